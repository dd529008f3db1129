"""B200-native implementation of Hetu-DiT's denoising-stage parallel hot path.

Host code is Python/PyTorch; every kernel lives in libhdit_b200.so (C ABI in
include/hdit.h, sources under csrc/). Nothing here falls back to a CPU or
library implementation: a missing extension raises at first use.
"""
__version__ = "0.1.0"
