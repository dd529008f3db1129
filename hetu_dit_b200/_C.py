"""ctypes binding of libhdit_b200.so (declared in include/hdit.h).

The library is the only compute path of this package: if it is missing or a
call fails, an exception is raised -- there is no eager/PyTorch fallback.
"""
import ctypes
import os
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libhdit_b200.so")

HDIT_OK = 0
HDIT_ERR_BAD_ARG = 1
HDIT_ERR_SHAPE = 2
HDIT_ERR_CUDA = 3
HDIT_ERR_NOT_INITIALISED = 4
HDIT_ERR_PEER_TIMEOUT = 5
HDIT_ERR_TOO_LARGE = 6

HDIT_BF16, HDIT_FP16, HDIT_FP32 = 0, 1, 2
HDIT_MAX_Q_SEG = 2
HDIT_MAX_KV_SEG = 10

ATTN_FINAL, ATTN_PARTIAL_FIRST, ATTN_PARTIAL_MERGE, ATTN_MERGE_FINAL = 0, 1, 2, 3


class HditError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code, message):
        super().__init__(f"hdit status {code}: {message}")
        self.code = code


class Seg(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("len", ctypes.c_int64),
        ("stride_b", ctypes.c_int64),
        ("stride_s", ctypes.c_int64),
        ("stride_h", ctypes.c_int64),
    ]


class AttnArgs(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("mode", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("n_q_seg", ctypes.c_int32),
        ("n_kv_seg", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("q", Seg * HDIT_MAX_Q_SEG),
        ("k", Seg * HDIT_MAX_KV_SEG),
        ("v", Seg * HDIT_MAX_KV_SEG),
        ("out", ctypes.c_void_p),
        ("out_stride_b", ctypes.c_int64),
        ("out_stride_s", ctypes.c_int64),
        ("out_stride_h", ctypes.c_int64),
        ("lse", ctypes.c_void_p),
        ("acc_out", ctypes.c_void_p),
        ("acc_lse", ctypes.c_void_p),
        ("stream", ctypes.c_void_p),
        ("n_out_dst", ctypes.c_int32),
        ("kv_interleave", ctypes.c_int32),
        ("out_dst", ctypes.c_void_p * 8),
        ("q_rows_per_dst", ctypes.c_int64 * HDIT_MAX_Q_SEG),
        ("q_dst_row0", ctypes.c_int64 * HDIT_MAX_Q_SEG),
        ("n_wait", ctypes.c_int32),
        ("reserved1", ctypes.c_int32),
        ("wait_slots", ctypes.c_void_p * 8),
        ("wait_epoch", ctypes.c_void_p),
        ("wait_spins", ctypes.c_int64),
    ]


class CopyPiece(ctypes.Structure):
    _fields_ = [
        ("src", ctypes.c_void_p),
        ("dst", ctypes.c_void_p),
        ("n_outer", ctypes.c_int64),
        ("src_outer_pitch", ctypes.c_int64),
        ("dst_outer_pitch", ctypes.c_int64),
        ("rows", ctypes.c_int64),
        ("src_pitch", ctypes.c_int64),
        ("dst_pitch", ctypes.c_int64),
        ("row_bytes", ctypes.c_int64),
    ]


class NormRopeTensor(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p),
        ("x_stride_b", ctypes.c_int64),
        ("x_stride_s", ctypes.c_int64),
        ("x_stride_h", ctypes.c_int64),
        ("norm_weight", ctypes.c_void_p),
        ("norm_bias", ctypes.c_void_p),
        ("do_norm", ctypes.c_int32),
        ("do_rope", ctypes.c_int32),
        ("dst", ctypes.c_void_p * 8),
        ("dst_stride_b", ctypes.c_int64),
        ("dst_stride_s", ctypes.c_int64),
        ("dst_stride_h", ctypes.c_int64),
        ("dst_seq_offset", ctypes.c_int64),
    ]


class NormRopeArgs(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("seq", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("n_tensors", ctypes.c_int32),
        ("n_dst", ctypes.c_int32),
        ("eps", ctypes.c_float),
        ("cos", ctypes.c_void_p),
        ("sin", ctypes.c_void_p),
        ("rope_rows", ctypes.c_int64),
        ("rope_seq_start", ctypes.c_int64),
        ("rope_row0", ctypes.c_int64),
        ("t", NormRopeTensor * 3),
        ("stream", ctypes.c_void_p),
        ("range2_start", ctypes.c_int64),
        ("range2_norm_weight", ctypes.c_void_p * 3),
        ("range2_norm_bias", ctypes.c_void_p * 3),
        ("range2_do_rope", ctypes.c_int32 * 3),
        ("reserved0", ctypes.c_int32),
        ("range2_rope_row0", ctypes.c_int64),
        ("n_signal", ctypes.c_int32),
        ("signal_me", ctypes.c_int32),
        ("signal_slots", ctypes.c_void_p * 8),
        ("epoch_counter", ctypes.c_void_p),
        ("ticket", ctypes.c_void_p),
    ]


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("epilogue", ctypes.c_int32),
        ("m", ctypes.c_int64),
        ("n", ctypes.c_int64),
        ("k", ctypes.c_int64),
        ("a", ctypes.c_void_p),
        ("lda", ctypes.c_int64),
        ("w", ctypes.c_void_p),
        ("ldw", ctypes.c_int64),
        ("bias", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("ldo", ctypes.c_int64),
        ("residual", ctypes.c_void_p),
        ("ldr", ctypes.c_int64),
        ("gate", ctypes.c_void_p),
        ("gate_batch_stride", ctypes.c_int64),
        ("rows_per_batch", ctypes.c_int64),
        ("tile_n", ctypes.c_int32),
        ("max_ctas", ctypes.c_int32),
        ("stream", ctypes.c_void_p),
        ("tile_m", ctypes.c_int32),
        ("cta_pair", ctypes.c_int32),
    ]


GEMM_BIAS, GEMM_BIAS_GELU_TANH, GEMM_BIAS_GATE_RESIDUAL = 0, 1, 2

_lib = None
_lock = threading.Lock()


def _declare(lib):
    lib.hdit_version.restype = ctypes.c_int
    lib.hdit_version.argtypes = []
    lib.hdit_last_error.restype = ctypes.c_char_p
    lib.hdit_last_error.argtypes = []
    lib.hdit_device_status.restype = ctypes.c_int
    lib.hdit_device_status.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int32), ctypes.c_int]
    lib.hdit_attn_fwd.restype = ctypes.c_int
    lib.hdit_attn_fwd.argtypes = [ctypes.POINTER(AttnArgs)]
    lib.hdit_attn_fwd_splitkv.restype = ctypes.c_int
    lib.hdit_attn_fwd_splitkv.argtypes = [ctypes.POINTER(AttnArgs), ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    lib.hdit_attn_fwd_split_static.restype = ctypes.c_int
    lib.hdit_attn_fwd_split_static.argtypes = [ctypes.POINTER(AttnArgs), ctypes.c_int32]
    lib.hdit_copy_pieces.restype = ctypes.c_int
    lib.hdit_copy_pieces.argtypes = [ctypes.POINTER(CopyPiece), ctypes.c_int64, ctypes.c_void_p]
    lib.hdit_kv_scatter.restype = ctypes.c_int
    lib.hdit_kv_scatter.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int64] * 7 + [
        ctypes.c_void_p]
    lib.hdit_qk_norm_rope.restype = ctypes.c_int
    lib.hdit_qk_norm_rope.argtypes = [ctypes.POINTER(NormRopeArgs)]
    lib.hdit_ln_modulate.restype = ctypes.c_int
    lib.hdit_ln_modulate.argtypes = [ctypes.c_int32] + [ctypes.c_void_p] * 4 + [ctypes.c_int64] * 6 + [
        ctypes.c_float, ctypes.c_void_p]
    lib.hdit_gate_residual.restype = ctypes.c_int
    lib.hdit_gate_residual.argtypes = [ctypes.c_int32] + [ctypes.c_void_p] * 4 + [ctypes.c_int64] * 7 + [ctypes.c_void_p]
    lib.hdit_gelu_tanh.restype = ctypes.c_int
    lib.hdit_gelu_tanh.argtypes = [ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int64] * 4 + [ctypes.c_void_p]
    lib.hdit_cfg_euler_step.restype = ctypes.c_int
    lib.hdit_cfg_euler_step.argtypes = [ctypes.c_int32] + [ctypes.c_void_p] * 5 + [ctypes.c_int64, ctypes.c_float,
                                                                                 ctypes.c_void_p, ctypes.c_int32,
                                                                                 ctypes.c_void_p]
    lib.hdit_linear_fused.restype = ctypes.c_int
    lib.hdit_linear_fused.argtypes = [ctypes.POINTER(GemmArgs)]
    lib.hdit_heap_alloc.restype = ctypes.c_int
    lib.hdit_heap_alloc.argtypes = [ctypes.c_int64, ctypes.POINTER(ctypes.c_void_p)]
    lib.hdit_heap_free.restype = ctypes.c_int
    lib.hdit_heap_free.argtypes = [ctypes.c_void_p]
    lib.hdit_ipc_export.restype = ctypes.c_int
    lib.hdit_ipc_export.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
    lib.hdit_ipc_open.restype = ctypes.c_int
    lib.hdit_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    lib.hdit_ipc_close.restype = ctypes.c_int
    lib.hdit_ipc_close.argtypes = [ctypes.c_void_p]
    lib.hdit_peer_barrier.restype = ctypes.c_int
    lib.hdit_peer_barrier.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                      ctypes.c_int, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    lib.hdit_peer_signal.restype = ctypes.c_int
    lib.hdit_peer_signal.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    lib.hdit_peer_wait.restype = ctypes.c_int
    lib.hdit_peer_wait.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                   ctypes.c_void_p]


def lib():
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise ImportError(
                        f"{LIB_PATH} is missing: build it with `python -m hetu_dit_b200.build` "
                        "(there is no fallback compute path)"
                    )
                handle = ctypes.CDLL(LIB_PATH)
                _declare(handle)
                _lib = handle
    return _lib


def check(code):
    if code != HDIT_OK:
        raise HditError(code, lib().hdit_last_error().decode("utf-8", "replace"))


def device_status(device, clear=False):
    """(code, block, where, iteration) written by the first failed bounded wait, or zeros."""
    out = (ctypes.c_int32 * 4)()
    check(lib().hdit_device_status(int(device), out, 1 if clear else 0))
    return tuple(out)
