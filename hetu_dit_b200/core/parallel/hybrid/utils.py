from ..ring import ring_flash_attn_func

# The reference also lists yunchang's "zigzag" and "strip" variants (hybrid/utils.py:7-11). They
# rebalance causal masks; DiT attention is non-causal, and neither works with the SP KV cache
# (hybrid/attn_layer.py:18,35-41), so only the basic ring is provided.
RING_IMPL_DICT = {
    "basic": ring_flash_attn_func,
}
