from .ring_flash_attn import ring_flash_attn_func, ring_flash_attn_forward

__all__ = ["ring_flash_attn_func", "ring_flash_attn_forward"]
