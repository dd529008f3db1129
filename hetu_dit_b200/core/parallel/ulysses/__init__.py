from .attn_layer import hetuDiTUlyssesAttention

__all__ = ["hetuDiTUlyssesAttention"]
