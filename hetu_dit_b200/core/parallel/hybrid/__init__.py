from .attn_layer import (hetuDiTFluxLongContextAttention, hetuDiTJointLongContextAttention,
                         hetuDiTLongContextAttention, xFuserFluxLongContextAttention,
                         xFuserJointLongContextAttention, xFuserLongContextAttention)

__all__ = [
    "hetuDiTLongContextAttention", "hetuDiTFluxLongContextAttention", "hetuDiTJointLongContextAttention",
    "xFuserLongContextAttention", "xFuserFluxLongContextAttention", "xFuserJointLongContextAttention",
]
