from .hybrid import (hetuDiTFluxLongContextAttention, hetuDiTJointLongContextAttention, hetuDiTLongContextAttention,
                     xFuserFluxLongContextAttention, xFuserJointLongContextAttention, xFuserLongContextAttention)
from .ulysses import hetuDiTUlyssesAttention

__all__ = [
    "hetuDiTLongContextAttention", "hetuDiTFluxLongContextAttention", "hetuDiTJointLongContextAttention",
    "hetuDiTUlyssesAttention", "xFuserLongContextAttention", "xFuserFluxLongContextAttention",
    "xFuserJointLongContextAttention",
]
