"""Ulysses-only attention operator.

Interface of the reference's hetuDiTUlyssesAttention
(hetu_dit/core/parallel/ulysses/attn_layer.py:12-155), which the reference's
processors pick when flash-attn is absent. Same exchange as the hybrid
operator with a ring of one; the KV-cache hook sits on the gathered K/V.
"""
import torch
from torch import Tensor

from .... import kernels
from ...distributed import parallel_state as ps
from ...resource_manager.cache_manager import get_cache_manager
from ..hybrid.attn_layer import _UlyssesExchange


class hetuDiTUlyssesAttention(torch.nn.Module):
    def __init__(self, scatter_idx: int = 2, gather_idx: int = 1, use_fa: bool = True, use_kv_cache: bool = True):
        super().__init__()
        if scatter_idx != 2 or gather_idx != 1:
            raise ValueError("only the (B, S, H, D) layout with scatter_idx=2, gather_idx=1 is supported")
        self.scatter_idx, self.gather_idx = scatter_idx, gather_idx
        self.use_fa = use_fa  # kept for signature compatibility: there is a single kernel path
        self.use_kv_cache = use_kv_cache
        self.ulysses_pg = ps.PROCESS_GROUP.ULYSSES_PG

    def forward(self, attn, query: Tensor, key: Tensor, value: Tensor, *, joint_tensor_query=None,
                joint_tensor_key=None, joint_tensor_value=None, dropout_p=0.0, softmax_scale=None, causal=False,
                window_size=(-1, -1), alibi_slopes=None, deterministic=False, return_attn_probs=False,
                joint_strategy="none") -> Tensor:
        self.ulysses_pg = ps.PROCESS_GROUP.ULYSSES_PG
        U = 1 if self.ulysses_pg is None else self.ulysses_pg.world_size
        has_joint = joint_tensor_key is not None and joint_tensor_value is not None and joint_tensor_query is not None
        if has_joint:
            if joint_strategy == "rear":
                query = torch.cat([query, joint_tensor_query], dim=1)
            elif joint_strategy == "front":
                query = torch.cat([joint_tensor_query, query], dim=1)
            elif joint_strategy == "none":
                raise ValueError(f"joint_strategy: {joint_strategy} not supported when joint tensors is not None.")
            else:
                raise ValueError(f"joint_strategy: {joint_strategy} not supported.")
            if U > 1:
                r = self.ulysses_pg.rank_in_group
                hpr = joint_tensor_key.shape[-2] // U
                joint_tensor_key = joint_tensor_key[..., hpr * r:hpr * (r + 1), :]
                joint_tensor_value = joint_tensor_value[..., hpr * r:hpr * (r + 1), :]
        if U > 1:
            xchg = _UlyssesExchange(self.ulysses_pg)
            query, key, value = xchg.gather_heads([query, key, value], ["q", "k", "v"])
        if self.use_kv_cache and attn is not None:
            key, value = get_cache_manager().update_and_get_kv_cache(new_kv=[key, value], layer=attn, slice_dim=1,
                                                                     layer_type="attn")
        ks, vs = [key], [value]
        if has_joint and joint_strategy == "rear":
            ks, vs = [key, joint_tensor_key], [value, joint_tensor_value]
        elif has_joint and joint_strategy == "front":
            ks, vs = [joint_tensor_key, key], [joint_tensor_value, value]
        if U == 1:
            return kernels.attn_fwd([query], ks, vs, softmax_scale=softmax_scale)
        # the reverse exchange rides on the attention epilogue: rows go straight into their owners' buffers
        B, S_g, Hl, D = query.shape
        out, plan = xchg.scatter_plan(B, S_g, Hl, D, query.dtype, "o")
        kernels.attn_fwd([query], ks, vs, softmax_scale=softmax_scale, out_dsts=plan["dsts"],
                         q_rows_per_dst=[plan["q"][0]], q_dst_row0=[plan["q"][1]])
        xchg.finish()
        return out
