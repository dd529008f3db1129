"""Block cache of the DiT transformer: which Linear layers tensor parallelism splits, and how.

Mirrors TransformerBlockCache (hetu_dit/model_executor/cache/transformer_cache.py:9-154):
q/k/v and added q/k/v projections and the first MLP projection split by rows (output features),
the output projections and the second MLP projection by columns (input features).
"""
from typing import List, Optional

import torch.nn as nn

from .base_cache import BaseBlockCache

_ROW_KEYS = ("to_q", "to_k", "to_v", "add_k_proj", "add_q_proj", "add_v_proj")
_COLUMN_KEYS = ("to_out", "to_add_out")
_ADJUSTED = {f"{a}.module.{n}" for a in ("attn", "attn1") for n in
             ("to_q", "to_k", "to_v", "add_k_proj", "add_q_proj", "add_v_proj", "to_add_out", "to_out.0")}
_ADJUSTED |= {"ff.module.net.0.proj", "ff.module.net.2", "ff_context.module.net.0.proj", "ff_context.module.net.2"}


class TransformerBlockCache(BaseBlockCache):
    def choose_tp_split_type(self, name: str) -> Optional[str]:
        return self.determine_tp_split_type_by_name(name) if name in _ADJUSTED else None

    def determine_tp_split_type_by_name(self, name: str) -> str:
        low = name.lower()
        if any(k in low for k in _ROW_KEYS):
            return "row"
        if any(k in low for k in _COLUMN_KEYS):
            return "column"
        if "net.0.proj" in low:
            return "row"
        if "net.2" in low:
            return "column"
        return "row"

    def block_list_names(self) -> List[str]:
        return ["transformer_blocks", "single_transformer_blocks"]

    def block_lists(self, model: nn.Module) -> List[nn.ModuleList]:
        return [getattr(model, n) for n in self.block_list_names() if hasattr(model, n)]
