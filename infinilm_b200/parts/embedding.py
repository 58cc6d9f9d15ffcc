"""Token embedding and output head.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:81,92` (embedding),
`python/infinilm/modeling_utils.py:15-23,258-263` (the table is multiplied by scale_emb when it
is loaded, in the model dtype) - here the table stays as stored and the gather multiplies in
f32, rounding through the model dtype once, which gives the value the pre-scaled table holds;
`minicpm4_for_causal_lm.cpp:117-125` (lm_head with alpha = dim_model_base / hidden),
`modeling_utils.py:342-351` (an absent lm_head.weight is taken from the unscaled embedding).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Part, register_part
from .linear import Linear
from .spec import WeightSpec


class TokenEmbedding(Part):
    """params: vocab, hidden, scale; name (local tensor name, default "weight"); exact (default False: on the bfloat16 path
    row x scale is rounded through bfloat16, the value a table scaled at load would hold; True: the float32 product enters
    the residual stream as it is)."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.vocab, self.hidden, self.scale = int(params["vocab"]), int(params["hidden"]), float(params.get("scale", 1.0))
        self.name, self.exact = str(params.get("name", "weight")), bool(params.get("exact", False))
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.vocab, self.hidden))]

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.table = t[self.name].to(self.dtype).contiguous()

    def forward(self, token_ids: torch.Tensor, resid: torch.Tensor) -> torch.Tensor:
        ops.embed(token_ids, self.table, self.scale, resid, round_bf16=(self.dtype == torch.bfloat16 and not self.exact))
        return resid


class OutputHead(Part):
    """params: vocab, hidden, scale, tied_to (full name of the embedding table or None), name (local tensor name,
    default "weight"), softcap (None, or c: logits = c * tanh(logits / c)). Logits are float32 on both paths."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.vocab, self.hidden = int(params["vocab"]), int(params["hidden"])
        self.linear = Linear(self.hidden, self.vocab, dtype, alpha=float(params.get("scale", 1.0)), use_tc5=True)
        self.tied_to = params.get("tied_to")
        self.name = str(params.get("name", "weight"))
        self.softcap = None if params.get("softcap") is None else float(params["softcap"])
        if self.softcap is not None and not self.softcap > 0.0:
            raise ValueError("output head: the soft cap must be positive")

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.vocab, self.hidden), fallback=self.tied_to)]

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.linear.set(t[self.name])

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        self.linear(x, out, out_f32=True)
        if self.softcap is not None:
            ops.softcap(out, self.softcap)
        return out


class PairPositionEmbedding(Part):
    """Token rows times a scale, plus - each optional - a row of a second table chosen by a hash of (previous token, token)
    and a sinusoidal position vector; the sum is made in float32 and not rounded.

    params: vocab, hidden, scale, name (tensor of the table); pair: None or {buckets, mul_prev, mul_cur, name} - row
    (prev * mul_prev + token * mul_cur) mod buckets of a [buckets + 1, hidden] table, its last row for a sequence's first
    token; sinusoid_base: None or b - entry 2i of position p is sin(p * b^(-2i/hidden)), entry 2i+1 the cosine.
    The previous token of a portion's first token is part of the request's state: one int32 word in a state slot
    (token + 1; the zero state means "none"), read and written on the device, so a step never needs the host to know it
    (a token sampled in the step before may still be on the device)."""
    graph_safe = True
    takes_context = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.vocab, self.hidden, self.scale = int(params["vocab"]), int(params["hidden"]), float(params.get("scale", 1.0))
        self.name = str(params.get("name", "weight"))
        self.pair = dict(params["pair"]) if params.get("pair") else None
        if self.pair is not None and int(self.pair["buckets"]) <= 0:
            raise ValueError("embedding: the pair table needs at least one bucket")
        self.base = None if params.get("sinusoid_base") is None else float(params["sinusoid_base"])
        self.table: Optional[torch.Tensor] = None
        self.pair_table: Optional[torch.Tensor] = None
        self.inv_freq: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.name, (self.vocab, self.hidden))]
        if self.pair is not None:
            specs.append(WeightSpec(str(self.pair.get("name", "pair")), (int(self.pair["buckets"]) + 1, self.hidden)))
        return specs

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.table = t[self.name].to(self.dtype).contiguous()
        if self.pair is not None:
            self.pair_table = t[str(self.pair.get("name", "pair"))].to(self.dtype).contiguous()
        if self.base is not None:
            i = torch.arange((self.hidden + 1) // 2, dtype=torch.float64)
            self.inv_freq = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / self.hidden).to(torch.float32).to(self.table.device)

    def cache_need(self):
        from .spec import CacheNeed
        return CacheNeed("state", shape=(1,), dtype="int32") if self.pair is not None else None

    def forward(self, token_ids: torch.Tensor, resid: torch.Tensor, ctx, cache) -> torch.Tensor:
        p = self.pair
        ops.embed_pair_pos(token_ids, ctx.tok_pos, ctx.tok_entry, ctx.entry_qstart, self.table, self.scale, self.pair_table,
                           int(p["buckets"]) if p else 0, int(p["mul_prev"]) if p else 0, int(p["mul_cur"]) if p else 0,
                           cache.storage if cache is not None else None, cache.read_slots if cache is not None else None,
                           cache.write_slots if cache is not None and cache.writable else None, self.inv_freq, resid)
        return resid


class RowTable(Part):
    """A table of residual-wide vectors kept in float32 (they are added to the float32 residual stream).
    params: rows, hidden, name."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.rows, self.hidden, self.name = int(params["rows"]), int(params["hidden"]), str(params.get("name", "weight"))
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.rows, self.hidden), role="vector", init=("normal", 0.5))]

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.table = t[self.name].to(torch.float32).contiguous()
        self._rows = [self.table[i] for i in range(self.rows)]

    def row(self, i: int) -> torch.Tensor:
        return self._rows[i]


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "pair_position_embedding", PairPositionEmbedding)
register_part("embedding", "row_table", RowTable)
register_part("head", "linear_head", OutputHead)
