"""Several mixers side by side on the same input: y = sum_i scale_i * mixer_i(h). Each keeps what it keeps (pages, states);
the part hands every branch its own share of the cache views.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List

import torch

from .. import ops
from .base import Mixer, ResidualTail, build_part, register_part
from .spec import PartSpec


def _needs_of(m: Mixer) -> list:
    n = m.cache_need()
    return [] if n is None else list(n) if isinstance(n, (tuple, list)) else [n]


class ParallelMixers(Mixer):
    """params: branches - a list of (PartSpec of a mixer, scale). A branch's prefix is relative to this part's and not
    empty: its tensors are this part's tensors `<branch prefix>.<name>`."""

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.branches, self.scales, self.rel = [], [], []
        for spec, scale in params["branches"]:
            if not spec.prefix:
                raise ValueError("parallel mixers: every branch needs a prefix of its own")
            self.branches.append(build_part("mixer", PartSpec(spec.kind, spec.params, f"{prefix}.{spec.prefix}" if prefix else spec.prefix), dtype))
            self.scales.append(float(scale))
            self.rel.append(spec.prefix)
        if len(self.branches) < 2 or len(set(self.rel)) != len(self.rel):
            raise ValueError("parallel mixers: at least two branches, each with its own prefix")
        self._n_needs = [len(_needs_of(m)) for m in self.branches]
        self._single = [not isinstance(m.cache_need(), (tuple, list)) for m in self.branches]

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self.branches)

    def weight_specs(self):
        return [dataclasses.replace(ws, name=f"{rel}.{ws.name}") for m, rel in zip(self.branches, self.rel) for ws in m.weight_specs()]

    def set_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for m, rel in zip(self.branches, self.rel):
            m.set_weights({k[len(rel) + 1:]: v for k, v in tensors.items() if k.startswith(rel + ".")})

    def cache_need(self):
        needs = [n for m in self.branches for n in _needs_of(m)]
        return tuple(needs) if needs else None

    # Rows whose norm is half done go to every branch's first product; with a tail every branch's output product adds its
    # share (scale_i x the tail's scale) into the residual itself, and the last one's view of the finished sum is the block's.
    def accepts_normed(self, T):
        return all(m.accepts_normed(T) for m in self.branches)

    def fuses_tail(self, T):
        return all(m.fuses_tail(T) for m in self.branches)

    def forward(self, x, ctx, cache, tail=None):
        views = list(cache) if isinstance(cache, (tuple, list)) else ([] if cache is None else [cache])
        at, ys = 0, []
        for m, n, single, scale in zip(self.branches, self._n_needs, self._single, self.scales):
            mine = views[at: at + n]
            at += n
            mine = (mine[0] if mine else None) if single else tuple(mine)
            if tail is not None:
                ys.append(m.forward(x, ctx, mine, tail=ResidualTail(tail.resid, tail.scale * scale, tail.norm)))
            else:
                ys.append(m.forward(x, ctx, mine))
        if tail is not None:
            return ys[-1]
        out = ctx.ws.rows("parallel_sum", x.shape[0], ys[0].shape[1], ys[0].dtype)
        ops.scaled_sum(ys[0], self.scales[0], ys[1], self.scales[1], out)
        for y, s in zip(ys[2:], self.scales[2:]):
            ops.scaled_sum(out, 1.0, y, s, out)
        return out


register_part("mixer", "parallel", ParallelMixers)
