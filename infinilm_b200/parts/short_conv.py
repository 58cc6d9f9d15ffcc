"""A short causal convolution over time, per channel, with its last inputs kept as per-request state.

y[t] = sum_j w[:, j] * u[t - (taps - 1) + j]: the last column of the weight meets the current token, inputs before the
sequence's start are zero. What a mixer builds on (like `Linear`): it owns the weights, says what state it needs
(`state_need`: float32 [taps - 1, channels], the inputs of the last taps - 1 tokens) and runs the two kernels of a step -
the convolution itself, which reads a portion's first inputs from the state, and the state's update.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops
from .spec import CacheNeed


class ShortConv:
    MAX_TAPS = 16

    def __init__(self, channels: int, taps: int):
        self.channels, self.taps = int(channels), int(taps)
        if not 1 <= self.taps <= self.MAX_TAPS:
            raise ValueError(f"short convolution: {taps} taps are not supported (1 to {self.MAX_TAPS})")
        self.weight: Optional[torch.Tensor] = None      # float32 [channels, taps]

    def state_need(self) -> CacheNeed:
        return CacheNeed("state", shape=(max(self.taps - 1, 1), self.channels), dtype="float32")

    def set(self, weights: Sequence[torch.Tensor]) -> None:
        """The weights of consecutive channel ranges, each [channels_i, taps]."""
        w = torch.cat([x.to(torch.float32) for x in weights], dim=0).contiguous()
        if tuple(w.shape) != (self.channels, self.taps):
            raise ValueError(f"short convolution: weights {tuple(w.shape)} != {(self.channels, self.taps)}")
        self.weight = w

    def run(self, x: torch.Tensor, x_off: int, ctx, state, out: torch.Tensor, segments: List[Tuple[int, int, int, int]], act: int = 0) -> None:
        """Convolves channels [x_off, x_off + channels) of `x`. `segments`: (first channel, number of segments, columns
        of a segment, first output column, columns it is written as - the surplus zero) per run of equal segments,
        given as (ch0, n_seg, seg_in, out_off, seg_out). Then leaves the state of the step's end in the write slots."""
        for ch0, n_seg, seg_in, out_off, seg_out in segments:
            ops.short_conv(x, x_off + ch0, self.weight[ch0: ch0 + n_seg * seg_in], state.storage, ch0, state.read_slots,
                           ctx.tok_entry, ctx.entry_qstart, out, out_off, n_seg, seg_in, seg_out, act)
        if state.writable:
            ops.short_conv_state(x, x_off, self.channels, self.taps, state.storage, 0, state.read_slots, state.write_slots,
                                 ctx.entry_qstart, ctx.n_entries)
