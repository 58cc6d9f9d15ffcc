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

    def run(self, x: torch.Tensor, x_off: int, ctx, state, out: torch.Tensor, segments: Tuple, act: int = 0) -> None:
        """Convolves channels [x_off, x_off + channels) of `x` into `out` from column 0: `segments` is (n_seg, seg_in, seg_out)
        or (n_seg, seg_in, n_seg2, seg_in2, seg_out) - that many segments of seg_in channels (then n_seg2 of seg_in2), each
        written seg_out columns wide, the surplus zero. Then leaves the state of the step's end in the write slots: for the
        single tokens the convolution kernel does it itself, for the portions behind them a second kernel."""
        if len(segments) == 3:
            n1, s1, n2, s2, so = segments[0], segments[1], 0, 0, segments[2]
        else:
            n1, s1, n2, s2, so = segments
        if n1 * s1 + n2 * s2 != self.channels:
            raise ValueError("short convolution: the segments do not add up to the channels")
        wr = state.write_slots if state.writable else None
        ops.short_conv(x, x_off, self.weight, state.storage, 0, state.read_slots, ctx.tok_entry, ctx.entry_qstart, out, 0, n1, s1, so, act,
                       n_seg2=n2, seg_in2=s2, write_slots=wr)
        if wr is not None and ctx.n_entries > ctx.n_decode:
            ops.short_conv_state(x, x_off, self.channels, self.taps, state.storage, 0, state.read_slots, wr, ctx.entry_qstart,
                                 ctx.n_entries - ctx.n_decode, first_entry=ctx.n_decode)
