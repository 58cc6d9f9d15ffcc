"""Softmax attention over the paged cache whose queries, keys and values pass a short convolution over time first, with
a key size that may differ from the value size, a score scale of its own, an optional window and one sigmoid gate per head.

    [q | k | v | g] = W h (+ b);  q, k, v <- short_conv(q), short_conv(k), short_conv(v)  (state: their last taps - 1 inputs)
    q, k rotated on their first rot_dim entries;  o_h = softmax(scale q_h . k over the window) v;  o_h *= sigmoid(g_h)
    y = W_o [o_1 .. o_H] (+ b_o)

The paged cache and the attention kernels hold keys and values of one size, so heads are laid out at
hd = max(key size, value size) rounded up to 16, the surplus columns zero (written so by the convolution kernel): a zero
column adds nothing to a score, and surplus value columns are dropped where the gate is applied.
Tensors (under the part's prefix): q, k, v, o [out, in]; q.b, k.b, v.b, o.b; q.conv, k.conv, v.conv [channels, taps]; g [heads, in].
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .attention import PagedAttend
from .base import Mixer, build_part, register_part
from .linear import Linear
from .short_conv import ShortConv
from .spec import CacheNeed, PartSpec, WeightSpec


class ConvGatedAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, qk_dim, v_dim, scale, window (None: all keys), conv_taps (None: no
    convolution), qkv_bias, out_bias, head_gate, position (PartSpec of a rotary encoding, or None)."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        p = params
        self.hidden, self.nh, self.nkv = int(p["hidden"]), int(p["n_heads"]), int(p["n_kv_heads"])
        self.dk, self.dv = int(p["qk_dim"]), int(p["v_dim"])
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads are not a multiple of {self.nkv} kv heads")
        self.hd = (max(self.dk, self.dv) + 15) // 16 * 16
        if self.hd > 256:
            raise ValueError(f"attention: key / value size {max(self.dk, self.dv)} is not supported (up to 256)")
        self.scale = float(p["scale"])
        self.window: Optional[int] = None if p.get("window") is None else int(p["window"])
        if self.window is not None and self.window < 1:
            raise ValueError("attention: a window holds at least the token itself")
        self.has_conv, self.taps = p.get("conv_taps") is not None, int(p.get("conv_taps") or 1)
        self.qkv_bias, self.out_bias, self.head_gate = bool(p.get("qkv_bias", False)), bool(p.get("out_bias", False)), bool(p.get("head_gate", False))
        self.nq, self.nk, self.nvv = self.nh * self.dk, self.nkv * self.dk, self.nkv * self.dv
        self.n_conv = self.nq + self.nk + self.nvv
        self.n_proj = self.n_conv + (self.nh if self.head_gate else 0)
        self.n_proj_pad = (self.n_proj + 7) // 8 * 8          # rows of 16-byte multiples for the kernels that read 8 at a time
        self.proj = Linear(self.hidden, self.n_proj_pad, dtype)
        self.o_proj = Linear(self.nh * self.dv, self.hidden, dtype)
        self.conv = ShortConv(self.n_conv, self.taps)
        self.position = build_part("position", p.get("position") or PartSpec("none"), dtype)
        if self.position.has_transform or self.position.rot_dim > self.dk or self.position.rot_dim % 2:
            raise ValueError("attention: the position encoding must be a rotary table over an even number of entries within the key size")
        self.core = PagedAttend(dtype, self.nh, self.nkv, self.hd, self.scale, self.window, bool(p.get("plain_kernel", False)),
                                str(p.get("prefill_kernel", "auto")))

    def weight_specs(self) -> List[WeightSpec]:
        H = self.hidden
        specs = [WeightSpec("q", (self.nq, H)), WeightSpec("k", (self.nk, H)), WeightSpec("v", (self.nvv, H)),
                 WeightSpec("o", (H, self.nh * self.dv))]
        if self.qkv_bias:
            specs += [WeightSpec(n + ".b", (c,), "vector", ("normal", 0.02)) for n, c in (("q", self.nq), ("k", self.nk), ("v", self.nvv))]
        if self.out_bias:
            specs.append(WeightSpec("o.b", (H,), "vector", ("normal", 0.02)))
        if self.has_conv:
            specs += [WeightSpec(n + ".conv", (c, self.taps), "vector", ("normal", 0.5)) for n, c in (("q", self.nq), ("k", self.nk), ("v", self.nvv))]
        if self.head_gate:
            specs.append(WeightSpec("g", (self.nh, H)))
        return specs

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        ws = [t["q"], t["k"], t["v"]] + ([t["g"]] if self.head_gate else [])
        pad = self.n_proj_pad - self.n_proj
        if pad:
            ws.append(torch.zeros((pad, self.hidden), dtype=ws[0].dtype, device=ws[0].device))
        b = None
        if self.qkv_bias:
            b = torch.cat([t["q.b"].float(), t["k.b"].float(), t["v.b"].float(),
                           torch.zeros(self.n_proj_pad - self.n_conv, dtype=torch.float32, device=t["q"].device)])
        self.proj.set(torch.cat(ws, dim=0), b)
        self.o_proj.set(t["o"], t.get("o.b"))
        if self.has_conv:
            self.conv.set([t["q.conv"], t["k.conv"], t["v.conv"]])
        else:
            self.conv.set([torch.ones((self.n_conv, 1), dtype=torch.float32, device=t["q"].device)])
        self.position.to_device(t["q"].device)

    def cache_need(self):
        return (CacheNeed("paged_kv", n_kv_heads=self.nkv, head_dim=self.hd, window=self.window), self.conv.state_need())

    # A decode step of a few bfloat16 rows: the first product may take rows whose norm is only half done (it divides by the
    # rms itself) and the output product may add into the residual and prepare the next norm, as the framework's other mixers do.
    def accepts_normed(self, T):
        return self.dtype == torch.bfloat16 and ops.skinny_ok(T, self.hidden)

    def fuses_tail(self, T):
        return self.dtype == torch.bfloat16 and ops.skinny_resid_ok(T, self.nh * self.dv, self.hidden)

    def forward(self, x, ctx, cache, tail=None):
        pages, state = cache
        T, hd = x.shape[0], self.hd
        proj = ctx.ws.rows("cga_proj", T, self.n_proj_pad, self.dtype)
        if isinstance(x, ops.NormedInput):
            ops.gemm_skinny(x.xw, self.proj.weight, proj, 1.0, self.proj.bias, norm_in=x)
        else:
            self.proj(x, proj)
        qkv = ctx.ws.rows("cga_qkv", T, (self.nh + 2 * self.nkv) * hd, self.dtype)
        # the convolution writes heads at the common size hd, the surplus columns zero
        self.conv.run(proj, 0, ctx, state, qkv, (self.nh + self.nkv, self.dk, self.nkv, self.dv, hd))
        pos = self.position
        ops.rope_store(qkv, ctx.tok_pos, ctx.tok_entry, pages.block_table, pages.storage if pages.writable else None,
                       pages.page_size, self.nh, self.nkv, hd, pos.rot_dim, pos.inv_freq, pos.mscale)
        att = ctx.ws.rows("cga_att", T, self.nh * hd, self.dtype)
        self.core.run(qkv, att, ctx, pages)
        if self.head_gate or hd != self.dv:
            gated = ctx.ws.rows("cga_gated", T, self.nh * self.dv, self.dtype)
            if self.head_gate:
                ops.head_gate(att, hd, proj, self.n_conv, gated, self.nh, self.dv)
            else:
                ops.head_gate(att, hd, None, 0, gated, self.nh, self.dv)
            att = gated
        if tail is not None:
            return ops.gemm_skinny_resid(att, self.o_proj.weight, self.o_proj.alpha, self.o_proj.bias, tail.resid, tail.scale,
                                         tail.norm.weight, tail.norm.eps, ctx.ws.rows("xw_mixer", T, self.hidden, self.dtype),
                                         ctx.ws.rows("sumsq_mixer", T, (self.hidden + 15) // 16, torch.float32))
        return self.o_proj(att, ctx.ws.rows("cga_branch", T, self.hidden, self.dtype))


register_part("mixer", "conv_gated_attention", ConvGatedAttention)
