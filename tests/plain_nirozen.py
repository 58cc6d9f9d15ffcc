"""A plain, slow implementation of the Nirozen design on whole sequences, one function per mechanism, in float64 on
the CPU. It is the oracle of the tests: written from the design's equations, sharing no code with the package.

Notation: W is the residual width, T the tokens of one sequence, `w` a dict of tensors by checkpoint name, `p` a name
prefix ("l3.mix", "l3.mlp"). Linear weights are [out, in] and applied as y = x W^T.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def _t(w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return w[name].to(F)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The block norm: the stored weight is a deviation from one: the factor is (1 + weight)."""
    return unit_rms(x, eps) * (1.0 + weight)


def plain_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight


def token_rows(cfg: dict, w, ids: List[int]) -> torch.Tensor:
    """embed[token] * scale."""
    return _t(w, "embed")[torch.tensor(ids, dtype=torch.long)] * float(cfg["embedding"]["scale"])


def bigram_rows(cfg: dict, w, ids: List[int]) -> torch.Tensor:
    """Row (prev * mul_prev + cur * mul_cur) mod buckets of the bigram table; the sequence's first token takes the
    table's last row (number `buckets`)."""
    b = cfg["embedding"]["bigram"]
    n, mp, mc = int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"])
    rows = [n if i == 0 else (ids[i - 1] * mp + ids[i] * mc) % n for i in range(len(ids))]
    return _t(w, "bigram")[torch.tensor(rows, dtype=torch.long)]


def sinusoid_rows(width: int, n: int, base: float = 10000.0) -> torch.Tensor:
    """Entry 2i of position p is sin(p * base^(-2i/width)), entry 2i+1 the cosine of the same angle."""
    out = torch.zeros(n, width, dtype=F)
    pos = torch.arange(n, dtype=F)[:, None]
    i = torch.arange((width + 1) // 2, dtype=F)[None, :]
    ang = pos * torch.pow(torch.tensor(base, dtype=F), -2.0 * i / width)
    out[:, 0::2] = torch.sin(ang)[:, : out[:, 0::2].shape[1]]
    out[:, 1::2] = torch.cos(ang)[:, : out[:, 1::2].shape[1]]
    return out


def embedding(cfg: dict, w, ids: List[int]) -> torch.Tensor:
    x = token_rows(cfg, w, ids)
    if cfg["embedding"].get("bigram"):
        x = x + bigram_rows(cfg, w, ids)
    return x + sinusoid_rows(int(cfg["width"]), len(ids))


def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, sink: torch.Tensor) -> torch.Tensor:
    """Causal attention of one head, q [T,d], k [T,d], v [T,e]. The softmax's denominator also holds exp(sink): a key
    without a value whose score is `sink` itself (not multiplied by `scale`)."""
    T = q.shape[0]
    s = (q @ k.t()) * scale
    s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), float("-inf"))
    m = torch.maximum(s.max(dim=1, keepdim=True).values, sink.reshape(1, 1))
    e = torch.exp(s - m)
    den = e.sum(dim=1, keepdim=True) + torch.exp(sink.reshape(1, 1) - m)
    return (e / den) @ v


def latent_attention(mix: dict, w, p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Queries through a latent (down, norm, up); keys and values from one shared normed latent per token; no position
    enters; a sink per head in the softmax; the heads gated by sigmoid(W_g h) before the output product."""
    H, d, e = int(mix["heads"]), int(mix["dim"]), int(mix["vdim"])
    scale = float(mix["scale"])
    cq = plain_norm(h @ _t(w, f"{p}.dq").t(), _t(w, f"{p}.dq.norm"), eps)
    q = cq @ _t(w, f"{p}.uq").t()                                   # [T, H*d]
    c = plain_norm(h @ _t(w, f"{p}.dkv").t(), _t(w, f"{p}.dkv.norm"), eps)
    k = c @ _t(w, f"{p}.uk").t()                                    # [T, H*d]
    v = c @ _t(w, f"{p}.uv").t()                                    # [T, H*e]
    sink = _t(w, f"{p}.sink")
    heads = []
    for j in range(H):
        heads.append(sink_softmax_attention(q[:, j * d:(j + 1) * d], k[:, j * d:(j + 1) * d], v[:, j * e:(j + 1) * e],
                                            scale, sink[j]))
    o = torch.cat(heads, dim=1) * torch.sigmoid(h @ _t(w, f"{p}.g").t())
    return o @ _t(w, f"{p}.o").t()


def gated_unit(w, p: str, h: torch.Tensor) -> torch.Tensor:
    """down(silu(gate h) * (up h)), no biases."""
    a = h @ _t(w, f"{p}.gate").t()
    return ((a * torch.sigmoid(a)) * (h @ _t(w, f"{p}.up").t())) @ _t(w, f"{p}.down").t()


def route(mlp: dict, w, p: str, h: torch.Tensor):
    """Router logits W h + b; the `top` largest are chosen, weighted by the softmax over the chosen logits alone.
    Returns (expert ids [T, top], weights [T, top], logits [T, experts])."""
    z = h @ _t(w, f"{p}.router").t() + _t(w, f"{p}.router.b")
    top = int(mlp["router"]["top"])
    val, idx = torch.topk(z, top, dim=1)
    return idx, torch.softmax(val, dim=1), z


def moe(mlp: dict, w, p: str, h: torch.Tensor, margins: Optional[list] = None) -> torch.Tensor:
    idx, wt, z = route(mlp, w, p, h)
    if margins is not None:                                         # how far the last chosen logit is from the first left out
        srt = z.sort(dim=1, descending=True).values
        k = idx.shape[1]
        if k < z.shape[1]:
            margins += (srt[:, k - 1] - srt[:, k]).tolist()
    out = torch.zeros(h.shape[0], _t(w, f"{p}.e0.down").shape[0], dtype=F)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            out[t] += wt[t, j] * gated_unit(w, f"{p}.e{int(idx[t, j])}", h[t:t + 1])[0]
    if mlp.get("shared"):
        out = out + gated_unit(w, f"{p}.shared", h)
    return out


def run_order(cfg: dict):
    """[(layer index, pass number or None)]: layers start..stop-1 run `times` times in a row, then the rest; the pass
    number is given at the first layer of each pass (where the pass vector is added)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop["stop"]) <= int(loop["start"]):
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg: dict, w, ids: List[int], taps: Optional[list] = None, margins: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence. `taps` receives the residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = embedding(cfg, w, ids)
    for i, pass_no in run_order(cfg):
        L = cfg["layers"][i]
        if pass_no is not None:
            x = x + _t(w, "loop.step")[pass_no]
        if L["type"] != "latent_attention":
            raise ValueError(f"layer type {L['type']!r} is not part of this oracle")
        x = x + latent_attention(L["mixer"], w, f"l{i}.mix", offset_norm(x, _t(w, f"l{i}.norm1"), eps), eps)
        if L.get("mlp"):
            if L["mlp"]["kind"] != "moe":
                raise ValueError(f"feed-forward kind {L['mlp']['kind']!r} is not part of this oracle")
            x = x + moe(L["mlp"], w, f"l{i}.mlp", offset_norm(x, _t(w, f"l{i}.norm2"), eps), margins)
        if taps is not None:
            taps.append(x.clone())
    return offset_norm(x, _t(w, "final.norm"), eps) @ _t(w, "head").t()


def greedy(cfg: dict, w, prompt: List[int], n_new: int) -> List[int]:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
