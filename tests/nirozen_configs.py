"""Small Nirozen configurations that differ from one another in every size and option, and weights for them: drawn
by the framework's random-weights mode (values that bfloat16 holds exactly, so every path and the oracle compute with
the same numbers), then changed so that faults show: token and pair rows as large as the position vector, the branches'
last products scaled up so that what a mixer or a feed-forward computes is of the residual stream's own size, queries
scaled up so that attention is peaked (a key that is lost, or one too many, moves the output), sinks large enough to
matter, pass vectors of visible size."""
from __future__ import annotations

from typing import Dict

import torch


def _layer(heads, dim, vdim, q_rank, kv_rank, scale, mlp):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale},
            "mlp": mlp}


def _moe(experts, top, ff, shared_ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": None if shared_ff is None else {"ff": shared_ff}}


def nz_a() -> dict:
    # latent of 64 (decode and tensor-memory prefill kernels), value size twice the key size, the loop starts at layer 0 and runs
    # three times, the last layer has no feed-forward, five experts, odd vocabulary
    return {"architecture": "Nirozen", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
            "embedding": {"scale": 3.0, "bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 7}},
            "layers": [_layer(3, 16, 32, 48, 64, 0.31, _moe(5, 2, 40, 24)), _layer(3, 16, 32, 48, 64, 0.31, _moe(5, 2, 40, None)),
                       _layer(2, 24, 8, 16, 64, 0.2, None)],
            "loop": {"start": 0, "stop": 2, "times": 3}}


def nz_b() -> dict:
    # latent of 48 (mma.sync prefill kernel), layers that differ in heads and ranks, top 1 in one layer, seven experts,
    # a loop in the middle that runs twice, eps and scales of their own
    return {"architecture": "Nirozen", "vocab": 300, "width": 160, "norm": {"eps": 1e-4},
            "embedding": {"scale": 0.5, "bigram": {"buckets": 13, "mul_prev": 5, "mul_cur": 3}},
            "layers": [_layer(5, 24, 16, 32, 48, 0.25, _moe(7, 3, 56, 72)), _layer(4, 8, 40, 72, 48, 0.5, _moe(7, 1, 24, 16)),
                       _layer(5, 24, 16, 32, 48, 0.25, _moe(3, 2, 56, None)), _layer(1, 32, 32, 8, 48, 0.18, _moe(2, 2, 16, 16))],
            "loop": {"start": 1, "stop": 3, "times": 2}}


def nz_c() -> dict:
    # no loop at all, a latent of 40 (no fast attention kernel takes it: the plain one runs), width not a multiple of 8, one bucket
    return {"architecture": "Nirozen", "vocab": 97, "width": 100, "norm": {"eps": 1e-6},
            "embedding": {"scale": 8.0, "bigram": {"buckets": 1, "mul_prev": 1, "mul_cur": 1}},
            "layers": [_layer(2, 12, 20, 24, 40, 0.4, _moe(4, 4, 28, 12)), _layer(7, 4, 4, 36, 40, 0.7, None)]}


def nz_d() -> dict:
    # latent of 128 (tensor-memory prefill at head size 128), every expert chosen (no discrete choice: long bfloat16 runs
    # compare position by position), a loop of one layer run four times, nine heads
    return {"architecture": "Nirozen", "vocab": 500, "width": 128, "norm": {"eps": 1e-5},
            "embedding": {"scale": 2.0, "bigram": {"buckets": 251, "mul_prev": 2, "mul_cur": 9}},
            "layers": [_layer(9, 16, 48, 64, 128, 0.3, _moe(3, 3, 48, 32)), _layer(4, 32, 16, 96, 128, 0.15, _moe(4, 4, 32, None))],
            "loop": {"start": 1, "stop": 2, "times": 4}}


def nz_e() -> dict:
    # a latent wider than any fast attention kernel takes (320: the plain kernel's wide form), one layer, no shared unit, a loop of all
    return {"architecture": "Nirozen", "vocab": 64, "width": 72, "norm": {"eps": 1e-5},
            "embedding": {"scale": 1.5, "bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 2}},
            "layers": [_layer(2, 8, 8, 40, 320, 0.35, _moe(3, 1, 16, None))], "loop": {"start": 0, "stop": 1, "times": 2}}


NIROZEN = {"a": nz_a, "b": nz_b, "c": nz_c, "d": nz_d, "e": nz_e}


def make_weights(raw: dict, seed: int, sharpen: float = 6.0) -> Dict[str, torch.Tensor]:
    from infinilm_b200.config import config_from_json
    from infinilm_b200.weights import random_tensors
    w = random_tensors(config_from_json(raw), seed, "cpu")
    g = torch.Generator().manual_seed(seed + 1000)
    for name in list(w):
        if name.endswith(".mix.uq"):
            w[name] = (w[name].float() * sharpen).to(torch.bfloat16)
        elif name.endswith(".mix.sink"):
            n = w[name].numel()
            w[name] = (torch.arange(n, dtype=torch.float32) % 3 * 2.5 - 1.0 + torch.randn(n, generator=g) * 0.3).to(torch.bfloat16)
        elif name == "loop.step":
            w[name] = (w[name].float() * 2.0).to(torch.bfloat16)
        elif name in ("embed", "bigram"):
            w[name] = (w[name].float() * 40.0 / float(raw["embedding"]["scale"] if name == "embed" else 1.0)).to(torch.bfloat16)
        elif name.endswith(".mix.o"):
            w[name] = (w[name].float() * 16.0).to(torch.bfloat16)
        elif name.endswith(".down"):
            w[name] = (w[name].float() * 30.0).to(torch.bfloat16)
    return w


def token_ids(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
