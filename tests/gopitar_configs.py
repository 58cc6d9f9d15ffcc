"""Small Gopitar configurations that differ from one another in every size and option, and weights for them: drawn by
the framework's random-weights mode (values that bfloat16 holds exactly, so every path and the oracle compute with the same
numbers), then changed so that faults show: queries scaled up so that attention is peaked (a key that is lost at a window's
edge, or one too many, moves the output), the branches' last products scaled up so that what a mixer computes is of the
residual stream's own size, decays and gates in ranges where the recurrent state matters for hundreds of tokens."""
from __future__ import annotations

from typing import Dict

import torch


def _left(heads, kv_heads, dim, vdim, conv, window, rot_dims, rot_base, scale):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "mask": {"size": window}, "scale": scale}
    if rot_dims:
        d["rot"] = {"base": rot_base, "dims": rot_dims}
    return d


def _parallel(left, heads, dim, vdim, decay, ls, rs, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
                                          "left_scale": ls, "right_scale": rs},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _delta(heads, kv_heads, dim, vdim, conv, ff):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def gp_a() -> dict:
    # grouped keys (4 heads on 2), key size 32 below value size 64 (tensor-memory prefill at 64), window 24 that is no multiple of
    # a page, rotation of half a head, 3 taps; a delta layer first; the loop covers the middle and runs three times
    return {"architecture": "Gopitar", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "logit_softcap": 10.0,
            "layers": [_delta(4, 2, 16, 24, 3, 72),
                       _parallel(_left(4, 2, 32, 64, 3, 24, 16, 1000.0, 0.2), 3, 16, 24, [0.9, 0.5, 0.99], 0.7, 1.1, 64),
                       _delta(3, 3, 24, 16, 2, None),
                       _parallel(_left(2, 1, 16, 16, 2, 7, 16, 50.0, 0.3), 1, 8, 40, [0.97], 1.0, 0.5, 40)],
            "loop": {"start": 1, "stop": 3, "times": 3}}


def gp_b() -> dict:
    # value size below key size (48 and 16: the mma.sync prefill at 48), window 33, full rotation, 5 taps, no loop, no cap,
    # one layer without a feed-forward, width not a multiple of 16
    return {"architecture": "Gopitar", "vocab": 300, "width": 120, "norm": {"eps": 1e-4}, "embedding": {"scale": 0.5},
            "layers": [_parallel(_left(6, 3, 48, 16, 5, 33, 48, 10000.0, 0.15), 2, 24, 8, [0.8, 0.95], 1.2, 0.4, None),
                       _delta(2, 1, 40, 32, 5, 100),
                       _parallel(_left(1, 1, 64, 64, 1, 16, 0, 0.0, 0.125), 4, 8, 8, [0.6, 0.7, 0.8, 0.9], 0.5, 0.5, 56)]}


def gp_c() -> dict:
    # head size 128 (tensor-memory prefill at 128), a window of one page exactly, a window of 1 (the token itself), loop from
    # layer 0 twice, one tap in the delta layer (no convolution)
    return {"architecture": "Gopitar", "vocab": 128, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
            "logit_softcap": 30.0,
            "layers": [_parallel(_left(2, 2, 128, 128, 4, 16, 64, 500000.0, 0.09), 2, 32, 32, [0.999, 0.7], 0.6, 0.9, 96),
                       _parallel(_left(3, 1, 8, 24, 2, 1, 8, 100.0, 0.5), 2, 16, 16, [0.9, 0.9], 1.0, 1.0, 48),
                       _delta(2, 2, 16, 48, 1, 64)],
            "loop": {"start": 0, "stop": 2, "times": 2}}


def gp_d() -> dict:
    # a window longer than any test sequence (all keys seen), key size 20 (no fast kernel takes heads padded to 32 ... the
    # padded size is 32: fast kernels run on zero columns), loop of everything four times
    return {"architecture": "Gopitar", "vocab": 64, "width": 72, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
            "logit_softcap": 5.0,
            "layers": [_parallel(_left(3, 3, 20, 12, 4, 4096, 10, 10000.0, 0.22), 2, 12, 20, [0.5, 0.9], 0.8, 0.8, 40),
                       _delta(6, 2, 8, 12, 4, 24)],
            "loop": {"start": 0, "stop": 2, "times": 4}}


GOPITAR = {"a": gp_a, "b": gp_b, "c": gp_c, "d": gp_d}


def make_weights(raw: dict, seed: int, sharpen: float = 5.0) -> Dict[str, torch.Tensor]:
    from infinilm_b200.config import config_from_json
    from infinilm_b200.weights import random_tensors
    w = random_tensors(config_from_json(raw), seed, "cpu")
    for name in list(w):
        x = w[name].float()
        if name == "embed":
            x = x * 40.0 / float(raw["embedding"]["scale"])
        elif name.endswith(".left.q"):
            x = x * sharpen * 4.0
        elif name.endswith(".left.k"):
            x = x * 4.0
        elif name.endswith((".left.o", ".right.o")) or (name.endswith(".mix.o")):
            x = x * 12.0
        elif name.endswith(".down"):
            x = x * 20.0
        elif name.endswith((".mix.q", ".mix.k", ".mix.v", ".right.q", ".right.k", ".right.v")):
            x = x * 5.0
        elif name.endswith((".mix.a", ".mix.b", ".g")):
            x = x * 4.0
        elif name.endswith("head"):
            x = x * 10.0
        else:
            continue
        w[name] = x.to(torch.bfloat16)
    return w


def token_ids(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
