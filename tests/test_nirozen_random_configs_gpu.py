"""Nirozen at sizes drawn from a seed: widths that are no multiple of 8, latents with and without a fast attention kernel,
one head or many, key and value sizes that differ, any number of experts and choices, layers without a feed-forward, loops
anywhere. Each configuration runs a prompt whole, in portions and token by token against the oracle, in both dtypes."""
import random
import warnings

import pytest
import torch

import plain_nirozen as P
from nirozen_configs import _layer, _moe, make_weights, token_ids

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 136, 200, 264])
    n_layers = rng.randint(1, 4)
    layers = []
    for _ in range(n_layers):
        dim = rng.choice([4, 8, 12, 16, 24, 40])
        mlp = None
        if rng.random() < 0.8:
            experts = rng.randint(1, 9)
            mlp = _moe(experts, rng.randint(1, experts), rng.choice([8, 20, 24, 56]), rng.choice([None, 8, 36]))
        layers.append(_layer(rng.randint(1, 9), dim, rng.choice([4, 8, 20, 32]), rng.choice([8, 24, 40, 64]),
                             rng.choice([16, 24, 32, 64, 80, 96, 128, 192, 256]), round(rng.uniform(0.1, 0.6), 3), mlp))
    raw = {"architecture": "Nirozen", "vocab": rng.choice([50, 129, 333]), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])},
           "embedding": {"scale": rng.choice([0.5, 4.0, 11.0]), "bigram": {"buckets": rng.choice([1, 7, 64, 1000]), "mul_prev": rng.randint(1, 99999),
                                                                        "mul_cur": rng.randint(1, 99999)}},
           "layers": layers}
    if rng.random() < 0.75:
        a = rng.randint(0, n_layers - 1)
        raw["loop"] = {"start": a, "stop": rng.randint(a + 1, n_layers), "times": rng.randint(1, 3)}
    return raw


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(10)))
def test_random_configuration(cuda_device, seed, dtype):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine, StepEntry
    raw = random_config(seed)
    w = make_weights(raw, seed)
    ids = token_ids(75, raw["vocab"], seed)
    margins = []
    ref = P.forward(raw, w, ids, margins=margins)
    sure = len(ids)
    if dtype == "bfloat16" and margins:                               # compare up to the first routing choice that rounding can turn
        m = torch.tensor(margins).view(-1, len(ids)).amin(0)
        close_calls = torch.nonzero(m < 0.08)
        sure = int(close_calls[0]) if close_calls.numel() else sure
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        eng = Engine.from_tensors(config_from_json(raw), w, dtype=dtype, page_size=16, num_pages=8, max_seqs=2, max_batch_tokens=128)
    tol = 4e-5 if dtype == "float32" else 5e-2
    for cuts in ([75], [33, 2, 17, 1, 1, 21], [16] + [1] * 59):
        seq, outs, a = eng.open(str(cuts[0])), [], 0
        for c in cuts:
            outs.append(eng.step([StepEntry(seq, ids[a:a + c], list(range(c)))]).clone())
            a += c
        eng.close(seq)
        got = torch.cat(outs, 0).double().cpu()[:sure]
        err = ((got - ref[:sure]).abs() / ref[:sure].abs().amax(dim=-1, keepdim=True)).amax(dim=-1)
        n_bad = int((err > tol).sum())
        worst = float(err.max()) if sure else 0.0
        assert torch.isfinite(got).all()
        assert n_bad <= (0 if dtype == "float32" else sure // 25) and (dtype == "float32" or worst <= 3 * tol), \
            f"seed {seed} cuts {cuts[:3]}: {n_bad} of {sure} positions over {tol:.0e}, worst {worst:.2e}; config {raw}"
    eng.synchronize()
    eng.cache.check_invariants()
