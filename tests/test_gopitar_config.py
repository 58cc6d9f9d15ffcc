"""Gopitar without a GPU: configuration reading, the run order of looped layers, the tensor names a model wants, the
random-weights folder, and properties of the plain implementation that the engine's kernels rest on (a convolution or a
recurrence continued from its state equals the whole; a head padded with zero columns scores the same)."""
import json
import os

import pytest
import torch

import plain_gopitar as P
from gopitar_configs import GOPITAR, make_weights, token_ids


def _cfg(raw):
    from infinilm_b200.config import config_from_json
    return config_from_json(raw)


@pytest.mark.parametrize("name", sorted(GOPITAR))
def test_config_and_tensor_names(name):
    from infinilm_b200.config.registry import describe_model
    from infinilm_b200.models.causal_lm import CausalLM
    raw = GOPITAR[name]()
    cfg = _cfg(raw)
    assert cfg.architecture == "Gopitar" and cfg.vocab_size == raw["vocab"] and cfg.hidden_size == raw["width"]
    model = CausalLM(describe_model(cfg), torch.float32)
    names = {p.full_name(ws.name): tuple(ws.shape) for p, ws in model.weight_specs()}
    W = raw["width"]
    assert names["embed"] == (raw["vocab"], W) and names["head"] == (raw["vocab"], W) and names["final.norm"] == (W,)
    for i, L in enumerate(raw["layers"]):
        m = L["mixer"]
        if L["type"] == "parallel":
            l, r = m["left"], m["right"]
            assert names[f"l{i}.mix.left.q"] == (l["heads"] * l["dim"], W)
            assert names[f"l{i}.mix.left.k"] == (l["kv_heads"] * l["dim"], W)
            assert names[f"l{i}.mix.left.v"] == (l["kv_heads"] * l["vdim"], W)
            assert names[f"l{i}.mix.left.v.conv"] == (l["kv_heads"] * l["vdim"], l["conv"])
            assert names[f"l{i}.mix.left.g"] == (l["heads"], W) and names[f"l{i}.mix.left.o.b"] == (W,)
            assert names[f"l{i}.mix.right.norm"] == (r["heads"] * r["vdim"],)
            assert names[f"l{i}.mix.right.o"] == (W, r["heads"] * r["vdim"])
        else:
            assert names[f"l{i}.mix.q"] == (m["kv_heads"] * m["dim"], W) and names[f"l{i}.mix.v"] == (m["heads"] * m["vdim"], W)
            assert names[f"l{i}.mix.A_log"] == (m["heads"],) and names[f"l{i}.mix.norm"] == (m["vdim"],)
            assert names[f"l{i}.mix.b"] == (m["heads"], W)
        assert (f"l{i}.mlp.down" in names) == (L["mlp"] is not None) == (f"l{i}.norm2" in names)
    # the run order: every pass of a loop is an entry with a cache of its own, later passes take the embedding in again
    order = [(st.layer, st.add_embedding) for st in model.order]
    assert order == P.run_order(raw)
    needs = model.cache_needs()
    assert len(needs) == len(order) and all(n is not None for n in needs)


def test_loop_of_one_pass_and_no_loop_are_the_same_order():
    raw = GOPITAR["b"]()
    raw["loop"] = {"start": 0, "stop": 2, "times": 1}
    assert [st.layer for st in __import__("infinilm_b200.models.gopitar", fromlist=["run_order"]).run_order(_cfg(raw))] == [0, 1, 2]
    assert P.run_order(raw) == [(0, False), (1, False), (2, False)]


def test_bad_configs_are_refused():
    from infinilm_b200.config.model_config import ConfigError
    raw = GOPITAR["a"]()
    raw["layers"][0]["type"] = "other"
    with pytest.raises(ConfigError):
        _cfg(raw)
    raw = GOPITAR["a"]()
    raw["layers"][1]["mixer"]["right"]["decay"] = [0.5]
    with pytest.raises(ConfigError):
        _cfg(raw)
    raw = GOPITAR["a"]()
    raw["loop"] = {"start": 2, "stop": 9, "times": 2}
    with pytest.raises(ConfigError):
        _cfg(raw)


def test_random_folder_round_trip(tmp_path):
    from infinilm_b200.config.registry import load_config
    from infinilm_b200.weights import write_model_folder
    from infinilm_b200.weights.safetensors_io import SafetensorsFile
    raw = GOPITAR["c"]()
    out = write_model_folder(_cfg(raw), 3, str(tmp_path / "m"))
    cfg = load_config(out)
    assert cfg.layers == _cfg(raw).layers and cfg.logit_softcap == raw["logit_softcap"]
    f = SafetensorsFile(os.path.join(out, "model.safetensors"))
    assert "l0.mix.left.q.conv" in f.names() and "l2.mix.dt_bias" in f.names()
    f.close()


def test_plain_convolution_continues_from_its_last_inputs():
    torch.manual_seed(0)
    u, w = torch.randn(23, 5, dtype=torch.float64), torch.randn(5, 4, dtype=torch.float64)
    whole = P.short_conv(u, w)
    for cut in (1, 2, 3, 10, 22):
        tail = P.short_conv(torch.cat([u[max(0, cut - 3):cut], u[cut:]]), w)[min(cut, 3):]
        assert torch.allclose(tail, whole[cut:], atol=1e-12)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (3, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(whole, ref, atol=1e-12)


def test_plain_recurrences_equal_their_closed_forms():
    torch.manual_seed(1)
    T, H, d, dv = 9, 2, 3, 4
    q, k, v = (torch.randn(T, H, n, dtype=torch.float64) for n in (d, d, dv))
    decay = torch.tensor([0.5, 0.9], dtype=torch.float64)
    o = P.decayed_linear_attention(q, k, v, decay)
    for t in range(T):
        for h in range(H):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(o[t, h], want, atol=1e-12)
    # the delta rule with beta = 1, g = 1 and orthonormal keys stores and returns values exactly
    k = torch.eye(3, dtype=torch.float64)[:, None, :].repeat(1, 1, 1)
    v = torch.randn(3, 1, dv, dtype=torch.float64)
    o = P.gated_delta_rule(k, k, v, torch.ones(3, 1, dtype=torch.float64), torch.ones(3, 1, dtype=torch.float64))
    assert torch.allclose(o, v, atol=1e-12)


def test_zero_columns_change_no_score():
    torch.manual_seed(2)
    T, H, d, dv = 7, 2, 5, 3
    q, k, v = torch.randn(T, H, d, dtype=torch.float64), torch.randn(T, 1, d, dtype=torch.float64), torch.randn(T, 1, dv, dtype=torch.float64)
    a = P.window_softmax_attention(q, k, v, 0.3, 4)
    pad = lambda x, n: torch.cat([x, torch.zeros(*x.shape[:-1], n - x.shape[-1], dtype=x.dtype)], -1)   # noqa: E731
    b = P.window_softmax_attention(pad(q, 16), pad(k, 16), pad(v, 16), 0.3, 4)[..., :dv]
    assert torch.allclose(a, b, atol=1e-12)
    # a window of w sees exactly w keys: the token itself and the w - 1 before it
    q0 = torch.zeros(T, 1, 1, dtype=torch.float64)
    ones = torch.ones(T, 1, 1, dtype=torch.float64)
    idx = torch.arange(T, dtype=torch.float64).view(T, 1, 1)
    mean_pos = P.window_softmax_attention(q0, ones, idx, 1.0, 3)[:, 0, 0]
    assert torch.allclose(mean_pos, torch.tensor([0, 0.5, 1, 2, 3, 4, 5], dtype=torch.float64))


def test_plain_forward_runs_every_configuration():
    for name in sorted(GOPITAR):
        raw = GOPITAR[name]()
        lg = P.forward(raw, make_weights(raw, 5), token_ids(12, raw["vocab"], 1))
        assert lg.shape == (12, raw["vocab"]) and torch.isfinite(lg).all()
        if raw.get("logit_softcap"):
            assert float(lg.abs().max()) <= raw["logit_softcap"]
