"""Nirozen on the CPU: configuration, run order, tensor names, the random-weights folder, and the oracle's own
identities (the rewriting that the package's mixer rests on is checked against the oracle's direct form)."""
import json
import os

import pytest
import torch

import plain_nirozen as P
from nirozen_configs import NIROZEN, make_weights, token_ids

from infinilm_b200.config import ConfigError, config_from_json, describe_model
from infinilm_b200.models.causal_lm import CausalLM
from infinilm_b200.weights import FolderSource, check_against, write_model_folder


@pytest.mark.parametrize("name", sorted(NIROZEN))
def test_run_order_matches_the_oracle(name):
    raw = NIROZEN[name]()
    spec = describe_model(config_from_json(raw))
    assert [(s.layer, s.add_row) for s in spec.order] == P.run_order(raw)
    assert all(s.cache_from is None for s in spec.order)            # every pass keeps a cache of its own
    assert (spec.pass_vectors is not None) == bool(raw.get("loop"))


def test_loop_that_is_empty_or_runs_once():
    raw = NIROZEN["a"]()
    raw["loop"] = {"start": 1, "stop": 1, "times": 5}
    spec = describe_model(config_from_json(raw))
    assert [s.layer for s in spec.order] == [0, 1, 2] and spec.pass_vectors is None
    raw["loop"] = {"start": 0, "stop": 3, "times": 1}
    spec = describe_model(config_from_json(raw))
    assert [(s.layer, s.add_row) for s in spec.order] == [(0, 0), (1, None), (2, None)]


@pytest.mark.parametrize("name", sorted(NIROZEN))
def test_tensor_names_and_cache_needs(name):
    raw = NIROZEN[name]()
    model = CausalLM(describe_model(config_from_json(raw)), torch.float32)
    names = {p.full_name(ws.name): ws.shape for p, ws in model.weight_specs()}
    W = raw["width"]
    assert names["embed"] == (raw["vocab"], W) and names["head"] == (raw["vocab"], W) and names["final.norm"] == (W,)
    assert names["bigram"] == (raw["embedding"]["bigram"]["buckets"] + 1, W)
    for i, L in enumerate(raw["layers"]):
        m = L["mixer"]
        assert names[f"l{i}.mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"]) and names[f"l{i}.mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
        assert names[f"l{i}.mix.sink"] == (m["heads"],) and names[f"l{i}.mix.g"] == (m["heads"] * m["vdim"], W)
        assert (f"l{i}.norm2" in names) == (L["mlp"] is not None)
        if L["mlp"]:
            assert names[f"l{i}.mlp.router.b"] == (L["mlp"]["router"]["experts"],)
            assert (f"l{i}.mlp.shared.up" in names) == (L["mlp"]["shared"] is not None)
    needs = model.cache_needs()
    assert len(needs) == len(model.order) + 1 and needs[-1].kind == "state" and needs[-1].dtype == "int32"
    for st, need in zip(model.order, needs):
        assert need.kind == "paged_kv" and need.n_kv_heads == 1 and need.head_dim == raw["layers"][st.layer]["mixer"]["kv_rank"]


def test_config_faults_name_the_key():
    raw = NIROZEN["a"]()
    raw["layers"][0]["type"] = "something_else"
    with pytest.raises(ConfigError, match="something_else"):
        config_from_json(raw)
    raw = NIROZEN["a"]()
    del raw["layers"][1]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError, match="kv_rank"):
        config_from_json(raw)
    raw = NIROZEN["a"]()
    raw["loop"] = {"start": 2, "stop": 5, "times": 2}
    with pytest.raises(ConfigError, match="loop"):
        config_from_json(raw)


def test_random_folder_round_trip(tmp_path):
    raw = NIROZEN["b"]()
    cfg = config_from_json(raw)
    d = write_model_folder(cfg, 3, str(tmp_path / "m"))
    assert json.load(open(os.path.join(d, "config.json"))) == raw
    model = CausalLM(describe_model(cfg), torch.bfloat16)
    src = FolderSource(d)
    check_against(model, src)
    src.close()


def test_oracle_first_token_and_pair_rows():
    raw = NIROZEN["a"]()
    w = make_weights(raw, 0)
    ids = [5, 9, 5, 9]
    b = raw["embedding"]["bigram"]
    rows = P.bigram_rows(raw, w, ids)
    assert torch.equal(rows[0], w["bigram"][b["buckets"]].double())
    assert torch.equal(rows[1], w["bigram"][(5 * b["mul_prev"] + 9 * b["mul_cur"]) % b["buckets"]].double())
    assert torch.equal(rows[3], rows[1]) and not torch.equal(rows[2], rows[1])
    s = P.sinusoid_rows(6, 3)
    assert torch.allclose(s[0], torch.tensor([0., 1., 0., 1., 0., 1.], dtype=torch.float64))
    assert abs(float(s[2, 2]) - float(torch.sin(torch.tensor(2.0 * 10000.0 ** (-2.0 / 6.0), dtype=torch.float64)))) < 1e-12


def test_oracle_sink_limits():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(5, 4, generator=g, dtype=torch.float64) for _ in range(3))
    plain = torch.softmax((q @ k.t() * 0.5).masked_fill(torch.ones(5, 5, dtype=torch.bool).triu(1), float("-inf")), dim=1) @ v
    assert torch.allclose(P.sink_softmax_attention(q, k, v, 0.5, torch.tensor(-1e9, dtype=torch.float64)), plain)       # no sink
    assert P.sink_softmax_attention(q, k, v, 0.5, torch.tensor(60.0, dtype=torch.float64)).abs().max() < 1e-20          # all mass on the sink
    half = P.sink_softmax_attention(q[:1], k[:1], v[:1], 0.5, (q[0] @ k[0] * 0.5).reshape(()))                          # sink = the only score
    assert torch.allclose(half, 0.5 * v[:1])


def test_attention_against_the_latents_equals_the_direct_form():
    """q.(W_uk c) = (W_uk^T q).c and sum p_i W_uv c_i = W_uv sum p_i c_i: what the package's mixer computes, checked with
    the oracle's one-head attention on both sides."""
    raw = NIROZEN["b"]()
    w = make_weights(raw, 1)
    m, p, eps = raw["layers"][1]["mixer"], "l1.mix", raw["norm"]["eps"]
    g = torch.Generator().manual_seed(2)
    h = torch.randn(9, raw["width"], generator=g, dtype=torch.float64)
    direct = P.latent_attention(m, w, p, h, eps)
    H, d, e = m["heads"], m["dim"], m["vdim"]
    cq = P.plain_norm(h @ w[f"{p}.dq"].double().t(), w[f"{p}.dq.norm"].double(), eps)
    q = cq @ w[f"{p}.uq"].double().t()
    c = P.plain_norm(h @ w[f"{p}.dkv"].double().t(), w[f"{p}.dkv.norm"].double(), eps)
    heads = []
    for j in range(H):
        uk, uv = w[f"{p}.uk"].double()[j * d:(j + 1) * d], w[f"{p}.uv"].double()[j * e:(j + 1) * e]
        o_lat = P.sink_softmax_attention(q[:, j * d:(j + 1) * d] @ uk, c, c, m["scale"], w[f"{p}.sink"].double()[j])
        heads.append(o_lat @ uv.t())
    o = torch.cat(heads, 1) * torch.sigmoid(h @ w[f"{p}.g"].double().t())
    assert torch.allclose(o @ w[f"{p}.o"].double().t(), direct, rtol=1e-10, atol=1e-12)


def test_oracle_routing_weights():
    raw = NIROZEN["b"]()
    w = make_weights(raw, 4)
    h = torch.randn(6, raw["width"], generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    idx, wt, z = P.route(raw["layers"][0]["mlp"], w, "l0.mlp", h)
    assert idx.shape == (6, 3) and torch.allclose(wt.sum(1), torch.ones(6, dtype=torch.float64))
    for t in range(6):
        chosen = z[t][idx[t]]
        assert chosen.min() >= z[t].sort().values[-3] - 1e-12
        assert torch.allclose(wt[t], torch.exp(chosen) / torch.exp(chosen).sum())
