"""Nirozen through the engine against the oracle under every way of cutting the work: whole prompts; a prompt and then
its last tokens one by one (long decoding, also replayed as graphs); portions of changing size down to two tokens;
up to four live requests mixed, unequal, with so few pages and state slots that both are used again; and greedy
generation through `LLM.generate` and the scheduler. float32 compares every position sharply. bfloat16 compares
position by position where no discrete choice can turn under rounding (configuration d chooses every expert), and up to
the first close routing call elsewhere."""
import warnings

import pytest
import torch

import plain_nirozen as P
from nirozen_configs import NIROZEN, make_weights, token_ids

pytestmark = pytest.mark.gpu

TOL = {"float32": 4e-5, "bfloat16": 5e-2}
LENGTHS = {"a": [1, 2, 17, 70, 130], "b": [3, 33, 100], "c": [5, 48, 90], "d": [4, 65, 300], "e": [2, 50, 60]}


def _engine(raw, w, dtype, num_pages=48, max_seqs=4, max_batch_tokens=512):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        return Engine.from_tensors(config_from_json(raw), w, dtype=dtype, page_size=16, num_pages=num_pages, max_seqs=max_seqs,
                                   max_batch_tokens=max_batch_tokens)


_oracle_cache = {}


def _oracle(name, seed, ids):
    """(logits, number of leading positions without a close routing call)."""
    key = (name, seed, tuple(ids))
    if key not in _oracle_cache:
        raw = NIROZEN[name]()
        margins = []
        lg = P.forward(raw, make_weights(raw, seed), ids, margins=margins)
        sure = len(ids)
        if margins:
            per_run = len(margins) // len(ids)
            m = torch.tensor(margins).view(per_run, len(ids)).amin(0)
            close_calls = torch.nonzero(m < 0.08)
            if close_calls.numel():
                sure = int(close_calls[0])
        _oracle_cache[key] = (lg, sure)
    return _oracle_cache[key]


def _check(got, name, seed, ids, dtype, what):
    ref, sure = _oracle(name, seed, ids)
    n = len(ids) if dtype == "float32" else sure
    got, ref = got.double().cpu()[:n], ref[:n]
    assert torch.isfinite(got).all(), what
    err = ((got - ref).abs() / ref.abs().amax(dim=-1, keepdim=True)).amax(dim=-1)
    bad = torch.nonzero(err > TOL[dtype])
    # float32: every position. bfloat16: the tests' weights make attention peaked and the branches large, so a few positions
    # carry several roundings at once: at most one position in 25 may pass the bound, none may pass three times the bound.
    allowed = 0 if dtype == "float32" else n // 25
    worst = float(err.max()) if n else 0.0
    assert bad.numel() <= allowed and (dtype == "float32" or worst <= 3 * TOL[dtype]), \
        f"{what}: first wrong position {int(bad[0])} of {n} (rel err {float(err[int(bad[0])]):.2e}, worst {worst:.2e}, {bad.numel()} wrong)"


def _run_cut(eng, ids, cuts, seq_id="r"):
    from infinilm_b200.engine import StepEntry
    assert sum(cuts) == len(ids)
    seq, outs, a = eng.open(seq_id), [], 0
    for c in cuts:
        outs.append(eng.step([StepEntry(seq, ids[a:a + c], list(range(c)))]).clone())
        a += c
    eng.close(seq)
    return torch.cat(outs, 0)


def _run_schedule(eng, requests, schedule):
    from infinilm_b200.engine import StepEntry
    done, seqs, outs = {k: 0 for k in requests}, {}, {k: [] for k in requests}
    for step in schedule:
        entries = []
        for rid, n in step:
            if rid not in seqs:
                seqs[rid] = eng.open(rid)
            entries.append(StepEntry(seqs[rid], requests[rid][done[rid]:done[rid] + n], list(range(n))))
            done[rid] += n
        logits, r = eng.step(entries).clone(), 0
        for rid, n in step:
            outs[rid].append(logits[r:r + n])
            r += n
            if done[rid] == len(requests[rid]):
                eng.close(seqs.pop(rid))
        eng.cache.check_invariants()
    assert all(done[k] == len(requests[k]) for k in requests)
    return {k: torch.cat(v, 0) for k, v in outs.items()}


CASES = [("a", 0), ("b", 1), ("c", 2), ("d", 3), ("e", 4)]
DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_whole_prompts(cuda_device, name, seed, dtype):
    raw = NIROZEN[name]()
    eng = _engine(raw, make_weights(raw, seed), dtype)
    for n in LENGTHS[name]:
        ids = token_ids(n, raw["vocab"], 100 + n)
        _check(_run_cut(eng, ids, [n]), name, seed, ids, dtype, f"{name} whole prompt of {n}")
    eng.synchronize()
    eng.cache.check_invariants()


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_prompt_then_token_by_token(cuda_device, name, seed, dtype, graphs):
    """Prefill against decoding through the cache: the last 40 tokens one by one; and a sequence decoded from its very
    first token on."""
    raw = NIROZEN[name]()
    eng = _engine(raw, make_weights(raw, seed), dtype)
    if graphs:
        eng.enable_graphs()
    n = LENGTHS[name][-1]
    ids = token_ids(n, raw["vocab"], 100 + n)
    _check(_run_cut(eng, ids, [n - 40] + [1] * 40), name, seed, ids, dtype, f"{name} {n - 40} + 40 single tokens")
    ids = token_ids(36, raw["vocab"], 136)
    _check(_run_cut(eng, ids, [1] * 36), name, seed, ids, dtype, f"{name} 36 single tokens from the start")
    eng.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_portions_of_changing_size(cuda_device, name, seed, dtype):
    raw = NIROZEN[name]()
    eng = _engine(raw, make_weights(raw, seed), dtype)
    n = LENGTHS[name][-1]
    ids = token_ids(n, raw["vocab"], 100 + n)
    for pattern in ([16, 7, 2, 5, 3, 17, 2, 1, 31, 2, 9], [2], [15, 1, 16, 17, 1, 1, 33]):
        cuts, left, i = [], n, 0
        while left > 0:
            cuts.append(min(pattern[i % len(pattern)], left))
            left -= cuts[-1]
            i += 1
        _check(_run_cut(eng, ids, cuts), name, seed, ids, dtype, f"{name} portions {cuts[:6]}...")
    eng.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_mixed_requests_pages_and_slots_used_again(cuda_device, name, seed, dtype):
    """Unequal requests side by side, portions of some beside single tokens of others, in a pool of 12 pages and 3 state
    slots: finished requests give theirs back and later ones get them (uncleared)."""
    raw = NIROZEN[name]()
    V = raw["vocab"]
    eng = _engine(raw, make_weights(raw, seed), dtype, num_pages=12, max_seqs=3)
    req = {"p": token_ids(70, V, 31), "q": token_ids(33, V, 32), "r": token_ids(2, V, 33), "s": token_ids(90, V, 34), "t": token_ids(1, V, 35),
           "u": token_ids(47, V, 36)}
    schedule = [[("p", 20), ("q", 1), ("r", 2)],           # r ends: its slot and page go back
                [("p", 2), ("q", 30), ("t", 1)],           # t takes them, and ends
                [("q", 2), ("p", 16)],                     # q ends
                [("p", 1), ("u", 17)]] + [[("p", 1), ("u", 2)]] * 15 + [[("p", 16)]]      # p ends at 70: five pages back
    schedule += [[("s", 50)]] + [[("s", 1)]] * 38 + [[("s", 2)]]          # s runs alone in pages that p, q and u held
    got = _run_schedule(eng, req, schedule)
    for k, ids in req.items():
        _check(got[k], name, seed, ids, dtype, f"{name} mixed, request {k}")
        alone = _run_cut(eng, ids, [len(ids)], seq_id=k + "_alone")
        d = (got[k].float() - alone.float()).abs().amax() / alone.float().abs().amax()
        if dtype == "float32":
            assert float(d) < 1e-5, f"request {k} in the mix against alone: {float(d):.2e}"
    eng.synchronize()
    eng.cache.check_invariants()
    assert eng.cache.free_pages() == {g: 12 for g in eng.cache.free_pages()}


def _lookup_weights(raw, w, ids, where):
    """Head 0 of layer 0 turned into a lookup: the query of the last token of `ids` is made to point at the latent of
    token `where`, whose score then stands 15 above zero while the others scatter around it by a few units."""
    eps, m, p = raw["norm"]["eps"], raw["layers"][0]["mixer"], "l0.mix"
    x = P.embedding(raw, w, ids)
    if P.run_order(raw)[0][1] is not None:
        x = x + w["loop.step"][0].double()
    h = P.offset_norm(x, w["l0.norm1"].double(), eps)
    c = P.plain_norm(h @ w[f"{p}.dkv"].double().t(), w[f"{p}.dkv.norm"].double(), eps)
    cq = P.plain_norm(h @ w[f"{p}.dq"].double().t(), w[f"{p}.dq.norm"].double(), eps)
    d = m["dim"]
    target = w[f"{p}.uk"].double()[:d] @ c[where]
    uq = w[f"{p}.uq"].double().clone()
    uq[:d] = torch.outer(target, cq[-1]) * (15.0 / (m["scale"] * float(target @ target) * float(cq[-1] @ cq[-1])))
    out = dict(w)
    out[f"{p}.uq"] = uq.to(torch.bfloat16)
    out[f"{p}.sink"] = torch.full_like(w[f"{p}.sink"], -2.0)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", [("a", 0), ("d", 3)])
def test_far_token_decides(cuda_device, name, seed, dtype):
    """A prompt whose last position looks one early token up (first of the sequence, last of a page, first of the next,
    the one after): the logits there change when that token changes, in the oracle and in the engine alike, whether
    the last position comes in a prompt, in a portion of two, or decoded after forty single tokens."""
    raw = NIROZEN[name]()
    base = token_ids(200, raw["vocab"], 77)
    for where in (0, 15, 16, 17):
        w = _lookup_weights(raw, make_weights(raw, seed), base, where)
        eng = _engine(raw, w, dtype)
        other = list(base)
        other[where] = (other[where] + 1) % raw["vocab"]
        ref_a, ref_b = P.forward(raw, w, base)[-1], P.forward(raw, w, other)[-1]
        moved = float((ref_a - ref_b).abs().max() / ref_a.abs().max())
        assert moved > 0.01, f"the test's weights do not carry token {where} to the end ({moved:.1e})"
        for ids, ref in ((base, ref_a), (other, ref_b)):
            for cuts in ([200], [198, 2], [160] + [1] * 40):
                got = _run_cut(eng, ids, cuts)[-1].double().cpu()
                err = float((got - ref).abs().max() / ref.abs().max())
                assert err < (TOL[dtype] if dtype == "float32" else max(TOL[dtype], 0.3 * moved)), f"token {where}, cuts {cuts[:2]}: {err:.2e} (the token moves {moved:.2e})"
        eng.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", [("a", 0), ("d", 3)])
def test_greedy_generation_through_llm(cuda_device, name, seed, dtype):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.llm import LLM, SamplingParams
    raw = NIROZEN[name]()
    w = make_weights(raw, seed)
    prompts = [token_ids(n, raw["vocab"], 50 + n) for n in (1, 19, 40)]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        llm = LLM.from_tensors(config_from_json(raw), w, dtype=dtype, num_blocks=24, block_size=16, max_batch_size=2, chunk_size=16,
                               enable_graph=True)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(top_k=1, max_tokens=12, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        tokens = out.outputs[0].token_ids
        assert len(tokens) == 12
        ids = list(prompt)
        for i, t in enumerate(tokens):                             # each token is the oracle's choice wherever that is clear
            lg = P.forward(raw, w, ids)[-1]
            top2 = torch.topk(lg, 2).values
            if dtype == "float32" or float(top2[0] - top2[1]) > 4 * TOL[dtype] * float(lg.abs().max()):
                assert t == int(torch.argmax(lg)), f"prompt of {len(prompt)}, token {i}: {t} != {int(torch.argmax(lg))}"
            ids.append(t)
    llm.close()


def test_command_line_on_a_random_folder(cuda_device, tmp_path, capsys):
    """The package's command line: write a folder of random weights for a configuration, then generate from it."""
    import json

    from infinilm_b200 import cli
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(NIROZEN["b"]()))
    folder = str(tmp_path / "m")
    assert cli.main(["--write-random-model", folder, "--config", str(cfg_path), "--seed", "3"]) == 0
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        rc = cli.main(["--model", folder, "--enable-paged-attn", "--block-size", "16", "--num-blocks", "32", "--prompt-len", "21",
                       "--max-new-tokens", "9", "--batch-size", "2", "--ignore-eos", "--enable-graph", "--log-level", "ERROR"])
    assert rc == 0


def test_trace_replay_as_a_process(cuda_device, tmp_path):
    """`bin/trace_run` on a folder of random weights, float32: five requests through four state slots and a pool of 192
    tokens, a request left out of a step, portions beside single tokens, steps in which nothing is wanted."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    from infinilm_b200.config import config_from_json
    from infinilm_b200.weights import random_tensors, write_model_folder
    raw = NIROZEN["a"]()
    cfg = config_from_json(raw)
    folder = write_model_folder(cfg, 9, str(tmp_path / "m"))
    w = random_tensors(cfg, 9, "cpu")
    V = raw["vocab"]
    seqs = {k: token_ids(n, V, 60 + n) for k, n in (("p", 40), ("q", 3), ("r", 1), ("s", 18), ("t", 33))}
    steps = [
        {"step": 0, "entries": [{"id": "p", "tokens": seqs["p"][:17], "want": [0, 16]}, {"id": "q", "tokens": seqs["q"][:2], "want": []},
                                {"id": "r", "tokens": seqs["r"], "want": [0]}, {"id": "s", "tokens": seqs["s"][:16], "want": [15]}], "end": ["r"]},
        {"step": 1, "entries": [{"id": "q", "tokens": seqs["q"][2:], "want": [0]}, {"id": "s", "tokens": seqs["s"][16:17], "want": [0]}], "end": ["q"]},
        {"step": 2, "entries": [{"id": "t", "tokens": seqs["t"][:31], "want": []}, {"id": "p", "tokens": seqs["p"][17:19], "want": [1]},
                                {"id": "s", "tokens": seqs["s"][17:], "want": [0]}], "end": ["s"]},
        {"step": 3, "entries": [{"id": "t", "tokens": seqs["t"][31:32], "want": [0]}, {"id": "p", "tokens": seqs["p"][19:], "want": [0, 20]}], "end": ["p"]},
        {"step": 4, "entries": [{"id": "t", "tokens": seqs["t"][32:], "want": [0]}], "end": ["t"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out_dir),
                           "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [x for i in range(5) for x in ("done", str(i))]
    ref = {k: P.forward(raw, w, ids) for k, ids in seqs.items()}
    want = {0: [ref["p"][0], ref["p"][16], ref["r"][0], ref["s"][15]], 1: [ref["q"][2], ref["s"][16]], 2: [ref["p"][18], ref["s"][17]],
            3: [ref["t"][31], ref["p"][19], ref["p"][39]], 4: [ref["t"][32]]}
    for step, rows in want.items():
        got = torch.from_numpy(np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(-1, V)).double()
        r = torch.stack(rows)
        assert float(((got - r).abs() / r.abs().amax(dim=-1, keepdim=True)).max()) < TOL["float32"], f"step {step}"
