"""Nirozen's mechanisms one at a time, each kernel or part against the oracle's function for it (float64 on the CPU),
at sizes of the tests' own: the embedding with its hashed pair row, sinusoid and previous-token state; the norm with
a weight offset and an added vector; the router; products over ragged groups and over heads; the routed feed-forward;
attention with a sink in every kernel that has one (plain, split-KV decode, mma.sync prefill, tensor-memory prefill),
with inputs built so that a fault shows: one far key that outweighs the rest, keys at page borders, a sink that
dominates or vanishes; and the latent-attention mixer as a whole."""
import math

import pytest
import torch

import plain_nirozen as P
from nirozen_configs import NIROZEN, make_weights, token_ids

pytestmark = pytest.mark.gpu

from infinilm_b200 import ops  # noqa: E402

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 2.5e-2}


def close(got, ref, dtype, what="", tol=None):
    tol = TOL[dtype] if tol is None else tol
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    got, ref = got.reshape(-1, got.shape[-1]), ref.reshape(-1, ref.shape[-1])
    err = ((got - ref).abs() / ref.abs().amax(dim=-1, keepdim=True).clamp_min(1e-6)).amax(dim=-1)
    bad = torch.nonzero(~(err <= tol))
    assert bad.numel() == 0, f"{what} row {int(bad[0])}: rel err {float(err[int(bad[0])]):.3e} > {tol:.1e} ({bad.numel()} of {err.numel()} rows)"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


# ---- embedding -----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "c"])
def test_embedding_rows_and_previous_token_state(cuda_device, dtype, name):
    raw = NIROZEN[name]()
    w = make_weights(raw, 5)
    V, W, b = raw["vocab"], raw["width"], raw["embedding"]["bigram"]
    seq0, seq1 = token_ids(9, V, 1), token_ids(30, V, 2)
    table, pair = w["embed"].to(DT[dtype]).cuda(), w["bigram"].to(DT[dtype]).cuda()
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange((W + 1) // 2, dtype=torch.float64) / W).float().cuda()
    state = torch.zeros(5, dtype=torch.int32, device="cuda")
    ref0, ref1 = P.embedding(raw, w, seq0), P.embedding(raw, w, seq1)

    def run(parts, read, write):
        """parts: [(tokens, first position)] one entry each."""
        ids = [t for p, _ in parts for t in p]
        pos = [s + i for p, s in parts for i in range(len(p))]
        ent = [e for e, (p, _) in enumerate(parts) for _ in p]
        qs = [0]
        for p, _ in parts:
            qs.append(qs[-1] + len(p))
        out = torch.empty(len(ids), W, device="cuda")
        ops.embed_pair_pos(i32(ids), i32(pos), i32(ent), i32(qs), table, raw["embedding"]["scale"], pair, b["buckets"], b["mul_prev"],
                           b["mul_cur"], state, i32(read), i32(write), inv, out)
        return out.cpu()
    # step 1: the first 4 tokens of seq0 (fresh: reads the zero slot, writes slot 2) beside the first token of seq1 (slot 3)
    out = run([(seq0[:4], 0), (seq1[:1], 0)], [0, 0], [2, 3])
    close(out[:4], ref0[:4], "float32", "first portion")
    close(out[4:], ref1[:1], "float32", "a sequence's first token")
    assert state.tolist() == [0, 0, seq0[3] + 1, seq1[0] + 1, 0]
    # step 2: one token of seq0 (decoding) beside 20 of seq1; step 3: two tokens and nine
    out = run([(seq0[4:5], 4), (seq1[1:21], 1)], [2, 3], [2, 3])
    close(out[:1], ref0[4:5], "float32", "single token after a portion")
    close(out[1:], ref1[1:21], "float32", "portion after a single token")
    out = run([(seq1[21:30], 21), (seq0[5:7], 5)], [3, 2], [3, 2])
    close(out[:9], ref1[21:30], "float32"), close(out[9:], ref0[5:7], "float32", "a portion of two")
    assert state.tolist() == [0, 0, seq0[6] + 1, seq1[29] + 1, 0]
    # a new request in a slot that was used: it reads the zero slot, so nothing of the old one shows
    out = run([(seq1[:3], 0)], [0], [2])
    close(out, ref1[:3], "float32", "slot used again")


# ---- norm ----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,W", [(1, 96), (19, 100), (3, 4100)])
def test_offset_norm_with_added_vector(cuda_device, dtype, T, W):
    from infinilm_b200.parts.norms import RMSNorm
    g = torch.Generator().manual_seed(T)
    resid, branch = torch.randn(T, W, generator=g) * 4, torch.randn(T, W, generator=g).to(DT[dtype])
    vec, wt = torch.randn(W, generator=g), (torch.randn(W, generator=g) * 0.2).bfloat16()
    norm = RMSNorm({"size": W, "eps": 1e-4, "weight_offset": 1.0, "name": "n"}, "x", DT[dtype])
    norm.set_weights({"n": wt.cuda()})
    r = resid.cuda()
    out = norm.add_norm(r, branch.cuda(), 1.0, torch.empty(T, W, device="cuda", dtype=DT[dtype]), vec=vec.cuda())
    x = resid.double() + branch.double() + vec.double()
    close(out, P.offset_norm(x, wt.double(), 1e-4), dtype)
    assert torch.allclose(r.cpu().double(), x, atol=1e-5)
    rows = i32([T - 1, 0])
    out2 = norm.add_norm(r, None, 1.0, torch.empty(2, W, device="cuda", dtype=DT[dtype]), rows=rows)
    close(out2, P.offset_norm(x[[T - 1, 0]], wt.double(), 1e-4), dtype)


# ---- router --------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,top,W", [(5, 2, 96), (7, 1, 160), (4, 4, 100), (64, 6, 72), (130, 32, 64)])
def test_router_against_the_oracle(cuda_device, E, top, W):
    g = torch.Generator().manual_seed(E)
    w = {"r.router": (torch.randn(E, W, generator=g) * 0.3).bfloat16(), "r.router.b": (torch.randn(E, generator=g)).bfloat16()}
    h = torch.randn(41, W, generator=g)
    idx_ref, wt_ref, _ = P.route({"router": {"top": top}}, w, "r", h.double())
    idx = torch.empty(41, top, dtype=torch.int32, device="cuda")
    wt = torch.empty(41, top, dtype=torch.float32, device="cuda")
    ops.moe_route(h.cuda(), w["r.router"].float().cuda(), w["r.router.b"].cuda(), idx, wt, top)
    assert torch.equal(idx.cpu().long(), idx_ref)                  # in the order of the logits, largest first
    assert torch.allclose(wt.cpu().double(), wt_ref, atol=2e-6)


@pytest.mark.parametrize("E,top,T", [(5, 2, 300), (64, 6, 41), (130, 32, 9), (9, 9, 17), (1, 1, 8)])
def test_choice_from_given_logits(cuda_device, E, top, T):
    """The choosing kernel alone (long portions in bfloat16 take their logits from a matrix product): rows of a wider
    buffer, the bias added here, the order of the choices, ties, the softmax over the chosen."""
    g = torch.Generator().manual_seed(E + T)
    z = torch.randn(T, E + 3, generator=g)[:, :E]
    z[T // 2] = z[T // 2].round()                                   # ties: the lower expert comes first
    b = torch.randn(E, generator=g).bfloat16()
    zz = (z + b.float()[None]).double()                             # the kernel adds the bias in float32
    order = torch.argsort(zz, dim=1, descending=True, stable=True)[:, :top]
    wt_ref = torch.softmax(torch.gather(zz, 1, order), dim=1)
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wt = torch.empty(T, top, dtype=torch.float32, device="cuda")
    zc = torch.zeros(T, E + 3, device="cuda")
    zc[:, :E] = z.cuda()
    ops.moe_select(zc[:, :E], b.cuda(), idx, wt, top)
    assert torch.equal(idx.cpu().long(), order)
    assert torch.allclose(wt.cpu().double(), wt_ref, atol=2e-6)


@pytest.mark.parametrize("E,top,W,T", [(64, 6, 2048, 8), (5, 2, 96, 1), (7, 7, 160, 16), (130, 32, 72, 3), (16, 4, 4088, 13)])
@pytest.mark.parametrize("unfinished", [False, True])
def test_router_of_a_few_rows_as_two_kernels(cuda_device, E, top, W, T, unfinished):
    """A decode step's router (logits a warp per token and expert, then one block that chooses and sorts) against the
    oracle and against the sort kernel; also on rows whose norm is unfinished, where it leaves rstd per row."""
    g = torch.Generator().manual_seed(E + T)
    w = {"r.router": (torch.randn(E, W, generator=g) * 0.3).bfloat16(), "r.router.b": (torch.randn(E, generator=g)).bfloat16()}
    resid = torch.randn(T, W, generator=g) * (2.0 if unfinished else 1.0)
    xw = resid.bfloat16()
    eps = 1e-5
    rstd_ref = torch.rsqrt((resid.double() ** 2).mean(-1, keepdim=True) + eps) if unfinished else torch.ones(T, 1, dtype=torch.float64)
    idx_ref, wt_ref, z_ref = P.route({"router": {"top": top}}, w, "r", xw.double() * rstd_ref)
    srt = z_ref.sort(dim=1, descending=True).values
    sure = ((srt[:, :top] - srt[:, 1:top + 1]).amin(1) > 1e-4) if top < E else ((srt[:, :-1] - srt[:, 1:]).amin(1) > 1e-4)
    dev = dict(device="cuda")
    idx, wt = torch.empty(T, top, dtype=torch.int32, **dev), torch.empty(T, top, dtype=torch.float32, **dev)
    z = torch.empty(T, E, **dev)
    group_off, pos, row = torch.empty(E + 1, dtype=torch.int32, **dev), torch.empty(T * top, dtype=torch.int32, **dev), torch.empty(T * top, dtype=torch.int32, **dev)
    norm_in, rstd = None, None
    if unfinished:
        pad = (-W) % 16
        sumsq = torch.nn.functional.pad(resid * resid, (0, pad)).view(T, -1, 16).sum(-1)
        norm_in, rstd = ops.NormedInput(xw.cuda(), sumsq.cuda().contiguous(), W, eps), torch.empty(T, **dev)
    assert ops.route_sort_small_ok(T, W, E)
    ops.moe_route_sort_small(xw.cuda(), w["r.router"].cuda(), w["r.router.b"].cuda(), z, idx, wt, top, group_off, pos, row, norm_in=norm_in, rstd_out=rstd)
    assert torch.allclose(z.cpu().double(), z_ref, atol=2e-4 * float(z_ref.abs().max()))
    assert torch.equal(idx.cpu().long()[sure], idx_ref[sure])
    assert torch.allclose(wt.cpu().double()[sure], wt_ref[sure], atol=1e-4)
    if unfinished:
        assert torch.allclose(rstd.cpu().double(), rstd_ref[:, 0], rtol=1e-5)
    # the sort: the same offsets as the sort kernel gives for these choices, every slot at a place of its expert's range
    g2, p2, r2 = torch.empty_like(group_off), torch.empty_like(pos), torch.empty_like(row)
    ops.moe_sort(idx, E, g2, p2, r2)
    assert torch.equal(group_off, g2)
    flat, off, pl, rw = idx.cpu().view(-1).tolist(), group_off.cpu().tolist(), pos.cpu().tolist(), row.cpu().tolist()
    assert sorted(pl) == list(range(T * top))
    for i, e in enumerate(flat):
        assert off[e] <= pl[i] < off[e + 1] and rw[pl[i]] == i // top


def test_router_ties_take_the_lower_expert(cuda_device):
    x = torch.ones(3, 8, device="cuda")
    w = torch.zeros(6, 8, device="cuda")
    w[4] = 0.5
    idx = torch.empty(3, 3, dtype=torch.int32, device="cuda")
    wt = torch.empty(3, 3, dtype=torch.float32, device="cuda")
    ops.moe_route(x, w, None, idx, wt, 3)
    assert idx.cpu().tolist() == [[4, 0, 1]] * 3
    ops.moe_select(x @ w.t(), None, idx, wt, 3)
    assert idx.cpu().tolist() == [[4, 0, 1]] * 3


# ---- products over groups ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("counts,N,K,glu", [([3, 0, 70, 1, 0], 40, 96, True), ([0, 0, 5], 100, 28, False), ([65, 64, 63], 24, 50, True),
                                            ([1], 7, 3, False)])
def test_ragged_products(cuda_device, dtype, counts, N, K, glu):
    g = torch.Generator().manual_seed(sum(counts))
    G, M = len(counts), sum(counts)
    n_src = M + 5
    a = torch.randn(n_src, K, generator=g).to(DT[dtype])
    w = (torch.randn(G, (2 if glu else 1) * N, K, generator=g) * 0.2).to(DT[dtype])
    rows = torch.randint(0, n_src, (M,), generator=g, dtype=torch.int32)
    off = [0]
    for c in counts:
        off.append(off[-1] + c)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=DT[dtype])
    ops.gemm_grouped(a.cuda(), w.cuda(), out, group_off=i32(off), a_rows=rows.cuda(), n_rows=M, glu=glu)
    ref = torch.empty(M, N, dtype=torch.float64)
    for e in range(G):
        x = a.double()[rows[off[e]:off[e + 1]].long()]
        y = x @ w[e].double().t()
        if glu:
            gate, up = y[:, :N].to(DT[dtype]).double(), y[:, N:].to(DT[dtype]).double()
            y = gate * torch.sigmoid(gate) * up
        ref[off[e]:off[e + 1]] = y
    close(out, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,G,K,N,gated", [(1, 3, 16, 64, False), (70, 5, 48, 16, True), (9, 1, 40, 20, True), (130, 9, 128, 48, False)])
def test_products_per_head(cuda_device, dtype, M, G, K, N, gated):
    g = torch.Generator().manual_seed(M)
    a = torch.randn(M, G * K + 8, generator=g).to(DT[dtype])[:, 8:]          # column ranges of wider rows
    w = (torch.randn(G, N, K, generator=g) * 0.2).to(DT[dtype])
    gate = torch.randn(M, G * N, generator=g).to(DT[dtype]) if gated else None
    out = torch.empty(M, G * N, device="cuda", dtype=DT[dtype])
    ops.gemm_grouped(a.cuda().view(M, G, K), w.cuda(), out.view(M, G, N), gate=gate.cuda().view(M, G, N) if gated else None)
    ref = torch.einsum("mgk,gnk->mgn", a.double().reshape(M, G, K), w.double())
    if gated:
        ref = ref.to(DT[dtype]).double() * torch.sigmoid(gate.double().view(M, G, N))
    close(out.view(M, G, N), ref, dtype)


# ---- routed feed-forward -----------------------------------------------------------------------------------------
class _Ctx:
    def __init__(self, dtype, max_tokens=512):
        from infinilm_b200.engine.step import Workspace
        self.ws, self.dtype, self.tap = Workspace(torch.device("cuda"), max_tokens), dtype, None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("a", 0), ("a", 1), ("b", 1), ("c", 0), ("b", 3)])
def test_routed_feed_forward_part(cuda_device, dtype, name, layer):
    from infinilm_b200.parts.moe import RoutedExperts
    raw = NIROZEN[name]()
    w = make_weights(raw, 7)
    mlp, W, p = raw["layers"][layer]["mlp"], raw["width"], f"l{layer}.mlp"
    part = RoutedExperts({"hidden": W, "n_experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "expert_ff": mlp["expert"]["ff"],
                          "shared_ff": mlp["shared"]["ff"] if mlp["shared"] else None}, p, DT[dtype])
    part.set_weights({ws.name: w[part.full_name(ws.name)].cuda() for ws in part.weight_specs()})
    ctx = _Ctx(DT[dtype])
    for T in (1, 2, 17, 150) + ((1100,) if name == "a" else ()):      # 1,100 tokens: bfloat16 hands the experts' products to the library
        h = torch.randn(T, W, generator=torch.Generator().manual_seed(T)).to(DT[dtype])
        margins = []
        ref = P.moe(mlp, w, p, h.double(), margins)
        got = part.forward(h.cuda(), ctx)
        if dtype == "bfloat16" and margins:                           # a choice that rounding can turn is not compared
            keep = torch.tensor(margins).view(T, -1).amin(1) > 0.05
            got, ref = got[keep.cuda()], ref[keep]
        close(got, ref, dtype, f"T={T}")
        # a token's result does not depend on what else is in the batch
        if T == 150:
            alone = part.forward(h[40:41].cuda(), ctx).clone()
            both = part.forward(h.cuda(), ctx)[40:41]
            assert torch.allclose(alone.float(), both.float(), rtol=0, atol=1e-6 if dtype == "float32" else 2e-2 * float(both.abs().max()))


@pytest.mark.parametrize("name,layer,T", [("a", 0, 1), ("a", 1, 8), ("b", 1, 16), ("d", 0, 5)])
def test_routed_feed_forward_takes_rows_whose_norm_is_unfinished(cuda_device, name, layer, T):
    """A decode step hands the feed-forward residual * norm weight and the sums of squares per 16 columns instead of
    normed rows: the router and the ragged product finish the norm themselves. Against the oracle on the normed rows."""
    from infinilm_b200.parts.moe import RoutedExperts
    raw = NIROZEN[name]()
    w = make_weights(raw, 11)
    mlp, W, p = raw["layers"][layer]["mlp"], raw["width"], f"l{layer}.mlp"
    part = RoutedExperts({"hidden": W, "n_experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "expert_ff": mlp["expert"]["ff"],
                          "shared_ff": mlp["shared"]["ff"] if mlp["shared"] else None}, p, torch.bfloat16)
    part.set_weights({ws.name: w[part.full_name(ws.name)].cuda() for ws in part.weight_specs()})
    assert part.accepts_normed(T)
    g = torch.Generator().manual_seed(T)
    resid, nw, eps = torch.randn(T, W, generator=g) * 3, 1.0 + torch.randn(W, generator=g) * 0.1, 1e-5
    xw = (resid * nw).bfloat16()
    pad = (-W) % 16
    sumsq = torch.nn.functional.pad(resid * resid, (0, pad)).view(T, -1, 16).sum(-1)
    ctx = _Ctx(torch.bfloat16)
    got = part.forward(ops.NormedInput(xw.cuda(), sumsq.cuda().contiguous(), W, eps), ctx)
    h = xw.double() * torch.rsqrt((resid.double() ** 2).mean(-1, keepdim=True) + eps)
    margins = []
    ref = P.moe(mlp, w, p, h, margins)
    if margins:
        keep = torch.tensor(margins).view(T, -1).amin(1) > 0.05
        got, ref = got[keep.cuda()], ref[keep]
    close(got, ref, "bfloat16", f"T={T}")


@pytest.mark.parametrize("T,W,top,shared", [(1, 96, 2, True), (8, 2048, 6, True), (16, 100, 3, False), (5, 4096, 1, True)])
def test_combine_that_ends_the_branch(cuda_device, T, W, top, shared):
    """The combine of a few rows with the residual add and the next norm's inputs, and the plain weight-streaming product
    that reads them: together they must give what add + norm + product give."""
    g = torch.Generator().manual_seed(T + W)
    n_slots = T * top
    y = torch.randn(n_slots + 3, W, generator=g).bfloat16()
    pos = torch.randperm(n_slots, generator=g).int()
    wt = torch.softmax(torch.randn(T, top, generator=g), -1)
    sh = torch.randn(T, W, generator=g).bfloat16() if shared else None
    resid = torch.randn(T, W, generator=g) * 3
    nw = 1.0 + torch.randn(W, generator=g) * 0.1
    eps, scale = 1e-5, 0.7
    branch = (wt.double()[:, :, None] * y.double()[pos.long().view(T, top)]).sum(1) + (sh.double() if shared else 0.0)
    new_resid = resid.double() + scale * branch.bfloat16().double()
    r = resid.cuda().clone()
    xw = torch.empty(T, W, dtype=torch.bfloat16, device="cuda")
    sumsq = torch.empty(T, (W + 15) // 16, device="cuda")
    ni = ops.moe_combine_resid(y.cuda(), pos.cuda(), wt.cuda(), sh.cuda() if shared else None, r, scale, nw.cuda(), eps, xw, sumsq)
    assert torch.allclose(r.cpu().double(), new_resid, atol=2e-2, rtol=0)            # a sum may round to the neighbouring bfloat16
    assert torch.allclose(sumsq.sum(1).cpu().double(), (r.cpu().double() ** 2).sum(1), rtol=1e-5)
    close(xw, r.cpu().double() * nw.double(), "bfloat16")
    if W % 8 == 0:
        wd = (torch.randn(40, W, generator=g) * 0.1).bfloat16()
        out = torch.empty(T, 40, dtype=torch.bfloat16, device="cuda")
        ops.gemm_skinny(ni.xw, wd.cuda(), out, 1.0, None, norm_in=ni)
        normed = xw.cpu().double() * torch.rsqrt((r.cpu().double() ** 2).mean(-1, keepdim=True) + eps)
        close(out, normed @ wd.double().t(), "bfloat16")


# ---- attention with a sink, kernel by kernel ---------------------------------------------------------------------
def _sink_case(nh, hd, starts, qlens, seed, far=None):
    """Entries with `starts[i]` cached positions and `qlens[i]` new ones over a cache whose K and V planes hold the same
    vectors, pages handed out in a shuffled order. `far`: (entry, key position): that key is scaled up and every query of
    the entry turned towards it, so that it outweighs all others together - a kernel that loses it shows."""
    g = torch.Generator().manual_seed(seed)
    E = len(starts)
    lens = [s + q for s, q in zip(starts, qlens)]
    n_pages = sum((n + 15) // 16 for n in lens)
    perm = torch.randperm(n_pages + 3, generator=g).tolist()
    width = max((n + 15) // 16 for n in lens)
    bt = torch.full((E, width), -1, dtype=torch.int32)
    lat = [torch.randn(n, hd, generator=g) for n in lens]
    q = [torch.randn(ql, nh, hd, generator=g) for ql in qlens]
    if far is not None:
        e, key = far
        lat[e][key] *= 3.0
        q[e] = q[e] * 0.3 + lat[e][key][None, None, :] * 0.4
    cache = torch.zeros(n_pages + 4, 2, 1, 16, hd)
    k = 0
    for e in range(E):
        for pi in range((lens[e] + 15) // 16):
            bt[e, pi] = perm[k]
            rows = lat[e][pi * 16:(pi + 1) * 16]
            cache[perm[k], 0, 0, :rows.shape[0]] = rows
            cache[perm[k], 1, 0, :rows.shape[0]] = rows
            k += 1
    sink = (torch.arange(nh, dtype=torch.float32) % 4) * 3.0 - 4.0 + torch.randn(nh, generator=g) * 0.2
    return dict(E=E, starts=starts, qlens=qlens, lens=lens, lat=lat, q=q, bt=bt, cache=cache, sink=sink)


def _sink_reference(c, scale, dtype):
    outs = []
    for e in range(c["E"]):
        lat = c["lat"][e].to(DT[dtype]).double()
        q = c["q"][e].to(DT[dtype]).double()
        s0 = c["starts"][e]
        per_head = []
        for j in range(q.shape[1]):
            full = torch.zeros(c["lens"][e], q.shape[2], dtype=torch.float64)      # rows before the portion: their queries do not matter
            full[s0:] = q[:, j]
            per_head.append(P.sink_softmax_attention(full, lat, lat, scale, c["sink"][j].double())[s0:])
        outs.append(torch.stack(per_head, 1))
    return torch.cat(outs, 0).reshape(sum(c["qlens"]), -1)


def _run_kernel(kernel, c, nh, hd, scale, dtype, splits=1):
    dt = DT[dtype]
    q = torch.cat(c["q"], 0).reshape(-1, nh * hd).to(dt).cuda()
    cache, bt, sink = c["cache"].to(dt).cuda(), c["bt"].cuda(), c["sink"].cuda()
    T = q.shape[0]
    out = torch.full((T, nh * hd), float("nan"), device="cuda", dtype=dt)
    qstart = [0]
    for ql in c["qlens"]:
        qstart.append(qstart[-1] + ql)
    if kernel == "plain":
        pos = [s + i for s, ql in zip(c["starts"], c["qlens"]) for i in range(ql)]
        ent = [e for e, ql in enumerate(c["qlens"]) for _ in range(ql)]
        ops.attention_plain(q, out, cache, bt, i32(pos), i32(ent), 16, nh, 1, hd, scale, None, sink)
    elif kernel in ("decode", "decode_k"):
        rows = T * nh * splits
        if kernel == "decode_k":                  # values that are the keys: the V plane must not even be read
            cache[:, 1] = float("nan")
            assert ops.kv_tensor_map(cache) is not None and bool(ops.kv_tensor_map(cache)[384:].any())
        ops.attention_decode(q, out, cache, bt, i32(c["lens"]), T, 16, nh, 1, hd, scale, None, 0, splits,
                             torch.empty(rows * hd, device="cuda"), torch.empty(rows * 2, device="cuda"),
                             kv_map=ops.kv_tensor_map(cache), sink=sink, v_is_k=kernel == "decode_k")
    elif kernel == "prefill":
        tpt = max(1, 64 // nh)
        ops.attention_prefill(q, out, cache, bt, i32(qstart), i32(c["lens"]), 0, c["E"], sum((x + tpt - 1) // tpt for x in c["qlens"]),
                              16, nh, 1, hd, scale, None, sink=sink)
    else:
        tpt = max(1, ops.prefill_tc5_rows(hd) // nh)
        ops.attention_prefill_tc5(q, out, ops.kv_tensor_map(cache), bt, i32(qstart), i32(c["lens"]), 0, c["E"],
                                  sum((x + tpt - 1) // tpt for x in c["qlens"]), 16, nh, 1, hd, scale, None, sink=sink)
    torch.cuda.synchronize()
    ops.check_status("cuda:0")
    return out


PORTIONS = dict(starts=[0, 250, 31, 16, 0], qlens=[70, 9, 2, 33, 1])
SINGLES = dict(starts=[0, 15, 16, 17, 399, 63], qlens=[1] * 6)


@pytest.mark.parametrize("kernel,dtype,nh,hd", [("plain", "float32", 3, 40), ("plain", "float32", 9, 128), ("plain", "bfloat16", 5, 48),
                                                ("prefill", "bfloat16", 5, 48), ("prefill", "bfloat16", 3, 64), ("prefill", "bfloat16", 7, 16),
                                                ("tc5", "bfloat16", 3, 64), ("tc5", "bfloat16", 9, 128), ("tc5", "bfloat16", 1, 64),
                                                ("tc5", "bfloat16", 12, 256), ("tc5", "bfloat16", 2, 256)])
@pytest.mark.parametrize("far", [None, (1, 3), (1, 16), (1, 255), (0, 0), (3, 15)])
def test_sink_attention_over_portions(cuda_device, kernel, dtype, nh, hd, far):
    c = _sink_case(nh, hd, PORTIONS["starts"], PORTIONS["qlens"], nh * hd, far)
    got = _run_kernel(kernel, c, nh, hd, 0.23, dtype)
    close(got.view(-1, nh, hd), _sink_reference(c, 0.23, dtype).view(-1, nh, hd), dtype, f"{kernel} far={far}")


@pytest.mark.parametrize("kernel,dtype,nh,hd,splits", [("plain", "float32", 3, 40, 1), ("decode", "bfloat16", 5, 48, 1), ("decode", "bfloat16", 3, 64, 4),
                                                       ("decode", "bfloat16", 9, 128, 1), ("decode", "bfloat16", 9, 128, 7), ("decode", "bfloat16", 20, 32, 13),
                                                       ("decode_k", "bfloat16", 3, 64, 4), ("decode_k", "bfloat16", 9, 128, 1), ("decode_k", "bfloat16", 9, 128, 7),
                                                       ("decode_k", "bfloat16", 20, 256, 5), ("decode_k", "bfloat16", 33, 192, 2), ("decode", "bfloat16", 5, 256, 3)])
@pytest.mark.parametrize("far", [None, (4, 2), (4, 16), (4, 383), (2, 15), (5, 0)])
def test_sink_attention_of_single_tokens(cuda_device, kernel, dtype, nh, hd, splits, far):
    c = _sink_case(nh, hd, SINGLES["starts"], SINGLES["qlens"], nh + hd, far)
    got = _run_kernel(kernel, c, nh, hd, 0.31, dtype, splits)
    close(got.view(-1, nh, hd), _sink_reference(c, 0.31, dtype).view(-1, nh, hd), dtype, f"{kernel} far={far} splits={splits}")


@pytest.mark.parametrize("kernel", ["plain", "decode", "prefill", "tc5"])
def test_sink_that_dominates_or_vanishes(cuda_device, kernel):
    nh, hd = 4, 64
    decode = kernel == "decode"
    c = _sink_case(nh, hd, [40, 0], [1, 1] if decode else [5, 3], 3)
    for sinks in ([80.0, -80.0, 0.0, 5.0], [-300.0] * 4):
        c["sink"] = torch.tensor(sinks)
        got = _run_kernel(kernel, c, nh, hd, 0.2, "bfloat16", 3 if decode else 1)
        ref = _sink_reference(c, 0.2, "bfloat16")
        close(got.view(-1, nh, hd), ref.view(-1, nh, hd), "bfloat16", f"{kernel} sinks={sinks}")
        if sinks[0] == 80.0:
            assert float(got.view(-1, nh, hd)[:, 0].float().abs().max()) < 1e-20      # all weight on the sink: nothing comes out


# ---- the mixer as a whole ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("a", 0), ("a", 2), ("b", 1), ("b", 3), ("c", 1), ("d", 0)])
def test_latent_attention_mixer(cuda_device, dtype, name, layer):
    """One whole sequence through the mixer (prompt kernels), then the same in three steps - a portion, a portion of two,
    single tokens - from the cache it wrote (decode kernels)."""
    from infinilm_b200.cache.manager import PagedKVView
    from infinilm_b200.parts.latent_attention import LatentAttention
    raw = NIROZEN[name]()
    w = make_weights(raw, 11)
    m, W, p = raw["layers"][layer]["mixer"], raw["width"], f"l{layer}.mix"
    part = LatentAttention({"hidden": W, "n_heads": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"], "q_rank": m["q_rank"],
                            "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": raw["norm"]["eps"]}, p, DT[dtype])
    part.set_weights({ws.name: w[part.full_name(ws.name)].cuda() for ws in part.weight_specs()})
    T = 53
    h = torch.randn(T, W, generator=torch.Generator().manual_seed(layer)).to(DT[dtype])
    ref = P.latent_attention(m, w, p, h.double(), raw["norm"]["eps"])
    storage = torch.zeros(9, 2, 1, 16, m["kv_rank"], device="cuda", dtype=DT[dtype])
    bt = i32([[6, 2, 7, 0]])
    view = PagedKVView(storage, bt, 16, True, 4, ops.kv_tensor_map(storage) if dtype == "bfloat16" else None)

    def step(a, b):
        ctx = _Ctx(DT[dtype])
        n = b - a
        ctx.T, ctx.n_entries, ctx.n_decode = n, 1, 1 if n == 1 else 0
        ctx.tok_pos, ctx.tok_entry = i32(list(range(a, b))), i32([0] * n)
        ctx.entry_qstart, ctx.entry_kvlen = i32([0, n]), i32([b])
        ctx.h_qlen, ctx.h_kvlen, ctx.lengths_are_bounds = [n], [b], False
        ctx.prompt_tiles = lambda tpt: (n + tpt - 1) // tpt if n > 1 else 0
        return part.forward(h[a:b].cuda(), ctx, view).clone()
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)      # a latent width without a fast kernel says so once
        # (queries are scaled up in the tests' weights: with scores of several units a bfloat16 step of a score moves a
        # weight by a few per cent, so the 16-bit path is given twice the usual room here; the 32-bit path is not)
        tol = 5e-2 if dtype == "bfloat16" else None
        close(step(0, T), ref, dtype, "whole", tol)
        storage.zero_()
        got = torch.cat([step(0, 30), step(30, 32)] + [step(t, t + 1) for t in range(32, T)], 0)
    close(got, ref, dtype, "in steps", tol)
