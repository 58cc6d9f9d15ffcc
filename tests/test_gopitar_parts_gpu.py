"""Each mechanism of the Gopitar parts alone, on the device, against the plain implementation: the short convolution with
its state (portions down to one token, slots used again), the two recurrences over a matrix state (whole against token by
token, a state that matters after hundreds of tokens), the delta rule's preparation, the grouped norm with a gate, the
head gate with packing, the soft cap, the weighted sum, the gelu form of the gated feed-forward in each of its kernels,
and the residual add of a row per token before a norm."""
import math

import pytest
import torch

import plain_gopitar as P

pytestmark = pytest.mark.gpu


def _i32(x, dev):
    return torch.tensor(x, dtype=torch.int32, device=dev)


def _step_arrays(lens, dev):
    qstart = [0]
    for n in lens:
        qstart.append(qstart[-1] + n)
    tok_entry = [e for e, n in enumerate(lens) for _ in range(n)]
    return _i32(qstart, dev), _i32(tok_entry, dev)


@pytest.mark.parametrize("fused_state", [False, True])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_short_conv_in_portions_with_state(cuda_device, taps, dtype, fused_state):
    from infinilm_b200 import ops
    dev = cuda_device
    torch.manual_seed(taps)
    C, seg_in, seg_out = 24, 6, 16
    seqs = {1: torch.randn(37, C).to(torch.bfloat16).float(), 2: torch.randn(9, C).to(torch.bfloat16).float(), 3: torch.randn(1, C).to(torch.bfloat16).float()}
    w = torch.randn(C, taps)
    want = {s: P.short_conv(u.double(), w.double()) for s, u in seqs.items()}
    state = torch.zeros(5, max(taps - 1, 1), C, device=dev)
    state[4] = 7.0                                # a slot that an earlier request left dirty: slot 3's first step reads slot 0 instead
    # steps: (slot, tokens) lists; a request's first step reads the zero slot
    plan = [[(1, 5), (2, 2)], [(1, 1), (2, 1), (3, 1)], [(1, 2), (2, 6)], [(1, 1)], [(1, 28)]]
    done = {s: 0 for s in seqs}
    got = {s: [] for s in seqs}
    for step in plan:
        lens = [n for _, n in step]
        x = torch.cat([seqs[s][done[s]: done[s] + n] for s, n in step]).to(dtype).to(dev)
        qstart, tok_entry = _step_arrays(lens, dev)
        rd = _i32([0 if done[s] == 0 else s for s, _ in step], dev)
        wr = _i32([s for s, _ in step], dev)
        out = torch.full((x.shape[0], 4 * seg_out + 3), 5.0, dtype=dtype, device=dev)
        if fused_state:                           # as a step runs it: single tokens first, their state moved on by the convolution itself
            n_single = sum(1 for _, n in step if n == 1)
            assert all(n == 1 for _, n in step[:n_single]) and all(n > 1 for _, n in step[n_single:])
            ops.short_conv(x, 0, w.to(dev), state, 0, rd, tok_entry, qstart, out, 3, C // seg_in // 2, seg_in, seg_out, 0,
                           n_seg2=C // seg_in - C // seg_in // 2, seg_in2=seg_in, write_slots=wr)
            ops.short_conv_state(x, 0, C, taps, state, 0, rd, wr, qstart, len(step) - n_single, first_entry=n_single)
        else:
            ops.short_conv(x, 0, w.to(dev), state, 0, rd, tok_entry, qstart, out, 3, C // seg_in, seg_in, seg_out, 0)
            ops.short_conv_state(x, 0, C, taps, state, 0, rd, wr, qstart, len(step))
        o = out[:, 3:].float().cpu().view(-1, C // seg_in, seg_out)
        assert float(o[:, :, seg_in:].abs().max()) == 0.0 and float(out[:, :3].float().min()) == 5.0
        r = 0
        for s, n in step:
            got[s].append(o[r: r + n, :, :seg_in].reshape(n, C))
            r += n
            done[s] += n
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for s in seqs:
        g = torch.cat(got[s]).double()
        assert g.shape == want[s].shape
        assert float((g - want[s]).abs().max()) <= tol * float(want[s].abs().max() + 1), (s, taps)


GENERIC = False                                   # which of the two recurrence kernels `_scan` runs; the tests run under both


@pytest.fixture(params=[False, True], ids=["registers", "shared"])
def scan_kernel(request):
    global GENERIC
    GENERIC = request.param
    yield request.param
    GENERIC = False


def _scan(ops, mode, q, k, v, H, G, d, dv, decay, beta, g, state, slot, first, dev, act=0):
    n = q.shape[0]
    qstart, _ = _step_arrays([n], dev)
    out = torch.empty(n, H * dv, device=dev)
    ops.matrix_state_scan(mode, q, k, v, H, G, d, dv, act, decay, beta, g, state, _i32([0 if first else slot], dev), _i32([slot], dev),
                          qstart, 1, out, generic=GENERIC, single=(n == 1))
    return out


@pytest.mark.parametrize("H,G,d,dv", [(2, 2, 32, 32), (3, 1, 8, 40), (4, 2, 64, 128), (1, 1, 20, 12), (2, 1, 128, 64), (1, 1, 256, 36), (2, 2, 136, 8), (2, 1, 10, 6), (1, 1, 50, 33)])
def test_decayed_sum_whole_and_token_by_token(cuda_device, scan_kernel, H, G, d, dv):
    from infinilm_b200 import ops
    dev = cuda_device
    torch.manual_seed(d)
    T = 300
    q, k, v = torch.randn(T, G * d), torch.randn(T, G * d), torch.randn(T, H * dv)
    decay = torch.tensor([0.999, 0.6, 0.95, 0.9][:H])
    rep = H // G
    want = P.decayed_linear_attention(P.silu(q.double()).view(T, G, d).repeat_interleave(rep, 1), P.silu(k.double()).view(T, G, d).repeat_interleave(rep, 1),
                                      P.silu(v.double()).view(T, H, dv), decay.double()).reshape(T, H * dv)
    state = torch.zeros(4, H, dv, d, device=dev)
    state[2] = 3.0
    qd, kd, vd, dd = q.to(dev), k.to(dev), v.to(dev), decay.to(dev)
    whole = _scan(ops, ops.SCAN_DECAY, qd, kd, vd, H, G, d, dv, dd, None, None, state, 1, True, dev, act=1)
    scale = float(want.abs().max())
    assert float((whole.cpu().double() - want).abs().max()) <= 2e-5 * scale
    # a prompt of 257 tokens, then one by one, into a slot that held something else
    parts = [_scan(ops, ops.SCAN_DECAY, qd[:257], kd[:257], vd[:257], H, G, d, dv, dd, None, None, state, 2, True, dev, act=1)]
    for t in range(257, T):
        parts.append(_scan(ops, ops.SCAN_DECAY, qd[t:t + 1], kd[t:t + 1], vd[t:t + 1], H, G, d, dv, dd, None, None, state, 2, False, dev, act=1))
    assert float((torch.cat(parts).cpu().double() - want).abs().max()) <= 2e-5 * scale
    assert float((state[1] - state[2]).abs().max()) <= 2e-5 * float(state[1].abs().max())
    # with a decay of 0.999 the first token still counts at the end: zero its value and the last output moves
    if H >= 1:
        v2 = vd.clone()
        v2[0] += 50.0
        moved = _scan(ops, ops.SCAN_DECAY, qd, kd, v2, H, G, d, dv, dd, None, None, state, 3, True, dev, act=1)
        assert float((moved[-1, :dv] - whole[-1, :dv]).abs().max()) > 1e-3 * scale


@pytest.mark.parametrize("H,G,d,dv", [(2, 1, 32, 64), (6, 2, 8, 12), (3, 3, 24, 16), (2, 2, 128, 128), (1, 1, 40, 32), (1, 1, 200, 130), (2, 1, 4, 4), (4, 2, 10, 6), (1, 1, 70, 33)])
def test_delta_rule_with_its_preparation(cuda_device, scan_kernel, H, G, d, dv):
    from infinilm_b200 import ops
    dev = cuda_device
    torch.manual_seed(dv)
    T = 200
    qk = torch.randn(T, 2 * G * d)
    v = torch.randn(T, H * dv)
    ab = torch.randn(T, 2 * H + 3) * 2
    a_log, dt_bias = torch.randn(H) * 0.5, torch.randn(H) * 0.5
    qn = P.unit(qk[:, :G * d].double().view(T, G, d)) * d ** -0.5
    kn = P.unit(qk[:, G * d:].double().view(T, G, d))
    beta = torch.sigmoid(ab[:, 1:1 + H].double())
    g = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(ab[:, 1 + H:1 + 2 * H].double() + dt_bias.double()))
    rep = H // G
    want = P.gated_delta_rule(qn.repeat_interleave(rep, 1), kn.repeat_interleave(rep, 1), v.double().view(T, H, dv), beta, g).reshape(T, H * dv)
    qkd, abd = qk.to(dev), ab.to(dev)
    b_dev, g_dev = torch.empty(T, H, device=dev), torch.empty(T, H, device=dev)
    ops.delta_prep(qkd, 0, G * d, G, d, d ** -0.5, 1e-6, abd, 1, 1 + H, a_log.to(dev), dt_bias.to(dev), b_dev, g_dev, H)
    assert float((b_dev.cpu().double() - beta).abs().max()) < 1e-6 and float((g_dev.cpu().double() - g).abs().max()) < 1e-6
    assert float((qkd[:, :G * d].cpu().double().view(T, G, d) - qn).abs().max()) < 1e-6
    state = torch.zeros(3, H, dv, d, device=dev)
    vd = v.to(dev)
    whole = _scan(ops, ops.SCAN_DELTA, qkd[:, :G * d], qkd[:, G * d:], vd, H, G, d, dv, None, b_dev, g_dev, state, 1, True, dev)
    scale = float(want.abs().max())
    assert float((whole.cpu().double() - want).abs().max()) <= 3e-5 * scale
    cuts, a, parts = [3, 1, 1, 64, 2, 129], 0, []
    for n in cuts:
        parts.append(_scan(ops, ops.SCAN_DELTA, qkd[a:a + n, :G * d], qkd[a:a + n, G * d:], vd[a:a + n], H, G, d, dv, None, b_dev[a:a + n], g_dev[a:a + n],
                           state, 2, a == 0, dev))
        a += n
    assert a == T and float((torch.cat(parts).cpu().double() - want).abs().max()) <= 3e-5 * scale


def test_scan_of_a_batch_equals_each_alone(cuda_device, scan_kernel):
    from infinilm_b200 import ops
    dev = cuda_device
    torch.manual_seed(7)
    H, d, dv, lens = 2, 16, 24, [5, 1, 40, 2]
    T = sum(lens)
    q, k, v = (torch.randn(T, H * n, device=dev) for n in (d, d, dv))
    decay = torch.tensor([0.9, 0.99], device=dev)
    state = torch.randn(6, H, dv, d, device=dev)
    state[0] = 0
    before = state.clone()
    qstart, _ = _step_arrays(lens, dev)
    out = torch.empty(T, H * dv, device=dev)
    rd, wr = _i32([0, 2, 3, 0], dev), _i32([1, 2, 3, 4], dev)
    ops.matrix_state_scan(ops.SCAN_DECAY, q, k, v, H, H, d, dv, 0, decay, None, None, state, rd, wr, qstart, 4, out, generic=GENERIC)
    a = 0
    for e, n in enumerate(lens):
        st = before.clone()
        one = _scan(ops, ops.SCAN_DECAY, q[a:a + n], k[a:a + n], v[a:a + n], H, H, d, dv, decay, None, None, st, int(wr[e]), int(rd[e]) == 0, dev)
        assert torch.equal(one, out[a:a + n]) and torch.equal(st[int(wr[e])], state[int(wr[e])])
        a += n
    assert torch.equal(state[5], before[5]) and float(state[0].abs().max()) == 0.0
    # as a step runs it: single tokens first, by the form made for them, the portions behind them by the chunked form
    lens2 = [1, 1, 5, 40]
    T2 = sum(lens2)
    qs2, _ = _step_arrays(lens2, dev)
    st2, out2 = before.clone(), torch.empty(T2, H * dv, device=dev)

    class Ctx:
        n_decode, n_entries, T = 2, 4, T2
    ops.matrix_state_scan_step(Ctx, ops.SCAN_DECAY, q[:T2], k[:T2], v[:T2], H, H, d, dv, 0, decay, None, None, st2, rd, wr, qs2, out=out2, generic=GENERIC)
    a = 0
    for e, n in enumerate(lens2):
        st = before.clone()
        one = _scan(ops, ops.SCAN_DECAY, q[a:a + n], k[a:a + n], v[a:a + n], H, H, d, dv, decay, None, None, st, int(wr[e]), int(rd[e]) == 0, dev)
        assert torch.equal(one, out2[a:a + n]) and torch.equal(st[int(wr[e])], st2[int(wr[e])])
        a += n


@pytest.mark.parametrize("H,d,dv", [(2, 32, 32), (3, 8, 40), (1, 128, 64), (2, 20, 12), (2, 10, 6), (1, 250, 9)])
def test_decayed_sum_in_segments(cuda_device, H, d, dv):
    """Long portions walked in segments that run at once, with the second pass that adds each segment's start: several
    entries of unequal length (one segment, an exact multiple, a ragged end), from states that hold something, against
    the plain implementation continued from those states; the request's state afterwards too."""
    from infinilm_b200 import ops
    dev = cuda_device
    torch.manual_seed(H + d)
    seg, lens = 64, [200, 64, 7, 129, 128]
    T = sum(lens)
    q, k, v = torch.randn(T, H * d) * 0.5, torch.randn(T, H * d) * 0.5, torch.randn(T, H * dv)
    decay = torch.tensor([0.999, 0.7, 0.97][:H])
    state = torch.randn(8, H, dv, d, device=dev) * 0.3
    state[0] = 0
    rd, wr = _i32([1, 0, 2, 0, 3], dev), _i32([1, 4, 2, 5, 3], dev)
    before = state.clone()
    qstart, _ = _step_arrays(lens, dev)
    out = torch.empty(T, H * dv, device=dev)
    n_tiles = sum((n + seg - 1) // seg for n in lens) + 2        # a bound: surplus blocks leave
    scratch = torch.empty(n_tiles * H * dv * d, device=dev)
    ops.matrix_state_scan(ops.SCAN_DECAY, q.to(dev), k.to(dev), v.to(dev), H, H, d, dv, 0, decay.to(dev), None, None, state, rd, wr, qstart,
                          len(lens), out, seg_len=seg, n_tiles=n_tiles, seg_state=scratch)
    a = 0
    for e, n in enumerate(lens):
        S = before[int(rd[e])].cpu().double().transpose(1, 2).clone()          # [H, d, dv]
        want = torch.zeros(n, H, dv, dtype=torch.float64)
        for t in range(n):
            S = decay.double()[:, None, None] * S + k[a + t].double().view(H, d)[:, :, None] * v[a + t].double().view(H, dv)[:, None, :]
            want[t] = torch.einsum("hde,hd->he", S, q[a + t].double().view(H, d))
        got = out[a:a + n].cpu().double().view(n, H, dv)
        assert float((got - want).abs().max()) <= 3e-5 * float(want.abs().max()), (e, n)
        assert float((state[int(wr[e])].cpu().double().transpose(1, 2) - S).abs().max()) <= 3e-5 * float(S.abs().max()), (e, n)
        a += n
    assert torch.equal(state[6], before[6]) and torch.equal(state[7], before[7])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_group_norm_gate_head_gate_softcap_sum(cuda_device, out_dtype):
    from infinilm_b200 import ops
    dev = cuda_device
    torch.manual_seed(3)
    T, H, dv = 11, 3, 20
    x = torch.randn(T, H * dv) * 3
    gate = torch.randn(T, 5 + H * dv)
    for group, n_w, act in ((dv, dv, ops.GATE_SILU), (H * dv, H * dv, ops.GATE_SIGMOID)):
        w = (1 + 0.1 * torch.randn(n_w)).to(torch.bfloat16)
        xx = x.double().view(T, -1, group)
        gz = gate[:, 5:].double()
        want = (P.rms_norm(xx, None, 1e-5).reshape(T, -1) * w.double().repeat(H * dv // n_w)
                * (P.silu(gz) if act == ops.GATE_SILU else torch.sigmoid(gz)))
        out = torch.empty(T, H * dv, dtype=out_dtype, device=dev)
        ops.group_norm_gate(x.to(dev), w.to(dev), 1e-5, gate.to(dev), 5, act, out, group)
        tol = 1e-5 if out_dtype == torch.float32 else 1e-2
        assert float((out.float().cpu().double() - want).abs().max()) <= tol * float(want.abs().max())
    # one gate per head, heads of 32 columns packed to 20
    hd = 32
    y = torch.randn(T, H * hd).to(out_dtype)
    gt = torch.randn(T, 4 + H).to(out_dtype)
    out = torch.empty(T, H * dv, dtype=out_dtype, device=dev)
    ops.head_gate(y.to(dev), hd, gt.to(dev), 4, out, H, dv)
    want = y.double().view(T, H, hd)[:, :, :dv] * torch.sigmoid(gt[:, 4:].double())[:, :, None]
    assert float((out.float().cpu().double().view(T, H, dv) - want).abs().max()) <= (1e-6 if out_dtype == torch.float32 else 2e-2)
    ops.head_gate(y.to(dev), hd, None, 0, out, H, dv)
    assert torch.equal(out.cpu().view(T, H, dv), y.view(T, H, hd)[:, :, :dv])
    a, b = torch.randn(T, 40).to(out_dtype), torch.randn(T, 40).to(out_dtype)
    o = torch.empty(T, 40, dtype=out_dtype, device=dev)
    ops.scaled_sum(a.to(dev), 0.6, b.to(dev), 0.9, o)
    assert float((o.float().cpu() - (0.6 * a.float() + 0.9 * b.float())).abs().max()) <= (1e-6 if out_dtype == torch.float32 else 3e-2)
    if out_dtype == torch.float32:
        z = torch.randn(7, 33) * 40
        zd = z.to(dev).contiguous()
        ops.softcap(zd, 15.0)
        assert float((zd.cpu().double() - 15.0 * torch.tanh(z.double() / 15.0)).abs().max()) < 1e-5


@pytest.mark.parametrize("T", [3, 16, 40, 100, 300])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_feed_forward_with_gelu(cuda_device, T, dtype):
    """Every kernel the gated feed-forward takes by row count (decode product, tensor-core product of 17..128 rows, library
    product with the activation kernel; the float32 kernels) with the tanh form of GELU as its gate."""
    from infinilm_b200.parts.base import build_part
    from infinilm_b200.parts.spec import PartSpec
    dev = cuda_device
    torch.manual_seed(T)
    H, I = 64, 96
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    ff = build_part("feed_forward", PartSpec("swiglu", {"hidden": H, "intermediate": I, "activation": "gelu_tanh",
                                                         "names": {"gate": "gate", "up": "up", "down": "down"}}, "x"), dt)
    assert [ws.name for ws in ff.weight_specs()] == ["gate", "up", "down"]
    w = {n: (torch.randn(s) * 0.2).to(torch.bfloat16) for n, s in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I)))}
    ff.set_weights({k: v.to(dev).to(dt) for k, v in w.items()})
    x = (torch.randn(T, H) * 1.5).to(torch.bfloat16)
    want = P.gated_mlp(x.double(), {k: v.double() for k, v in w.items()})

    class Ctx:
        pass
    from infinilm_b200.engine.step import Workspace
    ctx = Ctx()
    ctx.ws = Workspace(torch.device(dev), 512)
    got = ff.forward(x.to(dev).to(dt), ctx).float().cpu().double()
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert float((got - want).abs().max()) <= tol * float(want.abs().max())


def test_add_norm_with_a_row_per_token(cuda_device):
    from infinilm_b200 import ops
    dev = cuda_device
    torch.manual_seed(4)
    T, H = 9, 72
    resid, rows_add, branch = torch.randn(T, H), torch.randn(T, H), torch.randn(T, H)
    w = 1 + 0.1 * torch.randn(H)
    r = resid.to(dev).clone()
    out = torch.empty(T, H, device=dev)
    ops.add_rmsnorm(r, branch.to(dev), 0.5, w.to(dev), 1e-5, out, None, rows_add.to(dev).contiguous())
    x = resid.double() + 0.5 * branch.double() + rows_add.double()
    assert float((r.cpu().double() - x).abs().max()) < 1e-5
    assert float((out.cpu().double() - P.rms_norm(x, w.double(), 1e-5)).abs().max()) < 1e-5
