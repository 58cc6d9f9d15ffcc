"""A plain, slow implementation of the Gopitar design on whole sequences, one function per mechanism, written from the
design's equations in float64 (or any dtype given). It shares no code with the package: tensors in, tensors out, loops
over time where the design has a recurrence.

Notation: T tokens, W width; a linear weight is [out, in] and applied as x @ w.T; positions count from 0.
"""
import math

import torch


def rms_norm(x, w, eps):
    """y = x / sqrt(mean(x^2) + eps) * w over the last axis (w may be None)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(u, w):
    """Causal convolution over time, per channel. u [T, C], w [C, taps]; the last column of w meets the current token:
    y[t] = sum_j w[:, j] * u[t - (taps - 1) + j], with zeros before the sequence's start."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotate_half(x, pos, rot_dims, base):
    """x [T, heads, dim]; the first rot_dims entries of each head are rotated, entry i paired with i + rot_dims/2."""
    if rot_dims == 0:
        return x
    half = rot_dims // 2
    i = torch.arange(half, dtype=x.dtype)
    f = base ** (-2.0 * i / rot_dims)
    a = pos.to(x.dtype)[:, None] * f[None, :]                 # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:rot_dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:rot_dims] = v * c + u * s
    return out


def window_softmax_attention(q, k, v, scale, window):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h uses kv head h // (H // G); token i sees j with 0 <= i - j < window
    (window None: every j <= i). Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        ok = (j <= i) if window is None else ((i - j >= 0) & (i - j < window))
        s = s.masked_fill(~ok, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def conv_gated_attention(h, p, c):
    """The softmax branch: projections with biases, short convolution on q, k, v, partial rotation, windowed softmax,
    one sigmoid gate per head, output projection with bias. `p` maps local tensor names to tensors, `c` is the branch's
    configuration (heads, kv_heads, dim, vdim, conv, rot.base, rot.dims, scale, mask.size)."""
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = h @ p["q"].T + p["q.b"]
    k = h @ p["k"].T + p["k.b"]
    v = h @ p["v"].T + p["v.b"]
    if c.get("conv") is not None:
        q, k, v = short_conv(q, p["q.conv"]), short_conv(k, p["k.conv"]), short_conv(v, p["v.conv"])
    pos = torch.arange(T)
    rot = c.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_half(q.view(T, H, d), pos, rot["dims"], rot["base"])
    k = rotate_half(k.view(T, G, d), pos, rot["dims"], rot["base"])
    o = window_softmax_attention(q, k, v.view(T, G, dv), c["scale"], c["mask"]["size"] if c.get("mask") else None)
    gate = torch.sigmoid(h @ p["g"].T)                         # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ p["o"].T + p["o.b"]


def decayed_linear_attention(q, k, v, decay):
    """Per head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t. q, k [T, H, d], v [T, H, dv], decay [H]."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out


def lightning_branch(h, p, c, eps):
    T = h.shape[0]
    H, d, dv = c["heads"], c["dim"], c["vdim"]
    q = silu(h @ p["q"].T).view(T, H, d)
    k = silu(h @ p["k"].T).view(T, H, d)
    v = silu(h @ p["v"].T).view(T, H, dv)
    o = decayed_linear_attention(q, k, v, torch.tensor(c["decay"], dtype=h.dtype)).reshape(T, H * dv)
    o = rms_norm(o, p["norm"], eps) * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


def parallel_mixer(h, p, c, eps):
    left = conv_gated_attention(h, {k[5:]: v for k, v in p.items() if k.startswith("left.")}, c["left"])
    right = lightning_branch(h, {k[6:]: v for k, v in p.items() if k.startswith("right.")}, c["right"], eps)
    return c["left_scale"] * left + c["right_scale"] * right


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def gated_delta_rule(q, k, v, beta, g):
    """q, k [T, H, d] (already per value head), v [T, H, dv], beta and g [T, H]. Per head and token:
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out


def delta_mixer(h, p, c, eps):
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q, k, v = h @ p["q"].T, h @ p["k"].T, h @ p["v"].T
    if c.get("conv") is not None:
        q, k, v = short_conv(q, p["q.conv"]), short_conv(k, p["k.conv"]), short_conv(v, p["v.conv"])
    q, k, v = silu(q).view(T, G, d), silu(k).view(T, G, d), silu(v).view(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ p["b"].T)
    g = torch.exp(-torch.exp(p["A_log"]) * torch.nn.functional.softplus(h @ p["a"].T + p["dt_bias"]))
    o = gated_delta_rule(q, k, v, beta, g)                     # [T, H, dv]
    o = rms_norm(o, p["norm"], eps) * silu(h @ p["g"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ p["o"].T


def gated_mlp(h, p):
    return (gelu_tanh(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for t in range(times):
        order += [(i, t > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg, w, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one whole sequence. `w` maps tensor names to tensors; `layers_out`: a list that receives the
    residual stream after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    x0 = x.clone()
    for i, again in run_order(cfg):
        L = cfg["layers"][i]
        if again:
            x = x + x0
        pre = f"l{i}.mix."
        p = {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
        hin = rms_norm(x, w[f"l{i}.norm1"], eps)
        if L["type"] == "parallel":
            x = x + parallel_mixer(hin, p, L["mixer"], eps)
        elif L["type"] == "delta":
            x = x + delta_mixer(hin, p, L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            pre = f"l{i}.mlp."
            x = x + gated_mlp(rms_norm(x, w[f"l{i}.norm2"], eps), {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)})
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
