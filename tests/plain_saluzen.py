"""A plain, slow implementation of the Saluzen decoder, one function per mechanism, in float64.

It takes the configuration as the dictionary of config.json and the weights as a dictionary name -> tensor, runs ONE
sequence from its first token, and shares no code with the engine.  The tests compare the engine with it.

Notation: T tokens, E the width, H heads, G key/value heads (or groups), d the key size of a head, dv its value size,
N the size of a state-space head's state.
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotary_frequencies(rot):
    """The angle's frequency per pair i, with the three-band scaling when the file gives one."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
            wave = 2.0 * math.pi / f
            if wave > orig / low:
                f = f / factor
            elif not wave < orig / high:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate(x, positions, rot, layout):
    """x [T, heads, size]: the first rot.dims entries of each head turned by p * f_i; pair i is (i, i + dims/2) in the
    'halves' layout and (2i, 2i + 1) in the 'adjacent' one.  The other entries pass."""
    dims = int(rot["dims"])
    ang = positions.to(F64)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if layout == "halves":
        a, b = x[..., 0:dims // 2], x[..., dims // 2:dims]
        out[..., 0:dims // 2] = a * c - b * s
        out[..., dims // 2:dims] = b * c + a * s
    else:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    return out


def short_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j) (+ bias), zeros in front of the sequence."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j][None, :]
    return y if bias is None else y + bias[None, :]


def visible_keys(T, chunk=None):
    """[T, T] bool: key j <= row i, and (chunked) both in the same run of `chunk` positions counted from 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = j <= i
    if chunk:
        vis = vis & (i // chunk == j // chunk)
    return vis


def softmax_with_sink(scores, visible, sink):
    """scores [H, T, T] masked by visible [T, T]; the denominator also holds exp(sink_h) (sink None: ordinary softmax)."""
    scores = scores.masked_fill(~visible[None], float("-inf"))
    m = scores.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(scores - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def gated_attention(h, W, pre, m, sink_kind, gate_kind):
    """Grouped-query attention with biases, partly rotated heads ('halves'), a sink in the softmax and an output gate.
    sink_kind 'one': a sink of score 0; 'learned': the tensor .sink.  gate_kind 'full': sigmoid(W_g h) on every number of
    the heads' outputs; 'head': one number a head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).view(T, H, d)
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).view(T, G, d)
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).view(T, G, dv)
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"], "halves"), rotate(k, pos, m["rot"], "halves")
    rep = H // G
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * float(m["scale"])
    chunk = m["mask"]["size"] if m.get("mask") else None
    sink = torch.zeros(H, dtype=F64) if sink_kind == "one" else W[pre + "sink"]
    p = softmax_with_sink(scores, visible_keys(T, chunk), sink)
    o = torch.einsum("hij,jhd->ihd", p, vv)
    g = torch.sigmoid(h @ W[pre + "g"].T)
    o = o * (g.view(T, H, dv) if gate_kind == "full" else g.view(T, H, 1))
    return o.reshape(T, H * dv) @ W[pre + "o"].T


def state_space(h, W, pre, m, eps):
    """State-space duality: per head S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t."""
    T = h.shape[0]
    H, dv, N, G, R = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * dv
    u = h @ W[pre + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, W[pre + "conv"], W[pre + "conv.b"]))
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N).repeat_interleave(H // G, 1)
    C = xbc[:, inner + G * N:].view(T, G, N).repeat_interleave(H // G, 1)
    dt = softplus(dt + W[pre + "dt_bias"])                       # [T, H]
    a = torch.exp(-torch.exp(W[pre + "A_log"])[None, :] * dt)
    S = torch.zeros(H, N, dv, dtype=F64)
    y = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = a[t][:, None, None] * S + dt[t][:, None, None] * B[t][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, C[t]) + W[pre + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    y = y.view(T, R, inner // R)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    return (y.reshape(T, inner) * W[pre + "norm"]) @ W[pre + "o"].T


def gated_delta(h, W, pre, m, eps):
    """Gated delta rule: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[pre + "q"].T, W[pre + "q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ W[pre + "k"].T, W[pre + "k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ W[pre + "v"].T, W[pre + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1)
    beta = torch.sigmoid(h @ W[pre + "b"].T)                      # [T, H]
    g = torch.exp(-torch.exp(W[pre + "A_log"])[None, :] * softplus(h @ W[pre + "a"].T + W[pre + "dt_bias"]))
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * W[pre + "norm"]
    o = o * silu(h @ W[pre + "g"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ W[pre + "o"].T


def latent_kv(h, W, pre, m, eps):
    """What a latent attention layer keeps a position: the normalised latent and the rotated key part."""
    T = h.shape[0]
    r, dr = m["kv_rank"], m["rot_dim"]
    u = h @ W[pre + "dkv"].T
    c = rms_norm(u[:, :r], W[pre + "dkv.norm"], eps)
    kr = rotate(u[:, r:].view(T, 1, dr), torch.arange(T), m["rot"], "adjacent")[:, 0]
    return c, kr


def latent_attention(h, W, pre, m, eps, kv):
    """kv: (latent c [T, r], rotated key part [T, dr]) - the layer's own or an earlier layer's."""
    T = h.shape[0]
    H, d, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kv
    cq = rms_norm(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps)
    q = (cq @ W[pre + "uq"].T).view(T, H, d + dr)
    qn, qr = q[..., :d], rotate(q[..., d:], torch.arange(T), m["rot"], "adjacent")
    kn = (c @ W[pre + "uk"].T).view(T, H, d)
    v = (c @ W[pre + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * float(m["scale"])
    p = softmax_with_sink(scores, visible_keys(T), None)
    o = torch.einsum("hij,jhd->ihd", p, v)
    return o.reshape(T, H * dv) @ W[pre + "o"].T


def pair_mixer(h, W, pre, layer, eps):
    """Two mixers on the same input; 'parallel': half the sum of their normalised outputs, 'parallel_2': a weighted sum."""
    m = layer["mixer"]
    if layer["type"] == "parallel":
        left = gated_attention(h, W, pre + "left.", m["left"], "one", "full")
        right = state_space(h, W, pre + "right.", m["right"], eps)
        return 0.5 * (rms_norm(left, W[pre + "left.out"], eps) + rms_norm(right, W[pre + "right.out"], eps))
    left = gated_attention(h, W, pre + "left.", m["left"], "learned", "head")
    right = gated_delta(h, W, pre + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def dense_ff(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from its first token (and, on request, the stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)].to(F64)
    kept, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            m = layer["mixer"]
            if m.get("kv_from") is None:
                kept[i] = latent_kv(h, W, p + "mix.", m, eps)
            y = latent_attention(h, W, p + "mix.", m, eps, kept[m["kv_from"] if m.get("kv_from") is not None else i])
        else:
            y = pair_mixer(h, W, p + "mix.", layer, eps)
        x = x + rms_norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp"):
            x = x + rms_norm(dense_ff(rms_norm(x, W[p + "norm2"], eps), W, p + "mlp."), W[p + "norm2b"], eps)
        streams.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
