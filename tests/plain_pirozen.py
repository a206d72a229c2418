"""A plain, slow implementation of the Pirozen decoder, one function per mechanism, in float64.

It takes the configuration as the dictionary of config.json and the weights as a dictionary name -> tensor, runs ONE
sequence from its first token, and shares no code with the engine.  The tests compare the engine with it.

Notation: T tokens, E the width, H heads, G key/value heads, d the key size of a head, dv its value size, X routed experts,
I identity experts, R = X + I router outputs.

The design: every layer is  x <- x + mixer(n1(x)) + ff(n2(x))  with two RMS norms of the same x, followed by a per-layer token
input  x <- x + n_s(P (gelu(Gt x) * e_tok))  where e_tok is the layer's slice of a second embedding table.  The mixer is
grouped-query attention with biases, a per-head RMS norm of q and k, rotation of the first dimensions of a head (halves layout,
optionally with blended frequencies), a sliding window, and a sigmoid gate per head on the heads' outputs.  The feed-forward
is a mixture of gated experts with a softmax router, a selection bias, groups of experts, identity experts and a shared expert.
A span of layers may run several times, each pass starting from  W_in [x; embedding output].
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotary_table(rot, positions):
    """cos, sin [T, dims / 2] for the angles p * f_i; with "scaling" the frequencies are blended and both tables stretched."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def dim_of(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=F64)
        f = f / factor * ramp + f * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    ang = positions.to(F64)[:, None] * f[None, :]
    return torch.cos(ang) * amp, torch.sin(ang) * amp


def rotate_halves(x, positions, rot):
    """x [T, heads, size]: entry i < dims / 2 of a head pairs with entry i + dims / 2; the rest passes unchanged."""
    dims = int(rot["dims"])
    half = dims // 2
    c, s = rotary_table(rot, positions)
    c, s = c[:, None, :], s[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def window_mask(T, size):
    """visible[i, j]: 0 <= i - j < size (size None: every earlier key)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & (i - j < size)
    return ok


def attention_mixer(h, W, pre, m, eps):
    """h [T, E] -> [T, E]."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"])
    dv = int(m.get("vdim", d))
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).view(T, H, d)
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).view(T, G, d)
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).view(T, G, dv)
    q = rms_norm(q, W[pre + "q.norm"], eps)
    k = rms_norm(k, W[pre + "k.norm"], eps)
    pos = torch.arange(T)
    if m.get("rot"):
        q = rotate_halves(q, pos, m["rot"])
        k = rotate_halves(k, pos, m["rot"])
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)                              # query head h reads key/value head h // rep
    vv = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * float(m["scale"])
    size = int(m["mask"]["size"]) if m.get("mask") else None
    scores = scores.masked_fill(~window_mask(T, size)[None], float("-inf"))
    p = torch.softmax(scores, -1)
    o = torch.einsum("hij,jhd->ihd", p, vv)                           # [T, H, dv]
    gate = torch.sigmoid(h @ W[pre + "g"].T)                          # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ W[pre + "o"].T + W[pre + "o.b"]


def gated_expert(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def route(z, correction, r):
    """z [T, R] router logits -> (chosen [T, top] expert indices, weights [T, top])."""
    T, R = z.shape
    groups = r.get("groups") or {"count": 1, "keep": 1}              # no groups: one group of everything, kept
    top, count, keep = int(r["top"]), int(groups["count"]), int(groups.get("keep", groups["count"]))
    s = torch.softmax(z, -1)
    choice = s + correction
    per = R // count
    group_score = choice.view(T, count, per).max(-1).values            # [T, count]
    allowed = torch.zeros(T, count, dtype=torch.bool)
    allowed.scatter_(1, torch.topk(group_score, keep, dim=-1).indices, True)
    choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    chosen = torch.topk(choice, top, dim=-1).indices
    w = torch.gather(s, 1, chosen)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))
    return chosen, w


def moe(h, W, pre, mlp):
    r = mlp["router"]
    X, I = int(r["experts"]), int(r.get("identity", 0))
    z = h @ W[pre + "router"].T
    chosen, w = route(z, W[pre + "correction"], r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(chosen[t].tolist(), w[t]):
            if e >= X:
                assert e < X + I
                out[t] += we * h[t]
            else:
                out[t] += we * gated_expert(h[t:t + 1], W, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, W, pre + "shared.")
    return out


def token_side(x, tokens, W, pre, i, dim, eps):
    e = W["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ W[pre + "gate"].T) * e
    return rms_norm(g @ W[pre + "proj"].T, W[pre + "norm"], eps)


def layer(x, tokens, W, i, cfg):
    L = cfg["layers"][i]
    eps = float(cfg["norm"]["eps"])
    pre = f"l{i}."
    if L["type"] != "attention":
        raise ValueError(L["type"])
    y = attention_mixer(rms_norm(x, W[pre + "norm1"], eps), W, pre + "mix.", L["mixer"], eps)
    if L.get("mlp") is not None:
        y = y + moe(rms_norm(x, W[pre + "norm2"], eps), W, pre + "mlp.", L["mlp"])
    x = x + y
    if cfg.get("token_side"):
        x = x + token_side(x, tokens, W, pre + "side.", i, int(cfg["token_side"]["dim"]), eps)
    return x


def layer_order(cfg):
    """(layer, starts a pass) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(tokens, W, cfg, streams=None):
    """tokens: list of ids of one sequence from its start -> logits [T, vocab]; streams (a list) receives x after each run."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x0 = W["embed"][tokens]
    x = x0
    for i, enters in layer_order(cfg):
        if enters:
            x = torch.cat([x, x0], -1) @ W["loop.in"].T
        x = layer(x, tokens, W, i, cfg)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, W["final.norm"], float(cfg["norm"]["eps"])) @ W["head"].T
