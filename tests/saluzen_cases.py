"""Small Saluzen configurations and random weights for the tests, made here (names and shapes written out by hand, so a
loader that expects other names or shapes fails).

The configurations differ from one another in every size and option: width, vocabulary, heads and key/value heads (one,
some, as many as heads), key and value sizes (equal and unequal), rotated dimensions (all, some, none), scaled and plain
frequencies, chunks (shorter and longer than the sequences, around a page's edge, none), taps of the short convolutions
(1 to 4), state sizes, groups and norm groups (1, some, as many as heads), the two scales of a weighted pair, latent
sizes, layers that read an earlier layer's latents, layers without a feed-forward, and the order of layers.
"""
import json
import os

import torch

from plain_llama import write_safetensors


def attn(heads, kv_heads, dim, vdim, scale, rot=None, scaling=None, size=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if size is not None:
        m["mask"] = {"size": size}
    return m


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(left, right):
    return {"type": "parallel", "mixer": {"left": left, "right": right}}


def parallel_2(left, right, left_scale, right_scale):
    return {"type": "parallel_2", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, eps=1e-5):
    """layers: (mixer, mlp) pairs"""
    return {"architecture": "Saluzen", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [{"type": l["type"], "mixer": l["mixer"], "mlp": m} for l, m in layers]}


# every mixer, small everything, head sizes that are no power of two, a chunk shorter than a page
CASE_A = config(96, 211, [
    (latent(3, 16, 8, 24, 40, 48, 0.2, 10000.0), dense(80)),
    (parallel(attn(4, 2, 24, 40, 0.3, rot=(10000.0, 8)), ssm(3, 24, 16, 1, 4, 1)), dense(72)),
    (latent(2, 24, 8, 16, 40, 32, 0.25, 10000.0, kv_from=0), None),
    (parallel_2(attn(6, 3, 16, 16, 0.25, rot=(500.0, 16), size=9), delta(4, 2, 16, 24, 2), 0.7, 1.3), dense(64)),
], eps=1e-6)

# chunks of a page and of a page and one; one and as many key/value heads as heads; one tap; scaled frequencies; as many
# groups as heads; a left side without rotation
CASE_B = config(128, 300, [
    (parallel_2(attn(4, 1, 48, 48, 0.15, rot=(500000.0, 24), size=64), delta(2, 2, 48, 16, 4), 1.0, 0.25), dense(96)),
    (parallel(attn(2, 2, 16, 32, 0.25, rot=(1000.0, 16), scaling=(8.0, 1.0, 4.0, 64)), ssm(4, 16, 24, 4, 2, 4)), None),
    (latent(4, 24, 16, 40, 32, 72, 0.16, 50000.0), dense(64)),
    (parallel_2(attn(4, 2, 32, 24, 0.2, size=65), delta(6, 1, 8, 32, 1), 0.5, 0.5), dense(64)),
    (latent(4, 8, 16, 8, 32, 24, 0.3, 50000.0, kv_from=2), dense(48)),
])

# head sizes of 64 and 128 (the tensor-core kernels in bfloat16), states of 128 and 64 rows, a chunk past a page
CASE_C = config(256, 333, [
    (parallel(attn(4, 1, 64, 64, 0.1, rot=(300000.0, 64), scaling=(5.0, 1.0, 3.0, 128)), ssm(2, 64, 128, 1, 4, 2)), dense(128)),
    (latent(4, 64, 64, 128, 64, 64, 0.09, 10000.0), None),
    (parallel_2(attn(2, 1, 128, 128, 0.09, rot=(1000.0, 32), size=70), delta(2, 1, 128, 64, 3), 0.8, 0.6), dense(192)),
    (latent(2, 64, 64, 64, 64, 32, 0.1, 10000.0, kv_from=1), dense(64)),
    (parallel(attn(8, 2, 64, 64, 0.125), ssm(8, 16, 64, 8, 3, 1)), dense(96)),
])
CASE_D = config(64, 90, [(parallel_2(attn(2, 1, 16, 16, 0.25, rot=(1000.0, 16), size=8), delta(2, 1, 16, 16, 3), 1.0, 1.0), dense(40)),
                         (parallel(attn(2, 2, 16, 16, 0.25), ssm(2, 16, 8, 2, 3, 2)), dense(40))])

CASES = {"a": CASE_A, "b": CASE_B, "c": CASE_C, "d": CASE_D}


def attention_shapes(x, m, E, gate_per_head):
    rows = {"q": m["heads"] * m["dim"], "k": m["kv_heads"] * m["dim"], "v": m["kv_heads"] * m["vdim"]}
    shapes = {}
    for n, r in rows.items():
        shapes[x + n], shapes[x + n + ".b"] = (r, E), (r,)
    shapes[x + "g"] = (m["heads"] if gate_per_head else m["heads"] * m["vdim"], E)
    shapes[x + "o"] = (E, m["heads"] * m["vdim"])
    if gate_per_head:
        shapes[x + "sink"] = (m["heads"],)
    return shapes


def tensor_shapes(cfg):
    E = cfg["width"]
    shapes = {"embed": (cfg["vocab"], E), "head": (cfg["vocab"], E), "final.norm": (E,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (E,)
        x = p + "mix."
        if layer["type"] == "latent_attention":
            H = m["heads"]
            shapes[x + "dq"], shapes[x + "dq.norm"] = (m["q_rank"], E), (m["q_rank"],)
            shapes[x + "uq"] = (H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            if "kv_from" not in m:
                shapes[x + "dkv"], shapes[x + "dkv.norm"] = (m["kv_rank"] + m["rot_dim"], E), (m["kv_rank"],)
            shapes[x + "uk"], shapes[x + "uv"] = (H * m["dim"], m["kv_rank"]), (H * m["vdim"], m["kv_rank"])
            shapes[x + "o"] = (E, H * m["vdim"])
        elif layer["type"] == "parallel":
            shapes.update(attention_shapes(x + "left.", m["left"], E, False))
            r = m["right"]
            inner, gn = r["heads"] * r["vdim"], r["groups"] * r["state"]
            y = x + "right."
            shapes[y + "in"] = (2 * inner + 2 * gn + r["heads"], E)
            shapes[y + "conv"], shapes[y + "conv.b"] = (inner + 2 * gn, r["conv"]), (inner + 2 * gn,)
            shapes[y + "dt_bias"] = shapes[y + "A_log"] = shapes[y + "D"] = (r["heads"],)
            shapes[y + "norm"], shapes[y + "o"] = (inner,), (E, inner)
            shapes[x + "left.out"] = shapes[x + "right.out"] = (E,)
        else:
            shapes.update(attention_shapes(x + "left.", m["left"], E, True))
            r = m["right"]
            q, v = r["kv_heads"] * r["dim"], r["heads"] * r["vdim"]
            y = x + "right."
            for n, rows in (("q", q), ("k", q), ("v", v)):
                shapes[y + n], shapes[y + n + ".conv"] = (rows, E), (rows, r["conv"])
            shapes[y + "b"] = shapes[y + "a"] = (r["heads"], E)
            shapes[y + "A_log"] = shapes[y + "dt_bias"] = (r["heads"],)
            shapes[y + "norm"], shapes[y + "g"], shapes[y + "o"] = (r["vdim"],), (v, E), (E, v)
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            shapes[p + "norm2"] = shapes[p + "norm2b"] = (E,)
            shapes[p + "mlp.gate"] = shapes[p + "mlp.up"] = (F, E)
            shapes[p + "mlp.down"] = (E, F)
    return shapes


def random_weights(cfg, seed, sharp=1.0, sink=1.0, slow=0.0):
    """bfloat16 tensors: matrices ~ N(0, 1/in), norm weights ~ 1 + N(0, 0.2), biases ~ N(0, 0.3), taps ~ N(0, 0.5), sinks ~
    N(0, sink), A_log ~ N(-slow, 0.5), dt_bias ~ N(-slow, 1), D ~ 1 + N(0, 0.3), the table ~ N(0, 1).  ``sharp`` multiplies the
    query and key projections of the attention mixers, so that a few keys carry each softmax and a key that is wrongly seen
    or missed changes the result by much more than bfloat16 rounding does; ``slow`` makes the recurrent states forget slowly."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last in ("norm", "norm1", "norm1b", "norm2", "norm2b", "out"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.2
        elif last == "sink":
            t = torch.randn(shape, generator=g) * sink
        elif last == "conv":
            t = torch.randn(shape, generator=g) * 0.5
        elif last == "A_log":
            t = torch.randn(shape, generator=g) * 0.5 - slow
        elif last == "dt_bias":
            t = torch.randn(shape, generator=g) - slow
        elif last == "D":
            t = 1.0 + torch.randn(shape, generator=g) * 0.3
        elif len(shape) == 1:                       # biases
            t = torch.randn(shape, generator=g) * 0.3
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
            if (".left." in name and last in ("q", "k")) or last in ("uq", "dkv"):
                t = t * sharp
        W[name] = t.to(torch.bfloat16)
    return W


def write_model(path, cfg, W):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), W)
    return str(path)


def make_model(tmp_path, cfg, seed, sharp=1.0, sink=1.0, slow=0.0, change=None):
    """(model folder, float64 weights for the plain implementation); ``change(W)`` may edit the bfloat16 tensors first"""
    W = random_weights(cfg, seed, sharp, sink, slow)
    if change:
        change(W)
    d = write_model(tmp_path, cfg, W)
    return d, {k: v.to(torch.float64) for k, v in W.items()}
