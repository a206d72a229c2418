"""Small Pirozen configurations and random weights for the tests, made here (names and shapes written out by hand, so a
loader that expects other names or shapes fails).

The configurations differ from one another in every size and option: width, vocabulary, heads and key/value heads (one,
some, as many as heads), key and value sizes (equal and unequal, also the sizes the tensor-core attention takes), rotated
dimensions (all, some, none) with and without blended frequencies, windows (shorter and longer than the sequences, around a
page's edge, none), experts (few and many, one to four a token), identity experts (none, some), groups (none, some kept,
all kept), a shared expert (with, without), layers without a feed-forward, the token input (with, without), and the loop
(none; once; three times over a span in the middle; twice over everything).
"""
import copy
import json
import os

import torch

from plain_llama import write_safetensors


def attention(heads, kv_heads, dim, vdim, scale, size=None, rot=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "attention", "mixer": m}


def moe(ff, experts, top, scale=1.0, identity=None, groups=None, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if identity is not None:
        r["identity"] = identity
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def config(width, vocab, layers, loop=None, side=None, eps=1e-5):
    """layers: (mixer, mlp or None) pairs"""
    c = {"architecture": "Pirozen", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": [{"type": l["type"], "mixer": l["mixer"], "mlp": m} for l, m in layers]}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    if side is not None:
        c["token_side"] = {"dim": side}
    return c


# small everything, head sizes that are no power of two and differ for keys and values; a span in the middle runs three times
CASE_A = config(96, 211, [
    (attention(4, 2, 24, 40, 0.3, size=9, rot=(10000.0, 8), scaling=(4.0, 64, 8.0, 1.0)), moe(40, 6, 2, scale=2.0, identity=2, groups=(2, 1), shared=56)),
    (attention(3, 3, 16, 16, 0.4, size=5, rot=(300.0, 16)), moe(24, 5, 3)),
    (attention(6, 1, 32, 8, 0.2), None),
    (attention(2, 2, 16, 24, 0.25, size=70, rot=(500.0, 4)), moe(32, 9, 4, scale=0.7, identity=3, groups=(4, 2), shared=24)),
], loop=(1, 3, 3), side=8, eps=1e-6)

# no loop, no token input; head sizes 64 and 128 for keys and values alike; windows around a page's edge; one expert a token
CASE_B = config(128, 300, [
    (attention(4, 2, 64, 64, 0.125, size=64, rot=(500000.0, 64)), moe(64, 4, 1, scale=1.5, identity=1, shared=64)),
    (attention(6, 2, 128, 128, 0.09, size=65, rot=(10000.0, 32), scaling=(16.0, 128, 32.0, 1.0)), moe(48, 8, 2, scale=2.5, groups=(4, 2))),
    (attention(2, 1, 64, 64, 0.2, rot=(1000.0, 16)), None),
    (attention(8, 8, 64, 64, 0.15, size=130), moe(32, 3, 2, identity=3, groups=(3, 3))),
])

# a width the tensor-core contractions refuse, odd sizes everywhere, everything looped twice
CASE_C = config(100, 90, [
    (attention(5, 5, 12, 20, 0.35, size=33, rot=(50.0, 12), scaling=(2.0, 16, 4.0, 0.5)), moe(28, 7, 2, scale=1.2, identity=1, groups=(2, 2), shared=36)),
    (attention(3, 1, 40, 28, 0.18, size=1), moe(20, 2, 2)),
], loop=(0, 2, 2), side=5)

# a loop that runs once, in front of the last layer
CASE_D = config(64, 70, [(attention(2, 1, 16, 16, 0.25, size=8, rot=(1000.0, 16)), moe(24, 4, 2, identity=2, groups=(3, 2), shared=16)),
                         (attention(4, 2, 16, 32, 0.3), moe(16, 3, 1, scale=3.0))], loop=(1, 2, 1), side=12)

CASES = {"a": CASE_A, "b": CASE_B, "c": CASE_C, "d": CASE_D}


def without_choice(cfg):
    """The same model with every router output chosen (at most eight outputs a layer, all groups kept): the weights still come
    from the router's softmax, but no near tie can send a row to other experts - for position-by-position runs in bfloat16."""
    c = copy.deepcopy(cfg)
    for l in c["layers"]:
        if l["mlp"] is None:
            continue
        r = l["mlp"]["router"]
        ident = r.get("identity", 0)
        r["experts"] = min(r["experts"], 8 - ident)
        r["top"] = r["experts"] + ident
        if "groups" in r:
            count = r["groups"]["count"]
            if (r["experts"] + ident) % count:
                del r["groups"]
            else:
                r["groups"]["keep"] = count
    return c


def tensor_shapes(cfg):
    E = cfg["width"]
    shapes = {"embed": (cfg["vocab"], E), "head": (cfg["vocab"], E), "final.norm": (E,)}
    if "loop" in cfg:
        shapes["loop.in"] = (E, 2 * E)
    side = cfg.get("token_side", {}).get("dim")
    if side:
        shapes["side.embed"] = (cfg["vocab"], side * len(cfg["layers"]))
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (E,)
        x = p + "mix."
        rows = {"q": m["heads"] * m["dim"], "k": m["kv_heads"] * m["dim"], "v": m["kv_heads"] * m["vdim"]}
        for n, r in rows.items():
            shapes[x + n], shapes[x + n + ".b"] = (r, E), (r,)
        shapes[x + "q.norm"] = shapes[x + "k.norm"] = (m["dim"],)
        shapes[x + "g"] = (m["heads"], E)
        shapes[x + "o"], shapes[x + "o.b"] = (E, m["heads"] * m["vdim"]), (E,)
        mlp = layer["mlp"]
        if mlp is not None:
            f, F, r = p + "mlp.", mlp["expert"]["ff"], mlp["router"]
            shapes[p + "norm2"] = (E,)
            outputs = r["experts"] + r.get("identity", 0)
            shapes[f + "router"], shapes[f + "correction"] = (outputs, E), (outputs,)
            for e in range(r["experts"]):
                shapes[f + f"e{e}.gate"] = shapes[f + f"e{e}.up"] = (F, E)
                shapes[f + f"e{e}.down"] = (E, F)
            if "shared" in mlp:
                S = mlp["shared"]["ff"]
                shapes[f + "shared.gate"] = shapes[f + "shared.up"] = (S, E)
                shapes[f + "shared.down"] = (E, S)
        if side:
            shapes[p + "side.gate"], shapes[p + "side.proj"], shapes[p + "side.norm"] = (side, E), (E, side), (E,)
    return shapes


def random_weights(cfg, seed, sharp=1.0):
    """bfloat16 tensors: matrices ~ N(0, 1/in), norm weights ~ 1 + N(0, 0.2), biases ~ N(0, 0.3), tables ~ N(0, 1), routers
    four times wider (scores away from one another), selection biases ~ N(0, 0.1) - as large as the scores themselves, so that
    they change who is chosen.  ``sharp`` multiplies the query and key projections, so that a few keys carry each softmax and a
    key that is wrongly seen or missed changes the result by much more than bfloat16 rounding does."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last in ("norm", "norm1", "norm2"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.2
        elif last == "b":
            t = torch.randn(shape, generator=g) * 0.3
        elif last == "correction":
            t = torch.randn(shape, generator=g) * 0.1
        elif last == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
            if last == "router":
                t = t * 4.0
            if name.endswith((".mix.q", ".mix.k")):
                t = t * sharp
            if last == "g":
                t = t * 3.0                       # gates spread over (0, 1)
        W[name] = t.to(torch.bfloat16)
    return W


def write_model(path, cfg, W):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), W)
    return str(path)


def make_model(tmp_path, cfg, seed, sharp=1.0):
    """(model folder, float64 weights for the plain implementation)"""
    W = random_weights(cfg, seed, sharp)
    d = write_model(tmp_path, cfg, W)
    return d, {k: v.to(torch.float64) for k, v in W.items()}
