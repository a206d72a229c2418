"""The Pirozen decoder in the engine against the plain implementation (``plain_pirozen``): each mechanism alone, whole
prompts, portions, decoding, batches, reused slots and pages, and generation through the entry point.

Structure is tested in float32, where any key wrongly seen or missed, any expert wrongly chosen or weighed is orders of
magnitude above the tolerance.  The bfloat16 runs use sharpened attention (see ``pirozen_cases.random_weights``) so that the same
faults stay visible above rounding, and models in which every router output is chosen (``pirozen_cases.without_choice``), so that
a near tie between two experts cannot send a row elsewhere than the float64 implementation sends it."""
import numpy as np
import pytest
import torch

import plain_pirozen as pp
from helpers import rel_err
from pirozen_cases import CASES, attention, config, make_model, moe, random_weights, without_choice, write_model

pytestmark = pytest.mark.gpu

#: max |dlogit| / max |logit| against the float64 plain implementation.  float32: a key wrongly seen or an expert wrongly
#: chosen is at 1e-3 and above.  bfloat16 with sharpened attention and looped layers: rounding reaches 6e-2, a structural fault 0.3
TOL = {"float32": 2e-5, "bfloat16": 1e-1}


def tokens_for(case, n, seed):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, case["vocab"], size=n)]


def engine_for(model_dir, dtype, **kw):
    from fastgguf_b200.engine.api import Engine
    args = dict(dtype=dtype, max_tokens=4096, max_batch=8)
    args.update(kw)
    return Engine.from_dir(model_dir, **args)


def entry(slot, toks, want=None):
    from fastgguf_b200.engine.batch import StepEntry
    return StepEntry(slot, toks, list(range(len(toks))) if want is None else want)


def plain_logits(case, W, toks):
    return pp.forward(toks, W, case).numpy()


def f32(t):
    return np.ascontiguousarray(t.numpy(), dtype=np.float32)


class Rows:
    """Collects the errors of a whole model's logits, row by row, and judges them.

    The design divides by small numbers in places (the token input is normalised whatever its size, queries and keys are
    normalised per head), so at a few positions every rounding is amplified, in float32 as in bfloat16 and by the same factor.
    float32: at most one row in fifty (or one row) may exceed the tolerance, none five times the tolerance - a key wrongly seen
    or an expert wrongly chosen is fifty times above it.  bfloat16: ``cond`` holds, per sequence and position, the float32
    engine's error on the same model; a row's tolerance is the larger of the tolerance and 1e5 times that (bfloat16 rounds
    2^16 times coarser), so only positions that amplify get more room; the same count of rows may exceed it, none three times."""

    def __init__(self, dtype, cond=None):
        self.dtype, self.cond, self.n, self.over = dtype, cond, 0, []

    def add(self, got, want, what, seq=0, position=None):
        e, tol = rel_err(got, want), TOL[self.dtype]
        self.n += 1
        if self.cond is not None:
            tol = max(tol, 1e5 * self.cond[seq][position])
        assert e < (3 if self.cond is not None else 5) * tol, (what, e)
        if e >= tol:
            self.over.append((what, e))

    def done(self):
        assert len(self.over) <= max(1, self.n // 50), self.over


def conditioning(model_dir, case, W, sequences, dtype):
    """bfloat16: per sequence, the float32 engine's error at every position of the whole sequence; float32: None"""
    if dtype != "bfloat16":
        return None
    eng = engine_for(model_dir, "float32")
    out = []
    for toks in sequences:
        s = eng.acquire()
        got = eng.step_host([entry(s, toks)])
        want = plain_logits(case, W, toks)
        out.append([rel_err(got[p], want[p]) for p in range(len(toks))])
        eng.release(s)
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(case, "float32"): the case as it is; (case, "bfloat16"): attention sharpened and every router output chosen."""
    out = {}
    for i, (name, case) in enumerate(CASES.items()):
        d, W = make_model(tmp_path_factory.mktemp(f"p_{name}_f"), case, 100 + i, 1.0)
        out[(name, "float32")] = (d, case, W)
        wide = without_choice(case)
        d, W = make_model(tmp_path_factory.mktemp(f"p_{name}_b"), wide, 100 + i, 3.0)
        out[(name, "bfloat16")] = (d, wide, W)
    return out


# ------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("scaling", [None, (8.0, 256, 16.0, 2.0), (40.0, 64, 32.0, 1.0), (3.0, 2048, 24.0, 2.0)])
def test_rotary_tables_in_the_halves_layout(scaling):
    """The tables the rotation kernel reads: pair i of a position (entries i and i + dims / 2 of a head) holds amplitude * cos /
    sin of position * frequency, blended frequencies and the amplitude with scaling; the rest of the head is not rotated."""
    from fastgguf_b200.parts import position_tables
    rot = {"base": 5000.0, "dims": 24}
    params = {"head_dim": 32, "theta": 5000.0, "rotary_dim": 24, "layout": "halves", "scaling": None}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
        params["scaling"] = {"rope_type": "yarn", "factor": scaling[0], "original_max_position_embeddings": scaling[1],
                             "beta_fast": scaling[2], "beta_slow": scaling[3]}
    cos, sin, _ = position_tables("rope", params, 300)
    c, s = pp.rotary_table(rot, torch.arange(300))
    assert np.abs(cos[:, :12] - c.numpy()).max() < 2e-6
    assert np.abs(sin[:, :12] - s.numpy()).max() < 2e-6
    assert np.all(cos[:, 12:] == 1.0) and np.all(sin[:, 12:] == 0.0)
    if scaling:
        c0, _ = pp.rotary_table({"base": 5000.0, "dims": 24}, torch.arange(300))
        assert (c - c0).abs().max() > 0.05


def test_rotary_tables_over_random_parameters():
    """Two hundred drawn sets of base, rotated dimensions, factor, original length and the two turn counts - also ones whose ramp
    is empty, starts below zero or ends beyond the last dimension, and a factor of one: the tables follow the plain formulas."""
    from fastgguf_b200.parts import position_tables
    rng = np.random.default_rng(0)
    for _ in range(200):
        dims = int(rng.choice([2, 4, 8, 16, 24, 32, 64, 128]))
        hd = int(rng.choice([d for d in (2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 256) if d >= dims]))
        base = float(rng.choice([2.0, 10.0, 100.0, 1e4, 5e5, 1e6]))
        rot = {"base": base, "dims": dims}
        params = {"head_dim": hd, "theta": base, "rotary_dim": dims, "layout": "halves", "scaling": None}
        if rng.random() < 0.85:
            sc = (float(rng.choice([1.0, 1.5, 2.0, 4.0, 8.0, 32.0, 64.0])), float(rng.choice([8, 16, 64, 256, 1024, 4096, 32768])),
                  float(rng.choice([1.0, 4.0, 8.0, 32.0, 64.0])), float(rng.choice([0.25, 0.5, 1.0, 2.0, 32.0])))
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
            params["scaling"] = {"rope_type": "yarn", "factor": sc[0], "original_max_position_embeddings": sc[1], "beta_fast": sc[2],
                                 "beta_slow": sc[3]}
        cos, sin, _ = position_tables("rope", params, 150)
        c, s = pp.rotary_table(rot, torch.arange(150))
        h = dims // 2
        assert np.abs(cos[:, :h] - c.numpy()).max() < 3e-6 and np.abs(sin[:, :h] - s.numpy()).max() < 3e-6, rot
        assert np.all(cos[:, h:] == 1.0) and np.all(sin[:, h:] == 0.0)


def one_layer(layer, mlp=None, width=80, vocab=50, side=None):
    return config(width, vocab, [(layer, mlp)], side=side)


MIXERS = {
    "all keys, nothing rotated, keys and values of unequal size": attention(4, 2, 24, 40, 0.3),
    "window, one key/value head": attention(6, 1, 16, 16, 0.4, size=5),
    "window of one": attention(2, 2, 16, 16, 0.5, size=1, rot=(100.0, 16)),
    "some dimensions rotated, blended frequencies, odd output width": attention(3, 3, 32, 20, 0.2, size=11, rot=(100.0, 12), scaling=(4.0, 16, 8.0, 0.5)),
    "all dimensions rotated, a head a key/value head": attention(5, 5, 24, 24, 0.2, size=40, rot=(10000.0, 24)),
    "two rotated dimensions": attention(2, 1, 8, 8, 0.6, rot=(50.0, 2), scaling=(2.0, 8, 4.0, 1.0)),
    "long, window past a page, head 64": attention(4, 2, 64, 64, 0.125, size=70, rot=(250000.0, 64), scaling=(8.0, 64, 32.0, 1.0)),
    "long, window of a page, head 128, a quarter rotated": attention(3, 1, 128, 128, 0.09, size=64, rot=(1000.0, 32)),
    "long, all keys, keys 128 and values 64": attention(2, 1, 128, 64, 0.09, rot=(1000.0, 128)),
    "long, window beside a page's edge, head 64, nine heads on three": attention(9, 3, 64, 64, 0.11, size=65, rot=(5000.0, 32), scaling=(4.0, 512, 16.0, 1.0)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(MIXERS))
def test_mixer_alone(tmp_path, name, dtype):
    """One layer of the mixer alone (norm, mixer, residual add) on rows given by the test: a portion of 37 rows, then one of
    2, then single rows, so the second and later calls read what the first left in the cache (the long cases: 160, 30 and
    2 rows, then 38 single ones)."""
    case = one_layer(MIXERS[name])
    d, W = make_model(tmp_path, case, 7, sharp=2.0)
    eng = engine_for(d, dtype)
    g = torch.Generator().manual_seed(8)
    cuts = [160, 30, 2] + [1] * 38 if name.startswith("long") else [37, 2, 1, 1, 1, 1, 1, 1]
    T = sum(cuts)
    x = torch.randn(T, case["width"], generator=g, dtype=torch.float64)
    want = (x + pp.attention_mixer(pp.rms_norm(x, W["l0.norm1"], 1e-5), W, "l0.mix.", case["layers"][0]["mixer"], 1e-5)).numpy()
    slot = eng.acquire()
    got, at = [], 0
    for n in cuts:
        got.append(eng.block_forward(0, [(slot, n)], f32(x[at:at + n])))
        at += n
    got = np.concatenate(got)
    tol = 1e-5 if dtype == "float32" else 4e-2
    for r in range(T):
        assert rel_err(got[r], want[r]) < tol, (name, r)


def test_a_wide_batch_of_prompts(tmp_path):
    """Four prompts of 5 to 800 tokens in one step, sequences x longest prompt beyond 3,072 (the tensor-core attention then runs
    another of its forms), then one more token each."""
    name = "long, window past a page, head 64"
    case = one_layer(MIXERS[name])
    d, W = make_model(tmp_path, case, 12, sharp=2.0)
    eng = engine_for(d, "bfloat16", max_tokens=4096, max_batch=4)
    g = torch.Generator().manual_seed(9)
    lens = [800, 300, 50, 5]
    m = case["layers"][0]["mixer"]
    xs = [torch.randn(n + 1, case["width"], generator=g, dtype=torch.float64) for n in lens]
    want = [(x + pp.attention_mixer(pp.rms_norm(x, W["l0.norm1"], 1e-5), W, "l0.mix.", m, 1e-5)).numpy() for x in xs]
    slots = [eng.acquire() for _ in lens]
    got = eng.block_forward(0, list(zip(slots, lens)), f32(torch.cat([x[:n] for x, n in zip(xs, lens)])))
    at = 0
    for b, n in enumerate(lens):
        for r in (0, 1, n // 2, n - 2, n - 1):
            assert rel_err(got[at + r], want[b][r]) < 4e-2, (b, r)
        at += n
    got = eng.block_forward(0, [(s, 1) for s in slots], f32(torch.stack([x[n] for x, n in zip(xs, lens)])))
    for b, n in enumerate(lens):
        assert rel_err(got[b], want[b][n]) < 4e-2, (b, "decoded")


def test_the_gate_scales_each_head(tmp_path):
    """With gate rows that push the sigmoid towards 0 for one head and towards 1 for the others, that head's part of the output
    goes away and the others stay: the engine follows the plain implementation, which differs by far from the ungated mixer."""
    layer = attention(3, 1, 16, 24, 0.3, size=12)
    case = one_layer(layer)
    W = random_weights(case, 21)
    x = torch.randn(30, 80, generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    h = pp.rms_norm(x, W["l0.norm1"].double(), 1e-5)
    direction = (h.mean(0) / h.mean(0).norm()).to(torch.bfloat16)
    gate = W["l0.mix.g"].clone()
    gate[1] = -40.0 * direction                       # head 1 shut for rows along the common direction ...
    gate[0] = 40.0 * direction
    W["l0.mix.g"] = gate
    x = x + 3.0 * direction.double()[None, :]         # ... which every row now has
    d = write_model(tmp_path, case, W)
    W = {k: v.double() for k, v in W.items()}
    h = pp.rms_norm(x, W["l0.norm1"], 1e-5)
    want = x + pp.attention_mixer(h, W, "l0.mix.", layer["mixer"], 1e-5)
    open_gate = dict(W)
    open_gate["l0.mix.g"] = torch.zeros_like(W["l0.mix.g"])
    half = x + pp.attention_mixer(h, open_gate, "l0.mix.", layer["mixer"], 1e-5)
    for dtype, tol in (("float32", 1e-5), ("bfloat16", 4e-2)):
        eng = engine_for(d, dtype)
        got = eng.block_forward(0, [(eng.acquire(), 30)], f32(x))
        assert rel_err(got, want.numpy()) < tol
    assert rel_err(half.numpy(), want.numpy()) > 5e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_norms_of_the_same_stream(tmp_path, dtype):
    """x + mixer(norm1(x)) + ff(norm2(x)): both sublayers read the stream as the layer received it, each through a norm with a
    weight of its own."""
    mlp = moe(40, 6, 6, scale=1.3, shared=24)                  # every expert chosen: no tie can matter in bfloat16
    case = one_layer(attention(2, 1, 16, 16, 0.25, size=6, rot=(100.0, 8)), mlp)
    d, W = make_model(tmp_path, case, 9)
    eng = engine_for(d, dtype)
    x = torch.randn(20, 80, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    m = case["layers"][0]["mixer"]
    mixer = pp.attention_mixer(pp.rms_norm(x, W["l0.norm1"], 1e-5), W, "l0.mix.", m, 1e-5)
    want = x + mixer + pp.moe(pp.rms_norm(x, W["l0.norm2"], 1e-5), W, "l0.mlp.", mlp)
    one_norm = x + mixer + pp.moe(pp.rms_norm(x, W["l0.norm1"], 1e-5), W, "l0.mlp.", mlp)
    sequential = x + mixer
    sequential = sequential + pp.moe(pp.rms_norm(sequential, W["l0.norm2"], 1e-5), W, "l0.mlp.", mlp)
    got = eng.block_forward(0, [(eng.acquire(), 20)], f32(x))
    assert rel_err(got, want.numpy()) < (1e-5 if dtype == "float32" else 3e-2)
    assert rel_err(one_norm.numpy(), want.numpy()) > 5e-2 and rel_err(sequential.numpy(), want.numpy()) > 5e-2
    assert rel_err((x + mixer).numpy(), want.numpy()) > 5e-2


def moe_part(mlp, W, pre, width):
    """(parameters, tensors by their names inside the part) of the engine's feed-forward for one layer's mixture of experts"""
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    params = dict(hidden_size=width, d_ff=mlp["expert"]["ff"], n_experts=r["experts"], top_k=r["top"], router="softmax_grouped",
                  n_identity=r.get("identity", 0), n_groups=groups["count"], keep_groups=groups["keep"], route_scale=r.get("scale", 1.0),
                  shared_d_ff=(mlp.get("shared") or {}).get("ff", 0))
    t = {"router.weight": W[pre + "router"], "router.bias": W[pre + "correction"]}
    for e in range(r["experts"]):
        for n in ("gate", "up", "down"):
            t[f"experts.{e}.{n}_proj.weight"] = W[f"{pre}e{e}.{n}"]
    if mlp.get("shared"):
        for n in ("gate", "up", "down"):
            t[f"shared.{n}_proj.weight"] = W[f"{pre}shared.{n}"]
    return params, t


def run_moe(mlp, Wb, h, dtype="float32", width=80):
    """residual 0 + the engine's feed-forward of rows h (bfloat16 weights Wb)"""
    from fastgguf_b200.parts import run_part
    params, t = moe_part(mlp, Wb, "l0.mlp.", width)
    return run_part("feed_forward", "moe", params, t, dtype, x=f32(h), residual=np.zeros((h.shape[0], width), dtype=np.float32))


ROUTERS = {
    "two groups, one kept, identity experts, a shared expert": moe(40, 6, 2, scale=2.0, identity=2, groups=(2, 1), shared=56),
    "four groups, two kept, four a row": moe(32, 9, 4, scale=0.7, identity=3, groups=(4, 2), shared=24),
    "no groups, no identity experts, no shared expert": moe(24, 5, 3),
    "one a row": moe(64, 4, 1, scale=1.5, identity=1, shared=64),
    "groups all kept, as many identity experts as experts": moe(32, 3, 2, identity=3, groups=(3, 3)),
    "eight groups of two, three kept": moe(16, 16, 3, scale=2.5, groups=(8, 3)),
    "groups of one": moe(24, 5, 2, identity=1, groups=(6, 2), shared=8),
    "many rows an expert": moe(48, 3, 2, scale=1.1, groups=(3, 2)),
    "many outputs": moe(8, 44, 3, scale=1.3, identity=4, groups=(6, 3), shared=16),
}


@pytest.mark.parametrize("name", list(ROUTERS))
def test_router_and_experts_alone(name):
    """The feed-forward alone on rows given by the test, few rows (the decode step's kernels) and many (experts' runs of rows),
    in float32: who is chosen, with which weight, identity experts, the shared expert."""
    mlp = ROUTERS[name]
    case = one_layer(attention(2, 1, 16, 16, 0.25), mlp)
    Wb = random_weights(case, 31)
    W = {k: v.double() for k, v in Wb.items()}
    g = torch.Generator().manual_seed(32)
    # (many outputs and more than a thousand rows: the routing kernel's form that keeps no scores)
    for rows in (3, 150, 700) + ((1100,) if name == "many outputs" else ()):
        h = torch.randn(rows, 80, generator=g, dtype=torch.float64)
        want = pp.moe(h, W, "l0.mlp.", mlp).numpy()
        got = run_moe(mlp, Wb, h)
        for r in range(rows):
            assert rel_err(got[r], want[r]) < 2e-5, (name, rows, r)


def test_experts_in_bfloat16_on_many_rows():
    """700 rows with every output chosen (no tie can matter): the experts' runs of rows on the tensor cores."""
    mlp = moe(64, 6, 8, scale=1.7, identity=2, groups=(4, 4), shared=40)
    case = one_layer(attention(2, 1, 16, 16, 0.25), mlp)
    Wb = random_weights(case, 33)
    W = {k: v.double() for k, v in Wb.items()}
    h = torch.randn(700, 80, generator=torch.Generator().manual_seed(34), dtype=torch.float64)
    want = pp.moe(h, W, "l0.mlp.", mlp).numpy()
    for rows in (700, 5):
        got = run_moe(mlp, Wb, h[:rows], "bfloat16")
        assert rel_err(got, want[:rows]) < 3e-2


def test_groups_left_out_count_as_minus_infinity():
    """Selection biases so negative that every choice score is below zero: an output of a group that was left out must not be
    chosen although a masked score of 0 would now be the largest.  And the weights come from the scores WITHOUT the bias."""
    mlp = moe(24, 8, 2, scale=1.0, groups=(4, 2))
    case = one_layer(attention(2, 1, 16, 16, 0.25), mlp)
    Wb = random_weights(case, 35)
    Wb["l0.mlp.correction"] = (-3.0 + 0.5 * torch.randn(8, generator=torch.Generator().manual_seed(36))).to(torch.bfloat16)
    W = {k: v.double() for k, v in Wb.items()}
    h = torch.randn(40, 80, generator=torch.Generator().manual_seed(37), dtype=torch.float64)
    want = pp.moe(h, W, "l0.mlp.", mlp).numpy()
    got = run_moe(mlp, Wb, h)
    assert rel_err(got, want) < 2e-5
    # what masking with 0 would have chosen: outputs of the groups left out
    s = torch.softmax(h @ W["l0.mlp.router"].T, -1)
    choice = s + W["l0.mlp.correction"]
    assert float(choice.max()) < 0.0
    chosen, w = pp.route(h @ W["l0.mlp.router"].T, W["l0.mlp.correction"], mlp["router"])
    group_best = choice.view(40, 4, 2).max(-1).values
    kept = torch.topk(group_best, 2, dim=-1).indices
    assert all(int(e) // 2 in kept[t].tolist() for t in range(40) for e in chosen[t])
    assert torch.allclose(w.sum(-1), torch.ones(40, dtype=torch.float64))
    # weights from s + bias would be negative here
    assert float(torch.gather(choice, 1, chosen).max()) < 0.0 and float(w.min()) > 0.0


def test_identity_experts_return_their_input():
    """Biases that leave only the identity outputs to choose from: the routed part is route_scale times the input itself."""
    mlp = moe(24, 4, 2, scale=1.75, identity=2, shared=16)
    case = one_layer(attention(2, 1, 16, 16, 0.25), mlp)
    Wb = random_weights(case, 38)
    Wb["l0.mlp.correction"] = torch.tensor([0.0, 0.0, 0.0, 0.0, 5.0, 5.0]).to(torch.bfloat16)
    W = {k: v.double() for k, v in Wb.items()}
    h = torch.randn(12, 80, generator=torch.Generator().manual_seed(39), dtype=torch.float64)
    want = 1.75 * h + pp.gated_expert(h, W, "l0.mlp.shared.")
    assert torch.allclose(pp.moe(h, W, "l0.mlp.", mlp), want, atol=1e-12)
    got = run_moe(mlp, Wb, h)
    # (the engine's feed-forward reads its rows in float32 here; the plain one has them exactly)
    assert rel_err(got, want.numpy()) < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_input_alone(dtype):
    """x + norm(P (gelu(G x) * e)): e is the layer's columns of the second table's row of the token."""
    for D in (12, 1):
        token_input_case(dtype, D)


def token_input_case(dtype, D):
    """(D = 1: the normalised input is a fixed direction whose sign the gated number decides)"""
    from fastgguf_b200.parts import run_part
    E, V, layer, n_layers = 72, 40, 2, 4
    g = torch.Generator().manual_seed(41)
    Wb = {"side.embed": torch.randn(V, D * n_layers, generator=g).to(torch.bfloat16),
          "l2.side.gate": (torch.randn(D, E, generator=g) / E ** 0.5 * 2.0).to(torch.bfloat16),
          "l2.side.proj": (torch.randn(E, D, generator=g) / D ** 0.5).to(torch.bfloat16),
          "l2.side.norm": (1.0 + 0.3 * torch.randn(E, generator=g)).to(torch.bfloat16)}
    W = {k: v.double() for k, v in Wb.items()}
    for rows in (1, 17, 50):
        x = torch.randn(rows, E, generator=g, dtype=torch.float64) * 2.0
        toks = [int(t) for t in torch.randint(0, V, (rows,), generator=g)]
        if D == 1:
            # keep the one gated number away from zero, where the sign would hang on the last bit: the gate's input near 2,
            # tokens whose table entry is not small
            gate = W["l2.side.gate"][0]
            x = 0.1 * x + 2.0 * gate / (gate @ gate)
            big = [t for t in range(V) if abs(float(W["side.embed"][t, layer])) > 0.3]
            toks = [big[t % len(big)] for t in toks]
        want = x + pp.token_side(x, torch.tensor(toks), W, "l2.side.", layer, D, 1e-4)
        params = dict(hidden_size=E, vocab_size=V, dim=D, column=layer * D, table_dim=n_layers * D, eps=1e-4)
        t = {"table": Wb["side.embed"], "gate": Wb["l2.side.gate"], "proj": Wb["l2.side.proj"], "norm": Wb["l2.side.norm"]}
        got = run_part("token_input", "gated_token_embedding", params, t, dtype, tokens=toks, x=f32(x))
        assert rel_err(got, want.numpy()) < (1e-5 if dtype == "float32" else 2e-2)
        # the neighbouring layer's columns give something else (one number a token: the same up to the sign)
        other = x + pp.token_side(x, torch.tensor(toks), W, "l2.side.", layer + 1, D, 1e-4)
        assert D == 1 or rel_err(other.numpy(), want.numpy()) > 5e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", [7, 64, 65])
def test_one_key_at_the_windows_edge(tmp_path, size, dtype):
    """Weights and inputs made so that ONE key far outweighs all others for every later query: the key projection is the
    query projection with its input columns shifted, the special row is the later rows' common direction shifted back.
    The last row that still sees that key returns its value, the next row does not - in a prompt and decoded one by one."""
    layer = attention(2, 1, 16, 16, 1.5, size=size)
    case = one_layer(layer)
    E, special = 80, 20
    T = special + size + 20
    W = random_weights(case, 11)
    W["l0.mix.q"] = W["l0.mix.q"][:16].repeat(2, 1)                 # both query heads ask the one key head the same
    W["l0.mix.k"] = torch.roll(W["l0.mix.q"][:16], 1, dims=1)      # k(h) = q(h shifted back by one column)
    for k in ("l0.mix.q.b", "l0.mix.k.b"):
        W[k] = torch.zeros_like(W[k])
    for k in ("l0.norm1", "l0.mix.q.norm", "l0.mix.k.norm"):
        W[k] = torch.ones_like(W[k])
    d = write_model(tmp_path, case, W)
    W = {k: v.double() for k, v in W.items()}
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, E, generator=g, dtype=torch.float64)
    w = torch.randn(E, generator=g, dtype=torch.float64)
    x[special] = torch.roll(w, 1)                                   # its key is the query of direction w
    x[special + 1:] = w[None, :] + 0.05 * x[special + 1:]
    want = (x + pp.attention_mixer(pp.rms_norm(x, W["l0.norm1"], 1e-5), W, "l0.mix.", layer["mixer"], 1e-5)).numpy()
    last_in, first_out = special + size - 1, special + size
    mixed = want - x.numpy()
    assert np.abs(mixed[last_in] - mixed[first_out]).max() > 0.3 * np.abs(mixed[last_in]).max()      # the edge shows
    tol = 1e-5 if dtype == "float32" else 4e-2
    for cuts in ([T], [last_in - 3] + [1] * (T - last_in + 3), [special + 1, size - 3, 2, 2, 2] + [1] * 16):
        eng = engine_for(d, dtype)
        slot, at, got = eng.acquire(), 0, []
        for n in cuts:
            got.append(eng.block_forward(0, [(slot, n)], f32(x[at:at + n])))
            at += n
        got = np.concatenate(got)
        assert len(got) == T
        for r in (special, special + 1, last_in - 1, last_in, first_out, first_out + 1, T - 1):
            assert rel_err(got[r], want[r]) < tol, (size, cuts[0], r)


# ------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(CASES))
def test_whole_prompt(models, which, dtype):
    """Logits at every position of a prompt that passes every window and page edge of the case."""
    d, case, W = models[(which, dtype)]
    toks = tokens_for(case, 150, 11)
    want = plain_logits(case, W, toks)
    rows = Rows(dtype, conditioning(d, case, W, [toks], dtype))
    eng = engine_for(d, dtype)
    s = eng.acquire()
    got = eng.step_host([entry(s, toks)])
    for p in range(len(toks)):
        rows.add(got[p], want[p], (which, p), 0, p)
    rows.done()
    eng.release(s)
    eng.cache.check()


def test_the_stream_after_every_layer_run(models):
    """The residual stream behind each run of a layer (a looped layer counts each time), through the engine's single-layer
    entry: the token input's rows are those of token 0 there, so the plain layers run with that token too."""
    d, case, W = models[("a", "float32")]
    eng = engine_for(d, "float32")
    T = 40
    x = torch.randn(T, case["width"], generator=torch.Generator().manual_seed(5), dtype=torch.float64)
    zeros = torch.zeros(T, dtype=torch.long)
    slot = eng.acquire()
    for run, (i, _) in enumerate(pp.layer_order(case)):
        want = pp.layer(x, zeros, W, i, case).numpy()
        got = eng.block_forward(run, [(slot, T)], f32(x))
        assert rel_err(got, want) < 1e-5, (run, i)
        # the run wrote into a cache of its own: the same rows again continue the sequence there, and only there
        eng.release(slot)
        slot = eng.acquire()


def test_the_first_tokens(models):
    """Sequences of one, two, three and five tokens, as a prompt and one by one: windows that reach in front of the sequence's
    start see nothing there."""
    for which in CASES:
        d, case, W = models[(which, "float32")]
        eng = engine_for(d, "float32")
        for n in (1, 2, 3, 5):
            toks = tokens_for(case, n, 30 + n)
            want = plain_logits(case, W, toks)
            s = eng.acquire()
            assert rel_err(eng.step_host([entry(s, toks)]), want) < TOL["float32"], (which, n)
            eng.release(s)
            s = eng.acquire()
            got = np.concatenate([eng.step_host([entry(s, [t])]) for t in toks])
            assert rel_err(got, want) < TOL["float32"], (which, n)
            eng.release(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which,cuts", [("a", [2, 2, 3, 17, 33, 64, 65, 2, 31]), ("b", [63, 2, 64, 1, 1, 70, 2, 16]),
                                        ("c", [100, 28, 1, 2, 64, 24]), ("d", [3, 2, 40, 2])])
def test_portions_and_decoding(models, which, cuts, dtype):
    """A prompt cut into portions of many sizes, down to two tokens and one, then 40 tokens one by one: the same logits
    as the whole sequence at every position."""
    d, case, W = models[(which, dtype)]
    n = sum(cuts) + 40
    toks = tokens_for(case, n, 13)
    want = plain_logits(case, W, toks)
    rows = Rows(dtype, conditioning(d, case, W, [toks], dtype))
    eng = engine_for(d, dtype)
    s = eng.acquire()
    at = 0
    for c in cuts + [1] * 40:
        got = eng.step_host([entry(s, toks[at:at + c])])
        for i in range(c):
            rows.add(got[i], want[at + i], (which, at + i, c), 0, at + i)
        at += c
    rows.done()
    eng.release(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(CASES))
def test_batch_of_unequal_requests(models, which, dtype):
    """Five requests of 1 to 140 tokens in one step, then decoded together while the shorter ones leave: every
    request's logits equal those it has alone."""
    d, case, W = models[(which, dtype)]
    lens, total = [1, 140, 64, 7, 65], [9, 150, 70, 30, 66]
    toks = [tokens_for(case, t, 20 + i) for i, t in enumerate(total)]
    want = [plain_logits(case, W, t) for t in toks]
    rows = Rows(dtype, conditioning(d, case, W, toks, dtype))
    eng = engine_for(d, dtype)
    slots = [eng.acquire() for _ in toks]
    got = eng.step_host([entry(s, t[:n]) for s, t, n in zip(slots, toks, lens)])
    row = 0
    for b, n in enumerate(lens):
        for p in range(n):
            rows.add(got[row], want[b][p], (which, b, p), b, p)
            row += 1
    at = list(lens)
    alive = list(range(len(toks)))
    while alive:
        got = eng.step_host([entry(slots[b], [toks[b][at[b]]]) for b in alive])
        for i, b in enumerate(alive):
            rows.add(got[i], want[b][at[b]], (which, b, at[b]), b, at[b])
            at[b] += 1
        for b in [b for b in alive if at[b] == total[b]]:
            eng.release(slots[b])
            alive.remove(b)
    rows.done()
    eng.cache.check()
    assert eng.cache.live_slots() == []


def test_slots_and_pages_used_again(models):
    """Sequences come and go in a cache of two slots and few pages: a new sequence starts from nothing (pages of the one before
    are not read), also after a sequence that was released halfway."""
    d, case, W = models[("b", "float32")]
    eng = engine_for(d, "float32", max_tokens=512, max_batch=2)
    seqs = [tokens_for(case, n, 40 + i) for i, n in enumerate([200, 130, 90, 260, 70, 140])]
    for k, toks in enumerate(seqs):
        s = eng.acquire()
        other = eng.acquire()
        eng.step_host([entry(other, seqs[(k + 1) % len(seqs)][:50], [])])       # a neighbour that is dropped halfway
        want = plain_logits(case, W, toks)
        head = len(toks) - 20
        got = eng.step_host([entry(s, toks[:head], [head - 1])])
        assert rel_err(got[0], want[head - 1]) < TOL["float32"], k
        eng.release(other)
        for p in range(head, len(toks)):
            got = eng.step_host([entry(s, [toks[p]])])
            assert rel_err(got[0], want[p]) < TOL["float32"], (k, p)
        eng.release(s)
        eng.cache.check()


def test_long_decoding_past_windows_and_pages(models):
    """300 tokens one by one after a short prompt: windows slide over decoded tokens and pages leave the windowed groups, while
    the layer without a window keeps every key."""
    d, case, W = models[("b", "float32")]
    toks = tokens_for(case, 330, 50)
    want = plain_logits(case, W, toks)
    eng = engine_for(d, "float32")
    s = eng.acquire()
    eng.step_host([entry(s, toks[:30], [])])
    for p in range(30, 330):
        got = eng.step_host([entry(s, [toks[p]])])
        assert rel_err(got[0], want[p]) < TOL["float32"], p
    assert any(g["window"] for g in eng.cache.groups) and any(not g["window"] for g in eng.cache.groups)
    eng.release(s)
    eng.cache.check()


def test_a_far_token_is_remembered_without_a_window_only(tmp_path):
    """One early token differs between two prompts of 400 tokens.  Through a layer that sees every key the last logits differ by
    far more than rounding, in the engine exactly as in the plain implementation; with windows everywhere they do not differ
    at all (the token input adds nothing from earlier tokens, and two windowed layers reach 2 x 39 tokens back)."""
    for size, differs in ((None, True), (40, False)):
        case = config(64, 90, [(attention(2, 1, 16, 16, 0.5, size=size, rot=(10000.0, 16)), moe(24, 4, 2, identity=1, shared=16)),
                               (attention(2, 2, 16, 16, 0.25, size=40), None)], side=4)
        d, W = make_model(tmp_path / str(size), case, 60, sharp=2.0)
        a = tokens_for(case, 400, 61)
        b = list(a)
        b[3] = (a[3] + 1) % case["vocab"]
        eng = engine_for(d, "float32")
        last = []
        for toks in (a, b):
            s = eng.acquire()
            eng.step_host([entry(s, toks[:380], [])])
            for p in range(380, 400):
                got = eng.step_host([entry(s, [toks[p]])])
            last.append(got[0])
            eng.release(s)
            assert rel_err(got[0], plain_logits(case, W, toks)[-1]) < TOL["float32"]
        gap = np.abs(last[0] - last[1]).max() / np.abs(last[0]).max()
        assert (gap > 1e-4) if differs else (gap < 1e-6), (size, gap)


def test_many_prompt_steps_back_to_back():
    """Forty prompt steps of 2,048 tokens one after another at sizes where every contraction runs on the tensor cores and the
    small kernels between them (casts, gates, combines) are short against them: every step ends, with the same logits."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.registry import config_from_dict
    att = attention(16, 4, 64, 64, 0.125, size=512, rot=(1000000.0, 32), scaling=(8.0, 4096, 32.0, 1.0))
    mlp = moe(1024, 6, 2, scale=2.0, identity=2, groups=(2, 1), shared=1024)
    case = config(1024, 4096, [(att, mlp)] * 4, loop=(0, 4, 1), side=128, eps=1e-6)
    eng = Engine.from_random(config_from_dict(case), 3, dtype="bfloat16", max_tokens=4096, max_batch=2, max_seq_len=4096)
    toks = tokens_for(case, 2048, 90)
    first = None
    for _ in range(40):
        s = eng.acquire()
        got = eng.step_host([entry(s, toks, [2047])])
        eng.release(s)
        assert np.isfinite(got).all()
        if first is None:
            first = got
        assert np.array_equal(got, first)
    eng.cache.check()


# ------------------------------------------------------------------------------ generation through the entry point
@pytest.mark.parametrize("use_graphs", [False, True])
@pytest.mark.parametrize("which", ["a", "b"])
def test_greedy_generation(models, which, use_graphs):
    """Greedy decoding through Engine.generate - the scheduler's batches, the recorded decode step, slots that come
    back - follows the plain implementation: each token is the plain logits' best given the tokens before it (where the
    best two are closer than rounding, either counts)."""
    d, case, W = models[(which, "float32")]
    prompts = [tokens_for(case, n, 70 + i) for i, n in enumerate([5, 70, 1, 33, 12])]
    eng = engine_for(d, "float32", max_tokens=2048, max_batch=4, use_graphs=use_graphs)
    out = eng.generate(prompts, temp=0, max_tokens=24, ignore_eos=True, batch_size=3)
    for p, c in zip(prompts, out):
        assert len(c.tokens) == 24
        logits = plain_logits(case, W, p + c.tokens)
        for i, t in enumerate(c.tokens):
            row = logits[len(p) + i - 1]
            assert row[t] >= row.max() - 1e-4 * np.abs(row).max(), (which, i)
    eng.cache.check()
    assert eng.cache.live_slots() == []


def test_generation_in_bfloat16_runs_the_recorded_step(models):
    d, case, W = models[("c", "bfloat16")]
    prompts = [tokens_for(case, n, 80 + i) for i, n in enumerate([9, 40])]
    eng = engine_for(d, "bfloat16", max_tokens=1024, max_batch=2)
    out = eng.generate(prompts, temp=0, max_tokens=70, ignore_eos=True)
    for p, c in zip(prompts, out):
        logits = plain_logits(case, W, p + c.tokens)
        close = sum(logits[len(p) + i - 1][t] >= logits[len(p) + i - 1].max() - 0.05 * np.abs(logits[len(p) + i - 1]).max()
                    for i, t in enumerate(c.tokens))
        assert close >= 0.9 * len(c.tokens)
    eng.cache.check()


@pytest.mark.parametrize("which", ["a", "b"])
def test_trace_replay_three_cuts(tmp_path, models, which):
    """``bin/trace_run`` on a Pirozen folder in true 32-bit: the same requests whole, with their last 32 tokens one by one, and
    in batches of four unequal requests one batch after another (slots and pages are used again); a cache that holds just what
    the live requests need."""
    from trace_tools import batched_trace, collect, run_trace, tail_trace, whole_trace
    d, case, W = models[(which, "float32")]
    lengths = [5, 9, 1, 17, 3, 40, 11, 70, 33, 130]
    requests = {f"r{i}": tokens_for(case, n, 100 + i) for i, n in enumerate(lengths)}
    want = {rid: plain_logits(case, W, toks) for rid, toks in requests.items()}
    need = max(sum((len(requests[r]) + 63) // 64 * 64 for r in list(requests)[b:b + 4]) for b in range(0, 10, 4))
    cuts = {}
    for name, (steps, index), room in (("whole", whole_trace(requests), 192), ("tail", tail_trace(requests, 32), 192),
                                       ("batched", batched_trace(requests, 4), need)):
        run_trace(d, "float32", steps, str(tmp_path / name), max_tokens=room)
        rows = collect(str(tmp_path / name), steps, index, case["vocab"])
        assert len(rows) == sum(lengths), name
        judge = Rows("float32")
        for (rid, pos), row in rows.items():
            judge.add(row, want[rid][pos], (name, rid, pos))
        judge.done()
        cuts[name] = rows
    for key, row in cuts["whole"].items():
        scale = np.abs(row).max()
        assert np.abs(row - cuts["tail"][key]).max() < 2e-5 * scale and np.abs(row - cuts["batched"][key]).max() < 2e-5 * scale, key


def test_command_line_generates(models):
    """``python -m fastgguf_b200 generate`` on a Pirozen folder: the model class comes from config.json, the tokens are
    those of Engine.generate."""
    import json
    import os
    import subprocess
    import sys
    d, case, W = models[("a", "float32")]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "fastgguf_b200", "generate", d, "256", "--prompt", "5,17,3,200", "--prompt", "9",
                        "--temp", "0", "--max-tokens", "6", "--ignore-eos", "--dtype", "float32", "--json"],
                       cwd=root, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    got = [r["tokens"] for r in json.loads(p.stdout)]
    eng = engine_for(d, "float32", max_tokens=512, max_batch=2)
    want = [c.tokens for c in eng.generate([[5, 17, 3, 200], [9]], temp=0, max_tokens=6, ignore_eos=True)]
    assert got == want
