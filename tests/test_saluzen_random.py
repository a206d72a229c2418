"""Seeded random Saluzen configurations, engine against the plain implementation: every size, the order and mix of layers,
heads and groups, taps, chunks, rotated dimensions, frequency scaling, latent sizes, which layers read an earlier layer's
latents, and the pair's scales are drawn; then a batch of unequal prompts, portions, and decode steps during which sequences
leave.  float32 engines are held to the float32 tolerance everywhere; bfloat16 engines run the same model with sharpened
attention."""
import numpy as np
import pytest

from saluzen_cases import attn, config, delta, dense, latent, make_model, parallel, parallel_2, ssm
from test_saluzen import Rows, engine_for, entry, plain_logits

pytestmark = pytest.mark.gpu


def draw_left(rng, chunked):
    kv, dk = int(rng.choice([1, 2, 3])), int(rng.choice([16, 32, 64, 128, 24, 96]))
    dv = dk if rng.random() < 0.6 else int(rng.choice([16, 40, 64, 96]))
    rot, scaling = None, None
    if rng.random() < 0.85:
        rot = (float(rng.choice([10.0, 1e4, 1e6])), int(rng.choice([d for d in (8, 16, 24, 32, 64, 96, 128) if d <= dk])))
        if rng.random() < 0.5:
            low = float(rng.choice([1.0, 2.0]))
            scaling = (float(rng.choice([2.0, 4.0, 32.0])), low, low * float(rng.choice([2.0, 4.0])), int(rng.choice([16, 64, 2048])))
    size = int(rng.choice([1, 5, 17, 63, 64, 65, 100, 300])) if chunked else None
    return attn(kv * int(rng.choice([1, 2, 4, 5])), kv, dk, dv, float(rng.uniform(0.05, 0.3)), rot=rot, scaling=scaling, size=size)


def draw_config(rng):
    width = int(rng.choice([64, 96, 128, 160, 200, 72, 256]))
    n_layers = int(rng.integers(1, 6))
    layers, owners = [], []
    for i in range(n_layers):
        kind = rng.integers(3)
        if kind == 0:
            groups = int(rng.choice([1, 2, 3]))
            heads = groups * int(rng.choice([1, 2, 4]))
            vdim = int(rng.choice([8, 16, 32, 64, 24]))
            norm_groups = int(rng.choice([g for g in (1, 2, 4, heads, 2 * heads) if (heads * vdim) % g == 0]))
            mixer = parallel(draw_left(rng, False), ssm(heads, vdim, int(rng.choice([8, 16, 20, 64, 128])), groups, int(rng.integers(1, 5)), norm_groups))
        elif kind == 1:
            kv = int(rng.choice([1, 2, 3]))
            mixer = parallel_2(draw_left(rng, True), delta(kv * int(rng.choice([1, 2, 3])), kv, int(rng.choice([8, 16, 32, 64, 128, 24])),
                                                           int(rng.choice([8, 16, 32, 64, 128, 40])), int(rng.integers(1, 5))),
                               float(rng.uniform(0.3, 1.5)), float(rng.uniform(0.3, 1.5)))
        else:
            if owners and rng.random() < 0.5:
                j = int(rng.choice(owners))
                o = layers[j][0]["mixer"]
                mixer = latent(int(rng.integers(1, 7)), int(rng.choice([16, 32, 64, 24])), o["rot_dim"], int(rng.choice([16, 32, 64, 40])), o["kv_rank"],
                               int(rng.choice([24, 64, 96])), float(rng.uniform(0.05, 0.3)), o["rot"]["base"], kv_from=j)
            else:
                mixer = latent(int(rng.integers(1, 7)), int(rng.choice([16, 32, 64, 96, 24])), int(rng.choice([8, 16, 32, 64])),
                               int(rng.choice([16, 32, 64, 128, 40])), int(rng.choice([16, 40, 64, 128, 192])), int(rng.choice([24, 64, 96])),
                               float(rng.uniform(0.05, 0.3)), float(rng.choice([100.0, 1e4, 5e5])))
                owners.append(i)
        layers.append((mixer, None if rng.random() < 0.2 else dense(int(rng.choice([64, 100, 192, 320])))))
    return config(width, int(rng.integers(40, 500)), layers, eps=float(rng.choice([1e-5, 1e-6])))


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22])
def test_random_configuration(tmp_path, seed):
    rng = np.random.default_rng(seed)
    cfg = draw_config(rng)
    dtype = "bfloat16" if seed % 3 == 0 else "float32"
    d, W = make_model(tmp_path, cfg, seed, sharp=2.0 if dtype == "bfloat16" else 1.0)
    B = int(rng.integers(1, 5))
    total = [int(rng.integers(3, 200)) for _ in range(B)]
    first = [int(rng.integers(1, t)) for t in total]
    toks = [[int(t) for t in rng.integers(0, cfg["vocab"], size=n)] for n in total]
    want = [plain_logits(cfg, W, t) for t in toks]
    eng = engine_for(d, dtype)
    slots = [eng.acquire() for _ in toks]
    got = eng.step_host([entry(s, t[:n]) for s, t, n in zip(slots, toks, first)])
    row = 0
    judge = Rows(dtype)
    for b, n in enumerate(first):
        for p in range(n):
            judge.add(got[row], want[b][p], (seed, b, p))
            row += 1
    at = list(first)
    # one more portion for the first sequence, then everyone token by token
    if total[0] - at[0] > 3:
        n = int(rng.integers(2, total[0] - at[0]))
        got = eng.step_host([entry(slots[0], toks[0][at[0]:at[0] + n])])
        for i in range(n):
            judge.add(got[i], want[0][at[0] + i], (seed, "portion", at[0] + i))
        at[0] += n
    alive = [b for b in range(B) if at[b] < total[b]]
    for b in [b for b in range(B) if at[b] == total[b]]:
        eng.release(slots[b])
    while alive:
        got = eng.step_host([entry(slots[b], [toks[b][at[b]]]) for b in alive])
        for i, b in enumerate(alive):
            judge.add(got[i], want[b][at[b]], (seed, b, at[b]))
            at[b] += 1
        for b in [b for b in alive if at[b] == total[b]]:
            eng.release(slots[b])
            alive.remove(b)
    judge.done()
    eng.cache.check()
    assert eng.cache.live_slots() == []
