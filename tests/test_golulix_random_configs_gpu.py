"""Randomly drawn Golulix configurations through the engine against the plain implementation:
key and value sizes from 8 to 256 that agree or differ, any number of heads and kv heads, widths
and feed-forward sizes that are no multiple of 8, chunks from 1 position to longer than the
prompts, routers with and without groups, top from 1 to all experts, layers without feed-forward,
loops anywhere, with and without a cap; prompts whole or cut in two, then tokens one by one.
32-bit compares every position; bfloat16 those before the plain implementation's first close
routing call."""
import random

import pytest
import torch

from golulix_helpers import CLOSE_CALL, TOL, make_weights, random_tokens
from plain_golulix import plain_forward

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    n_layers = rng.choice([1, 2, 3])
    layers = []
    for _ in range(n_layers):
        G = rng.choice([1, 2, 3])
        H = G * rng.choice([1, 2, 4, 5])
        dim = rng.choice([8, 16, 24, 32, 64, 80, 128, 256])
        vdim = rng.choice([dim, dim, 8, 16, 40, 64, 128])
        mlp = None
        if rng.random() < 0.75:
            count = rng.choice([1, 1, 2, 4])
            per = rng.choice([1, 2, 3, 4])
            keep = rng.randint(1, count)
            top = rng.randint(1, keep * per)
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([8, 20, 32, 72]), "limit": rng.choice([0.8, 2.0, 7.0])},
                   "router": {"experts": count * per, "top": top, "groups": {"count": count, "keep": keep}},
                   "shared": rng.choice([None, {"ff": rng.choice([12, 40, 64]), "limit": rng.choice([1.0, 5.0])}])}
        layers.append({"type": "attention",
                       "mixer": {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim,
                                 "scale": rng.choice([0.05, 0.2, dim ** -0.5]),
                                 "mask": rng.choice([None, {"size": rng.choice([1, 7, 64, 65, 100, 128, 400])}])},
                       "mlp": mlp})
    start = rng.randint(0, n_layers - 1)
    cfg = {"architecture": "Golulix", "vocab": rng.choice([61, 256, 500]),
           "width": rng.choice([24, 64, 72, 100, 136]), "norm": {"eps": rng.choice([1e-5, 1e-6])},
           "embedding": {"bigram": {"buckets": rng.choice([1, 17, 4099]), "mul_prev": rng.choice([1, 29, 1000003]),
                                    "mul_cur": rng.choice([1, 13, 999983])}},
           "layers": layers,
           "loop": rng.choice([None, {"start": start, "stop": rng.randint(start + 1, n_layers),
                                      "times": rng.choice([1, 2, 3])}]),
           "logit_softcap": rng.choice([None, 8.0, 30.0])}
    lens = [rng.randint(1, 230) for _ in range(rng.choice([1, 2, 3]))]
    return cfg, lens, rng.random() < 0.5


# 207, 277, 295: key size 8 in prompts of more than 128 tokens (the q/k/v product's storing
# epilogue takes head sizes from 16 on; these once went to it)
@pytest.mark.parametrize("seed", list(range(21, 45)) + [207, 277, 295])
def test_a_random_configuration_matches_the_plain_model(seed):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, lens, cut = draw(seed)
    w = make_weights(cfg, 100 + seed)
    toks = [random_tokens(n + 6, cfg["vocab"], 7 * seed + i) for i, n in enumerate(lens)]
    refs, margins = [], []
    for t in toks:
        m: list = []
        refs.append(plain_forward(cfg, w, t, margins=m))
        margins.append(torch.stack(m).min(0).values if m else torch.full((len(t),), float("inf")))
    for dtype in ("float32", "bfloat16"):
        safe = []
        for m in margins:
            close = (m < CLOSE_CALL[dtype]).nonzero()
            safe.append(int(close[0]) if close.numel() else len(m))
        lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=len(lens), max_context=256,
                max_tokens=rng_tokens(lens))
        s = lm.acquire(len(lens))
        worst, seen = 0.0, 0

        def see(logits, i, pos):
            nonlocal worst, seen
            assert bool(torch.isfinite(logits).all()), (dtype, cfg, lens, i, pos)
            if pos < safe[i]:
                seen += 1
                worst = max(worst, float((logits - refs[i][pos]).abs().max() / refs[i].abs().max()))

        if cut:
            first = [max(1, n // 2) for n in lens]
            lg = lm.step([t[:c] for t, c in zip(toks, first)], s, [[c - 1] for c in first]).cpu()
            for i, c in enumerate(first):
                see(lg[i], i, c - 1)
            rest = [i for i, (c, n) in enumerate(zip(first, lens)) if n > c]
            if rest:
                lg = lm.step([toks[i][first[i]:lens[i]] for i in rest], [s[i] for i in rest],
                             [[lens[i] - first[i] - 1] for i in rest]).cpu()
                for k, i in enumerate(rest):
                    see(lg[k], i, lens[i] - 1)
        else:
            lg = lm.step([t[:n] for t, n in zip(toks, lens)], s, [[0, n - 1] for n in lens]).cpu()
            for i, n in enumerate(lens):
                see(lg[2 * i], i, 0)
                see(lg[2 * i + 1], i, n - 1)
        for k in range(6):
            lg = lm.step([[t[n + k]] for t, n in zip(toks, lens)], s, [[0]] * len(lens)).cpu()
            for i, n in enumerate(lens):
                see(lg[i], i, n + k)
        lm.release(s)
        lm.rt.check_status()
        assert worst <= TOL[dtype], (dtype, cfg, lens, cut, worst)
        assert seen > 0 or dtype != "float32"


def rng_tokens(lens):
    """The page budget of a trace with these requests (each count rounded up to a page)."""
    return sum((n + 6 + 63) // 64 * 64 for n in lens)
