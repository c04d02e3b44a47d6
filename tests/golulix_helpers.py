"""Shared pieces of the Golulix tests: small configurations that differ from each other in
every size and option, random weights by checkpoint name, crafted weights that make one key
stand out, and a comparison that leaves out positions whose routing was a close call."""
from __future__ import annotations

import copy
from typing import Dict, List, Optional

import torch

from plain_golulix import plain_forward


def _layer(heads, kv, dim, vdim, scale, mask, mlp):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                      "mask": None if mask is None else {"size": mask}},
            "mlp": mlp}


def _moe(experts, top, count, keep, ff, limit, shared):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


# three layers of which two run twice; key and value sizes that differ both ways; a layer without
# feed-forward; grouped and ungrouped routers, top 2 and top 1, with and without a shared expert
GOLU_A = {
    "architecture": "Golulix", "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 61, "mul_prev": 7, "mul_cur": 13}},
    "layers": [_layer(4, 2, 16, 32, 0.3, 24, _moe(8, 2, 4, 2, 48, 1.5, (40, 3.0))),
               _layer(3, 1, 32, 16, 0.2, 40, None),
               _layer(2, 2, 16, 16, 0.25, 17, _moe(6, 1, 1, 1, 32, 1.0, None))],
    "loop": {"start": 1, "stop": 3, "times": 2}, "logit_softcap": 20.0,
}
# head size 64 (the tensor-core attention kernels), a chunk that is no multiple of a page, a layer
# without a mask, more buckets than tokens and large multipliers, no loop, no cap
GOLU_B = {
    "architecture": "Golulix", "vocab": 300, "width": 96, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 1000, "mul_prev": 100003, "mul_cur": 7919}},
    "layers": [_layer(6, 3, 64, 64, 0.11, 100, _moe(4, 2, 2, 1, 64, 2.5, (32, 0.75))),
               _layer(4, 4, 64, 64, 0.15, None, _moe(4, 1, 4, 3, 24, 2.0, (16, 2.0)))],
    "loop": None, "logit_softcap": None,
}
# a width that is no multiple of 8 (products on the FMA kernel), head sizes 24 and 8, every expert
# chosen, the first layer alone run three times
GOLU_C = {
    "architecture": "Golulix", "vocab": 130, "width": 100, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 17, "mul_prev": 1, "mul_cur": 1}},
    "layers": [_layer(5, 5, 24, 8, 0.2, 33, _moe(3, 3, 3, 3, 20, 1.2, (12, 1.2))),
               _layer(2, 1, 8, 24, 0.35, 64, None)],
    "loop": {"start": 0, "stop": 1, "times": 3}, "logit_softcap": 5.0,
}
CONFIGS = {"golu_a": (GOLU_A, 11), "golu_b": (GOLU_B, 12), "golu_c": (GOLU_C, 13)}

TOL = {"float32": 2e-5, "bfloat16": 3e-2, "float16": 4e-3}
CLOSE_CALL = {"float32": 1e-4, "bfloat16": 0.04, "float16": 0.006}


def make_weights(cfg: dict, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    mat = lambda r, c, std: (std * torch.randn(r, c, generator=g)).to(dtype)
    vec = lambda n: (0.1 * torch.randn(n, generator=g)).to(dtype)
    w = {"embed": mat(V, D, 1.0), "final.norm": vec(D), "head": mat(V, D, 0.3)}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        w["bigram"] = mat(bg["buckets"] + 1, D, 0.5)
    s = D ** -0.5
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}"
        w[f"{p}.norm1"] = vec(D)
        w[f"{p}.mix.q"] = mat(m["heads"] * m["dim"], D, 2.0 * s)
        w[f"{p}.mix.k"] = mat(m["kv_heads"] * m["dim"], D, 2.0 * s)
        w[f"{p}.mix.v"] = mat(m["kv_heads"] * m["vdim"], D, s)
        w[f"{p}.mix.g"] = mat(m["heads"], D, 2.0 * s)
        w[f"{p}.mix.o"] = mat(D, m["heads"] * m["vdim"], (m["heads"] * m["vdim"]) ** -0.5)
        f = layer["mlp"]
        if f:
            w[f"{p}.norm2"] = vec(D)
            w[f"{p}.mlp.router"] = mat(f["router"]["experts"], D, 3.0 * s)
            shapes = [(f"e{j}", f["expert"]["ff"]) for j in range(f["router"]["experts"])]
            if f.get("shared"):
                shapes.append(("shared", f["shared"]["ff"]))
            for name, ff in shapes:
                w[f"{p}.mlp.{name}.gate"] = mat(ff, D, 1.5 * s)
                w[f"{p}.mlp.{name}.up"] = mat(ff, D, 1.5 * s)
                w[f"{p}.mlp.{name}.down"] = mat(D, ff, ff ** -0.5)
    return w


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def references(cfg, w, reqs, dtype: str):
    """Plain logits of every request and, per request, how many leading positions are safe to
    compare: those before the first position whose routing anywhere was a close call (the
    library may then choose the other expert, rightly, and what follows differs)."""
    refs, safe = {}, {}
    for rid, toks in reqs.items():
        margins: list = []
        refs[rid] = plain_forward(cfg, w, toks, margins=margins)
        n = len(toks)
        if margins:
            close = (torch.stack(margins).min(0).values < CLOSE_CALL[dtype]).nonzero()
            if close.numel():
                n = int(close[0])
        safe[rid] = n
    return refs, safe


def compare(tr, got, refs, safe, vocab: int, tol: float):
    """Largest error relative to the request's largest logit over the rows that are safe to
    compare; names the first wrong (step, request, position).  Returns (worst, rows compared)."""
    worst, n = 0.0, 0
    for step in sorted(tr.rows):
        rows = tr.rows[step]
        g = got[step].reshape(-1, vocab)
        assert g.shape[0] == len(rows), f"step {step}: {g.shape[0]} rows written, {len(rows)} wanted"
        for i, (rid, pos) in enumerate(rows):
            assert bool(torch.isfinite(g[i]).all()), f"step {step}, request {rid}, position {pos}: not finite"
            if pos >= safe[rid]:
                continue
            err = float((g[i] - refs[rid][pos]).abs().max() / refs[rid].abs().max())
            worst, n = max(worst, err), n + 1
            assert err <= tol, (f"first wrong row: step {step}, request {rid}, position {pos} "
                                f"(row {i} of {len(rows)}): error {err:.3e} > {tol:.1e}")
    return worst, n


def add_portions(tr, rid: str, toks: List[int], sizes: List[int], tag="p"):
    """One request whose prompt comes in portions of the given sizes (the last takes the rest),
    logits at every position."""
    name, at = f"{tag}-{rid}", 0
    tr.need([len(toks)])
    cuts = list(sizes)
    while at < len(toks):
        n = min(cuts.pop(0) if cuts else len(toks), len(toks) - at)
        last = at + n == len(toks)
        tr.add([{"id": name, "tokens": toks[at:at + n], "want": list(range(n))}], [name] if last else [],
               [(rid, p) for p in range(at, at + n)])
        at += n


# ---------------------------------------------------------------------------
# One attention layer without feed-forward whose weights make ONE key stand out: the token
# NEEDLE gets a key along a direction that only the token PROBE asks for, and a value that
# moves the logits.  Whether the needle is visible then decides the probe's logits, so a
# mask that is one position off shows as a large error, not as noise among hundreds of keys.
NEEDLE, PROBE = 3, 5


def needle_model(chunk: int, heads=2, kv=1, dim=16, vdim=16, width=32, vocab=40, scale=0.5):
    cfg = {"architecture": "Golulix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
           "embedding": {"bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 5}},
           "layers": [_layer(heads, kv, dim, vdim, scale, chunk, None)], "loop": None,
           "logit_softcap": None}
    g = torch.Generator().manual_seed(chunk)
    bf = torch.bfloat16
    E = 0.05 * torch.randn(vocab, width, generator=g)
    E[NEEDLE] = 0
    E[NEEDLE, 0] = 4.0
    E[PROBE] = 0
    E[PROBE, 1] = 4.0
    q = 0.02 * torch.randn(heads * dim, width, generator=g)
    k = 0.02 * torch.randn(kv * dim, width, generator=g)
    v = 0.02 * torch.randn(kv * vdim, width, generator=g)
    for h in range(heads):
        q[h * dim, 1] = 3.0                 # the probe asks along feature 0 of every head
    for h in range(kv):
        k[h * dim, 0] = 3.0                 # the needle answers there
        v[h * vdim + 1, 0] = 1.0            # and carries this value
    o = 0.05 * torch.randn(width, heads * vdim, generator=g)
    for h in range(heads):
        o[2, h * vdim + 1] = 1.0            # which lands on a feature of its own
    w = {"embed": E.to(bf), "bigram": torch.zeros(8, width).to(bf), "final.norm": torch.zeros(width).to(bf),
         "head": (0.5 * torch.randn(vocab, width, generator=g)).to(bf),
         "l0.norm1": torch.zeros(width).to(bf), "l0.mix.q": q.to(bf), "l0.mix.k": k.to(bf),
         "l0.mix.v": v.to(bf), "l0.mix.g": torch.zeros(heads, width).to(bf), "l0.mix.o": o.to(bf)}
    return cfg, w


def needle_tokens(n: int, needle_at: int, probes: List[int], vocab=40, seed=0) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(8, vocab, (n,), generator=g).tolist()
    toks[needle_at] = NEEDLE
    for p in probes:
        toks[p] = PROBE
    return toks


def with_sizes(cfg: dict, **changes) -> dict:
    out = copy.deepcopy(cfg)
    out.update(changes)
    return out
