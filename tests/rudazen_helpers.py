"""Shared pieces of the Rudazen tests: small configurations that differ from each other in every
size and option, random weights by checkpoint name, and crafted one-layer models in which ONE
key stands out, so that a mask that is one position off shows as a large error."""
from __future__ import annotations

import copy
from typing import Dict, List, Optional

import torch

from plain_rudazen import plain_forward


def _att(heads, kv, dim, vdim, scale, size, pool=None, rot=None):
    mask = {"size": size}
    if pool:
        mask["pool"] = pool
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": mask}
    if rot:
        m["rot"] = rot
    return m


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _mlp(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def attention_layer(mixer, ff):
    return {"type": "attention", "mixer": mixer, "mlp": _mlp(ff)}


def parallel_layer(left, right, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": dict(zip(("heads", "dim", "vdim"), right))},
            "mlp": _mlp(ff)}


# key and value sizes that differ in the left branch, rotation of a part of the head with YaRN,
# a layer without feed-forward, a pool smaller than its window and one larger than its window
RUDA_A = {
    "architecture": "Rudazen", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 1.7,
    "embedding": {"scale": 8.0},
    "layers": [parallel_layer(_att(4, 2, 16, 32, 0.3, 24, rot=_rot(1e4, 8, (4.0, 64, 16.0, 2.0))), (3, 24, 16), 96),
               attention_layer(_att(4, 1, 16, 16, 0.25, 20, pool=6, rot=_rot(5e5, 16)), None),
               attention_layer(_att(2, 2, 32, 32, 0.2, 16, pool=40, rot=_rot(1e4, 8)), 80)],
}
# head size 64, windows and pools that are no multiple of a page, alpha 1 and scale 1
RUDA_B = {
    "architecture": "Rudazen", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "postln_alpha": 1.0,
    "embedding": {"scale": 1.0},
    "layers": [attention_layer(_att(6, 3, 64, 64, 0.11, 100, pool=16, rot=_rot(1e6, 64)), 128),
               parallel_layer(_att(2, 2, 64, 64, 0.15, 70, rot=_rot(1e4, 32)), (1, 8, 40), 64)],
}
# a width that is no multiple of 8 (products on the FMA kernel), head sizes 24 / 8 and 20 / 12, a
# mixer without rotation, a pool of 3 before a window of 7
RUDA_C = {
    "architecture": "Rudazen", "vocab": 130, "width": 100, "norm": {"eps": 1e-5}, "postln_alpha": 3.0,
    "embedding": {"scale": 0.5},
    "layers": [parallel_layer(_att(5, 5, 24, 8, 0.2, 33, rot=_rot(1e4, 24, (8.0, 32, 8.0, 1.0))), (2, 20, 12), None),
               attention_layer(_att(3, 1, 8, 8, 0.35, 7, pool=3), 50)],
}
CONFIGS = {"ruda_a": (RUDA_A, 21), "ruda_b": (RUDA_B, 32), "ruda_c": (RUDA_C, 23)}

# Largest logit error relative to the request's largest logit.  The 16-bit bounds are wider than a
# pre-norm decoder's: every sublayer's input is the normed stream rounded to 16 bits, and a norm
# after the sum (and the scale-free norms of heads and branches) passes a rounding error on at
# full size instead of adding it to a large residual.
TOL = {"float32": 2e-5, "bfloat16": 6e-2, "float16": 8e-3}


def make_weights(cfg: dict, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    mat = lambda r, c, std: (std * torch.randn(r, c, generator=g)).to(dtype)
    ones = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g)).to(dtype)
    w = {"embed": mat(V, D, 1.0), "final.norm": ones(D), "head": mat(V, D, 0.3)}
    s = D ** -0.5

    def attention(p, m, own_values):
        w[f"{p}.q"] = mat(m["heads"] * m["dim"], D, 2.0 * s)
        w[f"{p}.k"] = mat(m["kv_heads"] * m["dim"], D, 2.0 * s)
        w[f"{p}.q.norm"] = ones(m["heads"] * m["dim"])
        w[f"{p}.k.norm"] = ones(m["kv_heads"] * m["dim"])
        w[f"{p}.o"] = mat(D, m["heads"] * m["vdim"], 2.0 * (m["heads"] * m["vdim"]) ** -0.5)
        if own_values:
            w[f"{p}.v"] = mat(m["kv_heads"] * m["vdim"], D, 2.0 * s)
            w[f"{p}.g"] = mat(m["heads"] * m["vdim"], D, 2.0 * s)
            w[f"{p}.temp"] = (1.0 + 0.3 * torch.randn(m["heads"], generator=g)).to(dtype)

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        w[f"{p}.norm1"] = ones(D)
        if layer["type"] == "attention":
            attention(f"{p}.mix", layer["mixer"], False)
        else:
            attention(f"{p}.mix.left", layer["mixer"]["left"], True)
            r = layer["mixer"]["right"]
            q = f"{p}.mix.right"
            w[f"{q}.q"] = mat(r["heads"] * r["dim"], D, 2.0 * s)
            w[f"{q}.f"] = mat(r["heads"] * r["dim"], D, 3.0 * s)
            w[f"{q}.f.b"] = torch.randn(r["heads"] * r["dim"], generator=g).to(dtype)
            w[f"{q}.lower"] = (0.9 * torch.rand(r["heads"] * r["dim"], generator=g)).to(dtype)
            w[f"{q}.v"] = mat(r["heads"] * r["vdim"], D, 2.0 * s)
            w[f"{q}.norm"] = ones(r["vdim"])
            w[f"{q}.o"] = mat(D, r["heads"] * r["vdim"], 2.0 * (r["heads"] * r["vdim"]) ** -0.5)
            w[f"{p}.mix.left.out"] = ones(D)
            w[f"{p}.mix.right.out"] = ones(D)
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            w[f"{p}.norm2"] = ones(D)
            w[f"{p}.mlp.gate"] = mat(ff, D, 1.5 * s)
            w[f"{p}.mlp.up"] = mat(ff, D, 1.5 * s)
            w[f"{p}.mlp.down"] = mat(D, ff, 2.0 * ff ** -0.5)
    return w


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def references(cfg, w, reqs) -> Dict[str, torch.Tensor]:
    return {rid: plain_forward(cfg, w, toks) for rid, toks in reqs.items()}


def plain_generate_greedy(cfg, w, prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(plain_forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


# ---------------------------------------------------------------------------
# One layer whose weights make ONE key stand out: the token NEEDLE gets a key along a feature
# that rotation leaves alone and that only the token PROBE asks for, and a value that moves the
# logits.  Whether the needle (or the pooled block that holds it) is visible then decides the
# probe's logits.
NEEDLE, PROBE = 3, 5


def needle_model(kind: str, size: int, pool: Optional[int] = None, heads=2, kv=1, dim=16, width=32,
                 vocab=40, scale=2.0, rot_dims=8):
    att = _att(heads, kv, dim, dim, scale, size, pool=pool, rot=_rot(1e4, rot_dims))
    layer = attention_layer(att, None) if kind == "attention" else parallel_layer(att, (1, 8, 8), None)
    cfg = {"architecture": "Rudazen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
           "postln_alpha": 1.0, "embedding": {"scale": 2.0}, "layers": [layer]}
    g = torch.Generator().manual_seed(size * 131 + (pool or 0))
    bf = torch.bfloat16
    E = 0.05 * torch.randn(vocab, width, generator=g)
    E[:, :2] = 0                                   # features 0 and 1 belong to the needle and the probe
    E[NEEDLE] = 0
    E[NEEDLE, 0] = 4.0
    E[PROBE] = 0
    E[PROBE, 1] = 4.0
    q = 0.02 * torch.randn(heads * dim, width, generator=g)
    k = 0.02 * torch.randn(kv * dim, width, generator=g)
    o = 0.05 * torch.randn(width, heads * dim, generator=g)
    f = rot_dims                                   # the first feature of a head that is not rotated
    for h in range(heads):
        q[h * dim + f] = 0
        q[h * dim + f, 1] = 3.0                    # the probe alone asks along that feature of every head
    for h in range(kv):
        k[h * dim + f] = 0
        k[h * dim + f, 0] = 3.0                    # the needle alone answers there
    p = "l0.mix" if kind == "attention" else "l0.mix.left"
    w = {"embed": E.to(bf), "final.norm": torch.ones(width).to(bf),
         "head": (0.5 * torch.randn(vocab, width, generator=g)).to(bf), "l0.norm1": torch.ones(width).to(bf),
         f"{p}.q": q.to(bf), f"{p}.k": k.to(bf), f"{p}.q.norm": torch.ones(heads * dim).to(bf),
         f"{p}.k.norm": torch.ones(kv * dim).to(bf)}
    if kind == "attention":
        for h in range(heads):
            o[2, h * dim + f] = 1.0                # the needle's value is its key as projected
    else:
        v = 0.02 * torch.randn(kv * dim, width, generator=g)
        for h in range(kv):
            v[h * dim + 1, 0] = 1.0
        for h in range(heads):
            o[2, h * dim + 1] = 1.0
        w.update({f"{p}.v": v.to(bf), f"{p}.g": torch.zeros(heads * dim, width).to(bf),
                  f"{p}.temp": torch.ones(heads).to(bf), "l0.mix.left.out": torch.ones(width).to(bf),
                  "l0.mix.right.out": torch.ones(width).to(bf)})
        r = "l0.mix.right"
        w.update({f"{r}.q": (0.1 * torch.randn(8, width, generator=g)).to(bf),
                  f"{r}.f": (0.1 * torch.randn(8, width, generator=g)).to(bf),
                  f"{r}.f.b": torch.zeros(8).to(bf), f"{r}.lower": torch.full((8,), 0.5).to(bf),
                  f"{r}.v": (0.1 * torch.randn(8, width, generator=g)).to(bf),
                  f"{r}.norm": torch.ones(8).to(bf), f"{r}.o": torch.zeros(width, 8).to(bf)})
    w[f"{p}.o"] = o.to(bf)
    return cfg, w


def needle_tokens(n: int, needle_at: int, probes: List[int], vocab=40, seed=0) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(8, vocab, (n,), generator=g).tolist()
    toks[needle_at] = NEEDLE
    for p in probes:
        toks[p] = PROBE
    return toks


def with_mask(cfg: dict, **mask) -> dict:
    """The one-layer configuration with other mask numbers (what a library that is one off computes)."""
    out = copy.deepcopy(cfg)
    m = out["layers"][0]["mixer"]
    (m if "mask" in m else m["left"])["mask"].update(mask)
    return out


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
