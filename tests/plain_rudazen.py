"""A plain, slow implementation of the Rudazen decoder for tests: whole sequences, no
cache, one function per mechanism, on the CPU.  It reads the raw ``config.json``
dictionary and tensors by their checkpoint names and shares no code with the library
under test.

The design in this file's notation (T tokens, width D, n(u, w) = u / sqrt(mean u^2 + eps) * w):

* embedding: x_t = E[tok_t] * s;
* layer: x <- n(a x + mixer(x), w1); x <- n(a x + ff(x), w2) when the layer has a
  feed-forward; the sublayers read x itself;
* mixer "attention": q = Wq x, k = Wk x; values are k as projected; q and k are each
  normed over the whole projection (all heads at once), then the first ``dims`` features
  of every head are rotated in neighbouring pairs (2i, 2i+1); query i sees the last
  ``size`` positions and, beside them, one (mean key, mean value) for every block of
  ``pool`` positions that lies wholly before that window; one softmax over both;
* mixer "parallel": half the sum of two branches, each normed over the width with a
  weight of its own.  Left: attention with its own value projection, the same whole-projection
  norms, rotation of pairs (i, i + dims/2) with YaRN-scaled frequencies, a factor per head on
  the scores, a plain window, and sigmoid(Wg x) on the concatenated heads before the output
  projection.  Right: a gated linear recurrence per head, S_t = diag(f_t) S_(t-1) +
  (1 - f_t) v_t^T, o_t = S_t^T q_t with q = silu(Wq x), f = l + (1 - l) sigmoid(Wf x + b),
  each head's o normed over its value size;
* feed-forward: down(silu(gate x) * (up x));
* output: n(x, w_final), head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def plain_norm(u: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    ms = (u * u).mean(-1, keepdim=True)
    return u / torch.sqrt(ms + eps) * weight.to(u.dtype)


def plain_embedding(w, cfg: dict, tokens: Sequence[int], dt) -> torch.Tensor:
    scale = float((cfg.get("embedding") or {}).get("scale", 1.0))
    return w["embed"].to(dt)[torch.tensor(list(tokens), dtype=torch.long)] * scale


# ----------------------------------------------------------------------------- rotation
def plain_frequencies(rot: dict, dt) -> (torch.Tensor, float):
    """The angle per position of every rotated pair, and the factor on cos and sin."""
    dims = int(rot["dims"])
    base = float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])
        where = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(where(float(sc["fast"]))), 0)
        hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    return f.to(dt), mult


def plain_rotate(u: torch.Tensor, rot: Optional[dict], layout: str, first_pos: int = 0) -> torch.Tensor:
    """u [T, heads, size]; the first rot['dims'] features of each head are rotated, the rest pass.
    layout 'pairs': (2i, 2i+1); 'halves': (i, i + dims/2)."""
    if not rot:
        return u
    T = u.shape[0]
    dims = int(rot["dims"])
    f, mult = plain_frequencies(rot, torch.float32)
    pos = torch.arange(first_pos, first_pos + T, dtype=torch.float32)
    ang = (pos[:, None] * f[None, :]).to(u.dtype)              # angles in 32 bits, as the design asks
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    out = u.clone()
    if layout == "pairs":
        a, b = u[..., 0:dims:2], u[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = u[..., :dims // 2], u[..., dims // 2:dims]
        out[..., :dims // 2] = a * c - b * s
        out[..., dims // 2:dims] = b * c + a * s
    return out


# ------------------------------------------------------------------------------- masks
def plain_window_mask(T: int, size: Optional[int]) -> torch.Tensor:
    """[T, T] bool: query i (row) sees key j (column): 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if size:
        m = m & (i - j < size)
    return m


def plain_pool_mask(T: int, size: int, pool: int) -> torch.Tensor:
    """[T, blocks] bool: query i sees block b (positions b pool .. b pool + pool - 1) when the
    block's last position is at most i - size."""
    n_blocks = T // pool
    i = torch.arange(T)[:, None]
    b = torch.arange(n_blocks)[None, :]
    return (b * pool + pool - 1) <= (i - size)


def plain_softmax_mix(scores: torch.Tensor, mask: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    """scores [T, K], mask [T, K], values [K, dv] -> [T, dv]."""
    s = scores.masked_fill(~mask, float("-inf"))
    return torch.softmax(s, -1) @ values


# -------------------------------------------------------------------------------- mixers
def plain_qk(w, p: str, m: dict, h: torch.Tensor, eps: float, layout: str):
    """Normed (over the whole projection) and rotated q [T, H, dk], k [T, G, dk], and the
    key projection as it came out, [T, G, dk]."""
    T = h.shape[0]
    H, G, dk = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q_raw = h @ w[f"{p}.q"].to(h.dtype).T
    k_raw = h @ w[f"{p}.k"].to(h.dtype).T
    q = plain_norm(q_raw, w[f"{p}.q.norm"], eps).view(T, H, dk)
    k = plain_norm(k_raw, w[f"{p}.k.norm"], eps).view(T, G, dk)
    rot = m.get("rot")
    return plain_rotate(q, rot, layout), plain_rotate(k, rot, layout), k_raw.view(T, G, dk)


def plain_pooled_attention(w, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """The 'attention' mixer: values are the keys as projected; window plus pooled blocks."""
    T = h.shape[0]
    H, G, dv = int(m["heads"]), int(m["kv_heads"]), int(m["vdim"])
    q, k, v = plain_qk(w, p, m, h, eps, "pairs")
    mask = m.get("mask") or {}
    size, pool = mask.get("size"), mask.get("pool")
    near = plain_window_mask(T, size)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        keys, vals, see = k[:, g], v[:, g], near
        if size and pool:
            nb = T // pool
            if nb:
                kb = k[:nb * pool, g].reshape(nb, pool, -1).mean(1)
                vb = v[:nb * pool, g].reshape(nb, pool, -1).mean(1)
                keys, vals = torch.cat([kb, keys], 0), torch.cat([vb, vals], 0)
                see = torch.cat([plain_pool_mask(T, int(size), int(pool)), near], 1)
        scores = (q[:, hh] @ keys.T) * float(m["scale"])
        out[:, hh] = plain_softmax_mix(scores, see, vals)
    return out.reshape(T, H * dv) @ w[f"{p}.o"].to(h.dtype).T


def plain_gated_window_attention(w, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """The left branch of 'parallel'."""
    T = h.shape[0]
    H, G, dv = int(m["heads"]), int(m["kv_heads"]), int(m["vdim"])
    q, k, _ = plain_qk(w, p, m, h, eps, "halves")
    v = (h @ w[f"{p}.v"].to(h.dtype).T).view(T, G, dv)
    see = plain_window_mask(T, (m.get("mask") or {}).get("size"))
    temp = w[f"{p}.temp"].to(h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        scores = (q[:, hh] @ k[:, g].T) * float(m["scale"]) * temp[hh]
        out[:, hh] = plain_softmax_mix(scores, see, v[:, g])
    gate = torch.sigmoid(h @ w[f"{p}.g"].to(h.dtype).T)
    return (out.reshape(T, H * dv) * gate) @ w[f"{p}.o"].to(h.dtype).T


def plain_gated_recurrence(w, p: str, m: dict, h: torch.Tensor, eps: float,
                           state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The right branch of 'parallel', token by token."""
    T = h.shape[0]
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = torch.nn.functional.silu(h @ w[f"{p}.q"].to(h.dtype).T).view(T, H, dk)
    v = (h @ w[f"{p}.v"].to(h.dtype).T).view(T, H, dv)
    low = w[f"{p}.lower"].to(h.dtype)
    f = low + (1.0 - low) * torch.sigmoid(h @ w[f"{p}.f"].to(h.dtype).T + w[f"{p}.f.b"].to(h.dtype))
    f = f.view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=h.dtype) if state is None else state
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = plain_norm(o, w[f"{p}.norm"], eps)
    return o.reshape(T, H * dv) @ w[f"{p}.o"].to(h.dtype).T


def plain_parallel(w, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    left = plain_gated_window_attention(w, f"{p}.left", m["left"], h, eps)
    right = plain_gated_recurrence(w, f"{p}.right", m["right"], h, eps)
    return 0.5 * (plain_norm(left, w[f"{p}.left.out"], eps) + plain_norm(right, w[f"{p}.right.out"], eps))


def plain_feed_forward(w, p: str, h: torch.Tensor) -> torch.Tensor:
    g = h @ w[f"{p}.gate"].to(h.dtype).T
    u = h @ w[f"{p}.up"].to(h.dtype).T
    return (torch.nn.functional.silu(g) * u) @ w[f"{p}.down"].to(h.dtype).T


# ------------------------------------------------------------------------------- model
def plain_forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
                  layers_out: Optional[List[torch.Tensor]] = None, dt=torch.float32) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layers_out`` collects x after every layer."""
    eps = float(cfg["norm"]["eps"])
    alpha = float(cfg.get("postln_alpha", 1.0))
    x = plain_embedding(w, cfg, tokens, dt)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        if layer["type"] == "attention":
            y = plain_pooled_attention(w, f"{p}.mix", layer["mixer"], x, eps)
        elif layer["type"] == "parallel":
            y = plain_parallel(w, f"{p}.mix", layer["mixer"], x, eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = plain_norm(alpha * x + y, w[f"{p}.norm1"], eps)
        if layer.get("mlp"):
            x = plain_norm(alpha * x + plain_feed_forward(w, f"{p}.mlp", x), w[f"{p}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return plain_norm(x, w["final.norm"], eps) @ w["head"].to(dt).T
