"""A plain, slow implementation of the Golulix decoder for tests: whole sequences,
no cache, one function per mechanism, 32-bit floats on the CPU.  It reads the raw
``config.json`` dictionary and tensors by their checkpoint names and shares no code
with the library under test.

The design in this file's notation (T tokens, width D):

* embedding: x_t = E[tok_t] + B[r_t], r_0 = buckets and
  r_t = (tok_{t-1} * mul_prev + tok_t * mul_cur) mod buckets for t > 0;
* layer order: layers ``start .. stop - 1`` run ``times`` times in a row with the
  same weights; before every repetition but the first the embedding output is
  added to x;
* layer: x += mixer(n1(x)); x += ff(n2(x)) when the layer has a feed-forward;
  n(x) = x / sqrt(mean(x^2) + eps) * (1 + w);
* mixer: q, k, v projections without rotation; score_ij = scale * q_i . k_j for
  j <= i with i // C == j // C (C = mask size); softmax; head outputs multiplied by
  sigmoid of a per-head projection of the mixer's input; output projection;
* feed-forward: routed experts (softmax over all experts, only experts of the
  ``keep`` best groups eligible, the ``top`` largest chosen, weighted by their
  scores as they are) plus a shared expert; an expert is
  down(min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u, -L, L) + 1));
* output: final norm, head, cap * tanh(logits / cap).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch


def plain_bigram_rows(tokens: Sequence[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def plain_embedding(w: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int]) -> torch.Tensor:
    x = w["embed"].float()[torch.tensor(list(tokens), dtype=torch.long)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        rows = plain_bigram_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))
        x = x + w["bigram"].float()[torch.tensor(rows, dtype=torch.long)]
    return x


def plain_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    ms = (x.float() ** 2).mean(-1, keepdim=True)
    return x.float() / torch.sqrt(ms + eps) * (1.0 + weight.float())


def plain_chunk_mask(T: int, size: Optional[int]) -> torch.Tensor:
    """[T, T] bool: query i (row) sees key j (column)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if size:
        m = m & ((i // size) == (j // size))
    return m


def plain_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    """h: [T, D], the mixer's input; returns the mixer's output [T, D]."""
    T = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[f"{p}.q"].float().T).view(T, H, dk)
    k = (h @ w[f"{p}.k"].float().T).view(T, G, dk)
    v = (h @ w[f"{p}.v"].float().T).view(T, G, dv)
    gate = torch.sigmoid(h @ w[f"{p}.g"].float().T)                    # [T, H]
    size = (m.get("mask") or {}).get("size")
    mask = plain_chunk_mask(T, size)
    out = torch.zeros(T, H, dv)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~mask, float("-inf"))
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[f"{p}.o"].float().T


def plain_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[f"{p}.gate"].float().T, max=limit)
    u = torch.clamp(h @ w[f"{p}.up"].float().T, min=-limit, max=limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return y @ w[f"{p}.down"].float().T


def plain_route(z: torch.Tensor, r: dict):
    """z: [T, E] router logits.  Returns (chosen [T, top] long, weights [T, top], margin [T]):
    margin is how far, relative to the score that was taken last, the nearest score that was
    not taken lies from it (a group's or an expert's): a small margin is a close call."""
    E, top = int(r["experts"]), int(r["top"])
    s = torch.softmax(z.float(), -1)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    n_g, keep = int(groups["count"]), int(groups["keep"])
    per = E // n_g
    best = s.view(-1, n_g, per).max(-1).values                           # [T, n_g]
    ranked = best.sort(-1, descending=True).values
    margin = torch.full((s.shape[0],), float("inf"))
    if keep < n_g:
        margin = (ranked[:, keep - 1] - ranked[:, keep]) / ranked[:, keep - 1]
    chosen_groups = best.topk(keep, -1).indices
    allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, chosen_groups, True)
    allowed = allowed[:, :, None].expand(-1, -1, per).reshape(-1, E)
    masked = s.masked_fill(~allowed, float("-inf"))
    order = masked.sort(-1, descending=True)
    idx = order.indices[:, :top]
    if top < keep * per:
        margin = torch.minimum(margin, (order.values[:, top - 1] - order.values[:, top]) / order.values[:, top - 1])
    return idx, s.gather(1, idx), margin


def plain_moe(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict,
              margins: Optional[list] = None) -> torch.Tensor:
    r = mlp["router"]
    z = h @ w[f"{p}.router"].float().T
    idx, wt, margin = plain_route(z, r)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros(h.shape[0], w[f"{p}.e0.down"].shape[0])
    limit = float(mlp["expert"]["limit"])
    for e in range(int(r["experts"])):
        for j in range(idx.shape[1]):
            rows = (idx[:, j] == e).nonzero()[:, 0]
            if rows.numel():
                out[rows] += wt[rows, j, None] * plain_expert(h[rows], w, f"{p}.e{e}", limit)
    if mlp.get("shared"):
        out = out + plain_expert(h, w, f"{p}.shared", float(mlp["shared"]["limit"]))
    return out


def plain_run_order(cfg: dict):
    """[(layer, adds the embedding output before it)]."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop["times"]) <= 1 or int(loop["stop"]) <= int(loop["start"]):
        return [(i, False) for i in range(L)]
    a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for rep in range(n):
        order += [(i, rep > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, L)]


def plain_forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
                  layers_out: Optional[list] = None, margins: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; ``layers_out`` collects the residual
    stream after every layer run, ``margins`` the routing margin [T] of every routed
    feed-forward that ran."""
    eps = float(cfg["norm"]["eps"])
    x0 = plain_embedding(w, cfg, tokens)
    x = x0.clone()
    for i, add in plain_run_order(cfg):
        layer = cfg["layers"][i]
        if add:
            x = x + x0
        assert layer["type"] == "attention", layer["type"]
        x = x + plain_attention(plain_norm(x, w[f"l{i}.norm1"], eps), w, f"l{i}.mix", layer["mixer"])
        if layer.get("mlp"):
            assert layer["mlp"]["kind"] == "moe", layer["mlp"]["kind"]
            x = x + plain_moe(plain_norm(x, w[f"l{i}.norm2"], eps), w, f"l{i}.mlp", layer["mlp"], margins)
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = plain_norm(x, w["final.norm"], eps) @ w["head"].float().T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits


def plain_generate_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int) -> List[int]:
    """Greedy continuation, recomputing the whole sequence for every new token."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(plain_forward(cfg, w, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
