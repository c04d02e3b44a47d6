"""Golulix on a GPU against the plain implementation: each added kernel alone, then the
engine -- whole prompts, the tail one token at a time, prompts in portions down to two tokens,
batches of unequal requests whose shorter ones end earlier (slots and pages used again), keys
just inside and just outside a chunk in prompts and in decoding, first tokens, long decoding
through the captured decode step, greedy generation through the entry point, and the trace
replay program.  32-bit runs compare every position; 16-bit runs leave out what follows a
routing decision that was a close call in the plain implementation."""
import pytest
import torch

from golulix_helpers import (CONFIGS, GOLU_A, NEEDLE, PROBE, TOL, add_portions, compare, make_weights,
                             needle_model, needle_tokens, random_tokens, references)
from plain_golulix import (plain_bigram_rows, plain_chunk_mask, plain_forward, plain_generate_greedy,
                           plain_route)
from trace_tools import (Trace, add_batches, add_tail, add_whole, forced_decode, run_in_process,
                         run_trace_run)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16", "float16"]
HALF = [(torch.bfloat16, 2 ** -8), (torch.float16, 2 ** -11)]


@pytest.fixture(scope="module")
def ops():
    from yalm_b200.csrc import ops as o
    o.lib()
    return o


class B:
    """The index arrays of a ragged batch."""

    def __init__(self, q_lens, slots, tokens=None):
        qs = [0]
        for q in q_lens:
            qs.append(qs[-1] + q)
        self.n_seqs, self.n_tokens, self.q_lens, self.slots = len(q_lens), qs[-1], q_lens, slots
        self.q_start = torch.tensor(qs, dtype=torch.int32, device=DEV)
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
        self.token_seq = torch.tensor(sum([[i] * q for i, q in enumerate(q_lens)], []),
                                      dtype=torch.int32, device=DEV)
        if tokens is not None:
            self.tokens = torch.tensor(tokens, dtype=torch.int32, device=DEV)


def _lm(cfg, w, dtype, **kw):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    return LM(config_from_dict(cfg), dict(w), dtype=dtype, **kw)


# ------------------------------------------------------------------ kernels alone
def test_hashed_pair_embedding_and_its_state(ops):
    V, D, buckets, mp, mc = 50, 24, 13, 100003, 7919
    g = torch.Generator().manual_seed(1)
    table = torch.randn(V, D, generator=g).to(torch.bfloat16).to(DEV)
    pair = torch.randn(buckets + 1, D, generator=g).to(torch.bfloat16).to(DEV)
    seqs = {2: random_tokens(9, V, 1), 0: random_tokens(5, V, 2)}
    prev = torch.zeros(4, 1, dtype=torch.int32, device=DEV)
    pos = torch.zeros(4, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = {s: [] for s in seqs}
    # portions of 4, then 1, then the rest: the state carries the previous token across steps
    at = {s: 0 for s in seqs}
    for sizes in ({2: 4, 0: 1}, {2: 1, 0: 1}, {2: 4, 0: 3}):
        slots = list(sizes)
        toks = sum([seqs[s][at[s]:at[s] + sizes[s]] for s in slots], [])
        b = B([sizes[s] for s in slots], slots, toks)
        x = torch.empty(b.n_tokens, D, device=DEV)
        xc = torch.empty_like(x)
        ops.embed_pair(b, table, pair, prev, pos, x, xc, mp, mc, status)
        assert torch.equal(x, xc)
        ops.advance(b, pos)
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            got[s].append(x[qs[i]:qs[i + 1]].cpu())
            at[s] += sizes[s]
    for s, toks in seqs.items():
        rows = plain_bigram_rows(toks, buckets, mp, mc)
        ref = table.float().cpu()[torch.tensor(toks)] + pair.float().cpu()[torch.tensor(rows)]
        assert torch.equal(torch.cat(got[s]), ref), s
        assert int(prev[s]) == toks[-1]
    assert status.item() == 0


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_head_gate_softcap_and_residual_add(ops, dt):
    g = torch.Generator().manual_seed(2)
    n, H, hd = 7, 5, 24
    o = torch.randn(n, H * hd, generator=g).to(dt).to(DEV)
    gate = torch.randn(3, n, H, generator=g).to(DEV)
    ref = (o.float().view(n, H, hd) * torch.sigmoid(gate.sum(0))[:, :, None]).view(n, H * hd)
    ops.head_gate(o, gate, 3, H, hd)
    assert (o.float() - ref).abs().max().item() <= (1e-6 if dt == torch.float32 else 2 ** -7) * ref.abs().max().item()
    if dt == torch.float32:
        v = (40 * torch.randn(5, 33, generator=g)).to(DEV)
        ref = 12.5 * torch.tanh(v / 12.5)
        ops.softcap(v, 12.5)
        assert (v - ref).abs().max().item() <= 1e-5
        x, y = torch.randn(6, 40, generator=g).to(DEV), torch.randn(6, 40, generator=g).to(DEV)
        parts = torch.randn(2, 6, 40, generator=g).to(DEV)
        ref = x + parts.sum(0) + y
        ops.residual_add(x, y, parts, 2)
        assert (x - ref).abs().max().item() <= 1e-5


@pytest.mark.parametrize("E, groups, keep, top", [(8, 4, 2, 2), (6, 1, 1, 1), (12, 3, 2, 5), (64, 8, 3, 6),
                                                  (3, 3, 3, 3), (40, 1, 1, 40)])
def test_router_choice_plan_and_weights(ops, E, groups, keep, top):
    g = torch.Generator().manual_seed(E)
    n = 37
    z = 2.0 * torch.randn(2, n, E, generator=g)
    idx, wt, _ = plain_route(z.sum(0), {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}})
    choice = torch.zeros(n * top, dtype=torch.int32, device=DEV)
    weight = torch.zeros(n * top, device=DEV)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    ops.route_topk(z.to(DEV), 2, n, E, groups, keep, top, False, choice, weight, counts)
    assert torch.equal(choice.cpu().view(n, top).long(), idx)
    assert (weight.cpu().view(n, top) - wt).abs().max().item() <= 1e-6
    assert counts.cpu().tolist() == torch.bincount(idx.reshape(-1), minlength=E).tolist()
    # the plan: rows sorted by expert, every pair exactly once, tiles cover each expert's rows
    i32 = dict(dtype=torch.int32, device=DEV)
    mt = ops.routed_max_tiles(n * top, E)
    first, pair_row, row_token = torch.zeros(E + 1, **i32), torch.zeros(n * top, **i32), torch.zeros(n * top, **i32)
    tile_e, tile_r0, n_tiles = torch.zeros(mt, **i32), torch.zeros(mt, **i32), torch.zeros(1, **i32)
    expected_counts = counts.cpu().tolist()
    ops.route_plan(counts, choice, n * top, top, E, first, pair_row, row_token, tile_e, tile_r0, n_tiles)
    assert counts.abs().sum().item() == 0
    f = first.cpu().tolist()
    assert f[0] == 0 and [f[e + 1] - f[e] for e in range(E)] == expected_counts
    pr = pair_row.cpu().tolist()
    assert sorted(pr) == list(range(n * top))
    for p, r in enumerate(pr):
        e = int(choice[p])
        assert f[e] <= r < f[e + 1] and int(row_token[r]) == p // top
    nt = int(n_tiles)
    covered = sum(min(ops.ROUTED_TILE, f[int(tile_e[i]) + 1] - int(tile_r0[i])) for i in range(nt))
    assert covered == n * top and nt <= mt
    # renormalised weights sum to one
    ops.route_topk(z.to(DEV), 2, n, E, groups, keep, top, True, choice, weight, counts)
    assert (weight.view(n, top).sum(1) - 1).abs().max().item() <= 1e-6
    counts.zero_()


@pytest.mark.parametrize("dt, tile", [(torch.float32, 0), (torch.bfloat16, 0), (torch.bfloat16, 16),
                                      (torch.float16, 32), (torch.bfloat16, 64), (torch.float16, 128), (torch.bfloat16, 256)])
def test_grouped_products_activation_and_weighted_sum(ops, dt, tile):
    """The routed feed-forward's kernels after the router: plan, gather, grouped gate/up product,
    clamped activation, grouped down product, weighted sum -- on the FMA kernel (tile 0) and on
    tcgen05 with every tile size; one expert has many rows (several tiles), one has none."""
    g = torch.Generator().manual_seed(5)
    n, D, F, E, top = 150, (264 if tile >= 128 else 72), 40, 5, 2       # 264: blocks of 256 features
    h = torch.randn(n, D, generator=g).to(dt)
    wgu = (0.2 * torch.randn(E, 2 * F, D, generator=g)).to(dt)
    wd = (0.2 * torch.randn(E, D, F, generator=g)).to(dt)
    choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    choice[:40] = torch.tensor([3, 1], dtype=torch.int32)
    choice[choice == 4] = 0
    choice[:, 1] = torch.where(choice[:, 1] == choice[:, 0], (choice[:, 0] + 1) % 4, choice[:, 1])
    weight = torch.rand(n, top, generator=g)
    x = torch.randn(n, D, generator=g)
    ref = x.clone()
    for t in range(n):
        for j in range(top):
            e = int(choice[t, j])
            gu = h[t].float() @ wgu[e].float().T
            gg, uu = torch.clamp(gu[:F], max=1.1), torch.clamp(gu[F:], -1.1, 1.1)
            y = gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)
            if dt != torch.float32:
                y = y.to(dt).float()
            ref[t] += weight[t, j] * (y @ wd[e].float().T)
    i32 = dict(dtype=torch.int32, device=DEV)
    rows_per_tile = tile or ops.ROUTED_TILE
    pairs, mt = n * top, ops.routed_max_tiles(n * top, E, rows_per_tile)
    counts = torch.bincount(choice.reshape(-1).long(), minlength=E).to(torch.int32).to(DEV)
    first, pair_row, row_token = torch.zeros(E + 1, **i32), torch.zeros(pairs, **i32), torch.zeros(pairs, **i32)
    tile_e, tile_r0, n_tiles = torch.zeros(mt, **i32), torch.zeros(mt, **i32), torch.zeros(1, **i32)
    ops.route_plan(counts, choice.reshape(-1).to(DEV), pairs, top, E, first, pair_row, row_token, tile_e,
                   tile_r0, n_tiles, tile_rows=rows_per_tile)
    plan = (first, tile_e, tile_r0, n_tiles, mt)
    rows = torch.empty(pairs, D, dtype=dt, device=DEV)
    ops.gather_rows(h.to(DEV), row_token, rows)
    act = torch.full((pairs, F), float("nan"), dtype=dt, device=DEV)
    y = torch.full((pairs, D), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    if tile:
        ops.gemm_grouped_tc(rows, wgu.to(DEV), act, *plan, tile, status, glu=(1.702, 1.1, 1.0))
        ops.gemm_grouped_tc(act, wd.to(DEV), y, *plan, tile, status)
    else:
        gu = torch.empty(pairs, 2 * F, device=DEV)
        ops.gemm_grouped(rows, wgu.to(DEV), gu, *plan)
        ops.glu_clamp(gu, act, 1, 1.702, 1.1, 1.0)
        ops.gemm_grouped(act, wd.to(DEV), y, *plan)
    xd = x.to(DEV)
    ops.routed_combine(xd, y, pair_row, weight.reshape(-1).to(DEV), top)
    assert status.item() == 0
    tol = 2e-5 if dt == torch.float32 else (2e-2 if dt == torch.bfloat16 else 3e-3)
    assert (xd.cpu() - ref).abs().max().item() <= tol * ref.abs().max().item()


@pytest.mark.parametrize("dt, eps", HALF)
@pytest.mark.parametrize("M, F, K", [(5, 64, 72), (40, 208, 256), (130, 96, 64), (300, 256, 136)])
def test_dense_products_with_the_clamped_activation_in_their_epilogue(ops, dt, eps, M, F, K):
    """The gate/up product of a dense feed-forward with g' sigmoid(slope g') (u' + shift) under
    clamps where SiLU(g) u would be: single-SM and two-SM kernels, gate and up rows stacked or
    interleaved in groups of 16, and the kernel that sums split-K slices, against 32-bit."""
    g = torch.Generator().manual_seed(M + F)
    a = torch.randn(M, K, generator=g).to(dt)
    wg = (0.3 * torch.randn(F, K, generator=g)).to(dt)
    wu = (0.3 * torch.randn(F, K, generator=g)).to(dt)
    slope, limit, shift = 1.702, 1.3, 1.0
    gg = torch.clamp(a.float() @ wg.float().T, max=limit)
    uu = torch.clamp(a.float() @ wu.float().T, -limit, limit)
    ref = gg * torch.sigmoid(slope * gg) * (uu + shift)
    stacked = torch.cat([wg, wu], 0).to(DEV)
    paired = torch.stack([wg.view(F // 16, 16, K), wu.view(F // 16, 16, K)], 1).reshape(2 * F, K).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ad = a.to(DEV)
    outs = {}
    for name, w, mode, pr in (("stacked", stacked, ops.GEMM_SILU_MUL, False), ("paired", paired, ops.GEMM_SILU_PAIRED, True)):
        o = torch.empty(M, F, dtype=dt, device=DEV)
        ops.gemm_tc(ad, w, o, mode, status, glu=(slope, limit, shift))
        outs["single-SM " + name] = o
        if M > 128:
            o = torch.empty(M, F, dtype=dt, device=DEV)
            ops.gemm_2sm(ad, w, o, mode, status, glu=(slope, limit, shift))
            outs["two-SM " + name] = o
        S = 2 if K >= 128 else 1
        parts = torch.empty(S, M, 2 * F, device=DEV)
        ops.gemm_tc(ad, w, parts, ops.GEMM_SPLIT, status, splits=S)
        o = torch.empty(M, F, dtype=dt, device=DEV)
        ops.glu_clamp(parts, o, S, slope, limit, shift, paired=pr)
        outs["slices summed " + name] = o
    # SiLU is the case (1, none, 0): the same bits as the kernels' own SiLU epilogue
    o1, o2 = torch.empty(M, F, dtype=dt, device=DEV), torch.empty(M, F, dtype=dt, device=DEV)
    ops.gemm_tc(ad, paired, o1, ops.GEMM_SILU_PAIRED, status)
    ops.gemm_tc(ad, paired, o2, ops.GEMM_SILU_PAIRED, status, glu=(1.0, 0.0, 0.0))
    assert torch.equal(o1, o2) and status.item() == 0
    for name, o in outs.items():
        err = (o.float().cpu() - ref).abs().max().item()
        assert err <= 4 * eps * max(1.0, ref.abs().max().item()), (name, err)


def _chunk_reference(q, k, v, scale, chunk):
    """q [T, H, hd], k, v [T, G, hd] of one sequence -> [T, H, hd], 32-bit, chunk mask."""
    T, H, _ = q.shape
    G = k.shape[1]
    mask = plain_chunk_mask(T, chunk)
    out = torch.zeros(T, H, v.shape[2])
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        out[:, h] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, h // (H // G)]
    return out


@pytest.mark.parametrize("dt, eps", [(torch.float32, 2 ** -20)] + HALF)
@pytest.mark.parametrize("H, G, hd, chunk, paged", [(4, 2, 64, 96, False), (6, 3, 64, 64, True),
                                                    (2, 1, 128, 200, True), (5, 5, 16, 33, False),
                                                    (3, 1, 48, 70, True)])
def test_attention_kernels_under_a_chunked_mask(ops, dt, eps, H, G, hd, chunk, paged):
    """Every attention kernel with a chunked mask, a scale of its own and a ring of one chunk:
    whole prompts longer than several chunks, a second portion on top of the cache, then single
    tokens across a chunk's edge.  One key per probed query is made to stand out, right at the
    chunk's first position or right before it (where only a wrong mask would see it)."""
    g = torch.Generator().manual_seed(hd + chunk)
    scale = 0.37 / hd ** 0.5
    n_slots, slots = 4, [2, 0, 3]
    zero_freq = torch.zeros(hd // 2, device=DEV)
    slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    pps = -(-chunk // 64)
    if paged:
        n_pages = n_slots * pps + 3
        kc = torch.zeros(G, n_pages, 64, hd, device=DEV, dtype=dt)
        perm = torch.randperm(n_pages, generator=g)[:n_slots * pps]
        pages = perm.view(n_slots, pps).to(torch.int32).to(DEV)
    else:
        kc = torch.zeros(n_slots, G, chunk, hd, device=DEV, dtype=dt)
        pages = None
    vc = torch.zeros_like(kc)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    hist = {s: torch.zeros(0, H + 2 * G, hd) for s in slots}
    half = dt != torch.float32
    steps = [[2 * chunk + 7, 1, chunk - 1], [chunk // 2, chunk - 1, 2]] + [[1, 1, 1]] * (chunk // 2 + 3)
    for si, lens in enumerate(steps):
        b = B(lens, slots)
        N = b.n_tokens
        qkv = torch.randn(N, H + 2 * G, hd, generator=g)
        # stand-out pairs: the token at a chunk's first position and the one before it get large
        # keys, and every later token of the step asks along the same direction
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            T0 = hist[s].shape[0]
            for t in range(lens[i]):
                if (T0 + t) % chunk in (0, chunk - 1):
                    qkv[qs[i] + t, H:H + G, 0] = 6.0
                qkv[qs[i] + t, :H, 0] = 5.0
        qkv = qkv.to(dt).float()
        flat = qkv.view(N, -1).to(DEV)
        q_out = torch.empty(N, H * hd, device=DEV, dtype=dt)
        kv_step = torch.empty(N, 2, G, hd, device=DEV, dtype=dt)
        past = [hist[s].shape[0] for s in slots]
        wraps = any(p > 0 and n > 1 and p + n > chunk for p, n in zip(past, lens))
        ops.rope_store(flat, 1, zero_freq, b, q_out, kv_step, kc, vc, slot_pos, H, G, hd, chunk,
                       write_cache=not wraps, pages=pages)
        outs = {}
        o = torch.empty(N, H * hd, device=DEV, dtype=dt)
        ops.attention(q_out, kv_step, kc, vc, b, slot_pos, o, H, G, hd, chunk, None, 1, pages=pages,
                      chunk=chunk, scale=scale)
        outs["simt"] = o
        if half and hd % 16 == 0 and max(lens) > 1:
            o = torch.empty_like(o)
            ops.attention_prefill_mma(q_out, kv_step, kc, vc, b, slot_pos, o, H, G, hd, chunk, None,
                                      pages=pages, chunk=chunk, scale=scale)
            outs["mma"] = o
        if half and hd in (64, 128) and max(lens) > 1 and all(p == 0 for p in past):
            o = torch.empty_like(o)
            ops.attention_prefill_tc(q_out, kv_step, b, o, H, G, hd, None, status, chunk=chunk, scale=scale)
            outs["tcgen05"] = o
        if half and hd in (64, 128) and max(lens) > 1 and not wraps and any(p > 0 for p in past):
            o = torch.empty_like(o)
            ops.attention_prefill_tc_cache(q_out, kc, vc, b, slot_pos, o, H, G, hd, chunk, None, status,
                                           pages=pages, chunk=chunk, scale=scale)
            outs["tcgen05 over the cache"] = o
        if wraps:
            ops.cache_write(kv_step, b, kc, vc, slot_pos, G, hd, chunk, pages=pages)
        if max(lens) == 1:
            bound = max(past) + 1
            seq_slot = b.seq_slot
            o = torch.empty(N, H * hd, device=DEV, dtype=dt)
            kb = 32
            parts = -(-min(bound, chunk) // kb)
            po, pml = torch.empty(N * H * parts * hd, device=DEV), torch.empty(N * H * parts * 2, device=DEV)
            cn = torch.zeros(N * G * -(-(H // G) // 4), dtype=torch.int32, device=DEV)
            ops.attention_decode(q_out, kc, vc, seq_slot, slot_pos, o, po, pml, cn, status, H, G, hd, chunk,
                                 None, kb, bound, pages=pages, mask_chunk=chunk, scale=scale)
            outs["simt decode"] = o
            if half and hd % 16 == 0:
                for warps in (4, 2):
                    for cpc in (1, 1000):
                        parts = ops.decode_mma_parts(bound, None, cpc, chunk)
                        po = torch.empty(N * H * parts * hd, device=DEV)
                        pml = torch.empty(N * H * parts * 2, device=DEV)
                        cn = torch.zeros(N * G * -(-(H // G) // 16), dtype=torch.int32, device=DEV)
                        o = torch.empty(N, H * hd, device=DEV, dtype=dt)
                        ops.attention_decode_mma(q_out, kc, vc, seq_slot, slot_pos, o, po, pml, cn, status, H, G,
                                                 hd, chunk, None, bound, cpc, pages=pages, warps=warps,
                                                 mask_chunk=chunk, scale=scale)
                        outs[f"mma decode {warps} warps, {cpc} chunks a block"] = o
        ops.advance(b, slot_pos)
        torch.cuda.synchronize()
        assert status.item() == 0
        for i, s in enumerate(slots):
            hist[s] = torch.cat([hist[s], qkv[qs[i]:qs[i + 1]]])
            a = hist[s]
            ref = _chunk_reference(a[:, :H], a[:, H:H + G], a[:, H + G:], scale, chunk)[-lens[i]:]
            for name, o in outs.items():
                got = o[qs[i]:qs[i + 1]].float().cpu().view(-1, H, hd)
                err = (got - ref).abs().max().item()
                assert err <= 8 * eps * max(1.0, ref.abs().max().item()), (name, si, lens, s, err)


# ------------------------------------------------------------------ the engine
REQUESTS = {
    "golu_a": {"lens": {"r0": 21, "r1": 49, "r2": 90, "r3": 2, "r4": 1, "r5": 130},
               "prompts": {"r0": 5, "r1": 24, "r2": 41, "r3": 1, "r4": 1, "r5": 100},
               "batches": [["r0", "r1", "r2", "r4"], ["r3", "r5", "r1"], ["r2", "r0"]]},
    "golu_b": {"lens": {"r0": 40, "r1": 230, "r2": 101, "r3": 129},
               "prompts": {"r0": 8, "r1": 199, "r2": 100, "r3": 128},
               "batches": [["r0", "r1", "r2"], ["r3", "r0"]]},
    "golu_c": {"lens": {"r0": 9, "r1": 70, "r2": 38},
               "prompts": {"r0": 2, "r1": 33, "r2": 37},
               "batches": [["r0", "r1", "r2"], ["r2", "r0"]]},
}
_cache = {}


def setup(name):
    if name not in _cache:
        cfg, seed = CONFIGS[name]
        w = make_weights(cfg, seed)
        reqs = {rid: random_tokens(n, cfg["vocab"], 100 + i)
                for i, (rid, n) in enumerate(REQUESTS[name]["lens"].items())}
        tr = Trace()
        add_whole(tr, reqs)
        add_tail(tr, reqs, tail=32)
        add_batches(tr, reqs, REQUESTS[name]["batches"], REQUESTS[name]["prompts"])
        longest = max(reqs, key=lambda r: len(reqs[r]))
        add_portions(tr, longest, reqs[longest], [2, 3, 17, 2, 40, 1, 2])
        add_portions(tr, "r0", reqs["r0"], [2] * 20, tag="q")
        _cache[name] = (cfg, w, reqs, tr, {dt: references(cfg, w, reqs, dt) for dt in DTYPES})
    return _cache[name]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["golu_a", "golu_b", "golu_c"])
def test_step_function_matches_plain_model(name, dtype):
    cfg, w, reqs, tr, refs = setup(name)
    ref, safe = refs[dtype]
    # the cache is sized by the tokens held: pages, handed back and taken again
    lm = _lm(cfg, w, dtype, max_batch=max(1, tr.max_tokens // 64), max_tokens=tr.max_tokens, max_context=256)
    for _ in range(2):                       # the second pass runs on slots and pages used before
        got = run_in_process(lm, tr)
        worst, n = compare(tr, got, ref, safe, cfg["vocab"], TOL[dtype])
        assert n >= (sum(len(r) for r in tr.rows.values()) if dtype == "float32" else 40)
        assert lm.engine.cache.slots.free_count == lm.max_batch
        assert all(f == g["pool"].n_slots for f, g in zip(lm.engine.cache.free_pages(),
                                                          [g for g in lm.engine.cache.groups if "pool" in g]))


def test_the_residual_stream_after_every_layer_run():
    cfg, w, reqs, tr, _ = setup("golu_a")
    lm = _lm(cfg, w, "float32", max_batch=2, max_context=256)
    toks = reqs["r2"]
    layers = []
    plain_forward(cfg, w, toks, layers_out=layers)
    taps = []
    lm.model.tap = lambda i, stream: taps.append(stream.resolve().clone().cpu())
    s = lm.acquire(1)
    lm.step([toks], s, [[]])
    lm.release(s)
    assert len(taps) == len(layers) == 5              # layers 1 and 2 run twice
    for i, (a, b) in enumerate(zip(taps, layers)):
        assert (a - b).abs().max().item() <= 2e-5 * b.abs().max().item(), i


def test_cutting_and_batching_do_not_change_32_bit_logits():
    cfg, w, reqs, tr, _ = setup("golu_a")
    lm = _lm(cfg, w, "float32", max_batch=max(1, tr.max_tokens // 64), max_context=256)
    got = run_in_process(lm, tr)
    seen = {}
    for step, rows in tr.rows.items():
        g = got[step].reshape(-1, cfg["vocab"])
        for i, key in enumerate(rows):
            if key in seen:
                assert float((g[i] - seen[key]).abs().max()) <= 2e-5 * float(seen[key].abs().max()), (step, key)
            else:
                seen[key] = g[i]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [24, 64, 70, 130])
def test_a_key_just_inside_and_just_outside_a_chunk(dtype, chunk):
    """One key stands out by construction.  Probes sit at the chunk's last position (sees a
    needle at the chunk's first position, not one right before it), at the next chunk's first
    positions, far from the needle and at page borders; in prompts and decoded one by one."""
    cfg, w = needle_model(chunk)
    n = 2 * chunk + 20
    cases = {}
    for needle in (chunk - 1, chunk, 0, 63 if chunk > 64 else 1, 64 if chunk > 65 else 2):
        probes = [p for p in (needle + 1, chunk - 1, chunk, chunk + 1, 2 * chunk - 1, 2 * chunk, 2 * chunk + 1,
                              64, 65, 128, n - 1) if needle < p < n]
        cases[f"needle{needle}"] = needle_tokens(n, needle, probes, seed=needle)
    refs = {rid: plain_forward(cfg, w, t) for rid, t in cases.items()}
    # the construction works: seeing the needle or not moves the probe's logits by far more
    # than the tolerance
    t = cases[f"needle{chunk}"]
    moved = plain_forward(cfg, w, [9 if x == NEEDLE else x for x in t])
    assert (moved[2 * chunk - 1] - refs[f"needle{chunk}"][2 * chunk - 1]).abs().max() > \
        0.2 * refs[f"needle{chunk}"].abs().max()
    assert torch.allclose(moved[2 * chunk:], refs[f"needle{chunk}"][2 * chunk:], atol=1e-4)
    tr = Trace()
    add_whole(tr, cases)
    add_tail(tr, cases, tail=chunk + 25)
    add_batches(tr, cases, [list(cases)], {rid: chunk - 3 + i for i, rid in enumerate(cases)})
    lm = _lm(cfg, w, dtype, max_batch=8, max_tokens=tr.max_tokens, max_context=512)
    got = run_in_process(lm, tr)
    compare(tr, got, refs, {rid: n for rid in cases}, cfg["vocab"], TOL[dtype])
    # and through the decode step that stays on the device (graphs after the third step)
    forced_decode(lm, cases, {rid: chunk - 2 for rid in cases}, refs, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(dtype):
    cfg, w, reqs, tr, refs = setup("golu_a")
    ref, safe = refs[dtype]
    lm = _lm(cfg, w, dtype, max_batch=4, max_context=256)
    one = {"r4": reqs["r4"], "r3": reqs["r3"]}
    t2 = Trace()
    add_whole(t2, one)
    add_batches(t2, one, [["r4", "r3"]], {"r4": 1, "r3": 1})
    compare(t2, run_in_process(lm, t2), ref, safe, cfg["vocab"], TOL[dtype])
    # 129 decode steps from a prompt of one token: five times around the smallest ring
    long_ones = {r: reqs[r][:safe[r]] for r in ("r5", "r2") if safe[r] > 40}
    assert long_ones or dtype != "float32"
    if long_ones:
        forced_decode(lm, long_ones, {r: 1 for r in long_ones}, ref, TOL[dtype])


def test_greedy_generation_through_the_entry_point():
    cfg, w, reqs, tr, _ = setup("golu_a")
    lm = _lm(cfg, w, "float32", max_batch=2, max_context=128)
    prompts = [reqs["r0"][:7], reqs["r1"][:30], reqs["r4"]]
    out = lm.generate(prompts, max_new_tokens=40, temperature=0.0)
    for p, c in zip(prompts, out):
        assert c.tokens == plain_generate_greedy(cfg, w, p, 40)
        assert c.finish_reason == "length"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(dtype, tmp_path):
    import json
    import os
    from yalm_b200.weights import write_file
    cfg, w, reqs, tr, refs = setup("golu_c")
    ref, safe = refs[dtype]
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(folder, "model.safetensors"), w)
    got = run_trace_run(folder, dtype, tr, str(tmp_path / "out"))
    compare(tr, got, ref, safe, cfg["vocab"], TOL[dtype])


def test_random_weights_of_a_configuration_run():
    from yalm_b200 import LM
    lm = LM.from_random(GOLU_A, seed=3, dtype="bfloat16", max_batch=2, max_context=128)
    out = lm.generate([[1, 2, 3]], max_new_tokens=5, temperature=0.0)
    assert len(out[0].tokens) == 5


def test_command_line_on_a_random_model_folder(tmp_path):
    """python -m yalm_b200: the random-weights mode writes a Golulix model folder, greedy
    completion of token-id prompts matches the plain implementation on the weights it wrote, and
    sampling with a temperature repeats under one seed."""
    import json
    import os
    import subprocess
    import sys
    from trace_tools import ROOT
    from yalm_b200.weights import load_checkpoint
    (tmp_path / "cfg.json").write_text(json.dumps(GOLU_A))
    model = str(tmp_path / "model")
    base = [sys.executable, "-m", "yalm_b200", model, "--dtype", "float32"]
    r = subprocess.run(base + ["--random-weights", str(tmp_path / "cfg.json"), "--seed", "3",
                               "--tokens", "5,6,7;9,10", "-n", "6", "-t", "0"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "Golulix" in r.stdout and os.path.isfile(os.path.join(model, "model.safetensors"))
    lines = [l for l in r.stdout.splitlines() if l.startswith("tokens:")]
    assert len(lines) == 2
    with open(os.path.join(model, "config.json")) as f:
        cfg = json.load(f)
    w = load_checkpoint(model)
    for line, prompt in zip(lines, ([5, 6, 7], [9, 10])):
        assert [int(t) for t in line.split("(")[0].split()[1:]] == plain_generate_greedy(cfg, w, prompt, 6)
    sampled = []
    for _ in range(2):
        r = subprocess.run(base + ["--tokens", "5,6,7", "-n", "8", "-t", "0.9", "--seed", "11"],
                           capture_output=True, text=True, cwd=ROOT, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        sampled.append([l for l in r.stdout.splitlines() if l.startswith("tokens:")])
    assert sampled[0] == sampled[1] and sampled[0]
