"""Rudazen on a GPU against the plain implementation: each added kernel alone, then the engine --
whole prompts, the tail one token at a time, prompts in portions down to two tokens, batches of
unequal requests whose shorter ones end earlier (slots and pages used again), keys just inside
and just outside a window and pooled blocks that are just seen or not yet, in prompts and in
decoding, far keys among hundreds, first tokens, long decoding through the captured decode step,
greedy generation through the entry point, and the trace replay program."""
import json
import os

import pytest
import torch

from plain_rudazen import (plain_forward, plain_gated_recurrence, plain_norm, plain_pool_mask, plain_rotate,
                           plain_softmax_mix, plain_window_mask)
from rudazen_helpers import (CONFIGS, PROBE, RUDA_A, TOL, add_portions, make_weights, needle_model,
                             needle_tokens, plain_generate_greedy, random_tokens, references)
from trace_tools import (Trace, add_batches, add_tail, add_whole, compare, forced_decode, run_in_process,
                         run_trace_run)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16", "float16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


@pytest.fixture(scope="module")
def ops():
    from yalm_b200.csrc import ops as o
    o.lib()
    return o


class B:
    """The index arrays of a ragged batch."""

    def __init__(self, q_lens, slots):
        qs = [0]
        for q in q_lens:
            qs.append(qs[-1] + q)
        self.n_seqs, self.n_tokens, self.q_lens, self.slots = len(q_lens), qs[-1], q_lens, slots
        self.q_start = torch.tensor(qs, dtype=torch.int32, device=DEV)
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
        self.token_seq = torch.tensor(sum([[i] * q for i, q in enumerate(q_lens)], []),
                                      dtype=torch.int32, device=DEV)


def _lm(cfg, w, dtype, **kw):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    return LM(config_from_dict(cfg), dict(w), dtype=dtype, **kw)


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dim, rows", [(64, 5), (100, 3), (1000, 300), (4100, 2)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_sum_norm(ops, dim, rows, dt):
    g = torch.Generator().manual_seed(dim)
    x = torch.randn(rows, dim, generator=g)
    wt = 1 + 0.1 * torch.randn(dim, generator=g)
    a, b = torch.randn(3, rows, dim, generator=g), torch.randn(2, rows, dim, generator=g)
    wa, wb = 1 + 0.1 * torch.randn(dim, generator=g), 1 + 0.1 * torch.randn(dim, generator=g)
    cases = {
        "one plain product": ([(a, 3, None, 1.0)], 2.5 * x + a.sum(0)),
        "two normed branches": ([(a, 3, wa, 0.5), (b, 2, wb, 0.5)],
                                1.5 * x + 0.5 * (plain_norm(a.sum(0), wa, 1e-5) + plain_norm(b.sum(0), wb, 1e-5))),
        "nothing pending": ([], 1.0 * x),
    }
    for name, (branches, v) in cases.items():
        alpha = {"one plain product": 2.5, "two normed branches": 1.5, "nothing pending": 1.0}[name]
        ref = plain_norm(v, wt, 1e-6)
        xd = x.clone().to(DEV)
        h = torch.empty(rows, dim, dtype=dt, device=DEV)
        ops.sum_norm(xd, alpha, [(s.to(DEV), n, None if w is None else w.to(DEV), f) for s, n, w, f in branches],
                     wt.to(DEV), 1e-6, h=h, branch_eps=1e-5)
        assert (xd.cpu() - ref).abs().max().item() <= 2e-5, name
        assert torch.equal(h.cpu(), xd.cpu().to(dt)), name


@pytest.mark.parametrize("layout", ["halves", "neighbours"])
@pytest.mark.parametrize("H, G, hd, dims, has_v", [(4, 2, 16, 8, True), (3, 1, 32, 32, False), (5, 5, 24, 0, True)])
def test_whole_projection_norm_rotation_and_store(ops, layout, H, G, hd, dims, has_v):
    g = torch.Generator().manual_seed(H * hd + dims)
    q_lens, slots, past = [5, 1, 3], [2, 0, 3], {2: 0, 0: 7, 3: 2}
    b = B(q_lens, slots)
    n = b.n_tokens
    row = (H + (2 if has_v else 1) * G) * hd
    parts = torch.randn(2, n, row, generator=g)
    qn, kn = 1 + 0.2 * torch.randn(H * hd, generator=g), 1 + 0.2 * torch.randn(G * hd, generator=g)
    freq = torch.tensor([50.0 ** (-2.0 * i / max(dims, 2)) for i in range(max(dims // 2, 1))])
    cap = 16
    slot_pos = torch.zeros(4, dtype=torch.int32, device=DEV)
    for s, p in past.items():
        slot_pos[s] = p
    q_out = torch.zeros(n, H * hd, device=DEV)
    kv_step = torch.zeros(n, 2, G, hd, device=DEV)
    kc, vc = torch.zeros(4, G, cap, hd, device=DEV), torch.zeros(4, G, cap, hd, device=DEV)
    ops.qk_norm_rope_store(parts.to(DEV), 2, qn.to(DEV), kn.to(DEV), H * hd, G * hd, 1e-5, freq.to(DEV), dims,
                           layout == "neighbours", 1.3, b, q_out, kv_step, kc, vc, slot_pos, H, G, hd, has_v, cap)
    full = parts.sum(0)
    at = 0
    for ql, s in zip(q_lens, slots):
        rows = full[at:at + ql]
        q = plain_norm(rows[:, :H * hd], qn, 1e-5).view(ql, H, hd)
        k_raw = rows[:, H * hd:(H + G) * hd]
        k = plain_norm(k_raw, kn, 1e-5).view(ql, G, hd)
        v = (rows[:, (H + G) * hd:] if has_v else k_raw).view(ql, G, hd)
        # cos and sin times 1.3: the rotation of the plain implementation with its factor forced
        pos = torch.arange(past[s], past[s] + ql, dtype=torch.float32)
        def turn(u):
            if not dims:
                return u
            ang = pos[:, None] * freq[None, :]
            c, sn = (torch.cos(ang) * 1.3)[:, None], (torch.sin(ang) * 1.3)[:, None]
            out = u.clone()
            if layout == "neighbours":
                a_, b_ = u[..., 0:dims:2], u[..., 1:dims:2]
                out[..., 0:dims:2], out[..., 1:dims:2] = a_ * c - b_ * sn, b_ * c + a_ * sn
            else:
                a_, b_ = u[..., :dims // 2], u[..., dims // 2:dims]
                out[..., :dims // 2], out[..., dims // 2:dims] = a_ * c - b_ * sn, b_ * c + a_ * sn
            return out
        assert (q_out[at:at + ql].cpu().view(ql, H, hd) - turn(q)).abs().max().item() <= 2e-5
        assert (kv_step[at:at + ql, 0].cpu() - turn(k)).abs().max().item() <= 2e-5
        assert (kv_step[at:at + ql, 1].cpu() - v).abs().max().item() <= 1e-6
        for j in range(ql):
            r = (past[s] + j) % cap
            assert torch.equal(kc[s, :, r], kv_step[at + j, 0]) and torch.equal(vc[s, :, r], kv_step[at + j, 1])
        at += ql


@pytest.mark.parametrize("window, pool, cap", [(7, 3, 7), (5, 8, 8), (16, 4, 16)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_pooled_blocks_beside_a_window(ops, window, pool, cap, dt):
    """Two sequences in portions (one token at a time at the end): the pooled rows are made when a
    block completes, from this step's rows or the ring's, and every query sees window + blocks."""
    g = torch.Generator().manual_seed(window * 31 + pool)
    H, G, hd, T = 4, 2, 16, 45
    tol = 1e-5 if dt == torch.float32 else 2e-2
    seqs = {1: T, 3: T - 9}
    data = {s: (torch.randn(n, H, hd, generator=g).to(dt), torch.randn(n, G, hd, generator=g).to(dt),
                torch.randn(n, G, hd, generator=g).to(dt)) for s, n in seqs.items()}
    kc, vc = torch.zeros(4, G, cap, hd, dtype=dt, device=DEV), torch.zeros(4, G, cap, hd, dtype=dt, device=DEV)
    pcap = -(-64 // pool)
    pk, pv = torch.zeros(4, G, pcap, hd, dtype=dt, device=DEV), torch.zeros(4, G, pcap, hd, dtype=dt, device=DEV)
    slot_pos = torch.zeros(4, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = {s: [] for s in seqs}
    at = {s: 0 for s in seqs}
    portions = [{1: 6, 3: 1}, {1: 1, 3: 9}, {1: 11, 3: 2}] + [{1: 1, 3: 1}] * 40
    for sizes in portions:
        sizes = {s: min(n, seqs[s] - at[s]) for s, n in sizes.items() if at[s] < seqs[s]}
        if not sizes:
            break
        slots = list(sizes)
        b = B([sizes[s] for s in slots], slots)
        q = torch.cat([data[s][0][at[s]:at[s] + sizes[s]] for s in slots]).reshape(b.n_tokens, H * hd).to(DEV)
        kv = torch.stack([torch.cat([data[s][1][at[s]:at[s] + sizes[s]] for s in slots]),
                          torch.cat([data[s][2][at[s]:at[s] + sizes[s]] for s in slots])], 1).contiguous().to(DEV)
        late = any(at[s] > 0 and sizes[s] > 1 and at[s] + sizes[s] > cap for s in slots)
        if not late:
            ops.cache_write(kv, b, kc, vc, slot_pos, G, hd, cap)
        ops.pool_blocks(kv, kc, vc, b, slot_pos, pk, pv, G, hd, cap, pool, pcap, status)
        out = torch.empty(b.n_tokens, H * hd, dtype=dt, device=DEV)
        nsplit = 3 if b.n_tokens == len(slots) else 1
        po = torch.empty(b.n_tokens, H, nsplit, hd, device=DEV)
        pml = torch.empty(b.n_tokens, H, nsplit, 2, device=DEV)
        ops.attention(q, kv, kc, vc, b, slot_pos, out, H, G, hd, cap, window, nsplit, po, pml, scale=0.3,
                      pooled=(pk, pv, pool, pcap, None))
        if late:
            ops.cache_write(kv, b, kc, vc, slot_pos, G, hd, cap)
        ops.advance(b, slot_pos)
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            got[s].append(out[qs[i]:qs[i + 1]].float().cpu())
            at[s] += sizes[s]
    assert status.item() == 0
    for s, n in seqs.items():
        q, k, v = (t.float() for t in data[s])
        nb = n // pool
        kb = k[:nb * pool].reshape(nb, pool, G, hd).mean(1).to(dt).float()
        vb = v[:nb * pool].reshape(nb, pool, G, hd).mean(1).to(dt).float()
        see = torch.cat([plain_pool_mask(n, window, pool), plain_window_mask(n, window)], 1)
        ref = torch.zeros(n, H, hd)
        for h in range(H):
            gg = h // (H // G)
            keys, vals = torch.cat([kb[:, gg], k[:, gg]]), torch.cat([vb[:, gg], v[:, gg]])
            ref[:, h] = plain_softmax_mix((q[:, h] @ keys.T) * 0.3, see, vals)
        out = torch.cat(got[s]).view(n, H, hd)
        err = (out - ref).abs().max(-1).values.max(-1).values
        bad = (err > tol * ref.abs().max()).nonzero()
        assert not bad.numel(), f"sequence {s}: first wrong position {int(bad[0])} (window {window}, pool {pool})"


@pytest.mark.parametrize("hd, window, pool", [(32, 40, 8), (64, 100, 16), (128, 70, 0), (64, 0, 0)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_tensor_core_attention_with_unrounded_weights(ops, hd, window, pool, dt):
    """Against the FMA kernel on the same cache: a first step fills ring and pooled rows, a second
    brings several tokens on top (one sequence from its first token, one that goes on)."""
    g = torch.Generator().manual_seed(hd + window)
    H, G, cap = 4, 2, max(window, pool) or 256
    pcap = 64
    kc, vc = torch.zeros(3, G, cap, hd, dtype=dt, device=DEV), torch.zeros(3, G, cap, hd, dtype=dt, device=DEV)
    pk, pv = torch.zeros(3, G, pcap, hd, dtype=dt, device=DEV), torch.zeros(3, G, pcap, hd, dtype=dt, device=DEV)
    slot_pos = torch.zeros(3, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pooled = (pk, pv, pool, pcap, None) if pool else None
    for q_lens, slots in (([37], [2]), ([90, 75], [0, 2]), ([3, 130], [0, 2])):
        b = B(q_lens, slots)
        n = b.n_tokens
        q = torch.randn(n, H * hd, generator=g).to(dt).to(DEV)
        kv = torch.randn(n, 2, G, hd, generator=g).to(dt).to(DEV)
        past = {s: int(slot_pos[s]) for s in slots}
        late = any(past[s] > 0 and ql > 1 and past[s] + ql > cap for s, ql in zip(slots, q_lens))
        if not late:
            ops.cache_write(kv, b, kc, vc, slot_pos, G, hd, cap)
        if pool:
            ops.pool_blocks(kv, kc, vc, b, slot_pos, pk, pv, G, hd, cap, pool, pcap, status)
        ref, got = torch.empty(n, H * hd, dtype=dt, device=DEV), torch.empty(n, H * hd, dtype=dt, device=DEV)
        ops.attention(q, kv, kc, vc, b, slot_pos, ref, H, G, hd, cap, window or None, 1, None, None, scale=0.2,
                      pooled=pooled)
        ops.attention_exact_prefill(q, kv, kc, vc, b, slot_pos, got, H, G, hd, cap, window or None, scale=0.2,
                                    pooled=pooled)
        if late:
            ops.cache_write(kv, b, kc, vc, slot_pos, G, hd, cap)
        ops.advance(b, slot_pos)
        err = (got.float() - ref.float()).abs().max(-1).values
        bad = (err > 2 ** -7 * ref.float().abs().max()).nonzero()
        assert not bad.numel(), f"step {q_lens}: first wrong token {int(bad[0])}, error {float(err.max()):.3e}"
    assert status.item() == 0


@pytest.mark.parametrize("H, dk, dv", [(3, 24, 16), (1, 8, 40), (2, 20, 12), (2, 128, 64), (1, 200, 9), (2, 64, 128), (1, 384, 24), (1, 301, 16)])
def test_gated_recurrence_in_portions(ops, H, dk, dv):
    g = torch.Generator().manual_seed(dk)
    D = 32
    w = {"r.q": torch.randn(H * dk, D, generator=g) * 0.3, "r.f": torch.randn(H * dk, D, generator=g) * 0.5,
         "r.v": torch.randn(H * dv, D, generator=g) * 0.3, "r.f.b": torch.randn(H * dk, generator=g),
         "r.lower": 0.9 * torch.rand(H * dk, generator=g), "r.norm": torch.ones(dv),
         "r.o": torch.eye(H * dv)}
    seqs = {2: torch.randn(41, D, generator=g), 0: torch.randn(19, D, generator=g)}
    m = {"heads": H, "dim": dk, "vdim": dv}
    wcat = torch.cat([w["r.q"], w["r.f"], w["r.v"]])
    state = torch.zeros(4, H, dk, dv, device=DEV)
    state[1] = 7.0                                        # another sequence's state stays as it is
    got = {s: [] for s in seqs}
    at = {s: 0 for s in seqs}
    for sizes in [{2: 17, 0: 2}, {2: 1, 0: 1}, {2: 20, 0: 16}, {2: 3}]:
        slots = list(sizes)
        b = B([sizes[s] for s in slots], slots)
        hcat = torch.cat([seqs[s][at[s]:at[s] + sizes[s]] for s in slots])
        proj = (hcat @ wcat.T)
        parts = torch.stack([0.25 * proj, 0.75 * proj]).contiguous().to(DEV)
        out = torch.empty(b.n_tokens, H * dv, device=DEV)
        act = torch.empty(b.n_tokens, 2 * H * dk + H * dv, device=DEV)
        ops.gated_recurrence(parts, 2, w["r.f.b"].to(DEV), w["r.lower"].to(DEV), b, state, out, H, dk, dv, act)
        normed = torch.empty(b.n_tokens, H * dv, device=DEV)
        ops.head_norm(out, w["r.norm"].to(DEV), normed, H, dv, 1e-5)
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            got[s].append(normed[qs[i]:qs[i + 1]].cpu())
            at[s] += sizes[s]
    for s, h in seqs.items():
        ref = plain_gated_recurrence(w, "r", m, h, 1e-5)
        assert (torch.cat(got[s]) - ref).abs().max().item() <= 3e-5 * max(1.0, ref.abs().max().item()), s
    assert bool((state[1] == 7.0).all())


# ------------------------------------------------------------------ the engine against the plain model
def _requests(cfg, seed):
    V = cfg["vocab"]
    return {"a": random_tokens(150, V, seed), "b": random_tokens(67, V, seed + 1), "c": random_tokens(1, V, seed + 2),
            "d": random_tokens(23, V, seed + 3), "e": random_tokens(131, V, seed + 4)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_schedules_against_the_plain_model(name, dtype):
    cfg, seed = CONFIGS[name]
    w = make_weights(cfg, seed, torch.float16 if dtype == "float16" else torch.bfloat16)
    reqs = _requests(cfg, seed)
    refs = references(cfg, w, reqs)
    tr = Trace()
    add_whole(tr, reqs)
    add_tail(tr, {k: reqs[k] for k in "abe"}, tail=48)
    add_portions(tr, "a", reqs["a"], [2, 2, 31, 64, 3, 2])
    add_portions(tr, "e", reqs["e"], [64, 1, 63, 2])
    add_portions(tr, "b", reqs["b"], [33, 32])
    add_batches(tr, reqs, [["a", "b", "c", "d"], ["e", "b"], ["d", "a", "e"]],
                {"a": 100, "b": 40, "c": 1, "d": 20, "e": 66})
    # few slots and a page pool sized by the tokens held: slots and pages are freed and used again
    lm = _lm(cfg, w, dtype, max_context=192, max_batch=4, max_tokens=tr.max_tokens)
    got = run_in_process(lm, tr)
    compare(tr, got, refs, cfg["vocab"], TOL[dtype])
    lm.rt.check_status()
    # and with one block per sequence in place of pages
    lm2 = _lm(cfg, w, dtype, max_context=192, max_batch=4)
    tr2 = Trace()
    add_batches(tr2, reqs, [["a", "b", "c", "d"], ["e", "b"]], {"a": 100, "b": 40, "c": 1, "d": 20, "e": 66})
    compare(tr2, run_in_process(lm2, tr2), refs, cfg["vocab"], TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_does_not_depend_on_its_batch(dtype):
    cfg, seed = CONFIGS["ruda_a"]
    w = make_weights(cfg, seed)
    reqs = _requests(cfg, seed)
    lm = _lm(cfg, w, dtype, max_context=192, max_batch=4)
    alone = {}
    for rid in "abd":
        s = lm.acquire(1)
        alone[rid] = lm.step([reqs[rid]], s, [list(range(len(reqs[rid])))]).cpu()
        lm.release(s)
    s = lm.acquire(3)
    both = lm.step([reqs[r] for r in "abd"], s, [list(range(len(reqs[r]))) for r in "abd"]).cpu()
    lm.release(s)
    at = 0
    for rid in "abd":
        n = len(reqs[rid])
        if dtype == "float32":
            assert torch.equal(both[at:at + n], alone[rid]), rid       # one chain of additions per output
        else:                                                          # the products' tiles follow the step's size
            assert (both[at:at + n] - alone[rid]).abs().max().item() <= TOL[dtype] * alone[rid].abs().max().item(), rid
        at += n


# ------------------------------------------------------------------ one key that stands out
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind, size, pool, dim", [("attention", 9, 4, 16), ("attention", 64, 16, 32),
                                                   ("attention", 70, 64, 16), ("attention", 30, 7, 64),
                                                   ("parallel", 9, None, 32), ("parallel", 64, None, 16),
                                                   ("parallel", 130, None, 64)])
def test_edges_of_windows_and_pooled_blocks(kind, size, pool, dim, dtype):
    cfg, w = needle_model(kind, size, pool, dim=dim)     # head sizes 32 and 64: the tensor-core prompt kernel
    at = 6
    edges = [at + size - 1, at + size]                          # the needle's last visible position, and the next
    if pool:
        first = (at // pool) * pool + pool - 1 + size            # its block is seen from here on
        edges += [first - 1, first]
    n = max(edges) + 70
    far = n - 2                                                 # hundreds of positions later (pooled designs still see it)
    probes = sorted(set(edges + [far]))
    toks = needle_tokens(n, at, probes)
    ref = {"n": plain_forward(cfg, w, toks)}
    lm = _lm(cfg, w, dtype, max_context=n + 1, max_batch=2, max_tokens=2 * (n + 64))
    # in a whole prompt, in a prompt cut right at the edges, and decoded token by token
    for cuts in ([n], [edges[0], 1, 1], [at + 1] + [1] * (n - at - 1), [2, 2, 2] + [64] * 8):
        tr = Trace()
        add_portions(tr, "n", toks, list(cuts))
        compare(tr, run_in_process(lm, tr), ref, cfg["vocab"], TOL[dtype])
    # the same through the captured decode step
    forced_decode(lm, {"n": toks}, {"n": at + 2}, ref, TOL[dtype])


# ------------------------------------------------------------------ decode path, generation, replay program
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_long_decoding_through_the_captured_step(name, dtype):
    cfg, seed = CONFIGS[name]
    w = make_weights(cfg, seed)
    V = cfg["vocab"]
    reqs = {"x": random_tokens(260, V, seed + 7), "y": random_tokens(150, V, seed + 8), "z": random_tokens(40, V, seed + 9)}
    refs = references(cfg, w, reqs)
    lm = _lm(cfg, w, dtype, max_context=320, max_batch=3, max_tokens=3 * 320)
    rows = forced_decode(lm, reqs, {"x": 30, "y": 3, "z": 1}, refs, TOL[dtype])
    assert rows.shape[0] > 400
    assert lm.engine._graphs, "decode steps of a lasting batch are captured"


def test_greedy_generation_through_the_entry_point():
    cfg, seed = CONFIGS["ruda_a"]
    w = make_weights(cfg, seed)
    lm = _lm(cfg, w, "float32", max_context=128, max_batch=3)
    prompts = [random_tokens(n, cfg["vocab"], 40 + n) for n in (9, 1, 30, 17)]
    out = lm.generate(prompts, max_new_tokens=24, temperature=0.0, ignore_eos=True)
    for p, c in zip(prompts, out):
        assert c.tokens == plain_generate_greedy(cfg, w, p, 24)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_replay_program_on_a_model_folder(tmp_path, dtype):
    from yalm_b200.weights import write_file
    cfg, seed = CONFIGS["ruda_b"]
    w = make_weights(cfg, seed)
    folder = tmp_path / "model"
    os.makedirs(folder)
    with open(folder / "config.json", "w") as f:
        json.dump(cfg, f)
    write_file(str(folder / "model.safetensors"), w)
    reqs = {k: v for k, v in _requests(cfg, seed).items() if k in "abd"}
    refs = references(cfg, w, reqs)
    tr = Trace()
    add_whole(tr, reqs)
    add_tail(tr, {"a": reqs["a"]}, tail=40)
    add_batches(tr, reqs, [["a", "b", "d"]], {"a": 110, "b": 30, "d": 5})
    out = tmp_path / "out"
    os.makedirs(out)
    compare(tr, run_trace_run(str(folder), dtype, tr, str(out)), refs, cfg["vocab"], TOL[dtype])


def test_command_line_on_a_random_model_folder(tmp_path):
    """python -m yalm_b200: the random-weights mode writes a Rudazen model folder, greedy completion
    of token-id prompts matches the plain implementation on the weights it wrote, and sampling with
    a temperature repeats under one seed."""
    import subprocess
    import sys
    from trace_tools import ROOT
    from yalm_b200.weights import load_checkpoint
    (tmp_path / "cfg.json").write_text(json.dumps(RUDA_A))
    model = str(tmp_path / "model")
    base = [sys.executable, "-m", "yalm_b200", model, "--dtype", "float32"]
    r = subprocess.run(base + ["--random-weights", str(tmp_path / "cfg.json"), "--seed", "3",
                               "--tokens", "5,6,7;9,10", "-n", "6", "-t", "0"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "Rudazen" in r.stdout and os.path.isfile(os.path.join(model, "model.safetensors"))
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
