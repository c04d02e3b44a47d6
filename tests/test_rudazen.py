"""Rudazen without a GPU: the configuration reader and its refusals, the tensors the model
declares, the plain implementation's own mechanisms (the pooled mask's edges, rotation layouts,
the recurrence carried from portion to portion), and that the crafted one-key models do show a
mask that is one position off."""
import copy
import math

import pytest
import torch

from plain_rudazen import (plain_forward, plain_frequencies, plain_gated_recurrence, plain_pool_mask,
                           plain_rotate, plain_window_mask)
from rudazen_helpers import (CONFIGS, PROBE, RUDA_A, RUDA_B, make_weights, needle_model, needle_tokens,
                             random_tokens, with_mask)
from yalm_b200.config import ConfigError, RudazenConfig, config_from_dict
from yalm_b200.engine.lm import tensor_needs_of


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoint_names(name):
    cfg, seed = CONFIGS[name]
    c = config_from_dict(cfg)
    assert isinstance(c, RudazenConfig) and c.to_dict() == cfg
    needs = tensor_needs_of(c)
    w = make_weights(cfg, seed)
    assert {k: tuple(v.shape) for k, v in needs.items()} == {k: tuple(v.shape) for k, v in w.items()}


def test_spec_carries_every_constant():
    spec = config_from_dict(RUDA_A).to_spec()
    assert [l.block for l in spec.layers] == ["postnorm"] * 3
    assert spec.embedding.params["scale"] == 8.0
    first = spec.layers[0]
    assert first.part("mixer").kind == "parallel_branches" and first.part("mixer_norm").params["residual_scale"] == 1.7
    left = dict(first.part("mixer").params["branches"])["left"].params
    assert (left["head_dim"], left["value_dim"], left["window"], left["pool"]) == (16, 32, 24, None)
    assert left["position"].params["layout"] == "halves" and left["position"].params["scaling"]["factor"] == 4.0
    second = spec.layers[1]
    assert "feed_forward" not in second.parts
    att = second.part("mixer").params
    assert att["values_from_keys"] and att["pool"] == 6 and att["position"].params["layout"] == "neighbours"
    assert "l1.mix.v" not in second.part("mixer").tensors.values()
    assert config_from_dict(RUDA_A).ignorable_tensor("l1.norm2") and not config_from_dict(RUDA_A).ignorable_tensor("l0.norm2")


def test_refusals():
    def broken(change):
        c = copy.deepcopy(RUDA_B)
        change(c)
        with pytest.raises(ConfigError):
            config_from_dict(c)
    broken(lambda c: c["layers"][0].update(type="convolution"))
    broken(lambda c: c["layers"][0]["mixer"].update(vdim=32))              # the values are the keys
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=4))           # 6 heads over 4
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=66))
    broken(lambda c: c["layers"][0]["mixer"]["mask"].pop("size"))          # a pool without a window
    broken(lambda c: c["layers"][1]["mlp"].update(kind="moe"))
    broken(lambda c: c["layers"][1]["mixer"].pop("right"))
    broken(lambda c: c.pop("norm"))


def test_pool_mask_edges():
    size, pool, T = 5, 3, 20
    m = plain_pool_mask(T, size, pool)
    for i in range(T):
        for b in range(T // pool):
            assert bool(m[i, b]) == (b * pool + pool - 1 <= i - size)
    # a position that has left the window is unseen until its whole block lies before the window
    near = plain_window_mask(T, size)
    i = 9                                           # window: 5..9; block 1 = 3..5 is not whole before it
    assert not near[i, 4] and not m[i, 1] and m[i, 0]


def test_rotation_layouts_and_yarn():
    u = torch.randn(6, 2, 12)
    rot = {"base": 100.0, "dims": 8}
    a, b = plain_rotate(u, rot, "pairs"), plain_rotate(u, rot, "halves")
    assert torch.equal(a[..., 8:], u[..., 8:]) and torch.equal(b[..., 8:], u[..., 8:])
    assert torch.allclose(a[0], u[0]) and torch.allclose(b[0], u[0])            # position 0 turns nothing
    # both layouts turn the same pairs by the same angles, only stored in another order
    perm = [0, 4, 1, 5, 2, 6, 3, 7]
    v = u.clone()
    v[..., :8] = u[..., perm]
    assert torch.allclose(plain_rotate(v, rot, "pairs")[..., [0, 2, 4, 6, 1, 3, 5, 7]], b[..., :8], atol=1e-6)
    f, mult = plain_frequencies({"base": 1e4, "dims": 16, "scaling": {"factor": 4.0, "original": 256,
                                                                     "fast": 16.0, "slow": 2.0}}, torch.float64)
    plain, one = plain_frequencies({"base": 1e4, "dims": 16}, torch.float64)
    assert one == 1.0 and abs(mult - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    # the ramp runs over pairs 0 .. 3: pair 0 keeps its frequency, pairs 3 and up are slowed down in full
    assert torch.equal(f[:1], plain[:1]) and torch.allclose(f[3:], plain[3:] / 4.0)
    assert bool(((f <= plain) & (f >= plain / 4.0)).all()) and bool((f[1:3] < plain[1:3]).all())


def test_recurrence_carries_its_state():
    cfg, seed = CONFIGS["ruda_a"]
    w = {k: v.float() for k, v in make_weights(cfg, seed).items()}
    m = cfg["layers"][0]["mixer"]["right"]
    h = torch.randn(11, cfg["width"])
    whole = plain_gated_recurrence(w, "l0.mix.right", m, h, 1e-5)
    # the same by hand, token by token, with the state handed on
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    S = torch.zeros(H, dk, dv)
    rows = []
    for t in range(11):
        x = h[t:t + 1]
        q = torch.nn.functional.silu(x @ w["l0.mix.right.q"].T).view(H, dk)
        low = w["l0.mix.right.lower"]
        f = (low + (1 - low) * torch.sigmoid(x @ w["l0.mix.right.f"].T + w["l0.mix.right.f.b"])).view(H, dk)
        v = (x @ w["l0.mix.right.v"].T).view(H, dv)
        S = f[:, :, None] * S + (1 - f)[:, :, None] * v[:, None, :]
        o = torch.einsum("hkv,hk->hv", S, q)
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5) * w["l0.mix.right.norm"]
        rows.append(o.reshape(1, -1) @ w["l0.mix.right.o"].T)
    assert torch.allclose(whole, torch.cat(rows), atol=1e-5)


@pytest.mark.parametrize("kind, size, pool", [("attention", 9, 4), ("parallel", 9, None)])
def test_the_crafted_models_show_a_mask_that_is_one_off(kind, size, pool):
    cfg, w = needle_model(kind, size, pool)
    n, at = 40, 6
    inside, outside = at + size - 1, at + size
    toks = needle_tokens(n, at, [inside, outside])
    ref = plain_forward(cfg, w, toks)
    wrong = plain_forward(with_mask(cfg, size=size + 1), w, toks)
    scale = float(ref.abs().max())
    far = float((ref[outside] - wrong[outside]).abs().max()) / scale
    near = float((ref[inside] - wrong[inside]).abs().max()) / scale     # one more ordinary key: little
    assert far > 0.05 and near < far / 3, (far, near)
    if pool:
        # the needle's block (positions 4..7) is seen from position 7 + size on
        first = (at // pool) * pool + pool - 1 + size
        toks = needle_tokens(n, at, [first - 1, first])
        ref = plain_forward(cfg, w, toks)
        for other in (with_mask(cfg, pool=pool + 1), with_mask(cfg, size=size + 1), with_mask(cfg, size=size - 1)):
            wrong = plain_forward(other, w, toks)
            assert max(float((ref[p] - wrong[p]).abs().max()) for p in (first - 1, first)) / scale > 0.02


def test_logits_of_a_prefix_do_not_change_with_what_follows():
    cfg, seed = CONFIGS["ruda_c"]
    w = make_weights(cfg, seed)
    toks = random_tokens(30, cfg["vocab"], 5)
    assert torch.allclose(plain_forward(cfg, w, toks)[:17], plain_forward(cfg, w, toks[:17]), atol=1e-5)
