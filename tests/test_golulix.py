"""Golulix without a GPU: the configuration reader, the run order of looped layers, the
tensors the model declares, and the plain implementation's own mechanisms."""
import copy

import pytest
import torch

from golulix_helpers import (CONFIGS, GOLU_A, GOLU_B, GOLU_C, NEEDLE, make_weights, needle_model,
                             needle_tokens, random_tokens)
from plain_golulix import (plain_bigram_rows, plain_chunk_mask, plain_forward, plain_route, plain_run_order)
from yalm_b200.config import ConfigError, GolulixConfig, config_from_dict
from yalm_b200.engine.lm import tensor_needs_of
from yalm_b200.weights import random_tensors


@pytest.mark.parametrize("name", list(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    cfg, seed = CONFIGS[name]
    c = config_from_dict(cfg)
    assert isinstance(c, GolulixConfig)
    needs = tensor_needs_of(c)
    w = make_weights(cfg, seed)
    assert {k: tuple(v.shape) for k, v in needs.items()} == {k: tuple(v.shape) for k, v in w.items()}
    assert c.to_dict() == cfg


def test_run_order_of_looped_layers():
    spec = config_from_dict(GOLU_A).to_spec()
    assert [(e.layer, e.adds_embedding) for e in spec.run_order] == \
        [(0, False), (1, False), (2, False), (1, True), (2, False)] == plain_run_order(GOLU_A)
    assert [(e.layer, e.adds_embedding) for e in config_from_dict(GOLU_B).to_spec().run_order] == \
        [(0, False), (1, False)]
    assert [(e.layer, e.adds_embedding) for e in config_from_dict(GOLU_C).to_spec().run_order] == \
        [(0, False), (0, True), (0, True), (1, False)] == plain_run_order(GOLU_C)
    once = copy.deepcopy(GOLU_A)
    once["loop"]["times"] = 1
    assert [e.layer for e in config_from_dict(once).to_spec().run_order] == [0, 1, 2]


def test_parts_get_the_constants_of_the_configuration():
    spec = config_from_dict(GOLU_A).to_spec()
    m = spec.layers[0].parts["mixer"].params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["value_dim"], m["scale"], m["chunk"]) == \
        (4, 2, 16, 32, 0.3, 24)
    f = spec.layers[0].parts["feed_forward"].params
    assert (f["experts"], f["top"], f["groups"], f["keep_groups"], f["limit"], f["shared"]["limit"]) == \
        (8, 2, 4, 2, 1.5, 3.0)
    assert "feed_forward" not in spec.layers[1].parts
    assert spec.layers[2].parts["feed_forward"].params["shared"] is None
    assert spec.head.params["softcap"] == 20.0 and spec.embedding.params["buckets"] == 61
    assert config_from_dict(GOLU_A).ignorable_tensor("l1.norm2")
    assert not config_from_dict(GOLU_A).ignorable_tensor("l0.norm2")


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="recurrent"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["loop"].update(stop=7), "loop"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_configurations_that_cannot_be_served_are_refused(change, message):
    cfg = copy.deepcopy(GOLU_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(cfg)


def test_random_weights_mode_draws_norm_weights_around_zero():
    needs = tensor_needs_of(config_from_dict(GOLU_C))
    w = random_tensors(needs, 5)
    assert abs(float(w["l0.norm1"].mean())) < 0.05 and float(w["l0.norm1"].abs().max()) < 0.2
    assert w["bigram"].shape == (18, 100)


def test_plain_mechanisms():
    assert plain_bigram_rows([5, 9, 9], 7, 3, 2) == [7, (5 * 3 + 9 * 2) % 7, (9 * 3 + 9 * 2) % 7]
    m = plain_chunk_mask(7, 3)
    assert m[2].tolist() == [True, True, True, False, False, False, False]
    assert m[3].tolist() == [False, False, False, True, False, False, False]
    assert m[6].tolist() == [False] * 6 + [True]
    # groups: the second-best expert overall is not eligible when its group is not kept
    z = torch.log(torch.tensor([[0.30, 0.05, 0.28, 0.27, 0.06, 0.04]]))
    idx, wt, margin = plain_route(z, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert idx.tolist() == [[0, 1]] and torch.allclose(wt, torch.tensor([[0.30, 0.05]]), atol=1e-6)
    idx, wt, _ = plain_route(z, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}})
    assert idx.tolist() == [[0, 2]]                   # weights are the scores, not renormalised
    assert abs(float(wt.sum()) - 0.58) < 1e-6
    assert 0.06 < float(margin) < 0.07                # groups at 0.30 against 0.28: (0.30 - 0.28) / 0.30


def test_the_needle_construction_decides_the_probes_logits():
    cfg, w = needle_model(24)
    toks = needle_tokens(60, 24, [47, 48], seed=1)
    a = plain_forward(cfg, w, toks)
    b = plain_forward(cfg, w, [9 if t == NEEDLE else t for t in toks])
    assert (a[47] - b[47]).abs().max() > 0.2 * a.abs().max()       # position 47 shares the needle's chunk
    assert torch.allclose(a[48], b[48], atol=1e-4)                   # position 48 starts the next one
