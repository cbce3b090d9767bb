"""Kefisun without a device: its configuration, its spec (parts, schedule, cache slots, tensor names) and the plain
implementation's own consistency (the window's edge, the bias, the recurrence's order, causality)."""
import copy

import pytest
import torch

import plain_kefisun as P
from firefly_b200.cache.spec import PagedKVSpec, StateSpec, filter_slot, sub_slot
from firefly_b200.config.base import ConfigError
from firefly_b200.config.kefisun import file_hints
from firefly_b200.models import config_from_dict, expected_weights, spec_for
from firefly_b200.models.decoder import DecoderModel
from firefly_b200.parts import Runtime

ATT = {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "conv": 3, "scale": 0.3, "mask": {"size": 10}, "v_mix": True}
PLAIN_ATT = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 40, "conv": 2, "scale": 0.5, "mask": {"size": 7}}
DELTA = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 4}
FF = {"kind": "dense", "ff": 40, "limit": 0.9}
CFG = {"architecture": "Kefisun", "vocab": 60, "width": 32, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
       "embedding": {"scale": 2.5}, "logit_scale": 0.75, "layers": [
           {"type": "channel_delta", "mixer": DELTA, "mlp": FF},
           {"type": "attention", "mixer": PLAIN_ATT, "mlp": None},
           {"type": "attention", "mixer": ATT, "mlp": FF},
           {"type": "channel_delta", "mixer": DELTA, "mlp": None},
           {"type": "attention", "mixer": ATT, "mlp": FF}]}
RANKS = {"a": 6, "g": 10}


def _cfg_with_ranks():
    shapes = P.tensor_shapes(CFG, RANKS)
    return config_from_dict(file_hints(CFG, shapes))


def test_the_spec_names_every_tensor_and_gives_every_run_its_caches():
    cfg = _cfg_with_ranks()
    spec = spec_for(cfg)
    assert len(spec.layers) == 5 and [e.layer for e in spec.schedule] == [0, 1, 2, 3, 4]
    names = {w.name: tuple(w.shape) for w in expected_weights(spec) if not w.optional}
    want = {k: tuple(v) for k, v in P.tensor_shapes(CFG, RANKS).items()}
    # the factor of a layer that does not blend (the first blending one, or one that blends nothing) is not needed
    for skip in ("l1.mix.vmix", "l2.mix.vmix"):
        want.pop(skip)
        assert skip not in names
    assert names == want
    assert [L.mixer.params.get("value_mix") for L in spec.layers if L.mixer.kind == "conv_attention"] == [None, "first", "blend"]
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    slots = model.cache_slot_specs()
    # every run keeps its filter's last inputs; a recurrent run one state; an attention run pages and a state
    assert sorted(slots) == sorted([filter_slot(i) for i in range(5)] + [0, 3] +
                                   [sub_slot(i, j) for i in (1, 2, 4) for j in (0, 1)])
    assert all(isinstance(slots[filter_slot(i)], StateSpec) and slots[filter_slot(i)].shape == (2 * 32,) for i in range(5))
    kv = slots[sub_slot(2, 0)]
    assert isinstance(kv, PagedKVSpec) and (kv.num_kv_heads, kv.head_dim, kv.window) == (2, 32, 10)      # heads of max(24, 16) -> 32
    kv = slots[sub_slot(1, 0)]
    assert (kv.num_kv_heads, kv.head_dim, kv.window) == (1, 48, 7)
    assert slots[sub_slot(2, 1)].shape == (2 * (4 * 24 + 2 * 24 + 2 * 16),)            # conv - 1 rows of q | k | v
    assert isinstance(slots[0], StateSpec) and slots[0].shape[0] >= 4 * 8 * 12 + 3 * (2 * 2 * 8 + 4 * 12)


def test_the_inner_sizes_of_the_two_step_projections_come_from_the_tensors():
    cfg = _cfg_with_ranks()
    p = spec_for(cfg).layers[0].mixer.params
    assert (p["decay_rank"], p["gate_rank"]) == (6, 10)
    other = config_from_dict(file_hints(CFG, P.tensor_shapes(CFG, {"a": 3, "g": 5})))
    p = spec_for(other).layers[3].mixer.params
    assert (p["decay_rank"], p["gate_rank"]) == (3, 5)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][2]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][2]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][2]["mixer"].update(heads=3), "kv_heads"),
    (lambda c: c["layers"][2]["mixer"].update(v_mix="yes"), "v_mix"),
    (lambda c: c["layers"][4].update(mixer=dict(ATT, vdim=8)), "mixes values"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["canon"].update(taps=17), "taps"),
    (lambda c: c.pop("norm"), "eps"),
    (lambda c: c.pop("embedding"), "scale"),
    (lambda c: c.pop("logit_scale"), "logit_scale"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_a_wrong_configuration_is_told_by_name(edit, word):
    raw = copy.deepcopy(CFG)
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_the_configuration_goes_to_a_dictionary_and_back():
    cfg = config_from_dict(CFG)
    assert config_from_dict(cfg.to_dict()) == cfg
    assert cfg.first_value_mixer() == 2 and cfg.vocab_size == 60


def test_the_plain_window_ends_exactly_at_its_size_and_the_bias_grows_with_distance():
    m = P.window_mask(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True] and m[1].tolist() == [True, True, False, False, False, False]
    b = P.distance_bias(torch.tensor([2.0]), torch.tensor([0.5]), 4)
    assert b[0, 3, 3] == 0 and abs(float(b[0, 3, 1]) - 2.0 * torch.log(torch.tensor(2.0)).item()) < 1e-6
    # a row of the attention depends on the rows inside its window (and the taps in front of them) only
    w = {k: v.double() for k, v in P.random_weights(CFG, 1, RANKS).items()}
    x = torch.randn(30, 32, generator=torch.Generator().manual_seed(0), dtype=torch.float64)
    out, _ = P.attention_mixer(x, w, "l1.mix", PLAIN_ATT, 1e-5, None)
    y = x.clone()
    y[:12] = torch.randn(12, 32, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    moved, _ = P.attention_mixer(y, w, "l1.mix", PLAIN_ATT, 1e-5, None)
    # row 19 sees keys 13..19, key 13 convolves rows 12 and 13: untouched; row 18 sees key 12, which convolves row 11
    assert torch.allclose(moved[19:], out[19:], atol=1e-12) and not torch.allclose(moved[18], out[18], atol=1e-6)


def test_the_plain_model_is_causal_and_blends_the_first_blending_layer_s_values():
    w = {k: v.double() for k, v in P.random_weights(CFG, 3, RANKS).items()}
    toks = [5, 9, 2, 33, 8, 1, 0, 59, 17, 4, 4, 21, 6, 40, 3]
    full = P.forward(CFG, w, toks)
    assert torch.allclose(P.forward(CFG, w, toks[:7]), full[:7], atol=1e-9)
    # with a factor of zero in the last layer its blend is switched off: the logits move
    off = dict(w, **{"l4.mix.vmix": torch.tensor(0.0, dtype=torch.float64)})
    assert float((P.forward(CFG, off, toks) - full).abs().max()) > 1e-3
    # the first blending layer's own factor is not used
    unused = dict(w, **{"l2.mix.vmix": torch.tensor(0.9, dtype=torch.float64)})
    assert torch.equal(P.forward(CFG, unused, toks), full)


def test_a_random_model_of_the_design_gets_every_tensor_it_needs():
    from firefly_b200.weights.random_init import random_weights_cpu
    cfg = _cfg_with_ranks()
    spec = spec_for(cfg)
    tensors = random_weights_cpu(expected_weights(spec), 0, dtype=torch.float32)
    for ws in expected_weights(spec):
        if not ws.optional:
            assert tuple(tensors[ws.name].shape) == tuple(ws.shape), ws.name
