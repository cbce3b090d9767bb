"""Papusun without a device: its configuration, its spec (parts, schedule, cache slots, tensor names) and the plain
implementation's own consistency (the window's edge, the score cap, the frequency bands, the recurrence's order)."""
import copy
import math

import pytest
import torch

import plain_papusun as P
from firefly_b200.cache.spec import PagedKVSpec, StateSpec, sub_slot
from firefly_b200.config.base import ConfigError
from firefly_b200.models import config_from_dict, expected_weights, spec_for
from firefly_b200.models.decoder import DecoderModel
from firefly_b200.parts import Runtime

ROT = {"base": 1000.0, "dims": 8}
LAT = {"heads": 3, "dim": 8, "rot_dim": 8, "vdim": 12, "kv_rank": 24, "q_rank": 16, "scale": 0.3, "mask": {"size": 9},
       "rot": ROT}
LEFT = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "softcap": 5.0,
        "rot": {"base": 500.0, "dims": 12, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}}
RIGHT = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3}
PAR = {"left": LEFT, "right": RIGHT, "left_scale": 0.8, "right_scale": 1.5}
FF = {"kind": "dense", "ff": 40}
CFG = {"architecture": "Papusun", "vocab": 60, "width": 32, "norm": {"eps": 1e-5}, "logit_scale": 1.5,
       "token_side": {"dim": 6}, "layers": [
           {"type": "parallel", "mixer": PAR, "mlp": FF},
           {"type": "latent_attention", "mixer": LAT, "mlp": None},
           {"type": "latent_attention", "mixer": dict(LAT, kv_from=1, mask={"size": 14}), "mlp": FF},
           {"type": "parallel", "mixer": PAR, "mlp": None},
           {"type": "latent_attention", "mixer": dict(LAT, mask={"size": 5}), "mlp": FF},
           {"type": "latent_attention", "mixer": dict(LAT, kv_from=1, vdim=4), "mlp": FF}]}


def test_the_spec_names_every_tensor_and_gives_every_run_its_caches():
    cfg = config_from_dict(CFG)
    spec = spec_for(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3, 4, 5]
    assert [(e.cache, e.write_cache) for e in spec.schedule] == [(None, True), (None, True), (1, False), (None, True),
                                                                 (None, True), (1, False)]
    names = {w.name: tuple(w.shape) for w in expected_weights(spec) if not w.optional}
    assert names == {k: tuple(v) for k, v in P.tensor_shapes(CFG).items()}
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    slots = model.cache_slot_specs()
    assert sorted(slots) == sorted([1, 4] + [sub_slot(i, j) for i in (0, 3) for j in (0, 1)])
    # the cache that layers 2 and 5 read keeps the longest of the three windows; layer 4 keeps its own
    assert slots[1] == PagedKVSpec(1, 32, 14, None, planes=1) and slots[4] == PagedKVSpec(1, 32, 5, None, planes=1)
    kv = slots[sub_slot(0, 0)]
    assert (kv.num_kv_heads, kv.head_dim, kv.window) == (2, 24, None)           # heads of max(16, 24)
    st = slots[sub_slot(0, 1)]
    assert isinstance(st, StateSpec) and st.shape[0] >= 4 * 8 * 12 + 2 * (2 * 2 * 8 + 4 * 12)
    tails = [b.tail for b in model.blocks]
    assert [t.col0 for t in tails] == [0, 6, 12, 18, 24, 30] and all(t.table_cols == 36 for t in tails)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].pop("right_scale"), "right_scale"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(conv=17), "taps"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=4), "earlier"),
    (lambda c: c["layers"][5]["mixer"].update(kv_from=2), "of its own"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=8), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c.pop("norm"), "eps"),
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
    assert cfg.vocab_size == 60 and cfg.kv_source(2) == 1 and cfg.kv_source(1) is None and cfg.cache_window(1) == 14


def test_the_frequency_bands_keep_short_waves_and_stretch_long_ones():
    from firefly_b200.parts.position import RotaryEncoding
    from firefly_b200.config.base import PartSpec
    rot = {"base": 500.0, "dims": 12, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
    f = P.rotary_frequencies(rot)
    plain = P.rotary_frequencies({"base": 500.0, "dims": 12})
    wave = 2 * math.pi / plain
    assert wave[0] < 16 and f[0] == plain[0]                                    # shorter than original / high: kept
    assert wave[-1] > 64 and abs(float(f[-1]) - float(plain[-1]) / 4.0) < 1e-15    # longer than original / low: divided
    mid = [i for i in range(6) if 16 <= wave[i] <= 64]
    assert mid and all(plain[i] / 4.0 < f[i] < plain[i] for i in mid)
    part = RotaryEncoding(PartSpec("rotary", dict(head_dim=16, rotary_dim=12, theta=500.0, pairing="interleaved",
                                                  scaling=dict(rot["scaling"], kind="wavelength_bands"))),
                          Runtime(torch.device("cpu"), torch.float32))
    assert torch.allclose(part.frequencies(), f, rtol=1e-14, atol=0) and part.magnitude == 1.0


def test_the_plain_rotation_turns_neighbours_and_leaves_the_rest():
    x = torch.arange(1.0, 9.0, dtype=torch.float64).view(1, 1, 8).repeat(3, 1, 1)
    f = torch.tensor([0.5, 0.25], dtype=torch.float64)
    y = P.rotate_pairs(x, f, torch.tensor([0, 1, 2]))
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, :, 4:], x[:, :, 4:])
    a = 2 * 0.25
    assert abs(float(y[2, 0, 2]) - (3 * math.cos(a) - 4 * math.sin(a))) < 1e-12
    assert abs(float(y[2, 0, 3]) - (4 * math.cos(a) + 3 * math.sin(a))) < 1e-12


def test_the_plain_window_ends_exactly_at_its_size_and_the_cap_bounds_the_scores():
    m = P.visible(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True] and m[1].tolist() == [True, True, False, False, False, False]
    assert P.visible(4, None)[3].tolist() == [True] * 4
    q = torch.tensor([[[10.0]], [[10.0]]], dtype=torch.float64)
    k = torch.tensor([[[10.0]], [[-10.0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[0.0]]], dtype=torch.float64)
    capped = P.softmax_attention(q, k, v, 1.0, P.visible(2, None), softcap=2.0)
    # scores 100 and -100 become 2 and -2: the second query still sees a little of the first value
    assert abs(float(capped[1, 0, 0]) - 1.0 / (1.0 + math.exp(-4.0))) < 1e-9
    assert float(P.softmax_attention(q, k, v, 1.0, P.visible(2, None))[1, 0, 0]) == 1.0


def test_the_plain_delta_rule_reads_out_after_its_own_write():
    """One head by hand: with k a unit vector, beta = 1 and no decay the state holds v exactly, and the read-out of
    the same token returns it."""
    mx = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "conv": 1}
    big = 40.0
    w = {"p.q": torch.eye(2, dtype=torch.float64), "p.k": torch.eye(2, dtype=torch.float64),
         "p.v": torch.tensor([[0.0, 1.0]], dtype=torch.float64), "p.q.conv": torch.ones(2, 1, dtype=torch.float64),
         "p.k.conv": torch.ones(2, 1, dtype=torch.float64), "p.v.conv": torch.ones(1, 1, dtype=torch.float64),
         "p.b": torch.tensor([[big, big]], dtype=torch.float64), "p.a": torch.zeros(1, 2, dtype=torch.float64),
         "p.A_log": torch.tensor([0.0], dtype=torch.float64), "p.dt_bias": torch.tensor([-big], dtype=torch.float64),
         "p.norm": torch.ones(1, dtype=torch.float64), "p.g": torch.tensor([[big, big]], dtype=torch.float64),
         "p.o": torch.ones(1, 1, dtype=torch.float64)}
    h = torch.tensor([[3.0, 3.0]], dtype=torch.float64)
    out = P.delta_rule(h, w, "p", mx, 0.0)
    # q = k = silu(3) (1, 1) -> unit vectors, q times 2^(-1/2): o = S^T q = v (k . q) = silu(3) / sqrt(2); the head norm
    # then makes it 1 (one value), the gate silu(2 big * 3) is that number itself
    assert abs(float(out) - 6 * big) < 1e-6


def test_the_plain_model_is_causal_and_a_shared_cache_is_the_other_layer_s_rows():
    w = {k: v.double() for k, v in P.random_weights(CFG, 3).items()}
    toks = [5, 9, 2, 33, 8, 1, 0, 59, 17, 4, 4, 21, 6, 40, 3, 11, 12, 13, 50, 7]
    full = P.forward(CFG, w, toks)
    assert torch.allclose(P.forward(CFG, w, toks[:7]), full[:7], atol=1e-9)
    # layer 2 reads layer 1's rows: changing layer 1's down projection's norm moves layer 2's output too, and the
    # token-side table moves every layer
    moved = dict(w, **{"l1.mix.dkv.norm": w["l1.mix.dkv.norm"] * 1.5})
    assert float((P.forward(CFG, moved, toks) - full).abs().max()) > 1e-3
    moved = dict(w, **{"side.embed": w["side.embed"] * 0.5})
    assert float((P.forward(CFG, moved, toks) - full).abs().max()) > 1e-3


def test_a_random_model_of_the_design_gets_every_tensor_it_needs():
    from firefly_b200.weights.random_init import random_weights_cpu
    spec = spec_for(config_from_dict(CFG))
    tensors = random_weights_cpu(expected_weights(spec), 0, dtype=torch.float32)
    for ws in expected_weights(spec):
        if not ws.optional:
            assert tuple(tensors[ws.name].shape) == tuple(ws.shape), ws.name
