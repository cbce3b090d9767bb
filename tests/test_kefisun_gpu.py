"""Kefisun on the device against the plain implementation in ``plain_kefisun.py``: every mechanism alone, then
whole models of several shapes through the replay session (whole prompts, decoding token by token, portions down
to two tokens, mixed batches with pages and state slots used again) and greedy generation through the engine and
its scheduler."""
import json
import os

import numpy as np
import pytest
import torch

import plain_kefisun as P
import replay_util as U

pytestmark = pytest.mark.gpu


def _att(heads, kv_heads, dim, vdim, window, conv=4, scale=None, v_mix=True):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
          "scale": scale or dim ** -0.5 * 1.5, "mask": {"size": window}}
    if v_mix is not None:
        mx["v_mix"] = v_mix
    return {"type": "attention", "mixer": mx}


def _delta(heads, kv_heads, dim, vdim, conv=4):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _dense(ff, limit=1.2):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _cfg(layers, width=48, vocab=101, taps=3, eps=1e-5, emb_scale=3.0, logit_scale=0.7):
    return {"architecture": "Kefisun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "embedding": {"scale": emb_scale}, "logit_scale": logit_scale, "layers": layers}


def _with(layer, mlp):
    return dict(layer, mlp=mlp)


CONFIGS = {
    # both kinds of mixer in an order of their own; value heads shorter and longer than key heads; windows that are
    # no multiple of a page and differ between layers; taps that differ between the filter and the mixers; the first
    # layer that blends values is not the first attention layer; a recurrent layer with and one without feed-forward
    "both_mixers": _cfg([_with(_att(4, 2, 24, 8, 37, conv=4, v_mix=False), _dense(72)),
                         _with(_delta(4, 2, 16, 24, conv=4), None),
                         _with(_att(4, 2, 24, 16, 37, conv=4), _dense(72)),
                         _with(_att(6, 2, 8, 16, 20, conv=2), None),
                         _with(_delta(3, 3, 8, 12, conv=2), _dense(40, 0.6)),
                         _with(_att(2, 1, 16, 32, 50, conv=3), _dense(72))]),
    # the values a model may happen to make equal or one: as many kv heads as heads, one q/k head for all recurrent
    # heads, key and value heads of one size, one tap (no convolution state at all), a window of one token and one
    # wider than any request, no layer that blends values (the key left out), scales of one
    "equal_or_one": _cfg([_with(_att(2, 2, 16, 16, 1 << 16, conv=1, scale=0.4, v_mix=None), _dense(64, 5.0)),
                          _with(_delta(2, 1, 32, 32, conv=1), _dense(64, 5.0)),
                          _with(_att(1, 1, 32, 32, 1, conv=2, v_mix=None), _dense(64, 5.0))],
                         width=64, vocab=131, taps=1, emb_scale=1.0, logit_scale=1.0),
    # sizes that no fast path takes: a width that is no multiple of 8, heads of 40, 12 and 20, three query heads on
    # a kv head, five taps, a window of one page, inner ranks of the two-step projections that differ
    "odd_sizes": _cfg([_with(_delta(3, 1, 20, 40, conv=5), _dense(50)),
                       _with(_att(6, 2, 40, 12, 8, conv=5), _dense(50)),
                       _with(_att(3, 1, 12, 24, 19, conv=3), None)], width=36, vocab=50, taps=5),
    # recurrent layers only: no pages at all, only state slots
    "recurrent_only": _cfg([_with(_delta(2, 2, 64, 16), _dense(40)), _with(_delta(4, 1, 8, 8, conv=3), None)], width=40),
    # attention only: every layer blends with the first layer's values
    "attention_only": _cfg([_with(_att(4, 4, 16, 16, 64), _dense(48)), _with(_att(8, 4, 16, 16, 33, conv=2), None),
                            _with(_att(4, 4, 32, 16, 16), _dense(48))], taps=4),
    # sizes that every fast path takes in bfloat16: heads of 64 (the tcgen05 attention kernel with the bias, the
    # 16-byte forms of the head preparation, the gate and the activation), blending layers with value heads as long as
    # and shorter than key heads, a recurrent layer with a key of 128 (two value columns a thread)
    "fast_paths": _cfg([_with(_att(4, 2, 64, 64, 70, conv=4), _dense(72)),
                        _with(_delta(2, 1, 128, 64, conv=4), None),
                        _with(_att(8, 2, 64, 64, 33, conv=3), _dense(64)),
                        _with(_att(2, 2, 128, 64, 100, conv=2), None)], width=64, vocab=97, taps=4),
}
RANKS = {"both_mixers": {"a": 8, "g": 12}, "odd_sizes": {"a": 5, "g": 3}}


def _model_dir(tmp_path, name, cfg, seed=1, edit=None, ranks=None):
    w = P.random_weights(cfg, seed, ranks or RANKS.get(name))
    if edit is not None:
        edit(w)
        w = {k: v.to(torch.bfloat16).to(v.dtype) for k, v in w.items()}        # what the file will hold
    U.write_model_dir(str(tmp_path / name), cfg, {k: v.float() for k, v in w.items()}, torch.bfloat16)
    return str(tmp_path / name), {k: v.double() for k, v in w.items()}       # the plain functions run in 64-bit


def _session(model_dir, dtype, max_tokens, block=16, max_requests=4):
    from firefly_b200.replay import ReplaySession
    return ReplaySession(model_dir, dtype=dtype, max_tokens=max_tokens, block_size=block, max_requests=max_requests)


def _compare_most(got, plain, tol, what, frac=0.9):
    """``frac`` of the rows within tol, and every row finite and within 8 tol: the head norm of the recurrent mixer
    divides by its output's root mean square, which magnifies bfloat16 rounding in a row whose output is small."""
    errs = sorted(U.rel_err(row, plain[rid.split("#")[0]][pos]) for (rid, pos), row in got.rows.items())
    assert errs and all(e == e for e in errs), what
    assert errs[-1] <= 8 * tol and errs[int(frac * (len(errs) - 1))] <= tol, \
        f"{what}: worst {errs[-1]:.3e}, {frac:.0%} quantile {errs[int(frac * (len(errs) - 1))]:.3e}, tol {tol:g}"


def _check(got, plain, dtype, what):
    if dtype == "float32":
        U.compare(got, plain, U.TOL[dtype], what)
    else:
        _compare_most(got, plain, U.TOL[dtype], what)


# ------------------------------------------------------------------ whole models, every cutting --
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_replay_in_every_cutting_matches_the_plain_model(tmp_path, name, dtype):
    cfg = CONFIGS[name]
    model_dir, w = _model_dir(tmp_path, name, cfg)
    reqs = U.make_requests(cfg["vocab"], [70, 3, 45, 1, 33, 58], 5)
    plain = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    twice = dict(reqs, **{"r0#2": reqs["r0"], "r4#2": reqs["r4"]})       # a request once more, on pages and slots used before
    for label, steps in (("whole", U.trace_whole(reqs)), ("decode", U.trace_tail_decode(reqs, tail=40)),
                         ("portions", U.trace_portions(reqs, sizes=(17, 5, 2, 9, 2, 31, 3, 2))),
                         ("mixed", U.trace_mixed(twice, seed=3, max_live=4, sizes=(13, 2, 7, 21, 3, 2, 16)))):
        sess = _session(model_dir, dtype, U.peak_tokens(steps), block=16 if label != "portions" else 8)
        got = U.run_trace(sess, steps)
        _check(got, plain, dtype, f"{name}/{dtype}/{label}")
        sess.cache.check()
        assert not sess.cache.live


def test_the_stream_matches_after_every_layer(tmp_path):
    cfg = CONFIGS["both_mixers"]
    model_dir, w = _model_dir(tmp_path, "stream", cfg)
    toks = U.make_requests(cfg["vocab"], [45], 8)["r0"]
    want = []
    P.forward(cfg, w, toks, layer_outputs=want)
    sess = _session(model_dir, "float32", 64)
    got = []

    def after(i, res, pending):
        x = res.detach().clone()
        if isinstance(pending, torch.Tensor):        # a block without feed-forward hands its mixer's output on unadded
            x += pending.float()
        got.append(x.cpu().double())
    sess.model.after_run = after
    sess.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [0]}], "end": ["a"]})
    assert len(got) == len(cfg["layers"]) == 6
    for i, g in enumerate(got):
        assert float((g - want[i]).abs().max()) < 2e-5 * float(want[i].abs().max()), f"after layer {i}"


# ------------------------------------------------------------------ mechanisms alone --
def _one_layer(tmp_path, layers, width=48, dtype="float32", seed=2, max_tokens=1024, block=16, edit=None, taps=3, ranks=None):
    cfg = _cfg(layers if isinstance(layers, list) else [layers], width=width, taps=taps)
    model_dir, w = _model_dir(tmp_path, "one", cfg, seed, edit=edit, ranks=ranks)
    return cfg, w, _session(model_dir, dtype, max_tokens, block=block)


def _step_context(sess, seqs):
    """A StepContext for sequences given as (request id, new tokens): admits, grows, builds."""
    from firefly_b200.engine.runner import StepEntry
    entries = []
    for rid, n in seqs:
        rc = sess.live.get(rid) or sess.cache.admit(rid)
        sess.live[rid] = rc
        assert sess.cache.grow(rc, rc.num_tokens + n)
        entries.append(StepEntry(rc, [0] * n, []))
    return sess.runner.build_context(entries), entries


def _advance(sess, entries):
    for e in entries:
        sess.cache.advance(e.cache, len(e.tokens))


def _run_cut(sess, call, x, cuts, rid):
    """``call(rows, ctx)`` on the portions of x one after the other, as one request; its pages and slot are then freed
    and go to the next cutting, which must start from zero."""
    rows, p = [], 0
    for n in cuts:
        ctx, entries = _step_context(sess, [(rid, n)])
        rows.append(call(x[p:p + n].cuda().contiguous(), ctx).float().cpu())
        _advance(sess, entries)
        p += n
    sess.cache.free(sess.live.pop(rid))
    return torch.cat(rows).double()


CUTS = ([57], [20, 2, 1, 1, 30, 3], [1] * 57)
TDT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_input_filter_alone_carries_its_last_inputs(tmp_path, taps):
    from firefly_b200.cache.spec import filter_slot
    cfg, w, sess = _one_layer(tmp_path, _with(_delta(1, 1, 8, 8), None), taps=taps)
    x = torch.randn(57, 48, generator=torch.Generator().manual_seed(taps))
    want = x.double() + P.causal_conv(x.double(), w["l0.canon1"])
    filt = sess.model.blocks[0].input_filter
    for cuts in CUTS:
        got = _run_cut(sess, lambda rows, ctx: filt.forward(rows, ctx, filter_slot(0)), x, cuts, f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max()), cuts


def test_norm_with_a_weight_around_zero_alone(tmp_path):
    cfg, w, sess = _one_layer(tmp_path, _with(_delta(1, 1, 8, 8), _dense(16)))
    ctx, _ = _step_context(sess, [("a", 11)])
    g = torch.Generator().manual_seed(3)
    res, delta = torch.randn(11, 48, generator=g) * 3 + 1, torch.randn(11, 48, generator=g)
    r = res.cuda()
    got = sess.model.blocks[0].norms[1].forward(r, delta.cuda(), ctx)
    summed = res.double() + delta.double()
    assert torch.allclose(r.cpu().double(), summed, atol=1e-6)                  # the sum goes into the stream, in 32-bit
    want = P.offset_norm(summed, w["l0.norm2"], cfg["norm"]["eps"])
    assert float((got.cpu().double() - want).abs().max()) < 1e-5
    assert float((want - P.rms(summed, cfg["norm"]["eps"]) * w["l0.norm2"]).abs().max()) > 0.5   # not a plain weight


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tokens", [1, 5, 150])
def test_dense_feed_forward_alone_with_inputs_that_reach_both_clamps(tmp_path, dtype, tokens):
    mlp = _dense(72, 0.8)
    cfg, w, sess = _one_layer(tmp_path, _with(_delta(1, 1, 8, 8), mlp), dtype=dtype)
    x = (torch.randn(tokens, 48, generator=torch.Generator().manual_seed(tokens)) * 1.5).to(TDT[dtype])
    gate = x.double() @ w["l0.mlp.gate"].T + w["l0.mlp.gate.b"]
    up = x.double() @ w["l0.mlp.up"].T + w["l0.mlp.up.b"]
    assert (gate > 0.8).any() and (up > 0.8).any() and (up < -0.8).any() and (gate < -0.8).any()
    want = P.dense_ff(x.double(), w, "l0.mlp", mlp)
    ctx, _ = _step_context(sess, [("a", tokens)])
    got = sess.model.blocks[0].feed_forward.forward(x.cuda(), ctx).float().cpu().double()
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert float((got - want).abs().max()) <= tol * float(want.abs().max())


DELTA_SHAPES = [(4, 2, 16, 24, 4), (1, 1, 40, 12, 2), (2, 2, 128, 128, 4), (6, 1, 8, 100, 3), (3, 3, 64, 32, 1), (2, 1, 192, 200, 4)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", DELTA_SHAPES)
def test_channel_delta_mixer_alone_whole_in_portions_and_token_by_token(tmp_path, dtype, shape):
    heads, kv, dim, vdim, conv = shape
    layer = _with(_delta(heads, kv, dim, vdim, conv), None)
    cfg, w, sess = _one_layer(tmp_path, layer, dtype=dtype, ranks={"a": 6, "g": 10})
    x = torch.randn(57, 48, generator=torch.Generator().manual_seed(0)).to(TDT[dtype])
    want = P.channel_delta_mixer(x.double(), w, "l0.mix", layer["mixer"], cfg["norm"]["eps"])
    mixer = sess.model.blocks[0].mixer
    tol = 3e-5 if dtype == "float32" else 3e-2
    for cuts in CUTS:
        got = _run_cut(sess, lambda rows, ctx: mixer.forward(rows, ctx, 0, True), x, cuts, f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts


def test_the_delta_rule_reads_out_after_its_own_write_and_decays_per_channel():
    """The recurrence by hand on three tokens: the read-out of a token contains that token's own write, and the
    decay of one key channel leaves the others alone."""
    q = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=torch.float64)
    k = torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.0, 0.0]], dtype=torch.float64)
    v = torch.tensor([[2.0], [3.0], [5.0]], dtype=torch.float64)
    beta = torch.tensor([1.0, 0.5, 1.0], dtype=torch.float64)
    g = torch.tensor([[1.0, 1.0], [0.5, 1.0], [1.0, 0.1]], dtype=torch.float64)
    o = P.delta_recurrence(q, k, v, beta, g)
    # t0: S = [[2],[0]], o = 2.  t1: S row 0 halves to 1, row 1 gets 0.5 * 3 = 1.5, o = 1.5.  t2: row 1 decays to 0.15, no write.
    assert torch.allclose(o.flatten(), torch.tensor([2.0, 1.5, 1.15], dtype=torch.float64))


def test_recurrent_state_of_a_freed_slot_does_not_leak_and_batches_equal_requests_alone(tmp_path):
    layer = _with(_delta(4, 2, 16, 24), None)
    cfg, w, sess = _one_layer(tmp_path, layer)
    g = torch.Generator().manual_seed(1)
    xs = {rid: torch.randn(n, 48, generator=g) * 2 for rid, n in (("a", 9), ("b", 1), ("c", 30), ("d", 2))}
    want = {rid: P.channel_delta_mixer(x.double(), w, "l0.mix", layer["mixer"], cfg["norm"]["eps"]) for rid, x in xs.items()}
    mixer = sess.model.blocks[0].mixer
    for rounds in range(2):                       # the second round runs on slots the first one used
        ctx, entries = _step_context(sess, [(rid, x.shape[0]) for rid, x in xs.items()])
        order = [e.cache.request_id for e in sorted(entries, key=lambda e: 0 if len(e.tokens) == 1 else 1)]
        got = mixer.forward(torch.cat([xs[r] for r in order]).cuda(), ctx, 0, True).cpu().double()
        p = 0
        for r in order:
            n = xs[r].shape[0]
            assert float((got[p:p + n] - want[r]).abs().max()) < 3e-5 * float(want[r].abs().max()), (rounds, r)
            p += n
        for rid in xs:
            sess.cache.free(sess.live.pop(rid))


# ------------------------------------------------------------------ attention: windows, far keys, blended values --
def _queries_like_keys(w, p, mx):
    """Every query head gets minus the matrix, and the convolution, of the key head it reads, and all the convolutions'
    last taps weigh the most.  A run of rows that is minus an earlier run then has a query equal to that run's last
    key (both pass the same convolution and the same norm) and against its own, and that one score stands far above
    the others: an attention that loses or wrongly sees that key gives another result."""
    d, rep = mx["dim"], mx["heads"] // mx["kv_heads"]
    for leaf in (".k.conv", ".v.conv"):
        w[p + leaf] = w[p + leaf] * 0.25
        w[p + leaf][:, -1] = 1.0
    for h in range(mx["heads"]):
        kh = h // rep
        w[p + ".q"][h * d:(h + 1) * d] = -w[p + ".k"][kh * d:(kh + 1) * d]
        w[p + ".q.conv"][h * d:(h + 1) * d] = w[p + ".k.conv"][kh * d:(kh + 1) * d]
    w[p + ".r1"] = w[p + ".r1"] * 0.25


def _standout_inputs(T, width, far, query, taps, seed):
    """Random rows; the last `taps` rows up to `query` are minus the rows up to `far` (rows in front of the sequence
    are zeros, as the convolution sees them)."""
    x = torch.randn(T, width, generator=torch.Generator().manual_seed(seed)) * 0.5
    for m in range(taps):
        if query - m > far:
            x[query - m] = -x[far - m] if far - m >= 0 else 0.0
    return x


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,far,query", [(37, 84, 120), (37, 83, 120), (64, 64, 127), (64, 63, 127), (64, 0, 63), (64, 0, 64),
                                              (16, 1, 16), (16, 0, 16), (200, 220, 419), (200, 219, 419), (40, 3, 40),
                                              (1000, 2, 700), (1000, 15, 700), (1000, 16, 700), (1000, 255, 700), (1000, 256, 700)])
def test_attention_alone_sees_its_window_and_nothing_else(tmp_path, dtype, window, far, query):
    """A key that stands out: just inside or just outside the query's window, at and off page borders, among the first
    tokens, hundreds of tokens back; with the query inside a prompt's portion, at the start of a portion, and decoded."""
    _window_case(tmp_path, dtype, window, far, query, (4, 2, 24, 16))


@pytest.mark.parametrize("window,far,query", [(64, 64, 127), (64, 63, 127), (200, 220, 419), (200, 219, 419), (130, 0, 129),
                                              (130, 0, 130), (300, 1, 300), (300, 2, 300)])
def test_window_edges_with_heads_of_64_on_the_tensor_cores(tmp_path, window, far, query):
    """Heads of 64 elements in bfloat16 take the tcgen05 kernel for a prompt's portions: the same edges there."""
    _window_case(tmp_path, "bfloat16", window, far, query, (4, 2, 64, 48))


def _window_case(tmp_path, dtype, window, far, query, sizes):
    layer = _with(_att(*sizes, window, conv=4, scale=1.5, v_mix=False), None)
    mx = layer["mixer"]
    cfg, w, sess = _one_layer(tmp_path, layer, dtype=dtype, edit=lambda w: _queries_like_keys(w, "l0.mix", mx))
    eps, T = cfg["norm"]["eps"], query + 1
    x = _standout_inputs(T, 48, far, query, 4, far).to(TDT[dtype])
    want, _ = P.attention_mixer(x.double(), w, "l0.mix", mx, eps, None)
    # the test can tell: with every key visible the query's row changes exactly when `far` lies outside the window
    every, _ = P.attention_mixer(x.double(), w, "l0.mix", dict(mx, mask={"size": 1 << 20}), eps, None)
    inside = query - far < window
    moved = float((every[-1] - want[-1]).abs().max()) > 0.1 * float(want[-1].abs().max())
    assert moved == (not inside)
    if inside:      # and a window one token shorter loses it, where it is the window's oldest key
        lost, _ = P.attention_mixer(x.double(), w, "l0.mix", dict(mx, mask={"size": query - far}), eps, None)
        assert float((lost[-1] - want[-1]).abs().max()) > 0.1 * float(want[-1].abs().max())
    mixer = sess.model.blocks[0].mixer
    tol = 3e-5 if dtype == "float32" else 4e-2
    cuttings = [[T], [T - 1, 1], [far + 1, T - far - 1], [max(1, T - 9)] + [1] * min(9, T - 1)]
    if T - far > 2 and far:
        cuttings.append([far, T - far - 2, 2])
    for cuts in cuttings:
        got = _run_cut(sess, lambda rows, ctx: mixer.forward(rows, ctx, 0, True), x, [c for c in cuts if c], f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts
        assert float((got[-1] - want[-1]).abs().max()) <= tol * float(want[-1].abs().max()), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(4, 2, 24, 16, 4), (2, 2, 16, 40, 2), (5, 1, 40, 12, 3), (8, 2, 64, 64, 4), (1, 1, 128, 128, 1),
                                   (34, 2, 16, 16, 2), (3, 1, 80, 72, 4), (2, 1, 192, 64, 3), (2, 2, 100, 256, 2)])
def test_attention_alone_in_other_sizes_whole_in_portions_and_token_by_token(tmp_path, dtype, shape):
    heads, kv, dim, vdim, conv = shape
    layer = _with(_att(heads, kv, dim, vdim, 23, conv=conv, v_mix=False), None)
    cfg, w, sess = _one_layer(tmp_path, layer, dtype=dtype)
    x = torch.randn(57, 48, generator=torch.Generator().manual_seed(0)).to(TDT[dtype])
    want, _ = P.attention_mixer(x.double(), w, "l0.mix", layer["mixer"], cfg["norm"]["eps"], None)
    mixer = sess.model.blocks[0].mixer
    tol = 3e-5 if dtype == "float32" else 3e-2
    for cuts in CUTS:
        got = _run_cut(sess, lambda rows, ctx: mixer.forward(rows, ctx, 0, True), x, cuts, f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts


def test_the_distance_bias_is_taken_off_the_scores(tmp_path):
    """With the bias scaled up, far keys inside the window all but vanish: the plain result moves, and the engine
    moves with it."""
    layer = _with(_att(2, 1, 16, 16, 64, v_mix=False), None)

    def edit(w):
        w["l0.mix.r1"] = w["l0.mix.r1"] * 6.0
    cfg, w, sess = _one_layer(tmp_path, layer, edit=edit)
    x = torch.randn(80, 48, generator=torch.Generator().manual_seed(5))
    want, _ = P.attention_mixer(x.double(), w, "l0.mix", layer["mixer"], cfg["norm"]["eps"], None)
    flat, _ = P.attention_mixer(x.double(), dict(w, **{"l0.mix.r1": w["l0.mix.r1"] * 0}), "l0.mix", layer["mixer"], cfg["norm"]["eps"], None)
    assert float((flat - want).abs().max()) > 0.2 * float(want.abs().max())
    mixer = sess.model.blocks[0].mixer
    for cuts in ([80], [50] + [1] * 30):
        got = _run_cut(sess, lambda rows, ctx: mixer.forward(rows, ctx, 0, True), x, cuts, f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= 3e-5 * float(want.abs().max()), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_values_are_blended_with_the_first_blending_layer_s_and_the_blend_is_what_the_cache_holds(tmp_path, dtype):
    layers = [_with(_att(4, 2, 24, 16, 30, conv=4), None), _with(_att(2, 1, 16, 32, 30, conv=2), None)]

    def edit(w):
        w["l1.mix.vmix"] = torch.tensor(0.75)
        w["l0.mix.vmix"] = torch.tensor(0.5)              # the first layer's factor is not used
    cfg, w, sess = _one_layer(tmp_path, layers, dtype=dtype, edit=edit)
    eps = cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(7)
    x0, x1 = torch.randn(57, 48, generator=g).to(TDT[dtype]), torch.randn(57, 48, generator=g).to(TDT[dtype])
    want0, v_first = P.attention_mixer(x0.double(), w, "l0.mix", layers[0]["mixer"], eps, None)
    want1, _ = P.attention_mixer(x1.double(), w, "l1.mix", layers[1]["mixer"], eps, v_first)
    alone, _ = P.attention_mixer(x1.double(), w, "l1.mix", layers[1]["mixer"], eps, None)
    assert float((alone - want1).abs().max()) > 0.2 * float(want1.abs().max())
    m0, m1 = sess.model.blocks[0].mixer, sess.model.blocks[1].mixer
    tol = 3e-5 if dtype == "float32" else 3e-2
    for cuts in CUTS:           # decoded tokens read blended values that earlier steps put into the cache
        rid, rows0, rows1, p = f"r{len(cuts)}", [], [], 0
        for n in cuts:
            ctx, entries = _step_context(sess, [(rid, n)])
            rows0.append(m0.forward(x0[p:p + n].cuda().contiguous(), ctx, 0, True).float().cpu())
            rows1.append(m1.forward(x1[p:p + n].cuda().contiguous(), ctx, 1, True).float().cpu())
            _advance(sess, entries)
            p += n
        sess.cache.free(sess.live.pop(rid))
        assert float((torch.cat(rows0).double() - want0).abs().max()) <= tol * float(want0.abs().max()), cuts
        assert float((torch.cat(rows1).double() - want1).abs().max()) <= tol * float(want1.abs().max()), cuts


def test_attention_in_a_batch_of_unequal_requests_on_reused_pages_and_slots(tmp_path):
    layers = [_with(_att(4, 2, 24, 16, 45, conv=4), None), _with(_att(2, 2, 8, 16, 70, conv=3), None)]
    cfg, w, sess = _one_layer(tmp_path, layers, max_tokens=512, block=8)
    eps = cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(4)
    mixers = [sess.model.blocks[0].mixer, sess.model.blocks[1].mixer]
    for rounds in range(3):
        xs = {rid: (torch.randn(n, 48, generator=g), torch.randn(n, 48, generator=g)) for rid, n in (("a", 70), ("b", 1), ("c", 129), ("d", 2))}
        want = {}
        for rid, (a, b) in xs.items():
            o0, vf = P.attention_mixer(a.double(), w, "l0.mix", layers[0]["mixer"], eps, None)
            want[rid] = (o0, P.attention_mixer(b.double(), w, "l1.mix", layers[1]["mixer"], eps, vf)[0])
        done = {rid: 0 for rid in xs}
        for take in ({"a": 33, "b": 1, "c": 64, "d": 1}, {"a": 36, "c": 1, "d": 1}, {"a": 1, "c": 64}):
            ctx, entries = _step_context(sess, list(take.items()))
            order = [e.cache.request_id for e in sorted(entries, key=lambda e: 0 if len(e.tokens) == 1 else 1)]
            for k in (0, 1):
                xin = torch.cat([xs[r][k][done[r]:done[r] + take[r]] for r in order])
                got = mixers[k].forward(xin.cuda(), ctx, k, True).cpu().double()
                p = 0
                for r in order:
                    ref = want[r][k][done[r]:done[r] + take[r]]
                    assert float((got[p:p + take[r]] - ref).abs().max()) < 3e-5 * float(want[r][k].abs().max()), (rounds, r, k)
                    p += take[r]
            for r in order:
                done[r] += take[r]
            _advance(sess, entries)
        for rid in xs:
            sess.cache.free(sess.live.pop(rid))
        sess.cache.check()


def _batch_step(sess, mixer, xs, take, done):
    """One step of the requests in ``take`` (id -> tokens) through ``mixer``; returns id -> rows."""
    ctx, entries = _step_context(sess, list(take.items()))
    order = [e.cache.request_id for e in sorted(entries, key=lambda e: 0 if len(e.tokens) == 1 else 1)]
    xin = torch.cat([xs[r][done[r]:done[r] + take[r]] for r in order])
    got = mixer.forward(xin.cuda(), ctx, 0, True).float().cpu().double()
    out, p = {}, 0
    for r in order:
        out[r] = got[p:p + take[r]]
        p += take[r]
        done[r] += take[r]
    _advance(sess, entries)
    return out


def test_long_steps_of_several_requests_prepare_their_heads_like_short_ones(tmp_path):
    """In long steps a block of the head-preparing kernel walks a run of neighbouring tokens, which may belong to
    several requests and start behind rows that an earlier step left in the slot."""
    layer = _with(_att(4, 2, 64, 48, 23, conv=4, v_mix=False), None)
    cfg, w, sess = _one_layer(tmp_path, layer, dtype="bfloat16", max_tokens=20480)
    mixer = sess.model.blocks[0].mixer
    g = torch.Generator().manual_seed(7)
    # a step of 1000 to 8000 tokens against the plain implementation: three requests, the third continued
    lens = {"a": 701, "b": 3, "c": 530}
    xs = {r: torch.randn(n, 48, generator=g).to(torch.bfloat16) for r, n in lens.items()}
    want = {r: P.attention_mixer(x.double(), w, "l0.mix", layer["mixer"], cfg["norm"]["eps"], None)[0] for r, x in xs.items()}
    done = {r: 0 for r in lens}
    got = {r: [] for r in lens}
    for take in ({"c": 29}, {"a": 701, "b": 3, "c": 501}):
        for r, rows in _batch_step(sess, mixer, xs, take, done).items():
            got[r].append(rows)
    for r in lens:
        rows = torch.cat(got[r])
        assert float((rows - want[r]).abs().max()) <= 3e-2 * float(want[r].abs().max()), r
        sess.cache.free(sess.live.pop(r))
    # a step of more than 8192 tokens against the same requests in portions of a few hundred
    lens = {"a": 3001, "b": 1, "c": 5203, "d": 2}
    xs = {r: torch.randn(n, 48, generator=g).to(torch.bfloat16) for r, n in lens.items()}
    done = {r: 0 for r in lens}
    whole = _batch_step(sess, mixer, xs, dict(lens), done)
    for r in lens:
        sess.cache.free(sess.live.pop(r))
    for r, n in lens.items():
        done, rows = {r: 0}, []
        while done[r] < n:
            rows.append(_batch_step(sess, mixer, xs, {r: min(613, n - done[r])}, done)[r])
        rows = torch.cat(rows)
        sess.cache.free(sess.live.pop(r))
        assert float((rows - whole[r]).abs().max()) <= 3e-2 * float(rows.abs().max()), r
    sess.cache.check()


# ------------------------------------------------------------------ long decoding, generation --
def test_long_decoding_moves_every_window_over_decoded_tokens(tmp_path):
    cfg = CONFIGS["both_mixers"]
    model_dir, w = _model_dir(tmp_path, "long", cfg, seed=4)
    toks = U.make_requests(cfg["vocab"], [230], 2)["r0"]
    plain = {"r0": P.forward(cfg, w, toks).numpy()}
    steps = U.trace_tail_decode({"r0": toks}, tail=220)
    sess = _session(model_dir, "float32", 64 + 16, block=8)          # less than the request: pages behind the windows go back
    U.compare(U.run_trace(sess, steps), plain, U.TOL["float32"], "long decoding")
    sess.cache.check()


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["both_mixers", "odd_sizes"])
def test_greedy_generation_through_the_engine(tmp_path, name, graphs):
    from firefly_b200 import LLM
    cfg = CONFIGS[name]
    model_dir, w = _model_dir(tmp_path, "gen", cfg, seed=6)
    prompts = [v for v in U.make_requests(cfg["vocab"], [19, 3, 41, 8, 27], 11).values()]
    llm = LLM(model_dir, dtype="float32", max_batch_size_limit=3, kv_block_size=8, num_kv_blocks=40,
              max_prefill_chunk_size=16, eos_token_ids=[], use_cuda_graphs=graphs)
    outs = llm.generate(prompts, max_tokens=10, ignore_eos=True)
    llm.engine.cache.check()
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        rows = P.forward(cfg, w, list(p) + o[:-1])
        for i, tok in enumerate(o):
            row = rows[len(p) - 1 + i]
            top2 = torch.topk(row, 2).values
            assert tok == int(row.argmax()) or float(top2[0] - top2[1]) < 1e-4 * float(row.abs().max()), (i, tok)


def test_the_command_line_generates_from_a_folder_and_from_a_configuration(tmp_path):
    import subprocess
    import sys
    cfg = CONFIGS["both_mixers"]
    model_dir, _ = _model_dir(tmp_path, "cli", cfg)
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "bin", "firefly")
    out = subprocess.run([sys.executable, exe, model_dir, "--prompt-ids", "5,9,2", "--max-tokens", "4", "--ignore-eos"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    assert len(json.loads(out.stdout.strip().splitlines()[-1])["tokens"]) == 4
    conf = tmp_path / "c.json"
    conf.write_text(json.dumps(CONFIGS["odd_sizes"]))
    out = subprocess.run([sys.executable, exe, "--random", str(conf), "--prompt-len", "9", "--num-prompts", "2",
                          "--max-tokens", "3", "--ignore-eos"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr


def test_the_trace_program_replays_a_mixed_schedule(tmp_path):
    import subprocess
    import sys
    cfg = CONFIGS["attention_only"]
    model_dir, w = _model_dir(tmp_path, "prog", cfg, seed=9)
    reqs = U.make_requests(cfg["vocab"], [40, 9, 77, 2, 31], 3)
    plain = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    steps = U.trace_mixed(reqs, seed=1, max_live=4)
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "bin", "trace_run")
    out = tmp_path / "out"
    run = subprocess.run([sys.executable, exe, "--model", model_dir, "--dtype", "float32", "--out", str(out),
                          "--max-tokens", str(U.peak_tokens(steps))], input="".join(json.dumps(s) + "\n" for s in steps),
                         capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stderr
    assert [ln for ln in run.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
    done = {}
    for rec in steps:
        arr = np.fromfile(out / f"{rec['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        k = 0
        for ent in rec["entries"]:
            base = done.get(ent["id"], 0)
            for wpos in ent["want"]:
                assert U.rel_err(arr[k], plain[ent["id"]][base + wpos]) <= U.TOL["float32"], (rec["step"], ent["id"], wpos)
                k += 1
            done[ent["id"]] = base + len(ent["tokens"])
        assert k == arr.shape[0]
