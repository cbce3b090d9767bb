"""Papusun on the device against the plain implementation in ``plain_papusun.py``: every mechanism alone, then
whole models of several shapes through the replay session (whole prompts, decoding token by token, portions down
to two tokens, mixed batches with pages and state slots used again) and greedy generation through the engine and
its scheduler."""
import json
import os

import numpy as np
import pytest
import torch

import plain_papusun as P
import replay_util as U

pytestmark = pytest.mark.gpu

BANDS = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}


def _lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, scale=None, base=3000.0, kv_from=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
          "scale": scale or (dim + rot_dim) ** -0.5 * 1.5, "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mx}


def _left(heads, kv_heads, dim, vdim, dims=None, softcap=6.0, scaling=BANDS, scale=None, base=700.0):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if scaling:
        rot["scaling"] = dict(scaling)
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5 * 2.0, "rot": rot}
    if softcap:
        out["softcap"] = softcap
    return out


def _right(heads, kv_heads, dim, vdim, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _par(left, right, left_scale=1.3, right_scale=0.6):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _cfg(layers, width=48, vocab=101, eps=1e-5, logit_scale=1.7, side=12):
    out = {"architecture": "Papusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
           "layers": layers}
    if side:
        out["token_side"] = {"dim": side}
    return out


def _with(layer, mlp):
    return dict(layer, mlp=mlp)


CONFIGS = {
    # both kinds of mixer in an order of their own; a layer that reads another layer's cache rows with a longer and
    # one with a shorter window than that layer's own; value heads shorter and longer than key heads; windows that
    # are no multiple of a page; a rotation over part of the head with rescaled frequencies; layers with and without
    # a feed-forward
    "both_mixers": _cfg([_with(_lat(4, 16, 8, 24, 24, 40, 21), _dense(72)),
                         _with(_par(_left(4, 2, 24, 40, dims=16), _right(4, 2, 16, 24)), None),
                         _with(_lat(2, 8, 8, 12, 24, 16, 37, kv_from=0), _dense(72)),
                         _with(_lat(3, 16, 16, 8, 32, 24, 30), None),
                         _with(_par(_left(6, 2, 16, 8, dims=8, scaling=None), _right(3, 3, 8, 12, conv=2)), _dense(40)),
                         _with(_lat(4, 16, 8, 8, 24, 8, 9, kv_from=0), _dense(72))]),
    # the values a model may happen to make equal or one: as many kv heads as heads, one q/k head for all recurrent
    # heads, key and value heads of one size, one tap (no convolution state), a window of one token and one wider
    # than any request, the whole head rotated, no rescaling, no cap, scales of one, equal ranks, a side input of one
    # number, one head
    "equal_or_one": _cfg([_with(_par(_left(2, 2, 16, 16, softcap=None, scaling=None), _right(2, 1, 32, 32, conv=1), 1.0, 1.0), _dense(64)),
                          _with(_lat(1, 16, 16, 16, 16, 16, 1 << 16, scale=0.2), _dense(64)),
                          _with(_lat(2, 8, 16, 8, 16, 16, 1, kv_from=1), _dense(64))],
                         width=64, vocab=131, logit_scale=1.0, side=1),
    # sizes that no fast path takes: a width that is no multiple of 8, heads of 20, 12 and 40, three query heads on a
    # kv head, five taps, a window of one page, a side input of five numbers, a cache row of 26 elements
    "odd_sizes": _cfg([_with(_par(_left(3, 1, 20, 12, dims=10), _right(3, 1, 20, 40, conv=5)), _dense(50)),
                       _with(_lat(3, 12, 6, 20, 20, 10, 16), _dense(50)),
                       _with(_lat(5, 4, 6, 12, 20, 12, 19, kv_from=1), None)], width=36, vocab=50, side=5),
    # recurrent and full attention only: state slots and pages that no window gives back
    "parallel_only": _cfg([_with(_par(_left(4, 1, 32, 16, dims=32), _right(2, 2, 64, 16)), _dense(40)),
                           _with(_par(_left(2, 2, 16, 32, dims=4, softcap=1.5), _right(4, 1, 8, 8, conv=4)), None)], width=40),
    # latent attention only, no side input: no state slots at all
    "latent_only": _cfg([_with(_lat(4, 16, 16, 16, 48, 32, 33), _dense(48)), _with(_lat(8, 8, 16, 8, 48, 16, 64, kv_from=0), None),
                         _with(_lat(2, 32, 8, 16, 24, 24, 16), _dense(48))], side=0),
    # sizes that every fast path takes in bfloat16: attention heads of 64 and 128 and a cache row of 64 and 128
    # elements (the tcgen05 attention kernel, with the cap and with a window), a recurrent key of 128
    "fast_paths": _cfg([_with(_par(_left(4, 2, 64, 64, dims=32), _right(2, 1, 128, 64, conv=4)), _dense(72)),
                        _with(_lat(4, 32, 16, 32, 48, 64, 70), _dense(64)),
                        _with(_par(_left(2, 1, 64, 128, dims=64, softcap=20.0), _right(4, 2, 64, 64)), None),
                        _with(_lat(2, 64, 32, 64, 96, 32, 100), None),
                        _with(_lat(8, 16, 16, 16, 48, 64, 33, kv_from=1), _dense(64))], width=64, vocab=97, side=8),
}


def _model_dir(tmp_path, name, cfg, seed=1, edit=None):
    w = P.random_weights(cfg, seed)
    if edit is not None:
        edit(w)
        w = {k: v.to(torch.bfloat16).to(v.dtype) for k, v in w.items()}        # what the file will hold
    U.write_model_dir(str(tmp_path / name), cfg, {k: v.float() for k, v in w.items()}, torch.bfloat16)
    return str(tmp_path / name), {k: v.double() for k, v in w.items()}       # the plain functions run in 64-bit


def _session(model_dir, dtype, max_tokens, block=16, max_requests=4):
    from firefly_b200.replay import ReplaySession
    return ReplaySession(model_dir, dtype=dtype, max_tokens=max_tokens, block_size=block, max_requests=max_requests)


def _compare_most(got, plain, tol, what, frac=0.9, worst=8.0):
    """``frac`` of the rows within tol, and every row finite and within ``worst`` tol: the head norm of the recurrent
    mixer and the norm of the side input divide by their input's root mean square, which magnifies bfloat16 rounding
    in a row where that input is small (a side input of few numbers is small wherever all its gates are closed)."""
    errs = sorted(U.rel_err(row, plain[rid.split("#")[0]][pos]) for (rid, pos), row in got.rows.items())
    assert errs and all(e == e for e in errs), what
    assert errs[-1] <= worst * tol and errs[int(frac * (len(errs) - 1))] <= tol, \
        f"{what}: worst {errs[-1]:.3e}, {frac:.0%} quantile {errs[int(frac * (len(errs) - 1))]:.3e}, tol {tol:g}"


def _check(got, plain, dtype, what, worst=8.0):
    if dtype == "float32":
        U.compare(got, plain, U.TOL[dtype], what)
    else:
        _compare_most(got, plain, U.TOL[dtype], what, worst=worst)


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
        # a side input of one number flips its sign where its one gate is about closed: in bfloat16 such a row is far off
        _check(got, plain, dtype, f"{name}/{dtype}/{label}", worst=25.0 if name == "equal_or_one" else 8.0)
        sess.cache.check()
        assert not sess.cache.live


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_requests_at_middling_sizes(tmp_path, dtype):
    """Requests of hundreds of tokens (whole, with a decoded tail, and mixed on reused pages and slots) through a model
    whose attention layers take, in bfloat16, the tcgen05 kernel (cache rows of 64 and 256, heads of 64) and the
    mma.sync kernel (heads of 80), with windows that end inside the prompts."""
    cfg = _cfg([_with(_lat(4, 24, 8, 40, 56, 48, 50), _dense(128)),
                _with(_par(_left(6, 2, 40, 80, dims=20), _right(4, 2, 24, 40, conv=4)), _dense(128)),
                _with(_lat(3, 16, 8, 24, 56, 24, 70, kv_from=0), None),
                _with(_par(_left(4, 4, 64, 32, dims=64, softcap=4.0), _right(2, 1, 64, 64)), _dense(96)),
                _with(_lat(2, 64, 64, 64, 192, 32, 33), _dense(128))], width=96, vocab=211, side=16)
    model_dir, w = _model_dir(tmp_path, "middling", cfg, seed=3)
    reqs = U.make_requests(cfg["vocab"], [600, 260, 90], 9)
    plain = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    twice = dict(reqs, **{"r1#2": reqs["r1"]})
    for label, steps in (("whole", U.trace_whole(reqs)), ("decode", U.trace_tail_decode(reqs, tail=48)),
                         ("mixed", U.trace_mixed(twice, seed=5, max_live=3, sizes=(64, 2, 129, 31, 3, 200)))):
        sess = _session(model_dir, dtype, U.peak_tokens(steps))
        _check(U.run_trace(sess, steps), plain, dtype, f"middling/{dtype}/{label}")
        sess.cache.check()
        assert not sess.cache.live


def test_the_stream_matches_after_every_layer(tmp_path):
    cfg = CONFIGS["both_mixers"]
    model_dir, w = _model_dir(tmp_path, "stream", cfg)
    toks = U.make_requests(cfg["vocab"], [45], 8)["r0"]
    want = []
    P.forward(cfg, w, toks, streams=want)
    sess = _session(model_dir, "float32", 64)
    got = []

    def after(i, res, pending):
        x = res.detach().clone()
        if isinstance(pending, torch.Tensor):
            x += pending.float()
        got.append(x.cpu().double())
    sess.model.after_run = after
    sess.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [0]}], "end": ["a"]})
    assert len(got) == len(cfg["layers"]) == 6
    for i, g in enumerate(got):
        assert float((g - want[i]).abs().max()) < 2e-5 * float(want[i].abs().max()), f"after layer {i}"


# ------------------------------------------------------------------ mechanisms alone --
def _one_layer(tmp_path, layers, width=48, dtype="float32", seed=2, max_tokens=1024, block=16, edit=None, side=6):
    cfg = _cfg(layers if isinstance(layers, list) else [layers], width=width, side=side)
    model_dir, w = _model_dir(tmp_path, "one", cfg, seed, edit=edit)
    return cfg, w, _session(model_dir, dtype, max_tokens, block=block)


def _step_context(sess, seqs, tokens=None):
    """A StepContext for sequences given as (request id, new tokens): admits, grows, builds."""
    from firefly_b200.engine.runner import StepEntry
    entries = []
    for rid, n in seqs:
        rc = sess.live.get(rid) or sess.cache.admit(rid)
        sess.live[rid] = rc
        assert sess.cache.grow(rc, rc.num_tokens + n)
        entries.append(StepEntry(rc, list(tokens[rid]) if tokens else [0] * n, []))
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
POS = torch.arange(57)


def test_layer_norm_without_a_bias_alone(tmp_path):
    cfg, w, sess = _one_layer(tmp_path, _with(_lat(1, 8, 8, 8, 8, 8, 4), _dense(16)))
    ctx, _ = _step_context(sess, [("a", 11)])
    g = torch.Generator().manual_seed(3)
    res, delta = torch.randn(11, 48, generator=g) * 3 + 1, torch.randn(11, 48, generator=g)
    r = res.cuda()
    norm = sess.model.blocks[0].norms[1]
    assert norm.bias is None
    got = norm.forward(r, delta.cuda(), ctx)
    summed = res.double() + delta.double()
    assert torch.allclose(r.cpu().double(), summed, atol=1e-6)                  # the sum goes into the stream, in 32-bit
    want = P.layer_norm(summed, w["l0.norm2"], cfg["norm"]["eps"])
    assert float((got.cpu().double() - want).abs().max()) < 1e-5
    assert float((want - P.rms(summed, cfg["norm"]["eps"]) * w["l0.norm2"]).abs().max()) > 0.1   # the mean is taken off


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tokens,side,layer", [(1, 6, 0), (5, 1, 1), (32, 12, 2), (33, 12, 0), (150, 20, 1), (70, 7, 2)])
def test_token_side_alone_reads_its_own_columns_of_the_table(tmp_path, dtype, tokens, side, layer):
    layers = [_with(_lat(1, 8, 8, 8, 8, 8, 4), None)] * 3
    cfg, w, sess = _one_layer(tmp_path, layers, dtype=dtype, side=side)
    g = torch.Generator().manual_seed(tokens)
    toks = torch.randint(0, cfg["vocab"], (tokens,), generator=g).tolist()
    x = torch.randn(tokens, 48, generator=g) * 2
    pending = (torch.randn(tokens, 48, generator=g) * 0.5).to(TDT[dtype])
    summed = x.double() + pending.double()
    want = P.token_side(summed, torch.tensor(toks), w, layer, side, cfg["norm"]["eps"])
    ctx, _ = _step_context(sess, [("a", tokens)], {"a": toks})
    r = x.cuda()
    res, left = sess.model.blocks[layer].tail.forward(r, pending.cuda(), ctx)
    assert left is None and res is r
    tol = 2e-5 if dtype == "float32" else 2e-2
    # what the part adds, against what it should add
    assert float((r.cpu().double() - want).abs().max()) <= tol * float((want - summed).abs().max())
    # and another layer's columns would have given something else
    other = P.token_side(summed, torch.tensor(toks), w, (layer + 1) % 3, side, cfg["norm"]["eps"])
    assert float((other - want).abs().max()) > 0.1


LEFT_SHAPES = [(4, 2, 24, 40, 16), (2, 2, 16, 16, 16), (3, 1, 20, 12, 10), (4, 2, 64, 64, 32), (2, 1, 64, 128, 64),
               (34, 2, 16, 16, 2), (2, 1, 192, 96, 96), (1, 1, 100, 256, 50)]


def _left_mixer(sess):
    from firefly_b200.cache.spec import sub_slot
    m = sess.model.blocks[0].mixer.mixers[0]
    return lambda rows, ctx: m.forward(rows, ctx, sub_slot(0, 0), True)


def _right_mixer(sess):
    from firefly_b200.cache.spec import sub_slot
    m = sess.model.blocks[0].mixer.mixers[1]
    return lambda rows, ctx: m.forward(rows, ctx, sub_slot(0, 1), True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", LEFT_SHAPES)
def test_capped_attention_alone_whole_in_portions_and_token_by_token(tmp_path, dtype, shape):
    heads, kv, dim, vdim, dims = shape
    left = _left(heads, kv, dim, vdim, dims=dims, softcap=3.0, scale=dim ** -0.5 * 4.0)
    cfg, w, sess = _one_layer(tmp_path, _with(_par(left, _right(1, 1, 8, 8)), None), dtype=dtype)
    x = torch.randn(57, 48, generator=torch.Generator().manual_seed(0)).to(TDT[dtype])
    want = P.capped_attention(x.double(), w, "l0.mix.left", left, POS)
    # the cap is at work: without it the result is another one
    free = P.capped_attention(x.double(), w, "l0.mix.left", dict(left, softcap=None), POS)
    assert float((free - want).abs().max()) > 0.02 * float(want.abs().max())
    tol = 3e-5 if dtype == "float32" else 3e-2
    for cuts in CUTS:
        got = _run_cut(sess, _left_mixer(sess), x, cuts, f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts


def _queries_like_keys(w, p, mx, gain):
    """Every query head becomes minus `gain` times the key head it reads, on the elements that do not turn (the
    turning ones are made small), without biases.  A row that is minus an earlier row then has a query along that
    row's key and against its own: that one score stands far above the others, and an attention that loses that key
    gives another result."""
    d, rep, dims = mx["dim"], mx["heads"] // mx["kv_heads"], mx["rot"]["dims"]
    for h in range(mx["heads"]):
        kh = h // rep
        w[p + ".q"][h * d:(h + 1) * d] = -gain * w[p + ".k"][kh * d:(kh + 1) * d]
        w[p + ".q"][h * d:h * d + dims] *= 0.02
    w[p + ".q.b"].zero_()
    w[p + ".k.b"].zero_()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes,far,query", [((4, 2, 24, 16, 8), 0, 700), ((4, 2, 24, 16, 8), 15, 700), ((4, 2, 24, 16, 8), 16, 700),
                                             ((4, 2, 24, 16, 8), 255, 700), ((4, 2, 24, 16, 8), 3, 40),
                                             ((4, 2, 64, 48, 16), 256, 700), ((4, 2, 64, 48, 16), 1, 300),
                                             ((2, 2, 128, 128, 32), 63, 419)])
def test_full_attention_finds_a_key_far_back(tmp_path, dtype, sizes, far, query):
    """A key that stands out among hundreds, at and off page borders, among the first tokens; with the query inside
    a prompt, at the start of a portion, and decoded.  The capped score stays the largest."""
    heads, kv, dim, vdim, dims = sizes
    left = _left(heads, kv, dim, vdim, dims=dims, softcap=20.0, scale=1.0)
    cfg, w, sess = _one_layer(tmp_path, _with(_par(left, _right(1, 1, 8, 8)), None), dtype=dtype,
                              edit=lambda w: _queries_like_keys(w, "l0.mix.left", left, 0.07))
    T = query + 1
    x = torch.randn(T, 48, generator=torch.Generator().manual_seed(far)) * 0.7
    x[far] *= 3.0                 # nothing norms a mixer's input here: the row's key and the query against it grow
    x[query] = -x[far]
    x = x.to(TDT[dtype])
    pos = torch.arange(T)
    want = P.capped_attention(x.double(), w, "l0.mix.left", left, pos)
    # the test can tell: without that key the query's row is another one
    y = x.double().clone()
    y[far] = 0.0
    lost = P.capped_attention(y, w, "l0.mix.left", left, pos)
    assert float((lost[-1] - want[-1]).abs().max()) > 0.2 * float(want[-1].abs().max())
    tol = 3e-5 if dtype == "float32" else 4e-2
    for cuts in ([T], [T - 1, 1], [far + 1, T - far - 1], [max(1, T - 9)] + [1] * min(9, T - 1)):
        got = _run_cut(sess, _left_mixer(sess), x, [c for c in cuts if c], f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts
        assert float((got[-1] - want[-1]).abs().max()) <= tol * float(want[-1].abs().max()), cuts


DELTA_SHAPES = [(4, 2, 16, 24, 4), (1, 1, 40, 12, 2), (2, 2, 128, 128, 4), (6, 1, 8, 100, 3), (3, 3, 64, 32, 1), (2, 1, 192, 200, 4)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", DELTA_SHAPES)
def test_gated_delta_mixer_alone_whole_in_portions_and_token_by_token(tmp_path, dtype, shape):
    heads, kv, dim, vdim, conv = shape
    right = _right(heads, kv, dim, vdim, conv)
    cfg, w, sess = _one_layer(tmp_path, _with(_par(_left(1, 1, 8, 8), right), None), dtype=dtype)
    x = torch.randn(57, 48, generator=torch.Generator().manual_seed(0)).to(TDT[dtype])
    want = P.delta_rule(x.double(), w, "l0.mix.right", right, cfg["norm"]["eps"])
    tol = 3e-5 if dtype == "float32" else 3e-2
    for cuts in CUTS:
        got = _run_cut(sess, _right_mixer(sess), x, cuts, f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), cuts


def test_a_head_s_decay_is_its_own(tmp_path):
    """With one head's decay made strong (a large A_log) that head forgets at once and the others do not: the plain
    result moves in that head's columns of the read-out only, and the engine moves with it."""
    right = _right(3, 1, 16, 8, 2)

    def edit(w):
        w["l0.mix.right.A_log"] = torch.tensor([-1.0, 4.0, -1.0])
        w["l0.mix.right.dt_bias"] = torch.tensor([0.0, 2.0, 0.0])
        w["l0.mix.right.o"] = torch.eye(48)[:, :24].contiguous()        # the heads' columns reach the output one to one
    cfg, w, sess = _one_layer(tmp_path, _with(_par(_left(1, 1, 8, 8), right), None), edit=edit)
    x = torch.randn(40, 48, generator=torch.Generator().manual_seed(4))
    want = P.delta_rule(x.double(), w, "l0.mix.right", right, cfg["norm"]["eps"])
    mild = P.delta_rule(x.double(), dict(w, **{"l0.mix.right.A_log": torch.tensor([-1.0, -1.0, -1.0]).double()}),
                        "l0.mix.right", right, cfg["norm"]["eps"])
    assert torch.allclose(mild[:, :8], want[:, :8]) and torch.allclose(mild[:, 16:24], want[:, 16:24])
    assert float((mild[:, 8:16] - want[:, 8:16]).abs().max()) > 0.05
    for cuts in ([40], [13, 2] + [1] * 25):
        got = _run_cut(sess, _right_mixer(sess), x, cuts, f"r{len(cuts)}")
        assert float((got - want).abs().max()) <= 3e-5 * float(want.abs().max()), cuts


def test_recurrent_state_of_a_freed_slot_does_not_leak_and_batches_equal_requests_alone(tmp_path):
    right = _right(4, 2, 16, 24)
    cfg, w, sess = _one_layer(tmp_path, _with(_par(_left(1, 1, 8, 8), right), None))
    g = torch.Generator().manual_seed(1)
    xs = {rid: torch.randn(n, 48, generator=g) * 2 for rid, n in (("a", 9), ("b", 1), ("c", 30), ("d", 2))}
    want = {rid: P.delta_rule(x.double(), w, "l0.mix.right", right, cfg["norm"]["eps"]) for rid, x in xs.items()}
    call = _right_mixer(sess)
    for rounds in range(2):                       # the second round runs on slots the first one used
        ctx, entries = _step_context(sess, [(rid, x.shape[0]) for rid, x in xs.items()])
        order = [e.cache.request_id for e in sorted(entries, key=lambda e: 0 if len(e.tokens) == 1 else 1)]
        got = call(torch.cat([xs[r] for r in order]).cuda(), ctx).cpu().double()
        p = 0
        for r in order:
            n = xs[r].shape[0]
            assert float((got[p:p + n] - want[r]).abs().max()) < 3e-5 * float(want[r].abs().max()), (rounds, r)
            p += n
        for rid in xs:
            sess.cache.free(sess.live.pop(rid))


LATENT_SHAPES = [(4, 16, 8, 24, 24, 40), (1, 16, 16, 16, 16, 16), (3, 12, 6, 20, 20, 10), (4, 32, 16, 32, 48, 64), (2, 64, 32, 64, 96, 32),
                 (20, 8, 4, 8, 28, 12), (2, 32, 64, 16, 192, 24)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", LATENT_SHAPES)
def test_latent_attention_alone_and_a_second_layer_on_the_first_one_s_rows(tmp_path, dtype, shape):
    heads, dim, rot, vdim, kv_rank, q_rank = shape
    own = _lat(heads, dim, rot, vdim, kv_rank, q_rank, 23)
    reader = _lat(max(1, heads // 2), dim + 4, rot, vdim + 8, kv_rank, q_rank + 8, 31, kv_from=0)
    cfg, w, sess = _one_layer(tmp_path, [_with(own, None), _with(reader, None)], dtype=dtype)
    eps = cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(0)
    x0, x1 = torch.randn(57, 48, generator=g).to(TDT[dtype]), torch.randn(57, 48, generator=g).to(TDT[dtype])
    rows = P.latent_rows(x0.double(), w, "l0.mix", own["mixer"], POS, eps)
    want0 = P.latent_attention(x0.double(), w, "l0.mix", own["mixer"], POS, eps, rows)
    want1 = P.latent_attention(x1.double(), w, "l1.mix", reader["mixer"], POS, eps, rows)
    m0, m1 = sess.model.blocks[0].mixer, sess.model.blocks[1].mixer
    assert m1.cache_spec() == m0.cache_spec() and m0.cache_spec().window == 31
    tol = 3e-5 if dtype == "float32" else 3e-2

    def both(rows_in, ctx):
        n = rows_in.shape[0] // 2
        a = m0.forward(rows_in[:n].contiguous(), ctx, 0, True).float().clone()
        b = m1.forward(rows_in[n:].contiguous(), ctx, 0, False).float()
        return torch.cat([a, b], dim=1)
    for cuts in CUTS:
        # the two layers' inputs travel side by side through the cutting
        out, p = [], 0
        for n in cuts:
            ctx, entries = _step_context(sess, [("r", n)])
            out.append(both(torch.cat([x0[p:p + n], x1[p:p + n]]).cuda(), ctx).cpu())
            _advance(sess, entries)
            p += n
        sess.cache.free(sess.live.pop("r"))
        got = torch.cat(out).double()
        assert float((got[:, :48] - want0).abs().max()) <= tol * float(want0.abs().max()), cuts
        assert float((got[:, 48:] - want1).abs().max()) <= tol * float(want1.abs().max()), cuts


def _latent_queries_like_keys(w, p, mx, gain):
    """The queries' latent is made the keys' (same down projection, same norm) and every head's plain query rows minus
    `gain` times its key rows; the turning part is made small.  A row that is minus an earlier row then has a query
    along that row's key and against its own."""
    H, d, rd, r = mx["heads"], mx["dim"], mx["rot_dim"], mx["kv_rank"]
    w[p + ".dq"] = w[p + ".dkv"][:r].clone()
    w[p + ".dq.norm"] = w[p + ".dkv.norm"].clone()
    uq = w[p + ".uq"].view(H, d + rd, r)
    uq[:, :d] = -gain * w[p + ".uk"].view(H, d, r)
    uq[:, d:] *= 0.02
    w[p + ".dkv"][r:] *= 0.1


def _window_case(tmp_path, dtype, window, far, query, sizes, block=16):
    heads, dim, rot, vdim, rank = sizes
    layer = _with(_lat(heads, dim, rot, vdim, rank, rank, window, scale=0.8), None)
    mx = layer["mixer"]
    cfg, w, sess = _one_layer(tmp_path, layer, dtype=dtype, block=block,
                              edit=lambda w: _latent_queries_like_keys(w, "l0.mix", mx, 1.5))
    eps, T = cfg["norm"]["eps"], query + 1
    x = torch.randn(T, 48, generator=torch.Generator().manual_seed(far + 1)) * 0.7
    x[query] = -x[far]
    x = x.to(TDT[dtype])
    pos = torch.arange(T)

    def plain(m):
        return P.latent_attention(x.double(), w, "l0.mix", m, pos, eps, P.latent_rows(x.double(), w, "l0.mix", m, pos, eps))
    want = plain(mx)
    # the test can tell: with every key visible the query's row changes exactly when `far` lies outside the window
    every = plain(dict(mx, mask={"size": 1 << 20}))
    inside = query - far < window
    moved = float((every[-1] - want[-1]).abs().max()) > 0.1 * float(want[-1].abs().max())
    assert moved == (not inside)
    if inside:      # and a window one token shorter loses it, where it is the window's oldest key
        lost = plain(dict(mx, mask={"size": query - far}))
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
@pytest.mark.parametrize("window,far,query", [(37, 84, 120), (37, 83, 120), (64, 64, 127), (64, 63, 127), (64, 0, 63), (64, 0, 64),
                                              (16, 1, 16), (16, 0, 16), (200, 220, 419), (200, 219, 419), (40, 3, 40), (40, 0, 40),
                                              (1000, 2, 700), (1000, 16, 700), (1000, 255, 700)])
def test_latent_attention_sees_its_window_and_nothing_else(tmp_path, dtype, window, far, query):
    """A key that stands out: just inside or just outside the query's window, at and off page borders, among the first
    tokens, hundreds of tokens back; with the query inside a prompt's portion, at the start of a portion, and decoded."""
    _window_case(tmp_path, dtype, window, far, query, (3, 24, 8, 16, 24))


@pytest.mark.parametrize("window,far,query", [(64, 64, 127), (64, 63, 127), (200, 220, 419), (200, 219, 419), (130, 0, 129),
                                              (130, 0, 130), (300, 1, 300), (300, 2, 300)])
def test_window_edges_with_cache_rows_of_64_on_the_tensor_cores(tmp_path, window, far, query):
    """Cache rows of 64 elements in bfloat16 take the tcgen05 kernel for a prompt's portions: the same edges there."""
    _window_case(tmp_path, "bfloat16", window, far, query, (4, 32, 16, 32, 48))


def test_a_reader_with_a_longer_window_still_finds_its_keys(tmp_path):
    """The layer that writes the rows has a window of 8, the layer that reads them one of 50: the cache must keep 50."""
    own, reader = _lat(2, 16, 8, 16, 24, 24, 8), _lat(2, 16, 8, 16, 24, 24, 50, kv_from=0)
    cfg = _cfg([_with(own, _dense(40)), _with(reader, None)])
    model_dir, w = _model_dir(tmp_path, "reader", cfg, seed=5)
    toks = U.make_requests(cfg["vocab"], [150], 2)["r0"]
    plain = {"r0": P.forward(cfg, w, toks).numpy()}
    short = {"r0": P.forward(dict(cfg, layers=[cfg["layers"][0], _with(_lat(2, 16, 8, 16, 24, 24, 8, kv_from=0), None)]), w, toks).numpy()}
    assert U.rel_err(short["r0"][-1], plain["r0"][-1]) > 1e-2
    for steps in (U.trace_tail_decode({"r0": toks}, tail=100), U.trace_portions({"r0": toks}, sizes=(17, 5, 2, 9, 2, 31, 3, 2))):
        sess = _session(model_dir, "float32", 128, block=8)      # fewer pages than tokens: pages behind the window go back
        U.compare(U.run_trace(sess, steps), plain, U.TOL["float32"], "longer reader window")
        sess.cache.check()


# ------------------------------------------------------------------ long decoding, generation --
def test_long_decoding_moves_every_window_over_decoded_tokens(tmp_path):
    cfg = CONFIGS["latent_only"]
    model_dir, w = _model_dir(tmp_path, "long", cfg, seed=4)
    toks = U.make_requests(cfg["vocab"], [230], 2)["r0"]
    plain = {"r0": P.forward(cfg, w, toks).numpy()}
    steps = U.trace_tail_decode({"r0": toks}, tail=220)
    sess = _session(model_dir, "float32", 64 + 32, block=8)          # less than the request: pages behind the windows go back
    U.compare(U.run_trace(sess, steps), plain, U.TOL["float32"], "long decoding")
    sess.cache.check()


def test_long_decoding_with_both_mixers(tmp_path):
    cfg = CONFIGS["both_mixers"]
    model_dir, w = _model_dir(tmp_path, "long2", cfg, seed=4)
    toks = U.make_requests(cfg["vocab"], [300], 3)["r0"]
    plain = {"r0": P.forward(cfg, w, toks).numpy()}
    for dtype in ("float32", "bfloat16"):
        sess = _session(model_dir, dtype, 320, block=16)
        _check(U.run_trace(sess, U.trace_tail_decode({"r0": toks}, tail=280)), plain, dtype, f"long decoding {dtype}")
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


def test_generation_in_bfloat16_with_graphs_stays_near_the_plain_model_s_best(tmp_path):
    from firefly_b200 import LLM
    cfg = CONFIGS["fast_paths"]
    model_dir, w = _model_dir(tmp_path, "genbf", cfg, seed=7)
    prompts = [v for v in U.make_requests(cfg["vocab"], [90, 5, 33], 12).values()]
    llm = LLM(model_dir, dtype="bfloat16", max_batch_size_limit=4, num_kv_blocks=64, max_prefill_chunk_size=64,
              eos_token_ids=[], use_cuda_graphs=True)
    outs = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    llm.engine.cache.check()
    for p, o in zip(prompts, outs):
        rows = P.forward(cfg, w, list(p) + o[:-1])
        for i, tok in enumerate(o):
            row = rows[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 5e-2 * float(row.abs().max()), (i, tok)


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
    cfg = CONFIGS["both_mixers"]
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
