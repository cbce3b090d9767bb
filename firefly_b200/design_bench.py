"""Throughput of a design beside the closest existing model at equal size: Kolorax beside Qwen3 dense, Pepolorn
beside Kolorax, Kefisun beside Qwen3 dense, Papusun beside Kefisun.

``python bench.py --design kolorax`` (or ``pepolorn``, ``kefisun``, ``papusun``) calls `main` here; the default workload of bench.py is untouched.
For each size, both models are built with seeded random weights at layer sizes that resemble a real
model's (same width, same number of layers, the dense feed-forward as wide as the experts a token
uses plus the shared one) and run through the engine's own loop (`Engine`: scheduler, captured decode
steps): a batch of prompts is prefilled, then decoded.  Times are wall clock around the engine loop with
a device synchronisation on both sides, after one untimed run of the same shape; prefill tokens per
second come from a run that generates one token, decode tokens per second from the extra time of a run
that generates N more.

The second part times the design's own kernels alone (CUDA events, inputs larger than L2 or an L2 flush
between iterations) against the bytes they must move or the operations they must do, next to the like
kernel of the dense model: the recurrence against the decode attention (both stream per-request state),
the grouped expert products against the dense feed-forward's product, layer norm against RMS norm.
"""
from __future__ import annotations

import json
import time
from types import SimpleNamespace

import torch

SIZES = {
    # width, layers, heads of the recurrent mixer (dim 64), attention heads, experts (top 4 of 16, 4 groups keep 2)
    "w1024": dict(width=1024, layers=8, ff=512, shared_ff=1024),
    "w2048": dict(width=2048, layers=8, ff=1024, shared_ff=2048),
}
VOCAB = 32768
TOP, EXPERTS, GROUPS, KEEP = 4, 16, 4, 2


def pepolorn_config(width: int, layers: int, ff: int, shared_ff: int = 0) -> dict:
    """Six state-space layers (inner size twice the width, heads of 64, a state of 128) around two layers of chunked
    attention beside linear attention (heads of 128); the first layer's feed-forward dense, the others routed."""
    moe = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP, "groups": {"count": GROUPS, "keep": KEEP}}, "expert": {"ff": ff}}
    ssm = {"type": "mamba2", "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8}}
    heads = width // 128
    par = {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5 * 4.0,
                 "mask": {"size": 8192}, "rot": {"base": 10000.0, "dims": 64,
                                                 "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
        "right": {"heads": heads, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** -(3 + 5 * h / max(1, heads - 1)) for h in range(heads)]},
        "left_scale": 1.0, "right_scale": 1.0}}
    out = []
    for i in range(layers):
        L = dict(par if i % 4 == 3 else ssm)
        L["mlp"] = {"kind": "dense", "ff": TOP * ff} if i == 0 else moe
        out.append(L)
    return {"architecture": "Pepolorn", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6}, "layers": out}


def kolorax_config(width: int, layers: int, ff: int, shared_ff: int) -> dict:
    heads = width // 64
    mlp = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP, "groups": {"count": GROUPS, "keep": KEEP}},
           "expert": {"ff": ff, "limit": 7.0}, "shared": {"ff": shared_ff, "limit": 7.0} if shared_ff else None}
    wkv = {"type": "wkv", "mixer": {"heads": heads, "dim": 64, "decay_rank": 64}, "mlp": mlp}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": heads, "dim": 64, "rot_dim": 64, "vdim": 64, "kv_rank": 192, "scale": 128 ** -0.5,
                     "rot": {"base": 10000.0, "dims": 64}}}
    return {"architecture": "Kolorax", "vocab": VOCAB, "width": width, "residual_mult": 0.5, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": [lat if i % 4 == 3 else wkv for i in range(layers)], "loop": None}


def qwen3_config(width: int, layers: int, ff: int, shared_ff: int, max_len: int) -> dict:
    heads = width // 128
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=width, intermediate_size=TOP * ff + shared_ff,
                num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=max(1, heads // 4), head_dim=128,
                vocab_size=VOCAB, max_position_embeddings=max_len, rms_norm_eps=1e-6, rope_theta=1e4,
                tie_word_embeddings=False)


def run_engine(raw_cfg: dict, dtype: str, batch: int, prompt: int, new_tokens: int) -> dict:
    from .engine.engine import Engine, EngineOptions
    from .engine.loading import random_model
    from .engine.request import GenerationRequest
    from .models import config_from_dict
    from .ops import kernels as K
    from .sampling import SamplingParams
    cfg = config_from_dict(raw_cfg)
    model = random_model(cfg, 0, dtype=dtype)
    pages = batch * (-(-(prompt + new_tokens + 8) // 16) + 2)
    eng = Engine(model, options=EngineOptions(max_batch_size_limit=batch, kv_block_size=16, num_kv_blocks=pages,
                                              max_prefill_chunk_size=prompt, max_num_batched_tokens=max(8192, prompt),
                                              eos_token_ids=[]))
    g = torch.Generator().manual_seed(7)
    serial = [0]

    def once(n_new: int):
        reqs = []
        for _ in range(batch):
            toks = torch.randint(0, VOCAB, (prompt,), generator=g).tolist()
            serial[0] += 1
            reqs.append(GenerationRequest(f"b{serial[0]}", toks, SamplingParams(max_tokens=n_new, ignore_eos=True)))
        torch.cuda.synchronize()
        l0, t0 = K.LAUNCHES, time.perf_counter()
        for r in reqs:
            eng.add_request(r)
        while eng.has_unfinished_requests():
            eng.step()
        torch.cuda.synchronize()
        return time.perf_counter() - t0, K.LAUNCHES - l0
    once(new_tokens + 1)                      # kernels built, step shapes captured
    t_pre = min(once(1)[0] for _ in range(2))
    t_all, launches = min(once(new_tokens + 1) for _ in range(2))
    eng.runner.check_status()
    params = sum(t.numel() for t in model.weight_arena.tensors().values())
    del eng, model
    torch.cuda.empty_cache()
    return {"prefill_tok_s": round(batch * prompt / t_pre), "decode_tok_s": round(batch * new_tokens / max(t_all - t_pre, 1e-9)),
            "prefill_ms": round(t_pre * 1e3, 2), "decode_ms_per_step": round((t_all - t_pre) / new_tokens * 1e3, 3),
            "parameters_m": round(params / 1e6, 1), "launches": launches}


def _time(fn, iters: int = 10, flush=None) -> float:
    """Median microseconds of fn() by CUDA events; ``flush`` (a buffer larger than L2) is rewritten between runs."""
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    return times[len(times) // 2]


def kernel_table(width: int, ff: int, batch: int, prompt: int, peaks: dict) -> list:
    """The design's kernels alone against their floors, and the dense model's like kernels at equal size."""
    from .ops import kernels as K
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rows = []

    def add(name, us, bytes_=0, flops=0, like=None):
        floor = max(bytes_ / hbm, flops / tflops) * 1e6
        rows.append({"kernel": name, "us": round(us, 1), "floor_us": round(floor, 2),
                     "of_floor": round(floor / us, 3) if us else None, "bound": "memory" if bytes_ / hbm >= flops / tflops else "tensor",
                     "like": like})
    heads, dim = width // 64, 64
    hd = heads * dim
    for label, n_seqs, q in (("prefill", batch, prompt), ("decode", batch * 8, 1)):
        T = n_seqs * q
        ctx = SimpleNamespace(cu_q=torch.arange(0, T + 1, q, dtype=torch.int32, device=dev), num_seqs=n_seqs,
                              state_slots=torch.arange(1, n_seqs + 1, dtype=torch.int32, device=dev),
                              seq_fresh=torch.zeros(n_seqs, dtype=torch.int32, device=dev))
        state = torch.zeros(n_seqs + 1, hd * dim + width, dtype=torch.float32, device=dev)
        rkvg = torch.randn(4, T, hd, device=dev).to(bf) * 0.1
        dlog = torch.randn(T, hd, device=dev)
        w0, u = torch.zeros(hd, device=dev), torch.randn(hd, device=dev)
        x, o = torch.randn(T, width, device=dev).to(bf), torch.empty(T, hd, device=dev)
        us = _time(lambda: K.wkv_scan(rkvg, dlog, w0, u, state, hd * dim, x, ctx, o, heads, dim), flush=flush)   # dim 64: its own size
        add(f"wkv_scan {label} ({n_seqs} x {q})", us, bytes_=3 * T * hd * 2 + 2 * T * hd * 4 + 2 * n_seqs * hd * dim * 4)
        # routed experts: gate|up with the activation, then down
        E, top = EXPERTS, TOP
        xa = torch.randn(T, width, device=dev).to(bf)
        z = torch.randn(T, E, device=dev)
        ids, wts = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, device=dev)
        K.moe_route(z, ids, wts, GROUPS, KEEP)
        n = T * top
        mt = K.moe_max_tiles(n, E, True)
        ints = [torch.empty(k, dtype=torch.int32, device=dev) for k in (E + 1, n, n, mt, mt, 1)]
        K.moe_plan(ids, E, *ints, True)
        plan = (ints[0], ints[3], ints[4], ints[5], mt)
        wg, wu = (torch.randn(E, ff, width, device=dev).to(bf) * 0.02 for _ in range(2))
        wd = torch.randn(E, width, ff, device=dev).to(bf) * 0.02
        act, outs = torch.empty(n, ff, dtype=bf, device=dev), torch.empty(n, width, device=dev)
        used = min(E, n)
        us = _time(lambda: K.moe_grouped(xa, ints[2], wg, wu, plan, act, 7.0, True), flush=flush)
        add(f"moe gate|up {label} ({n} rows)", us, bytes_=used * 2 * ff * width * 2 + n * (width + ff) * 2, flops=4 * n * ff * width)
        us = _time(lambda: K.moe_grouped(act, ints[2], wd, None, plan, outs, 0.0, True), flush=flush)
        add(f"moe down {label} ({n} rows)", us, bytes_=used * ff * width * 2 + n * (ff * 2 + width * 4), flops=2 * n * ff * width)
        # the dense model's like kernel: its gate|up product at the same number of operations
        inter = top * ff
        wdense = torch.randn(2 * inter, width, device=dev).to(bf) * 0.02
        yd = torch.empty(T, 2 * inter, dtype=bf, device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        if T <= K.GEMM_TC_MAX_TOKENS:
            us = _time(lambda: K.gemm_tc(xa, wdense, yd, K.EPI_BF16, 4, st), flush=flush)
        else:
            us = _time(lambda: K.linear(xa, wdense, yd), flush=flush)
        add(f"dense gate|up {label} ({T} tokens)", us, bytes_=2 * inter * width * 2 + T * (width + 2 * inter) * 2,
            flops=4 * T * inter * width, like="moe gate|up")
        # norms
        res, dl = torch.randn(T, width, device=dev), torch.randn(T, width, device=dev).to(bf)
        wn, bn, on = torch.ones(width, device=dev), torch.zeros(width, device=dev), torch.empty(T, width, dtype=bf, device=dev)
        if label == "prefill":
            us = _time(lambda: K.add_layer_norm(res, dl, wn, bn, 1e-6, on, None, 0.5), flush=flush)
            add(f"add_layer_norm ({T} rows)", us, bytes_=T * width * (4 + 4 + 2 + 2))
            us = _time(lambda: K.add_rms_norm(res, dl, wn, 1e-6, on), flush=flush)
            add(f"add_rms_norm ({T} rows)", us, bytes_=T * width * (4 + 4 + 2 + 2), like="add_layer_norm")
    return rows


def pepolorn_kernel_table(width: int, ff: int, batch: int, prompt: int, peaks: dict) -> list:
    """Pepolorn's own kernels alone against their floors, each beside the like kernel of Kolorax at equal size."""
    from .ops import kernels as K
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    hbm = peaks["hbm_gbs"] * 1e9
    rows = []

    def add(name, us, bytes_, like=None):
        floor = bytes_ / hbm * 1e6
        rows.append({"kernel": name, "us": round(us, 1), "floor_us": round(floor, 2), "of_floor": round(floor / us, 3) if us else None,
                     "bound": "memory", "like": like})
    heads, V, N, G, taps = 2 * width // 64, 64, 128, 8, 4
    inner, C = heads * V, heads * V + 2 * G * N
    P_ = 2 * inner + 2 * G * N + heads
    for label, n_seqs, q in (("prefill", batch, prompt), ("decode", batch * 8, 1)):
        T = n_seqs * q
        ctx = SimpleNamespace(cu_q=torch.arange(0, T + 1, q, dtype=torch.int32, device=dev), num_seqs=n_seqs,
                              token_seq=torch.arange(T, dtype=torch.int32, device=dev) // q,
                              positions=(torch.arange(T, dtype=torch.int32, device=dev) % q) + (0 if q > 1 else 2048),
                              state_slots=torch.arange(1, n_seqs + 1, dtype=torch.int32, device=dev),
                              seq_fresh=torch.zeros(n_seqs, dtype=torch.int32, device=dev),
                              status=torch.zeros(1, dtype=torch.int32, device=dev))
        sf = K.scan_state_floats(heads, N, V)
        state = torch.zeros(n_seqs + 1, sf + (taps - 1) * C, dtype=torch.float32, device=dev)
        proj = (torch.randn(T, P_, device=dev) * 0.5).to(bf)
        xbc = torch.empty(T, C, dtype=bf, device=dev)
        cw, cb = torch.randn(C, taps, device=dev) * 0.3, torch.zeros(C, device=dev)
        us = _time(lambda: K.causal_conv_silu(proj, inner, C, cw, cb, state, sf, ctx, xbc), flush=flush)
        add(f"causal_conv_silu {label} ({n_seqs} x {q})", us, T * C * 4 + 2 * n_seqs * (taps - 1) * C * 4, like="wkv_shift_mix")
        o = torch.empty(T, inner, device=dev)
        db, al, sk = (torch.zeros(heads, device=dev) for _ in range(3))
        us = _time(lambda: K.scalar_decay_scan((xbc, inner + G * N), (xbc, inner), (xbc, 0), state, 0, ctx, o, heads, N, V,
                                               heads_per_group=heads // G, step=(proj, 2 * inner + 2 * G * N), step_bias=db,
                                               a_log=al, skip=sk), flush=flush)
        add(f"scalar_decay_scan state-space {label} ({n_seqs} x {q})", us, T * C * 2 + T * inner * 4 + 2 * n_seqs * heads * N * V * 4, like="wkv_scan")
        y = torch.empty(T, inner, dtype=bf, device=dev)
        nw = torch.ones(inner, device=dev)
        us = _time(lambda: K.gated_rms_norm(o, (proj, 0), nw, 1e-6, y, 8, True), flush=flush)
        add(f"gated_rms_norm {label} ({T} rows)", us, T * inner * (4 + 2 + 2), like="wkv_out")
        # linear attention: heads of 128
        lh = width // 128
        lproj = (torch.randn(T, 4 * lh * 128, device=dev) * 0.5).to(bf)
        lstate = torch.zeros(n_seqs + 1, K.scan_state_floats(lh, 128, 128), dtype=torch.float32, device=dev)
        lo = torch.empty(T, lh * 128, device=dev)
        dec = torch.full((lh,), 0.99, device=dev)
        us = _time(lambda: K.scalar_decay_scan((lproj, 0), (lproj, lh * 128), (lproj, 2 * lh * 128), lstate, 0, ctx, lo, lh, 128, 128,
                                               silu_inputs=True, decay=dec), flush=flush)
        add(f"scalar_decay_scan linear attention {label} ({n_seqs} x {q})", us, T * 3 * lh * 128 * 2 + T * lh * 128 * 4 + 2 * n_seqs * lh * 128 * 128 * 4,
            like="wkv_scan")
        # the like kernels of Kolorax: its recurrence (heads of 64), the five shifted mixes, its output norm
        kh, kd = width // 64, 64
        hd = kh * kd
        kstate = torch.zeros(n_seqs + 1, hd * kd + width, dtype=torch.float32, device=dev)
        rkvg = torch.randn(4, T, hd, device=dev).to(bf) * 0.1
        dlog = torch.randn(T, hd, device=dev)
        w0, u = torch.zeros(hd, device=dev), torch.randn(hd, device=dev)
        x, ko = torch.randn(T, width, device=dev).to(bf), torch.empty(T, hd, device=dev)
        us = _time(lambda: K.wkv_scan(rkvg, dlog, w0, u, kstate, hd * kd, x, ctx, ko, kh, kd), flush=flush)
        add(f"wkv_scan {label} ({n_seqs} x {q})", us, 3 * T * hd * 2 + 2 * T * hd * 4 + 2 * n_seqs * hd * kd * 4)
        mu, mixes = torch.rand(5, width, device=dev), torch.empty(5, T, width, dtype=bf, device=dev)
        us = _time(lambda: K.wkv_shift_mix(x, mu, kstate, hd * kd, ctx, mixes), flush=flush)
        add(f"wkv_shift_mix {label} ({T} rows)", us, T * width * 2 * 6)
        ky = torch.empty(T, hd, dtype=bf, device=dev)
        us = _time(lambda: K.wkv_out(ko, rkvg[3], torch.ones(hd, device=dev), 1e-6, ky, kh, kd), flush=flush)
        add(f"wkv_out {label} ({T} rows)", us, T * hd * (4 + 2 + 2))
        # the norm on a part's output beside the layer norm with the residual add
        res, dl = torch.randn(T, width, device=dev), torch.randn(T, width, device=dev)
        wn, bn, on = torch.ones(width, device=dev), torch.zeros(width, device=dev), torch.empty(T, width, dtype=bf, device=dev)
        us = _time(lambda: K.norm_add(res, dl, wn, 1e-6, on), flush=flush)
        add(f"norm_add {label} ({T} rows)", us, T * width * (4 + 4 + 4 + 2), like="add_layer_norm")
        us = _time(lambda: K.add_layer_norm(res, dl.to(bf), wn, bn, 1e-6, on, None, 0.5), flush=flush)
        add(f"add_layer_norm {label} ({T} rows)", us, T * width * (4 + 4 + 2 + 2))
        # finishing the heads: rotation, unit norm, cache write
        ah, akv, d = width // 128, max(1, width // 512), 128
        qkv = torch.randn(T, (ah + 2 * akv) * d, device=dev).to(bf)
        pages = torch.zeros(T // 16 + n_seqs + 2, 2, akv, 16, d, dtype=bf, device=dev)
        per = -(-(q + 2048) // 16)
        table = (torch.arange(n_seqs * per, dtype=torch.int32, device=dev) % (pages.shape[0] - 1) + 1).view(n_seqs, per).contiguous()
        freq = torch.rand(32, dtype=torch.float64, device=dev)
        us = _time(lambda: K.rope_unit_norm_store(qkv, ah, akv, d, d, 1e-6, freq, 1.2, ctx, table, pages), flush=flush)
        add(f"rope_unit_norm_store {label} ({T} rows)", us, T * (ah + 2 * akv) * d * 2 * 2, like="qk_norm_rope_store")
    return rows


def main(args, peaks: dict) -> int:
    if args.design == "pepolorn":
        return pepolorn_main(args, peaks)
    if args.design == "kefisun":
        return kefisun_main(args, peaks)
    if args.design == "papusun":
        return papusun_main(args, peaks)
    out = {"design": "Kolorax", "beside": "Qwen3 dense at equal width, layers and feed-forward width per token",
           "dtype": args.dtype, "batch": args.batch, "prompt_len": args.prompt_len, "new_tokens": args.steps,
           "data": "synthetic token ids, seeded random weights", "peaks": peaks.get("source"), "sizes": {}}
    for name, size in SIZES.items():
        if args.design_sizes and name not in args.design_sizes.split(","):
            continue
        max_len = args.prompt_len + args.steps + 64
        ours = run_engine(kolorax_config(**size), args.dtype, args.batch, args.prompt_len, args.steps)
        dense = run_engine(qwen3_config(max_len=max_len, **size), args.dtype, args.batch, args.prompt_len, args.steps)
        out["sizes"][name] = {"shape": size, "kolorax": ours, "qwen3": dense,
                              "kernels": kernel_table(size["width"], size["ff"], args.batch, args.prompt_len, peaks)}
    print(json.dumps(out))
    return 0


def pepolorn_main(args, peaks: dict) -> int:
    out = {"design": "Pepolorn", "beside": "Kolorax at equal width, layers and experts (no shared expert)",
           "dtype": args.dtype, "batch": args.batch, "prompt_len": args.prompt_len, "new_tokens": args.steps,
           "data": "synthetic token ids, seeded random weights", "peaks": peaks.get("source"), "sizes": {}}
    for name, size in SIZES.items():
        if args.design_sizes and name not in args.design_sizes.split(","):
            continue
        shape = dict(size, shared_ff=0)
        ours = run_engine(pepolorn_config(**shape), args.dtype, args.batch, args.prompt_len, args.steps)
        beside = run_engine(kolorax_config(**shape), args.dtype, args.batch, args.prompt_len, args.steps)
        out["sizes"][name] = {"shape": shape, "pepolorn": ours, "kolorax": beside,
                              "kernels": pepolorn_kernel_table(size["width"], size["ff"], args.batch, args.prompt_len, peaks)}
    print(json.dumps(out))
    return 0


# --------------------------------------------------------------------------- #
# Kefisun beside Qwen3 dense
KEFISUN_WINDOW = 1024


def kefisun_config(width: int, layers: int, ff: int, shared_ff: int = 0) -> dict:
    """Attention layers (heads of 128, four query heads a kv head, a window of 1024 tokens, four taps, values blended
    with the first layer's) with every fourth layer a channel_delta mixer (heads of 128 x 128, two heads a q/k head)
    that has no feed-forward; the dense feed-forward as wide as the dense model's beside it."""
    heads = width // 128
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "conv": 4,
                                          "scale": 128 ** -0.5, "mask": {"size": KEFISUN_WINDOW}, "v_mix": True},
           "mlp": {"kind": "dense", "ff": TOP * ff + shared_ff, "limit": 7.0}}
    delta = {"type": "channel_delta", "mlp": None,
             "mixer": {"heads": heads, "kv_heads": max(1, heads // 2), "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64, "gate_rank": 64}}
    return {"architecture": "Kefisun", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "embedding": {"scale": float(width) ** 0.5}, "logit_scale": 0.5,
            "layers": [delta if i % 4 == 2 else att for i in range(layers)]}


def kefisun_kernel_table(width: int, batch: int, prompt: int, peaks: dict) -> list:
    """Kefisun's own kernels alone against their floors, each beside the like kernel of the models that were there."""
    from .ops import kernels as K
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rows = []

    def add(name, us, bytes_=0, flops=0, like=None):
        floor = max(bytes_ / hbm, flops / tflops) * 1e6
        rows.append({"kernel": name, "us": round(us, 1), "floor_us": round(floor, 2), "of_floor": round(floor / us, 3) if us else None,
                     "bound": "memory" if bytes_ / hbm >= flops / tflops else "tensor", "like": like})
    H, d, taps, window = width // 128, 128, 4, KEFISUN_WINDOW
    G = max(1, H // 4)
    C = (H + 2 * G) * d
    block = 16
    for label, n_seqs, q, ctx_len in (("prefill", batch, prompt, 0), ("decode", batch * 8, 1, prompt)):
        T = n_seqs * q
        per = -(-(q + ctx_len) // block)
        ctx = SimpleNamespace(cu_q=torch.arange(0, T + 1, q, dtype=torch.int32, device=dev), num_seqs=n_seqs,
                              token_seq=torch.arange(T, dtype=torch.int32, device=dev) // q,
                              positions=(torch.arange(T, dtype=torch.int32, device=dev) % q) + ctx_len,
                              state_slots=torch.arange(1, n_seqs + 1, dtype=torch.int32, device=dev),
                              seq_fresh=torch.zeros(n_seqs, dtype=torch.int32, device=dev),
                              status=torch.zeros(1, dtype=torch.int32, device=dev))
        ctx_lens = torch.full((n_seqs,), ctx_len, dtype=torch.int32, device=dev)
        pages = (torch.randn(n_seqs * per + 1, 2, G, block, d, device=dev) * 0.5).to(bf)
        table = (torch.arange(n_seqs * per, dtype=torch.int32, device=dev) + 1).view(n_seqs, per).contiguous()
        # the input filter: a convolution added to its 32-bit input
        xn = torch.randn(T, width, device=dev)
        fstate = torch.zeros(n_seqs + 1, (taps - 1) * width, dtype=torch.float32, device=dev)
        fw, fo = torch.randn(width, taps, device=dev) * 0.3, torch.empty(T, width, dtype=bf, device=dev)
        us = _time(lambda: K.causal_conv(xn, 0, width, fw, None, fstate, 0, ctx, fo, add_input=True), flush=flush)
        add(f"causal_conv filter {label} ({n_seqs} x {q})", us, T * width * (4 + 2) + 2 * n_seqs * (taps - 1) * width * 4, like="causal_conv_silu")
        # attention heads: convolution, norm over the projection, blend, cache write
        proj = (torch.randn(T, C + H * d, device=dev) * 0.5).to(bf)
        cstate = torch.zeros(n_seqs + 1, (taps - 1) * C, dtype=torch.float32, device=dev)
        cw = torch.randn(C, taps, device=dev) * 0.3
        cwt = cw.t().contiguous()
        qn, kn = torch.ones(H * d, device=dev), torch.ones(G * d, device=dev)
        qo = torch.empty(T, H * d, dtype=bf, device=dev)
        shared, f = torch.randn(T, G * d, device=dev), torch.full((1,), 0.3, device=dev)
        us = _time(lambda: K.conv_norm_store(proj, 0, cw, qn, kn, 1e-6, cstate, 0, ctx, table, pages, qo, H, G, d, d, d,
                                             mix=2, mix_factor=f, shared=shared, conv_w_t=cwt), flush=flush)
        add(f"conv_norm_store {label} ({T} rows)", us, T * C * 2 * 2 + T * G * d * 4, like="qk_norm_rope_store")
        us = _time(lambda: K.conv_state_update(proj, 0, C, taps, cstate, 0, ctx), flush=flush)
        add(f"conv_state_update {label} ({n_seqs} sequences)", us, n_seqs * (taps - 1) * C * (2 + 4))
        # the dense model's like kernel: q/k norm per head, rotation, cache write
        qkv = (torch.randn(T, C, device=dev) * 0.5).to(bf)
        cs = torch.randn(q + ctx_len + 1, d // 2, 2, device=dev)
        hn = torch.ones(d, device=dev)
        us = _time(lambda: K.qk_norm_rope_store(qkv, H, G, d, hn, hn, 1e-6, cs, d, ctx.positions, ctx.token_seq, table, pages, ctx.status),
                   flush=flush)
        add(f"qk_norm_rope_store {label} ({T} rows)", us, T * C * 2 * 2)
        # attention itself, with the bias by distance and without
        bias = (torch.rand(H, 1) * torch.log1p(torch.rand(H, 1) * torch.arange(window).view(1, -1))).float().to(dev).contiguous()
        att = torch.empty(T, H * d, dtype=bf, device=dev)
        keys = min(window, q + ctx_len)
        if q > 1:
            visible = sum(min(window, i + 1) for i in range(q)) * n_seqs
            flops = 4 * visible * H * d
            kv_bytes = T * (2 * H + 2 * G) * d * 2
            tiles = n_seqs * -(-(q * (H // G)) // 64)
            us = _time(lambda: K.attn_tiled(qo, H * d, pages, table, ctx.cu_q, ctx_lens, n_seqs, tiles, att, H, G, d, d ** -0.5, window,
                                            ctx.status, bias), flush=flush)
            add(f"attention mma.sync, window and bias {label}", us, kv_bytes, flops, like="attention mma.sync, window")
            us = _time(lambda: K.attn_tiled(qo, H * d, pages, table, ctx.cu_q, ctx_lens, n_seqs, tiles, att, H, G, d, d ** -0.5, window,
                                            ctx.status), flush=flush)
            add(f"attention mma.sync, window {label}", us, kv_bytes, flops)
            tiles = n_seqs * -(-(q * (H // G)) // 128)
            for name, bt in (("attention tcgen05, window and bias", bias), ("attention tcgen05, window", None)):
                try:
                    us = _time(lambda: K.attn_tc(qo, H * d, pages, table, ctx.cu_q, ctx_lens, n_seqs, tiles, att, H, G, d, d ** -0.5, window,
                                                 ctx.status, **({"dist_bias": bt} if bt is not None else {})), flush=flush)
                    add(f"{name} {label}", us, kv_bytes, flops, like=None if bt is None else "attention tcgen05, window")
                except TypeError:
                    pass
        else:
            ctx_lens1 = torch.full((n_seqs,), ctx_len, dtype=torch.int32, device=dev)
            splits = K.decode_splits(n_seqs, G, keys)
            part_o = torch.empty(n_seqs * H * splits * d, device=dev)
            part_ml = torch.empty(n_seqs * H * splits * 2, device=dev)
            kv_bytes = n_seqs * keys * 2 * G * d * 2 + T * 2 * H * d * 2
            for name, bt in (("attention decode, window and bias", bias), ("attention decode, window", None)):
                us = _time(lambda: K.attn_decode(qo, H * d, pages, table, ctx.cu_q, ctx_lens1, n_seqs, att, part_o, part_ml, H, G, d,
                                                 d ** -0.5, window, splits, ctx.status, bt), flush=flush)
                add(f"{name} ({n_seqs} x {keys} keys)", us, kv_bytes, like=None if bt is None else "attention decode, window")
        y = torch.empty(T, H * d, dtype=bf, device=dev)
        us = _time(lambda: K.head_gate(att, (proj, C), y, H, d, d), flush=flush)
        add(f"head_gate {label} ({T} rows)", us, T * H * d * 2 * 3, like="silu_mul")
        # feed-forward activation with biases and clamps beside the dense model's
        I = 3 * width
        gu, act, gb = (torch.randn(T, 2 * I, device=dev)).to(bf), torch.empty(T, I, dtype=bf, device=dev), torch.zeros(2 * I, device=dev)
        us = _time(lambda: K.glu_act(gu, act, "clamped_swish", gb, 7.0), flush=flush)
        add(f"glu_act clamped, biases {label} ({T} rows)", us, T * I * 2 * 3, like="silu_mul")
        us = _time(lambda: K.silu_mul(gu, act), flush=flush)
        add(f"silu_mul {label} ({T} rows)", us, T * I * 2 * 3)
        # the recurrent mixer: convolution with SiLU, the delta rule, head norm and gate; beside Kolorax's recurrence
        dh, dg, N, V = H, max(1, H // 2), 128, 128
        DC = 2 * dg * N + dh * V
        sf = K.delta_state_floats(dh, N, V)
        dstate = torch.zeros(n_seqs + 1, sf + (taps - 1) * DC, dtype=torch.float32, device=dev)
        dproj = (torch.randn(T, DC + dh, device=dev) * 0.5).to(bf)
        dqkv = torch.empty(T, DC, dtype=bf, device=dev)
        dcw = torch.randn(DC, taps, device=dev) * 0.3
        us = _time(lambda: K.causal_conv(dproj, 0, DC, dcw, None, dstate, sf, ctx, dqkv, silu=True), flush=flush)
        add(f"causal_conv with SiLU {label} ({n_seqs} x {q})", us, T * DC * 4 + 2 * n_seqs * (taps - 1) * DC * 4, like="causal_conv_silu")
        ag = torch.randn(T, dh * N + dh * V, device=dev)
        do = torch.empty(T, dh * V, device=dev)
        dtb, al = torch.zeros(dh * N, device=dev), torch.zeros(dh, device=dev)
        us = _time(lambda: K.delta_rule_scan((dqkv, 0), (dqkv, dg * N), (dqkv, 2 * dg * N), (dproj, DC), (ag, 0), dtb, al, dstate, 0, ctx, do,
                                             dh, N, V, heads_per_group=dh // dg, q_scale=N ** -0.5), flush=flush)
        add(f"delta_rule_scan {label} ({n_seqs} x {q})", us, T * (DC * 2 + dh * N * 4 + dh * V * 4) + 2 * n_seqs * dh * N * V * 4, like="wkv_scan")
        dy = torch.empty(T, dh * V, dtype=bf, device=dev)
        nw = torch.ones(V, device=dev)
        us = _time(lambda: K.head_norm_gate(do, (ag, dh * N), nw, 1e-6, dy, dh, V), flush=flush)
        add(f"head_norm_gate {label} ({T} rows)", us, T * dh * V * (4 + 4 + 2), like="wkv_out")
        kh, kd = width // 64, 64
        hd = kh * kd
        kstate = torch.zeros(n_seqs + 1, hd * kd + width, dtype=torch.float32, device=dev)
        rkvg = torch.randn(4, T, hd, device=dev).to(bf) * 0.1
        dlog = torch.randn(T, hd, device=dev)
        w0, u = torch.zeros(hd, device=dev), torch.randn(hd, device=dev)
        x, ko = torch.randn(T, width, device=dev).to(bf), torch.empty(T, hd, device=dev)
        us = _time(lambda: K.wkv_scan(rkvg, dlog, w0, u, kstate, hd * kd, x, ctx, ko, kh, kd), flush=flush)
        add(f"wkv_scan {label} ({n_seqs} x {q})", us, 3 * T * hd * 2 + 2 * T * hd * 4 + 2 * n_seqs * hd * kd * 4)
        ky = torch.empty(T, hd, dtype=bf, device=dev)
        us = _time(lambda: K.wkv_out(ko, rkvg[3], torch.ones(hd, device=dev), 1e-6, ky, kh, kd), flush=flush)
        add(f"wkv_out {label} ({T} rows)", us, T * hd * (4 + 2 + 2))
        # the recurrence of the state-space design at the same key and value size
        lproj = (torch.randn(T, 3 * dh * 128, device=dev) * 0.5).to(bf)
        lstate = torch.zeros(n_seqs + 1, K.scan_state_floats(dh, 128, 128), dtype=torch.float32, device=dev)
        lo = torch.empty(T, dh * 128, device=dev)
        dec = torch.full((dh,), 0.99, device=dev)
        us = _time(lambda: K.scalar_decay_scan((lproj, 0), (lproj, dh * 128), (lproj, 2 * dh * 128), lstate, 0, ctx, lo, dh, 128, 128,
                                               silu_inputs=True, decay=dec), flush=flush)
        add(f"scalar_decay_scan 128 x 128 {label} ({n_seqs} x {q})", us, T * 3 * dh * 128 * 2 + T * dh * 128 * 4 + 2 * n_seqs * dh * 128 * 128 * 4)
    return rows


def kefisun_main(args, peaks: dict) -> int:
    out = {"design": "Kefisun", "beside": "Qwen3 dense at equal width, layers and feed-forward width (its attention sees every key, "
                                          f"Kefisun's the last {KEFISUN_WINDOW}; two of Kefisun's eight layers are recurrent and have no feed-forward)",
           "dtype": args.dtype, "batch": args.batch, "prompt_len": args.prompt_len, "new_tokens": args.steps,
           "data": "synthetic token ids, seeded random weights", "peaks": peaks.get("source"), "sizes": {}}
    for name, size in SIZES.items():
        if args.design_sizes and name not in args.design_sizes.split(","):
            continue
        max_len = args.prompt_len + args.steps + 64
        ours = run_engine(kefisun_config(**size), args.dtype, args.batch, args.prompt_len, args.steps)
        dense = run_engine(qwen3_config(max_len=max_len, **size), args.dtype, args.batch, args.prompt_len, args.steps)
        out["sizes"][name] = {"shape": size, "kefisun": ours, "qwen3": dense,
                              "kernels": kefisun_kernel_table(size["width"], args.batch, args.prompt_len, peaks)}
        print(json.dumps({"partial": name, **out["sizes"][name]}), flush=True)
    print(json.dumps(out))
    return 0


# --------------------------------------------------------------------------- #
# Papusun beside Kefisun
PAPUSUN_WINDOW = 1024


def papusun_config(width: int, layers: int, ff: int, shared_ff: int = 0) -> dict:
    """Latent-attention layers (heads of 128 + 64 rotated, a latent of 192 for keys and values and of half the width for the
    queries, a window of 1024 tokens; every second one of them reads the rows of the one in front) with every fourth
    layer two mixers side by side (attention over every key with heads of 128, four query heads a kv head, half of
    the head rotated, capped scores; a delta rule with heads of 128 x 128, two heads a q/k head); the dense
    feed-forward as wide as the model's beside it; a side input of 256 numbers a token and layer."""
    heads = width // 128
    lat = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 192, "q_rank": max(256, width // 2),
           "scale": 192 ** -0.5, "mask": {"size": PAPUSUN_WINDOW}, "rot": {"base": 10000.0, "dims": 64}}
    par = {"left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                    "softcap": 50.0, "rot": {"base": 500000.0, "dims": 64,
                                             "scaling": {"factor": 16.0, "low": 1.0, "high": 8.0, "original": 8192}}},
           "right": {"heads": heads, "kv_heads": max(1, heads // 2), "dim": 128, "vdim": 128, "conv": 4},
           "left_scale": 1.0, "right_scale": 1.0}
    mlp = {"kind": "dense", "ff": TOP * ff + shared_ff}
    out, last_writer = [], None
    for i in range(layers):
        if i % 4 == 2:
            out.append({"type": "parallel", "mixer": par, "mlp": mlp})
            continue
        mx = dict(lat)
        if last_writer is not None and i % 4 in (1, 3):
            mx["kv_from"] = last_writer
        else:
            last_writer = i
        out.append({"type": "latent_attention", "mixer": mx, "mlp": mlp})
    return {"architecture": "Papusun", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
            "token_side": {"dim": 256}, "layers": out}


def papusun_kernel_table(width: int, batch: int, prompt: int, peaks: dict) -> list:
    """The kernels that Papusun added or changed, alone against their floors, each beside the like kernel (or the
    same kernel without the new option) of the models that were there."""
    from .ops import kernels as K
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rows = []

    def add(name, us, bytes_=0, flops=0, like=None):
        floor = max(bytes_ / hbm, flops / tflops) * 1e6
        rows.append({"kernel": name, "us": round(us, 1), "floor_us": round(floor, 2), "of_floor": round(floor / us, 3) if us else None,
                     "bound": "memory" if bytes_ / hbm >= flops / tflops else "tensor", "like": like})
    H, d, block = width // 128, 128, 16
    G = max(1, H // 4)
    C = (H + 2 * G) * d
    rank, rot, window = 192, 64, PAPUSUN_WINDOW
    ld = rank + rot
    for label, n_seqs, q, ctx_len in (("prefill", batch, prompt, 0), ("decode", batch * 8, 1, prompt)):
        T = n_seqs * q
        per = -(-(q + ctx_len) // block)
        ctx = SimpleNamespace(cu_q=torch.arange(0, T + 1, q, dtype=torch.int32, device=dev), num_seqs=n_seqs,
                              token_seq=torch.arange(T, dtype=torch.int32, device=dev) // q,
                              positions=(torch.arange(T, dtype=torch.int32, device=dev) % q) + ctx_len,
                              state_slots=torch.arange(1, n_seqs + 1, dtype=torch.int32, device=dev),
                              seq_fresh=torch.zeros(n_seqs, dtype=torch.int32, device=dev),
                              status=torch.zeros(1, dtype=torch.int32, device=dev))
        ctx_lens = torch.full((n_seqs,), ctx_len, dtype=torch.int32, device=dev)
        table = (torch.arange(n_seqs * per, dtype=torch.int32, device=dev) + 1).view(n_seqs, per).contiguous()
        # -- the attention over every key: heads finished (biases, interleaved rotation, cache write), capped scores
        pages = (torch.randn(n_seqs * per + 1, 2, G, block, d, device=dev) * 0.5).to(bf)
        qkv = (torch.randn(T, C, device=dev) * 0.5).to(bf)
        freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -torch.arange(32, dtype=torch.float64) / 32).to(dev)
        bias = torch.randn(C, device=dev) * 0.1
        us = _time(lambda: K.rope_unit_norm_store(qkv, H, G, d, d, 1e-6, freq, 1.0, ctx, table, pages, interleaved=True,
                                                  normalize=False, bias=bias), flush=flush)
        add(f"head finish: biases, interleaved rotation, cache write {label} ({T} rows)", us, T * C * 2 * 2,
            like="head finish: rotation by halves, unit norm, cache write")
        us = _time(lambda: K.rope_unit_norm_store(qkv, H, G, d, d, 1e-6, freq, 1.0, ctx, table, pages), flush=flush)
        add(f"head finish: rotation by halves, unit norm, cache write {label} ({T} rows)", us, T * C * 2 * 2)
        att = torch.empty(T, H * d, dtype=bf, device=dev)
        if q > 1:
            flops = 4 * n_seqs * (q * (q + 1) // 2) * H * d
            kv_bytes = T * (2 * H + 2 * G) * d * 2
            tiles = n_seqs * -(-(q * (H // G)) // 128)
            for name, cap in (("attention tcgen05, every key, capped scores", 50.0), ("attention tcgen05, every key", 0.0)):
                us = _time(lambda: K.attn_tc(qkv, C, pages, table, ctx.cu_q, ctx_lens, n_seqs, tiles, att, H, G, d, d ** -0.5, 0,
                                             ctx.status, softcap=cap), flush=flush)
                add(f"{name} {label}", us, kv_bytes, flops, like="attention tcgen05, every key" if cap else None)
        else:
            keys = ctx_len + 1
            splits = K.decode_splits(n_seqs, G, keys)
            part_o = torch.empty(n_seqs * H * splits * d, device=dev)
            part_ml = torch.empty(n_seqs * H * splits * 2, device=dev)
            kv_bytes = n_seqs * keys * 2 * G * d * 2 + T * 2 * H * d * 2
            for name, cap in (("attention decode, every key, capped scores", 50.0), ("attention decode, every key", 0.0)):
                us = _time(lambda: K.attn_decode(qkv, C, pages, table, ctx.cu_q, ctx_lens, n_seqs, att, part_o, part_ml, H, G, d,
                                                 d ** -0.5, 0, splits, ctx.status, None, cap), flush=flush)
                add(f"{name} ({n_seqs} x {keys} keys)", us, kv_bytes, like="attention decode, every key" if cap else None)
        # -- the delta rule with one decay a head beside the one with a decay a key channel
        dh, dg, N, V, taps = H, max(1, H // 2), 128, 128, 4
        DC = 2 * dg * N + dh * V
        sf = K.delta_state_floats(dh, N, V)
        dstate = torch.zeros(n_seqs + 1, sf + (taps - 1) * DC, dtype=torch.float32, device=dev)
        dproj = (torch.randn(T, DC + dh, device=dev) * 0.5).to(bf)
        dqkv = (torch.randn(T, DC, device=dev) * 0.5).to(bf)
        do = torch.empty(T, dh * V, device=dev)
        io = T * (DC * 2 + dh * V * 4) + 2 * n_seqs * dh * N * V * 4
        for name, per_head in (("delta rule, a decay a head", True), ("delta rule, a decay a key channel", False)):
            rows_a = dh if per_head else dh * N
            ag = torch.randn(T, rows_a + dh * V, device=dev)
            dtb, al = torch.zeros(rows_a, device=dev), torch.zeros(dh, device=dev)
            us = _time(lambda: K.delta_rule_scan((dqkv, 0), (dqkv, dg * N), (dqkv, 2 * dg * N), (dproj, DC), (ag, 0), dtb, al, dstate, 0, ctx,
                                                 do, dh, N, V, heads_per_group=dh // dg, q_scale=N ** -0.5, decay_per_head=per_head),
                       flush=flush)
            add(f"{name} {label} ({n_seqs} x {q})", us, io + T * rows_a * 4, like=None if not per_head else "delta rule, a decay a key channel")
            dy = torch.empty(T, dh * V, dtype=bf, device=dev)
            nw = torch.ones(V, device=dev)
            act = "silu" if per_head else "sigmoid"
            us = _time(lambda: K.head_norm_gate(do, (ag, rows_a), nw, 1e-6, dy, dh, V, act), flush=flush)
            add(f"head norm and {act} gate {label} ({T} rows)", us, T * dh * V * (4 + 4 + 2),
                like="head norm and sigmoid gate" if per_head else None)
        # -- latent attention: queries finished and rows written, attention inside a window over one-plane pages, head gates
        lpages = (torch.randn(n_seqs * per + 1, 1, 1, block, ld, device=dev) * 0.5).to(bf)
        lq = (torch.randn(T, H * (d + rot), device=dev) * 0.5).to(bf)
        dkv = (torch.randn(T, ld, device=dev) * 0.5).to(bf)
        q_abs = (torch.randn(H, T, rank, device=dev) * 0.5).to(bf)
        q_full = torch.empty(T, H * ld, dtype=bf, device=dev)
        cn = torch.ones(rank, device=dev)
        for name, inter in (("latent rows and queries, interleaved rotation", True), ("latent rows and queries, rotation by halves", False)):
            us = _time(lambda: K.latent_finish(lq, dkv, q_abs, cn, 1e-6, freq, ctx, table, lpages, q_full, H, d, rot, rank, rot, inter),
                       flush=flush)
            add(f"{name} {label} ({T} rows)", us, T * (H * (d + rot) + ld + 2 * H * rank + H * rot + ld) * 2,
                like=None if not inter else "latent rows and queries, rotation by halves")
        latt = torch.empty(T, H * ld, dtype=bf, device=dev)
        for name, win in (("latent attention inside a window", window), ("latent attention over every key", 0)):
            keys_seen = sum(min(win or (1 << 30), i + 1 + ctx_len) for i in range(q)) * n_seqs
            step_ctx = SimpleNamespace(**vars(ctx), ctx_lens=ctx_lens, q_lens=[q] * n_seqs, ctx_lens_host=[ctx_len] * n_seqs,
                                       num_decode_seqs=n_seqs if q == 1 else 0, max_kv_len=q + ctx_len, ranges_by_length=False,
                                       workspace=_Scratch(dev), captured=False, memo={}, key_share_level=0)
            us = _time(lambda: K.paged_attention(q_full, H * ld, lpages, table, step_ctx, latt, H, 1, ld, 192 ** -0.5, win), flush=flush)
            kv_b = (n_seqs * min(win or (1 << 30), q + ctx_len) * ld * 2 if q == 1 else T * ld * 2) + T * 2 * H * ld * 2
            add(f"{name} {label}", us, kv_b, 2 * keys_seen * H * (ld + rank), like=None if not win else "latent attention over every key")
        val = (torch.randn(H, T, d, device=dev) * 0.5).to(bf)
        y = torch.empty(T, H * d, dtype=bf, device=dev)
        for name, per_head in (("latent head gates, one a head", True), ("latent head gates, one an element", False)):
            g = (torch.randn(T, H if per_head else H * d, device=dev)).to(bf)
            us = _time(lambda: K.latent_gate(val, g, y, H, d, per_head), flush=flush)
            add(f"{name} {label} ({T} rows)", us, T * H * d * 2 * 2 + g.numel() * 2, like=None if not per_head else "latent head gates, one an element")
        # -- the token's side input: gated table rows, and the norm that adds the result to the stream
        side = 256
        tbl = (torch.randn(VOCAB, 8 * side, device=dev) * 0.5).to(bf)
        ids = torch.randint(0, VOCAB, (T,), dtype=torch.int32, device=dev)
        gate, gout = (torch.randn(T, side, device=dev)).to(bf), torch.empty(T, side, dtype=bf, device=dev)
        us = _time(lambda: K.act_mul_table_rows(gate, ids, tbl, 3 * side, gout, "gelu_tanh", ctx.status), flush=flush)
        add(f"side input: GELU gate times table rows {label} ({T} rows)", us, T * side * 2 * 3, like="silu_mul")
        gu, act_o = (torch.randn(T, 2 * side, device=dev)).to(bf), torch.empty(T, side, dtype=bf, device=dev)
        us = _time(lambda: K.silu_mul(gu, act_o), flush=flush)
        add(f"silu_mul {label} ({T} rows of {side})", us, T * side * 2 * 3)
        res, yy, nw2 = torch.randn(T, width, device=dev), torch.randn(T, width, device=dev), torch.ones(width, device=dev)
        us = _time(lambda: K.norm_add(res, yy, nw2, 1e-6), flush=flush)
        add(f"side input: RMS norm added to the stream {label} ({T} rows)", us, T * width * 4 * 3, like="layer norm with the residual add")
        out_n, lw = torch.empty(T, width, dtype=bf, device=dev), torch.ones(width, device=dev)
        us = _time(lambda: K.add_layer_norm(res, yy, lw, None, 1e-6, out_n, None, 1.0), flush=flush)
        add(f"layer norm with the residual add {label} ({T} rows)", us, T * width * (4 * 3 + 2))
    return rows


class _Scratch:
    """Named scratch buffers for a kernel timed alone (the engine's workspace in small)."""

    def __init__(self, device):
        self.device, self._bufs = device, {}

    def get(self, tag, shape, dtype):
        n = 1
        for s_ in shape:
            n *= int(s_)
        buf = self._bufs.get((tag, dtype))
        if buf is None or buf.numel() < n:
            buf = self._bufs[(tag, dtype)] = torch.empty(max(n, 1), dtype=dtype, device=self.device)
        return buf[:n].view(*shape)


def papusun_main(args, peaks: dict) -> int:
    out = {"design": "Papusun", "beside": "Kefisun at equal width, layers and feed-forward width (six of Papusun's eight layers are latent "
                                          f"attention inside a window of {PAPUSUN_WINDOW}, two are attention over every key beside a delta rule; "
                                          "two of Kefisun's eight layers are recurrent and have no feed-forward)",
           "dtype": args.dtype, "batch": args.batch, "prompt_len": args.prompt_len, "new_tokens": args.steps,
           "data": "synthetic token ids, seeded random weights", "peaks": peaks.get("source"), "sizes": {}}
    for name, size in SIZES.items():
        if args.design_sizes and name not in args.design_sizes.split(","):
            continue
        ours = run_engine(papusun_config(**size), args.dtype, args.batch, args.prompt_len, args.steps)
        beside = run_engine(kefisun_config(**size), args.dtype, args.batch, args.prompt_len, args.steps)
        out["sizes"][name] = {"shape": size, "papusun": ours, "kefisun": beside,
                              "kernels": papusun_kernel_table(size["width"], args.batch, args.prompt_len, peaks)}
        print(json.dumps({"partial": name, **out["sizes"][name]}), flush=True)
    print(json.dumps(out))
    return 0
