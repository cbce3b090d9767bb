"""Python faces of the CUDA kernels in ``csrc/``.

Every function takes CUDA tensors, launches on torch's current stream (so the
calls can be captured into a CUDA graph) and writes into buffers the caller
provides; nothing is allocated here.  There is no CPU or library fallback: a
tensor that is not on a CUDA device, or a kernel that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_size_t, c_void_p
from typing import Optional

import torch

from .build import compile_many, load_module

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream's handle.  Asked for at every launch: the raw getter costs well under a
    microsecond where ``torch.cuda.current_stream()`` builds an object each time (15 us)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {t.dtype}") from None


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None:
            if not t.is_cuda:
                raise KernelError("firefly_b200 kernels run on a CUDA device only; got a "
                                  f"{t.device} tensor (there is no CPU implementation)")
            if not t.is_contiguous():
                raise KernelError("kernel operand must be contiguous")


LAUNCHES = 0   # launches of this package's own kernels (library products are not counted)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code == -1:
        raise KernelError(f"{what}: bad argument")
    if code == -2:
        raise KernelError(f"{what}: size not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code}")


_MODULES = {
    "elementwise": ("elementwise.cu", None),
    "qk_rope_store": ("qk_rope_store.cu", None),
    "attention_simt": ("attention_simt.cu", None),
    "sampling": ("sampling.cu", None),
    "gemm_tcgen05": ("gemm_tcgen05.cu", None),
    "gemm_pair": ("gemm_pair.cu", None),
    "weights": ("weights.cu", None),
    "layer_norm": ("layer_norm.cu", None),
    "wkv": ("wkv.cu", None),
    "latent_attention": ("latent_attention.cu", None),
    "moe": ("moe.cu", None),
    "ssm": ("ssm.cu", None),
    "head_finish": ("head_finish.cu", None),
    "conv_attention": ("conv_attention.cu", None),
    "delta_rule": ("delta_rule.cu", None),
}


USE_PDL = True      # programmatic dependent launch: a kernel's prologue overlaps its predecessor's tail
_pdl_state = {}     # id(library) -> flag it was last given


def _configured(lib: ctypes.CDLL) -> ctypes.CDLL:
    if _pdl_state.get(id(lib)) != USE_PDL:
        lib.ff_set_pdl(c_int(1 if USE_PDL else 0))
        _pdl_state[id(lib)] = USE_PDL
    return lib


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch on or off for all kernels of this package."""
    global USE_PDL
    USE_PDL = bool(on)


def _lib(name: str) -> ctypes.CDLL:
    src, defs = _MODULES[name]
    return _configured(load_module(src, defs))


DEFAULT_HEAD_DIMS = (128,)


def build_all(head_dims=DEFAULT_HEAD_DIMS) -> None:
    """Compile every module (used by the build check; needs no GPU).  The
    tensor-core attention is compiled per head size; others are built when a
    model with that head size is first run."""
    mods = list(_MODULES.values()) + [("attention_mma.cu", {"FF_HEAD_DIM": int(d)}) for d in head_dims] + \
        [("attention_tc.cu", {"FF_HEAD_DIM": int(d)}) for d in head_dims if int(d) % 64 == 0]
    compile_many(mods)


# --------------------------------------------------------------------------- #
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
              scale: float = 1.0) -> None:
    """out[t,:] = float(table[ids[t],:]) * scale; ids int32 [T], out float32 [T,H]."""
    _need_cuda(ids, table, out, status)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32
    T, H = out.shape
    V = table.shape[0]
    assert table.shape[1] == H and ids.numel() == T
    _check(_lib("elementwise").ff_embedding(_p(ids), _p(table), c_int(_dt(table)), _p(out), c_int(T),
                                           c_int(H), c_int(V), c_float(scale), _p(status), _stream()), "embedding")


def scatter_int(buf: torch.Tensor, updates: torch.Tensor, cap: int) -> None:
    """buf[updates[1 + 2i]] = updates[2 + 2i] for i < min(updates[0], cap); all int32."""
    _need_cuda(buf, updates)
    assert buf.dtype == torch.int32 and updates.dtype == torch.int32 and updates.numel() >= 1 + 2 * cap
    _check(_lib("elementwise").ff_scatter_int(_p(buf), _p(updates), c_int(cap), c_int(buf.numel()), _stream()),
           "scatter_int")


def add_rms_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                 eps: float, out: torch.Tensor, row_idx: Optional[torch.Tensor] = None) -> None:
    """residual (+= delta), out = rms_norm(residual) * weight.

    residual float32 [T,H], updated in place when ``delta`` is given and
    ``row_idx`` is not.  With ``row_idx`` (int32 [n]) only those rows are
    normalised, into ``out`` [n,H], and the residual is left as it is.
    """
    _need_cuda(residual, delta, weight, out, row_idx)
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32
    H = residual.shape[-1]
    rows = out.shape[0]
    assert out.shape[-1] == H and weight.numel() == H
    if row_idx is None:
        assert rows == residual.shape[0]
    else:
        assert row_idx.dtype == torch.int32 and row_idx.numel() == rows
    if delta is not None:
        assert delta.shape == residual.shape
    _check(_lib("elementwise").ff_add_rms_norm(
        _p(residual), _p(delta), c_int(_dt(delta) if delta is not None else _dt(out)), _p(row_idx),
        _p(weight), c_float(eps), _p(out), c_int(_dt(out)), c_int(rows), c_int(H),
        c_int(1 if row_idx is None else 0), _stream()), "add_rms_norm")


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    _need_cuda(residual, delta)
    assert residual.dtype == torch.float32 and residual.shape == delta.shape
    _check(_lib("elementwise").ff_residual_add(_p(residual), _p(delta), c_int(_dt(delta)),
                                              c_size_t(residual.numel()), _stream()), "residual_add")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out[t,i] = silu(gate) * up, gate = gate_up[t,i], up = gate_up[t,I+i]; with
    ``interleaved`` the columns hold gate and up in alternating groups of 16."""
    _need_cuda(gate_up, out)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype == out.dtype
    _check(_lib("elementwise").ff_silu_mul(_p(gate_up), _p(out), c_int(_dt(out)), c_int(T), c_int(I),
                                          c_int(1 if interleaved else 0), _stream()), "silu_mul")


def cast(src: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(src, out)
    assert src.numel() == out.numel()
    _check(_lib("elementwise").ff_cast(_p(src), c_int(_dt(src)), _p(out), c_int(_dt(out)),
                                      c_size_t(src.numel()), _stream()), "cast")


def qk_norm_rope_store(qkv: torch.Tensor, nq: int, nkv: int, d: int, q_norm_w, k_norm_w, eps: float,
                       cos_sin: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
                       token_seq: torch.Tensor, block_table: Optional[torch.Tensor],
                       cache: Optional[torch.Tensor], status: torch.Tensor) -> None:
    """Per-head RMSNorm of q and k, rotation, and the write of k, v into the
    paged cache ``[blocks, 2, nkv, block_size, d]``; q is rewritten in place in
    ``qkv`` [T, (nq+2nkv)*d].  ``nkv == 0``: q only, no cache write."""
    _need_cuda(qkv, q_norm_w, k_norm_w, cos_sin, positions, token_seq, block_table, cache, status)
    T, width = qkv.shape
    if nkv:
        assert cache is not None and block_table is not None and cache.dtype == qkv.dtype
        num_blocks, two, ckv, block_size, cd = cache.shape
        assert two == 2 and ckv == nkv and cd == d
        max_blocks = block_table.shape[1]
    else:
        num_blocks = block_size = max_blocks = 1
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.shape[1] * cos_sin.shape[2] == rotary_dim
    _check(_lib("qk_rope_store").ff_qk_norm_rope_store(
        _p(qkv), c_int(_dt(qkv)), c_int(width), c_int(T), c_int(nq), c_int(nkv), c_int(d),
        _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(cos_sin), c_int(rotary_dim), c_int(max_pos),
        _p(positions), _p(token_seq), _p(block_table), c_int(max_blocks), c_int(block_size),
        c_int(num_blocks), _p(cache), _p(status), _stream()), "qk_norm_rope_store")


def _check_dist_bias(dist_bias: Optional[torch.Tensor], nq: int, window: int) -> None:
    """A table of biases by distance covers a window: one row a query head, one entry per distance the window
    lets through."""
    if dist_bias is None:
        return
    if dist_bias.dtype != torch.float32 or dist_bias.dim() != 2 or dist_bias.shape[0] != nq or not dist_bias.is_contiguous():
        raise KernelError("attention: the bias by distance is a contiguous float32 table [query heads, distances]")
    if window <= 0 or dist_bias.shape[1] < window:
        raise KernelError("attention: a bias by distance needs a window no longer than its table")


def paged_attention_simt(q: torch.Tensor, q_stride: int, cache: torch.Tensor, block_table: torch.Tensor,
                         token_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                         nq: int, nkv: int, d: int, scale: float, window: int,
                         status: torch.Tensor, dist_bias: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Attention of every query token over its sequence's cached keys 0..pos
    (or the last ``window`` of them; 0 = all).  ``q`` is read with row stride
    ``q_stride`` elements (it may be the head of a wider qkv buffer).  ``dist_bias`` float32 [nq, L]:
    entry (h, i - j) is taken off the score of query position i and key position j.  ``softcap`` c > 0: the scaled score
    s becomes c tanh(s / c) (before the bias)."""
    _need_cuda(cache, block_table, token_seq, positions, out, status, dist_bias)
    _check_dist_bias(dist_bias, nq, window)
    if not q.is_cuda:
        raise KernelError("firefly_b200 kernels run on a CUDA device only")
    T = out.shape[0]
    num_blocks, planes, ckv, block_size, cd = cache.shape
    assert ckv == nkv and cd == d and cache.dtype == q.dtype == out.dtype
    lib = _lib("attention_simt") if planes == 2 else _configured(load_module("attention_simt.cu", _planes_defs({}, planes)))
    _check(lib.ff_paged_attention_simt(
        _p(q), c_int(_dt(q)), c_int(q_stride), _p(cache), _p(block_table), c_int(block_table.shape[1]),
        _p(token_seq), _p(positions), _p(out), c_int(out.shape[1]), c_int(T), c_int(nq), c_int(nkv),
        c_int(d), c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), _p(dist_bias),
        c_int(dist_bias.shape[1] if dist_bias is not None else 0), c_float(softcap), _p(status), _stream()), "paged_attention_simt")


_sample_scratch = {}


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           seeds: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None) -> None:
    """out[r] = arg-max of logits[r] (lowest index on ties), or, where
    temperature[r] > 0, a draw from softmax(logits[r] / temperature[r]) with the
    random numbers of (seeds[r], counters[r]).

    The one wrapper that keeps memory of its own: the partial results of rows split over several
    blocks live in a scratch pair per device that grows when more rows come.  It never grows while
    the stream is being captured (an error then: the run before the capture sizes it)."""
    global LAUNCHES
    _need_cuda(logits, out, temperature, seeds, counters)
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and logits.dim() == 2
    rows, V = logits.shape
    if temperature is not None:
        assert temperature.dtype == torch.float32 and seeds.dtype == torch.int64 \
            and counters.dtype == torch.int64
    # a row is split over several blocks so that few rows still fill the GPU
    chunks = max(1, min(64, _sm_target_ctas() // 2 // max(rows, 1), V // 2048))
    pv = pi = None
    if chunks > 1:
        key = logits.device
        buf = _sample_scratch.get(key)
        if buf is None or buf[0].numel() < rows * chunks:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("sample: its scratch memory would have to grow while a CUDA graph is being "
                                  "captured; run the same step once before the capture")
            n = max(rows * chunks, 4096)
            buf = (torch.empty(n, dtype=torch.float32, device=key), torch.empty(n, dtype=torch.int32, device=key))
            _sample_scratch[key] = buf
        pv, pi = buf
    _check(_lib("sampling").ff_sample(_p(logits), c_int(rows), c_int(V), c_size_t(logits.stride(0)),
                                     _p(temperature), _p(seeds), _p(counters), _p(out), c_int(chunks),
                                     _p(pv), _p(pi), _stream()), "sample")
    if chunks > 1:
        LAUNCHES += 1


# --------------------------------------------------------------------------- #
# matrix products: a library routine (cuBLAS through torch), as the reference
# uses a library (CUTLASS, src/kernels/linear.cu:15-104) for them.
def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out = x @ weight^T with 32-bit accumulation.  ``weight`` [N,K] row-major
    as stored in checkpoints.  ``out`` may be float32 for bfloat16 operands."""
    _need_cuda(x, weight, out)
    if x.dtype != weight.dtype:
        raise KernelError(f"linear: operand types differ ({x.dtype} vs {weight.dtype})")
    if out.dtype == x.dtype:
        torch.mm(x, weight.t(), out=out)
    elif out.dtype == torch.float32:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    else:
        raise KernelError(f"linear: cannot write {out.dtype} from {x.dtype}")


def linear_add(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor) -> None:
    """residual (float32) += x @ weight^T through the library, the sum formed in 32-bit: the product
    never exists rounded to the operands' type, and the norm behind it has one tensor less to read."""
    _need_cuda(x, weight, residual)
    if x.dtype != weight.dtype or residual.dtype != torch.float32:
        raise KernelError(f"linear_add: {x.dtype} x {weight.dtype} into {residual.dtype}")
    if x.dtype == torch.float32:
        torch.addmm(residual, x, weight.t(), out=residual)
    else:
        torch.addmm(residual, x, weight.t(), out_dtype=torch.float32, out=residual)


LIBRARY_ADDS_INTO_RESIDUAL = True   # products of more than GEMM_TC_MAX_TOKENS tokens add into the 32-bit residual themselves
EPI_BF16, EPI_F32, EPI_RESIDUAL_ADD, EPI_SWIGLU = 0, 1, 2, 3
GEMM_TC_MAX_TOKENS = 64    # up to here the one-block tcgen05 product runs
# From there to GEMM_PAIR_MAX_TOKENS the two-SM product (cta_group::2, csrc/gemm_pair.cu) can take over,
# with the same fused epilogues.  Off: alone it reaches 0.7 to 1.0 of the library's speed at 128 to 512
# tokens (the gate|up product at 128 tokens: 41 us against 41), but inside a step its blocks, one per SM
# with nearly all of the shared memory, leave no room for the next kernel to move in early, and a
# 256-token step of the 8B shape takes 8.2 ms with it against 5.9 ms with the library's products.
USE_PAIR_GEMM = False
GEMM_PAIR_MAX_TOKENS = 512
USE_TCGEN05_GEMM = True    # tests flip this to compare with the library route
FOLD_NORM = True           # fold the RMSNorm between two tcgen05 products into their epilogues


def gemm_tc_plan(T: int, N: int, K: int, want_splits: int):
    """(tokens per tile, K ranges) the tensor-core product would use."""
    tok, splits = c_int(), c_int()
    _lib("gemm_tcgen05").ff_gemm_tc_plan(c_int(T), c_int(N), c_int(K), c_int(want_splits), ctypes.byref(tok),
                                       ctypes.byref(splits))
    return tok.value, splits.value


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int, want_splits: int,
            status: torch.Tensor, *, norm_out: Optional[tuple] = None, norm_in: Optional[tuple] = None) -> None:
    """out (op)= x @ weight^T on tcgen05 tensor cores; bfloat16 operands, 32-bit accumulation.

    epilogue: EPI_BF16 store bfloat16, EPI_F32 store float32, EPI_RESIDUAL_ADD add into a float32
    ``out``, EPI_SWIGLU store silu(gate)*up as bfloat16 [T, N/2] for a weight whose rows interleave
    gate and up in groups of 16.  ``want_splits`` K ranges (at most 8) share a thread-block cluster.

    An RMSNorm between two products can be folded into them.  Producing side (EPI_RESIDUAL_ADD):
    ``norm_out`` = (xw bfloat16 [T, N], norm weight float32 [N], ssq float32 [ceil(N/128), T]) receives
    bfloat16(out * w) and each row tile's sum of squares per token.  Consuming side: ``norm_in`` =
    (ssq [parts, T], norm_dim, eps) scales token t's result by rsqrt(sum_p ssq[p, t] / norm_dim + eps)."""
    _need_cuda(x, weight, out, status)
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    T, Kd = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == Kd
    if epilogue == EPI_BF16 or epilogue == EPI_SWIGLU:
        assert out.dtype == torch.bfloat16
    else:
        assert out.dtype == torch.float32
    assert out.shape[0] == T and out.shape[1] == (N // 2 if epilogue == EPI_SWIGLU else N)
    xw = xw_w = ssq_out = ssq_in = None
    parts = dim = 0
    eps = 0.0
    if norm_out is not None:
        xw, xw_w, ssq_out = norm_out
        _need_cuda(xw, xw_w, ssq_out)
        assert epilogue == EPI_RESIDUAL_ADD and xw.dtype == torch.bfloat16 and xw.shape == (T, N)
        assert xw_w.dtype == torch.float32 and xw_w.numel() == N
        assert ssq_out.dtype == torch.float32 and ssq_out.numel() >= -(-N // 128) * T
    if norm_in is not None:
        ssq_in, dim, eps = norm_in
        _need_cuda(ssq_in)
        assert ssq_in.dtype == torch.float32 and ssq_in.dim() == 2 and ssq_in.shape[1] == T
        parts = ssq_in.shape[0]
    _check(_lib("gemm_tcgen05").ff_gemm_tc(
        _p(x), _p(weight), _p(out), c_int(out.stride(0)), c_int(T), c_int(N), c_int(Kd), c_int(epilogue),
        c_int(want_splits), c_int(1 if USE_PDL else 0), _p(xw), _p(xw_w), _p(ssq_out), _p(ssq_in),
        c_int(parts), c_int(dim), c_float(eps), _p(status), _stream()), "gemm_tc")


def gemm_pair_plan(T: int, N: int, K: int, want_ranges: int):
    """(tokens per tile, K ranges) the two-SM product would use."""
    tok, ranges = c_int(), c_int()
    _lib("gemm_pair").ff_gemm_pair_plan(c_int(T), c_int(N), c_int(K), c_int(want_ranges), ctypes.byref(tok),
                                        ctypes.byref(ranges))
    return tok.value, ranges.value


def gemm_pair(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int, want_ranges: int,
              status: torch.Tensor, *, norm_out: Optional[tuple] = None, norm_in: Optional[tuple] = None) -> None:
    """out (op)= x @ weight^T on pairs of SMs (tcgen05 with cta_group::2), for steps of about a hundred to
    a few hundred tokens.  Arguments as `gemm_tc`; ``want_ranges`` K ranges (at most 4)."""
    _need_cuda(x, weight, status)
    if not out.is_cuda or out.dim() != 2 or out.stride(1) != 1:
        raise KernelError("gemm_pair: the output must be a CUDA matrix with contiguous rows")
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    T, Kd = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == Kd
    assert out.dtype == (torch.bfloat16 if epilogue in (EPI_BF16, EPI_SWIGLU) else torch.float32)
    assert out.shape[0] == T and out.shape[1] == (N // 2 if epilogue == EPI_SWIGLU else N)
    xw = xw_w = ssq_out = ssq_in = None
    parts = dim = 0
    eps = 0.0
    if norm_out is not None:
        xw, xw_w, ssq_out = norm_out
        _need_cuda(xw, xw_w, ssq_out)
        assert epilogue == EPI_RESIDUAL_ADD and xw.dtype == torch.bfloat16 and xw.shape == (T, N)
        assert xw_w.dtype == torch.float32 and xw_w.numel() == N
        assert ssq_out.dtype == torch.float32 and ssq_out.numel() >= -(-N // 128) * T
    if norm_in is not None:
        ssq_in, dim, eps = norm_in
        _need_cuda(ssq_in)
        assert ssq_in.dtype == torch.float32 and ssq_in.dim() == 2 and ssq_in.shape[1] == T
        parts = ssq_in.shape[0]
    _check(_lib("gemm_pair").ff_gemm_pair(
        _p(x), _p(weight), _p(out), c_int(out.stride(0)), c_int(T), c_int(N), c_int(Kd), c_int(epilogue),
        c_int(want_ranges), c_int(1 if USE_PDL else 0), _p(xw), _p(xw_w), _p(ssq_out), _p(ssq_in),
        c_int(parts), c_int(dim), c_float(eps), _p(status), _stream()), "gemm_pair")


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stack gate and up rows in groups of 16: rows [32g, 32g+16) are gate rows [16g, 16g+16),
    rows [32g+16, 32g+32) the up rows of the same columns.  Needs I % 16 == 0."""
    I, H = gate.shape
    assert I % 16 == 0 and up.shape == gate.shape
    return torch.stack([gate.view(I // 16, 16, H), up.view(I // 16, 16, H)], dim=1).reshape(2 * I, H).contiguous()


def set_exact_matmul() -> None:
    """No reduced-precision matrix mode anywhere: 32-bit products are true
    32-bit (no TF32), 16-bit products accumulate and reduce in 32-bit."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    try:
        torch.set_float32_matmul_precision("highest")
    except Exception:  # noqa: BLE001
        pass


_ATTN_FORCE_SIMT = False      # tests flip this to compare the two kernels


@functools.lru_cache(maxsize=None)
def sm_count(device_index: Optional[int] = None) -> int:
    """Streaming multiprocessors of the device (the current one by default), asked of the driver
    once.  Grid sizes, K splits and scratch extents are derived from it; no file holds the figure."""
    if device_index is None:
        device_index = torch.cuda.current_device()
    return int(torch.cuda.get_device_properties(device_index).multi_processor_count)


def _sm_target_ctas() -> int:
    """Blocks that the decode attention's scratch memory is sized for: four per SM."""
    return 4 * sm_count()


def _planes_defs(defs: dict, planes: int) -> dict:
    """Build definitions for a cache of `planes` planes a page (2: keys and values; 1: one vector that is both)."""
    if planes not in (1, 2):
        raise KernelError(f"a cache page has 1 or 2 planes, got {planes}")
    return dict(defs, FF_KV_PLANES=1) if planes == 1 else defs


def _attn_lib(d: int, planes: int = 2) -> ctypes.CDLL:
    return _configured(load_module("attention_mma.cu", _planes_defs({"FF_HEAD_DIM": d}, planes)))


def mma_attention_supported(dtype: torch.dtype, d: int) -> bool:
    return dtype == torch.bfloat16 and d % 16 == 0 and 16 <= d <= 256


def _bias_args(dist_bias: Optional[torch.Tensor], nq: int, window: int):
    _check_dist_bias(dist_bias, nq, window)
    return _p(dist_bias), c_int(dist_bias.shape[1] if dist_bias is not None else 0)


def attn_tiled(q, q_stride, pages, table, cu_q, ctx_lens, n_seqs, total_tiles, out, nq, nkv, d, scale,
               window, status: Optional[torch.Tensor] = None, dist_bias: Optional[torch.Tensor] = None,
               softcap: float = 0.0) -> None:
    """Tensor-core attention for any mix of sequences (bfloat16).  ``status`` (int32 [1]) is set to 4
    when a key that must be read has no valid page in the block table.  ``dist_bias``: as for
    `paged_attention_simt`."""
    _need_cuda(pages, table, cu_q, ctx_lens, out, status, dist_bias)
    num_blocks, planes, _, block_size, _ = pages.shape
    _check(_attn_lib(d, planes).ff_attn_tiled(
        _p(q), c_int(q_stride), _p(pages), _p(table), c_int(table.shape[1]), _p(cu_q), _p(ctx_lens),
        c_int(n_seqs), c_int(total_tiles), _p(out), c_int(out.shape[1]), c_int(nq), c_int(nkv),
        c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), *_bias_args(dist_bias, nq, window),
        c_float(softcap), _p(status), _stream()), "attn_tiled")


def attn_decode(q, q_stride, pages, table, cu_q, ctx_lens, n_seqs, out, part_o, part_ml, nq, nkv, d,
                scale, window, num_splits, status: Optional[torch.Tensor] = None,
                dist_bias: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Split-KV tensor-core attention when every sequence has one token (bfloat16).  ``status`` and
    ``dist_bias`` as for `attn_tiled`."""
    _need_cuda(pages, table, cu_q, ctx_lens, out, part_o, part_ml, status, dist_bias)
    num_blocks, planes, _, block_size, _ = pages.shape
    _check(_attn_lib(d, planes).ff_attn_decode(
        _p(q), c_int(q_stride), _p(pages), _p(table), c_int(table.shape[1]), _p(cu_q), _p(ctx_lens),
        c_int(n_seqs), _p(out), c_int(out.shape[1]), _p(part_o), _p(part_ml), c_int(nq), c_int(nkv),
        c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), c_int(num_splits),
        *_bias_args(dist_bias, nq, window), c_float(softcap), _p(status), _stream()), "attn_decode")
    global LAUNCHES
    if num_splits > 1:
        LAUNCHES += 1     # the kernel that joins the splits


DECODE_FINISHES_HEADS = True    # pure decode steps: per-head norm, rotation and cache write inside the attention kernel


def decode_finishes_heads(ctx, dtype: torch.dtype, nq: int, nkv: int, d: int, rotary_dim: int) -> bool:
    """True if this step's attention kernel can take the raw q|k|v projection: every sequence
    decodes one token, bfloat16, a head size in steps of 64 that is rotated whole or not at all,
    and at most 16 query heads per kv head."""
    return (DECODE_FINISHES_HEADS and not _ATTN_FORCE_SIMT and ctx.num_seqs > 0
            and ctx.num_decode_seqs == ctx.num_seqs and dtype == torch.bfloat16 and d % 64 == 0 and d <= 256
            and nkv > 0 and nq // nkv <= 16 and rotary_dim in (0, d))


def attn_decode_heads(qkv, pages, table, ctx, out, nq, nkv, d, scale, window, q_norm_w, k_norm_w, eps,
                      cos_sin, num_splits: Optional[int] = None) -> None:
    """The split-KV decode attention fed with the raw q|k|v projection ``[T, (nq + 2 nkv) d]``:
    it finishes the heads itself (per-head RMSNorm, rotation, cache write of the newest key and
    value) and replaces `qk_norm_rope_store` + `attn_decode` in steps that only decode."""
    _need_cuda(qkv, pages, table, out, q_norm_w, k_norm_w, cos_sin)
    num_blocks, _, _, block_size, _ = pages.shape
    n = ctx.num_seqs
    global LAUNCHES
    units = 0 if num_splits else decode_units(n, nkv, d, ctx.ranges_by_length)
    splits = num_splits or decode_splits(n, nkv, ctx.max_kv_len)
    part_o, part_ml, seq_ranges = _decode_scratch(ctx.workspace, n, nq, nkv, d, splits)
    if units:
        attn_decode_units(qkv, qkv.shape[1], pages, table, ctx.cu_q, ctx.ctx_lens, n, out, part_o, part_ml,
                          seq_ranges, nq, nkv, d, scale, window, units, DECODE_MAX_RANGES,
                          heads=(q_norm_w, k_norm_w, eps, cos_sin), status=ctx.status)
        return
    _check(_attn_lib(d).ff_attn_decode_heads(
        _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(table), c_int(table.shape[1]), _p(ctx.cu_q), _p(ctx.ctx_lens),
        c_int(n), _p(out), c_int(out.shape[1]), _p(part_o), _p(part_ml), c_int(nq), c_int(nkv),
        c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), c_int(splits),
        _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(cos_sin), c_int(cos_sin.shape[0] if cos_sin is not None else 0),
        _p(ctx.status), _stream()), "attn_decode_heads")
    if splits > 1:
        LAUNCHES += 1     # the kernel that joins the splits


USE_TC_ATTENTION = True     # tcgen05 attention for prompt portions where the sizes allow


def _attn_tc_lib(d: int, page_list: Optional[int] = None, planes: int = 2) -> ctypes.CDLL:
    defs = _planes_defs({"FF_HEAD_DIM": d}, planes)
    if page_list is not None:
        defs["FF_ATC_PAGE_LIST"] = int(page_list)       # a test build with a tiny ring of page ids
    return _configured(load_module("attention_tc.cu", defs))


def tc_attention_supported(dtype: torch.dtype, d: int, block_size: int, max_kv_len: int = 0) -> bool:
    """The tcgen05 attention kernel takes head sizes 64..256 in steps of 64 and pages of 8..64 tokens
    that divide 64; contexts of any length (it walks the block table in pieces)."""
    return dtype == torch.bfloat16 and d % 64 == 0 and 64 <= d <= 256 and block_size in (8, 16, 32, 64)


def attn_tc(q, q_stride, pages, table, cu_q, ctx_lens, n_seqs, total_tiles, out, nq, nkv, d, scale, window,
            status, page_list: Optional[int] = None, shares=None, dist_bias: Optional[torch.Tensor] = None,
            softcap: float = 0.0) -> None:
    """tcgen05 flash attention over the paged cache (bfloat16); total_tiles counts row tiles of 128.
    ``shares`` = (count, part_o, part_ml, first row, rows): every row tile's keys are shared out over
    ``count`` blocks and a second kernel joins their partial results (for prompts so short that their
    row tiles alone would leave most SMs idle); the scratch tensors are float32 with at least
    (first row + rows) * nq * count * d and ... * 2 elements.  ``dist_bias``: as for `paged_attention_simt`."""
    _need_cuda(pages, table, cu_q, ctx_lens, out, status, dist_bias)
    num_blocks, planes, _, block_size, _ = pages.shape
    count, part_o, part_ml, row0, rows = shares if shares is not None else (1, None, None, 0, 0)
    if count > 1:
        _need_cuda(part_o, part_ml)
        need = (row0 + rows) * nq * count
        assert part_o.dtype == part_ml.dtype == torch.float32 and part_o.numel() >= need * d and part_ml.numel() >= need * 2
    _check(_attn_tc_lib(d, page_list, planes).ff_attn_tc(
        _p(q), c_int(q_stride), _p(pages), _p(table), c_int(table.shape[1]), _p(cu_q), _p(ctx_lens),
        c_int(n_seqs), c_int(total_tiles), _p(out), c_int(out.shape[1]), c_int(nq), c_int(nkv),
        c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), _p(status), c_int(count), _p(part_o),
        _p(part_ml), c_int(row0), c_int(rows), *_bias_args(dist_bias, nq, window), c_float(softcap), _stream()), "attn_tc")
    if count > 1:
        global LAUNCHES
        LAUNCHES += 1     # the kernel that joins the shares


USE_TC_SHARES = True       # short portions behind long contexts share their keys out over several blocks


def attn_tc_shares(total_tiles: int, nkv: int, max_key_tiles: int) -> int:
    """Over how many blocks a row tile's keys are shared out: 1 unless the row tiles alone would fill
    less than three quarters of the places (two per SM) and each would walk at least eight tiles of
    keys; then as many as fill the places once, each share at least four key tiles long, at most 8."""
    places = 2 * sm_count()
    units = total_tiles * nkv
    if not USE_TC_SHARES or units * 4 >= places * 3 or max_key_tiles < 8:
        return 1
    return max(1, min(8, places // units, max_key_tiles // 4))


def decode_splits(n_seqs: int, nkv: int, max_kv_len: int) -> int:
    """Ranges of keys per (sequence, kv head).  Three blocks of the decode kernel fit an SM: few
    sequences get as many ranges as fill those places once (at most 20), many sequences three.
    Measured on the 8B shape at context 2100 (ms per step, ranges): batch 1 3.29 (24), 4 3.51 (13),
    8 3.70 (6) against 3.83 (8), 16 4.18 (3) against 4.39 (8), 32 5.43 (3) against 5.70 (8),
    64 8.08 (3) against 8.34 (8)."""
    tiles = max(1, -(-max_kv_len // 64))
    places = 3 * sm_count()
    want = max(3, min(places // max(1, n_seqs * nkv), 20))
    return max(1, min(want, tiles, 64))


DECODE_BY_UNITS = True      # few sequences: ranges of keys shared out by length so that the blocks fill the SMs once
DECODE_MAX_RANGES = 64      # a sequence is cut into at most this many ranges (and a range holds 1.5 tiles of keys at least)


@functools.lru_cache(maxsize=None)
def _decode_places_per_kv_head(nkv: int, d: int) -> int:
    return sm_count() * int(_attn_lib(d).ff_attn_decode_blocks_per_sm()) // nkv


def lengths_differ_much(ctx_lens) -> bool:
    """True if the longest of these decoding sequences has a quarter more tiles of keys than the
    average: then a fixed number of ranges per sequence makes blocks of very different length, and
    the attention shares its blocks out by length instead (`decode_units`).  Also true for one or
    two sequences of 3000 tokens or more."""
    tiles = [c // 64 + 1 for c in ctx_lens]
    if len(tiles) <= 2:
        # one or two long sequences: the fixed 20 ranges leave two thirds of the SMs' places empty and every
        # block waits for its own tiles one after the other (batch 1 behind 32 000 tokens: 2.3 TB/s);
        # shared out by length a sequence gets as many ranges as there are places
        return bool(tiles) and max(tiles) >= 48
    return max(tiles) >= 4 and max(tiles) * len(tiles) >= 1.25 * sum(tiles)


BY_LENGTH_CALLS = 0         # how often the kernel that shares its blocks out by length was chosen


def decode_units(n_seqs: int, nkv: int, d: int, by_length: bool) -> int:
    """Blocks per kv head when the ranges of keys are shared out by length (as many as fill every
    SM's places once, at most `DECODE_MAX_RANGES` a sequence), or 0 for the fixed number of ranges
    of `decode_splits`.  Measured on the 8B shape, kernel and join alone, us: eight sequences of
    200 to 6000 tokens 18.6 against 31.4 (six ranges each); seven of 100 and one of 16000 28 against
    70; eight of 2100 17.7 against 17.2 (the share-out costs every block a scan of the lengths), so
    equal lengths keep the fixed ranges.  Each sequence should get two units at least."""
    if not (DECODE_BY_UNITS and by_length):
        return 0
    units = min(_decode_places_per_kv_head(nkv, d), n_seqs * DECODE_MAX_RANGES)
    return units if 2 * n_seqs <= units and n_seqs <= 128 else 0


def _decode_scratch(ws, n: int, nq: int, nkv: int, d: int, splits: int):
    """Scratch memory of the decode attention: partial outputs, their (max, sum) pairs and the
    number of ranges per sequence.  The extent never shrinks as the batch grows (captured graphs
    of every batch size share the buffers that the largest one sized)."""
    units = _decode_places_per_kv_head(nkv, d) if DECODE_BY_UNITS else 0
    cap = max(n * nq * splits, (nq // nkv) * _sm_target_ctas() + n * nq, nq * units * (units // 2))
    return (ws.get("attn.part_o", (cap * d,), torch.float32), ws.get("attn.part_ml", (cap * 2,), torch.float32),
            ws.get("attn.seq_ranges", (max(n, 128),), torch.int32))


def attn_decode_units(q, q_stride, pages, table, cu_q, ctx_lens, n_seqs, out, part_o, part_ml, seq_ranges,
                      nq, nkv, d, scale, window, units, max_ranges, heads=None, status=None,
                      dist_bias: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Split-KV decode attention with `units` blocks per kv head shared out among the sequences
    in proportion to their lengths.  ``heads = (q_norm_w, k_norm_w, eps, cos_sin)``: q is the raw
    q|k|v projection and the kernel finishes the heads itself."""
    _need_cuda(q, pages, table, cu_q, ctx_lens, out, part_o, part_ml, seq_ranges)
    num_blocks, planes, _, block_size, _ = pages.shape
    assert part_o.numel() >= n_seqs * nq * units * d and part_ml.numel() >= n_seqs * nq * units * 2
    qw, kw, eps, cos_sin = heads if heads is not None else (None, None, 0.0, None)
    _need_cuda(qw, kw, cos_sin, status, dist_bias)
    _check(_attn_lib(d, planes).ff_attn_decode_units(
        _p(q), c_int(q_stride), _p(pages), _p(table), c_int(table.shape[1]), _p(cu_q), _p(ctx_lens),
        c_int(n_seqs), _p(out), c_int(out.shape[1]), _p(part_o), _p(part_ml), _p(seq_ranges), c_int(nq),
        c_int(nkv), c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), c_int(units),
        c_int(max_ranges), c_int(1 if heads is not None else 0), _p(qw), _p(kw), c_float(eps), _p(cos_sin),
        c_int(cos_sin.shape[0] if cos_sin is not None else 0), *_bias_args(dist_bias, nq, window), c_float(softcap),
        _p(status), _stream()), "attn_decode_units")
    global LAUNCHES, BY_LENGTH_CALLS
    BY_LENGTH_CALLS += 1
    if units > n_seqs and max_ranges > 1:
        LAUNCHES += 1     # the kernel that joins the ranges


def paged_attention(q: torch.Tensor, q_stride: int, pages: torch.Tensor, table: torch.Tensor, ctx,
                    out: torch.Tensor, nq: int, nkv: int, d: int, scale: float, window: int,
                    dist_bias: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Attention of a step's tokens over the paged cache; picks the kernel: the
    tensor-core kernels for bfloat16 and head sizes in steps of 16, the plain
    kernel for 32-bit and every other head size up to 256.  ``dist_bias`` float32 [nq, L >= window]: entry
    (h, i - j) is taken off the score of query position i and key position j.  ``softcap`` c > 0: the scaled score s
    becomes c tanh(s / c), before the bias."""
    if _ATTN_FORCE_SIMT or not mma_attention_supported(q.dtype, d):
        paged_attention_simt(q, q_stride, pages, table, ctx.token_seq, ctx.positions, out, nq, nkv, d,
                             scale, window, ctx.status, dist_bias, softcap)
        return
    G = nq // nkv
    n = ctx.num_seqs
    n_dec = ctx.num_decode_seqs if G <= 16 else 0      # these come first in the step's arrays
    if n_dec:
        # one-token sequences: split-KV kernel
        splits = decode_splits(n_dec, nkv, ctx.max_kv_len)
        units = decode_units(n_dec, nkv, d, ctx.ranges_by_length)
        part_o, part_ml, seq_ranges = _decode_scratch(ctx.workspace, n_dec, nq, nkv, d, splits)
        if units:
            attn_decode_units(q, q_stride, pages, table, ctx.cu_q, ctx.ctx_lens, n_dec, out, part_o, part_ml,
                              seq_ranges, nq, nkv, d, scale, window, units, DECODE_MAX_RANGES, status=ctx.status,
                              dist_bias=dist_bias, softcap=softcap)
        else:
            attn_decode(q, q_stride, pages, table, ctx.cu_q, ctx.ctx_lens, n_dec, out, part_o, part_ml, nq, nkv,
                        d, scale, window, splits, ctx.status, dist_bias, softcap)
    if n_dec < n:
        # portions of prompts: tiled kernel over the remaining sequences (token offsets in cu_q are absolute)
        # every layer of a step asks the same of the step's arrays: worked out once and kept with the step
        memo = getattr(ctx, "memo", None)
        tail = memo.get(("attn_tail", id(table), n_dec)) if memo is not None else None
        if tail is None:
            tail = (table[n_dec:], ctx.cu_q[n_dec:], ctx.ctx_lens[n_dec:])
            if memo is not None:
                memo[("attn_tail", id(table), n_dec)] = tail
        table_t, cu_q_t, ctx_lens_t = tail
        if USE_TC_ATTENTION and tc_attention_supported(q.dtype, d, pages.shape[3], ctx.max_kv_len):
            plan = memo.get(("attn_tc_plan", G, nkv, n_dec, ctx.captured)) if memo is not None else None
            if plan is None:
                tiles = sum(-(-(ql * G) // 128) for ql in ctx.q_lens[n_dec:])
                # a captured step does not know its requests' lengths: the level it was captured for stands in
                key_tiles = 4 * getattr(ctx, "key_share_level", 0) if ctx.captured else \
                    max(-(-(c + ql) // 64) for c, ql in zip(ctx.ctx_lens_host[n_dec:], ctx.q_lens[n_dec:]))
                count = attn_tc_shares(tiles, nkv, key_tiles)
                plan = (tiles, count, sum(ctx.q_lens[:n_dec]), sum(ctx.q_lens[n_dec:]))
                if memo is not None:
                    memo[("attn_tc_plan", G, nkv, n_dec, ctx.captured)] = plan
            tiles, count, row0, rows = plan
            shares = None
            if count > 1:
                cells = (row0 + rows) * nq * count
                shares = (count, ctx.workspace.get("attn.tc_part_o", (cells * d,), torch.float32),
                          ctx.workspace.get("attn.tc_part_ml", (cells * 2,), torch.float32), row0, rows)
            attn_tc(q, q_stride, pages, table_t, cu_q_t, ctx_lens_t, n - n_dec, tiles,
                    out, nq, nkv, d, scale, window, ctx.status, shares=shares, dist_bias=dist_bias, softcap=softcap)
        else:
            tiles = sum(-(-(ql * G) // 64) for ql in ctx.q_lens[n_dec:])
            attn_tiled(q, q_stride, pages, table_t, cu_q_t, ctx_lens_t, n - n_dec,
                       tiles, out, nq, nkv, d, scale, window, ctx.status, dist_bias, softcap)


# --------------------------------------------------------------------------- #
# layer norm and the row kernels at the head of a pass of a looped range of layers
def add_layer_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                   bias: Optional[torch.Tensor], eps: float, out: torch.Tensor,
                   row_idx: Optional[torch.Tensor] = None, delta_scale: float = 1.0) -> None:
    """residual (+= delta_scale * delta); out = (v - mean) / sqrt(var + eps) * weight + bias over each row v
    of the residual (float32 [T,H]).  With ``row_idx`` only those rows, and the residual is not written."""
    _need_cuda(residual, delta, weight, bias, out, row_idx)
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32
    H = residual.shape[-1]
    rows = out.shape[0]
    assert out.shape[-1] == H and weight.numel() == H and (bias is None or (bias.numel() == H and bias.dtype == torch.float32))
    if row_idx is None:
        assert rows == residual.shape[0]
    else:
        assert row_idx.dtype == torch.int32 and row_idx.numel() == rows
    if delta is not None:
        assert delta.shape == residual.shape
    _check(_lib("layer_norm").ff_add_layer_norm(
        _p(residual), _p(delta), c_int(_dt(delta) if delta is not None else 0), c_float(delta_scale), _p(row_idx),
        _p(weight), _p(bias), c_float(eps), _p(out), c_int(_dt(out)), c_int(rows), c_int(H),
        c_int(1 if row_idx is None else 0), _stream()), "add_layer_norm")


def concat_cast(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [a[t] | b[t]] for two float32 [T,H] streams, in out's type [T,2H]."""
    _need_cuda(a, b, out)
    T, H = a.shape
    assert a.dtype == b.dtype == torch.float32 and b.shape == a.shape and out.shape == (T, 2 * H)
    _check(_lib("layer_norm").ff_concat_cast(_p(a), _p(b), _p(out), c_int(_dt(out)), c_int(T), c_int(H), _stream()),
           "concat_cast")


def add_row_vector(x: torch.Tensor, v: torch.Tensor, scale: float = 1.0) -> None:
    """x[t,:] += scale * v for float32 x [T,H], v [H]."""
    _need_cuda(x, v)
    assert x.dtype == v.dtype == torch.float32 and v.numel() == x.shape[1]
    _check(_lib("layer_norm").ff_add_row_vector(_p(x), _p(v), c_float(scale), c_int(x.shape[0]), c_int(x.shape[1]),
                                               _stream()), "add_row_vector")


def linear_scaled_add(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, alpha: float) -> None:
    """residual (float32) += alpha * x @ weight^T through the library, summed in 32-bit."""
    _need_cuda(x, weight, residual)
    if x.dtype != weight.dtype or residual.dtype != torch.float32:
        raise KernelError(f"linear_scaled_add: {x.dtype} x {weight.dtype} into {residual.dtype}")
    if x.dtype == torch.float32:
        torch.addmm(residual, x, weight.t(), alpha=alpha, out=residual)
    else:
        torch.addmm(residual, x, weight.t(), alpha=alpha, out_dtype=torch.float32, out=residual)


def batched_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = x[b] @ weight[b]^T for b in a batch (the library's batched product); x [B,T,K] and weight
    [B,N,K] may be strided views with unit inner stride, out [B,T,N] is contiguous."""
    if not (x.is_cuda and weight.is_cuda and out.is_cuda):
        raise KernelError("firefly_b200 kernels run on a CUDA device only")
    if x.dtype != weight.dtype or out.dtype != x.dtype or not out.is_contiguous():
        raise KernelError("batched_linear: operands and result share one type; the result is contiguous")
    torch.bmm(x, weight.transpose(1, 2), out=out)


# --------------------------------------------------------------------------- #
# the recurrent mixer with a matrix state per head (csrc/wkv.cu)
def wkv_shift_mix(x, mu, state, prev_off: int, ctx, mixes) -> None:
    """mixes[s, t] = x[t] + (x[t-1] - x[t]) * mu[s] for the five inputs of the mixer; the row in front of a
    portion's first token comes from the request's state slot (zeros for a fresh request)."""
    _need_cuda(x, mu, state, mixes)
    T, W = x.shape
    assert mu.dtype == torch.float32 and mu.shape == (5, W) and state.dtype == torch.float32 and state.dim() == 2
    assert mixes.shape == (5, T, W) and mixes.dtype == x.dtype
    _check(_lib("wkv").ff_wkv_shift_mix(_p(x), c_int(_dt(x)), _p(mu), _p(state), ctypes.c_longlong(state.stride(0)),
                                       c_int(prev_off), _p(ctx.token_seq), _p(ctx.cu_q), _p(ctx.state_slots),
                                       _p(ctx.seq_fresh), _p(mixes), c_int(T), c_int(W), _stream()), "wkv_shift_mix")


def tanh_cast(src: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(src, out)
    assert src.dtype == torch.float32 and src.numel() == out.numel()
    _check(_lib("wkv").ff_tanh_cast(_p(src), _p(out), c_int(_dt(out)), ctypes.c_longlong(src.numel()), _stream()),
           "tanh_cast")


WKV_MAX_DIM = 128


def wkv_state_dim(dim: int) -> int:
    """The head size the recurrence kernel keeps its state for (the next of 32, 64, 128): a head's state takes
    that many squared floats in the request's slot, in the kernel's own order."""
    if not (0 < dim <= WKV_MAX_DIM):
        raise KernelError(f"wkv: head size {dim} is not supported (1..{WKV_MAX_DIM})")
    return 32 if dim <= 32 else (64 if dim <= 64 else 128)


def wkv_scan(rkvg, dlog, w0, u, state, prev_off: int, x, ctx, o, heads: int, dim: int) -> None:
    """The recurrence, token by token, one block per (sequence, head).  rkvg [4,T,heads*dim] (r, k, v, gate
    projections; the gate is not read here), dlog float32 [T,heads*dim] (the decay's inner logarithm without
    its offset w0), state float32 [slots, prev_off + W] with prev_off >= heads * wkv_state_dim(dim)^2 (read unless
    the request is fresh, written back in the kernel's own order, the portion's last row of x saved at prev_off),
    o float32 [T, heads*dim]."""
    _need_cuda(rkvg, dlog, w0, u, state, x, o)
    T, W = x.shape
    HD = heads * dim
    assert rkvg.shape == (4, T, HD) and rkvg.dtype == x.dtype and dlog.shape == (T, HD) and dlog.dtype == torch.float32
    assert o.shape == (T, HD) and o.dtype == torch.float32 and state.dtype == torch.float32
    assert w0.dtype == u.dtype == torch.float32 and w0.numel() == HD and u.numel() == HD
    assert state.shape[1] >= prev_off + W and prev_off >= heads * wkv_state_dim(dim) ** 2
    _check(_lib("wkv").ff_wkv_scan(_p(rkvg), c_int(_dt(rkvg)), _p(dlog), _p(w0), _p(u), _p(state),
                                  ctypes.c_longlong(state.stride(0)), c_int(prev_off), _p(x), c_int(W), _p(ctx.cu_q),
                                  _p(ctx.state_slots), _p(ctx.seq_fresh), _p(o), c_int(T), c_int(ctx.num_seqs),
                                  c_int(heads), c_int(dim), _stream()), "wkv_scan")


def wkv_out(o, gate, norm_w, eps: float, y, heads: int, dim: int) -> None:
    """y = o / rms(o over a head) * norm_w * silu(gate); o float32 [T, heads*dim], gate and y in the activation type."""
    _need_cuda(o, gate, norm_w, y)
    T = o.shape[0]
    assert o.dtype == torch.float32 and norm_w.dtype == torch.float32 and gate.dtype == y.dtype
    assert gate.shape == o.shape == y.shape and o.shape[1] == heads * dim
    _check(_lib("wkv").ff_wkv_out(_p(o), _p(gate), c_int(_dt(gate)), _p(norm_w), c_float(eps), _p(y), c_int(T),
                                 c_int(heads), c_int(dim), _stream()), "wkv_out")


# --------------------------------------------------------------------------- #
# attention over a cached latent vector (csrc/latent_attention.cu)
def latent_finish(q, dkv, q_abs, c_norm_w, eps: float, freq, ctx, table, pages, q_full,
                  heads: int, dim: int, rot: int, kv_rank: int, rotary_dims: Optional[int] = None,
                  interleaved: bool = False) -> None:
    """Finish a step's query rows and write its cache rows.  ``q`` [T, heads * (dim + rot)] and ``dkv`` [T, kv_rank +
    rot] (the down projection; None: the layer reads a cache that another layer writes, only the queries are
    finished) may be column ranges of wider matrices; q_abs [heads, T, kv_rank]; freq float64 [rotary_dims/2]
    (rotary_dims <= rot, by default rot: the first that many elements of the rotated part turn, the rest pass;
    ``interleaved``: element 2i turns with element 2i + 1, else i with i + rotary_dims/2);
    pages [blocks, planes, 1, block, kv_rank + rot]; q_full [T, heads * (kv_rank + rot)]."""
    rdims = rot if rotary_dims is None else int(rotary_dims)
    _need_cuda(q_abs, c_norm_w, freq, table, pages, q_full)
    for m in (q, dkv):
        if m is not None and (not m.is_cuda or m.stride(1) != 1):
            raise KernelError("latent_finish: q and dkv are CUDA matrices with contiguous rows")
    T = q.shape[0]
    d = kv_rank + rot
    num_blocks, planes, one, block_size, cd = pages.shape
    assert planes in (1, 2) and one == 1 and cd == d and pages.dtype == q.dtype == q_abs.dtype == q_full.dtype
    assert q.shape[1] == heads * (dim + rot) and (dkv is None or (dkv.shape == (T, d) and dkv.dtype == q.dtype))
    assert q_abs.shape == (heads, T, kv_rank) and q_full.shape == (T, heads * d)
    assert freq.dtype == torch.float64 and freq.numel() == rdims // 2 and c_norm_w.dtype == torch.float32
    _check(_lib("latent_attention").ff_latent_finish(
        c_void_p(q.data_ptr()), c_int(q.stride(0)), c_void_p(dkv.data_ptr() if dkv is not None else None),
        c_int(dkv.stride(0) if dkv is not None else 0), c_int(_dt(q)), _p(q_abs), _p(c_norm_w),
        c_float(eps), _p(freq), _p(ctx.positions), _p(ctx.token_seq), _p(table), c_int(table.shape[1]),
        c_int(block_size), c_int(num_blocks), c_int(planes), _p(pages), _p(q_full), c_int(T), c_int(heads), c_int(dim),
        c_int(rot), c_int(rdims), c_int(kv_rank), c_int(1 if interleaved else 0), _p(ctx.status), _stream()), "latent_finish")


def latent_gate(val, g, y, heads: int, vdim: int, per_head: bool = False) -> None:
    """y[t, h*vdim + j] = val[h, t, j] * sigmoid(g[t, h*vdim + j]) (``per_head``: sigmoid(g[t, h])); g may be a column
    range of a wider matrix."""
    if not g.is_cuda or g.stride(1) != 1:
        raise KernelError("latent_gate: the gate must be a CUDA matrix with contiguous rows")
    _need_cuda(val, y)
    T = y.shape[0]
    assert val.shape == (heads, T, vdim) and y.shape == (T, heads * vdim) and val.dtype == g.dtype == y.dtype
    assert g.shape[1] == (heads if per_head else heads * vdim)
    _check(_lib("latent_attention").ff_latent_gate(_p(val), c_void_p(g.data_ptr()), c_int(g.stride(0)), c_int(_dt(y)),
                                                  _p(y), c_int(T), c_int(heads), c_int(vdim),
                                                  c_int(1 if per_head else 0), _stream()), "latent_gate")


# --------------------------------------------------------------------------- #
# routed experts (csrc/moe.cu)
MOE_FORCE_PLAIN = False     # tests flip this to hold the tensor-core grouped product against the plain one


def moe_on_tensor_cores(dtype: torch.dtype, k_sizes) -> bool:
    """True if a layer's grouped products run on the tensor-core kernel: bfloat16 and every K a multiple of 8."""
    return not MOE_FORCE_PLAIN and dtype == torch.bfloat16 and all(int(k) % 8 == 0 for k in k_sizes)


@functools.lru_cache(maxsize=None)
def moe_row_tile(tensor_cores: bool) -> int:
    """Rows of a row tile of the grouped product (the plan is made for the kernel that will run)."""
    return int(_lib("moe").ff_moe_row_tile(c_int(1 if tensor_cores else 0)))


ROUTE_SOFTMAX, ROUTE_SIGMOID = 0, 1            # how router logits become scores
GROUP_BY_BEST, GROUP_BY_TWO_BEST = 0, 1        # a group's score: its largest choice score, or the sum of its two largest
GLU_CLAMPED_SWISH, GLU_SILU = 0, 1             # an expert's activation


def moe_route(z, ids, wts, groups: int, keep: int, *, score: int = ROUTE_SOFTMAX, correction=None,
              group_score: int = GROUP_BY_BEST, renormalize: bool = True) -> None:
    """Choice of experts per token from router logits z float32 [T,E]: ids int32 [T,top], wts float32 [T,top].
    ``correction`` float32 [E]: added to the scores for the choice only (the weights are the plain scores)."""
    _need_cuda(z, ids, wts, correction)
    T, E = z.shape
    top = ids.shape[1]
    assert z.dtype == torch.float32 and ids.dtype == torch.int32 and wts.dtype == torch.float32 and wts.shape == ids.shape
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == E)
    _check(_lib("moe").ff_moe_route(_p(z), _p(correction), c_int(T), c_int(E), c_int(top), c_int(groups), c_int(keep),
                                   c_int(score), c_int(group_score), c_int(1 if renormalize else 0), _p(ids), _p(wts),
                                   _stream()), "moe_route")


def moe_max_tiles(entries: int, E: int, tensor_cores: bool = False) -> int:
    """The most row tiles `entries` rows spread over E experts can make."""
    return entries // moe_row_tile(bool(tensor_cores)) + min(E, entries)


def moe_plan(ids, E: int, seg, row_of, src_tok, tile_expert, tile_row0, n_tiles, tensor_cores: bool = False) -> None:
    """Sort the step's (token, choice) pairs by expert, on the device (all int32), and list the row tiles for
    the grouped kernel that will run (``tensor_cores``)."""
    _need_cuda(ids, seg, row_of, src_tok, tile_expert, tile_row0, n_tiles)
    T, top = ids.shape
    cap = moe_max_tiles(T * top, E, tensor_cores)
    assert seg.numel() >= E + 1 and row_of.numel() >= T * top and src_tok.numel() >= T * top
    assert tile_expert.numel() >= cap and tile_row0.numel() >= cap
    _check(_lib("moe").ff_moe_plan(_p(ids), c_int(T * top), c_int(top), c_int(E), c_int(moe_row_tile(bool(tensor_cores))),
                                  _p(seg), _p(row_of), _p(src_tok), _p(tile_expert), _p(tile_row0), _p(n_tiles),
                                  _stream()), "moe_plan")


def moe_grouped(a, src_tok, b0, b1, plan, out, limit: float = 0.0, tensor_cores: bool = False,
                act: int = GLU_CLAMPED_SWISH) -> None:
    """Grouped product over the experts' stacked matrices.  With ``b1`` (gate|up): rows of ``a`` [T,K] gathered
    by src_tok, b0/b1 [E,N,K], out[row] = g * sigmoid(1.702 g) * (u + 1) with the clamps of ``limit``
    (``act`` GLU_CLAMPED_SWISH) or silu(g) * u (GLU_SILU), in a's type.  Without: a [rows,K] in place, out float32 [rows,N].  ``plan`` = (seg, tile_expert, tile_row0, n_tiles,
    max_tiles), made with the same ``tensor_cores``: the mma.sync kernel (bfloat16, K % 8 == 0) or the plain one."""
    seg, tile_expert, tile_row0, n_tiles, max_tiles = plan
    _need_cuda(a, src_tok, b0, b1, out)
    E, N, Kd = b0.shape
    assert a.shape[1] == Kd and a.dtype == b0.dtype and out.shape[1] == N
    assert out.dtype == (a.dtype if b1 is not None else torch.float32)
    assert not tensor_cores or (a.dtype == torch.bfloat16 and Kd % 8 == 0)
    _check(_lib("moe").ff_moe_grouped(_p(a), _p(src_tok), _p(b0), _p(b1), c_int(_dt(a)), c_int(1 if b1 is not None else 0),
                                     _p(seg), _p(tile_expert), _p(tile_row0), _p(n_tiles), _p(out), c_int(max_tiles),
                                     c_int(N), c_int(Kd), c_float(limit), c_int(act),
                                     c_int(1 if tensor_cores else 0), _stream()), "moe_grouped")


def clamped_glu(gu, y, limit: float) -> None:
    """y = g * sigmoid(1.702 g) * (u + 1), g = min(gu[:, :F], limit), u = clamp(gu[:, F:], -limit, limit)."""
    _need_cuda(gu, y)
    T, F = y.shape
    assert gu.shape == (T, 2 * F) and gu.dtype == y.dtype
    _check(_lib("moe").ff_clamped_glu(_p(gu), _p(y), c_int(_dt(y)), c_int(T), c_int(F), c_float(limit), _stream()),
           "clamped_glu")


def moe_combine(residual, rows, row_of, wts, shared, mult: float) -> None:
    """residual[t] += mult * (sum_k wts[t,k] * rows[row_of[t,k]] + shared[t]); everything float32."""
    _need_cuda(residual, rows, row_of, wts, shared)
    T, W = residual.shape
    top = wts.shape[1]
    assert residual.dtype == rows.dtype == wts.dtype == torch.float32 and rows.shape[1] == W
    assert shared is None or (shared.dtype == torch.float32 and shared.shape == residual.shape)
    _check(_lib("moe").ff_moe_combine(_p(residual), _p(rows), _p(row_of), _p(wts), _p(shared), c_float(mult), c_int(T),
                                     c_int(top), c_int(W), _stream()), "moe_combine")


# --------------------------------------------------------------------------- #
# norms on a part's output, gated linear units with a choice of activation
def norm_add(residual: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float,
             copy: Optional[torch.Tensor] = None) -> None:
    """residual (float32 [T,H]) += rms_norm(delta) * weight, statistics and sum in 32-bit; ``copy`` [T,H]
    (any engine type) receives the updated rows."""
    _need_cuda(residual, delta, weight, copy)
    T, H = residual.shape
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == H
    assert delta.shape == residual.shape and (copy is None or copy.shape == residual.shape)
    _check(_lib("elementwise").ff_norm_add(_p(residual), _p(delta), c_int(_dt(delta)), _p(weight), c_float(eps), _p(copy),
                                          c_int(_dt(copy) if copy is not None else 0), c_int(T), c_int(H), _stream()),
           "norm_add")


GLU_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}


def glu_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str, bias: Optional[torch.Tensor] = None,
            limit: float = 0.0) -> None:
    """out[t,i] = act(g) * u with g = gate_up[t,i] (+ bias[i]) and u = gate_up[t,I+i] (+ bias[I+i]); act: "silu",
    "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))) or "clamped_swish"
    (min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1)).  ``bias`` float32 [2I]."""
    _need_cuda(gate_up, out, bias)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype == out.dtype
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * I)
    _check(_lib("elementwise").ff_glu_act(_p(gate_up), _p(bias), _p(out), c_int(_dt(out)), c_int(T), c_int(I),
                                         c_int(GLU_ACTIVATIONS[activation]), c_float(limit), _stream()), "glu_act")


def act_mul_table_rows(g: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, col0: int, out: torch.Tensor,
                       activation: str, status: torch.Tensor) -> None:
    """out[t, j] = act(g[t, j]) * table[ids[t], col0 + j] for the n columns of ``g``; act "silu" or "gelu_tanh"."""
    _need_cuda(g, ids, table, out, status)
    T, n = g.shape
    assert g.dtype == table.dtype == out.dtype and out.shape == g.shape and g.is_contiguous() and out.is_contiguous()
    assert ids.dtype == torch.int32 and ids.numel() == T and table.is_contiguous() and col0 + n <= table.shape[1]
    _check(_lib("elementwise").ff_act_mul_table_rows(
        _p(g), _p(ids), _p(table), c_int(table.shape[1]), c_int(col0), c_int(table.shape[0]), _p(out), c_int(_dt(out)),
        c_int(T), c_int(n), c_int({"silu": 0, "gelu_tanh": 1}[activation]), _p(status), _stream()), "act_mul_table_rows")


def scale_(x: torch.Tensor, a: float) -> None:
    """x *= a for a contiguous float32 tensor."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(_lib("elementwise").ff_scale(_p(x), c_float(a), c_size_t(x.numel()), _stream()), "scale")


def rope_unit_norm_store(qkv: torch.Tensor, nq: int, nkv: int, d: int, norm_dim: int, eps: float, freq: torch.Tensor,
                         mag: float, ctx, block_table: Optional[torch.Tensor], cache: Optional[torch.Tensor], *,
                         interleaved: bool = False, normalize: bool = True, bias: Optional[torch.Tensor] = None) -> None:
    """Heads whose unit norm comes behind the rotation: q and k heads of ``qkv`` [T, (nq + 2 nkv) d] are turned
    (their first 2 * len(freq) elements; cos and sin times ``mag``), divided by their root mean square over
    ``norm_dim`` elements, q written back in place, k and v into the paged cache [blocks, 2, nkv, block, d].
    ``nkv == 0``: q only.  ``interleaved``: element 2i turns with element 2i + 1 (else i with i + len(freq));
    ``normalize`` False: no unit norm; ``bias`` float32 [(nq + 2 nkv) d]: added to q, k and v first, in 32-bit."""
    _need_cuda(qkv, freq, block_table, cache, bias)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == (nq + 2 * nkv) * d and bias.is_contiguous()
    T, width = qkv.shape
    assert freq.dtype == torch.float64 and width == (nq + 2 * nkv) * d
    if nkv:
        num_blocks, two, ckv, block_size, cd = cache.shape
        assert two == 2 and ckv == nkv and cd == d and cache.dtype == qkv.dtype
        max_blocks = block_table.shape[1]
    else:
        num_blocks = block_size = max_blocks = 1
    _check(_lib("head_finish").ff_rope_unit_norm_store(
        _p(qkv), c_int(_dt(qkv)), c_int(width), c_int(T), c_int(nq), c_int(nkv), c_int(d), c_int(norm_dim), c_float(eps),
        _p(freq), c_int(2 * freq.numel()), c_float(mag), _p(ctx.positions), _p(ctx.token_seq), _p(block_table),
        c_int(max_blocks), c_int(block_size), c_int(num_blocks), _p(cache), _p(ctx.status),
        c_int(1 if interleaved else 0), c_int(1 if normalize else 0), _p(bias), _stream()),
        "rope_unit_norm_store")


# --------------------------------------------------------------------------- #
# recurrences with one scalar decay per head and token (csrc/ssm.cu)
SCAN_MAX_KEY, SCAN_MAX_VALUE = 256, 256


def scan_plan(N: int, V: int):
    """(key size the kernel is built for, threads that share a value column, blocks a head's columns are split
    over, columns a block, threads a block): the recurrence kernel's layout for key size N and value size V
    (the twin of `scan_plan` in csrc/ssm.cu; `scan_state_floats_of_kernel` is the kernel's own figure)."""
    if not (0 < N <= SCAN_MAX_KEY and 0 < V <= SCAN_MAX_VALUE):
        raise KernelError(f"recurrence: key size {N} / value size {V} not supported "
                          f"(up to {SCAN_MAX_KEY} / {SCAN_MAX_VALUE})")
    pad = 16 if N <= 16 else (32 if N <= 32 else (64 if N <= 64 else (128 if N <= 128 else 256)))
    parts = 8 if pad >= 32 else 4
    max_cols = 512 // parts
    vsplit = -(-V // max_cols)
    vb = -(-V // vsplit)
    return pad, parts, vsplit, vb, -(-(vb * parts) // 32) * 32


def scan_state_floats(heads: int, N: int, V: int) -> int:
    """Floats of a request's state for `heads` heads of key size N and value size V, in the recurrence
    kernel's own layout (sizes rounded up to what the kernel is instantiated for)."""
    pad, parts, vsplit, _, threads = scan_plan(N, V)
    return heads * vsplit * (pad // parts) * threads


def scan_state_floats_of_kernel(heads: int, N: int, V: int) -> int:
    fn = _lib("ssm").ff_scan_state_floats
    fn.restype = ctypes.c_longlong
    return int(fn(c_int(heads), c_int(N), c_int(V)))


def causal_conv_silu(x: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: torch.Tensor,
                     state: torch.Tensor, conv_off: int, ctx, out: torch.Tensor) -> None:
    """out[t,c] = silu(bias[c] + sum_j weight[c,j] * x[t - (taps-1) + j, col0 + c]) along each sequence; the inputs
    in front of a portion come from the request's state slot ([taps-1, channels] floats at ``conv_off``, zeros for
    a fresh request), which is then brought up to date."""
    _need_cuda(x, weight, bias, state, out)
    T = x.shape[0]
    taps = weight.shape[1]
    assert weight.dtype == bias.dtype == state.dtype == torch.float32 and weight.shape[0] == channels == bias.numel()
    assert out.shape == (T, channels) and out.dtype == x.dtype and state.dim() == 2
    assert state.shape[1] >= conv_off + (taps - 1) * channels
    _check(_lib("ssm").ff_causal_conv_silu(
        _p(x), c_int(_dt(x)), c_int(x.stride(0)), c_int(col0), _p(weight), _p(bias), _p(state),
        ctypes.c_longlong(state.stride(0)), c_int(conv_off), _p(ctx.token_seq), _p(ctx.cu_q), _p(ctx.state_slots),
        _p(ctx.seq_fresh), _p(out), c_int(T), c_int(ctx.num_seqs), c_int(channels), c_int(taps), _stream()),
        "causal_conv_silu")
    global LAUNCHES
    if taps > 1:
        LAUNCHES += 1     # the kernel that saves the last inputs


CONV_SILU, CONV_ADD_INPUT = 1, 2


def causal_conv(x: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                state: torch.Tensor, conv_off: int, ctx, out: torch.Tensor, *, silu: bool = False,
                add_input: bool = False) -> None:
    """`causal_conv_silu` with the activation and the bias as options: out[t,c] = act(bias[c] + sum_j weight[c,j] *
    x[t - (taps-1) + j, col0 + c]) (+ x[t, col0 + c] with ``add_input``).  ``out`` may be of the engine's type while
    ``x`` is 32-bit."""
    _need_cuda(x, weight, bias, state, out)
    T = x.shape[0]
    taps = weight.shape[1]
    assert weight.dtype == state.dtype == torch.float32 and weight.shape[0] == channels and state.dim() == 2
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == channels)
    assert out.shape == (T, channels) and (out.dtype == x.dtype or x.dtype == torch.float32)
    assert state.shape[1] >= conv_off + (taps - 1) * channels
    _check(_lib("ssm").ff_causal_conv(
        _p(x), c_int(_dt(x)), c_int(x.stride(0)), c_int(col0), _p(weight), _p(bias), _p(state),
        ctypes.c_longlong(state.stride(0)), c_int(conv_off), _p(ctx.token_seq), _p(ctx.cu_q), _p(ctx.state_slots),
        _p(ctx.seq_fresh), _p(out), c_int(_dt(out)), c_int(T), c_int(ctx.num_seqs), c_int(channels), c_int(taps),
        c_int((CONV_SILU if silu else 0) | (CONV_ADD_INPUT if add_input else 0)), _stream()), "causal_conv")
    global LAUNCHES
    if taps > 1:
        LAUNCHES += 1     # the kernel that saves the last inputs


def conv_state_update(x: torch.Tensor, col0: int, channels: int, taps: int, state: torch.Tensor, conv_off: int, ctx) -> None:
    """The last taps-1 rows of x[:, col0 : col0 + channels] of every sequence into its state slot ([taps-1, channels]
    floats at ``conv_off``), for a part that convolves inside a kernel of its own."""
    _need_cuda(x, state)
    assert state.dtype == torch.float32 and state.shape[1] >= conv_off + (taps - 1) * channels
    if taps <= 1:
        return
    _check(_lib("ssm").ff_conv_state_update(
        _p(x), c_int(_dt(x)), c_int(x.stride(0)), c_int(col0), _p(state), ctypes.c_longlong(state.stride(0)),
        c_int(conv_off), _p(ctx.cu_q), _p(ctx.state_slots), _p(ctx.seq_fresh), c_int(ctx.num_seqs), c_int(channels),
        c_int(taps), _stream()), "conv_state_update")


# --------------------------------------------------------------------------- #
# attention heads behind a short convolution and a norm over the whole projection (csrc/conv_attention.cu)
def conv_norm_store(proj: torch.Tensor, col0: int, conv_w: torch.Tensor, q_norm_w: torch.Tensor, k_norm_w: torch.Tensor,
                    eps: float, state: torch.Tensor, conv_off: int, ctx, table: torch.Tensor, pages: torch.Tensor,
                    q_out: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int, d: int, *, mix: int = 0,
                    mix_factor: Optional[torch.Tensor] = None, shared: Optional[torch.Tensor] = None,
                    conv_w_t: Optional[torch.Tensor] = None) -> None:
    """q | k | v from column ``col0`` of ``proj`` pass a causal convolution per channel (``conv_w`` [C, taps], no bias,
    the inputs in front of a portion from the state slot), q and k an RMS norm over their whole projection with the
    weights given; q goes to ``q_out`` [T, heads * d], k and v into ``pages`` [blocks, 2, kv_heads, block, d] (heads
    filled up to d with zeros).  ``mix`` 1: the values are also kept in ``shared`` float32 [T, kv_heads * dv];
    2: v <- (1 - f) v + f shared with f = ``mix_factor`` (one float32 on the device).  The state is not updated
    here (`conv_state_update`).  ``conv_w_t``: the weights once more as [taps, C]; the bfloat16 kernel for sizes in
    steps of 8 reads those."""
    _need_cuda(proj, conv_w, q_norm_w, k_norm_w, state, table, pages, q_out, mix_factor, shared, conv_w_t)
    T = proj.shape[0]
    C = heads * dk + kv_heads * (dk + dv)
    taps = conv_w.shape[1]
    num_blocks, two, ckv, block_size, cd = pages.shape
    assert two == 2 and ckv == kv_heads and cd == d and pages.dtype == proj.dtype == q_out.dtype
    assert conv_w.shape[0] == C and conv_w.dtype == torch.float32 and conv_w.is_contiguous()
    assert q_norm_w.numel() == heads * dk and k_norm_w.numel() == kv_heads * dk and q_out.shape == (T, heads * d)
    assert state.dtype == torch.float32 and state.shape[1] >= conv_off + (taps - 1) * C
    assert shared is None or (shared.dtype == torch.float32 and shared.shape == (T, kv_heads * dv))
    assert conv_w_t is None or (conv_w_t.shape == (taps, C) and conv_w_t.dtype == torch.float32 and conv_w_t.is_contiguous())
    _check(_lib("conv_attention").ff_conv_norm_store(
        _p(proj), c_int(_dt(proj)), c_int(proj.stride(0)), c_int(col0), _p(conv_w), _p(q_norm_w), _p(k_norm_w), _p(state),
        ctypes.c_longlong(state.stride(0)), c_int(conv_off), _p(ctx.token_seq), _p(ctx.cu_q), _p(ctx.positions),
        _p(ctx.state_slots), _p(ctx.seq_fresh), _p(table), c_int(table.shape[1]), c_int(block_size), c_int(num_blocks),
        c_int(T), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv), c_int(d), c_int(taps), c_float(eps), c_int(mix),
        _p(mix_factor), _p(shared), _p(q_out), _p(pages), _p(ctx.status), _p(conv_w_t), _stream()), "conv_norm_store")


def head_gate(att: torch.Tensor, gate, y: torch.Tensor, heads: int, d: int, dv: int) -> None:
    """y[t, h*dv + i] = att[t, h*d + i] * sigmoid(g[t, h*dv + i]) for i < dv; ``gate`` = (matrix, first column)."""
    gm, g0 = gate
    _need_cuda(att, gm, y)
    T = y.shape[0]
    assert att.shape == (T, heads * d) and y.shape == (T, heads * dv) and att.dtype == gm.dtype == y.dtype
    assert att.is_contiguous() and gm.stride(1) == 1
    _check(_lib("conv_attention").ff_head_gate(_p(att), _p(gm), c_int(gm.stride(0)), c_int(g0), c_int(_dt(y)), _p(y),
                                              c_int(T), c_int(heads), c_int(d), c_int(dv), _stream()), "head_gate")


# --------------------------------------------------------------------------- #
# the gated delta rule with a decay per key channel (csrc/delta_rule.cu)
def delta_plan(N: int, V: int):
    """(key size the kernel is built for, threads that share a value column, blocks a head's columns are split over,
    columns a block, threads a block): the twin of `delta_plan` in csrc/delta_rule.cu (`delta_state_floats` is the
    kernel's own figure)."""
    if not (0 < N <= 256 and 0 < V <= 256):
        raise KernelError(f"delta rule: key size {N} / value size {V} not supported (up to 256 each)")
    pad = 16 if N <= 16 else (32 if N <= 32 else (64 if N <= 64 else (128 if N <= 128 else 256)))
    parts = 16 if pad >= 128 else (8 if pad >= 32 else 4)
    vj = 2 if pad >= 128 else 1                 # value columns a thread
    max_cols = 512 // parts * vj
    vsplit = -(-V // max_cols)
    vb = -(-V // vsplit)
    return pad, parts, vsplit, vb, -(-(-(-vb // vj) * parts) // 32) * 32


def delta_state_floats_plan(heads: int, N: int, V: int) -> int:
    """Floats of a request's state for `heads` heads of key size N and value size V (worked out on the host)."""
    pad, parts, vsplit, _, threads = delta_plan(N, V)
    return heads * vsplit * (pad // parts) * (2 if pad >= 128 else 1) * threads


def delta_state_floats(heads: int, N: int, V: int) -> int:
    """Floats of a request's state for `heads` heads of key size N and value size V, in the kernel's own layout."""
    fn = _lib("delta_rule").ff_delta_state_floats
    fn.restype = ctypes.c_longlong
    n = int(fn(c_int(heads), c_int(N), c_int(V)))
    if n < 0:
        raise KernelError(f"delta rule: key size {N} / value size {V} not supported (up to 256 each)")
    return n


def delta_rule_scan(q, k, v, beta, a, dt_bias: torch.Tensor, a_log: torch.Tensor, state: torch.Tensor, state_off: int,
                    ctx, o: torch.Tensor, heads: int, N: int, V: int, *, heads_per_group: int = 1, q_scale: float = 1.0,
                    unit_eps: float = 1e-6, decay_per_head: bool = False) -> None:
    """S = diag(g) S; u = beta (v - S^T k); S += k u^T; o = S^T q per head, token by token.  ``q``, ``k``, ``v``,
    ``beta``, ``a``: (matrix [T, *], first column); a q/k row holds [groups, N] (made unit vectors here, q also times
    ``q_scale``), a v row [heads, V], a beta row [heads] (its sigmoid is taken here), an ``a`` row float32
    [heads, N] with g = exp(-exp(a_log) softplus(a + dt_bias)) (``decay_per_head``: an ``a`` row is [heads], dt_bias
    [heads], and a head's key channels all decay alike).  ``state`` float32 [slots, *]: `delta_state_floats`
    floats from ``state_off``; o float32 [T, heads * V]."""
    (qm, q0), (km, k0), (vm, v0), (bm, b0), (am, a0) = q, k, v, beta, a
    _need_cuda(qm, km, vm, bm, am, dt_bias, a_log, state, o)
    T = o.shape[0]
    assert qm.dtype == km.dtype == vm.dtype == bm.dtype and am.dtype == torch.float32
    assert all(m.stride(1) == 1 for m in (qm, km, vm, bm, am))
    assert dt_bias.dtype == a_log.dtype == torch.float32 and a_log.numel() == heads
    assert dt_bias.numel() == (heads if decay_per_head else heads * N)
    assert o.dtype == torch.float32 and o.shape == (T, heads * V) and state.dtype == torch.float32
    _check(_lib("delta_rule").ff_delta_rule_scan(
        _p(qm), c_int(qm.stride(0)), c_int(q0), _p(km), c_int(km.stride(0)), c_int(k0), _p(vm), c_int(vm.stride(0)),
        c_int(v0), _p(bm), c_int(bm.stride(0)), c_int(b0), c_int(_dt(qm)), _p(am), c_int(am.stride(0)), c_int(a0),
        _p(dt_bias), _p(a_log), c_int(1 if decay_per_head else 0), c_int(heads_per_group), c_float(q_scale), c_float(unit_eps), _p(state),
        ctypes.c_longlong(state.stride(0)), c_int(state_off), _p(ctx.cu_q), _p(ctx.state_slots), _p(ctx.seq_fresh),
        _p(o), c_int(T), c_int(ctx.num_seqs), c_int(heads), c_int(N), c_int(V), _stream()), "delta_rule_scan")


def head_norm_gate(o: torch.Tensor, gate, weight: torch.Tensor, eps: float, y: torch.Tensor, heads: int, V: int,
                   gate_activation: str = "sigmoid") -> None:
    """y[t, h, :] = rms_norm(o[t, h, :]) * weight * act(g[t, h, :]): the norm over each head's V values, one weight
    row [V] for all heads; ``gate`` = (float32 matrix, first column); act = "sigmoid" or "silu"."""
    gm, g0 = gate
    _need_cuda(o, gm, weight, y)
    T = o.shape[0]
    assert o.dtype == gm.dtype == weight.dtype == torch.float32 and weight.numel() == V and gm.stride(1) == 1
    assert o.shape == (T, heads * V) and y.shape == o.shape and o.is_contiguous() and y.is_contiguous()
    _check(_lib("delta_rule").ff_head_norm_gate(_p(o), _p(gm), c_int(gm.stride(0)), c_int(g0), _p(weight), c_float(eps),
                                               _p(y), c_int(_dt(y)), c_int(T), c_int(heads), c_int(V),
                                               c_int({"sigmoid": 0, "silu": 1}[gate_activation]), _stream()),
           "head_norm_gate")


def scalar_decay_scan(q, k, v, state: torch.Tensor, state_off: int, ctx, o: torch.Tensor, heads: int, N: int, V: int, *,
                      heads_per_group: int = 1, silu_inputs: bool = False, decay: Optional[torch.Tensor] = None,
                      step=None, step_bias=None, a_log=None, skip=None) -> None:
    """S = a S + b k v^T, o = S^T q (+ skip * v) per head, token by token, one block per (sequence, head).
    ``q``, ``k``, ``v``: (matrix [T, *], first column); a q/k row holds [groups, N], a v row [heads, V].
    Either ``decay`` float32 [heads] (a constant, b = 1) or ``step`` = (matrix, first column) with ``step_bias``,
    ``a_log``, ``skip`` float32 [heads]: s = softplus(step + bias), a = exp(-exp(a_log) s), b = s.
    ``state`` float32 [slots, *]: `scan_state_floats` floats from ``state_off``; o float32 [T, heads * V]."""
    (qm, q0), (km, k0), (vm, v0) = q, k, v
    _need_cuda(state, o, decay, step_bias, a_log, skip)
    T = o.shape[0]
    assert qm.dtype == km.dtype == vm.dtype and qm.stride(1) == km.stride(1) == vm.stride(1) == 1
    assert o.dtype == torch.float32 and o.shape == (T, heads * V) and state.dtype == torch.float32
    assert state.shape[1] >= state_off + scan_state_floats(heads, N, V)
    mode = 0 if decay is not None else 1
    sm, s0 = step if step is not None else (None, 0)
    if mode == 1:
        assert sm.dtype == qm.dtype and step_bias is not None and a_log is not None
    _check(_lib("ssm").ff_scalar_decay_scan(
        _p(qm), c_int(qm.stride(0)), c_int(q0), _p(km), c_int(km.stride(0)), c_int(k0), _p(vm), c_int(vm.stride(0)),
        c_int(v0), c_int(_dt(qm)), c_int(heads_per_group), c_int(1 if silu_inputs else 0), c_int(mode), _p(decay),
        _p(sm), c_int(sm.stride(0) if sm is not None else 0), c_int(s0), _p(step_bias), _p(a_log), _p(skip), _p(state),
        ctypes.c_longlong(state.stride(0)), c_int(state_off), _p(ctx.cu_q), _p(ctx.state_slots), _p(ctx.seq_fresh),
        _p(o), c_int(T), c_int(ctx.num_seqs), c_int(heads), c_int(N), c_int(V), _stream()), "scalar_decay_scan")


def gated_rms_norm(o: torch.Tensor, gate, weight: torch.Tensor, eps: float, y: torch.Tensor, parts: int,
                   gate_first: bool) -> None:
    """``gate_first``: y = rms_norm(o * silu(g)) * weight, the norm over each of ``parts`` equal parts of a row;
    else y = rms_norm(o) * weight * sigmoid(g).  o float32 [T, width]; ``gate`` = (matrix, first column)."""
    gm, g0 = gate
    _need_cuda(o, weight, y)
    T, width = o.shape
    assert o.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == width
    assert y.shape == o.shape and y.dtype == gm.dtype and gm.stride(1) == 1
    _check(_lib("ssm").ff_gated_rms_norm(_p(o), _p(gm), c_int(_dt(gm)), c_int(gm.stride(0)), c_int(g0), _p(weight),
                                        c_float(eps), _p(y), c_int(T), c_int(width), c_int(parts),
                                        c_int(0 if gate_first else 1), _stream()), "gated_rms_norm")
