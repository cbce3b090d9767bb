// Recurrent mixers whose state decays by one scalar per head and token:
//
//   S_t = a_t S_(t-1) + b_t k_t v_t^T        S: [key channel, value channel] per head, 32-bit, starts at 0
//   o_t = S_t^T q_t  (+ D v_t)
//
// Two designs use it.  A state-space mixer (Mamba-2 style): k = B_t and q = C_t (shared by the heads of a
// group), v = x_t, step = softplus(raw_t + bias), a_t = exp(-exp(A_log) step), b_t = step, with a skip
// term D x_t; its inputs x, B, C come out of a short causal convolution per channel with SiLU
// (`causal_conv_silu_kernel`), whose last taps-1 inputs are part of the request's state.  And linear
// attention with a constant decay per head: a = decay_h, b = 1, q, k, v = SiLU of three projections.
//
// The state lives in the request's state slot in 32-bit and is carried from step to step; a fresh request
// starts from zeros.  Decays, steps, S and every sum are 32-bit.  A sequence's tokens are walked in order
// with the same order of additions however the prompt was cut into steps.
#include "common.cuh"

namespace ff {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ----------------------------------------------------------------------------- convolution --
// out[t, c] = act(bias[c] + sum_j w[c, j] * in[t - (taps-1) + j, c]) (+ in[t, c]); inputs in front of the portion
// come from the state slot (`conv_off`: [(taps-1), C] floats, oldest first; zeros for a fresh request).
// `flags`: CONV_SILU the activation is SiLU (else none), CONV_ADD_INPUT the token's own input is added to the
// result (a filter whose output is x + conv(x)).  `bias` may be null.  The output type TO may differ from the
// input's (32-bit rows in, rows of the engine's type out).
// A thread takes VEC neighbouring channels (one 16-byte load where the layout allows it, else one channel)
// and walks `tile` tokens with the last taps-1 inputs in registers, so every input of a long step is read once
// (steps of few tokens get a thread a token, so that they still fill the GPU).
constexpr int CONV_MAX_TAPS = 16;
constexpr int CONV_SILU = 1, CONV_ADD_INPUT = 2;

// TAPS > 0: the number of taps is known when the kernel is built (the window stays in registers); 0: any number
// up to CONV_MAX_TAPS.
template <typename T, typename TO, int VEC, int TAPS>
__global__ void causal_conv_silu_kernel(const T* in, int in_stride, int in_off,
                                        const float* __restrict__ w /*[C,taps]*/, const float* __restrict__ bias,
                                        const float* state, size_t state_stride, int conv_off,
                                        const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                                        const int* __restrict__ state_slots, const int* __restrict__ seq_fresh,
                                        TO* __restrict__ out /*[T,C]*/, int Ttot, int C, int taps_rt, int tile,
                                        int flags) {
    pdl_prologue();
    in = pdl_fresh(in);
    state = pdl_fresh(state);
    constexpr int MT = TAPS ? TAPS : CONV_MAX_TAPS;
    const int taps = TAPS ? TAPS : taps_rt;
    const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
    if (c0 >= C) return;
    const int tile0 = blockIdx.x * tile, tile1 = min(Ttot, tile0 + tile);
    float win[MT > 1 ? MT - 1 : 1][VEC];          // the inputs of the taps-1 tokens in front, oldest first
    float wt[MT][VEC], bs[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        bs[e] = bias ? bias[c0 + e] : 0.f;
#pragma unroll
        for (int j = 0; j < MT; ++j) wt[j][e] = j < taps ? w[(size_t)(c0 + e) * taps + j] : 0.f;
    }
    auto load_row = [&](int tt, float* dst) {           // the inputs of token tt (a row of this step)
        const T* src = in + (size_t)tt * in_stride + in_off + c0;
        if constexpr (VEC == 1) dst[0] = to_float(src[0]);
        else {
            const uint4 raw = *reinterpret_cast<const uint4*>(src);
            const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int e = 0; e < VEC; ++e) dst[e] = to_float(v[e]);
        }
    };
    // the window in front of token t of sequence s: rows of this step where they exist, else the saved rows
    auto fill_window = [&](int t, int s) {
        const int t0 = cu_q[s];
        const bool fresh = seq_fresh[s] != 0;
        const float* st = state + (size_t)state_slots[s] * state_stride + conv_off;
#pragma unroll
        for (int j = 0; j < MT - 1; ++j) {
            if (j < taps - 1) {
                const int tt = t - (taps - 1) + j;
                if (tt >= t0) load_row(tt, win[j]);
                else {
                    const int r = (taps - 1) + (tt - t0);       // row of the saved inputs: 0 oldest
#pragma unroll
                    for (int e = 0; e < VEC; ++e) win[j][e] = fresh ? 0.f : st[(size_t)r * C + c0 + e];
                }
            }
        }
    };
    int s_prev = -1;
    for (int t = tile0; t < tile1; ++t) {
        const int s = token_seq[t];
        if (t == tile0 || s != s_prev) fill_window(t, s);
        s_prev = s;
        float cur[VEC], acc[VEC];
        load_row(t, cur);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = bs[e];
#pragma unroll
        for (int j = 0; j < MT - 1; ++j)
            if (j < taps - 1) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] += wt[j][e] * win[j][e];
            }
#pragma unroll
        for (int j = 0; j < MT; ++j)
            if (j == taps - 1) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] += wt[j][e] * cur[e];
            }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            if (flags & CONV_SILU) acc[e] = silu_f(acc[e]);
            if (flags & CONV_ADD_INPUT) acc[e] += cur[e];
        }
        TO* dst = out + (size_t)t * C + c0;
        if constexpr (VEC == 1) dst[0] = from_float<TO>(acc[0]);
        else {
            struct alignas(VEC * sizeof(TO)) Pack { TO v[VEC]; };
            Pack raw;
#pragma unroll
            for (int e = 0; e < VEC; ++e) raw.v[e] = from_float<TO>(acc[e]);
            *reinterpret_cast<Pack*>(dst) = raw;
        }
        // slide: the oldest row leaves, the current one comes in
#pragma unroll
        for (int j = 0; j < MT - 1; ++j) {
            if (j < taps - 2) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) win[j][e] = win[j + 1][e];
            } else if (j == taps - 2) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) win[j][e] = cur[e];
            }
        }
    }
}

// The last taps-1 inputs of every sequence, for its next step.  One thread per (sequence, channel) reads what
// it needs of the old rows before it writes.
template <typename T>
__global__ void conv_state_update_kernel(const T* in, int in_stride, int in_off, float* __restrict__ state,
                                         size_t state_stride, int conv_off, const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slots, const int* __restrict__ seq_fresh,
                                         int C, int taps) {
    pdl_prologue();
    in = pdl_fresh(in);
    constexpr int MAX_KEEP = 15;
    const int s = blockIdx.x;
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    const int keep = taps - 1, n = t1 - t0;
    if (n <= 0) return;
    const bool fresh = seq_fresh[s] != 0;
    float* st = state + (size_t)state_slots[s] * state_stride + conv_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float nv[MAX_KEEP];
#pragma unroll
        for (int r = 0; r < MAX_KEEP; ++r) {
            if (r < keep) {
                const int tt = t1 - keep + r;
                if (tt >= t0) nv[r] = to_float(in[(size_t)tt * in_stride + in_off + c]);
                else nv[r] = fresh ? 0.f : st[(size_t)(keep + (tt - t0)) * C + c];
            }
        }
#pragma unroll
        for (int r = 0; r < MAX_KEEP; ++r)
            if (r < keep) st[(size_t)r * C + c] = nv[r];
    }
}

// ----------------------------------------------------------------------------- the recurrence --
struct ScanArgs {
    const void* q; int q_stride, q_off;          // [T, ...] key-sized rows per group: q_off + group * N + i
    const void* k; int k_stride, k_off;
    const void* v; int v_stride, v_off;          // value rows per head: v_off + h * V + j
    int heads_per_group;                         // heads that share one q/k row (1: a row per head)
    int act;                                     // 1: q, k, v pass SiLU as they are read
    const float* decay;                          // [heads] constant a (mode 0)
    const void* step; int step_stride, step_off; // mode 1: raw step per (token, head)
    const float* step_bias; const float* a_log; const float* skip;   // [heads] each (mode 1; skip may be null)
    int mode;
};

constexpr int SCAN_CHUNK = 8;
constexpr int SCAN_MAX_THREADS = 512;

// How the recurrence is laid out for key size N and value size V: the key size it is instantiated for (NP),
// the threads that share a value column (PARTS, each with NP / PARTS key channels in registers), over how many
// blocks a head's value columns are split (vsplit, Vb columns each) and the threads of a block.  A token costs a
// thread NP / PARTS steps of a serial chain, so long keys get many threads a column and the columns of a head go
// to several blocks.  (Sixteen threads a column were tried for keys of 128: a head of 64 columns then needs two
// blocks of 512 threads, eight sequences of 32 heads no longer fit the GPU at once, and the prompt pass was slower.)
struct ScanPlan { int NP, PARTS, vsplit, Vb, threads; };
static inline bool scan_plan(int N, int V, ScanPlan* p) {
    if (N <= 0 || N > 256 || V <= 0 || V > 256) return false;
    p->NP = N <= 16 ? 16 : (N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256)));
    p->PARTS = p->NP >= 32 ? 8 : 4;
    const int max_cols = SCAN_MAX_THREADS / p->PARTS;
    p->vsplit = (V + max_cols - 1) / max_cols;
    p->Vb = (V + p->vsplit - 1) / p->vsplit;
    p->threads = ((p->Vb * p->PARTS + 31) / 32) * 32;
    return true;
}

// One block per (sequence, head, share of the value columns).  Value column j is held by PARTS neighbouring
// threads, each with NP / PARTS key channels of column j in registers.
// PF: the next chunk's inputs are asked for (into registers) before the current chunk is computed, so their
// latency hides behind the recurrence; it needs a block with enough threads for SCAN_PFQ q and k values and
// SCAN_PFV v values each a chunk (the launcher checks), else the chunk is staged when it is needed.
constexpr int SCAN_PFQ = 2, SCAN_PFV = 1;

template <typename T, int NP, int PARTS, bool PF>
__global__ void __launch_bounds__(SCAN_MAX_THREADS, 2) scalar_decay_scan_kernel(
    ScanArgs A, float* __restrict__ state, size_t state_stride, int state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, const int* __restrict__ seq_fresh, float* __restrict__ o /*[T, heads*V]*/,
    int heads, int N, int V, int Vb) {
    pdl_prologue();
    constexpr int KP = NP / PARTS;
    static_assert(KP % 4 == 0, "a thread reads its key channels four at a time");
    __shared__ __align__(16) float s_q[SCAN_CHUNK][NP], s_k[SCAN_CHUNK][NP];
    __shared__ float s_v[SCAN_CHUNK][128];
    __shared__ float s_a[SCAN_CHUNK], s_d[SCAN_CHUNK];
    const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x;
    const int jl = tid / PARTS, part = tid % PARTS;
    const int j0 = blockIdx.z * Vb, j = j0 + jl;
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    const bool live = jl < Vb && j < V;
    const bool fresh = seq_fresh[s] != 0;
    // a block's share of a head's state is kept as its threads hold it: register i of thread tid at i * threads + tid
    float* S_g = state + (size_t)state_slots[s] * state_stride + state_off +
                 ((size_t)h * gridDim.z + blockIdx.z) * KP * nthr;
    float S[KP];
#pragma unroll
    for (int i = 0; i < KP; ++i) S[i] = fresh ? 0.f : S_g[(size_t)i * nthr + tid];
    const int group = h / A.heads_per_group;
    const T* qp = pdl_fresh((const T*)A.q) + A.q_off + (size_t)group * N;
    const T* kp = pdl_fresh((const T*)A.k) + A.k_off + (size_t)group * N;
    const T* vp = pdl_fresh((const T*)A.v) + A.v_off + (size_t)h * V + j0;
    const T* stepp = pdl_fresh((const T*)A.step);
    const int cols = min(Vb, V - j0);
    float a_const = 1.f, rate = 0.f, sbias = 0.f, skip = 0.f;
    if (A.mode == 0) a_const = A.decay[h];
    else { rate = expf(A.a_log[h]); sbias = A.step_bias[h]; skip = A.skip ? A.skip[h] : 0.f; }
    // the values a thread stages: element u of a thread is flat index tid + u * threads of the chunk's [8][NP] or [8][cols]
    float rq[PF ? SCAN_PFQ : 1], rk[PF ? SCAN_PFQ : 1], rv[PF ? SCAN_PFV : 1], rstep = 0.f;
    auto fetch = [&](int c0) {
        const int n = min(SCAN_CHUNK, t1 - c0);
#pragma unroll
        for (int u = 0; u < SCAN_PFQ; ++u) {
            const int idx = tid + u * nthr, c = idx / NP, i = idx - c * NP;
            const bool ok = idx < SCAN_CHUNK * NP && c < n && i < N;
            rq[u] = ok ? to_float(qp[(size_t)(c0 + c) * A.q_stride + i]) : 0.f;
            rk[u] = ok ? to_float(kp[(size_t)(c0 + c) * A.k_stride + i]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < SCAN_PFV; ++u) {
            const int idx = tid + u * nthr, c = idx / cols, jj = idx - c * cols;
            rv[u] = (idx < SCAN_CHUNK * cols && c < n) ? to_float(vp[(size_t)(c0 + c) * A.v_stride + jj]) : 0.f;
        }
        if (A.mode == 1 && tid < n) rstep = to_float(stepp[(size_t)(c0 + tid) * A.step_stride + A.step_off + h]);
    };
    if constexpr (PF) fetch(t0);
    for (int c0 = t0; c0 < t1; c0 += SCAN_CHUNK) {
        const int n = min(SCAN_CHUNK, t1 - c0);
        __syncthreads();
        // staging: the chunk's q, k, v, decays and input scales in 32-bit
        if (tid < SCAN_CHUNK) {
            float a = a_const, b = 1.f;
            if (A.mode == 1 && tid < n) {
                const float raw = PF ? rstep : to_float(stepp[(size_t)(c0 + tid) * A.step_stride + A.step_off + h]);
                const float dt = softplus_f(raw + sbias);
                a = expf(-rate * dt);
                b = dt;
            }
            s_a[tid] = a;
            s_d[tid] = b;
        }
        if constexpr (PF) {
#pragma unroll
            for (int u = 0; u < SCAN_PFQ; ++u) {
                const int idx = tid + u * nthr;
                if (idx < SCAN_CHUNK * NP) {
                    (&s_q[0][0])[idx] = A.act ? silu_f(rq[u]) : rq[u];
                    (&s_k[0][0])[idx] = A.act ? silu_f(rk[u]) : rk[u];
                }
            }
#pragma unroll
            for (int u = 0; u < SCAN_PFV; ++u) {
                const int idx = tid + u * nthr, c = idx / cols, jj = idx - c * cols;
                if (idx < SCAN_CHUNK * cols) s_v[c][jj] = A.act ? silu_f(rv[u]) : rv[u];
            }
        } else {
            for (int idx = tid; idx < SCAN_CHUNK * NP; idx += nthr) {
                const int c = idx / NP, i = idx - c * NP;
                float qv = 0.f, kv = 0.f;
                if (c < n && i < N) {
                    qv = to_float(qp[(size_t)(c0 + c) * A.q_stride + i]);
                    kv = to_float(kp[(size_t)(c0 + c) * A.k_stride + i]);
                    if (A.act) { qv = silu_f(qv); kv = silu_f(kv); }
                }
                s_q[c][i] = qv;
                s_k[c][i] = kv;
            }
            for (int idx = tid; idx < SCAN_CHUNK * cols; idx += nthr) {
                const int c = idx / cols, jj = idx - c * cols;
                float vv = 0.f;
                if (c < n) {
                    vv = to_float(vp[(size_t)(c0 + c) * A.v_stride + jj]);
                    if (A.act) vv = silu_f(vv);
                }
                s_v[c][jj] = vv;
            }
        }
        __syncthreads();
        if constexpr (PF) {
            if (c0 + SCAN_CHUNK < t1) fetch(c0 + SCAN_CHUNK);
        }
#pragma unroll
        for (int c = 0; c < SCAN_CHUNK; ++c) {
            if (c < n) {
                const float vj = live ? s_v[c][jl] : 0.f;
                const float a = s_a[c], bv = s_d[c] * vj;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int i = 0; i < KP; i += 4) {
                    // thread `part` holds key channels 4 PARTS m + 4 part + e (m = i / 4, e < 4)
                    const int at = i * PARTS + part * 4;
                    const float4 q4 = *reinterpret_cast<const float4*>(&s_q[c][at]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&s_k[c][at]);
                    S[i]     = a * S[i]     + k4.x * bv;  a0 += q4.x * S[i];
                    S[i + 1] = a * S[i + 1] + k4.y * bv;  a1 += q4.y * S[i + 1];
                    S[i + 2] = a * S[i + 2] + k4.z * bv;  a2 += q4.z * S[i + 2];
                    S[i + 3] = a * S[i + 3] + k4.w * bv;  a3 += q4.w * S[i + 3];
                }
                float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
                for (int off = 1; off < PARTS; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                if (live && part == 0) o[(size_t)(c0 + c) * heads * V + (size_t)h * V + j] = acc + skip * vj;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < KP; ++i) S_g[(size_t)i * nthr + tid] = S[i];
}

// ----------------------------------------------------------------------------- gate and norm --
// One block per (token, part).  order 0: y = rms(o * silu(z)) * w  (the gate in front of the norm, norm over
// each of `parts` equal parts);  order 1: y = rms(o) * w * sigmoid(z)  (the gate behind it).
template <typename T>
__global__ void gated_rms_norm_kernel(const float* o, const T* z, int z_stride, int z_off,
                                      const float* __restrict__ w, float eps, T* __restrict__ y, int width, int parts,
                                      int order) {
    pdl_prologue();
    o = pdl_fresh(o);
    z = pdl_fresh(z);
    __shared__ float scratch[32];
    const int t = blockIdx.x, g = blockIdx.y;
    const int per = width / parts;
    const float* orow = o + (size_t)t * width + (size_t)g * per;
    const T* zrow = z + (size_t)t * z_stride + z_off + (size_t)g * per;
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        float v = orow[i];
        if (order == 0) v *= silu_f(to_float(zrow[i]));
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)per + eps);
    T* yrow = y + (size_t)t * width + (size_t)g * per;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const float zv = to_float(zrow[i]);
        float v = orow[i];
        if (order == 0) v = v * silu_f(zv) * inv * w[g * per + i];
        else v = v * inv * w[g * per + i] / (1.0f + expf(-zv));
        yrow[i] = from_float<T>(v);
    }
}

}  // namespace ff

using namespace ff;

template <typename T, typename TO>
static int conv_launch(const void* in, int in_stride, int in_off, const float* w, const float* bias, float* state,
                       long long state_stride, int conv_off, const int* token_seq, const int* cu_q, const int* state_slots,
                       const int* seq_fresh, void* out, int T_, int n_seqs, int C, int taps, int flags,
                       cudaStream_t stream) {
    constexpr int V = 16 / (int)sizeof(T);
    const bool vec = taps >= 2 && taps <= 4 && C % V == 0 && in_off % V == 0 && in_stride % V == 0 &&
                     (((uintptr_t)in | (uintptr_t)out) & 15) == 0;
    const int per = vec ? V : 1;
    const int lanes = (C + per - 1) / per;
    const int threads = lanes >= 128 ? 128 : ((lanes + 31) / 32) * 32;
    const int tile = T_ >= 4096 ? 16 : (T_ >= 512 ? 4 : 1);
    dim3 grid((T_ + tile - 1) / tile, (lanes + threads - 1) / threads);
#define FF_CONV(VV, TT)                                                                                              \
    FF_LAUNCH((causal_conv_silu_kernel<T, TO, VV, TT>), grid, threads, 0, stream, (const T*)in, in_stride, in_off, w, bias, \
              (const float*)state, (size_t)state_stride, conv_off, token_seq, cu_q, state_slots, seq_fresh, (TO*)out, T_, C, taps, \
              tile, flags)
    if (vec) {
        switch (taps) {
            case 2: FF_CONV(V, 2); break;
            case 3: FF_CONV(V, 3); break;
            case 4: FF_CONV(V, 4); break;
            default: return FF_ERR_BAD_ARG;      // not reached: `vec` holds only for 2 to 4 taps
        }
    } else {
        switch (taps) {
            case 2: FF_CONV(1, 2); break;
            case 3: FF_CONV(1, 3); break;
            case 4: FF_CONV(1, 4); break;
            default: FF_CONV(1, 0); break;
        }
    }
#undef FF_CONV
    if (taps > 1) {
        const int cy = min(64, (C + 255) / 256);
        FF_LAUNCH((conv_state_update_kernel<T>), dim3(n_seqs, cy), 256, 0, stream, (const T*)in, in_stride, in_off, state,
                  (size_t)state_stride, conv_off, cu_q, state_slots, seq_fresh, C, taps);
    }
    FF_LAUNCH_CHECK();
    return 0;
}

// `out_dtype`: the type of `out` (the input's, or the engine's type for 32-bit input rows).
FF_EXPORT int ff_causal_conv(const void* in, int dtype, int in_stride, int in_off, const float* w, const float* bias,
                             float* state, long long state_stride, int conv_off, const int* token_seq,
                             const int* cu_q, const int* state_slots, const int* seq_fresh, void* out, int out_dtype,
                             int T, int n_seqs, int C, int taps, int flags, cudaStream_t stream) {
    if (T <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS) return FF_ERR_UNSUPPORTED;
#define FF_CONV_TYPES(TI, TOUT)                                                                                          \
    return conv_launch<TI, TOUT>(in, in_stride, in_off, w, bias, state, state_stride, conv_off, token_seq, cu_q, state_slots, \
                                 seq_fresh, out, T, n_seqs, C, taps, flags, stream)
    if (dtype == 0 && out_dtype == 0) FF_CONV_TYPES(float, float);
    if (dtype == 1 && out_dtype == 1) FF_CONV_TYPES(bf16, bf16);
    if (dtype == 0 && out_dtype == 1) FF_CONV_TYPES(float, bf16);
#undef FF_CONV_TYPES
    return FF_ERR_BAD_ARG;
}

FF_EXPORT int ff_causal_conv_silu(const void* in, int dtype, int in_stride, int in_off, const float* w, const float* bias,
                                  float* state, long long state_stride, int conv_off, const int* token_seq,
                                  const int* cu_q, const int* state_slots, const int* seq_fresh, void* out, int T,
                                  int n_seqs, int C, int taps, cudaStream_t stream) {
    return ff_causal_conv(in, dtype, in_stride, in_off, w, bias, state, state_stride, conv_off, token_seq, cu_q, state_slots,
                          seq_fresh, out, dtype, T, n_seqs, C, taps, CONV_SILU, stream);
}

// Only the second half of the convolution: the last taps-1 rows of `in` of every sequence go into its state
// slot, for a part that convolves inside a kernel of its own.
FF_EXPORT int ff_conv_state_update(const void* in, int dtype, int in_stride, int in_off, float* state, long long state_stride,
                                   int conv_off, const int* cu_q, const int* state_slots, const int* seq_fresh, int n_seqs,
                                   int C, int taps, cudaStream_t stream) {
    if (n_seqs <= 0 || C <= 0 || taps <= 1) return 0;
    if (taps > CONV_MAX_TAPS) return FF_ERR_UNSUPPORTED;
    const int cy = min(64, (C + 255) / 256);
    if (dtype == 0)
        FF_LAUNCH((conv_state_update_kernel<float>), dim3(n_seqs, cy), 256, 0, stream, (const float*)in, in_stride, in_off, state,
                  (size_t)state_stride, conv_off, cu_q, state_slots, seq_fresh, C, taps);
    else if (dtype == 1)
        FF_LAUNCH((conv_state_update_kernel<bf16>), dim3(n_seqs, cy), 256, 0, stream, (const bf16*)in, in_stride, in_off, state,
                  (size_t)state_stride, conv_off, cu_q, state_slots, seq_fresh, C, taps);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

// floats of a request's state for `heads` heads of key size N and value size V (-1: sizes not supported)
FF_EXPORT long long ff_scan_state_floats(int heads, int N, int V) {
    ScanPlan p;
    if (!scan_plan(N, V, &p)) return -1;
    return (long long)heads * p.vsplit * (p.NP / p.PARTS) * p.threads;
}

template <typename T>
static int scan_launch(const ScanArgs& A, float* state, long long state_stride, int state_off, const int* cu_q,
                       const int* state_slots, const int* seq_fresh, float* o, int n_seqs, int heads, int N, int V,
                       cudaStream_t stream) {
    ScanPlan p;
    if (!scan_plan(N, V, &p)) return FF_ERR_UNSUPPORTED;
    dim3 grid(n_seqs, heads, p.vsplit);
    const bool pf = SCAN_CHUNK * p.NP <= SCAN_PFQ * p.threads && SCAN_CHUNK * p.Vb <= SCAN_PFV * p.threads;
#define FF_SCAN(NP, PARTS)                                                                                              \
    do {                                                                                                                \
        if (pf)                                                                                                         \
            FF_LAUNCH((scalar_decay_scan_kernel<T, NP, PARTS, true>), grid, p.threads, 0, stream, A, state,             \
                      (size_t)state_stride, state_off, cu_q, state_slots, seq_fresh, o, heads, N, V, p.Vb);             \
        else                                                                                                            \
            FF_LAUNCH((scalar_decay_scan_kernel<T, NP, PARTS, false>), grid, p.threads, 0, stream, A, state,            \
                      (size_t)state_stride, state_off, cu_q, state_slots, seq_fresh, o, heads, N, V, p.Vb);             \
    } while (0)
    switch (p.NP) {
        case 16: FF_SCAN(16, 4); break;
        case 32: FF_SCAN(32, 8); break;
        case 64: FF_SCAN(64, 8); break;
        case 128: FF_SCAN(128, 8); break;
        case 256: FF_SCAN(256, 8); break;
        default: return FF_ERR_UNSUPPORTED;
    }
#undef FF_SCAN
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_scalar_decay_scan(const void* q, int q_stride, int q_off, const void* k, int k_stride, int k_off,
                                   const void* v, int v_stride, int v_off, int dtype, int heads_per_group, int act,
                                   int mode, const float* decay, const void* step, int step_stride, int step_off,
                                   const float* step_bias, const float* a_log, const float* skip, float* state,
                                   long long state_stride, int state_off, const int* cu_q, const int* state_slots,
                                   const int* seq_fresh, float* o, int T, int n_seqs, int heads, int N, int V,
                                   cudaStream_t stream) {
    if (T <= 0 || n_seqs <= 0) return 0;
    if (heads_per_group <= 0 || (mode != 0 && mode != 1)) return FF_ERR_BAD_ARG;
    ScanArgs A{q, q_stride, q_off, k, k_stride, k_off, v, v_stride, v_off, heads_per_group, act, decay,
               step, step_stride, step_off, step_bias, a_log, skip, mode};
    if (dtype == 0)
        return scan_launch<float>(A, state, state_stride, state_off, cu_q, state_slots, seq_fresh, o, n_seqs, heads, N, V, stream);
    if (dtype == 1)
        return scan_launch<bf16>(A, state, state_stride, state_off, cu_q, state_slots, seq_fresh, o, n_seqs, heads, N, V, stream);
    return FF_ERR_BAD_ARG;
}

FF_EXPORT int ff_gated_rms_norm(const float* o, const void* z, int dtype, int z_stride, int z_off, const float* w,
                                float eps, void* y, int T, int width, int parts, int order, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (parts <= 0 || width % parts || (order != 0 && order != 1)) return FF_ERR_BAD_ARG;
    const int per = width / parts;
    const int threads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
    if (dtype == 0)
        FF_LAUNCH((gated_rms_norm_kernel<float>), dim3(T, parts), threads, 0, stream, o, (const float*)z, z_stride, z_off, w, eps,
                  (float*)y, width, parts, order);
    else if (dtype == 1)
        FF_LAUNCH((gated_rms_norm_kernel<bf16>), dim3(T, parts), threads, 0, stream, o, (const bf16*)z, z_stride, z_off, w, eps,
                  (bf16*)y, width, parts, order);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
