// A recurrent mixer that corrects its state by the error of its own prediction (the gated delta rule), with a
// decay per head and key channel (or one per head: `decay_per_head`, the raw decay inputs are then rows of
// [heads] and dt_bias has one entry a head; g_t[i] is the same for every key channel i):
//
//   S_t   = diag(g_t) S_(t-1)                         S: [key channel, value channel] per head, 32-bit, starts at 0
//   u_t   = beta_t (v_t - S_t^T k_t)
//   S_t  += k_t u_t^T
//   o_t   = S_t^T q_t                                  (the read-out sees the token's own write)
//         = (diag(g_t) S_(t-1))^T q_t + u_t (k_t . q_t)      the form the kernel uses: both sums over key channels in one walk
//
// with q and k made unit vectors per head on the way in (x / sqrt(sum x^2 + unit_eps), q also times q_scale),
// beta_t = sigmoid(raw beta) and g_t[i] = exp(-exp(A_log_h) * softplus(a_t[i] + dt_bias[i])).  Everything behind
// the projections is 32-bit.  The state lives in the request's state slot and is carried from step to step; a
// fresh request starts from zeros.  A sequence's tokens are walked in order with the same order of additions
// however the prompt was cut into steps.
//
// One block per (sequence, head, share of the value columns).  Value column j is held by PARTS neighbouring
// threads, each with NP / PARTS key channels of column j in registers; the two sums over key channels of a
// token (the prediction and the read-out) are joined over those threads by shuffles.  For keys of 128 and more a
// thread holds the same key channels of two neighbouring columns: what it reads of the staged q, k and g serves
// both, and a head needs half the blocks.
#include "common.cuh"

namespace ff {

__device__ __forceinline__ float dr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct DeltaArgs {
    const void* q; int q_stride, q_off;          // rows of [groups, N]
    const void* k; int k_stride, k_off;
    const void* v; int v_stride, v_off;          // rows of [heads, V]
    const void* beta; int beta_stride, beta_off; // raw, rows of [heads]
    const float* a; int a_stride, a_off;         // raw decay inputs, rows of [heads, N], 32-bit
    const float* dt_bias;                        // [heads * N]
    const float* a_log;                          // [heads]
    int heads_per_group;
    float q_scale, unit_eps;
    int decay_per_head;                          // 1: `a` rows of [heads], dt_bias [heads]
};

constexpr int DR_CHUNK = 8;
constexpr int DR_AHEAD = 2;     // elements of a chunk's inputs a thread may hold for the chunk to come
constexpr int DR_MAX_THREADS = 512;

struct DeltaPlan { int NP, PARTS, VJ, vsplit, Vb, threads; };
static inline bool delta_plan(int N, int V, DeltaPlan* p) {
    if (N <= 0 || N > 256 || V <= 0 || V > 256) return false;
    p->NP = N <= 16 ? 16 : (N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256)));
    p->PARTS = p->NP >= 128 ? 16 : (p->NP >= 32 ? 8 : 4);
    p->VJ = p->NP >= 128 ? 2 : 1;              // value columns a thread: long keys share their staged q, k, g over two
    const int max_cols = DR_MAX_THREADS / p->PARTS * p->VJ;
    p->vsplit = (V + max_cols - 1) / max_cols;
    p->Vb = (V + p->vsplit - 1) / p->vsplit;
    p->threads = (((p->Vb + p->VJ - 1) / p->VJ * p->PARTS + 31) / 32) * 32;
    return true;
}

template <typename T, int NP, int PARTS, int VJ>
__global__ void __launch_bounds__(DR_MAX_THREADS) delta_rule_scan_kernel(
    DeltaArgs A, float* __restrict__ state, size_t state_stride, int state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, const int* __restrict__ seq_fresh, float* __restrict__ o /*[T, heads*V]*/,
    int heads, int N, int V, int Vb) {
    pdl_prologue();
    constexpr int KP = NP / PARTS;
    constexpr int CH = NP >= 256 ? DR_CHUNK : 2 * DR_CHUNK;     // tokens staged at a time (shared memory bounds the longest keys)
    constexpr int AH = NP >= 256 ? DR_AHEAD : 2 * DR_AHEAD;
    static_assert(KP % 4 == 0, "a thread reads its key channels four at a time");
    __shared__ __align__(16) float s_q[CH][NP], s_k[CH][NP], s_g[CH][NP];
    __shared__ float s_v[CH][128];
    __shared__ float s_b[CH], s_kq[CH];
    const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    const int jl = tid / PARTS, part = tid % PARTS;
    const int j0 = blockIdx.z * Vb;                       // the block's first column; the thread's are j0 + jl * VJ + x
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    bool live[VJ];
#pragma unroll
    for (int x = 0; x < VJ; ++x) live[x] = jl * VJ + x < Vb && j0 + jl * VJ + x < V;
    const bool fresh = seq_fresh[s] != 0;
    // a block's share of a head's state is kept as its threads hold it: register (x, i) of thread tid at
    // (x * KP + i) * threads + tid
    float* S_g = state + (size_t)state_slots[s] * state_stride + state_off +
                 ((size_t)h * gridDim.z + blockIdx.z) * KP * VJ * nthr;
    float S[VJ][KP];
#pragma unroll
    for (int x = 0; x < VJ; ++x) {
#pragma unroll
        for (int i = 0; i < KP; ++i) S[x][i] = fresh ? 0.f : S_g[(size_t)(x * KP + i) * nthr + tid];
    }
    const int group = h / A.heads_per_group;
    const T* qp = pdl_fresh((const T*)A.q) + A.q_off + (size_t)group * N;
    const T* kp = pdl_fresh((const T*)A.k) + A.k_off + (size_t)group * N;
    const T* vp = pdl_fresh((const T*)A.v) + A.v_off + (size_t)h * V + j0;
    const T* bp = pdl_fresh((const T*)A.beta) + A.beta_off + h;
    const int an = A.decay_per_head ? 0 : 1;            // 0: every key channel reads the head's one decay input
    const float* ap = pdl_fresh(A.a) + A.a_off + (A.decay_per_head ? (size_t)h : (size_t)h * N);
    const float* dtb = A.dt_bias + (A.decay_per_head ? (size_t)h : (size_t)h * N);
    const int cols = min(Vb, V - j0);
    const float rate = expf(A.a_log[h]);
    // Where a chunk's inputs are at most AH elements a thread, the next chunk's are asked for (into registers)
    // before the current chunk's tokens are walked, so that their way from memory passes under the recurrence.
    const bool ahead = CH * NP <= AH * nthr && CH * cols <= AH * nthr;
    T nq[AH], nk[AH], nv[AH], nb = from_float<T>(0.f);
    float na[AH];
    auto ask = [&](int c0) {
        const int n = min(CH, t1 - c0);
#pragma unroll
        for (int r = 0; r < AH; ++r) {
            const int idx = tid + r * nthr, c = idx / NP, i = idx - c * NP;
            const bool in = idx < CH * NP && c < n && i < N;
            nq[r] = in ? qp[(size_t)(c0 + c) * A.q_stride + i] : from_float<T>(0.f);
            nk[r] = in ? kp[(size_t)(c0 + c) * A.k_stride + i] : from_float<T>(0.f);
            na[r] = in ? ap[(size_t)(c0 + c) * A.a_stride + i * an] : 0.f;
            const int cv = idx / cols, jj = idx - cv * cols;
            nv[r] = (idx < CH * cols && cv < n) ? vp[(size_t)(c0 + cv) * A.v_stride + jj] : from_float<T>(0.f);
        }
        nb = tid < n ? bp[(size_t)(c0 + tid) * A.beta_stride] : from_float<T>(0.f);
    };
    if (ahead && t0 < t1) ask(t0);
    for (int c0 = t0; c0 < t1; c0 += CH) {
        const int n = min(CH, t1 - c0);
        __syncthreads();
        // staging: the chunk's q, k (raw), decays, v and beta in 32-bit
        if (ahead) {
#pragma unroll
            for (int r = 0; r < AH; ++r) {
                const int idx = tid + r * nthr, c = idx / NP, i = idx - c * NP;
                if (idx < CH * NP) {
                    const bool in = c < n && i < N;
                    s_q[c][i] = to_float(nq[r]);
                    s_k[c][i] = to_float(nk[r]);
                    s_g[c][i] = in ? expf(-rate * dr_softplus(na[r] + dtb[i * an])) : 0.f;
                }
                if (idx < CH * cols) s_v[idx / cols][idx % cols] = to_float(nv[r]);
            }
            if (tid < CH) s_b[tid] = tid < n ? 1.0f / (1.0f + expf(-to_float(nb))) : 0.f;
            if (c0 + CH < t1) ask(c0 + CH);
        } else {
        for (int idx = tid; idx < CH * NP; idx += nthr) {
            const int c = idx / NP, i = idx - c * NP;
            float qv = 0.f, kv = 0.f, gv = 0.f;
            if (c < n && i < N) {
                qv = to_float(qp[(size_t)(c0 + c) * A.q_stride + i]);
                kv = to_float(kp[(size_t)(c0 + c) * A.k_stride + i]);
                gv = expf(-rate * dr_softplus(ap[(size_t)(c0 + c) * A.a_stride + i * an] + dtb[i * an]));
            }
            s_q[c][i] = qv;
            s_k[c][i] = kv;
            s_g[c][i] = gv;
        }
        for (int idx = tid; idx < CH * cols; idx += nthr) {
            const int c = idx / cols, jj = idx - c * cols;
            s_v[c][jj] = c < n ? to_float(vp[(size_t)(c0 + c) * A.v_stride + jj]) : 0.f;
        }
        if (tid < CH)
            s_b[tid] = tid < n ? 1.0f / (1.0f + expf(-to_float(bp[(size_t)(c0 + tid) * A.beta_stride]))) : 0.f;
        }
        __syncthreads();
        // unit vectors: a warp per token
        for (int c = warp; c < n; c += nwarps) {
            float sq = 0.f, sk = 0.f, kq = 0.f;
            for (int i = lane; i < NP; i += 32) {
                sq += s_q[c][i] * s_q[c][i];
                sk += s_k[c][i] * s_k[c][i];
                kq += s_q[c][i] * s_k[c][i];
            }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            kq = warp_sum(kq);
            const float fq = A.q_scale / sqrtf(sq + A.unit_eps), fk = 1.0f / sqrtf(sk + A.unit_eps);
            for (int i = lane; i < NP; i += 32) { s_q[c][i] *= fq; s_k[c][i] *= fk; }
            if (lane == 0) s_kq[c] = kq * fq * fk;
        }
        __syncthreads();
#pragma unroll 1
        for (int c = 0; c < n; ++c) {
            float vj[VJ];
#pragma unroll
            for (int x = 0; x < VJ; ++x) vj[x] = live[x] ? s_v[c][jl * VJ + x] : 0.f;
            const float beta = s_b[c];
            // one walk over the decayed state gives both sums over key channels: the prediction S^T k and the
            // read-out of the state before the write, S^T q; the write k u^T then adds u (k . q) to the read-out
            float d[VJ][4], a[VJ][4];
#pragma unroll
            for (int x = 0; x < VJ; ++x) {
#pragma unroll
                for (int e = 0; e < 4; ++e) { d[x][e] = 0.f; a[x][e] = 0.f; }
            }
#pragma unroll
            for (int i = 0; i < KP; i += 4) {
                // thread `part` holds key channels 4 PARTS m + 4 part + e (m = i / 4, e < 4)
                const int at = i * PARTS + part * 4;
                const float4 g4 = *reinterpret_cast<const float4*>(&s_g[c][at]);
                const float4 k4 = *reinterpret_cast<const float4*>(&s_k[c][at]);
                const float4 q4 = *reinterpret_cast<const float4*>(&s_q[c][at]);
#pragma unroll
                for (int x = 0; x < VJ; ++x) {
                    S[x][i]     *= g4.x;  d[x][0] += k4.x * S[x][i];      a[x][0] += q4.x * S[x][i];
                    S[x][i + 1] *= g4.y;  d[x][1] += k4.y * S[x][i + 1];  a[x][1] += q4.y * S[x][i + 1];
                    S[x][i + 2] *= g4.z;  d[x][2] += k4.z * S[x][i + 2];  a[x][2] += q4.z * S[x][i + 2];
                    S[x][i + 3] *= g4.w;  d[x][3] += k4.w * S[x][i + 3];  a[x][3] += q4.w * S[x][i + 3];
                }
            }
            float dot[VJ], acc[VJ];
#pragma unroll
            for (int x = 0; x < VJ; ++x) {
                dot[x] = (d[x][0] + d[x][1]) + (d[x][2] + d[x][3]);
                acc[x] = (a[x][0] + a[x][1]) + (a[x][2] + a[x][3]);
            }
#pragma unroll
            for (int off = 1; off < PARTS; off <<= 1) {
#pragma unroll
                for (int x = 0; x < VJ; ++x) {
                    dot[x] += __shfl_xor_sync(0xffffffffu, dot[x], off);
                    acc[x] += __shfl_xor_sync(0xffffffffu, acc[x], off);
                }
            }
            float u[VJ];
#pragma unroll
            for (int x = 0; x < VJ; ++x) {
                u[x] = beta * (vj[x] - dot[x]);
                acc[x] += u[x] * s_kq[c];
            }
#pragma unroll
            for (int i = 0; i < KP; i += 4) {
                const int at = i * PARTS + part * 4;
                const float4 k4 = *reinterpret_cast<const float4*>(&s_k[c][at]);
#pragma unroll
                for (int x = 0; x < VJ; ++x) {
                    S[x][i]     += k4.x * u[x];
                    S[x][i + 1] += k4.y * u[x];
                    S[x][i + 2] += k4.z * u[x];
                    S[x][i + 3] += k4.w * u[x];
                }
            }
            if (part == 0) {
#pragma unroll
                for (int x = 0; x < VJ; ++x)
                    if (live[x]) o[(size_t)(c0 + c) * heads * V + (size_t)h * V + j0 + jl * VJ + x] = acc[x];
            }
        }
    }
#pragma unroll
    for (int x = 0; x < VJ; ++x) {
#pragma unroll
        for (int i = 0; i < KP; ++i) S_g[(size_t)(x * KP + i) * nthr + tid] = S[x][i];
    }
}

// y[t, h*V + i] = o[t, h*V + i] / sqrt(mean_i o[t, h, :]^2 + eps) * w[i] * act(gate[t, gate_off + h*V + i]):
// a norm over each head's values with one weight row for all heads, then a gate, act = sigmoid (gate_act 0) or
// SiLU (gate_act 1).  One warp per (token, head).
template <typename T>
__global__ void head_norm_gate_kernel(const float* o, const float* gate, int gate_stride, int gate_off,
                                      const float* __restrict__ w, float eps, T* __restrict__ y, int rows, int heads, int V,
                                      int gate_act) {
    pdl_prologue();
    o = pdl_fresh(o);
    gate = pdl_fresh(gate);
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int t = row / heads, h = row - t * heads;
    const float* orow = o + (size_t)row * V;
    const float* grow = gate + (size_t)t * gate_stride + gate_off + (size_t)h * V;
    float ss = 0.f;
    for (int i = lane; i < V; i += 32) ss += orow[i] * orow[i];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)V + eps);
    for (int i = lane; i < V; i += 32) {
        const float g = grow[i], sg = 1.0f / (1.0f + expf(-g));
        y[(size_t)row * V + i] = from_float<T>(orow[i] * inv * w[i] * (gate_act ? g * sg : sg));
    }
}

}  // namespace ff

using namespace ff;

// floats of a request's state for `heads` heads of key size N and value size V (-1: sizes not supported)
FF_EXPORT long long ff_delta_state_floats(int heads, int N, int V) {
    DeltaPlan p;
    if (!delta_plan(N, V, &p)) return -1;
    return (long long)heads * p.vsplit * (p.NP / p.PARTS) * p.VJ * p.threads;
}

template <typename T>
static int delta_launch(const DeltaArgs& A, float* state, long long state_stride, int state_off, const int* cu_q,
                        const int* state_slots, const int* seq_fresh, float* o, int n_seqs, int heads, int N, int V,
                        cudaStream_t stream) {
    DeltaPlan p;
    if (!delta_plan(N, V, &p)) return FF_ERR_UNSUPPORTED;
    if (p.Vb > 128) return FF_ERR_UNSUPPORTED;
    dim3 grid(n_seqs, heads, p.vsplit);
#define FF_DELTA(NP, PARTS, VJ)                                                                                    \
    FF_LAUNCH((delta_rule_scan_kernel<T, NP, PARTS, VJ>), grid, p.threads, 0, stream, A, state, (size_t)state_stride, \
              state_off, cu_q, state_slots, seq_fresh, o, heads, N, V, p.Vb)
    switch (p.NP) {
        case 16: FF_DELTA(16, 4, 1); break;
        case 32: FF_DELTA(32, 8, 1); break;
        case 64: FF_DELTA(64, 8, 1); break;
        case 128: FF_DELTA(128, 16, 2); break;
        case 256: FF_DELTA(256, 16, 2); break;
        default: return FF_ERR_UNSUPPORTED;
    }
#undef FF_DELTA
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_delta_rule_scan(const void* q, int q_stride, int q_off, const void* k, int k_stride, int k_off,
                                 const void* v, int v_stride, int v_off, const void* beta, int beta_stride, int beta_off,
                                 int dtype, const float* a, int a_stride, int a_off, const float* dt_bias,
                                 const float* a_log, int decay_per_head, int heads_per_group, float q_scale, float unit_eps, float* state,
                                 long long state_stride, int state_off, const int* cu_q, const int* state_slots,
                                 const int* seq_fresh, float* o, int T, int n_seqs, int heads, int N, int V,
                                 cudaStream_t stream) {
    if (T <= 0 || n_seqs <= 0) return 0;
    if (heads_per_group <= 0 || heads % heads_per_group) return FF_ERR_BAD_ARG;
    DeltaArgs A{q, q_stride, q_off, k, k_stride, k_off, v, v_stride, v_off, beta, beta_stride, beta_off,
                a, a_stride, a_off, dt_bias, a_log, heads_per_group, q_scale, unit_eps, decay_per_head ? 1 : 0};
    if (dtype == 0)
        return delta_launch<float>(A, state, state_stride, state_off, cu_q, state_slots, seq_fresh, o, n_seqs, heads, N, V, stream);
    if (dtype == 1)
        return delta_launch<bf16>(A, state, state_stride, state_off, cu_q, state_slots, seq_fresh, o, n_seqs, heads, N, V, stream);
    return FF_ERR_BAD_ARG;
}

FF_EXPORT int ff_head_norm_gate(const float* o, const float* gate, int gate_stride, int gate_off, const float* w, float eps,
                                void* y, int dtype, int T, int heads, int V, int gate_act, cudaStream_t stream) {
    const int rows = T * heads;
    if (rows <= 0) return 0;
    const int warps = 4;
    const unsigned blocks = (unsigned)((rows + warps - 1) / warps);
    if (dtype == 0)
        FF_LAUNCH((head_norm_gate_kernel<float>), blocks, warps * 32, 0, stream, o, gate, gate_stride, gate_off, w, eps, (float*)y, rows, heads, V, gate_act);
    else if (dtype == 1)
        FF_LAUNCH((head_norm_gate_kernel<bf16>), blocks, warps * 32, 0, stream, o, gate, gate_stride, gate_off, w, eps, (bf16*)y, rows, heads, V, gate_act);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
