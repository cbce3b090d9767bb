// Preparation of attention heads whose projections pass a short causal convolution and a norm over the whole
// projection, and the gate on the attention's output:
//
//   u      = [q | k | v] rows of the projection (Cq, Ck, Cv channels)
//   y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]                  zeros in front of the sequence, no bias
//   q      = y_q / sqrt(mean(y_q^2) + eps) * wq                       the mean over all Cq channels (all heads at once)
//   k      = y_k / sqrt(mean(y_k^2) + eps) * wk                       likewise over all Ck channels
//   v      = y_v, or (1 - lambda) y_v + lambda * shared_t             (values blended with another layer's of the same token)
//
// q goes to a buffer of heads of `d` elements (the attention kernels' head size; a true head size below d is
// filled up with zeros), k and v into the paged cache [blocks, 2, G, block, d].  The inputs in front of a
// portion come from the request's state slot ([taps-1, C] floats, oldest first; zeros for a fresh request);
// bringing that up to date is the convolution module's kernel.  The convolution, both norms and the blend are
// 32-bit; only what is stored is rounded.  One block per token.
#include "common.cuh"

namespace ff {

constexpr int CA_MAX_TAPS = 16;

struct ConvHeadArgs {
    const void* proj; int stride, col0;          // q | k | v from column col0
    const float* w;                              // [C, taps]
    const float* w_t;                            // the same transposed, [taps, C], or null (the 16-byte form reads this one)
    int T;
    const float* wq; const float* wk;            // [Cq], [Ck]
    const float* state; long long state_stride; int conv_off;
    const int* token_seq; const int* cu_q; const int* positions; const int* state_slots; const int* seq_fresh;
    const int* block_table; int max_blocks, block_size, num_blocks;
    int H, G, dk, dv, d, taps;
    float eps;
    int mix;                                     // 0: values as they are; 1: also kept in `shared`; 2: blended with `shared`
    const float* lambda;                         // one float on the device (mix 2)
    float* shared;                               // [T, G * dv] floats
    int* status;
};

template <typename T>
__global__ void conv_norm_store_kernel(ConvHeadArgs A, T* __restrict__ q_out /*[T, H*d]*/, T* __restrict__ cache) {
    pdl_prologue();
    extern __shared__ float y[];                  // [C]
    __shared__ float scratch[32];
    const T* proj = pdl_fresh((const T*)A.proj);
    const float* state = pdl_fresh(A.state);
    const float* shared_in = pdl_fresh((const float*)A.shared);
    const int t = blockIdx.x;
    const int Cq = A.H * A.dk, Ck = A.G * A.dk, Cv = A.G * A.dv, C = Cq + Ck + Cv;
    const int s = A.token_seq[t], t0 = A.cu_q[s], pos = A.positions[t];
    const bool fresh = A.seq_fresh[s] != 0;
    const float* st = state + (size_t)A.state_slots[s] * A.state_stride + A.conv_off;
    const int keep = A.taps - 1;
    float ssq_q = 0.f, ssq_k = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < A.taps; ++j) {
            const int tt = t - keep + j;
            float u;
            if (tt >= t0) u = to_float(proj[(size_t)tt * A.stride + A.col0 + c]);
            else u = fresh ? 0.f : st[(size_t)(keep + (tt - t0)) * C + c];
            acc += A.w[(size_t)c * A.taps + j] * u;
        }
        y[c] = acc;
        if (c < Cq) ssq_q += acc * acc;
        else if (c < Cq + Ck) ssq_k += acc * acc;
    }
    ssq_q = block_sum(ssq_q, scratch);
    ssq_k = block_sum(ssq_k, scratch);
    __syncthreads();
    const float inv_q = 1.0f / sqrtf(ssq_q / (float)Cq + A.eps);
    const float inv_k = 1.0f / sqrtf(ssq_k / (float)Ck + A.eps);
    // q rows, heads filled up to d
    T* qrow = q_out + (size_t)t * A.H * A.d;
    for (int idx = threadIdx.x; idx < A.H * A.d; idx += blockDim.x) {
        const int h = idx / A.d, i = idx - h * A.d;
        float v = 0.f;
        if (i < A.dk) { const int c = h * A.dk + i; v = y[c] * inv_q * A.wq[c]; }
        qrow[idx] = from_float<T>(v);
    }
    // k and v into the token's cache row
    const int page = A.block_table[(size_t)s * A.max_blocks + pos / A.block_size];
    if (page < 0 || page >= A.num_blocks) {
        if (threadIdx.x == 0) atomicExch(A.status, 3);
        return;
    }
    const float lam = A.mix == 2 ? A.lambda[0] : 0.f;
    const size_t plane = (size_t)A.G * A.block_size * A.d;
    T* krow0 = cache + (size_t)page * 2 * plane + (size_t)(pos % A.block_size) * A.d;
    for (int idx = threadIdx.x; idx < A.G * A.d; idx += blockDim.x) {
        const int g = idx / A.d, i = idx - g * A.d;
        float kv = 0.f, vv = 0.f;
        if (i < A.dk) { const int c = g * A.dk + i; kv = y[Cq + c] * inv_k * A.wk[c]; }
        if (i < A.dv) {
            const int c = g * A.dv + i;
            vv = y[Cq + Ck + c];
            if (A.mix == 1) A.shared[(size_t)t * Cv + c] = vv;
            else if (A.mix == 2) vv = (1.0f - lam) * vv + lam * shared_in[(size_t)t * Cv + c];
        }
        T* kdst = krow0 + (size_t)g * A.block_size * A.d + i;
        kdst[0] = from_float<T>(kv);
        kdst[plane] = from_float<T>(vv);
    }
}

// The bfloat16 form for sizes in steps of 8 (dk, dv, d, the projection's stride and first column; at most 8192
// channels): a thread owns eight neighbouring channels, which lie in one head of q, k or v, keeps their sums in
// registers, reads the projection 16 bytes at a time and writes each head's part with one 16-byte store.  The
// arithmetic, element by element, is that of the kernel above.  The weights come transposed ([taps, C]) so that
// neighbouring threads read neighbouring addresses.  A block takes TT neighbouring tokens of the step and asks for
// all their rows at once, before it knows which sequences they belong to (a row in front of its sequence's portion
// is replaced from the slot afterwards): one trip to memory for the rows, and one reduction for all the tokens' sums.
template <int TAPS, int TT>
__global__ void conv_norm_store_vec8_kernel(ConvHeadArgs A, bf16* __restrict__ q_out, bf16* __restrict__ cache) {
    pdl_prologue();
    __shared__ float scratch[2 * TT][32];
    const bf16* proj = pdl_fresh((const bf16*)A.proj);
    const float* state = pdl_fresh(A.state);
    const float* shared_in = pdl_fresh((const float*)A.shared);
    const int Cq = A.H * A.dk, Ck = A.G * A.dk, Cv = A.G * A.dv, C = Cq + Ck + Cv;
    constexpr int keep = TAPS - 1, NR = TT + keep;
    const int c = threadIdx.x * 8;
    const bool active = c < C;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    const int t_begin = blockIdx.x * TT, n = min(TT, A.T - t_begin);
    // the rows of the step that the block's tokens may read: t_begin - keep .. t_begin + TT - 1
    uint4 raw[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int tt = t_begin - keep + r;
        raw[r] = (active && tt >= 0 && tt < A.T) ? *reinterpret_cast<const uint4*>(proj + (size_t)tt * A.stride + A.col0 + c)
                                                 : make_uint4(0u, 0u, 0u, 0u);
    }
    // whose rows those are: a row belongs to a token's portion exactly when it is a row of the token's sequence
    // (a sequence's tokens lie together in a step), so nothing here waits for the sequences' first rows
    int row_seq[NR], pos[TT];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int tt = t_begin - keep + r;
        row_seq[r] = tt >= 0 ? A.token_seq[min(tt, A.T - 1)] : -1;
    }
#pragma unroll
    for (int i = 0; i < TT; ++i) pos[i] = A.positions[min(t_begin + i, A.T - 1)];
    // what this thread's channels are: a head of q, of k or of v
    const bool is_q = c < Cq, is_k = !is_q && c < Cq + Ck;
    const int cc = is_q ? c : (is_k ? c - Cq : c - Cq - Ck);
    const int hsize = (is_q || is_k) ? A.dk : A.dv;
    const int head = cc / hsize, within = cc - head * hsize;
    // the other layer's values for the blend
    float sv[TT][8];
    const bool blend = A.mix == 2 && active && !is_q && !is_k;
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        if (blend && i < n) {
            const float* src = shared_in + (size_t)(t_begin + i) * Cv + cc;
            *reinterpret_cast<float4*>(&sv[i][0]) = *reinterpret_cast<const float4*>(src);
            *reinterpret_cast<float4*>(&sv[i][4]) = *reinterpret_cast<const float4*>(src + 4);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) sv[i][e] = 0.f;
        }
    }
    float wr[TAPS][8];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
        const float4 a = active ? __ldg(reinterpret_cast<const float4*>(A.w_t + (size_t)j * C + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 b = active ? __ldg(reinterpret_cast<const float4*>(A.w_t + (size_t)j * C + c + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        wr[j][0] = a.x; wr[j][1] = a.y; wr[j][2] = a.z; wr[j][3] = a.w;
        wr[j][4] = b.x; wr[j][5] = b.y; wr[j][6] = b.z; wr[j][7] = b.w;
    }
    float nw[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
    if (active && (is_q || is_k)) {
        const float* src = (is_q ? A.wq : A.wk) + cc;
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(src)), w1 = __ldg(reinterpret_cast<const float4*>(src + 4));
        nw[0] = w0.x; nw[1] = w0.y; nw[2] = w0.z; nw[3] = w0.w; nw[4] = w1.x; nw[5] = w1.y; nw[6] = w1.z; nw[7] = w1.w;
    }
    const float lam = A.mix == 2 ? A.lambda[0] : 0.f;
    int page[TT];
    float acc[TT][8];
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        page[i] = A.block_table[(size_t)row_seq[keep + i] * A.max_blocks + pos[i] / A.block_size];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
    }
    // row by row: a row is widened once and goes into every token of the block that reads it (tap j = row - token)
    bool outside = false;                     // some token of the block reads rows in front of its portion (the same for all threads)
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        float u[8];
        {
            const bf16* rr = reinterpret_cast<const bf16*>(&raw[r]);
#pragma unroll
            for (int e = 0; e < 8; ++e) u[e] = __bfloat162float(rr[e]);
        }
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            const int j = r - i;
            if (j < 0 || j >= TAPS) continue;
            if (row_seq[r] == row_seq[keep + i]) {
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[i][e] += wr[j][e] * u[e];
            } else if (i < n) {
                outside = true;
            }
        }
    }
    if (outside && active) {
        // the rows in front of a portion come from the sequence's slot (zeros for a fresh request)
#pragma unroll 1
        for (int i = 0; i < n; ++i) {
            const int sq = row_seq[keep + i];
            if (A.seq_fresh[sq] != 0) continue;
            const int t0 = A.cu_q[sq];
            const float* st = state + (size_t)A.state_slots[sq] * A.state_stride + A.conv_off;
#pragma unroll 1
            for (int j = 0; j < keep; ++j) {
                const int tt = t_begin + i - keep + j;
                if (tt >= t0) continue;
                const float* row = st + (size_t)(keep + (tt - t0)) * C + c;
                const float4 s0 = *reinterpret_cast<const float4*>(row), s1 = *reinterpret_cast<const float4*>(row + 4);
                const float su[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int ii = 0; ii < TT; ++ii) {
                    if (ii != i) continue;
#pragma unroll
                    for (int jj = 0; jj < keep; ++jj) {
                        if (jj != j) continue;
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[ii][e] += wr[jj][e] * su[e];
                    }
                }
            }
        }
    }
    // every token's two sums of squares in one reduction over the block; a warp that holds no channel of q (of k)
    // leaves that sum out
    const bool warp_q = __any_sync(0xffffffffu, active && is_q), warp_k = __any_sync(0xffffffffu, active && is_k);
    float part[2 * TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        float ssq = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ssq += acc[i][e] * acc[i][e];
        part[2 * i] = warp_q ? warp_sum(active && is_q ? ssq : 0.f) : 0.f;
        part[2 * i + 1] = warp_k ? warp_sum(active && is_k ? ssq : 0.f) : 0.f;
    }
    if (lane == 0) {
#pragma unroll
        for (int v = 0; v < 2 * TT; ++v) scratch[v][warp] = part[v];
    }
    __syncthreads();
    {
        float mine = 0.f;                      // lane v adds up sum v over the warps, in the warps' order
        if (lane < 2 * TT)
            for (int w = 0; w < nwarps; ++w) mine += scratch[lane][w];
#pragma unroll
        for (int v = 0; v < 2 * TT; ++v) part[v] = __shfl_sync(0xffffffffu, mine, v);
    }
    const size_t plane = (size_t)A.G * A.block_size * A.d;
    const bf16 zero = __float2bfloat16_rn(0.f);
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        if (i >= n) break;
        const int t = t_begin + i;
        const float inv = is_q ? 1.0f / sqrtf(part[2 * i] / (float)Cq + A.eps) : 1.0f / sqrtf(part[2 * i + 1] / (float)Ck + A.eps);
        const bool page_ok = page[i] >= 0 && page[i] < A.num_blocks;
        if (!page_ok && threadIdx.x == 0) atomicExch(A.status, 3);
        bf16* krow0 = cache + (size_t)(page_ok ? page[i] : 0) * 2 * plane + (size_t)(pos[i] % A.block_size) * A.d;
        bf16* qrow = q_out + (size_t)t * A.H * A.d;
        if (active) {
            uint4 ov;
            bf16* o = reinterpret_cast<bf16*>(&ov);
            if (is_q || is_k) {
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __float2bfloat16_rn(acc[i][e] * inv * nw[e]);
                if (is_q) *reinterpret_cast<uint4*>(qrow + (size_t)head * A.d + within) = ov;
                else if (page_ok) *reinterpret_cast<uint4*>(krow0 + (size_t)head * A.block_size * A.d + within) = ov;
            } else {
                if (A.mix == 1) {
                    float* dst = A.shared + (size_t)t * Cv + cc;
                    *reinterpret_cast<float4*>(dst) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
                } else if (A.mix == 2) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[i][e] = (1.0f - lam) * acc[i][e] + lam * sv[i][e];
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __float2bfloat16_rn(acc[i][e]);
                if (page_ok) *reinterpret_cast<uint4*>(krow0 + plane + (size_t)head * A.block_size * A.d + within) = ov;
            }
        }
        // heads filled up to d with zeros
        if (A.d > A.dk) {
            const int pad = A.d - A.dk;
            for (int idx = threadIdx.x; idx < (A.H + A.G) * pad; idx += blockDim.x) {
                const int h = idx / pad, k = A.dk + (idx - h * pad);
                if (h < A.H) qrow[(size_t)h * A.d + k] = zero;
                else if (page_ok) krow0[(size_t)(h - A.H) * A.block_size * A.d + k] = zero;
            }
        }
        if (A.d > A.dv && page_ok) {
            const int pad = A.d - A.dv;
            for (int idx = threadIdx.x; idx < A.G * pad; idx += blockDim.x) {
                const int g = idx / pad, k = A.dv + (idx - g * pad);
                krow0[plane + (size_t)g * A.block_size * A.d + k] = zero;
            }
        }
    }
}

// y[t, h*dv + i] = att[t, h*d + i] * sigmoid(g[t, g_off + h*dv + i])      (i < dv; the attention's heads have d >= dv elements)
template <typename T>
__global__ void head_gate_kernel(const T* att, const T* g, int g_stride, int g_off, T* __restrict__ y, int H, int d, int dv,
                                 size_t total) {
    pdl_prologue();
    att = pdl_fresh(att);
    g = pdl_fresh(g);
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int W = H * dv;
    const size_t t = idx / W;
    const int c = (int)(idx - t * W), h = c / dv, i = c - h * dv;
    const float a = to_float(att[t * (size_t)H * d + (size_t)h * d + i]);
    const float z = to_float(g[t * (size_t)g_stride + g_off + c]);
    y[idx] = from_float<T>(a / (1.0f + expf(-z)));
}

// The same with eight bfloat16 elements a thread (dv, d, g_stride and g_off multiples of 8, 16-byte aligned rows).
__global__ void head_gate_vec8_kernel(const bf16* att, const bf16* g, int g_stride, int g_off, bf16* __restrict__ y, int H,
                                      int d, int dv) {
    pdl_prologue();
    att = pdl_fresh(att);
    g = pdl_fresh(g);
    const int W = H * dv;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    const size_t t = blockIdx.y;
    if (c >= W) return;
    const int h = c / dv, i = c - h * dv;
    const uint4 av = *reinterpret_cast<const uint4*>(att + t * (size_t)H * d + (size_t)h * d + i);
    const uint4 gv = *reinterpret_cast<const uint4*>(g + t * (size_t)g_stride + g_off + c);
    const bf16* a = reinterpret_cast<const bf16*>(&av);
    const bf16* z = reinterpret_cast<const bf16*>(&gv);
    uint4 ov;
    bf16* o = reinterpret_cast<bf16*>(&ov);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(__bfloat162float(a[j]) / (1.0f + expf(-__bfloat162float(z[j]))));
    *reinterpret_cast<uint4*>(y + t * (size_t)W + c) = ov;
}

}  // namespace ff

using namespace ff;

FF_EXPORT int ff_conv_norm_store(const void* proj, int dtype, int stride, int col0, const float* w, const float* wq,
                                 const float* wk, const float* state, long long state_stride, int conv_off,
                                 const int* token_seq, const int* cu_q, const int* positions, const int* state_slots,
                                 const int* seq_fresh, const int* block_table, int max_blocks, int block_size,
                                 int num_blocks, int T, int H, int G, int dk, int dv, int d, int taps, float eps, int mix,
                                 const float* lambda, float* shared, void* q_out, void* cache, int* status,
                                 const float* w_t, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || d < dk || d < dv || taps < 1 || mix < 0 || mix > 2) return FF_ERR_BAD_ARG;
    if (taps > CA_MAX_TAPS) return FF_ERR_UNSUPPORTED;
    if (mix && !shared) return FF_ERR_BAD_ARG;
    if (mix == 2 && !lambda) return FF_ERR_BAD_ARG;
    const int C = H * dk + G * dk + G * dv;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return FF_ERR_UNSUPPORTED;
    ConvHeadArgs A{proj, stride, col0, w, w_t, T, wq, wk, state, state_stride, conv_off, token_seq, cu_q, positions, state_slots,
                   seq_fresh, block_table, max_blocks, block_size, num_blocks, H, G, dk, dv, d, taps, eps, mix, lambda,
                   shared, status};
    if (dtype == 1 && w_t && ((uintptr_t)w_t & 15) == 0 && taps >= 2 && taps <= 4 && dk % 8 == 0 && dv % 8 == 0 && d % 8 == 0 &&
        stride % 8 == 0 && col0 % 8 == 0 && C <= 8192 && state_stride % 4 == 0 && conv_off % 4 == 0 &&
        (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)cache | (uintptr_t)state | (uintptr_t)shared | (uintptr_t)wq |
          (uintptr_t)wk) & 15) == 0) {
        const int vthreads = (C / 8 + 31) / 32 * 32;
        // steps of many tokens give a block four of them; short steps keep one token a block and fill more SMs
        const bool four = T >= 1024;
        const int vblocks = four ? (T + 3) / 4 : T;
#define FF_CNS_LAUNCH(TAPS_)                                                                                               \
        if (four) FF_LAUNCH((conv_norm_store_vec8_kernel<TAPS_, 4>), vblocks, vthreads, 0, stream, A, (bf16*)q_out, (bf16*)cache); \
        else FF_LAUNCH((conv_norm_store_vec8_kernel<TAPS_, 1>), vblocks, vthreads, 0, stream, A, (bf16*)q_out, (bf16*)cache)
        if (taps == 2) { FF_CNS_LAUNCH(2); }
        else if (taps == 3) { FF_CNS_LAUNCH(3); }
        else { FF_CNS_LAUNCH(4); }
#undef FF_CNS_LAUNCH
        FF_LAUNCH_CHECK();
        return 0;
    }
    const int threads = C >= 2048 ? 256 : (C >= 512 ? 128 : 64);
    if (dtype == 0) {
        if (smem > 48 * 1024) FF_SMEM_LIMIT(conv_norm_store_kernel<float>, smem);
        FF_LAUNCH((conv_norm_store_kernel<float>), T, threads, smem, stream, A, (float*)q_out, (float*)cache);
    } else if (dtype == 1) {
        if (smem > 48 * 1024) FF_SMEM_LIMIT(conv_norm_store_kernel<bf16>, smem);
        FF_LAUNCH((conv_norm_store_kernel<bf16>), T, threads, smem, stream, A, (bf16*)q_out, (bf16*)cache);
    } else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_head_gate(const void* att, const void* g, int g_stride, int g_off, int dtype, void* y, int T, int H, int d,
                           int dv, cudaStream_t stream) {
    const size_t total = (size_t)T * H * dv;
    if (total == 0) return 0;
    if (d < dv) return FF_ERR_BAD_ARG;
    if (dtype == 1 && dv % 8 == 0 && d % 8 == 0 && g_stride % 8 == 0 && g_off % 8 == 0 && T <= 65535 &&
        (((uintptr_t)att | (uintptr_t)g | (uintptr_t)y) & 15) == 0) {
        FF_LAUNCH(head_gate_vec8_kernel, dim3((H * dv / 8 + 127) / 128, T), 128, 0, stream, (const bf16*)att, (const bf16*)g,
                  g_stride, g_off, (bf16*)y, H, d, dv);
        FF_LAUNCH_CHECK();
        return 0;
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) FF_LAUNCH((head_gate_kernel<float>), blocks, 256, 0, stream, (const float*)att, (const float*)g, g_stride, g_off, (float*)y, H, d, dv, total);
    else if (dtype == 1) FF_LAUNCH((head_gate_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)att, (const bf16*)g, g_stride, g_off, (bf16*)y, H, d, dv, total);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
