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

}  // namespace ff

using namespace ff;

FF_EXPORT int ff_conv_norm_store(const void* proj, int dtype, int stride, int col0, const float* w, const float* wq,
                                 const float* wk, const float* state, long long state_stride, int conv_off,
                                 const int* token_seq, const int* cu_q, const int* positions, const int* state_slots,
                                 const int* seq_fresh, const int* block_table, int max_blocks, int block_size,
                                 int num_blocks, int T, int H, int G, int dk, int dv, int d, int taps, float eps, int mix,
                                 const float* lambda, float* shared, void* q_out, void* cache, int* status,
                                 cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || d < dk || d < dv || taps < 1 || mix < 0 || mix > 2) return FF_ERR_BAD_ARG;
    if (taps > CA_MAX_TAPS) return FF_ERR_UNSUPPORTED;
    if (mix && !shared) return FF_ERR_BAD_ARG;
    if (mix == 2 && !lambda) return FF_ERR_BAD_ARG;
    const int C = H * dk + G * dk + G * dv;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return FF_ERR_UNSUPPORTED;
    ConvHeadArgs A{proj, stride, col0, w, wq, wk, state, state_stride, conv_off, token_seq, cu_q, positions, state_slots,
                   seq_fresh, block_table, max_blocks, block_size, num_blocks, H, G, dk, dv, d, taps, eps, mix, lambda,
                   shared, status};
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
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) FF_LAUNCH((head_gate_kernel<float>), blocks, 256, 0, stream, (const float*)att, (const float*)g, g_stride, g_off, (float*)y, H, d, dv, total);
    else if (dtype == 1) FF_LAUNCH((head_gate_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)att, (const bf16*)g, g_stride, g_off, (bf16*)y, H, d, dv, total);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
