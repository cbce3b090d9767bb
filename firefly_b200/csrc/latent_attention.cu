// The per-token work around attention over a cached latent vector.
//
// A token's cache row is [c (kv_rank), k_rot (rot_dim)]: c = rms_norm(first kv_rank outputs of
// the down projection) * weight, k_rot = the rotated last rot_dim outputs, shared by all heads.
// With q_abs[h] = W_uk[h]^T q_plain[h] (made by a batched product in front of this kernel),
//   score(h, j) = (q_abs[h] . c_j + q_rot[h] . k_rot_j) * scale,   out_latent[h] = sum_j p_j c_j,
// which is attention with one key/value head of size kv_rank + rot_dim whose values are the
// cache rows themselves (the last rot_dim outputs are dropped; the cache has one plane and the
// attention kernels are built to read values from it); the head's value is then
// W_uv[h] out_latent[h].  This file finishes the query rows and writes the cache rows; the
// attention itself is the paged attention the other mixers use.
//
// Rotation: the first rdims (<= rot_dim) elements of the rotated part, pairs (i, i + rdims/2) or, with
// `interleaved`, (2i, 2i + 1), angle = position * f_i; elements past rdims pass unchanged.  A layer that reads
// another layer's cache passes no down projection (`dkv` null): only its queries are finished.  The angle is formed in double from
// the 64-bit frequency table and reduced there, so cos and sin are right to 32-bit rounding at
// any position; norms and the rotation are 32-bit.
#include "common.cuh"

namespace ff {

template <typename T>
__global__ void latent_finish_kernel(
    const T* q_src, int q_stride,                                          // [T, ...]: q heads [H, dim + rot]
    const T* dkv_src, int dkv_stride,                                      // [T, ...]: dkv [kv_rank + rot], or null
    const T* __restrict__ q_abs,                                          // [H, T, kv_rank]
    const float* __restrict__ c_norm_w, float eps, const double* __restrict__ freq /*[rot/2]*/,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ block_table,
    int max_blocks, int block_size, int num_blocks, int planes, T* __restrict__ cache /*[blocks, planes, 1, block, d]*/,
    T* __restrict__ q_full /*[T, H, d]*/, int Ttot, int H, int dim, int rot, int rdims, int kv_rank,
    int interleaved, int* __restrict__ status) {
    pdl_prologue();
    q_src = pdl_fresh(q_src);
    dkv_src = pdl_fresh(dkv_src);
    q_abs = pdl_fresh(q_abs);
    extern __shared__ float sh[];           // cos[rdims/2], sin[rdims/2]
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int half = rdims / 2, rest = rot - rdims;
    const int d = kv_rank + rot;
    const int pos = positions[t];
    float* s_cos = sh;
    float* s_sin = sh + half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double sn, cs;
        sincos((double)pos * freq[i], &sn, &cs);
        s_cos[i] = (float)cs;
        s_sin[i] = (float)sn;
    }
    // the partners of a pair: element `lo_of(i)` turns with element `hi_of(i)` by angle i
    const int step = interleaved ? 2 : 1, gap = interleaved ? 1 : half;
    const T* dkv = dkv_src ? dkv_src + (size_t)t * dkv_stride : nullptr;
    float ss = 0.f;
    if (dkv)
        for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) { const float v = to_float(dkv[i]); ss += v * v; }
    ss = block_sum(ss, scratch);             // also orders the writes of s_cos / s_sin before their use
    const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    // the cache row
    const int seq = token_seq[t];
    const int page = dkv ? block_table[(size_t)seq * max_blocks + pos / block_size] : 0;
    if (!dkv) {
    } else if (page < 0 || page >= num_blocks) {
        if (threadIdx.x == 0) atomicExch(status, 2);
    } else {
        // one plane: the row is read as key and as value; two: the value plane repeats c, with zeros behind it
        T* krow = cache + (((size_t)page * planes) * block_size + pos % block_size) * d;
        T* vrow = planes == 2 ? krow + (size_t)block_size * d : nullptr;
        for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
            const T c = from_float<T>(to_float(dkv[i]) * inv * c_norm_w[i]);
            krow[i] = c;
            if (vrow) vrow[i] = c;
        }
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const int e0 = kv_rank + i * step, e1 = e0 + gap;
            const float a = to_float(dkv[e0]), b = to_float(dkv[e1]);
            krow[e0] = from_float<T>(a * s_cos[i] - b * s_sin[i]);
            krow[e1] = from_float<T>(b * s_cos[i] + a * s_sin[i]);
            if (vrow) {
                vrow[e0] = from_float<T>(0.f);
                vrow[e1] = from_float<T>(0.f);
            }
        }
        for (int i = threadIdx.x; i < rest; i += blockDim.x) {
            krow[kv_rank + rdims + i] = dkv[kv_rank + rdims + i];
            if (vrow) vrow[kv_rank + rdims + i] = from_float<T>(0.f);
        }
    }
    // the query rows: [q_abs | rotated part] per head
    T* qf = q_full + (size_t)t * H * d;
    for (int idx = threadIdx.x; idx < H * kv_rank; idx += blockDim.x) {
        const int h = idx / kv_rank, i = idx - h * kv_rank;
        qf[(size_t)h * d + i] = q_abs[((size_t)h * Ttot + t) * kv_rank + i];
    }
    const T* q = q_src + (size_t)t * q_stride;
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const T* qr = q + (size_t)h * (dim + rot) + dim;
        const int e0 = i * step, e1 = e0 + gap;
        const float a = to_float(qr[e0]), b = to_float(qr[e1]);
        qf[(size_t)h * d + kv_rank + e0] = from_float<T>(a * s_cos[i] - b * s_sin[i]);
        qf[(size_t)h * d + kv_rank + e1] = from_float<T>(b * s_cos[i] + a * s_sin[i]);
    }
    for (int idx = threadIdx.x; idx < H * rest; idx += blockDim.x) {
        const int h = idx / rest, i = idx - h * rest;
        qf[(size_t)h * d + kv_rank + rdims + i] = q[(size_t)h * (dim + rot) + dim + rdims + i];
    }
}

// y[t, h * vdim + j] = val[h, t, j] * sigmoid(g[t, h * vdim + j]), or, with one gate a head, sigmoid(g[t, h])
template <typename T>
__global__ void latent_gate_kernel(const T* val /*[H,T,vdim]*/, const T* g, int g_stride,
                                   T* __restrict__ y, int Ttot, int H, int vdim, size_t total, int per_head) {
    pdl_prologue();
    val = pdl_fresh(val);
    g = pdl_fresh(g);
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int hv = H * vdim;
    const size_t t = idx / hv;
    const int c = (int)(idx - t * hv);
    const int h = c / vdim, j = c - h * vdim;
    const float gv = to_float(g[t * g_stride + (per_head ? h : c)]);
    y[idx] = from_float<T>(to_float(val[((size_t)h * Ttot + t) * vdim + j]) / (1.0f + expf(-gv)));
}

}  // namespace ff

using namespace ff;

FF_EXPORT int ff_latent_finish(const void* q, int q_stride, const void* dkv, int dkv_stride, int dtype, const void* q_abs,
                               const float* c_norm_w, float eps, const double* freq, const int* positions,
                               const int* token_seq, const int* block_table, int max_blocks, int block_size,
                               int num_blocks, int planes, void* cache, void* q_full, int T, int H, int dim, int rot,
                               int rdims, int kv_rank, int interleaved, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (planes != 1 && planes != 2) return FF_ERR_BAD_ARG;
    if (rot < 0 || rdims < 0 || rdims > rot || rdims % 2 || kv_rank <= 0) return FF_ERR_BAD_ARG;
    const size_t smem = (size_t)(rdims > 0 ? rdims : 2) * sizeof(float);
    if (smem > 40 * 1024) return FF_ERR_UNSUPPORTED;
    if (dtype == 0)
        FF_LAUNCH((latent_finish_kernel<float>), T, 256, smem, stream, (const float*)q, q_stride, (const float*)dkv, dkv_stride,
                  (const float*)q_abs, c_norm_w, eps, freq, positions, token_seq, block_table, max_blocks, block_size,
                  num_blocks, planes, (float*)cache, (float*)q_full, T, H, dim, rot, rdims, kv_rank, interleaved, status);
    else if (dtype == 1)
        FF_LAUNCH((latent_finish_kernel<bf16>), T, 256, smem, stream, (const bf16*)q, q_stride, (const bf16*)dkv, dkv_stride,
                  (const bf16*)q_abs, c_norm_w, eps, freq, positions, token_seq, block_table, max_blocks, block_size,
                  num_blocks, planes, (bf16*)cache, (bf16*)q_full, T, H, dim, rot, rdims, kv_rank, interleaved, status);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_latent_gate(const void* val, const void* g, int g_stride, int dtype, void* y, int T, int H, int vdim,
                             int per_head, cudaStream_t stream) {
    const size_t total = (size_t)T * H * vdim;
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0)
        FF_LAUNCH((latent_gate_kernel<float>), blocks, 256, 0, stream, (const float*)val, (const float*)g, g_stride,
                  (float*)y, T, H, vdim, total, per_head);
    else if (dtype == 1)
        FF_LAUNCH((latent_gate_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)val, (const bf16*)g, g_stride,
                  (bf16*)y, T, H, vdim, total, per_head);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
