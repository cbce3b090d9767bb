// Finishing a step's query and key heads when the unit norm comes behind the rotation:
//
//   rotate the first `rdims` elements of every q and k head (pairs (i, i + rdims/2), angle = position * f_i,
//   cos and sin times `mag`), then divide the head by its root mean square over its `norm_dim` elements
//   (no weight), write q back in place and k, v into the paged cache.
//
// The frequencies come as a 64-bit table (a scaled rotation changes the table, not this kernel); the angle is
// formed and reduced in double, so cos and sin are right to 32-bit rounding at any position.  Heads are laid out
// with `d` elements each (q | k | v in a row of the projection); a head whose true size is smaller than d has
// zeros behind it (its matrix rows are zero), so sums over d are sums over the head.
//
// Options: `interleaved` pairs element 2i with element 2i + 1 instead of i with i + rdims/2; `normalize` 0 leaves
// the unit norm out (rotation and cache write only); `bias` (float [(nq + 2 nkv) d] in the row's layout, or null) is
// added to q, k and v in 32-bit in front of everything else.
#include "common.cuh"

namespace ff {

template <typename T>
__global__ void rope_unit_norm_store_kernel(
    T* __restrict__ qkv, int width, int nq, int nkv, int d, int norm_dim, float eps, const double* __restrict__ freq,
    int rdims, float mag, const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks, int block_size, int num_blocks,
    T* __restrict__ cache /*[blocks, 2, nkv, block, d]*/, int* __restrict__ status, int interleaved, int normalize,
    const float* __restrict__ bias) {
    pdl_prologue();
    extern __shared__ float sh[];           // cos[half], sin[half], then one head of d floats per warp
    const int t = blockIdx.x;
    const int half = rdims / 2;
    const int pos = positions[t];
    float* s_cos = sh;
    float* s_sin = sh + half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double sn, cs;
        sincos((double)pos * freq[i], &sn, &cs);
        s_cos[i] = (float)cs * mag;
        s_sin[i] = (float)sn * mag;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    float* hbuf = sh + 2 * half + (size_t)warp * d;
    T* row = qkv + (size_t)t * width;
    T* krow = nullptr;
    T* vrow = nullptr;
    if (nkv > 0) {
        const int seq = token_seq[t];
        const int page = block_table[(size_t)seq * max_blocks + pos / block_size];
        if (page < 0 || page >= num_blocks) {
            if (threadIdx.x == 0) atomicExch(status, 2);
        } else {
            krow = cache + (((size_t)page * 2) * nkv * block_size + pos % block_size) * d;
            vrow = krow + (size_t)nkv * block_size * d;
        }
    }
    for (int h = warp; h < nq + 2 * nkv; h += nwarps) {
        T* src = row + (size_t)h * d;
        const float* brow = bias ? bias + (size_t)h * d : nullptr;
        if (h >= nq + nkv) {               // a value head: copied as it is (plus its bias)
            if (vrow) {
                T* dst = vrow + (size_t)(h - nq - nkv) * block_size * d;
                if (brow)
                    for (int i = lane; i < d; i += 32) dst[i] = from_float<T>(to_float(src[i]) + brow[i]);
                else
                    for (int i = lane; i < d; i += 32) dst[i] = src[i];
            }
            continue;
        }
        for (int i = lane; i < d; i += 32) hbuf[i] = to_float(src[i]) + (brow ? brow[i] : 0.f);
        __syncwarp();
        // element i after the rotation: its partner and the sign of the sine term depend on the pairing
        auto turned = [&](int i) -> float {
            float v = hbuf[i];
            if (i >= rdims) return v;
            if (interleaved) {
                const int f = i >> 1;
                return (i & 1) ? v * s_cos[f] + hbuf[i - 1] * s_sin[f] : v * s_cos[f] - hbuf[i + 1] * s_sin[f];
            }
            return i < half ? v * s_cos[i] - hbuf[i + half] * s_sin[i] : v * s_cos[i - half] + hbuf[i - half] * s_sin[i - half];
        };
        float inv = 1.0f;
        if (normalize) {
            float ss = 0.f;
            for (int i = lane; i < d; i += 32) { const float v = turned(i); ss += v * v; }
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)norm_dim + eps);
        }
        T* dst = h < nq ? src : (krow ? krow + (size_t)(h - nq) * block_size * d : nullptr);
        if (dst)
            for (int i = lane; i < d; i += 32) dst[i] = from_float<T>(turned(i) * inv);
        __syncwarp();
    }
}

}  // namespace ff

using namespace ff;

FF_EXPORT int ff_rope_unit_norm_store(void* qkv, int dtype, int width, int T, int nq, int nkv, int d, int norm_dim,
                                      float eps, const double* freq, int rdims, float mag, const int* positions,
                                      const int* token_seq, const int* block_table, int max_blocks, int block_size,
                                      int num_blocks, void* cache, int* status, int interleaved, int normalize,
                                      const float* bias, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rdims < 0 || rdims % 2 || rdims > d || norm_dim <= 0 || norm_dim > d || d > 1024) return FF_ERR_BAD_ARG;
    const int heads = nq + 2 * nkv;
    const int threads = heads >= 4 ? 128 : 32 * (heads > 0 ? heads : 1);
    const size_t smem = ((size_t)rdims + (size_t)(threads / 32) * d) * sizeof(float);
    if (dtype == 0)
        FF_LAUNCH((rope_unit_norm_store_kernel<float>), T, threads, smem, stream, (float*)qkv, width, nq, nkv, d, norm_dim, eps,
                  freq, rdims, mag, positions, token_seq, block_table, max_blocks, block_size, num_blocks, (float*)cache, status, interleaved, normalize, bias);
    else if (dtype == 1)
        FF_LAUNCH((rope_unit_norm_store_kernel<bf16>), T, threads, smem, stream, (bf16*)qkv, width, nq, nkv, d, norm_dim, eps,
                  freq, rdims, mag, positions, token_seq, block_table, max_blocks, block_size, num_blocks, (bf16*)cache, status, interleaved, normalize, bias);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
