// Row-wise and element-wise kernels: embedding gather, (residual add +) RMSNorm,
// SiLU-gate product, casts.  Statistics and sums are 32-bit whatever the storage.
//
// Arithmetic follows the reference's kernels (src/kernels/embedding.cu:19-37,
// src/kernels/norm.cu:73-131, src/kernels/activation.cu:15-19, src/kernels/add.cu:33-39)
// but the residual add is folded into the norm and the residual stream is kept in
// 32-bit, so a layer's output is rounded once.
#include "common.cuh"

namespace ff {

// ---------------------------------------------------------------- embedding --
template <typename TT>
__global__ void embedding_kernel(const int* __restrict__ ids, const TT* __restrict__ table,
                                 float* __restrict__ out, int H, int V, float scale, int* __restrict__ status) {
    pdl_prologue();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {  // never read outside the table; report it
        if (threadIdx.x == 0) atomicExch(status, 1);
        id = 0;
    }
    const TT* src = table + (size_t)id * H;
    float* dst = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_float(src[i]) * scale;
}

// ------------------------------------------------------ residual add + norm --
// residual[src,:] (+= delta[src,:]);  out[r,:] = v * rsqrt(mean(v^2)+eps) * w
// src = row_idx ? row_idx[r] : r.  With row_idx the residual is not written back.
// four consecutive elements of either type
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

// VEC = 4: four elements a thread and step (needs H % 4 == 0); VEC = 1: any H.
template <typename TD, typename TO, int VEC>
__global__ void add_rms_norm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                    const int* __restrict__ row_idx, const float* __restrict__ w,
                                    float eps, TO* __restrict__ out, int H, int write_residual,
                                    int use_smem) {
    pdl_prologue();
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = row_idx ? row_idx[r] : r;
    float* res = residual + (size_t)src * H;
    const TD* dl = delta ? delta + (size_t)src * H : nullptr;
    float ss = 0.f;
    if (VEC == 4) {
#pragma unroll 4
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 v = load4(res + i);
            if (dl) {
                const float4 d = load4(dl + i);
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
                if (write_residual) store4(res + i, v);
            }
            if (use_smem) store4(row + i, v);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = res[i];
            if (dl) v += to_float(dl[i]);
            if (use_smem) row[i] = v;
            if (dl && write_residual) res[i] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)r * H;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 v;
            if (use_smem) v = load4(row + i);
            else {
                v = load4(res + i);
                if (dl && !write_residual) { const float4 d = load4(dl + i); v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w; }
            }
            const float4 ww = load4(w + i);
            store4(o + i, make_float4(v.x * inv * ww.x, v.y * inv * ww.y, v.z * inv * ww.z, v.w * inv * ww.w));
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v;
            if (use_smem) v = row[i];
            else { v = res[i]; if (dl && !write_residual) v += to_float(dl[i]); }
            o[i] = from_float<TO>(v * inv * w[i]);
        }
    }
}

// ------------------------------------------------------------------ SwiGLU --
// out[t,i] = silu(g) * u with g = gu[t,i], u = gu[t,I+i]; or, when the columns of gu
// interleave gate and up in groups of 16 (the layout the fused product uses for its
// weight), g = gu[t, 32*(i/16) + i%16], u = gu[t, 32*(i/16) + 16 + i%16].
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total,
                                int interleaved) {
    pdl_prologue();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    size_t t = idx / I;
    int i = (int)(idx - t * I);
    const T* row = gu + t * 2 * I;
    const int gi = interleaved ? 32 * (i / 16) + (i % 16) : i;
    const int ui = interleaved ? gi + 16 : I + i;
    float g = to_float(row[gi]);
    float u = to_float(row[ui]);
    out[idx] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

// Four outputs a thread (needs I % 4 == 0, and I % 16 == 0 when interleaved).
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total4,
                                    int interleaved) {
    pdl_prologue();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    const int per_row = I / 4;
    size_t t = idx / per_row;
    int i = (int)(idx - t * per_row) * 4;
    const T* row = gu + t * 2 * I;
    const int gi = interleaved ? 32 * (i / 16) + (i % 16) : i;
    const int ui = interleaved ? gi + 16 : I + i;
    const float4 g = load4(row + gi), u = load4(row + ui);
    store4(out + t * I + i, make_float4(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y,
                                        g.z / (1.0f + expf(-g.z)) * u.z, g.w / (1.0f + expf(-g.w)) * u.w));
}

// Eight bfloat16 outputs a thread (needs I % 8 == 0, and I % 16 == 0 when interleaved): 16-byte
// loads and stores, the form long prompts use.  (Four such groups a thread measured slower.)
__global__ void silu_mul_vec8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I, int T,
                                     int interleaved) {
    pdl_prologue();
    const int per_row = I / 8;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= per_row) return;
    const int i = c * 8;
    const bf16* row = gu + (size_t)t * 2 * I;
    const int gi = interleaved ? 32 * (i / 16) + (i % 16) : i;
    const int ui = interleaved ? gi + 16 : I + i;
    const uint4 gv = *reinterpret_cast<const uint4*>(row + gi), uv = *reinterpret_cast<const uint4*>(row + ui);
    const bf16* g = reinterpret_cast<const bf16*>(&gv);
    const bf16* u = reinterpret_cast<const bf16*>(&uv);
    uint4 ov;
    bf16* o = reinterpret_cast<bf16*>(&ov);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float x = __bfloat162float(g[j]);
        o[j] = __float2bfloat16_rn(x / (1.0f + expf(-x)) * __bfloat162float(u[j]));
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * I + i) = ov;
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* in, TO* __restrict__ out, size_t n) {
    pdl_prologue();
    in = pdl_fresh(in);
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_float<TO>(to_float(in[i]));
}

// out[r,:] += delta[r,:]   (32-bit residual, delta of either type)
template <typename TD>
__global__ void add_kernel(float* __restrict__ res, const TD* __restrict__ delta, size_t n) {
    pdl_prologue();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) res[i] += to_float(delta[i]);
}

// ----------------------------------------------------------- metadata updates --
// buf[upd[1 + 2i]] = upd[2 + 2i] for i < min(upd[0], cap): a step's few changed block-table
// entries are written into the table that stays on the device, so that the host uploads what
// changed and not the table.  Indices outside [0, len) are skipped.
// The kernels behind this one look pages up in the tables before they wait for the kernel in front of
// them, so this one does not let its dependents start early: they are launched when it has ended,
// with its writes in place.
__global__ void scatter_int_kernel(int* __restrict__ buf, const int* __restrict__ upd, int cap, int len) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int n = min(upd[0], cap);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int idx = upd[1 + 2 * i];
        if (idx >= 0 && idx < len) buf[idx] = upd[2 + 2 * i];
    }
}

// A row's threads: 16 elements each, so that many rows share an SM and each thread has four loads in flight.
static inline int norm_threads(int H) {
    int t = (H + 15) / 16;
    t = ((t + 31) / 32) * 32;
    if (t < 32) t = 32;
    if (t > 1024) t = 1024;
    return t;
}

}  // namespace ff

using namespace ff;

// dtype codes: 0 = float32, 1 = bfloat16
FF_EXPORT int ff_scatter_int(int* buf, const int* upd, int cap, int len, cudaStream_t stream) {
    if (cap <= 0) return 0;
    const unsigned blocks = (unsigned)((cap + 255) / 256);
    FF_LAUNCH((scatter_int_kernel), blocks, 256, 0, stream, buf, upd, cap, len);
    FF_LAUNCH_CHECK();
    return 0;
}
FF_EXPORT int ff_embedding(const int* ids, const void* table, int table_dtype, float* out, int T,
                           int H, int V, float scale, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
    if (table_dtype == 0)
        FF_LAUNCH((embedding_kernel<float>), T, threads, 0, stream, ids, (const float*)table, out, H, V, scale, status);
    else if (table_dtype == 1)
        FF_LAUNCH((embedding_kernel<bf16>), T, threads, 0, stream, ids, (const bf16*)table, out, H, V, scale, status);
    else
        return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

template <typename TD, typename TO>
static int launch_add_rms_norm(float* residual, const void* delta, const int* row_idx, const float* w,
                               float eps, void* out, int rows, int H, int write_residual,
                               cudaStream_t stream) {
    size_t smem = (size_t)H * sizeof(float);
    int use_smem = smem <= 200 * 1024;
    if (!use_smem) smem = 0;
    const bool vec = (H % 4) == 0;
    auto kern = vec ? add_rms_norm_kernel<TD, TO, 4> : add_rms_norm_kernel<TD, TO, 1>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    FF_LAUNCH((kern), rows, norm_threads(H), smem, stream, residual, (const TD*)delta, row_idx, w, eps, (TO*)out,
                                                  H, write_residual, use_smem);
    FF_LAUNCH_CHECK();
    return 0;
}

// delta may be null (plain norm).  delta_dtype / out_dtype: 0 f32, 1 bf16.
FF_EXPORT int ff_add_rms_norm(float* residual, const void* delta, int delta_dtype, const int* row_idx,
                              const float* w, float eps, void* out, int out_dtype, int rows, int H,
                              int write_residual, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0) return FF_ERR_BAD_ARG;
    if (delta_dtype == 0 && out_dtype == 0)
        return launch_add_rms_norm<float, float>(residual, delta, row_idx, w, eps, out, rows, H, write_residual, stream);
    if (delta_dtype == 1 && out_dtype == 1)
        return launch_add_rms_norm<bf16, bf16>(residual, delta, row_idx, w, eps, out, rows, H, write_residual, stream);
    if (delta_dtype == 0 && out_dtype == 1)
        return launch_add_rms_norm<float, bf16>(residual, delta, row_idx, w, eps, out, rows, H, write_residual, stream);
    if (delta_dtype == 1 && out_dtype == 0)
        return launch_add_rms_norm<bf16, float>(residual, delta, row_idx, w, eps, out, rows, H, write_residual, stream);
    return FF_ERR_BAD_ARG;
}

FF_EXPORT int ff_silu_mul(const void* gate_up, void* out, int dtype, int T, int I, int interleaved,
                          cudaStream_t stream) {
    if (interleaved && (I % 16)) return FF_ERR_BAD_ARG;
    size_t total = (size_t)T * I;
    if (total == 0) return 0;
    if (dtype != 0 && dtype != 1) return FF_ERR_BAD_ARG;
    if (dtype == 1 && I % 8 == 0 && T <= 65535 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const int per_row = I / 8;
        FF_LAUNCH(silu_mul_vec8_kernel, dim3((per_row + 127) / 128, T), 128, 0, stream, (const bf16*)gate_up,
                  (bf16*)out, I, T, interleaved);
        return 0;
    }
    if (I % 4 == 0) {
        const size_t total4 = total / 4;
        unsigned blocks = (unsigned)((total4 + 255) / 256);
        if (dtype == 0) FF_LAUNCH((silu_mul_vec_kernel<float>), blocks, 256, 0, stream, (const float*)gate_up, (float*)out, I, total4, interleaved);
        else FF_LAUNCH((silu_mul_vec_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)gate_up, (bf16*)out, I, total4, interleaved);
        return 0;
    }
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) FF_LAUNCH((silu_mul_kernel<float>), blocks, 256, 0, stream, (const float*)gate_up, (float*)out, I, total, interleaved);
    else FF_LAUNCH((silu_mul_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)gate_up, (bf16*)out, I, total, interleaved);
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_cast(const void* in, int in_dtype, void* out, int out_dtype, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == 0 && out_dtype == 1) FF_LAUNCH((cast_kernel<float, bf16>), blocks, 256, 0, stream, (const float*)in, (bf16*)out, n);
    else if (in_dtype == 1 && out_dtype == 0) FF_LAUNCH((cast_kernel<bf16, float>), blocks, 256, 0, stream, (const bf16*)in, (float*)out, n);
    else if (in_dtype == 0 && out_dtype == 0) FF_LAUNCH((cast_kernel<float, float>), blocks, 256, 0, stream, (const float*)in, (float*)out, n);
    else if (in_dtype == 1 && out_dtype == 1) FF_LAUNCH((cast_kernel<bf16, bf16>), blocks, 256, 0, stream, (const bf16*)in, (bf16*)out, n);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_residual_add(float* residual, const void* delta, int delta_dtype, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (delta_dtype == 0) FF_LAUNCH((add_kernel<float>), blocks, 256, 0, stream, residual, (const float*)delta, n);
    else if (delta_dtype == 1) FF_LAUNCH((add_kernel<bf16>), blocks, 256, 0, stream, residual, (const bf16*)delta, n);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

// --------------------------------------------------- norm on a part's output, added into the stream --
// residual[t] += rms_norm(delta[t]) * w   (a block whose norms sit on the parts' outputs: the parts read the
// stream itself), statistics and sum in 32-bit.  `copy` (optional, [T,H] in the activation type) receives the
// updated row for the next part's products.
namespace ff {
template <typename TD, typename TO>
__global__ void norm_add_kernel(float* __restrict__ residual, const TD* delta, const float* __restrict__ w,
                                float eps, TO* __restrict__ copy, int H) {
    pdl_prologue();
    delta = pdl_fresh(delta);
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* res = residual + (size_t)r * H;
    const TD* dl = delta + (size_t)r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = to_float(dl[i]); ss += v * v; }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = res[i] + to_float(dl[i]) * inv * w[i];
        res[i] = v;
        if (copy) copy[(size_t)r * H + i] = from_float<TO>(v);
    }
}

// The same with four elements a thread and step, the row's delta and stream kept in registers between the two
// passes (H % 4 == 0, H <= 16 * threads): one round trip to memory instead of two in a row.
template <typename TD, typename TO>
__global__ void norm_add_vec_kernel(float* __restrict__ residual, const TD* delta, const float* __restrict__ w,
                                    float eps, TO* __restrict__ copy, int H) {
    pdl_prologue();
    delta = pdl_fresh(delta);
    constexpr int IT = 4;
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* res = residual + (size_t)r * H;
    const TD* dl = delta + (size_t)r * H;
    float4 d[IT], x[IT];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < IT; ++u) {
        const int i = (threadIdx.x + u * blockDim.x) * 4;
        if (i < H) {
            d[u] = load4(dl + i);
            x[u] = load4(res + i);
            ss += d[u].x * d[u].x + d[u].y * d[u].y + d[u].z * d[u].z + d[u].w * d[u].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int u = 0; u < IT; ++u) {
        const int i = (threadIdx.x + u * blockDim.x) * 4;
        if (i < H) {
            const float4 ww = load4(w + i);
            const float4 v = make_float4(x[u].x + d[u].x * inv * ww.x, x[u].y + d[u].y * inv * ww.y,
                                         x[u].z + d[u].z * inv * ww.z, x[u].w + d[u].w * inv * ww.w);
            store4(res + i, v);
            if (copy) store4(copy + (size_t)r * H + i, v);
        }
    }
}

// out[t,i] = act(g) * u with g = gu[t,i] (+ bias[i]), u = gu[t,I+i] (+ bias[I+i]); act 0: SiLU, 1: the tanh form
// of GELU, 2: the clamped form min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1).
// `bias` float32 [2I] or null.
template <typename T>
__global__ void glu_act_kernel(const T* gu, const float* __restrict__ bias, T* __restrict__ out, int I, size_t total,
                               int act, float limit) {
    pdl_prologue();
    gu = pdl_fresh(gu);
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    float g = to_float(gu[t * 2 * I + i]), u = to_float(gu[t * 2 * I + I + i]);
    if (bias) { g += bias[i]; u += bias[I + i]; }
    float a;
    if (act == 0) a = g / (1.0f + expf(-g));
    else if (act == 1) a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    else {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit) + 1.0f;
        a = g / (1.0f + expf(-1.702f * g));
    }
    out[idx] = from_float<T>(a * u);
}

// out[t, j] = act(g[t, j]) * table[ids[t], col0 + j] for j < n: a projection's rows gated into the rows that a table
// holds per token id (one slice of `n` columns of a wider table).  act 0: SiLU, 1: the tanh form of GELU; 32-bit
// arithmetic.  An id outside the table raises status 1 and reads row 0.
template <typename T>
__global__ void act_mul_table_rows_kernel(const T* g, const int* __restrict__ ids, const T* __restrict__ table,
                                          int table_cols, int col0, int vocab, T* __restrict__ out, int n, size_t total,
                                          int act, int* __restrict__ status) {
    pdl_prologue();
    g = pdl_fresh(g);
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / n;
    const int j = (int)(idx - t * n);
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (j == 0) atomicExch(status, 1);
        id = 0;
    }
    const float z = to_float(g[idx]);
    const float a = act == 0 ? z / (1.0f + expf(-z))
                             : 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    out[idx] = from_float<T>(a * to_float(table[(size_t)id * table_cols + col0 + j]));
}

// Eight bfloat16 outputs a thread (I % 8 == 0, rows 16-byte aligned): 16-byte loads and stores, the form long
// prompts use.  The arithmetic is that of glu_act_kernel, element by element.
template <int ACT>
__global__ void glu_act_vec8_kernel(const bf16* gu, const float* __restrict__ bias, bf16* __restrict__ out, int I,
                                    float limit) {
    pdl_prologue();
    gu = pdl_fresh(gu);
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= I / 8) return;
    const int i = c * 8;
    const bf16* row = gu + (size_t)t * 2 * I;
    const uint4 gv = *reinterpret_cast<const uint4*>(row + i), uv = *reinterpret_cast<const uint4*>(row + I + i);
    const bf16* gp = reinterpret_cast<const bf16*>(&gv);
    const bf16* up = reinterpret_cast<const bf16*>(&uv);
    float gb[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, ub[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (bias) {
        *reinterpret_cast<float4*>(gb) = __ldg(reinterpret_cast<const float4*>(bias + i));
        *reinterpret_cast<float4*>(gb + 4) = __ldg(reinterpret_cast<const float4*>(bias + i + 4));
        *reinterpret_cast<float4*>(ub) = __ldg(reinterpret_cast<const float4*>(bias + I + i));
        *reinterpret_cast<float4*>(ub + 4) = __ldg(reinterpret_cast<const float4*>(bias + I + i + 4));
    }
    uint4 ov;
    bf16* o = reinterpret_cast<bf16*>(&ov);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float g = __bfloat162float(gp[j]) + gb[j], u = __bfloat162float(up[j]) + ub[j];
        float a;
        if (ACT == 0) a = g / (1.0f + expf(-g));
        else if (ACT == 1) a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
        else {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit) + 1.0f;
            a = g / (1.0f + expf(-1.702f * g));
        }
        o[j] = __float2bfloat16_rn(a * u);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * I + i) = ov;
}

// x *= a
__global__ void scale_kernel(float* x, float a, size_t total) {
    pdl_prologue();
    x = pdl_fresh(x);
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) x[idx] *= a;
}
}  // namespace ff

FF_EXPORT int ff_norm_add(float* residual, const void* delta, int delta_dtype, const float* w, float eps, void* copy,
                          int copy_dtype, int rows, int H, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0) return FF_ERR_BAD_ARG;
    if (H % 4 == 0 && H <= 16 * 1024 && (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)copy | (uintptr_t)w) & 15) == 0) {
        int threads = ((H / 4 + 3) / 4 + 31) / 32 * 32;          // four steps a thread where the row is long enough
        if (threads < 32) threads = 32;
        if (threads > 1024) threads = 1024;
        while (threads * 16 < H) threads += 32;
        if (delta_dtype == 0 && copy_dtype == 0)
            FF_LAUNCH((norm_add_vec_kernel<float, float>), rows, threads, 0, stream, residual, (const float*)delta, w, eps, (float*)copy, H);
        else if (delta_dtype == 0 && copy_dtype == 1)
            FF_LAUNCH((norm_add_vec_kernel<float, bf16>), rows, threads, 0, stream, residual, (const float*)delta, w, eps, (bf16*)copy, H);
        else if (delta_dtype == 1 && copy_dtype == 1)
            FF_LAUNCH((norm_add_vec_kernel<bf16, bf16>), rows, threads, 0, stream, residual, (const bf16*)delta, w, eps, (bf16*)copy, H);
        else if (delta_dtype == 1 && copy_dtype == 0)
            FF_LAUNCH((norm_add_vec_kernel<bf16, float>), rows, threads, 0, stream, residual, (const bf16*)delta, w, eps, (float*)copy, H);
        else return FF_ERR_BAD_ARG;
        FF_LAUNCH_CHECK();
        return 0;
    }
    const int threads = norm_threads(H);
    if (delta_dtype == 0 && copy_dtype == 0)
        FF_LAUNCH((norm_add_kernel<float, float>), rows, threads, 0, stream, residual, (const float*)delta, w, eps, (float*)copy, H);
    else if (delta_dtype == 0 && copy_dtype == 1)
        FF_LAUNCH((norm_add_kernel<float, bf16>), rows, threads, 0, stream, residual, (const float*)delta, w, eps, (bf16*)copy, H);
    else if (delta_dtype == 1 && copy_dtype == 1)
        FF_LAUNCH((norm_add_kernel<bf16, bf16>), rows, threads, 0, stream, residual, (const bf16*)delta, w, eps, (bf16*)copy, H);
    else if (delta_dtype == 1 && copy_dtype == 0)
        FF_LAUNCH((norm_add_kernel<bf16, float>), rows, threads, 0, stream, residual, (const bf16*)delta, w, eps, (float*)copy, H);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_glu_act(const void* gate_up, const float* bias, void* out, int dtype, int T, int I, int act, float limit,
                         cudaStream_t stream) {
    const size_t total = (size_t)T * I;
    if (total == 0) return 0;
    if (act < 0 || act > 2) return FF_ERR_BAD_ARG;
    if (dtype == 1 && I % 8 == 0 && T <= 65535 && (((uintptr_t)gate_up | (uintptr_t)out | (uintptr_t)bias) & 15) == 0) {
        const dim3 grid((I / 8 + 127) / 128, T);
        if (act == 0) FF_LAUNCH((glu_act_vec8_kernel<0>), grid, 128, 0, stream, (const bf16*)gate_up, bias, (bf16*)out, I, limit);
        else if (act == 1) FF_LAUNCH((glu_act_vec8_kernel<1>), grid, 128, 0, stream, (const bf16*)gate_up, bias, (bf16*)out, I, limit);
        else FF_LAUNCH((glu_act_vec8_kernel<2>), grid, 128, 0, stream, (const bf16*)gate_up, bias, (bf16*)out, I, limit);
        FF_LAUNCH_CHECK();
        return 0;
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) FF_LAUNCH((glu_act_kernel<float>), blocks, 256, 0, stream, (const float*)gate_up, bias, (float*)out, I, total, act, limit);
    else if (dtype == 1) FF_LAUNCH((glu_act_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)gate_up, bias, (bf16*)out, I, total, act, limit);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_scale(float* x, float a, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    FF_LAUNCH(scale_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, a, n);
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_act_mul_table_rows(const void* g, const int* ids, const void* table, int table_cols, int col0, int vocab,
                                    void* out, int dtype, int T, int n, int act, int* status, cudaStream_t stream) {
    const size_t total = (size_t)T * n;
    if (total == 0) return 0;
    if (act < 0 || act > 1 || col0 < 0 || col0 + n > table_cols) return FF_ERR_BAD_ARG;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0)
        FF_LAUNCH((act_mul_table_rows_kernel<float>), blocks, 256, 0, stream, (const float*)g, ids, (const float*)table,
                  table_cols, col0, vocab, (float*)out, n, total, act, status);
    else if (dtype == 1)
        FF_LAUNCH((act_mul_table_rows_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)g, ids, (const bf16*)table,
                  table_cols, col0, vocab, (bf16*)out, n, total, act, status);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
