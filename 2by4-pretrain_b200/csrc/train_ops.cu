// Two element-wise / reduction kernels of the GPT-2 trainer that sit between the sparse GEMMs: layer normalisation
// (float32 residual stream in, 16-bit GEMM operand out, and its backward pass with the gamma / beta gradients taken
// in the same pass) and the cross-entropy loss over 16-bit logits (log-sum-exp forward, gradient written as 16-bit
// values).  Both are HBM-bound streaming kernels on 16-byte accesses; neither has a counterpart in the reference,
// whose training scripts live in another repository.
#include "sp24_common.cuh"

namespace sp24 {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// ---------------------------------------------------------------------------------------------
// layer norm: one warp per row, the row in registers (d <= 128 * MAXV, d % 128 == 0)
// ---------------------------------------------------------------------------------------------
constexpr int MAXV = 8;    // float4 per lane: rows of up to 1024 elements (the row, and in the backward pass five
                           // values per element, live in registers); NV = d / 128 is a template parameter

template <typename TOut> __device__ __forceinline__ void store4(TOut *p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float *p, float a, float b, float c, float d) {
    *reinterpret_cast<float4 *>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16 *p, float a, float b, float c, float d) {
    uint2 o;
    o.x = Elem<__nv_bfloat16>::pack2(a, b);
    o.y = Elem<__nv_bfloat16>::pack2(c, d);
    *reinterpret_cast<uint2 *>(p) = o;
}
template <> __device__ __forceinline__ void store4<__half>(__half *p, float a, float b, float c, float d) {
    uint2 o;
    o.x = Elem<__half>::pack2(a, b);
    o.y = Elem<__half>::pack2(c, d);
    *reinterpret_cast<uint2 *>(p) = o;
}
template <typename TIn> __device__ __forceinline__ float4 load4(const TIn *p);
template <> __device__ __forceinline__ float4 load4<float>(const float *p) { return *reinterpret_cast<const float4 *>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16 *p) {
    const uint2 r = *reinterpret_cast<const uint2 *>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162 *>(&r.x), b = *reinterpret_cast<const __nv_bfloat162 *>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <> __device__ __forceinline__ float4 load4<__half>(const __half *p) {
    const uint2 r = *reinterpret_cast<const uint2 *>(p);
    const __half2 a = *reinterpret_cast<const __half2 *>(&r.x), b = *reinterpret_cast<const __half2 *>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

// y = (x - mean) * rstd * gamma + beta, statistics in float32 (two passes over the registers)
template <typename TOut, int NV>
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const float *x, const float *gamma, const float *beta, TOut *out,
                                                            float *mean_out, float *rstd_out, int64_t rows, float eps) {
    constexpr int d = NV * 128, nv = NV;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float4 v[NV];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (i < nv) {
            v[i] = load4<float>(x + row * d + (i * 32 + lane) * 4);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    const float mean = warp_sum(s) / (float)d;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (i < nv) {
            const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
            q += (a * a + b * b) + (c * c + e * e);
        }
    const float rstd = rsqrtf(warp_sum(q) / (float)d + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (i < nv) {
            const int c0 = (i * 32 + lane) * 4;
            const float4 g = load4<float>(gamma + c0), b = load4<float>(beta + c0);
            store4<TOut>(out + row * d + c0, (v[i].x - mean) * rstd * g.x + b.x, (v[i].y - mean) * rstd * g.y + b.y,
                         (v[i].z - mean) * rstd * g.z + b.z, (v[i].w - mean) * rstd * g.w + b.w);
        }
    if (lane == 0) {
        mean_out[row] = mean;
        rstd_out[row] = rstd;
    }
}

// dx = rstd * (g dy - mean(g dy) - xhat mean(g dy xhat));  dgamma += sum_rows dy xhat;  dbeta += sum_rows dy.
// Persistent warps: each walks rows warp, warp + nwarps, ... and keeps its column sums in registers; one reduction
// over the block's eight warps in shared memory, then one atomic per column and block.
template <typename TDy, int NV>
__global__ void __launch_bounds__(256) layernorm_bwd_kernel(const TDy *dy, const float *x, const float *gamma, const float *mean,
                                                            const float *rstd, float *dx, float *dgamma, float *dbeta,
                                                            int64_t rows) {
    extern __shared__ float red[];           // 2 x 8 x d floats
    constexpr int d = NV * 128, nv = NV;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float4 g[NV], ag[NV], ab[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (i < nv) {
            g[i] = load4<float>(gamma + (i * 32 + lane) * 4);
            ag[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    const int64_t nwarps = (int64_t)gridDim.x * 8;
    for (int64_t row = (int64_t)blockIdx.x * 8 + warp; row < rows; row += nwarps) {
        const float mu = mean[row], rs = rstd[row];
        float4 xh[NV], gy[NV];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (i < nv) {
                const int c0 = (i * 32 + lane) * 4;
                const float4 xv = load4<float>(x + row * d + c0);
                const float4 dv = load4<TDy>(dy + row * d + c0);
                xh[i] = make_float4((xv.x - mu) * rs, (xv.y - mu) * rs, (xv.z - mu) * rs, (xv.w - mu) * rs);
                gy[i] = make_float4(dv.x * g[i].x, dv.y * g[i].y, dv.z * g[i].z, dv.w * g[i].w);
                s1 += (gy[i].x + gy[i].y) + (gy[i].z + gy[i].w);
                s2 += (gy[i].x * xh[i].x + gy[i].y * xh[i].y) + (gy[i].z * xh[i].z + gy[i].w * xh[i].w);
                ag[i].x += dv.x * xh[i].x; ag[i].y += dv.y * xh[i].y; ag[i].z += dv.z * xh[i].z; ag[i].w += dv.w * xh[i].w;
                ab[i].x += dv.x; ab[i].y += dv.y; ab[i].z += dv.z; ab[i].w += dv.w;
            }
        const float m1 = warp_sum(s1) / (float)d, m2 = warp_sum(s2) / (float)d;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (i < nv) {
                const int c0 = (i * 32 + lane) * 4;
                store4<float>(dx + row * d + c0, rs * (gy[i].x - m1 - xh[i].x * m2), rs * (gy[i].y - m1 - xh[i].y * m2),
                              rs * (gy[i].z - m1 - xh[i].z * m2), rs * (gy[i].w - m1 - xh[i].w * m2));
            }
    }
    float *rg = red, *rb = red + 8 * d;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (i < nv) {
            const int c0 = (i * 32 + lane) * 4;
            *reinterpret_cast<float4 *>(rg + warp * d + c0) = ag[i];
            *reinterpret_cast<float4 *>(rb + warp * d + c0) = ab[i];
        }
    __syncthreads();
    for (int c = threadIdx.x; c < d; c += 256) {
        float sg = 0.f, sb = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            sg += rg[w * d + c];
            sb += rb[w * d + c];
        }
        atomicAdd(dgamma + c, sg);
        atomicAdd(dbeta + c, sb);
    }
}

// ---------------------------------------------------------------------------------------------
// cross entropy over 16-bit logits: one block per row
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_reduce(float v, bool is_max, float *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();                       // scratch may still be read from the previous reduction
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = scratch[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
    return r;
}

template <typename T> __device__ __forceinline__ void unpack8(const uint4 &r, float (&f)[8]) {
    const T *h = reinterpret_cast<const T *>(&r);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = Elem<T>::to_f32(h[j]);
}

// lse[row] = log sum exp(logits[row, :]),  loss[row] = lse[row] - logits[row, target[row]]   (float32)
template <typename T>
__global__ void __launch_bounds__(256) ce_fwd_kernel(const T *logits, const int64_t *targets, float *lse, float *loss,
                                                     int64_t v, int64_t ld) {
    __shared__ float scratch[8];
    const int64_t row = blockIdx.x;
    const T *p = logits + row * ld;
    const int64_t nvec = v / 8;
    float m = -INFINITY, s = 0.f;          // running maximum and sum of exp(x - m) of this thread's elements
    for (int64_t i = threadIdx.x; i < nvec; i += 256) {
        float f[8];
        unpack8<T>(*reinterpret_cast<const uint4 *>(p + i * 8), f);
        float vm = f[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) vm = fmaxf(vm, f[j]);
        const float nm = fmaxf(m, vm);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
        s = s * __expf(m - nm) + acc;
        m = nm;
    }
    const float gm = block_reduce(m, true, scratch);
    const float gs = block_reduce(m == -INFINITY ? 0.f : s * __expf(m - gm), false, scratch);
    if (threadIdx.x == 0) {
        const float l = gm + logf(gs);
        lse[row] = l;
        loss[row] = l - Elem<T>::to_f32(p[targets[row]]);
    }
}

// dlogits[row, c] = (exp(logits[row, c] - lse[row]) - [c == target[row]]) * scale * *upstream
template <typename T>
__global__ void __launch_bounds__(256) ce_bwd_kernel(const T *logits, const int64_t *targets, const float *lse,
                                                     const float *upstream, float scale, T *dlogits, int64_t v, int64_t ld,
                                                     int64_t ld_out) {
    const int64_t row = blockIdx.x;
    const T *p = logits + row * ld;
    T *q = dlogits + row * ld_out;
    const float l = lse[row], sc = scale * (upstream ? *upstream : 1.f);
    const int64_t tgt = targets[row];
    const int64_t nvec = v / 8;
    for (int64_t i = threadIdx.x; i < nvec; i += 256) {
        float f[8];
        unpack8<T>(*reinterpret_cast<const uint4 *>(p + i * 8), f);
        uint4 o;
        uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t c = i * 8 + 2 * j;
            const float a = (__expf(f[2 * j] - l) - (c == tgt ? 1.f : 0.f)) * sc;
            const float b = (__expf(f[2 * j + 1] - l) - (c + 1 == tgt ? 1.f : 0.f)) * sc;
            ow[j] = Elem<T>::pack2(a, b);
        }
        *reinterpret_cast<uint4 *>(q + i * 8) = o;
    }
}

}  // namespace
}  // namespace sp24

using namespace sp24;

extern "C" int sp24_layernorm_fwd(const float *x, const float *gamma, const float *beta, void *out, int out_dtype, float *mean,
                                  float *rstd, int64_t rows, int64_t d, float eps, void *stream) {
    if (!x || !gamma || !beta || !out || !mean || !rstd) return SP24_ERR_ARG;
    if (out_dtype != SP24_F32 && out_dtype != SP24_F16 && out_dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (rows <= 0 || d <= 0 || d % 128 || d > 128 * MAXV) return SP24_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(gamma) || !aligned16(beta) || !aligned16(out)) return SP24_ERR_ALIGN;
    if (!(eps >= 0.f)) return SP24_ERR_ARG;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (unsigned)((rows + 7) / 8);
#define SP24_LN_FWD(T_, NV_) \
    layernorm_fwd_kernel<T_, NV_><<<blocks, 256, 0, st>>>(x, gamma, beta, static_cast<T_ *>(out), mean, rstd, rows, eps)
#define SP24_LN_FWD_NV(T_) \
    switch (d / 128) { \
        case 1: SP24_LN_FWD(T_, 1); break; case 2: SP24_LN_FWD(T_, 2); break; case 3: SP24_LN_FWD(T_, 3); break; \
        case 4: SP24_LN_FWD(T_, 4); break; case 5: SP24_LN_FWD(T_, 5); break; case 6: SP24_LN_FWD(T_, 6); break; \
        case 7: SP24_LN_FWD(T_, 7); break; default: SP24_LN_FWD(T_, 8); break; \
    }
    if (out_dtype == SP24_F32) { SP24_LN_FWD_NV(float) }
    else if (out_dtype == SP24_F16) { SP24_LN_FWD_NV(__half) }
    else { SP24_LN_FWD_NV(__nv_bfloat16) }
#undef SP24_LN_FWD_NV
#undef SP24_LN_FWD
    return launch_status();
}

extern "C" int sp24_layernorm_bwd(const void *dy, int dy_dtype, const float *x, const float *gamma, const float *mean,
                                  const float *rstd, float *dx, float *dgamma, float *dbeta, int64_t rows, int64_t d,
                                  void *stream) {
    if (!dy || !x || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta) return SP24_ERR_ARG;
    if (dy_dtype != SP24_F32 && dy_dtype != SP24_F16 && dy_dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (rows <= 0 || d <= 0 || d % 128 || d > 128 * MAXV) return SP24_ERR_SHAPE;
    if (!aligned16(dy) || !aligned16(x) || !aligned16(gamma) || !aligned16(dx)) return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t blocks = (rows + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 2;       // persistent: about one resident block per SM, each ends with 2 d atomics
    if (blocks > cap) blocks = cap;
    const size_t smem = (size_t)2 * 8 * d * sizeof(float);       // at most 64 KB (d = 1024)
    static bool attr_set[3][8][64];
    int dev = 0;
    cudaGetDevice(&dev);
    const int which = dy_dtype == SP24_F32 ? 0 : (dy_dtype == SP24_F16 ? 1 : 2);
#define SP24_LN_BWD(T_, NV_) \
    do { \
        auto kern = layernorm_bwd_kernel<T_, NV_>; \
        if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_set[which][NV_ - 1][dev]) { \
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
                return launch_status(); \
            attr_set[which][NV_ - 1][dev] = true; \
        } \
        kern<<<(unsigned)blocks, 256, smem, st>>>(static_cast<const T_ *>(dy), x, gamma, mean, rstd, dx, dgamma, dbeta, rows); \
    } while (0)
#define SP24_LN_BWD_NV(T_) \
    switch (d / 128) { \
        case 1: SP24_LN_BWD(T_, 1); break; case 2: SP24_LN_BWD(T_, 2); break; case 3: SP24_LN_BWD(T_, 3); break; \
        case 4: SP24_LN_BWD(T_, 4); break; case 5: SP24_LN_BWD(T_, 5); break; case 6: SP24_LN_BWD(T_, 6); break; \
        case 7: SP24_LN_BWD(T_, 7); break; default: SP24_LN_BWD(T_, 8); break; \
    }
    if (dy_dtype == SP24_F32) { SP24_LN_BWD_NV(float) }
    else if (dy_dtype == SP24_F16) { SP24_LN_BWD_NV(__half) }
    else { SP24_LN_BWD_NV(__nv_bfloat16) }
#undef SP24_LN_BWD_NV
#undef SP24_LN_BWD
    return launch_status();
}

extern "C" int sp24_cross_entropy_fwd(const void *logits, int dtype, const int64_t *targets, float *lse, float *loss, int64_t rows,
                                      int64_t v, int64_t ld, void *stream) {
    if (!logits || !targets || !lse || !loss) return SP24_ERR_ARG;
    if (dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (rows <= 0 || v <= 0 || v % 8) return SP24_ERR_SHAPE;
    if (ld < v || ld % 8) return SP24_ERR_STRIDE;
    if (!aligned16(logits)) return SP24_ERR_ALIGN;
    if (rows > 0x7FFFFFFF) return SP24_ERR_TOO_LARGE;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == SP24_F16)
        ce_fwd_kernel<__half><<<(unsigned)rows, 256, 0, st>>>(static_cast<const __half *>(logits), targets, lse, loss, v, ld);
    else
        ce_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(logits), targets, lse, loss, v, ld);
    return launch_status();
}

extern "C" int sp24_cross_entropy_bwd(const void *logits, int dtype, const int64_t *targets, const float *lse,
                                      const float *upstream, float scale, void *dlogits, int64_t rows, int64_t v, int64_t ld,
                                      int64_t ld_out, void *stream) {
    if (!logits || !targets || !lse || !dlogits) return SP24_ERR_ARG;
    if (dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (rows <= 0 || v <= 0 || v % 8) return SP24_ERR_SHAPE;
    if (ld < v || ld % 8 || ld_out < v || ld_out % 8) return SP24_ERR_STRIDE;
    if (!aligned16(logits) || !aligned16(dlogits)) return SP24_ERR_ALIGN;
    if (rows > 0x7FFFFFFF) return SP24_ERR_TOO_LARGE;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == SP24_F16)
        ce_bwd_kernel<__half><<<(unsigned)rows, 256, 0, st>>>(static_cast<const __half *>(logits), targets, lse, upstream, scale,
                                                             static_cast<__half *>(dlogits), v, ld, ld_out);
    else
        ce_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(logits), targets, lse, upstream,
                                                                    scale, static_cast<__nv_bfloat16 *>(dlogits), v, ld, ld_out);
    return launch_status();
}
