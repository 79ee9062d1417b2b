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

// y = (r - mean) * rstd * gamma + beta with r = x (+ delta, then also written to res_out as float32): statistics in
// float32, two passes over the registers.  delta / res_out: both null, or the branch output that joins the residual
// stream in front of this norm (same element type as the output) and the new residual stream.
template <typename TOut, int NV>
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const float *x, const TOut *delta, float *res_out, const float *gamma,
                                                            const float *beta, TOut *out, float *mean_out, float *rstd_out,
                                                            int64_t rows, float eps) {
    constexpr int d = NV * 128, nv = NV;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float4 v[NV];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (i < nv) {
            const int64_t at = row * d + (i * 32 + lane) * 4;
            v[i] = load4<float>(x + at);
            if (delta) {
                const float4 dl = load4<TOut>(delta + at);
                v[i] = make_float4(v[i].x + dl.x, v[i].y + dl.y, v[i].z + dl.z, v[i].w + dl.w);
                store4<float>(res_out + at, v[i].x, v[i].y, v[i].z, v[i].w);
            }
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

// dx = rstd * (g dy - mean(g dy) - xhat mean(g dy xhat)) (+ dres);  dgamma += sum_rows dy xhat;  dbeta += sum_rows dy.
// dres (optional): the gradient that reaches the norm's input along the residual stream, added before the store;
// ddelta (optional): the same dx again in dy's element type, the gradient of the branch that was added in front.
// Persistent warps: each walks rows warp, warp + nwarps, ... and keeps its column sums in its own slice of shared
// memory; one reduction over the block's eight warps at the end, then one atomic per column and block.
// The kernel is bound by the latency of a row's two dependent memory round trips (statistics, then outputs), so what
// counts is the number of rows in flight: with the column sums in shared memory instead of registers a thread needs
// under 64 registers and an SM holds 32 warps instead of 16; they form ONE block per SM (LnBwdWarps<NV> warps: 32 up
// to d = 768, 16 beyond, by the shared memory their sums take), so that the closing atomics are one set per SM.
// A row is read twice: once for the two row-wide sums and the column sums, once more (L1 / L2) together with the
// residual-stream gradient.  (L2 prefetches of that gradient and of the warp's next row made it slower.)
template <int NV> struct LnBwdWarps { static constexpr int value = NV <= 6 ? 32 : 16; };

template <typename TDy, int NV>
__global__ void __launch_bounds__(32 * LnBwdWarps<NV>::value, 1)
    layernorm_bwd_kernel(const TDy *dy, const float *x, const float *gamma, const float *mean, const float *rstd, const float *dres,
                         float *dx, TDy *ddelta, float *dgamma, float *dbeta, int64_t rows) {
    extern __shared__ float red[];           // 2 x W x d floats: [gamma sums | beta sums] x warp x column
    constexpr int d = NV * 128, W = LnBwdWarps<NV>::value;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float4 *ag = reinterpret_cast<float4 *>(red + warp * d) + lane;
    float4 *ab = reinterpret_cast<float4 *>(red + W * d + warp * d) + lane;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        ag[i * 32] = make_float4(0.f, 0.f, 0.f, 0.f);
        ab[i * 32] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float4 *g4 = reinterpret_cast<const float4 *>(gamma) + lane;
    const int64_t nwarps = (int64_t)gridDim.x * W;
    for (int64_t row = (int64_t)blockIdx.x * W + warp; row < rows; row += nwarps) {
        const float mu = mean[row], rs = rstd[row];
        const float shift = -mu * rs;
        const int64_t base = row * d + lane * 4;
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float4 xv = load4<float>(x + base + i * 128);
            const float4 dv = load4<TDy>(dy + base + i * 128);
            const float4 g = __ldg(g4 + i * 32);
            const float4 xh = make_float4(fmaf(xv.x, rs, shift), fmaf(xv.y, rs, shift), fmaf(xv.z, rs, shift), fmaf(xv.w, rs, shift));
            const float4 gy = make_float4(dv.x * g.x, dv.y * g.y, dv.z * g.z, dv.w * g.w);
            s1 += (gy.x + gy.y) + (gy.z + gy.w);
            s2 += (gy.x * xh.x + gy.y * xh.y) + (gy.z * xh.z + gy.w * xh.w);
            float4 a = ag[i * 32], b = ab[i * 32];
            a.x = fmaf(dv.x, xh.x, a.x); a.y = fmaf(dv.y, xh.y, a.y); a.z = fmaf(dv.z, xh.z, a.z); a.w = fmaf(dv.w, xh.w, a.w);
            b.x += dv.x; b.y += dv.y; b.z += dv.z; b.w += dv.w;
            ag[i * 32] = a;
            ab[i * 32] = b;
        }
        const float m1 = warp_sum(s1) / (float)d, m2 = warp_sum(s2) / (float)d;
        const float c1 = -rs * m1, c2 = -rs * m2;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int64_t at = base + i * 128;
            const float4 xv = load4<float>(x + at);
            const float4 dv = load4<TDy>(dy + at);
            const float4 g = __ldg(g4 + i * 32);
            // rs (g dy - m1 - xhat m2) = (rs g) dy + c1 + c2 xhat
            float4 o = make_float4(fmaf(c2, fmaf(xv.x, rs, shift), fmaf(rs * g.x, dv.x, c1)),
                                   fmaf(c2, fmaf(xv.y, rs, shift), fmaf(rs * g.y, dv.y, c1)),
                                   fmaf(c2, fmaf(xv.z, rs, shift), fmaf(rs * g.z, dv.z, c1)),
                                   fmaf(c2, fmaf(xv.w, rs, shift), fmaf(rs * g.w, dv.w, c1)));
            if (dres) {
                const float4 r = load4<float>(dres + at);
                o = make_float4(o.x + r.x, o.y + r.y, o.z + r.z, o.w + r.w);
            }
            store4<float>(dx + at, o.x, o.y, o.z, o.w);
            if (ddelta) store4<TDy>(ddelta + at, o.x, o.y, o.z, o.w);
        }
    }
    const float *rg = red, *rb = red + W * d;
    __syncthreads();
    for (int c = threadIdx.x; c < d; c += 32 * W) {
        float sg = 0.f, sb = 0.f;
#pragma unroll
        for (int w = 0; w < W; ++w) {
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
        const int64_t tgt = targets[row];
        loss[row] = (tgt >= 0 && tgt < v) ? l - Elem<T>::to_f32(p[tgt]) : 0.f;     // a target outside [0, v) reads nothing
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

// Forward and gradient in one kernel: the row is read from HBM once and the gradient for an upstream gradient of 1 is
// written in the same launch: dlogits[row, c] = (exp(logits[row, c] - lse[row]) - [c == target[row]]) * scale.
// STAGED: the whole row is brought into shared memory by asynchronous 16-byte copies, all issued before the first
// wait (one memory round trip per row and block, two blocks per SM), and the three passes (maximum, sum, gradient)
// read it from there; otherwise (rows beyond the shared-memory budget) the passes re-read the row, mostly from L2.
// The kernel is bound by instruction issue and the exponential unit, not by memory, unless the passes are lean: the
// maximum is taken on packed 16-bit pairs, an exponential is one multiply-add (log2 e and the offset folded) plus one
// ex2, the gradient's scale rides in that offset, and the target's -1 is patched in by one thread afterwards instead
// of being compared for in every element.
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <typename T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
    typedef __nv_bfloat162 type;
    static __device__ __forceinline__ void unpack(uint32_t w, float &lo, float &hi) {
        lo = __uint_as_float(w << 16);
        hi = __uint_as_float(w & 0xFFFF0000u);
    }
    static __device__ __forceinline__ type lowest() { return __float2bfloat162_rn(-INFINITY); }
};
template <> struct Pair16<__half> {
    typedef __half2 type;
    static __device__ __forceinline__ void unpack(uint32_t w, float &lo, float &hi) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
        lo = f.x;
        hi = f.y;
    }
    static __device__ __forceinline__ type lowest() { return __float2half2_rn(-INFINITY); }
};

template <typename T, bool STAGED>
__global__ void __launch_bounds__(512) ce_fused_kernel(const T *logits, const int64_t *targets, float *lse, float *loss,
                                                       float scale, T *dlogits, int64_t v, int64_t ld, int64_t ld_out) {
    extern __shared__ uint4 staged[];        // the row as 16-byte pieces (STAGED only)
    __shared__ float scratch[16];
    typedef typename Pair16<T>::type P2;
    constexpr float L2E = 1.4426950408889634f;
    const int64_t row = blockIdx.x;
    const uint4 *p = reinterpret_cast<const uint4 *>(logits + row * ld);
    uint4 *q = reinterpret_cast<uint4 *>(dlogits + row * ld_out);
    const int nvec = (int)(v / 8);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (STAGED) {
        for (int i = threadIdx.x; i < nvec; i += 512) {
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(staged + i);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(p + i) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        // every pass below gives a thread the pieces it copied itself: no barrier needed before reading them
    }
    // pass 1: maximum, on packed pairs (exact)
    P2 m2 = Pair16<T>::lowest();
    for (int i = threadIdx.x; i < nvec; i += 512) {
        const uint4 r = STAGED ? staged[i] : p[i];
        const P2 *h = reinterpret_cast<const P2 *>(&r);
        m2 = __hmax2(__hmax2(m2, h[0]), __hmax2(h[1], __hmax2(h[2], h[3])));
    }
    float lo, hi;
    Pair16<T>::unpack(*reinterpret_cast<const uint32_t *>(&m2), lo, hi);
    const float wm = warp_max(fmaxf(lo, hi));
    if (lane == 0) scratch[warp] = wm;
    __syncthreads();
    float gm = scratch[0];
#pragma unroll
    for (int w = 1; w < 16; ++w) gm = fmaxf(gm, scratch[w]);
    __syncthreads();
    // pass 2: sum of exp(x - max)
    const float off1 = -gm * L2E;
    float s0 = 0.f, s1 = 0.f;
    for (int i = threadIdx.x; i < nvec; i += 512) {
        const uint4 r = STAGED ? staged[i] : p[i];
        const uint32_t *w = reinterpret_cast<const uint32_t *>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            Pair16<T>::unpack(w[j], lo, hi);
            s0 += ex2_fast(fmaf(lo, L2E, off1));
            s1 += ex2_fast(fmaf(hi, L2E, off1));
        }
    }
    const float ws = warp_sum(s0 + s1);
    if (lane == 0) scratch[warp] = ws;
    __syncthreads();
    float gs = 0.f;
#pragma unroll
    for (int w = 0; w < 16; ++w) gs += scratch[w];
    const float l = gm + logf(gs);
    const int64_t tgt = targets[row];
    const bool tgt_ok = tgt >= 0 && tgt < v;
    const T *pe = reinterpret_cast<const T *>(p);
    if (threadIdx.x == 0) {
        lse[row] = l;
        loss[row] = tgt_ok ? l - Elem<T>::to_f32(pe[tgt]) : 0.f;      // a target outside [0, v) reads nothing
    }
    // pass 3: scale * exp(x - lse) = ex2(x log2 e - lse log2 e + log2 scale)   (scale = 0 gives ex2(-inf) = 0)
    const float off2 = fmaf(-l, L2E, log2f(scale));
    for (int i = threadIdx.x; i < nvec; i += 512) {
        const uint4 r = STAGED ? staged[i] : p[i];
        const uint32_t *w = reinterpret_cast<const uint32_t *>(&r);
        uint4 o;
        uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            Pair16<T>::unpack(w[j], lo, hi);
            ow[j] = Elem<T>::pack2(ex2_fast(fmaf(lo, L2E, off2)), ex2_fast(fmaf(hi, L2E, off2)));
        }
        q[i] = o;
    }
    if (tgt_ok) {
        __syncthreads();                                            // the vector holding the target's entry is written
        if (threadIdx.x == 0) {
            const float x = Elem<T>::to_f32(STAGED ? reinterpret_cast<const T *>(staged)[tgt] : pe[tgt]);
            const uint16_t one = (uint16_t)(Elem<T>::pack2(ex2_fast(fmaf(x, L2E, off2)) - scale, 0.f) & 0xFFFFu);
            reinterpret_cast<uint16_t *>(q)[tgt] = one;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// token + position embedding: one warp per token
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void red_add_v4(float *addr, const float4 &v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// out[row, :] = wte[ids[row], :] + wpe[row % t, :]; an id outside [0, vocab) contributes zeros
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const int64_t *ids, const float *wte, const float *wpe, float *out,
                                                            int64_t rows, int64_t t, int64_t d, int64_t vocab) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int64_t id = ids[row];
    const bool ok = id >= 0 && id < vocab;
    const float *a = wte + (ok ? id : 0) * d, *b = wpe + (row % t) * d;
    for (int64_t c = lane * 4; c < d; c += 128) {
        const float4 u = ok ? load4<float>(a + c) : make_float4(0.f, 0.f, 0.f, 0.f), v = load4<float>(b + c);
        store4<float>(out + row * d + c, u.x + v.x, u.y + v.y, u.z + v.z, u.w + v.w);
    }
}

// dwte[ids[row], :] += dx[row, :];  dwpe[row % t, :] += dx[row, :]   (float32 vector reductions in L2; the order in
// which rows that share a token or a position are added is not fixed)
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const float *dx, const int64_t *ids, float *dwte, float *dwpe,
                                                            int64_t rows, int64_t t, int64_t d, int64_t vocab) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int64_t id = ids[row];
    const bool ok = id >= 0 && id < vocab;
    float *a = dwte + (ok ? id : 0) * d, *b = dwpe + (row % t) * d;
    for (int64_t c = lane * 4; c < d; c += 128) {
        const float4 v = load4<float>(dx + row * d + c);
        if (ok) red_add_v4(a + c, v);
        red_add_v4(b + c, v);
    }
}

// ---------------------------------------------------------------------------------------------
// GELU (tanh form) over 16-bit tensors: 16-byte accesses, float32 arithmetic, tanh.approx
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float gelu_f(float x) {
    const float u = x * fmaf(0.0356774081f, x * x, 0.7978845608f);          // sqrt(2/pi) (x + 0.044715 x^3)
    return 0.5f * x * (1.f + tanh_fast(u));
}
__device__ __forceinline__ float dgelu_f(float x) {
    const float x2 = x * x;
    const float t = tanh_fast(x * fmaf(0.0356774081f, x2, 0.7978845608f));
    // 0.5 (1 + t) + 0.5 x (1 - t^2) sqrt(2/pi) (1 + 3 * 0.044715 x^2)
    return fmaf(0.5f * x * (1.f - t * t), fmaf(0.1070322243f, x2, 0.7978845608f), 0.5f * (1.f + t));
}

// BWD: out = dy * gelu'(x); otherwise out = gelu(x).  Two 16-byte pieces per thread and trip.
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) gelu_kernel(const uint4 *x, const uint4 *dy, uint4 *out, int64_t nvec) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nvec; i += 2 * stride) {
        const int64_t i2 = i + stride;
        const bool two = i2 < nvec;
        uint4 a0 = x[i], a1, g0, g1;
        if (two) a1 = x[i2];
        if (BWD) {
            g0 = dy[i];
            if (two) g1 = dy[i2];
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (h == 1 && !two) break;
            const uint4 &a = h ? a1 : a0;
            const uint4 &g = h ? g1 : g0;
            const uint32_t *aw = reinterpret_cast<const uint32_t *>(&a), *gw = reinterpret_cast<const uint32_t *>(&g);
            uint4 o;
            uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float lo, hi;
                Pair16<T>::unpack(aw[j], lo, hi);
                if (BWD) {
                    float glo, ghi;
                    Pair16<T>::unpack(gw[j], glo, ghi);
                    ow[j] = Elem<T>::pack2(glo * dgelu_f(lo), ghi * dgelu_f(hi));
                } else {
                    ow[j] = Elem<T>::pack2(gelu_f(lo), gelu_f(hi));
                }
            }
            out[h ? i2 : i] = o;
        }
    }
}

// g *= *factor unless *factor == 1 (the usual case: nothing is read or written then)
template <typename T>
__global__ void __launch_bounds__(256) scale_unless_one_kernel(T *g, const float *factor, int64_t nvec) {
    const float f = *factor;
    if (f == 1.f) return;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * 256) {
        uint4 r = reinterpret_cast<uint4 *>(g)[i];
        float x[8];
        unpack8<T>(r, x);
        uint32_t *w = reinterpret_cast<uint32_t *>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = Elem<T>::pack2(x[2 * j] * f, x[2 * j + 1] * f);
        reinterpret_cast<uint4 *>(g)[i] = r;
    }
}

}  // namespace
}  // namespace sp24

using namespace sp24;

static int layernorm_fwd_impl(const float *x, const void *delta, float *res_out, const float *gamma, const float *beta, void *out,
                              int out_dtype, float *mean, float *rstd, int64_t rows, int64_t d, float eps, void *stream) {
    if (!x || !gamma || !beta || !out || !mean || !rstd) return SP24_ERR_ARG;
    if ((delta == nullptr) != (res_out == nullptr)) return SP24_ERR_ARG;
    if (out_dtype != SP24_F32 && out_dtype != SP24_F16 && out_dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (rows <= 0 || d <= 0 || d % 128 || d > 128 * MAXV) return SP24_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(gamma) || !aligned16(beta) || !aligned16(out) || !aligned16(delta) || !aligned16(res_out))
        return SP24_ERR_ALIGN;
    if (!(eps >= 0.f)) return SP24_ERR_ARG;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (unsigned)((rows + 7) / 8);
#define SP24_LN_FWD(T_, NV_) \
    layernorm_fwd_kernel<T_, NV_><<<blocks, 256, 0, st>>>(x, static_cast<const T_ *>(delta), res_out, gamma, beta, \
                                                          static_cast<T_ *>(out), mean, rstd, rows, eps)
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

extern "C" int sp24_layernorm_fwd(const float *x, const float *gamma, const float *beta, void *out, int out_dtype, float *mean,
                                  float *rstd, int64_t rows, int64_t d, float eps, void *stream) {
    return layernorm_fwd_impl(x, nullptr, nullptr, gamma, beta, out, out_dtype, mean, rstd, rows, d, eps, stream);
}

extern "C" int sp24_add_layernorm_fwd(const float *x, const void *delta, float *res_out, const float *gamma, const float *beta,
                                      void *out, int out_dtype, float *mean, float *rstd, int64_t rows, int64_t d, float eps,
                                      void *stream) {
    if (!delta || !res_out) return SP24_ERR_ARG;
    return layernorm_fwd_impl(x, delta, res_out, gamma, beta, out, out_dtype, mean, rstd, rows, d, eps, stream);
}

static int layernorm_bwd_impl(const void *dy, int dy_dtype, const float *dres, const float *x, const float *gamma, const float *mean,
                              const float *rstd, float *dx, void *ddelta, float *dgamma, float *dbeta, int64_t rows, int64_t d,
                              void *stream) {
    if (!dy || !x || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta) return SP24_ERR_ARG;
    if (dy_dtype != SP24_F32 && dy_dtype != SP24_F16 && dy_dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (rows <= 0 || d <= 0 || d % 128 || d > 128 * MAXV) return SP24_ERR_SHAPE;
    if (!aligned16(dy) || !aligned16(x) || !aligned16(gamma) || !aligned16(dx) || !aligned16(dres) || !aligned16(ddelta))
        return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    static bool attr_set[3][8][64];
    int dev = 0;
    cudaGetDevice(&dev);
    const int which = dy_dtype == SP24_F32 ? 0 : (dy_dtype == SP24_F16 ? 1 : 2);
#define SP24_LN_BWD(T_, NV_) \
    do { \
        constexpr int W = LnBwdWarps<NV_>::value; \
        const size_t smem = (size_t)2 * W * d * sizeof(float);           /* 32 warps x 6 KB = 192 KB at d = 768 */ \
        auto kern = layernorm_bwd_kernel<T_, NV_>; \
        if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_set[which][NV_ - 1][dev]) { \
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
                return launch_status(); \
            attr_set[which][NV_ - 1][dev] = true; \
        } \
        int resident = 0;                                                /* persistent grid: every block resident at once */ \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, 32 * W, smem) != cudaSuccess || resident < 1) resident = 1; \
        int64_t blocks = (rows + W - 1) / W; \
        const int64_t cap = (int64_t)sm_count() * resident; \
        if (blocks > cap) blocks = cap; \
        kern<<<(unsigned)blocks, 32 * W, smem, st>>>(static_cast<const T_ *>(dy), x, gamma, mean, rstd, dres, dx, \
                                                  static_cast<T_ *>(ddelta), dgamma, dbeta, rows); \
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

extern "C" int sp24_layernorm_bwd(const void *dy, int dy_dtype, const float *x, const float *gamma, const float *mean,
                                  const float *rstd, float *dx, float *dgamma, float *dbeta, int64_t rows, int64_t d,
                                  void *stream) {
    return layernorm_bwd_impl(dy, dy_dtype, nullptr, x, gamma, mean, rstd, dx, nullptr, dgamma, dbeta, rows, d, stream);
}

extern "C" int sp24_add_layernorm_bwd(const void *dy, int dy_dtype, const float *dres, const float *x, const float *gamma,
                                      const float *mean, const float *rstd, float *dx, void *ddelta, float *dgamma, float *dbeta,
                                      int64_t rows, int64_t d, void *stream) {
    return layernorm_bwd_impl(dy, dy_dtype, dres, x, gamma, mean, rstd, dx, ddelta, dgamma, dbeta, rows, d, stream);
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

template <typename T>
static int ce_fused_launch(const void *logits, const int64_t *targets, float *lse, float *loss, float scale, void *dlogits,
                           int64_t rows, int64_t v, int64_t ld, int64_t ld_out, cudaStream_t st) {
    const size_t row_bytes = (size_t)v * sizeof(T);
    const bool staged = row_bytes <= 110 * 1024;           // two resident blocks per SM
    if (staged) {
        auto kern = ce_fused_kernel<T, true>;
        static bool attr_set[64];
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !attr_set[dev]) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024) != cudaSuccess)
                return launch_status();
            attr_set[dev] = true;
        }
        kern<<<(unsigned)rows, 512, row_bytes, st>>>(static_cast<const T *>(logits), targets, lse, loss, scale,
                                                     static_cast<T *>(dlogits), v, ld, ld_out);
    } else {
        ce_fused_kernel<T, false><<<(unsigned)rows, 512, 0, st>>>(static_cast<const T *>(logits), targets, lse, loss, scale,
                                                                  static_cast<T *>(dlogits), v, ld, ld_out);
    }
    return launch_status();
}

extern "C" int sp24_cross_entropy_fused(const void *logits, int dtype, const int64_t *targets, float *lse, float *loss, float scale,
                                        void *dlogits, int64_t rows, int64_t v, int64_t ld, int64_t ld_out, void *stream) {
    if (!logits || !targets || !lse || !loss || !dlogits) return SP24_ERR_ARG;
    if (dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (rows <= 0 || v <= 0 || v % 8) return SP24_ERR_SHAPE;
    if (ld < v || ld % 8 || ld_out < v || ld_out % 8) return SP24_ERR_STRIDE;
    if (!aligned16(logits) || !aligned16(dlogits)) return SP24_ERR_ALIGN;
    if (!(scale >= 0.f) || !(scale < INFINITY)) return SP24_ERR_ARG;
    if (rows > 0x7FFFFFFF || v / 8 > 0x7FFFFFFF) return SP24_ERR_TOO_LARGE;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == SP24_F16 ? ce_fused_launch<__half>(logits, targets, lse, loss, scale, dlogits, rows, v, ld, ld_out, st)
                             : ce_fused_launch<__nv_bfloat16>(logits, targets, lse, loss, scale, dlogits, rows, v, ld, ld_out, st);
}

extern "C" int sp24_scale_unless_one(void *g, int dtype, const float *factor, int64_t count, void *stream) {
    if (!g || !factor) return SP24_ERR_ARG;
    if (dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (count <= 0 || count % 8) return SP24_ERR_SHAPE;
    if (!aligned16(g)) return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t nvec = count / 8;
    int64_t blocks = (nvec + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (dtype == SP24_F16)
        scale_unless_one_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<__half *>(g), factor, nvec);
    else
        scale_unless_one_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(static_cast<__nv_bfloat16 *>(g), factor, nvec);
    return launch_status();
}

extern "C" int sp24_embedding_fwd(const int64_t *ids, const float *wte, const float *wpe, float *out, int64_t rows, int64_t t,
                                  int64_t d, int64_t vocab, void *stream) {
    if (!ids || !wte || !wpe || !out) return SP24_ERR_ARG;
    if (rows <= 0 || t <= 0 || d <= 0 || d % 4 || vocab <= 0) return SP24_ERR_SHAPE;
    if (!aligned16(wte) || !aligned16(wpe) || !aligned16(out)) return SP24_ERR_ALIGN;
    if ((rows + 7) / 8 > 0x7FFFFFFF) return SP24_ERR_TOO_LARGE;
    if (int rc = check_device()) return rc;
    embedding_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(ids, wte, wpe, out, rows, t, d,
                                                                                                     vocab);
    return launch_status();
}

extern "C" int sp24_embedding_bwd(const float *dx, const int64_t *ids, float *dwte, float *dwpe, int64_t rows, int64_t t, int64_t d,
                                  int64_t vocab, void *stream) {
    if (!dx || !ids || !dwte || !dwpe) return SP24_ERR_ARG;
    if (rows <= 0 || t <= 0 || d <= 0 || d % 4 || vocab <= 0) return SP24_ERR_SHAPE;
    if (!aligned16(dx) || !aligned16(dwte) || !aligned16(dwpe)) return SP24_ERR_ALIGN;
    if ((rows + 7) / 8 > 0x7FFFFFFF) return SP24_ERR_TOO_LARGE;
    if (int rc = check_device()) return rc;
    embedding_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(dx, ids, dwte, dwpe, rows, t, d,
                                                                                                     vocab);
    return launch_status();
}

extern "C" int sp24_gelu(const void *x, const void *dy, void *out, int dtype, int64_t count, void *stream) {
    if (!x || !out) return SP24_ERR_ARG;
    if (dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (count <= 0 || count % 8) return SP24_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(dy) || !aligned16(out)) return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t nvec = count / 8;
    int64_t blocks = (nvec + 511) / 512;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    const uint4 *xv = static_cast<const uint4 *>(x), *gv = static_cast<const uint4 *>(dy);
    uint4 *ov = static_cast<uint4 *>(out);
    if (dtype == SP24_F16) {
        if (dy) gelu_kernel<__half, true><<<(unsigned)blocks, 256, 0, st>>>(xv, gv, ov, nvec);
        else gelu_kernel<__half, false><<<(unsigned)blocks, 256, 0, st>>>(xv, gv, ov, nvec);
    } else {
        if (dy) gelu_kernel<__nv_bfloat16, true><<<(unsigned)blocks, 256, 0, st>>>(xv, gv, ov, nvec);
        else gelu_kernel<__nv_bfloat16, false><<<(unsigned)blocks, 256, 0, st>>>(xv, gv, ov, nvec);
    }
    return launch_status();
}
