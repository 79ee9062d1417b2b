// 2:4 sparse GEMM for sm_100a:  D (Ms x N) = A_sparse (Ms x K) * B (K x N)  [+ bias per row] [activation]
//
// The sparse operand is always the tensor-core "A" operand of tcgen05.mma.sp: compressed values are
// staged in shared memory by TMA (128-byte swizzle), its metadata goes shared memory -> tensor memory
// with tcgen05.cp, the dense operand B is staged by TMA, accumulators live in tensor memory and are read
// back with tcgen05.ld by eight epilogue warps.
//
// Warp roles in a CTA of 320 threads: warp 0 = TMA producer (one elected lane), warp 1 = tensor-memory
// allocation + MMA issue (one elected lane), warps 2..9 = epilogue (two per TMEM lane quadrant, half of the
// columns each).
// One CTA computes one 128 x BN output tile; the K loop runs over stages of 128 bytes of compressed A
// per row (logical K 128 for 16-bit types, 256 for 8-bit types) through a STAGES-deep mbarrier ring.
//
// Every wait on an mbarrier is bounded: when a wait gives up, the CTA records a code in *status,
// raises a shared abort flag that cuts all other waits short, drains its own copies in flight (again
// bounded), frees its tensor memory and returns.  Nothing traps.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>

#include "sp24_common.cuh"

namespace sp24 {
namespace {

constexpr int BM = 128;            // rows of the sparse operand per CTA tile (= TMEM lanes)
constexpr int A_STAGE_BYTES = BM * 128;
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // polls of mbarrier.try_wait before a wait gives up

// ------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when it gave up (limit reached or another role raised the abort flag).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code,
                                          uint32_t limit = WAIT_LIMIT) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 0xFFu) == 0xFFu && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (status) atomicCAS(status, 0, code);
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_128x128b(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
template <bool F8>
__device__ __forceinline__ void mma_sp(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t e_tmem, uint32_t idesc,
                                       uint32_t accumulate, int int8 = 0) {
    if constexpr (F8) {
        if (int8) {   // signed 8-bit integers, 32-bit integer accumulators; same operand geometry as fp8
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
                "tcgen05.mma.sp.cta_group::1.kind::i8 [%0], %1, %2, [%3], %4, p;\n\t}" ::"r"(d_tmem),
                "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
                : "memory");
        } else {
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
                "tcgen05.mma.sp.cta_group::1.kind::f8f6f4 [%0], %1, %2, [%3], %4, p;\n\t}" ::"r"(d_tmem),
                "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
                : "memory");
        }
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
            "tcgen05.mma.sp.cta_group::1.kind::f16 [%0], %1, %2, [%3], %4, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
// fp32 vector reduction into global memory (sm_90+), address 16-byte aligned
__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets (all >> 4),
// descriptor version 1, swizzle mode in bits 61..63 (0 none, 2 = 128-byte).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)swizzle << 61;
    return d;
}

struct SpmmParams {
    const void *e_tc;       // metadata in tensor-core atom order
    void *out;
    const void *bias;       // per sparse row (output feature), in the output type, or null
    int64_t ms, n, k;       // sparse rows, dense columns, logical K
    int64_t ld_out;
    int64_t k_atoms;        // number of 128-column metadata atoms per 128-row block (K padded up)
    int *status;
    uint32_t idesc;         // instruction descriptor without the metadata selector bits
    int activation;         // 0 none, 1 relu, 2 silu, 3 gelu (tanh form)
    unsigned long long *trace;  // timing trace of CTA 0: only developer builds (-DSP24_TRACE_BUILD) ever set it
    int int8;               // 8-bit operands are signed integers (kind::i8, int32 accumulators and output)
    int k_splits;           // work units per tile along K (> 1 only for the accumulating fp32 output)
    int mblk_per_tile;      // 128-row blocks per tile: 2 (B staged once per 256 rows) or 1 (more, smaller tiles)
    float alpha;            // float32 outputs: D = alpha * (A * B) (+ bias); 16-bit and integer outputs ignore it
    int bias_f32;           // bias holds float32 values instead of values of the output type
    void *aux;              // fused MLP epilogues (CTA-pair kernel): second tensor shaped and pitched like out
    int64_t ld_aux;
};

// Epilogue forms of the CTA-pair kernel.  PRE_GELU: aux = h = acc + bias rounded to the output type, out = gelu(h)
// (tanh form, evaluated on the rounded h, so that out is exactly the activation of what aux holds).  DGELU: out =
// acc * gelu'(aux): the input gradient of a layer whose input was gelu(aux), written as the gradient of aux.
enum { EPI_PLAIN = 0, EPI_PRE_GELU = 1, EPI_DGELU = 2 };

__device__ __forceinline__ float tanh_fast(float v) {
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
// GELU, tanh form: 0.5 v (1 + tanh(u)), u = sqrt(2 / pi) (v + 0.044715 v^3); one MUFU per value
__device__ __forceinline__ float gelu_tanh(float v) {
    const float t = tanh_fast(0.7978845608f * fmaf(0.044715f * v * v, v, v));
    return 0.5f * v * (1.f + t);
}
// its derivative: 0.5 (1 + t) + 0.5 v (1 - t^2) sqrt(2 / pi) (1 + 3 * 0.044715 v^2)
__device__ __forceinline__ float gelu_tanh_grad(float v) {
    const float v2 = v * v;
    const float t = tanh_fast(0.7978845608f * fmaf(0.044715f * v2, v, v));
    return 0.5f * (1.f + t) + 0.5f * v * (1.f - t * t) * (0.7978845608f * fmaf(0.134145f, v2, 1.f));
}

template <typename OutT> __device__ __forceinline__ OutT to_out(float v);
template <> __device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ int32_t to_out<int32_t>(float v) { return __float_as_int(v); }
template <typename OutT> __device__ __forceinline__ float from_out(OutT v);
template <> __device__ __forceinline__ float from_out<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float from_out<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float from_out<float>(float v) { return v; }
template <> __device__ __forceinline__ float from_out<int32_t>(int32_t) { return 0.f; }   // no bias for integer GEMMs

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == 1) return v > 0.f ? v : 0.f;
    if (act == 2) return v / (1.f + __expf(-v));
    if (act == 3) {  // GELU, tanh form: v * sigmoid(2 * sqrt(2 / pi) * (v + 0.044715 v^3))
        const float u = 1.5957691216f * (v + 0.044715f * v * v * v);
        return v / (1.f + __expf(-u));
    }
    return v;
}

// The activation is compiled in only for launches that ask for one (template parameter ACT): the plain
// epilogue carries no per-element tests.
template <bool ACT> __device__ __forceinline__ float finish(float v, int act) {
    if constexpr (ACT) return apply_act(v, act);
    return v;
}

// One accumulator word -> one output value.  Integer accumulators pass through untouched: no float operation may
// see their bits (an add of 0.0f would rewrite -0.0 and signalling-NaN patterns, which are ordinary integers).
// float32 outputs are scaled first: alpha * acc + bias in one fused multiply-add (alpha = 1 gives acc + bias exactly).
template <typename OutT, bool ACT> __device__ __forceinline__ OutT emit(uint32_t acc_bits, float bias, int act, float alpha) {
    if constexpr (std::is_same<OutT, int32_t>::value) return (int32_t)acc_bits;
    else if constexpr (std::is_same<OutT, float>::value) return finish<ACT>(fmaf(__uint_as_float(acc_bits), alpha, bias), act);
    else return to_out<OutT>(finish<ACT>(__uint_as_float(acc_bits) + bias, act));
}
// the same, as the 32-bit container of a 4-byte output type
template <typename OutT, bool ACT> __device__ __forceinline__ uint32_t emit_bits(uint32_t acc_bits, float bias, int act, float alpha) {
    if constexpr (std::is_same<OutT, int32_t>::value) return acc_bits;
    else return __float_as_uint(finish<ACT>(fmaf(__uint_as_float(acc_bits), alpha, bias), act));
}

__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// trace layout: 3 roles x 256 slots of nanosecond timestamps, CTA 0 only.  Compiled out of the shipped library:
// a developer build (-DSP24_TRACE_BUILD) stores through P.trace, which that build takes from the environment.
#ifdef SP24_TRACE_BUILD
#define SP24_TRACE(role, slot) do { if (P.trace && blockIdx.x == 0 && (slot) < 256) P.trace[(role) * 256 + (slot)] = globaltimer(); } while (0)
#else
#define SP24_TRACE(role, slot) do { } while (0)
#endif

__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Geometry shared by the kernel and its launcher.
template <int BN, bool F8, bool TRANS_OUT, typename OutT> struct SpmmCfg {
    static constexpr int E_BYTES = F8 ? 4096 : 2048;          // metadata of one 128-row block and one stage
    static constexpr int B_BYTES = BN * 256;                  // two 128-byte K atoms per row of B
    static constexpr int STAGE_BYTES = 2 * A_STAGE_BYTES + B_BYTES + 2 * E_BYTES;
    // transposed output: each accumulator is first copied row by row (16-byte stores) into a staging
    // buffer of 128 rows x STG_COLS columns (+16 bytes of padding per row against bank conflicts), then
    // written out column by column
    static constexpr int STG_COLS = sizeof(OutT) == 4 ? 64 : BN;
    static constexpr int STG_ROW_BYTES = STG_COLS * (int)sizeof(OutT) + 16;
    // 16-bit outputs of wide tiles go through the staging buffer in both output orders (the second accumulator
    // waits in registers, so the tensor memory is free again early); narrow tiles keep a third operand stage
    static constexpr bool STAGED16 = sizeof(OutT) == 2 && (TRANS_OUT || BN > 128);
    static constexpr int STG_BYTES = (TRANS_OUT || STAGED16) ? BM * STG_ROW_BYTES : 0;
    static constexpr int AVAIL = 227 * 1024 - 2048 - STG_BYTES;
    static constexpr int STAGES = AVAIL / STAGE_BYTES >= 4 ? 4 : AVAIL / STAGE_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + STG_BYTES + 1024;
    static_assert(STAGES >= 2, "tile too large for a two-stage ring");
    static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
};

// Persistent kernel: CTA c processes tiles c, c + gridDim.x, ... ; a tile is (256 sparse rows) x (BN dense
// columns), computed as two 128-row blocks that share every stage of B.  The operand ring keeps filling
// across tile boundaries; the epilogue drains tensor memory into a staging buffer and releases each
// accumulator as soon as it has been read, so the next tile's MMAs overlap the global stores.
template <int BN, bool F8, bool A_MN, bool B_MN, bool TRANS_OUT, typename OutT, bool ACT>
__global__ void __launch_bounds__(320, 1)
spmm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, SpmmParams P) {
    using Cfg = SpmmCfg<BN, F8, TRANS_OUT, OutT>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int E_BYTES = Cfg::E_BYTES;
    constexpr int OFF_B = 2 * A_STAGE_BYTES, OFF_E = OFF_B + Cfg::B_BYTES;
    constexpr int KSTEPS = 4;                 // MMA instructions per stage and row block (32 bytes of compressed A each)
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int E_COL0 = 2 * BN;            // metadata columns behind the two accumulators
    constexpr int E_SLOT = F8 ? 8 : 4;        // metadata columns of one row block and one stage
    // 16-bit operands with a direct fp32 output: the accumulating form (D += A * B), the only one that splits K
    constexpr bool ACCUM = !F8 && !TRANS_OUT && sizeof(OutT) == 4;
    static_assert(E_COL0 + 4 * E_SLOT <= 512, "tensor memory columns exhausted");
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "invalid tile width");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 3];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles_n = (int)((P.n + BN - 1) / BN);
    const int n_mblocks = (int)(P.ms / BM);
    const int mpt = P.mblk_per_tile;
    // tile index -> (row tile, column tile) with the row tile varying fastest: the CTAs running at one time
    // cover whole rows of the transposed output (long contiguous runs in DRAM) and share their B tiles in L2
    const int n_tiles_m = (n_mblocks + mpt - 1) / mpt;
    const int n_tiles = n_tiles_n * n_tiles_m;
    // work unit u = (tile u % n_tiles, K slice u / n_tiles); one slice unless the output accumulates
    const int n_units = n_tiles * P.k_splits;
    const int logical_k_per_stage = F8 ? 256 : 128;
    const int k_iters = (int)((P.k + logical_k_per_stage - 1) / logical_k_per_stage);

    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t tmem_full = smem_u32(&bars[2 * STAGES]), tmem_empty0 = smem_u32(&bars[2 * STAGES + 1]);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty0, 8);      // one arrival per epilogue warp
        mbar_init(tmem_empty0 + 8, 8);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_smem), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int g = 0;  // stages issued so far (ring position across tiles)
            bool ok = true;
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                const int tile = unit % n_tiles, ks = unit / n_tiles;
                const int it0 = (int)((int64_t)ks * k_iters / P.k_splits), it1 = (int)((int64_t)(ks + 1) * k_iters / P.k_splits);
                const int mblk0 = (tile % n_tiles_m) * mpt;
                const int n_mblk = (n_mblocks - mblk0) >= mpt ? mpt : 1;
                const int64_t m0 = (int64_t)mblk0 * BM, n0 = (int64_t)(tile / n_tiles_m) * BN;
                const uint32_t stage_tx = (uint32_t)(n_mblk * (A_STAGE_BYTES + E_BYTES) + Cfg::B_BYTES);
                for (int it = it0; it < it1; ++it, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (g / STAGES) & 1;
                    if (g >= STAGES && !mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, P.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint32_t sb = sa + OFF_B;
                    const uint32_t se = sa + OFF_E;
                    const uint32_t full = full0 + 8 * s;
                    mbar_expect_tx(full, stage_tx);
                    for (int mb = 0; mb < n_mblk; ++mb) {
                        const int mrow = (int)m0 + mb * BM;
                        const uint32_t sam = sa + mb * A_STAGE_BYTES;
                        // compressed A: 128 rows x 128 bytes
                        if constexpr (!A_MN) {
                            tma_load_2d(sam, &map_a, it * (F8 ? 128 : 64), mrow, full);
                        } else {
                            tma_load_2d(sam, &map_a, mrow, it * 64, full);
                            tma_load_2d(sam + 8192, &map_a, mrow + 64, it * 64, full);
                        }
                        // metadata atoms of this 128-row block
                        const uint8_t *e_src = static_cast<const uint8_t *>(P.e_tc) +
                                               ((size_t)(mblk0 + mb) * P.k_atoms + (size_t)it * (E_BYTES / 2048)) * 2048;
                        bulk_load(se + mb * E_BYTES, e_src, E_BYTES, full);
                    }
                    // dense B: BN rows x 2 atoms of 128 bytes (K-major) or column blocks of 64 x 128 K-rows (MN-major)
                    if constexpr (!B_MN) {
                        const int kx = it * (F8 ? 256 : 128);
                        tma_load_2d(sb, &map_b, kx, (int)n0, full);
                        tma_load_2d(sb + BN * 128, &map_b, kx + (F8 ? 128 : 64), (int)n0, full);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(sb + j * 16384, &map_b, (int)n0 + j * 64, it * 128, full);
                    }
                    SP24_TRACE(0, g);
                }
            }
            if (abort_flag) {
                // drain: wait (bounded) for the copies already issued so that none lands after exit
                for (int q = (g > STAGES ? g - STAGES : 0); q < g; ++q) {
                    const int s = q % STAGES;
                    const uint32_t ph = (q / STAGES) & 1;
                    for (uint32_t w = 0; w < WAIT_LIMIT; ++w)
                        if (mbar_try_wait(full0 + 8 * s, ph)) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart, 32 (A) / 64 (B) bytes per MMA inside
            // the atom.  MN-major: 64-element column blocks one TMA box apart, 8 K-rows per 1024 bytes.
            constexpr uint32_t A_LBO = A_MN ? 8192 : 16, A_KSTEP = A_MN ? 2048 : 32;
            constexpr uint32_t B_LBO = B_MN ? 16384 : 16, B_KSTEP = B_MN ? 4096 : 64;
            int g = 0, tl = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x, ++tl) {
                const int tile = unit % n_tiles, ks = unit / n_tiles;
                const int it0 = (int)((int64_t)ks * k_iters / P.k_splits), it1 = (int)((int64_t)(ks + 1) * k_iters / P.k_splits);
                const int mblk0 = (tile % n_tiles_m) * mpt;
                const int n_mblk = (n_mblocks - mblk0) >= mpt ? mpt : 1;
                for (int it = it0; it < it1 && ok; ++it, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (g / STAGES) & 1;
                    ok = mbar_wait(full0 + 8 * s, ph, &abort_flag, P.status, 2);
                    if (!ok) break;
                    SP24_TRACE(1, 2 * g);
                    const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint32_t sb = sa + OFF_B;
                    const uint32_t se = sa + OFF_E;
                    for (int mb = 0; mb < n_mblk && ok; ++mb) {
                        if (it == it0) {
                            // the epilogue of this CTA's previous tile must have drained this accumulator
                            ok = mbar_wait(tmem_empty0 + 8 * mb, (tl & 1) ^ 1, &abort_flag, P.status, 4);
                            if (!ok) break;
                        }
                        tc_fence_after();
                        const uint32_t e_cols = E_COL0 + ((g & 1) * 2 + mb) * E_SLOT;
                        // metadata: shared memory -> tensor memory, 128 lanes x 16 bytes per atom
                        tc_cp_128x128b(tmem_base + e_cols, make_desc(se + mb * E_BYTES, 16, 128, 0));
                        if constexpr (F8)
                            tc_cp_128x128b(tmem_base + e_cols + 4, make_desc(se + mb * E_BYTES + 2048, 16, 128, 0));
#pragma unroll
                        for (int j = 0; j < KSTEPS; ++j) {
                            const uint64_t adesc = make_desc(sa + mb * A_STAGE_BYTES + j * A_KSTEP, A_LBO, 1024, 2);
                            const uint32_t b_off = B_MN ? j * B_KSTEP : (uint32_t)(j >> 1) * (BN * 128) + (j & 1) * B_KSTEP;
                            const uint64_t bdesc = make_desc(sb + b_off, B_LBO, 1024, 2);
                            const uint32_t ecol = e_cols + (F8 ? 2 * j : j);
                            // 16-bit types: the instruction takes the even column of a pair plus a 1-bit selector
                            const uint32_t e_addr = tmem_base + (F8 ? ecol : (ecol & ~1u));
                            const uint32_t idesc = P.idesc | (F8 ? 0u : (ecol & 1u));
                            mma_sp<F8>(tmem_base + mb * BN, adesc, bdesc, e_addr, idesc, (it > it0 || j > 0) ? 1u : 0u, P.int8);
                        }
                    }
                    tc_commit(empty0 + 8 * s);  // frees the stage when these MMAs have read it
                    SP24_TRACE(1, 2 * g + 1);
                }
                tc_commit(tmem_full);           // accumulators of this tile complete (also arrives after an abort)
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        // Two warps per tensor-memory lane quadrant, each taking half of the tile's columns.  No early exit
        // here: the eight warps meet at named barrier 1, so after an abort they keep walking the tile list
        // (waits return at once) and simply skip the work.
        const int quad = warp & 3;          // TMEM lane quadrant this warp may read
        const int half = (warp - 2) >> 2;   // which half of the columns
        const int tid = (warp - 2) * 32 + lane;
        OutT *out = static_cast<OutT *>(P.out);
        OutT *stg = reinterpret_cast<OutT *>(smem + (size_t)STAGES * STAGE_BYTES);
        int tl = 0;
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++tl) {
            const int tile = unit % n_tiles;
            const int mblk0 = (tile % n_tiles_m) * mpt;
            const int n_mblk = (n_mblocks - mblk0) >= mpt ? mpt : 1;
            const int64_t m0 = (int64_t)mblk0 * BM, n0 = (int64_t)(tile / n_tiles_m) * BN;
            const bool ok = mbar_wait(tmem_full, tl & 1, &abort_flag, P.status, 3);
            tc_fence_after();
            if (threadIdx.x == 64) SP24_TRACE(2, 4 * tl);
            const bool run = ok && !abort_flag;
            const int row_in_blk = quad * 32 + lane;
            if constexpr (Cfg::STAGED16) {
                // 16-bit output through the staging buffer.  Row r of the staging buffer holds one feature's BN values; its
                // 16-byte pieces are permuted by (r / 8) % 4 so that the column-wise reads below (four groups
                // of eight rows per warp instruction) fall on 32 different banks.
                constexpr int HC = BN / 2;                  // columns per warp
                constexpr int NREG = HC / 2;
                uint8_t *stg_row = reinterpret_cast<uint8_t *>(stg) + (size_t)row_in_blk * Cfg::STG_ROW_BYTES;
                const int swz = 2 * ((row_in_blk >> 3) & 3);
                uint32_t held[NREG];                        // second accumulator, converted, two values per word
                float bias0 = 0.f, bias1 = 0.f;
                if (run && P.bias) {
                    bias0 = from_out<OutT>(static_cast<const OutT *>(P.bias)[m0 + row_in_blk]);
                    if (n_mblk == 2) bias1 = from_out<OutT>(static_cast<const OutT *>(P.bias)[m0 + BM + row_in_blk]);
                }
                const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + half * HC;
                if (run) {
#pragma unroll
                    for (int c = 0; c < HC / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(acc + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            Vec<OutT, 8> o;
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                o.v[i] = emit<OutT, ACT>(v[q * 8 + i], bias0, P.activation, P.alpha);
                            const int piece = (half * HC + c * 32) / 8 + q;
                            *reinterpret_cast<uint4 *>(stg_row + ((piece ^ swz) << 4)) = *reinterpret_cast<const uint4 *>(&o);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty0);
                if (n_mblk == 2) {
                    if (run) {
#pragma unroll
                        for (int c = 0; c < HC / 32; ++c) {
                            uint32_t v[32];
                            tmem_ld32(acc + BN + c * 32, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                Vec<OutT, 2> o;
                                o.v[0] = emit<OutT, ACT>(v[2 * i], bias1, P.activation, P.alpha);
                                o.v[1] = emit<OutT, ACT>(v[2 * i + 1], bias1, P.activation, P.alpha);
                                held[c * 16 + i] = *reinterpret_cast<const uint32_t *>(&o);
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                }
                // both accumulators are in shared memory / registers now: the next tile's MMAs may start
                if (lane == 0) mbar_arrive(tmem_empty0 + 8);
                if (threadIdx.x == 64) SP24_TRACE(2, 4 * tl + 1);
                for (int mb = 0; mb < n_mblk; ++mb) {
                    if (mb == 1) {
                        if (run) {
#pragma unroll
                            for (int q = 0; q < NREG / 4; ++q) {
                                const int piece = (half * HC) / 8 + q;
                                *reinterpret_cast<uint4 *>(stg_row + ((piece ^ swz) << 4)) =
                                    make_uint4(held[4 * q], held[4 * q + 1], held[4 * q + 2], held[4 * q + 3]);
                            }
                        }
                    }
                    epilogue_bar_sync();
                    if (run) {
                        const int64_t mrow0 = m0 + mb * BM;
                        const uint8_t *stg_b = reinterpret_cast<const uint8_t *>(stg);
                        if constexpr (TRANS_OUT) {
                            // thread = two adjacent output rows (dense columns n, n+1) x 8 consecutive features;
                            // a warp instruction covers 8 row pairs x 4 feature groups: 64-byte runs per row
                            for (int i = tid; i < (BN / 2) * (BM / 8); i += 256) {
                                const int mg = (i & 3) + 4 * ((i >> 5) & 3), np = ((i >> 2) & 7) + 8 * (i >> 7);
                                const int word = np ^ ((i & 3) << 3);   // rows mg*8..mg*8+7 share (r / 8) % 4 = mg % 4
                                uint32_t w[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    w[j] = *reinterpret_cast<const uint32_t *>(stg_b + (size_t)(mg * 8 + j) * Cfg::STG_ROW_BYTES + word * 4);
                                uint4 lo, hi;
                                lo.x = __byte_perm(w[0], w[1], 0x5410); hi.x = __byte_perm(w[0], w[1], 0x7632);
                                lo.y = __byte_perm(w[2], w[3], 0x5410); hi.y = __byte_perm(w[2], w[3], 0x7632);
                                lo.z = __byte_perm(w[4], w[5], 0x5410); hi.z = __byte_perm(w[4], w[5], 0x7632);
                                lo.w = __byte_perm(w[6], w[7], 0x5410); hi.w = __byte_perm(w[6], w[7], 0x7632);
                                const int64_t nrow = n0 + 2 * np;
                                OutT *dst = out + nrow * P.ld_out + mrow0 + mg * 8;
                                if (nrow < P.n) *reinterpret_cast<uint4 *>(dst) = lo;
                                if (nrow + 1 < P.n) *reinterpret_cast<uint4 *>(dst + P.ld_out) = hi;
                            }
                        } else {
                            // thread = 8 consecutive columns of one row; a warp writes 512 contiguous bytes
                            constexpr int PIECES = BN / 8;
                            for (int i = tid; i < PIECES * BM; i += 256) {
                                const int row = i / PIECES, piece = i % PIECES;
                                const uint4 v = *reinterpret_cast<const uint4 *>(
                                    stg_b + (size_t)row * Cfg::STG_ROW_BYTES + ((piece ^ (2 * ((row >> 3) & 3))) << 4));
                                const int64_t nb = n0 + piece * 8;
                                OutT *dst = out + (mrow0 + row) * P.ld_out + nb;
                                if (nb + 8 <= P.n) {
                                    *reinterpret_cast<uint4 *>(dst) = v;
                                } else {
                                    const OutT *e = reinterpret_cast<const OutT *>(&v);
                                    for (int j = 0; j < 8; ++j)
                                        if (nb + j < P.n) dst[j] = e[j];
                                }
                            }
                        }
                    }
                    epilogue_bar_sync();
                }
            } else {
                for (int mb = 0; mb < n_mblk; ++mb) {
                    const int64_t mrow0 = m0 + mb * BM;
                    const int64_t m = mrow0 + row_in_blk;
                    float bias = 0.f;
                    if (run && P.bias) bias = from_out<OutT>(static_cast<const OutT *>(P.bias)[m]);
                    const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + mb * BN;
                    if constexpr (TRANS_OUT) {
                        // 4-byte transposed output, STG_COLS columns at a time; each warp copies its half of a chunk
                        constexpr int CHUNKS = BN / Cfg::STG_COLS;
                        constexpr int HC = Cfg::STG_COLS / 2;
                        static_assert(HC % 32 == 0, "a warp reads whole 32-column pieces");
                        uint8_t *stg_row = reinterpret_cast<uint8_t *>(stg) + (size_t)row_in_blk * Cfg::STG_ROW_BYTES;
#pragma unroll 1
                        for (int ch = 0; ch < CHUNKS; ++ch) {
                            if (run) {
#pragma unroll 1
                                for (int c = 0; c < HC / 32; ++c) {
                                    uint32_t v[32];
                                    const int col = half * HC + c * 32;
                                    tmem_ld32(acc + ch * Cfg::STG_COLS + col, v);
                                    tmem_ld_wait();
#pragma unroll
                                    for (int q = 0; q < 8; ++q) {
                                        float4 o;
                                        o.x = __uint_as_float(emit_bits<OutT, ACT>(v[q * 4 + 0], bias, P.activation, P.alpha));
                                        o.y = __uint_as_float(emit_bits<OutT, ACT>(v[q * 4 + 1], bias, P.activation, P.alpha));
                                        o.z = __uint_as_float(emit_bits<OutT, ACT>(v[q * 4 + 2], bias, P.activation, P.alpha));
                                        o.w = __uint_as_float(emit_bits<OutT, ACT>(v[q * 4 + 3], bias, P.activation, P.alpha));
                                        *reinterpret_cast<float4 *>(stg_row + (col + q * 4) * 4) = o;
                                    }
                                }
                            }
                            if (ch == CHUNKS - 1) {
                                // this accumulator has been read completely: hand it back to the MMA warp
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(tmem_empty0 + 8 * mb);
                                if (threadIdx.x == 64) SP24_TRACE(2, 4 * tl + 1 + mb);
                            }
                            epilogue_bar_sync();
                            if (run) {
                                // thread = one output row x 4 consecutive features; lane pairs cover 8 features of
                                // the same row, so every warp instruction writes whole 32-byte sectors
                                const int64_t nbase = n0 + ch * Cfg::STG_COLS;
                                const uint8_t *stg_b = reinterpret_cast<const uint8_t *>(stg);
                                for (int i = tid; i < Cfg::STG_COLS * (BM / 4); i += 256) {
                                    const int pr = i >> 1;
                                    const int nn = pr % Cfg::STG_COLS, mg = 2 * (pr / Cfg::STG_COLS) + (i & 1);
                                    uint4 o;
                                    o.x = *reinterpret_cast<const uint32_t *>(stg_b + (size_t)(mg * 4 + 0) * Cfg::STG_ROW_BYTES + nn * 4);
                                    o.y = *reinterpret_cast<const uint32_t *>(stg_b + (size_t)(mg * 4 + 1) * Cfg::STG_ROW_BYTES + nn * 4);
                                    o.z = *reinterpret_cast<const uint32_t *>(stg_b + (size_t)(mg * 4 + 2) * Cfg::STG_ROW_BYTES + nn * 4);
                                    o.w = *reinterpret_cast<const uint32_t *>(stg_b + (size_t)(mg * 4 + 3) * Cfg::STG_ROW_BYTES + nn * 4);
                                    if (nbase + nn < P.n)
                                        *reinterpret_cast<uint4 *>(out + (nbase + nn) * P.ld_out + mrow0 + mg * 4) = o;
                                }
                            }
                            epilogue_bar_sync();
                        }
                    } else {
                        constexpr int HC = BN / 2;
                        if (run) {
#pragma unroll 1
                            for (int c = 0; c < HC / 32; ++c) {
                                uint32_t v[32];
                                const int col = half * HC + c * 32;
                                tmem_ld32(acc + col, v);
                                tmem_ld_wait();
                                const int64_t nb = n0 + col;
                                OutT *row = out + m * P.ld_out + nb;
                                if constexpr (ACCUM) {
                                    // D += partial product: fp32 reductions in L2, 16 bytes each, no return value
                                    if (nb + 32 <= P.n) {
#pragma unroll
                                        for (int q = 0; q < 8; ++q)
                                            red_add_v4(reinterpret_cast<float *>(row) + q * 4, __uint_as_float(v[q * 4]), __uint_as_float(v[q * 4 + 1]),
                                                       __uint_as_float(v[q * 4 + 2]), __uint_as_float(v[q * 4 + 3]));
                                    } else {
                                        for (int i = 0; i < 32; ++i)
                                            if (nb + i < P.n) atomicAdd(reinterpret_cast<float *>(row) + i, __uint_as_float(v[i]));
                                    }
                                } else if (nb + 32 <= P.n) {
                                    constexpr int PER = 16 / sizeof(OutT);
#pragma unroll
                                    for (int q = 0; q < 32 / PER; ++q) {
                                        Vec<OutT, PER> o;
#pragma unroll
                                        for (int i = 0; i < PER; ++i)
                                            o.v[i] = emit<OutT, ACT>(v[q * PER + i], bias, P.activation, P.alpha);
                                        store_vec<OutT, PER>(row + q * PER, o);
                                    }
                                } else {
                                    for (int i = 0; i < 32; ++i)
                                        if (nb + i < P.n)
                                            row[i] = emit<OutT, ACT>(v[i], bias, P.activation, P.alpha);
                                }
                            }
                        }
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tmem_empty0 + 8 * mb);
                    }
                }
                if (n_mblk == 1) {
                    // keep the second accumulator's barrier in step with the tile count
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tmem_empty0 + 8);
                }
            }
            if (threadIdx.x == 64) SP24_TRACE(2, 4 * tl + 3);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// Two-CTA form (cluster of 2, tcgen05 cta_group::2) for 16-bit types, B stored (n, k), output (n, ms).
// ------------------------------------------------------------------------------------------------
// A CTA pair computes tiles of 256 sparse rows x 192 dense columns: every MMA instruction has M = 256 (128
// rows per CTA) and N = 192, and reads half of its B operand from each CTA's shared memory, so a CTA stages
// only 96 rows of B per stage: 42 KB per stage and 128-row block, where the single-CTA kernel needs 66 KB
// (or 84 KB for two blocks).  One accumulator per tile leaves room for two accumulator buffers in tensor
// memory, so the epilogue of a tile runs entirely under the next tile's MMAs, and five operand stages fit.
// Each CTA loads its own A block, metadata and B half with TMA (cta_group::2 form, completing on the leader's
// barrier), drains its own accumulator and reports its release to the leader's barrier.  CTA 0 of the pair
// (the leader) issues all MMAs and metadata copies; its commits arrive on the barriers of both CTAs.  No load
// is multicast.
namespace two {
constexpr int BN2 = 192;                                   // columns of a pair tile
constexpr int B_HALF_BYTES = (BN2 / 2) * 256;              // 96 rows x two 128-byte K atoms
constexpr int STAGE2_BYTES = A_STAGE_BYTES + B_HALF_BYTES + 2048;   // 43008
constexpr int STAGES2 = 5;
constexpr int SMEM2 = STAGES2 * STAGE2_BYTES + 1024;
static_assert(STAGE2_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
static_assert(SMEM2 <= 227 * 1024, "shared memory budget");
}  // namespace two

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cta address -> shared::cluster address of the same location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void tc_cp_128x128b_pair(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void mma_sp_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t e_tmem, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.sp.cta_group::2.kind::f16 [%0], %1, %2, [%3], %4, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
        : "memory");
}

template <bool A_MN, typename OutT, int EPI>
__global__ void __launch_bounds__(320, 1)
spmm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_e, SpmmParams P) {
    using namespace two;
    constexpr int BN = BN2;
    constexpr int STAGES = STAGES2;
    constexpr int OFF_B = A_STAGE_BYTES, OFF_E = OFF_B + B_HALF_BYTES;
    constexpr int KSTEPS = 4;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int E_COL0 = 2 * BN, E_SLOT = 4;    // two accumulator buffers, then two metadata slots
    static_assert(sizeof(OutT) == 2, "16-bit outputs only");
    static_assert(E_COL0 + 2 * E_SLOT <= 512, "tensor memory columns exhausted");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_tiles_n = (int)((P.n + BN - 1) / BN);
    const int n_tiles_m = (int)(P.ms / (2 * BM));     // 256-row blocks: one 128-row block per CTA
    const int n_tiles = n_tiles_n * n_tiles_m;        // row block varies fastest over the tile index
    const int k_iters = (int)((P.k + 127) / 128);

    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t tmem_full0 = smem_u32(&bars[2 * STAGES]), tmem_empty0 = smem_u32(&bars[2 * STAGES + 2]);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);      // used in the leader only: one expect_tx arrival, bytes of both CTAs
            mbar_init(empty0 + 8 * s, 1);     // one commit arrival per CTA
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full0 + 8 * b, 1);
            mbar_init(tmem_empty0 + 8 * b, 16);   // used in the leader only: eight epilogue warps of each CTA
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tmem_base_smem), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                       // the peer's barriers are initialised before anything targets them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (one per CTA)
        if (lane == 0) {
            int g = 0;
            bool ok = true;
            constexpr uint32_t cta_tx = A_STAGE_BYTES + 2048 + B_HALF_BYTES;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                const int mblk = (tile % n_tiles_m) * 2 + (int)rank;
                const int mrow = mblk * BM;
                const int brow = (tile / n_tiles_m) * BN + (int)rank * (BN / 2);
                for (int it = 0; it < k_iters; ++it, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (g / STAGES) & 1;
                    if (g >= STAGES && !mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, P.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_u32(smem + (size_t)s * STAGE2_BYTES);
                    const uint32_t sb = sa + OFF_B;
                    const uint32_t full_leader = map_to_cta(full0 + 8 * s, 0);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * cta_tx);
                    if constexpr (!A_MN) {
                        tma_load_2d_pair(sa, &map_a, it * 64, mrow, full_leader);
                    } else {
                        tma_load_2d_pair(sa, &map_a, mrow, it * 64, full_leader);
                        tma_load_2d_pair(sa + 8192, &map_a, mrow + 64, it * 64, full_leader);
                    }
                    // metadata atom of this row block and K step: two rows of 1024 bytes in the atom table
                    tma_load_2d_pair(sa + OFF_E, &map_e, 0, (int)(((int64_t)mblk * P.k_atoms + it) * 2), full_leader);
                    // this CTA's half of B: 96 rows x two 128-byte K atoms
                    tma_load_2d_pair(sb, &map_b, it * 128, brow, full_leader);
                    tma_load_2d_pair(sb + (BN / 2) * 128, &map_b, it * 128 + 64, brow, full_leader);
                    SP24_TRACE(0, g);
                }
            }
            if (abort_flag && rank == 0) {
                for (int q = (g > STAGES ? g - STAGES : 0); q < g; ++q) {
                    const int s = q % STAGES;
                    const uint32_t ph = (q / STAGES) & 1;
                    for (uint32_t w = 0; w < WAIT_LIMIT; ++w)
                        if (mbar_try_wait(full0 + 8 * s, ph)) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t A_LBO = A_MN ? 8192 : 16, A_KSTEP = A_MN ? 2048 : 32;
            const uint32_t idesc0 = P.idesc;   // M = 256, N = 192 set by the launcher
            int g = 0, tl = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++tl) {
                const int buf = tl & 1;
                // the epilogues of both CTAs must have drained this accumulator buffer (two tiles ago)
                ok = mbar_wait(tmem_empty0 + 8 * buf, ((tl >> 1) & 1) ^ 1, &abort_flag, P.status, 4);
                for (int it = 0; it < k_iters && ok; ++it, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (g / STAGES) & 1;
                    ok = mbar_wait(full0 + 8 * s, ph, &abort_flag, P.status, 2);
                    if (!ok) break;
                    SP24_TRACE(1, 2 * g);
                    const uint32_t sa = smem_u32(smem + (size_t)s * STAGE2_BYTES);
                    const uint32_t sb = sa + OFF_B;
                    tc_fence_after();
                    const uint32_t e_cols = E_COL0 + (g & 1) * E_SLOT;
                    tc_cp_128x128b_pair(tmem_base + e_cols, make_desc(sa + OFF_E, 16, 128, 0));
#pragma unroll
                    for (int j = 0; j < KSTEPS; ++j) {
                        const uint64_t adesc = make_desc(sa + j * A_KSTEP, A_LBO, 1024, 2);
                        const uint32_t b_off = (uint32_t)(j >> 1) * ((BN / 2) * 128) + (j & 1) * 64;
                        const uint64_t bdesc = make_desc(sb + b_off, 16, 1024, 2);
                        const uint32_t ecol = e_cols + j;
                        mma_sp_pair(tmem_base + buf * BN, adesc, bdesc, tmem_base + (ecol & ~1u), idesc0 | (ecol & 1u),
                                    (it > 0 || j > 0) ? 1u : 0u);
                    }
                    tc_commit_pair(empty0 + 8 * s);
                    SP24_TRACE(1, 2 * g + 1);
                }
                tc_commit_pair(tmem_full0 + 8 * buf);   // also arrives after an abort
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9 of both CTAs)
        // No staging buffer: a warp packs its 96 columns of the accumulator into 48 registers, hands the buffer
        // back, then stores 16-bit values directly; the 32 lanes of a store are 32 consecutive features of one
        // token, 64 contiguous bytes.
        const int quad = warp & 3, half = (warp - 2) >> 2;
        constexpr int HC = BN / 2, NREG = HC / 2;
        OutT *out = static_cast<OutT *>(P.out);
        const uint32_t empty_leader0 = map_to_cta(tmem_empty0, 0);
        int tl = 0;
        for (int tile = pair; tile < n_tiles; tile += n_pairs, ++tl) {
            const int buf = tl & 1;
            const int mrow = ((tile % n_tiles_m) * 2 + (int)rank) * BM + quad * 32 + lane;
            const int64_t tok0 = (int64_t)(tile / n_tiles_m) * BN + half * HC;
            const bool ok = mbar_wait(tmem_full0 + 8 * buf, (tl >> 1) & 1, &abort_flag, P.status, 3);
            tc_fence_after();
            if (threadIdx.x == 64) SP24_TRACE(2, 4 * tl);
            const bool run = ok && !abort_flag;
            uint32_t held[NREG];
            if (run) {
                float bias = 0.f;
                if (P.bias) bias = P.bias_f32 ? static_cast<const float *>(P.bias)[mrow] : from_out<OutT>(static_cast<const OutT *>(P.bias)[mrow]);
                const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + half * HC;
#pragma unroll
                for (int c = 0; c < HC / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(acc + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        Vec<OutT, 2> o;
                        if constexpr (EPI == EPI_DGELU) {   // no bias; the factor gelu'(aux) is applied at store time
                            o.v[0] = to_out<OutT>(__uint_as_float(v[2 * i]));
                            o.v[1] = to_out<OutT>(__uint_as_float(v[2 * i + 1]));
                        } else {
                            o.v[0] = to_out<OutT>(__uint_as_float(v[2 * i]) + bias);
                            o.v[1] = to_out<OutT>(__uint_as_float(v[2 * i + 1]) + bias);
                        }
                        held[c * 16 + i] = *reinterpret_cast<const uint32_t *>(&o);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(empty_leader0 + 8 * buf);
            if (threadIdx.x == 64) SP24_TRACE(2, 4 * tl + 1);
            if (run) {
                uint16_t *dst = reinterpret_cast<uint16_t *>(out) + tok0 * P.ld_out + mrow;
                uint16_t *aux = reinterpret_cast<uint16_t *>(P.aux) + tok0 * P.ld_aux + mrow;
                if constexpr (EPI == EPI_PLAIN) {
                    if (tok0 + HC <= P.n) {
#pragma unroll
                        for (int c2 = 0; c2 < NREG; ++c2) {
                            dst[0] = (uint16_t)(held[c2] & 0xFFFFu);
                            dst[P.ld_out] = (uint16_t)(held[c2] >> 16);
                            dst += 2 * P.ld_out;
                            asm volatile("" : "+l"(dst));   // one running pointer, not 96 precomputed addresses
                        }
                    } else {
#pragma unroll
                        for (int c2 = 0; c2 < NREG; ++c2) {
                            if (tok0 + 2 * c2 < P.n) dst[0] = (uint16_t)(held[c2] & 0xFFFFu);
                            if (tok0 + 2 * c2 + 1 < P.n) dst[P.ld_out] = (uint16_t)(held[c2] >> 16);
                            dst += 2 * P.ld_out;
                            asm volatile("" : "+l"(dst));
                        }
                    }
                } else {
                    const bool full = tok0 + HC <= P.n;
                    auto as_f = [](uint16_t bits) { return from_out<OutT>(*reinterpret_cast<const OutT *>(&bits)); };
                    auto as_b = [](float v) { const OutT o = to_out<OutT>(v); return *reinterpret_cast<const uint16_t *>(&o); };
                    // chunks of 16 tokens: all loads of a chunk are issued before the first use, all its stores after
                    constexpr int CHUNK = 8;
#pragma unroll
                    for (int c0 = 0; c0 < NREG; c0 += CHUNK) {
                        uint16_t a[2 * CHUNK];
                        if constexpr (EPI == EPI_DGELU) {
#pragma unroll
                            for (int j = 0; j < 2 * CHUNK; ++j)
                                a[j] = (full || tok0 + 2 * c0 + j < P.n) ? aux[(int64_t)j * P.ld_aux] : (uint16_t)0;
                        }
#pragma unroll
                        for (int j = 0; j < 2 * CHUNK; ++j) {
                            const uint32_t hw = held[c0 + (j >> 1)];
                            const uint16_t h_bits = (j & 1) ? (uint16_t)(hw >> 16) : (uint16_t)(hw & 0xFFFFu);
                            if (full || tok0 + 2 * c0 + j < P.n) {
                                if constexpr (EPI == EPI_PRE_GELU) {
                                    aux[(int64_t)j * P.ld_aux] = h_bits;
                                    dst[(int64_t)j * P.ld_out] = as_b(gelu_tanh(as_f(h_bits)));
                                } else {
                                    dst[(int64_t)j * P.ld_out] = as_b(as_f(h_bits) * gelu_tanh_grad(as_f(a[j])));
                                }
                            }
                        }
                        dst += 2 * CHUNK * P.ld_out;
                        aux += 2 * CHUNK * P.ld_aux;
                        asm volatile("" : "+l"(dst), "+l"(aux));   // running pointers per chunk
                    }
                }
            }
            if (threadIdx.x == 64) SP24_TRACE(2, 4 * tl + 3);
        }
        tc_fence_before();
    }
    // nobody leaves while the peer may still read this CTA's shared memory or signal its barriers
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// Two-CTA form of the weight-gradient GEMM: D (ms x n, fp32) += A_sparse (ms x k) * B (k x n, stored row-major).
// ------------------------------------------------------------------------------------------------
// Tiles of 256 sparse rows x 256 dense columns per CTA pair (M = 256, N = 256 per instruction); a CTA stages its 128
// rows of A (16 KB), its 128 columns of B as two 64-column boxes of 128 K-rows (32 KB) and 2 KB of metadata per K
// step of 128: 50 KB for 8.4 dense-equivalent MFLOP, four stages.  K is cut into slices (work unit = tile x slice)
// so that the units fill the pairs; every unit adds its partial product with fp32 vector reductions.  One
// accumulator of 256 columns per CTA: a pair that owns more than one unit drains it before the next unit's MMAs.
namespace two {
constexpr int BN3 = 256;
constexpr int B3_BYTES = (BN3 / 2) * 256;                  // 128 columns x 128 K-rows x 2 bytes
constexpr int STAGE3_BYTES = A_STAGE_BYTES + B3_BYTES + 2048;   // 51200
constexpr int STAGES3 = 4;
constexpr int SMEM3 = STAGES3 * STAGE3_BYTES + 1024;
static_assert(STAGE3_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
static_assert(SMEM3 <= 227 * 1024, "shared memory budget");
}  // namespace two

template <bool A_MN>
__global__ void __launch_bounds__(320, 1)
spmm_pair_acc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_e, SpmmParams P) {
    using namespace two;
    constexpr int BN = BN3;
    constexpr int STAGES = STAGES3;
    constexpr int OFF_B = A_STAGE_BYTES, OFF_E = OFF_B + B3_BYTES;
    constexpr int KSTEPS = 4;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int E_COL0 = BN, E_SLOT = 4;       // one accumulator, then two metadata slots

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_tiles_n = (int)((P.n + BN - 1) / BN);
    const int n_tiles_m = (int)(P.ms / (2 * BM));
    const int n_tiles = n_tiles_n * n_tiles_m;
    const int n_units = n_tiles * P.k_splits;     // unit u = (tile u % n_tiles, K slice u / n_tiles)
    const int k_iters = (int)((P.k + 127) / 128);

    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t tmem_full = smem_u32(&bars[2 * STAGES]), tmem_empty = smem_u32(&bars[2 * STAGES + 1]);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, 16);            // used in the leader only: eight epilogue warps of each CTA
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tmem_base_smem), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (one per CTA)
        if (lane == 0) {
            int g = 0;
            bool ok = true;
            constexpr uint32_t cta_tx = A_STAGE_BYTES + 2048 + B3_BYTES;
            for (int unit = pair; unit < n_units && ok; unit += n_pairs) {
                const int tile = unit % n_tiles, ks = unit / n_tiles;
                const int it0 = (int)((int64_t)ks * k_iters / P.k_splits), it1 = (int)((int64_t)(ks + 1) * k_iters / P.k_splits);
                const int mblk = (tile % n_tiles_m) * 2 + (int)rank;
                const int mrow = mblk * BM;
                const int bcol = (tile / n_tiles_m) * BN + (int)rank * (BN / 2);
                for (int it = it0; it < it1; ++it, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (g / STAGES) & 1;
                    if (g >= STAGES && !mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, P.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_u32(smem + (size_t)s * STAGE3_BYTES);
                    const uint32_t sb = sa + OFF_B;
                    const uint32_t full_leader = map_to_cta(full0 + 8 * s, 0);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * cta_tx);
                    if constexpr (!A_MN) {
                        tma_load_2d_pair(sa, &map_a, it * 64, mrow, full_leader);
                    } else {
                        tma_load_2d_pair(sa, &map_a, mrow, it * 64, full_leader);
                        tma_load_2d_pair(sa + 8192, &map_a, mrow + 64, it * 64, full_leader);
                    }
                    tma_load_2d_pair(sa + OFF_E, &map_e, 0, (int)(((int64_t)mblk * P.k_atoms + it) * 2), full_leader);
                    // this CTA's 128 columns of B: two boxes of 64 columns x 128 K-rows
                    tma_load_2d_pair(sb, &map_b, bcol, it * 128, full_leader);
                    tma_load_2d_pair(sb + 16384, &map_b, bcol + 64, it * 128, full_leader);
                }
            }
            if (abort_flag && rank == 0) {
                for (int q = (g > STAGES ? g - STAGES : 0); q < g; ++q) {
                    const int s = q % STAGES;
                    const uint32_t ph = (q / STAGES) & 1;
                    for (uint32_t w = 0; w < WAIT_LIMIT; ++w)
                        if (mbar_try_wait(full0 + 8 * s, ph)) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t A_LBO = A_MN ? 8192 : 16, A_KSTEP = A_MN ? 2048 : 32;
            const uint32_t idesc0 = P.idesc;   // M = 256, N = 256, B MN-major set by the launcher
            int g = 0, tl = 0;
            bool ok = true;
            for (int unit = pair; unit < n_units && ok; unit += n_pairs, ++tl) {
                const int ks = unit / n_tiles;
                const int it0 = (int)((int64_t)ks * k_iters / P.k_splits), it1 = (int)((int64_t)(ks + 1) * k_iters / P.k_splits);
                // the epilogues of both CTAs must have drained the accumulator of the previous unit
                ok = mbar_wait(tmem_empty, (tl & 1) ^ 1, &abort_flag, P.status, 4);
                for (int it = it0; it < it1 && ok; ++it, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (g / STAGES) & 1;
                    ok = mbar_wait(full0 + 8 * s, ph, &abort_flag, P.status, 2);
                    if (!ok) break;
                    const uint32_t sa = smem_u32(smem + (size_t)s * STAGE3_BYTES);
                    const uint32_t sb = sa + OFF_B;
                    tc_fence_after();
                    const uint32_t e_cols = E_COL0 + (g & 1) * E_SLOT;
                    tc_cp_128x128b_pair(tmem_base + e_cols, make_desc(sa + OFF_E, 16, 128, 0));
#pragma unroll
                    for (int j = 0; j < KSTEPS; ++j) {
                        const uint64_t adesc = make_desc(sa + j * A_KSTEP, A_LBO, 1024, 2);
                        // MN-major B: 64-column blocks 16384 bytes apart, 32 K-rows (4096 bytes) per MMA
                        const uint64_t bdesc = make_desc(sb + j * 4096, 16384, 1024, 2);
                        const uint32_t ecol = e_cols + j;
                        mma_sp_pair(tmem_base, adesc, bdesc, tmem_base + (ecol & ~1u), idesc0 | (ecol & 1u),
                                    (it > it0 || j > 0) ? 1u : 0u);
                    }
                    tc_commit_pair(empty0 + 8 * s);
                }
                tc_commit_pair(tmem_full);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9 of both CTAs)
        const int quad = warp & 3, half = (warp - 2) >> 2;
        constexpr int HC = BN / 2;                     // 128 columns per warp
        float *out = static_cast<float *>(P.out);
        const uint32_t empty_leader = map_to_cta(tmem_empty, 0);
        int tl = 0;
        for (int unit = pair; unit < n_units; unit += n_pairs, ++tl) {
            const int tile = unit % n_tiles;
            const int mrow = ((tile % n_tiles_m) * 2 + (int)rank) * BM + quad * 32 + lane;
            const int64_t col0 = (int64_t)(tile / n_tiles_m) * BN + half * HC;
            const bool ok = mbar_wait(tmem_full, tl & 1, &abort_flag, P.status, 3);
            tc_fence_after();
            const bool run = ok && !abort_flag;
            if (run) {
                const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + half * HC;
                float *row = out + (int64_t)mrow * P.ld_out + col0;
#pragma unroll 1
                for (int c = 0; c < HC / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(acc + c * 32, v);
                    tmem_ld_wait();
                    const int64_t nb = col0 + c * 32;
                    if (nb + 32 <= P.n) {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            red_add_v4(row + c * 32 + q * 4, __uint_as_float(v[q * 4]), __uint_as_float(v[q * 4 + 1]),
                                       __uint_as_float(v[q * 4 + 2]), __uint_as_float(v[q * 4 + 3]));
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (nb + i < P.n) atomicAdd(row + c * 32 + i, __uint_as_float(v[i]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(empty_leader);
        }
        tc_fence_before();
    }
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// metadata: reference (reordered) layout -> tensor-core atom order
// ------------------------------------------------------------------------------------------------
// 16-bit types: atom = 128 rows x 128 logical columns = 2048 bytes, byte 16*L + 4*q + 2*h with
// L = 16*(r/16) + 8*(c%2) + r%8, q = (c/2)%4, h = (r/8)%2 for row r (inside the 128-row block) and
// 16-column metadata word c.  8-bit types: atom = 128 rows x 16 bytes, row-major.
template <int MB>
__global__ void meta_to_tc_kernel(const void *meta_api, uint8_t *e_tc, int64_t m, int64_t ncols, int64_t k_atoms) {
    const int64_t words_per_atom = 2048 / MB;
    const int64_t total = (m / 128) * k_atoms * words_per_atom;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t atom = idx / words_per_atom;
    const int w = (int)(idx % words_per_atom);
    const int64_t mb = atom / k_atoms, kb = atom % k_atoms;
    int r, cw;  // row inside the block, metadata word inside the atom's 128 columns
    if constexpr (MB == 2) {
        const int L = w >> 3, q = (w >> 1) & 3, h = w & 1;
        r = 16 * (L >> 4) + 8 * h + (L & 7);
        cw = 2 * q + ((L >> 3) & 1);
    } else {
        r = w >> 2;
        cw = w & 3;
    }
    const int64_t c = kb * (MB == 2 ? 8 : 4) + cw;
    using MetaT = typename VecBytes<MB>::type;
    MetaT val = 0;
    if (c < ncols) val = static_cast<const MetaT *>(meta_api)[meta_offset<MB>(mb * 128 + r, c, m)];
    reinterpret_cast<MetaT *>(e_tc)[idx] = val;
}

CUtensorMapDataType tmap_dtype(int dt) {
    switch (dt) {
        case SP24_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        case SP24_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    }
}

// cuTensorMapEncodeTiled is looked up through the runtime so that the library has no link-time
// dependency on the driver library (it must load on machines without a GPU driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D tensor map over a row-major (rows, cols) array with leading dimension ld (elements), 128-byte swizzle.
int make_map(CUtensorMap *map, const void *base, int dt, int64_t rows, int64_t cols, int64_t ld, uint32_t box_cols,
             uint32_t box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * dtype_size(dt)};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return SP24_ERR_CUDA;
    CUresult r = encode(map, tmap_dtype(dt), 2, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_ERROR_INVALID_CONTEXT) {
        // a host thread that has made no runtime call yet (an autograd worker) has no current context for this
        // driver entry point: let the runtime bind the primary context, then encode again
        cudaFree(nullptr);
        r = encode(map, tmap_dtype(dt), 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS && getenv("SP24_DEBUG"))
        fprintf(stderr, "sparse24_b200: cuTensorMapEncodeTiled failed (%d): base %p rows %lld cols %lld ld %lld box %u x %u\n",
                (int)r, base, (long long)rows, (long long)cols, (long long)ld, box_cols, box_rows);
    return r == CUDA_SUCCESS ? SP24_OK : SP24_ERR_CUDA;
}

// SP24_SPMM_PAIR=0 in the environment keeps every GEMM on the single-CTA kernels (read once per process)
bool pair_kernels_enabled() {
    static const bool enabled = [] {
        const char *env = getenv("SP24_SPMM_PAIR");
        return !(env && atoi(env) == 0);
    }();
    return enabled;
}

int sm_count_cached() { return sm_count(); }

template <int BN, bool F8, bool A_MN, bool B_MN, bool TRANS, typename OutT>
int launch_spmm(const CUtensorMap &ma, const CUtensorMap &mb, SpmmParams P, cudaStream_t st) {
    using Cfg = SpmmCfg<BN, F8, TRANS, OutT>;
    auto kern = P.activation ? spmm_kernel<BN, F8, A_MN, B_MN, TRANS, OutT, true>
                             : spmm_kernel<BN, F8, A_MN, B_MN, TRANS, OutT, false>;
    static bool attr_set[64][2];
    int dev = 0;
    cudaGetDevice(&dev);
    const int which = P.activation ? 1 : 0;
    if (dev >= 0 && dev < 64 && !attr_set[dev][which]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
            return launch_status();
        attr_set[dev][which] = true;
    }
    P.idesc |= (uint32_t)(BN >> 3) << 17;
    const int64_t tiles = ((P.n + BN - 1) / BN) * ((P.ms / BM + P.mblk_per_tile - 1) / P.mblk_per_tile) * P.k_splits;
    const int sms = sm_count_cached();
    kern<<<(unsigned)(tiles < sms ? tiles : sms), 320, Cfg::SMEM, st>>>(ma, mb, P);
    return launch_status();
}

// Metadata atoms as a 2-D tensor for TMA: rows of 1024 bytes (256 int32), two rows per 2048-byte atom, no swizzle.
int make_map_e(CUtensorMap *map, const void *e_tc, int64_t n_atoms) {
    const cuuint64_t dims[2] = {256, (cuuint64_t)(2 * n_atoms)};
    const cuuint64_t strides[1] = {1024};
    const cuuint32_t box[2] = {256, 2};
    const cuuint32_t estr[2] = {1, 1};
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return SP24_ERR_CUDA;
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void *>(e_tc), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_ERROR_INVALID_CONTEXT) {
        cudaFree(nullptr);   // see make_map
        r = encode(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void *>(e_tc), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    return r == CUDA_SUCCESS ? SP24_OK : SP24_ERR_CUDA;
}

template <bool A_MN, typename OutT, int EPI = EPI_PLAIN>
int launch_spmm_pair(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &me, SpmmParams P, cudaStream_t st) {
    auto kern = spmm_pair_kernel<A_MN, OutT, EPI>;
    static bool attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, two::SMEM2) != cudaSuccess)
            return SP24_ERR_CUDA;
        attr_set[dev] = true;
    }
    // M = 256 over the CTA pair, N = 192
    P.idesc = (P.idesc & ~(0x1Fu << 24)) | ((uint32_t)(256 >> 4) << 24) | ((uint32_t)(two::BN2 >> 3) << 17);
    const int64_t tiles = ((P.n + two::BN2 - 1) / two::BN2) * (P.ms / 256);
    const int64_t pairs_max = sm_count_cached() / 2;
    const unsigned pairs = (unsigned)(tiles < pairs_max ? tiles : pairs_max);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(320, 1, 1);
    cfg.dynamicSmemBytes = two::SMEM2;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, ma, mb, me, P) != cudaSuccess) return SP24_ERR_CUDA;
    return launch_status();
}

template <bool A_MN>
int launch_spmm_pair_acc(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &me, SpmmParams P, int k_splits,
                         cudaStream_t st) {
    auto kern = spmm_pair_acc_kernel<A_MN>;
    static bool attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, two::SMEM3) != cudaSuccess)
            return launch_status();
        attr_set[dev] = true;
    }
    // M = 256 over the CTA pair, N = 256
    P.idesc = (P.idesc & ~(0x1Fu << 24)) | ((uint32_t)(256 >> 4) << 24) | ((uint32_t)(two::BN3 >> 3) << 17);
    const int64_t tiles = ((P.n + two::BN3 - 1) / two::BN3) * (P.ms / 256);
    const int64_t pairs_max = sm_count_cached() / 2;
    const int64_t k_iters = (P.k + 127) / 128;
    int64_t splits = k_splits ? k_splits : pairs_max / tiles;
    if (splits < 1) splits = 1;
    if (splits > k_iters) splits = k_iters;
    P.k_splits = (int)splits;
    const int64_t units = tiles * splits;
    const unsigned pairs = (unsigned)(units < pairs_max ? units : pairs_max);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(320, 1, 1);
    cfg.dynamicSmemBytes = two::SMEM3;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, ma, mb, me, P) != cudaSuccess) return launch_status();
    return launch_status();
}

// Tile shape: wide / tall tiles stage fewer operand bytes per output, small ones fill the SMs more evenly.
// Cost model per candidate (BN, row blocks per tile): rounds of tiles per CTA x bytes staged per K iteration.
void pick_tile(int64_t ms, int64_t n, int sm_count, int &bn_out, int &mpt_out) {
    const int cand_bn[2] = {192, 128};
    double best_cost = 1e300;
    for (int mpt = 2; mpt >= 1; --mpt) {
        for (int i = 0; i < 2; ++i) {
            const int bn = cand_bn[i];
            const int64_t tiles = ((n + bn - 1) / bn) * ((ms / BM + mpt - 1) / mpt);
            const double rounds = (double)((tiles + sm_count - 1) / sm_count);
            const double cost = rounds * (mpt * (A_STAGE_BYTES + 2048) + bn * 256);
            if (cost < best_cost) { best_cost = cost; bn_out = bn; mpt_out = mpt; }
        }
    }
}

template <bool F8, bool A_MN, bool B_MN, bool TRANS, typename OutT>
int dispatch_bn(int bn, const void *b, int dtype, int64_t n, int64_t k, int64_t ld_b, const CUtensorMap &ma,
                const SpmmParams &P, cudaStream_t st) {
    CUtensorMap mb;
    int rc;
    if (!B_MN) rc = make_map(&mb, b, dtype, n, k, ld_b, F8 ? 128 : 64, (uint32_t)bn);
    else rc = make_map(&mb, b, dtype, k, n, ld_b, 64, 128);
    if (rc) return rc;
    if (bn == 192) return launch_spmm<192, F8, A_MN, B_MN, TRANS, OutT>(ma, mb, P, st);
    return launch_spmm<128, F8, A_MN, B_MN, TRANS, OutT>(ma, mb, P, st);
}

}  // namespace
}  // namespace sp24

using namespace sp24;

extern "C" int sp24_meta_to_tc(const void *meta, int meta_itemsize, int64_t m, int64_t k, void *e_tc, void *stream) {
    if (!meta || !e_tc) return SP24_ERR_ARG;
    if (meta_itemsize != 2 && meta_itemsize != 4) return SP24_ERR_DTYPE;
    if (m <= 0 || k <= 0 || m % 128 || k % (meta_itemsize == 2 ? 64 : 128)) return SP24_ERR_SHAPE;
    if (!aligned16(meta) || !aligned16(e_tc)) return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    const int64_t k_atoms = (k + 127) / 128;
    const int64_t total = (m / 128) * k_atoms * (2048 / meta_itemsize);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (meta_itemsize == 2)
        meta_to_tc_kernel<2><<<blocks, 256, 0, st>>>(meta, static_cast<uint8_t *>(e_tc), m, k / 16, k_atoms);
    else
        meta_to_tc_kernel<4><<<blocks, 256, 0, st>>>(meta, static_cast<uint8_t *>(e_tc), m, k / 32, k_atoms);
    return launch_status();
}

extern "C" int64_t sp24_meta_tc_bytes(int64_t m, int64_t k) {
    if (m <= 0 || k <= 0) return 0;
    return ((m + 127) / 128) * ((k + 127) / 128) * 2048;
}

// Argument checks of sp24_spmm (everything except the metadata pointer); no CUDA call.
static int validate_spmm_args(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, int64_t ms, int64_t k,
                              const void *b, int b_mn_major, int64_t ld_b, int64_t n, const void *out, int out_dtype,
                              int trans_out, int64_t ld_out, const void *bias, int activation) {
    if (!a_packed || !b || !out) return SP24_ERR_ARG;
    const bool i8 = dtype == SP24_I8;
    const bool f8 = dtype == SP24_E4M3 || dtype == SP24_E5M2 || i8;   // 8-bit operand geometry
    if (!f8 && dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (i8 ? out_dtype != SP24_I32 : (f8 ? out_dtype != SP24_F32 : out_dtype != dtype)) return SP24_ERR_DTYPE;
    if (f8 && (a_mn_major || b_mn_major)) return SP24_ERR_DTYPE;  // 8-bit operands are K-major only
    if (i8 && (bias || activation)) return SP24_ERR_ARG;          // integer GEMM: plain product only
    if (activation < 0 || activation > 3) return SP24_ERR_ARG;
    const int esz = f8 ? 1 : 2;
    if (ms <= 0 || n <= 0 || k <= 0 || ms % 128 || k % (f8 ? 128 : 64)) return SP24_ERR_SHAPE;
    // n is free when B is stored (n, k) and the output (n, ms): rows past n are zero-filled on load and skipped
    // on store.  The other layouts have n as a contiguous extent, which must keep 16-byte row pitches.
    if ((b_mn_major || !trans_out) && n % 8) return SP24_ERR_SHAPE;
    const int64_t a_inner = a_mn_major ? ms : k / 2, b_inner = b_mn_major ? n : k, o_inner = trans_out ? ms : n;
    if (ld_a < a_inner || (ld_a * esz) % 16 || ld_b < b_inner || (ld_b * esz) % 16 || ld_out < o_inner) return SP24_ERR_STRIDE;
    if ((ld_out * dtype_size(out_dtype)) % 16) return SP24_ERR_STRIDE;
    if (!aligned16(a_packed) || !aligned16(b) || !aligned16(out)) return SP24_ERR_ALIGN;
    return SP24_OK;
}

static int spmm_impl(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *e_tc, int64_t ms,
                     int64_t k, const void *b, int b_mn_major, int64_t ld_b, int64_t n, void *out, int out_dtype,
                     int trans_out, int64_t ld_out, const void *bias, int activation, float alpha, int *status, void *stream,
                     int bias_f32 = 0, int epi = EPI_PLAIN, void *aux = nullptr, int64_t ld_aux = 0) {
    if (!e_tc) return SP24_ERR_ARG;
    if (int rc = validate_spmm_args(a_packed, dtype, a_mn_major, ld_a, ms, k, b, b_mn_major, ld_b, n, out, out_dtype,
                                    trans_out, ld_out, bias, activation))
        return rc;
    if (!aligned16(e_tc)) return SP24_ERR_ALIGN;
    const bool i8 = dtype == SP24_I8;
    const bool f8 = dtype == SP24_E4M3 || dtype == SP24_E5M2 || i8;   // 8-bit operand geometry
    // CTA-pair kernel: 16-bit types, token-major B and output, whole 256-row blocks, no activation; the fused MLP
    // epilogues and the float32 bias exist in that kernel only
    const bool pair_ok = !f8 && !b_mn_major && trans_out && ms % 256 == 0 && activation == 0;
    if (epi != EPI_PLAIN && (!pair_ok || !aux || ld_aux < ms || (ld_aux * 2) % 16 || !aligned16(aux))) return SP24_ERR_ARG;
    if (bias_f32 && !pair_ok) return SP24_ERR_ARG;
    if (int rc = check_device()) return rc;

    CUtensorMap map_a;
    int rc;
    if (!a_mn_major) rc = make_map(&map_a, a_packed, dtype, ms, k / 2, ld_a, f8 ? 128 : 64, 128);
    else rc = make_map(&map_a, a_packed, dtype, k / 2, ms, ld_a, 64, 64);
    if (rc) return rc;

    SpmmParams P{};
    P.e_tc = e_tc; P.out = out; P.bias = bias; P.ms = ms; P.n = n; P.k = k; P.ld_out = ld_out;
    P.k_atoms = (k + 127) / 128; P.status = status; P.activation = activation;
    P.trace = nullptr;
    P.k_splits = 1;
    P.alpha = alpha;
    P.bias_f32 = bias_f32;
    P.aux = aux;
    P.ld_aux = ld_aux;
#ifdef SP24_TRACE_BUILD
    if (const char *env = getenv("SP24_SPMM_TRACE_PTR")) P.trace = reinterpret_cast<unsigned long long *>(strtoull(env, nullptr, 0));
#endif
    // operand format codes: f16 0 / bf16 1; e4m3 0 / e5m2 1; unsigned 0 / signed 1 for the integer kind
    const uint32_t fmt = (dtype == SP24_BF16 || dtype == SP24_E5M2 || i8) ? 1u : 0u;
    // sparse flag, accumulator format (fp32 = 1, int32 = 2), operand formats, operand majors, M = 128 (N is added
    // by the launcher)
    P.int8 = i8 ? 1 : 0;
    P.idesc = (1u << 2) | ((i8 ? 2u : 1u) << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(a_mn_major ? 1 : 0) << 15) |
              ((uint32_t)(b_mn_major ? 1 : 0) << 16) | ((uint32_t)(BM >> 4) << 24);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    bool pair_form = pair_ok && n >= 1024 && pair_kernels_enabled();
    if (epi != EPI_PLAIN || bias_f32) pair_form = true;      // checked above: these forms exist in the pair kernel only
    if (pair_form) {
        CUtensorMap map_b, map_e;
        rc = make_map(&map_b, b, dtype, n, k, ld_b, 64, two::BN2 / 2);
        if (rc) return rc;
        rc = make_map_e(&map_e, e_tc, (ms / 128) * P.k_atoms);
        if (rc) return rc;
#define SP24_PAIR(EPI_) \
        do { \
            if (out_dtype == SP24_F16) \
                return a_mn_major ? launch_spmm_pair<true, __half, EPI_>(map_a, map_b, map_e, P, st) \
                                  : launch_spmm_pair<false, __half, EPI_>(map_a, map_b, map_e, P, st); \
            return a_mn_major ? launch_spmm_pair<true, __nv_bfloat16, EPI_>(map_a, map_b, map_e, P, st) \
                              : launch_spmm_pair<false, __nv_bfloat16, EPI_>(map_a, map_b, map_e, P, st); \
        } while (0)
        if (epi == EPI_PRE_GELU) SP24_PAIR(EPI_PRE_GELU);
        if (epi == EPI_DGELU) SP24_PAIR(EPI_DGELU);
        SP24_PAIR(EPI_PLAIN);
#undef SP24_PAIR
    }
    int bn = 128, mpt = 2;
    pick_tile(ms, n, sm_count_cached(), bn, mpt);
    P.mblk_per_tile = mpt;
#define SP24_GO(F8_, AMN_, BMN_, TR_, OT_) return dispatch_bn<F8_, AMN_, BMN_, TR_, OT_>(bn, b, dtype, n, k, ld_b, map_a, P, st)
    if (i8) {
        if (trans_out) SP24_GO(true, false, false, true, int32_t);
        SP24_GO(true, false, false, false, int32_t);
    }
    if (f8) {
        if (trans_out) SP24_GO(true, false, false, true, float);
        SP24_GO(true, false, false, false, float);
    }
    if (dtype == SP24_F16) {
        if (!a_mn_major && !b_mn_major) { if (trans_out) SP24_GO(false, false, false, true, __half); SP24_GO(false, false, false, false, __half); }
        if (a_mn_major && !b_mn_major) { if (trans_out) SP24_GO(false, true, false, true, __half); SP24_GO(false, true, false, false, __half); }
        if (!a_mn_major && b_mn_major) { if (trans_out) SP24_GO(false, false, true, true, __half); SP24_GO(false, false, true, false, __half); }
        if (trans_out) SP24_GO(false, true, true, true, __half);
        SP24_GO(false, true, true, false, __half);
    }
    if (!a_mn_major && !b_mn_major) { if (trans_out) SP24_GO(false, false, false, true, __nv_bfloat16); SP24_GO(false, false, false, false, __nv_bfloat16); }
    if (a_mn_major && !b_mn_major) { if (trans_out) SP24_GO(false, true, false, true, __nv_bfloat16); SP24_GO(false, true, false, false, __nv_bfloat16); }
    if (!a_mn_major && b_mn_major) { if (trans_out) SP24_GO(false, false, true, true, __nv_bfloat16); SP24_GO(false, false, true, false, __nv_bfloat16); }
    if (trans_out) SP24_GO(false, true, true, true, __nv_bfloat16);
    SP24_GO(false, true, true, false, __nv_bfloat16);
#undef SP24_GO
}


extern "C" int sp24_spmm(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *e_tc, int64_t ms,
                         int64_t k, const void *b, int b_mn_major, int64_t ld_b, int64_t n, void *out, int out_dtype,
                         int trans_out, int64_t ld_out, const void *bias, int activation, int *status, void *stream) {
    return spmm_impl(a_packed, dtype, a_mn_major, ld_a, e_tc, ms, k, b, b_mn_major, ld_b, n, out, out_dtype, trans_out, ld_out,
                     bias, activation, 1.f, status, stream);
}

// The 16-bit GEMM of a transformer MLP with its neighbours fused into the epilogue (CTA-pair kernel): see the header.
extern "C" int sp24_spmm_mlp(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *e_tc, int64_t ms,
                             int64_t k, const void *b, int64_t ld_b, int64_t n, void *out, int64_t ld_out, const void *bias,
                             int bias_is_f32, int epilogue, void *aux, int64_t ld_aux, int *status, void *stream) {
    if (dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (epilogue < 0 || epilogue > 2) return SP24_ERR_ARG;
    if (epilogue == EPI_DGELU && bias) return SP24_ERR_ARG;
    return spmm_impl(a_packed, dtype, a_mn_major, ld_a, e_tc, ms, k, b, 0, ld_b, n, out, dtype, 1, ld_out, bias, 0, 1.f, status,
                     stream, bias_is_f32 ? 1 : 0, epilogue, aux, ld_aux);
}

// The float8 GEMM with the dequantisation folded into the epilogue: D = alpha * (A_sparse * B) [+ bias] [activation],
// alpha = the product of the operands' per-tensor scales.  Float8 operands (float32 output) only.
extern "C" int sp24_spmm_scaled(const void *a_packed, int dtype, int64_t ld_a, const void *e_tc, int64_t ms, int64_t k,
                                const void *b, int64_t ld_b, int64_t n, float *out, int trans_out, int64_t ld_out,
                                const float *bias, int activation, float alpha, int *status, void *stream) {
    if (dtype != SP24_E4M3 && dtype != SP24_E5M2) return SP24_ERR_DTYPE;
    if (!(alpha == alpha)) return SP24_ERR_ARG;
    return spmm_impl(a_packed, dtype, 0, ld_a, e_tc, ms, k, b, 0, ld_b, n, out, SP24_F32, trans_out, ld_out, bias, activation,
                     alpha, status, stream);
}


// ------------------------------------------------------------------------------------------------
// Self-test of the bounded wait: one CTA waits on a barrier that nothing ever signals, with a small
// poll limit.  The wait must give up, record code 9 in *status and let the kernel return normally.
// ------------------------------------------------------------------------------------------------
namespace sp24 {
namespace {
__global__ void wait_selftest_kernel(int *status, uint32_t limit) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 9, limit);
    __syncthreads();
}
}  // namespace
}  // namespace sp24

extern "C" int sp24_selftest_bounded_wait(int *status, int polls, void *stream) {
    if (!status || polls <= 0 || polls > (1 << 20)) return SP24_ERR_ARG;
    if (int rc = check_device()) return rc;
    wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, (uint32_t)polls);
    return launch_status();
}

// ------------------------------------------------------------------------------------------------
// Sparse GEMM for callers that must not allocate
// ------------------------------------------------------------------------------------------------
// Some hosts of this library cannot call cudaMalloc at the point where they run the GEMM: code replayed
// under a memory plan fixed in advance, a real-time loop that may not touch the allocator, or a plug-in
// whose host application owns all device memory.  sp24_spmm needs one piece of scratch besides its
// inputs and outputs - the metadata re-ordered for the tensor cores - and normally the caller allocates
// it.  This variant keeps that scratch in a fixed array inside the library image instead.  Every GPU
// that loads the library carries the array until the process exits.
constexpr int64_t NOALLOC_SCRATCH_BYTES = 4ll << 20;  // enough for ms * k <= 32 Mi elements
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

namespace sp24 {
namespace {
// Device address of the array, looked up once per device.  In host code the array's name is only a
// handle; the address a kernel can use comes from cudaGetSymbolAddress with that device current.
int noalloc_scratch(void **out) {
    static void *cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return SP24_ERR_CUDA;
    if (dev < 0 || dev >= 64) return SP24_ERR_DEVICE;
    if (!cached[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return SP24_ERR_CUDA;
        cached[dev] = p;
    }
    *out = cached[dev];
    return SP24_OK;
}
}  // namespace
}  // namespace sp24

extern "C" int64_t sp24_spmm_noalloc_max_bytes(void) { return NOALLOC_SCRATCH_BYTES; }

extern "C" int sp24_spmm_noalloc(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *meta,
                                 int64_t ms, int64_t k, const void *b, int b_mn_major, int64_t ld_b, int64_t n, void *out,
                                 int out_dtype, int trans_out, int64_t ld_out, const void *bias, int activation,
                                 int *status, void *stream) {
    // every check of sp24_spmm comes first: a rejected call launches nothing and leaves the shared array alone
    if (!meta) return SP24_ERR_ARG;
    if (int rc = validate_spmm_args(a_packed, dtype, a_mn_major, ld_a, ms, k, b, b_mn_major, ld_b, n, out, out_dtype,
                                    trans_out, ld_out, bias, activation))
        return rc;
    if (!aligned16(meta)) return SP24_ERR_ALIGN;
    // fp8 and int8 operands carry 32-bit metadata words, the 16-bit types 16-bit words
    const bool f8 = dtype == SP24_E4M3 || dtype == SP24_E5M2 || dtype == SP24_I8;
    if (sp24_meta_tc_bytes(ms, k) > NOALLOC_SCRATCH_BYTES) return SP24_ERR_TOO_LARGE;
    if (int rc = check_device()) return rc;
    void *scratch = nullptr;
    if (int rc = noalloc_scratch(&scratch)) return rc;
    // the conversion rewrites every word the GEMM will read (padding included), so whatever an earlier
    // call left in the array does not matter
    if (int rc = sp24_meta_to_tc(meta, f8 ? 4 : 2, ms, k, scratch, stream)) return rc;
    return sp24_spmm(a_packed, dtype, a_mn_major, ld_a, scratch, ms, k, b, b_mn_major, ld_b, n, out, out_dtype, trans_out,
                     ld_out, bias, activation, status, stream);
}


// D (ms x n, fp32, row-major) += A_sparse (ms x k) * B (k x n, stored row-major): the weight-gradient form.
// K is cut into slices so that tiles x slices fills the SMs; every slice adds its partial product with fp32
// reductions, so the caller zeroes D for a plain product or passes a gradient buffer to accumulate into.
extern "C" int sp24_spmm_accumulate_f32(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *e_tc,
                                        int64_t ms, int64_t k, const void *b, int64_t ld_b, int64_t n, float *out,
                                        int64_t ld_out, int k_splits, int *status, void *stream) {
    if (!a_packed || !e_tc || !b || !out || !status) return SP24_ERR_ARG;
    if (dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (ms <= 0 || n <= 0 || k <= 0 || ms % 128 || k % 64 || n % 8) return SP24_ERR_SHAPE;
    if (k_splits < 0) return SP24_ERR_ARG;
    const int64_t a_inner = a_mn_major ? ms : k / 2;
    if (ld_a < a_inner || (ld_a * 2) % 16 || ld_b < n || (ld_b * 2) % 16 || ld_out < n || (ld_out * 4) % 16) return SP24_ERR_STRIDE;
    if (!aligned16(a_packed) || !aligned16(e_tc) || !aligned16(b) || !aligned16(out)) return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;

    CUtensorMap map_a, map_b;
    int rc;
    if (!a_mn_major) rc = make_map(&map_a, a_packed, dtype, ms, k / 2, ld_a, 64, 128);
    else rc = make_map(&map_a, a_packed, dtype, k / 2, ms, ld_a, 64, 64);
    if (rc) return rc;
    rc = make_map(&map_b, b, dtype, k, n, ld_b, 64, 128);
    if (rc) return rc;

    SpmmParams P{};
    P.e_tc = e_tc; P.out = out; P.bias = nullptr; P.ms = ms; P.n = n; P.k = k; P.ld_out = ld_out;
    P.k_atoms = (k + 127) / 128; P.status = status; P.activation = 0; P.trace = nullptr;
    P.alpha = 1.f;
    const uint32_t fmt = dtype == SP24_BF16 ? 1u : 0u;
    P.idesc = (1u << 2) | (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(a_mn_major ? 1 : 0) << 15) | (1u << 16) |
              ((uint32_t)(BM >> 4) << 24);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // CTA-pair kernel for whole 256-row blocks and at least one full tile of columns
    bool pair_form = ms % 256 == 0 && n >= 256;
    pair_form = pair_form && pair_kernels_enabled();
    if (pair_form) {
        CUtensorMap map_e;
        rc = make_map_e(&map_e, e_tc, (ms / 128) * P.k_atoms);
        if (rc) return rc;
        return a_mn_major ? launch_spmm_pair_acc<true>(map_a, map_b, map_e, P, k_splits, st)
                          : launch_spmm_pair_acc<false>(map_a, map_b, map_e, P, k_splits, st);
    }
    // widest tile (least operand traffic per output), then as many K slices as idle SMs allow
    const int sms = sm_count_cached();
    const bool wide = n >= 192;
    const int bn = wide ? 192 : 128;
    P.mblk_per_tile = ms >= 256 ? 2 : 1;
    const int64_t tiles = ((n + bn - 1) / bn) * ((ms / BM + P.mblk_per_tile - 1) / P.mblk_per_tile);
    const int64_t k_iters = (k + 127) / 128;
    int64_t splits = k_splits ? k_splits : sms / tiles;
    if (splits < 1) splits = 1;
    if (splits > k_iters) splits = k_iters;
    P.k_splits = (int)splits;
    // fp16 and bf16 operands share these kernels: the element type only enters through the tensor maps and the
    // instruction descriptor
    if (a_mn_major) return wide ? launch_spmm<192, false, true, true, false, float>(map_a, map_b, P, st)
                                : launch_spmm<128, false, true, true, false, float>(map_a, map_b, P, st);
    return wide ? launch_spmm<192, false, false, true, false, float>(map_a, map_b, P, st)
                : launch_spmm<128, false, false, true, false, float>(map_a, map_b, P, st);
}
