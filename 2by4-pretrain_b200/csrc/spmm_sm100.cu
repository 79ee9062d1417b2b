// 2:4 sparse GEMM for sm_100a:  D (Ms x N) = A_sparse (Ms x K) * B (K x N)  [+ bias per row] [activation]
//
// The sparse operand is always the tensor-core "A" operand of tcgen05.mma.sp: compressed values are
// staged in shared memory by TMA (128-byte swizzle), its metadata goes shared memory -> tensor memory
// with tcgen05.cp, the dense operand B is staged by TMA, accumulators live in tensor memory and are read
// back with tcgen05.ld by four epilogue warps.
//
// Warp roles in a CTA of 192 threads: warp 0 = TMA producer (one elected lane), warp 1 = tensor-memory
// allocation + MMA issue (one elected lane), warps 2..5 = epilogue (one TMEM lane quadrant each).
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
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
                                       uint32_t accumulate) {
    if constexpr (F8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
            "tcgen05.mma.sp.cta_group::1.kind::f8f6f4 [%0], %1, %2, [%3], %4, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
            : "memory");
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
    int activation;         // 0 none, 1 relu, 2 silu
};

template <typename OutT> __device__ __forceinline__ OutT to_out(float v);
template <> __device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <typename OutT> __device__ __forceinline__ float from_out(OutT v);
template <> __device__ __forceinline__ float from_out<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float from_out<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float from_out<float>(float v) { return v; }

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == 1) return v > 0.f ? v : 0.f;
    if (act == 2) return v / (1.f + __expf(-v));
    return v;
}

__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Geometry shared by the kernel and its launcher.
template <int BN, bool F8> struct SpmmCfg {
    static constexpr int E_BYTES = F8 ? 4096 : 2048;          // metadata of one 128-row block and one stage
    static constexpr int B_BYTES = BN * 256;                  // two 128-byte K atoms per row of B
    static constexpr int STAGE_BYTES = 2 * A_STAGE_BYTES + B_BYTES + 2 * E_BYTES;
    static constexpr int STAGES = (227 * 1024 - 2048) / STAGE_BYTES >= 4 ? 4 : (227 * 1024 - 2048) / STAGE_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;
    static_assert(STAGES >= 2, "tile too large for a two-stage ring");
    static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
};

// One CTA computes a (256 x BN) output tile as two 128-row blocks that share every stage of B
// (each byte of B staged once per 256 sparse rows).  A_MN / B_MN: operand stored with the non-K axis
// contiguous.  TRANS_OUT: write out[n][m] (row-major (N, Ms)) instead of out[m][n].
template <int BN, bool F8, bool A_MN, bool B_MN, bool TRANS_OUT, typename OutT>
__global__ void __launch_bounds__(192, 1)
spmm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, SpmmParams P) {
    using Cfg = SpmmCfg<BN, F8>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int E_BYTES = Cfg::E_BYTES;
    constexpr int OFF_B = 2 * A_STAGE_BYTES, OFF_E = OFF_B + Cfg::B_BYTES;
    constexpr int KSTEPS = 4;                 // MMA instructions per stage and row block (32 bytes of compressed A each)
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int E_COL0 = 2 * BN;            // metadata columns behind the two accumulators
    constexpr int E_SLOT = F8 ? 8 : 4;        // metadata columns of one row block and one stage
    static_assert(E_COL0 + 4 * E_SLOT <= 512, "tensor memory columns exhausted");
    static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "invalid MMA N");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 1];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_blk = blockIdx.x;
    const int mblk0 = blockIdx.y * 2;                                    // first 128-row block of this CTA
    const int n_mblk = (P.ms / BM - mblk0) >= 2 ? 2 : 1;                   // 1 on a ragged last CTA
    const int64_t m0 = (int64_t)mblk0 * BM, n0 = (int64_t)n_blk * BN;
    const int logical_k_per_stage = F8 ? 256 : 128;
    const int k_iters = (int)((P.k + logical_k_per_stage - 1) / logical_k_per_stage);
    const uint32_t stage_tx = (uint32_t)(n_mblk * (A_STAGE_BYTES + E_BYTES) + Cfg::B_BYTES);

    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), accum_bar = smem_u32(&bars[2 * STAGES]);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum_bar, 1);
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
            int issued = 0;
            for (int it = 0; it < k_iters; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (it >= STAGES && !mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, P.status, 1)) break;
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
                    for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 16384, &map_b, (int)n0 + j * 64, it * 128, full);
                }
                ++issued;
            }
            if (abort_flag) {
                // drain: wait (bounded) for the copies already issued so that none lands after exit
                for (int it = (issued > STAGES ? issued - STAGES : 0); it < issued; ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
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
            bool ok = true;
            for (int it = 0; it < k_iters && ok; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                ok = mbar_wait(full0 + 8 * s, ph, &abort_flag, P.status, 2);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
                const uint32_t sb = sa + OFF_B;
                const uint32_t se = sa + OFF_E;
                for (int mb = 0; mb < n_mblk; ++mb) {
                    const uint32_t e_cols = E_COL0 + ((it & 1) * 2 + mb) * E_SLOT;
                    // metadata: shared memory -> tensor memory, 128 lanes x 16 bytes per atom
                    tc_cp_128x128b(tmem_base + e_cols, make_desc(se + mb * E_BYTES, 16, 128, 0));
                    if constexpr (F8) tc_cp_128x128b(tmem_base + e_cols + 4, make_desc(se + mb * E_BYTES + 2048, 16, 128, 0));
#pragma unroll
                    for (int j = 0; j < KSTEPS; ++j) {
                        const uint64_t adesc = make_desc(sa + mb * A_STAGE_BYTES + j * A_KSTEP, A_LBO, 1024, 2);
                        const uint32_t b_off = B_MN ? j * B_KSTEP : (uint32_t)(j >> 1) * (BN * 128) + (j & 1) * B_KSTEP;
                        const uint64_t bdesc = make_desc(sb + b_off, B_LBO, 1024, 2);
                        const uint32_t ecol = e_cols + (F8 ? 2 * j : j);
                        // 16-bit types: the instruction takes the even column of a pair plus a 1-bit selector
                        const uint32_t e_addr = tmem_base + (F8 ? ecol : (ecol & ~1u));
                        const uint32_t idesc = P.idesc | (F8 ? 0u : (ecol & 1u));
                        mma_sp<F8>(tmem_base + mb * BN, adesc, bdesc, e_addr, idesc, (it > 0 || j > 0) ? 1u : 0u);
                    }
                }
                tc_commit(empty0 + 8 * s);  // frees the stage when these MMAs have read it
            }
            tc_commit(accum_bar);           // accumulators complete (arrives even after an abort)
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..5)
        const int quad = warp & 3;  // TMEM lane quadrant this warp may read
        const bool ok = mbar_wait(accum_bar, 0, &abort_flag, P.status, 3);
        tc_fence_after();
        const bool run = ok && !abort_flag;
        OutT *out = static_cast<OutT *>(P.out);
        for (int mb = 0; mb < n_mblk; ++mb) {
            const int64_t mrow0 = m0 + mb * BM;
            const int64_t m = mrow0 + quad * 32 + lane;
            float bias = 0.f;
            if (run && P.bias) bias = from_out<OutT>(static_cast<const OutT *>(P.bias)[m]);
            if constexpr (TRANS_OUT) {
                // stage the 128 x BN block transposed in shared memory (the operand ring is idle now), then
                // write rows of 128 consecutive outputs with 16-byte stores
                OutT *stg = reinterpret_cast<OutT *>(smem);
                if (mb > 0) epilogue_bar_sync();
                if (run) {
#pragma unroll 1
                    for (int c = 0; c < BN / 16; ++c) {
                        uint32_t v[16];
                        tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + mb * BN + c * 16, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            stg[(c * 16 + i) * BM + quad * 32 + lane] =
                                to_out<OutT>(apply_act(__uint_as_float(v[i]) + bias, P.activation));
                    }
                }
                epilogue_bar_sync();
                if (run) {
                    constexpr int PER = 16 / sizeof(OutT);          // elements per 16-byte piece
                    constexpr int PIECES = BM / PER;                // pieces per output row
                    const int tid = (warp - 2) * 32 + lane;
                    for (int i = tid; i < BN * PIECES; i += 128) {
                        const int nrow = i / PIECES, piece = i % PIECES;
                        if (n0 + nrow < P.n)
                            *reinterpret_cast<uint4 *>(out + (n0 + nrow) * P.ld_out + mrow0 + piece * PER) =
                                *reinterpret_cast<const uint4 *>(stg + nrow * BM + piece * PER);
                    }
                }
            } else if (run) {
#pragma unroll 1
                for (int c = 0; c < BN / 16; ++c) {
                    uint32_t v[16];
                    tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + mb * BN + c * 16, v);
                    tmem_ld_wait();
                    const int64_t nb = n0 + c * 16;
                    OutT *row = out + m * P.ld_out + nb;
                    if (nb + 16 <= P.n) {
                        constexpr int PER = 16 / sizeof(OutT);
#pragma unroll
                        for (int q = 0; q < 16 / PER; ++q) {
                            Vec<OutT, PER> o;
#pragma unroll
                            for (int i = 0; i < PER; ++i)
                                o.v[i] = to_out<OutT>(apply_act(__uint_as_float(v[q * PER + i]) + bias, P.activation));
                            store_vec<OutT, PER>(row + q * PER, o);
                        }
                    } else {
                        for (int i = 0; i < 16; ++i)
                            if (nb + i < P.n) row[i] = to_out<OutT>(apply_act(__uint_as_float(v[i]) + bias, P.activation));
                    }
                }
            }
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
    const CUresult r = encode(map, tmap_dtype(dt), 2, const_cast<void *>(base), dims, strides, box, estr,
                                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? SP24_OK : SP24_ERR_CUDA;
}

template <int BN, bool F8, bool A_MN, bool B_MN, bool TRANS, typename OutT>
int launch_spmm(const CUtensorMap &ma, const CUtensorMap &mb, SpmmParams P, cudaStream_t st) {
    using Cfg = SpmmCfg<BN, F8>;
    auto kern = spmm_kernel<BN, F8, A_MN, B_MN, TRANS, OutT>;
    static bool attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
            return SP24_ERR_CUDA;
        attr_set[dev] = true;
    }
    P.idesc |= (uint32_t)(BN >> 3) << 17;
    dim3 grid((unsigned)((P.n + BN - 1) / BN), (unsigned)((P.ms / BM + 1) / 2));
    kern<<<grid, 192, Cfg::SMEM, st>>>(ma, mb, P);
    return launch_status();
}

// Tile width: the candidates trade operand traffic per output (wide is better) against how evenly the
// CTAs fill the SMs.  Cost model: waves x K iterations x bytes staged per iteration.
int pick_bn(int64_t ms, int64_t n, int sm_count, bool b_mn) {
    const int cand[3] = {240, 176, 128};
    int best = 128;
    double best_cost = 1e300;
    for (int i = 0; i < 3; ++i) {
        const int bn = cand[i];
        if (b_mn && bn % 64) continue;  // MN-major B is staged in 64-column blocks
        const int64_t ctas = ((n + bn - 1) / bn) * ((ms / BM + 1) / 2);
        const double waves = (double)((ctas + sm_count - 1) / sm_count);
        const double cost = waves * (2 * A_STAGE_BYTES + bn * 256 + 4096);
        if (cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

int sm_count_cached() {
    static int cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

template <bool F8, bool A_MN, bool B_MN, bool TRANS, typename OutT>
int dispatch_bn(int bn, const void *b, int dtype, int64_t n, int64_t k, int64_t ld_b, const CUtensorMap &ma,
                const SpmmParams &P, cudaStream_t st) {
    CUtensorMap mb;
    int rc;
    if (!B_MN) rc = make_map(&mb, b, dtype, n, k, ld_b, F8 ? 128 : 64, (uint32_t)bn);
    else rc = make_map(&mb, b, dtype, k, n, ld_b, 64, 128);
    if (rc) return rc;
    if constexpr (B_MN) {
        if (bn == 128) return launch_spmm<128, F8, A_MN, B_MN, TRANS, OutT>(ma, mb, P, st);
        return launch_spmm<192, F8, A_MN, B_MN, TRANS, OutT>(ma, mb, P, st);
    } else {
        if (bn == 240) return launch_spmm<240, F8, A_MN, B_MN, TRANS, OutT>(ma, mb, P, st);
        if (bn == 176) return launch_spmm<176, F8, A_MN, B_MN, TRANS, OutT>(ma, mb, P, st);
        return launch_spmm<128, F8, A_MN, B_MN, TRANS, OutT>(ma, mb, P, st);
    }
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

extern "C" int sp24_spmm(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *e_tc, int64_t ms,
                         int64_t k, const void *b, int b_mn_major, int64_t ld_b, int64_t n, void *out, int out_dtype,
                         int trans_out, int64_t ld_out, const void *bias, int activation, int *status, void *stream) {
    if (!a_packed || !e_tc || !b || !out) return SP24_ERR_ARG;
    const bool f8 = dtype == SP24_E4M3 || dtype == SP24_E5M2;
    if (!f8 && dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (f8 ? out_dtype != SP24_F32 : out_dtype != dtype) return SP24_ERR_DTYPE;
    if (f8 && (a_mn_major || b_mn_major)) return SP24_ERR_DTYPE;  // 8-bit operands are K-major only
    if (activation < 0 || activation > 2) return SP24_ERR_ARG;
    const int esz = f8 ? 1 : 2;
    if (ms <= 0 || n <= 0 || k <= 0 || ms % 128 || k % (f8 ? 128 : 64) || n % 8) return SP24_ERR_SHAPE;
    const int64_t a_inner = a_mn_major ? ms : k / 2, b_inner = b_mn_major ? n : k, o_inner = trans_out ? ms : n;
    if (ld_a < a_inner || (ld_a * esz) % 16 || ld_b < b_inner || (ld_b * esz) % 16 || ld_out < o_inner) return SP24_ERR_STRIDE;
    if ((ld_out * dtype_size(out_dtype)) % 16) return SP24_ERR_STRIDE;
    if (!aligned16(a_packed) || !aligned16(e_tc) || !aligned16(b) || !aligned16(out)) return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;

    CUtensorMap map_a;
    int rc;
    if (!a_mn_major) rc = make_map(&map_a, a_packed, dtype, ms, k / 2, ld_a, f8 ? 128 : 64, 128);
    else rc = make_map(&map_a, a_packed, dtype, k / 2, ms, ld_a, 64, 64);
    if (rc) return rc;

    SpmmParams P{};
    P.e_tc = e_tc; P.out = out; P.bias = bias; P.ms = ms; P.n = n; P.k = k; P.ld_out = ld_out;
    P.k_atoms = (k + 127) / 128; P.status = status; P.activation = activation;
    const uint32_t fmt = (dtype == SP24_BF16 || dtype == SP24_E5M2) ? 1u : 0u;
    // sparse flag, fp32 accumulate, operand formats, operand majors, M = 128 (N is added by the launcher)
    P.idesc = (1u << 2) | (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(a_mn_major ? 1 : 0) << 15) |
              ((uint32_t)(b_mn_major ? 1 : 0) << 16) | ((uint32_t)(BM >> 4) << 24);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int bn;
    if (b_mn_major) {
        // candidates 192 and 128 (multiples of the 64-column staging block)
        const int sms = sm_count_cached();
        const int64_t mp = (ms / BM + 1) / 2;
        const double c192 = (double)((((n + 191) / 192) * mp + sms - 1) / sms) * (2 * A_STAGE_BYTES + 192 * 256 + 4096);
        const double c128 = (double)((((n + 127) / 128) * mp + sms - 1) / sms) * (2 * A_STAGE_BYTES + 128 * 256 + 4096);
        bn = c192 <= c128 ? 192 : 128;
    } else {
        bn = pick_bn(ms, n, sm_count_cached(), false);
    }
#define SP24_GO(F8_, AMN_, BMN_, TR_, OT_) return dispatch_bn<F8_, AMN_, BMN_, TR_, OT_>(bn, b, dtype, n, k, ld_b, map_a, P, st)
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
