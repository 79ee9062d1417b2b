// Transposable 4x4 mask select, alone and fused with the 2:4 compression of W and of W^T.
//
// One thread owns one 4x4 block.  The 90 admissible patterns (two ones per row and per column), in
// descending lexicographic order of the row-major bit string, are the nested order "row 0 pair, row 1
// pair, row 2 pair, row 3 pair" over the pair list (0,1) (0,2) (0,3) (1,2) (1,3) (2,3).  Scores are
// float32 with a fixed association, (s0 + s1) + (s2 + s3), s_i = v[i][a] + v[i][b], and the first
// maximum wins.  The search is hierarchical (best bottom per top pair, then first top, then first
// bottom) and returns exactly what the flat scan over the 90 patterns would.
#include "sp24_common.cuh"

namespace sp24 {
namespace {

// ---------------------------------------------------------------------------------------------
// compile-time description of the 90 patterns
// ---------------------------------------------------------------------------------------------
// Column pairs in table order: 0:(0,1) 1:(0,2) 2:(0,3) 3:(1,2) 4:(1,3) 5:(2,3); pair 5-p is the complement of p.
__host__ __device__ constexpr int pair_a(int i) { return i < 3 ? 0 : (i < 5 ? 1 : 2); }
__host__ __device__ constexpr int pair_b(int i) { return i < 3 ? i + 1 : (i < 5 ? i - 1 : 3); }
__host__ __device__ constexpr int row_bits(int i) { return (1 << pair_a(i)) | (1 << pair_b(i)); }
__host__ __device__ constexpr int pair_of(int c0, int c1) {
    const int lo = c0 < c1 ? c0 : c1, hi = c0 < c1 ? c1 : c0;
    return lo == 0 ? hi - 1 : (lo == 1 ? hi + 1 : 5);
}
// A pattern is (a, b, c, d) = the pairs of rows 0..3.  Given the pairs (a, b) of the two top rows, the
// admissible bottoms are: a == b -> only (5-a, 5-a); b == 5-a -> (c, 5-c) for every c; otherwise the two
// top rows share one column s and leave one column r unused, and the bottoms are {r,p},{r,q} in either
// order (p, q = the unshared columns of a and b).
__host__ __device__ constexpr int top_type(int a, int b) { return a == b ? 0 : (b == 5 - a ? 2 : 1); }
__host__ __device__ constexpr int shared_bottom(int a, int b, int which) {
    const int a0 = pair_a(a), a1 = pair_b(a), b0 = pair_a(b), b1 = pair_b(b);
    const int s = (a0 == b0 || a0 == b1) ? a0 : a1;
    const int p = a0 == s ? a1 : a0, q = b0 == s ? b1 : b0;
    const int r = 6 - s - p - q;
    const int x0 = pair_of(r, p), y0 = pair_of(r, q);
    const int x = x0 < y0 ? x0 : y0, y = x0 < y0 ? y0 : x0;
    return which == 0 ? x : y;
}
constexpr uint32_t PATTERN0 = 0x33CCu & 0xFFFFu;  // rows (0,1),(0,1),(2,3),(2,3): bits 0011 0011 1100 1100 read high to low

// Lookup words.  [0,36): per top (a*6+b): bits 0..7 rows 0-1, 8..15 first bottom, 16..23 second bottom,
// 24..25 type.  [36,42): bottoms (c, 5-c).  [48,64): per 4-bit keep mask: bits 0..3 metadata code
// idx0 | idx1 << 2, bits 8..23 byte-permute selector that gathers the 16-bit elements idx0, idx1 of
// a (lo, hi) register pair.
struct SelectLut { uint32_t v[64]; };
__host__ __device__ constexpr uint32_t encode_nibble_c(uint32_t mask) {
    const uint32_t m0 = mask & 1u, m1 = (mask >> 1) & 1u, m2 = (mask >> 2) & 1u;
    const uint32_t bit0 = (m0 ^ 1u) & m1, bit1 = (m0 ^ 1u) & (m1 ^ 1u);
    const uint32_t bit2 = bit1 | (m2 ^ 1u), bit3 = bit0 | (m1 ^ 1u) | m2;
    return bit0 | (bit1 << 1) | (bit2 << 2) | (bit3 << 3);
}
constexpr SelectLut make_select_lut() {
    SelectLut L{};
    for (int a = 0; a < 6; ++a)
        for (int b = 0; b < 6; ++b) {
            const int ty = top_type(a, b);
            uint32_t bot0 = 0, bot1 = 0;
            if (ty == 0) bot0 = row_bits(5 - a) | (row_bits(5 - a) << 4);
            if (ty == 1) {
                const int x = shared_bottom(a, b, 0), y = shared_bottom(a, b, 1);
                bot0 = row_bits(x) | (row_bits(y) << 4);
                bot1 = row_bits(y) | (row_bits(x) << 4);
            }
            L.v[a * 6 + b] = (uint32_t)(row_bits(a) | (row_bits(b) << 4)) | (bot0 << 8) | (bot1 << 16) | ((uint32_t)ty << 24);
        }
    for (int c = 0; c < 6; ++c) L.v[36 + c] = row_bits(c) | (row_bits(5 - c) << 4);
    for (uint32_t k = 0; k < 16; ++k) {
        const uint32_t nib = encode_nibble_c(k), i0 = nib & 3u, i1 = nib >> 2;
        const uint32_t sel = (2 * i0) | ((2 * i0 + 1) << 4) | ((2 * i1) << 8) | ((2 * i1 + 1) << 12);
        L.v[48 + k] = nib | (sel << 8);
    }
    return L;
}
__constant__ SelectLut kSelectLut = make_select_lut();

// v: the 4x4 block (already |.| when requested); lut: shared-memory copy of kSelectLut.
// Returns the 16-bit pattern (bit 4*i+j = keep (i, j)) that a scan over all 90 patterns in table order with
// "replace only when strictly greater" would return, with far fewer instructions: the best bottom for every
// top pair is a max over at most six sums (rounding is monotone, so max-then-add equals add-then-max), the
// 36 top pairs are scanned once in table order with a running strict maximum, and the winning bottom is the
// first admissible one that reaches the maximum with the winning top.
__device__ __forceinline__ uint32_t select_pattern(const float (&v)[4][4], const uint32_t *lut) {
    float s[4][6];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int p = 0; p < 6; ++p) s[i][p] = __fadd_rn(v[i][pair_a(p)], v[i][pair_b(p)]);
    auto top = [&](int a, int b) { return __fadd_rn(s[0][a], s[1][b]); };
    auto bot = [&](int c, int d) { return __fadd_rn(s[2][c], s[3][d]); };
    float max_c = bot(0, 5);
#pragma unroll
    for (int c = 1; c < 6; ++c) max_c = fmaxf(max_c, bot(c, 5 - c));
    // One pass over the 36 top pairs in table order, as two independent chains of 18 (instruction-level
    // parallelism): a candidate replaces the running best only when strictly greater, so the first maximum
    // wins inside a chain, and the second chain replaces the first only when strictly greater.  NaN totals
    // never win; if nothing ever exceeds -inf the answer stays at top 0 (pattern 0), like the flat scan.
    float best[2] = {-INFINITY, -INFINITY}, tv[2] = {0.f, 0.f}, c0v[2] = {0.f, 0.f};
    int ts[2] = {0, 18};
#pragma unroll
    for (int t = 0; t < 36; ++t) {
        const int a = t / 6, b = t % 6, h = t / 18;
        const float tp = top(a, b);
        float bb, first_bot = 0.f;
        if (top_type(a, b) == 0) bb = bot(5 - a, 5 - a);
        else if (top_type(a, b) == 2) bb = max_c;
        else {
            first_bot = bot(shared_bottom(a, b, 0), shared_bottom(a, b, 1));
            bb = fmaxf(first_bot, bot(shared_bottom(a, b, 1), shared_bottom(a, b, 0)));
        }
        const float tot = __fadd_rn(tp, bb);
        if (tot > best[h]) {
            best[h] = tot;
            ts[h] = t;
            tv[h] = tp;
            if (top_type(a, b) == 1) c0v[h] = first_bot;
        }
    }
    const bool second = best[1] > best[0];
    const float m = second ? best[1] : best[0];
    const int tstar = second ? ts[1] : ts[0];
    const float t_val = second ? tv[1] : tv[0];
    const float cand0 = second ? c0v[1] : c0v[0];
    const bool first = __fadd_rn(t_val, cand0) == m;
    int cstar = 0;
#pragma unroll
    for (int c = 5; c >= 0; --c)
        if (__fadd_rn(t_val, bot(c, 5 - c)) == m) cstar = c;
    const uint32_t e = lut[tstar];
    const uint32_t ty = e >> 24;
    const uint32_t bot_bits = ty == 2 ? lut[36 + cstar] : ((ty == 1 && !first) ? ((e >> 16) & 0xFFu) : ((e >> 8) & 0xFFu));
    uint32_t bits = (e & 0xFFu) | (bot_bits << 8);
    if (!(m > -INFINITY)) bits = row_bits(0) | (row_bits(0) << 4) | (row_bits(5) << 8) | (row_bits(5) << 12);
    return bits;
}

__device__ __forceinline__ void load_select_lut(uint32_t *lut) {
    if (threadIdx.x < 64) lut[threadIdx.x] = kSelectLut.v[threadIdx.x];
    __syncthreads();
}

template <typename T> __device__ __forceinline__ void load_row4(const T *p, T (&out)[4]) {
    Vec<T, 4> v = load_vec<T, 4>(p);
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = v.v[j];
}

// keep bits of one row -> four mask bytes (0 / 1)
__device__ __forceinline__ uint32_t spread_mask_bytes(uint32_t rb) { return (rb * 0x00204081u) & 0x01010101u; }
// four mask bytes (non-zero = keep) -> keep bits
__device__ __forceinline__ uint32_t gather_mask_bytes(uint32_t mw) {
    return ((__vcmpne4(mw, 0u) & 0x01010101u) * 0x01020408u) >> 24;
}

// ---------------------------------------------------------------------------------------------
// select only: x -> (sparse, mask)
// block = 8 warps = 8 block-rows (32 rows) x 32 block-columns (128 columns)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) ts_select_kernel(const T *x, T *sparse, uint8_t *mask, int64_t k, int64_t ld_x,
                                                        int64_t ld_s, int64_t ld_m, int use_abs) {
    __shared__ uint32_t lut[64];
    load_select_lut(lut);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t r = (int64_t)blockIdx.y * 32 + warp * 4;
    const int64_t c = (int64_t)blockIdx.x * 128 + lane * 4;
    if (c >= k) return;
    T w[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) load_row4<T>(x + (r + i) * ld_x + c, w[i]);
    float v[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float f = Elem<T>::to_f32(w[i][j]);
            v[i][j] = use_abs ? fabsf(f) : f;
        }
    const uint32_t bits = select_pattern(v, lut);
    const T zero = Elem<T>::from_f32(0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t rb = (bits >> (4 * i)) & 0xFu;
        *reinterpret_cast<uint32_t *>(mask + (r + i) * ld_m + c) = spread_mask_bytes(rb);
        if (sparse) {
            Vec<T, 4> o;
#pragma unroll
            for (int j = 0; j < 4; ++j) o.v[j] = ((rb >> j) & 1u) ? w[i][j] : zero;
            store_vec<T, 4>(sparse + (r + i) * ld_s + c, o);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// select (or read mask) + compress W and W^T.  Same thread mapping as above.
// ---------------------------------------------------------------------------------------------
struct DualParams {
    const void *w;
    uint8_t *mask;
    void *packed_w, *packed_t;
    int16_t *meta_w, *meta_t;
    int64_t m, k, ld_w, ld_mask, ld_pw, ld_pt;
    // optional second copy of the metadata in the order the sparse GEMM reads (2048-byte atoms per 128 rows x 128
    // columns, int16 index 8*L + 2*q + h with L = 16*(r/16) + 8*(c%2) + r%8, q = (c/2)%4, h = (r/8)%2 for row r of
    // the 128-row block and metadata word column c); requires m % 128 == 0 and k % 128 == 0
    int16_t *tc_w, *tc_t;
    int64_t tc_w_bytes, tc_t_bytes;   // sizes of the two copies: every store is checked against them
};

// four elements of a row as two registers of packed 16-bit output values (low half = lower column)
template <typename T, typename TOut> __device__ __forceinline__ void pack_row(const T (&w)[4], uint32_t &lo, uint32_t &hi) {
    if constexpr (std::is_same<T, TOut>::value) {
        lo = *reinterpret_cast<const uint32_t *>(&w[0]);
        hi = *reinterpret_cast<const uint32_t *>(&w[2]);
    } else {
        TOut o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = convert<TOut>(w[j]);
        lo = (uint32_t) * reinterpret_cast<const uint16_t *>(&o[0]) | ((uint32_t) * reinterpret_cast<const uint16_t *>(&o[1]) << 16);
        hi = (uint32_t) * reinterpret_cast<const uint16_t *>(&o[2]) | ((uint32_t) * reinterpret_cast<const uint16_t *>(&o[3]) << 16);
    }
}

// Work of one block: 64 rows x 128 columns at block coordinates (bx, by) of the matrix P describes.
template <typename T, typename TOut, bool SELECT, bool TC>
__device__ __forceinline__ void ts_dual_block(const DualParams &P, const unsigned bx, const unsigned by) {
    // Metadata words are staged in the order they are produced (one cheap store per producer); the few threads
    // that write them out gather them into the reference's run order (and the tensor-core order) afterwards.
    __shared__ __align__(8) uint16_t wlin[8 * 8 * 4];   // W: [warp = 4-row group][word column][row in group]
    __shared__ __align__(4) uint16_t tlin[2 * 128];     // W^T: [word column parity][W column]
    __shared__ __align__(4) uint8_t nib_t[8][128];      // [block row][W column]
    __shared__ uint32_t lut[64];
    load_select_lut(lut);

    // A block covers 64 rows x 128 columns as two 32-row halves.  Both halves are loaded up front so that
    // the second half's global loads are in flight while the first half is being searched.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t c0 = (int64_t)bx * 128, c = c0 + lane * 4;
    const bool active = c < P.k;
    const T *w_ptr = static_cast<const T *>(P.w);
    uint16_t *pw = static_cast<uint16_t *>(P.packed_w);
    uint16_t *pt = static_cast<uint16_t *>(P.packed_t);

    T w[4][4], w_next[4][4];
    uint32_t mw[4] = {0, 0, 0, 0}, mw_next[4] = {0, 0, 0, 0};
    if (active) {
        const int64_t ra = (int64_t)by * 64 + warp * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            load_row4<T>(w_ptr + (ra + i) * P.ld_w + c, w[i]);
            load_row4<T>(w_ptr + (ra + 32 + i) * P.ld_w + c, w_next[i]);
            if constexpr (!SELECT) {
                mw[i] = *reinterpret_cast<const uint32_t *>(P.mask + (ra + i) * P.ld_mask + c);
                mw_next[i] = *reinterpret_cast<const uint32_t *>(P.mask + (ra + 32 + i) * P.ld_mask + c);
            }
        }
    }

#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
        const int64_t r0 = (int64_t)by * 64 + half * 32;
        const int64_t r = r0 + warp * 4;
        uint32_t bits = 0;
        uint32_t h[4][2] = {{0, 0}, {0, 0}, {0, 0}, {0, 0}};  // the block as packed 16-bit output values
        if (active) {
#pragma unroll
            for (int i = 0; i < 4; ++i) pack_row<T, TOut>(w[i], h[i][0], h[i][1]);
            if constexpr (SELECT) {
                float v[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[i][j] = fabsf(Elem<T>::to_f32(w[i][j]));
                bits = select_pattern(v, lut);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<uint32_t *>(P.mask + (r + i) * P.ld_mask + c) = spread_mask_bytes((bits >> (4 * i)) & 0xFu);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) bits |= gather_mask_bytes(mw[i]) << (4 * i);
            }
        }
        // rows of W: table lookup gives the metadata code and the byte-permute selector of the two kept values
        uint32_t nib01 = 0, nib23 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t e = lut[48 + ((bits >> (4 * i)) & 0xFu)];
            if (active) *reinterpret_cast<uint32_t *>(pw + (r + i) * P.ld_pw + (c >> 1)) = __byte_perm(h[i][0], h[i][1], e >> 8);
            if (i < 2) nib01 |= (e & 0xFu) << (16 * i);
            else nib23 |= (e & 0xFu) << (16 * (i - 2));
        }
        // four horizontally adjacent lanes make one 16-bit metadata word per row (two rows per register)
        nib01 <<= 4 * (lane & 3);
        nib23 <<= 4 * (lane & 3);
        nib01 |= __shfl_xor_sync(0xFFFFFFFFu, nib01, 1);
        nib23 |= __shfl_xor_sync(0xFFFFFFFFu, nib23, 1);
        nib01 |= __shfl_xor_sync(0xFFFFFFFFu, nib01, 2);
        nib23 |= __shfl_xor_sync(0xFFFFFFFFu, nib23, 2);
        if ((lane & 3) == 0)   // word column lane / 4, rows warp*4 .. warp*4+3: (row 0, row 1) and (row 2, row 3)
            *reinterpret_cast<uint2 *>(&wlin[(warp * 8 + (lane >> 2)) * 4]) = make_uint2(nib01, nib23);
        // columns of W (= rows of W^T): transpose the 4x4 block of 16-bit values, then the same table lookup
        {
            uint32_t pj[4], nibs = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t sel_t = (j & 1) ? 0x7632u : 0x5410u;
                const uint32_t c_lo = __byte_perm(h[0][j >> 1], h[1][j >> 1], sel_t);  // (w[0][j], w[1][j])
                const uint32_t c_hi = __byte_perm(h[2][j >> 1], h[3][j >> 1], sel_t);  // (w[2][j], w[3][j])
                const uint32_t cb = ((((bits >> j) & 0x1111u) * 0x1248u) >> 12) & 0xFu;  // keep bits of column j
                const uint32_t e = lut[48 + cb];
                pj[j] = __byte_perm(c_lo, c_hi, e >> 8);
                nibs |= (e & 0xFu) << (8 * j);
            }
            // one 32-bit store per thread: [block row][column] keeps the four columns of a thread together
            *reinterpret_cast<uint32_t *>(&nib_t[0][0] + (warp * 128 + lane * 4)) = nibs;
            if (active) {
                uint2 o0, o1;
                o0.x = __byte_perm(pj[0], pj[1], 0x5410u); o0.y = __byte_perm(pj[2], pj[3], 0x5410u);
                o1.x = __byte_perm(pj[0], pj[1], 0x7632u); o1.y = __byte_perm(pj[2], pj[3], 0x7632u);
                *reinterpret_cast<uint2 *>(pt + (r >> 1) * P.ld_pt + c) = o0;
                *reinterpret_cast<uint2 *>(pt + ((r >> 1) + 1) * P.ld_pt + c) = o1;
            }
        }
        __syncthreads();
        {
            // thread t: W column t>>1, metadata column parity t&1 of the transposed matrix; the bytes of
            // block rows 4*par .. 4*par+3 for that column sit 128 bytes apart
            const int col = threadIdx.x >> 1, par = threadIdx.x & 1;
            const uint8_t *nb = &nib_t[0][0] + (par * 4) * 128 + col;
            const uint32_t word = (uint32_t)nb[0] | ((uint32_t)nb[128] << 4) | ((uint32_t)nb[256] << 8) | ((uint32_t)nb[384] << 12);
            tlin[par * 128 + col] = (uint16_t)word;
        }
        __syncthreads();
        // Write-out.  In the reference layout the 64 words of (32 rows x one word-column pair) form one 128-byte
        // run; its 16-byte piece p holds, in this order, the words (row, parity) = (p,0) (8+p,0) (p,1) (8+p,1)
        // (16+p,0) (24+p,0) (16+p,1) (24+p,1).
        if (threadIdx.x < 32) {
            // W: 4 word-column pairs x 8 pieces
            const int pair = threadIdx.x >> 3, piece = threadIdx.x & 7;
            const int64_t cp = c0 / 32 + pair;
            if (cp * 2 < P.k / 16) {
                auto wd = [&](int q, int par) { return (uint32_t)wlin[((2 * q + (piece >> 2)) * 8 + pair * 2 + par) * 4 + (piece & 3)]; };
                uint4 o;
                o.x = wd(0, 0) | (wd(1, 0) << 16); o.y = wd(0, 1) | (wd(1, 1) << 16);
                o.z = wd(2, 0) | (wd(3, 0) << 16); o.w = wd(2, 1) | (wd(3, 1) << 16);
                char *dst = reinterpret_cast<char *>(P.meta_w) + (cp * 2 * P.m + 2 * r0) * 2 + piece * 16;
                *reinterpret_cast<uint4 *>(dst) = o;
            }
        } else if (threadIdx.x < 64) {
            // W^T: 4 groups of 32 W columns x 8 pieces, one word-column pair (the 32 rows of this half)
            const int grp = (threadIdx.x - 32) >> 3, piece = threadIdx.x & 7;
            const int64_t cols_here = (P.k - c0 < 128) ? (P.k - c0) : 128;
            if (grp * 32 < cols_here) {
                auto wd = [&](int q, int par) { return (uint32_t)tlin[par * 128 + grp * 32 + q * 8 + piece]; };
                uint4 o;
                o.x = wd(0, 0) | (wd(1, 0) << 16); o.y = wd(0, 1) | (wd(1, 1) << 16);
                o.z = wd(2, 0) | (wd(3, 0) << 16); o.w = wd(2, 1) | (wd(3, 1) << 16);
                const int64_t cp = r0 / 32;  // column pair of the (k, m) metadata matrix
                char *dst = reinterpret_cast<char *>(P.meta_t) + (cp * 2 * P.k + 2 * c0) * 2 + (grp * 8 + piece) * 16;
                *reinterpret_cast<uint4 *>(dst) = o;
            }
        }
        if constexpr (TC) {
            // tensor-core order: line L = 16*(r/16) + 8*(c%2) + r%8 of 16 bytes holds the int16 slots 2*((c/2)%4) + (r/8)%2
            if (threadIdx.x >= 64 && threadIdx.x < 96) {
                // W: 32 lines, contiguous in the atom of (row block r0/128, column block c0/128)
                const int L = threadIdx.x - 64, par = (L >> 3) & 1;
                auto wd = [&](int q, int hh) {
                    const int rr = 16 * (L >> 4) + 8 * hh + (L & 7);
                    return (uint32_t)wlin[((rr >> 2) * 8 + 2 * q + par) * 4 + (rr & 3)];
                };
                uint4 o;
                o.x = wd(0, 0) | (wd(0, 1) << 16); o.y = wd(1, 0) | (wd(1, 1) << 16);
                o.z = wd(2, 0) | (wd(2, 1) << 16); o.w = wd(3, 0) | (wd(3, 1) << 16);
                const int64_t off = ((r0 >> 7) * (P.k >> 7) + (c0 >> 7)) * 2048 + ((r0 & 127) + L) * 16;
                if (off >= 0 && off + 16 <= P.tc_w_bytes) *reinterpret_cast<uint4 *>(reinterpret_cast<char *>(P.tc_w) + off) = o;
            }
            if (threadIdx.x >= 128) {
                // W^T: row block c0/128, word columns r0/16 and r0/16 + 1: one 4-byte piece (h = 0, 1) per line L
                const int L = threadIdx.x - 128, par = (L >> 3) & 1;
                const int col = 16 * (L >> 4) + (L & 7);
                const uint32_t o = (uint32_t)tlin[par * 128 + col] | ((uint32_t)tlin[par * 128 + col + 8] << 16);
                const int64_t wc = r0 >> 4;
                const int64_t off = ((c0 >> 7) * (P.m >> 7) + (wc >> 3)) * 2048 + L * 16 + ((wc >> 1) & 3) * 4;
                if (off >= 0 && off + 4 <= P.tc_t_bytes) *reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(P.tc_t) + off) = o;
            }
        }
        __syncthreads();  // the staging arrays are rewritten by the next half
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j) w[i][j] = w_next[i][j];
            mw[i] = mw_next[i];
        }
    }
}

template <typename T, typename TOut, bool SELECT, bool TC>
// three CTAs per SM for 16-bit inputs (80 registers); fp32 inputs need more registers and keep two
__global__ void __launch_bounds__(256, sizeof(T) == 2 ? 3 : 2) ts_dual_kernel(DualParams P) {
    ts_dual_block<T, TOut, SELECT, TC>(P, blockIdx.x, blockIdx.y);
}

// Several matrices in one launch (the per-step recompression of all the layers of a model: each matrix alone is
// too small to fill the GPU).  Blocks are numbered through the matrices one after the other; first[i] is the first
// block of matrix i.
constexpr int kDualBatchMax = 48;
struct DualBatch {
    DualParams p[kDualBatchMax];
    unsigned first[kDualBatchMax + 1];
    int count;
};
template <typename T, typename TOut, bool SELECT, bool TC>
__global__ void __launch_bounds__(256, sizeof(T) == 2 ? 3 : 2) ts_dual_batch_kernel(const __grid_constant__ DualBatch B) {
    int i = 0;
    while (i + 1 < B.count && blockIdx.x >= B.first[i + 1]) ++i;
    const DualParams &P = B.p[i];
    const unsigned local = blockIdx.x - B.first[i];
    const unsigned ncb = (unsigned)((P.k + 127) / 128);
    ts_dual_block<T, TOut, SELECT, TC>(P, local % ncb, local / ncb);
}

template <typename T, typename TOut> int launch_dual(const DualParams &P, int select, cudaStream_t st) {
    dim3 grid((unsigned)((P.k + 127) / 128), (unsigned)(P.m / 64));
    const bool tc = P.tc_w != nullptr;
    if (select) {
        if (tc) ts_dual_kernel<T, TOut, true, true><<<grid, 256, 0, st>>>(P);
        else ts_dual_kernel<T, TOut, true, false><<<grid, 256, 0, st>>>(P);
    } else {
        if (tc) ts_dual_kernel<T, TOut, false, true><<<grid, 256, 0, st>>>(P);
        else ts_dual_kernel<T, TOut, false, false><<<grid, 256, 0, st>>>(P);
    }
    return launch_status();
}

template <typename T, typename TOut> int launch_dual_batch(const DualBatch &B, int select, bool tc, cudaStream_t st) {
    const unsigned grid = B.first[B.count];
    if (select) {
        if (tc) ts_dual_batch_kernel<T, TOut, true, true><<<grid, 256, 0, st>>>(B);
        else ts_dual_batch_kernel<T, TOut, true, false><<<grid, 256, 0, st>>>(B);
    } else {
        if (tc) ts_dual_batch_kernel<T, TOut, false, true><<<grid, 256, 0, st>>>(B);
        else ts_dual_batch_kernel<T, TOut, false, false><<<grid, 256, 0, st>>>(B);
    }
    return launch_status();
}

template <typename T> int dispatch_dual_batch(const DualBatch &B, int packed_dtype, int select, bool tc, cudaStream_t st) {
    if (packed_dtype == SP24_F16) return launch_dual_batch<T, __half>(B, select, tc, st);
    if (packed_dtype == SP24_BF16) return launch_dual_batch<T, __nv_bfloat16>(B, select, tc, st);
    return SP24_ERR_DTYPE;
}

template <typename T> int dispatch_dual(const DualParams &P, int packed_dtype, int select, cudaStream_t st) {
    if (packed_dtype == SP24_F16) return launch_dual<T, __half>(P, select, st);
    if (packed_dtype == SP24_BF16) return launch_dual<T, __nv_bfloat16>(P, select, st);
    return SP24_ERR_DTYPE;
}

}  // namespace
}  // namespace sp24

using namespace sp24;

extern "C" int sp24_transposable_select(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int use_abs,
                                        void *sparse_out, int64_t ld_sparse, void *mask_out, int64_t ld_mask,
                                        void *stream) {
    if (!x || !mask_out) return SP24_ERR_ARG;
    if (dtype != SP24_F32 && dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (m <= 0 || k <= 0 || m % 32 || k % 64) return SP24_ERR_SHAPE;
    const int sz = dtype_size(dtype);
    if (ld_x < k || (ld_x * sz) % 16 || ld_mask < k || ld_mask % 16) return SP24_ERR_STRIDE;
    if (sparse_out && (ld_sparse < k || (ld_sparse * sz) % 16)) return SP24_ERR_STRIDE;
    if (!aligned16(x) || !aligned16(mask_out) || (sparse_out && !aligned16(sparse_out))) return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)((k + 127) / 128), (unsigned)(m / 32));
    uint8_t *mk = static_cast<uint8_t *>(mask_out);
    switch (dtype) {
        case SP24_F32:
            ts_select_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float *>(x), static_cast<float *>(sparse_out), mk,
                                                          k, ld_x, ld_sparse, ld_mask, use_abs);
            break;
        case SP24_F16:
            ts_select_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half *>(x), static_cast<__half *>(sparse_out),
                                                           mk, k, ld_x, ld_sparse, ld_mask, use_abs);
            break;
        default:
            ts_select_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(x),
                                                                  static_cast<__nv_bfloat16 *>(sparse_out), mk, k, ld_x,
                                                                  ld_sparse, ld_mask, use_abs);
    }
    return launch_status();
}

// Argument checks of one matrix; fills P.  No CUDA call.
static int make_dual_params(const void *w, int dtype, int64_t m, int64_t k, int64_t ld_w, void *mask, int64_t ld_mask,
                            void *packed_w, int packed_dtype, int64_t ld_packed_w, void *meta_w, void *packed_t,
                            int64_t ld_packed_t, void *meta_t, void *tc_w, void *tc_t, DualParams *P) {
    if (!w || !mask || !packed_w || !meta_w || !packed_t || !meta_t) return SP24_ERR_ARG;
    if (dtype != SP24_F32 && dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (packed_dtype != SP24_F16 && packed_dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (m <= 0 || k <= 0 || m % 64 || k % 64) return SP24_ERR_SHAPE;
    if ((tc_w || tc_t) && (m % 128 || k % 128)) return SP24_ERR_SHAPE;
    const int sz = dtype_size(dtype);
    if (ld_w < k || (ld_w * sz) % 16 || ld_mask < k || ld_mask % 16) return SP24_ERR_STRIDE;
    if (ld_packed_w < k / 2 || ld_packed_w % 8 || ld_packed_t < k || ld_packed_t % 8) return SP24_ERR_STRIDE;
    if (!aligned16(w) || !aligned16(mask) || !aligned16(packed_w) || !aligned16(meta_w) || !aligned16(packed_t) ||
        !aligned16(meta_t) || (tc_w && !aligned16(tc_w)) || (tc_t && !aligned16(tc_t)))
        return SP24_ERR_ALIGN;
    *P = DualParams{w, static_cast<uint8_t *>(mask), packed_w, packed_t, static_cast<int16_t *>(meta_w),
                    static_cast<int16_t *>(meta_t), m, k, ld_w, ld_mask, ld_packed_w, ld_packed_t,
                    static_cast<int16_t *>(tc_w), static_cast<int16_t *>(tc_t), (m / 128) * (k / 128) * 2048,
                    (k / 128) * (m / 128) * 2048};
    return SP24_OK;
}

static int select_dual_compress_impl(const void *w, int dtype, int64_t m, int64_t k, int64_t ld_w, int select, void *mask,
                                     int64_t ld_mask, void *packed_w, int packed_dtype, int64_t ld_packed_w, void *meta_w,
                                     void *packed_t, int64_t ld_packed_t, void *meta_t, void *tc_w, void *tc_t,
                                     void *stream) {
    DualParams P;
    if (int rc = make_dual_params(w, dtype, m, k, ld_w, mask, ld_mask, packed_w, packed_dtype, ld_packed_w, meta_w,
                                  packed_t, ld_packed_t, meta_t, tc_w, tc_t, &P))
        return rc;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case SP24_F32: return dispatch_dual<float>(P, packed_dtype, select, st);
        case SP24_F16: return dispatch_dual<__half>(P, packed_dtype, select, st);
        default: return dispatch_dual<__nv_bfloat16>(P, packed_dtype, select, st);
    }
}

// Same conversion for `count` matrices of one element type in as few launches as possible (48 matrices per launch).
// Either every descriptor carries both tensor-core metadata pointers or none does.
extern "C" int sp24_select_dual_compress_batch(const sp24_dual_desc *descs, int count, int dtype, int packed_dtype,
                                               int select, void *stream) {
    if (!descs || count <= 0) return SP24_ERR_ARG;
    const bool tc = descs[0].tc_w != nullptr;
    for (int i = 0; i < count; ++i)
        if ((descs[i].tc_w != nullptr) != tc || (descs[i].tc_t != nullptr) != tc) return SP24_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    bool device_checked = false;
    for (int base = 0; base < count; base += kDualBatchMax) {
        DualBatch B;
        B.count = count - base < kDualBatchMax ? count - base : kDualBatchMax;
        uint64_t blocks = 0;
        for (int i = 0; i < B.count; ++i) {
            const sp24_dual_desc &d = descs[base + i];
            if (int rc = make_dual_params(d.w, dtype, d.m, d.k, d.ld_w, d.mask, d.ld_mask, d.packed_w, packed_dtype,
                                          d.ld_packed_w, d.meta_w, d.packed_t, d.ld_packed_t, d.meta_t, d.tc_w, d.tc_t,
                                          &B.p[i]))
                return rc;
            B.first[i] = (unsigned)blocks;
            blocks += (uint64_t)((d.k + 127) / 128) * (uint64_t)(d.m / 64);
            if (blocks > 0x7FFFFFFFull) return SP24_ERR_TOO_LARGE;
        }
        B.first[B.count] = (unsigned)blocks;
        if (!device_checked) {
            if (int rc = check_device()) return rc;
            device_checked = true;
        }
        int rc;
        switch (dtype) {
            case SP24_F32: rc = dispatch_dual_batch<float>(B, packed_dtype, select, tc, st); break;
            case SP24_F16: rc = dispatch_dual_batch<__half>(B, packed_dtype, select, tc, st); break;
            default: rc = dispatch_dual_batch<__nv_bfloat16>(B, packed_dtype, select, tc, st);
        }
        if (rc) return rc;
    }
    return SP24_OK;
}

extern "C" int sp24_select_dual_compress(const void *w, int dtype, int64_t m, int64_t k, int64_t ld_w, int select,
                                         void *mask, int64_t ld_mask, void *packed_w, int packed_dtype,
                                         int64_t ld_packed_w, void *meta_w, void *packed_t, int64_t ld_packed_t,
                                         void *meta_t, void *stream) {
    return select_dual_compress_impl(w, dtype, m, k, ld_w, select, mask, ld_mask, packed_w, packed_dtype, ld_packed_w,
                                     meta_w, packed_t, ld_packed_t, meta_t, nullptr, nullptr, stream);
}

// Same pass, which also writes the metadata of W (tc_w, sp24_meta_tc_bytes(m, k) bytes) and of W^T (tc_t,
// sp24_meta_tc_bytes(k, m) bytes) in the order the sparse GEMM reads, so that no conversion launch is needed
// before sp24_spmm.  Requires m % 128 == 0 and k % 128 == 0.
extern "C" int sp24_select_dual_compress_tc(const void *w, int dtype, int64_t m, int64_t k, int64_t ld_w, int select,
                                            void *mask, int64_t ld_mask, void *packed_w, int packed_dtype,
                                            int64_t ld_packed_w, void *meta_w, void *packed_t, int64_t ld_packed_t,
                                            void *meta_t, void *tc_w, void *tc_t, void *stream) {
    if (!tc_w || !tc_t) return SP24_ERR_ARG;
    return select_dual_compress_impl(w, dtype, m, k, ld_w, select, mask, ld_mask, packed_w, packed_dtype, ld_packed_w,
                                     meta_w, packed_t, ld_packed_t, meta_t, tc_w, tc_t, stream);
}
