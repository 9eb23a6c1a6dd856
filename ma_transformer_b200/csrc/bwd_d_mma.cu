// 16-bit backward of window attention for head widths other than 64 on the warp-level tensor-core
// instructions.
//
// The reference's backward takes any head width (sparse_attention_backward_kernel,
// src/cuda/sparse_attention_kernel.cu:265-346).  The TMA-staged kernels of bwd_mma.cu are laid out for 128-byte
// rows (D = 64); other widths used to fall to the one-warp-per-row kernels of backward.cu.  This file has the
// control flow of the fp32 tensor-core backward (bwd_f32_mma.cu: 64-row tiles, the band walked in 64-column
// chunks through two cp.async buffers, a rows pass with two sweeps, a dV pass and a dK pass, statistics in the
// workspace) with the products of the 16-bit forward for these widths (mma_window_d.cu: ldmatrix from rows padded
// by 16 bytes, mma.sync.m16n8k16, the accumulator tiles of one product packed into the A fragments of the next;
// P and dS rounded to the input type for the second products, as in bwd_mma.cu).
#include <algorithm>
#include <cstring>

#include "mat_common.cuh"
#include "ptx.cuh"

namespace mat {
namespace {

constexpr int kT = 64, kThreads = 128;

struct BwdDArgs {
    const void *q, *k, *v, *go;
    void *dq, *dk, *dv;
    float2 *stats;             // [B, HH, S]: (log2-sum-exp of the scaled scores, delta * scale)
    int32_t S, HH;             // rows and heads of the (possibly dilated) view
    int32_t left, right;
    float scale;
    int32_t D;                 // head width (read by the kernel for wide heads only)
    float *scr_dq, *scr_dk, *scr_dv;   // wide heads, walks of more than two passes: fp32 copies of the three outputs' shape, or null
};

__device__ __forceinline__ void cp_async16(void *dst, const void *src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(ptx::smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ float quad_max(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    return fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x + __shfl_xor_sync(0xffffffffu, x, 2);
}

constexpr int kRows = 0, kColsV = 1, kColsK = 2;

// PASS = kRows: tile rows are queries, columns keys.  kColsV / kColsK: tile rows are keys, columns queries.
// NS = 0: the band is walked in 64-column chunks shared by the four warps (two buffers).  NS > 0, for narrow windows:
// every warp walks the columns from a base of its own, the first column its first row meets, in passes of NS
// 16-column steps, so that no step is without a visible column but the last of the walk (5 steps instead of 8 at 64
// causal taps); the CTA stages the 48 + 16 NS rows the four warps' passes span, in one buffer.
template <typename T, int D, int PASS, int NS>
__global__ void __launch_bounds__(kThreads)
bwd_d_kernel(const BwdDArgs a) {
    using M = ptx::Mma<T>;
    constexpr int LD = D + 8, KS = D / 16;   // padded row (elements); 16-wide steps of the head dimension
    constexpr bool COLS = PASS != kRows, DIAG = NS > 0;
    constexpr int STEPS = DIAG ? NS : 4;                        // 16-column steps a warp takes per chunk or pass
    constexpr int kRowsStaged = DIAG ? 48 + 16 * NS : 2 * kT;   // rows of each operand in shared memory
    extern __shared__ __align__(16) uint8_t smem_raw[];
    T *sY1 = reinterpret_cast<T *>(smem_raw);          // rows pass K, cols passes Q
    T *sY2 = sY1 + kRowsStaged * LD;                   // rows pass V, cols passes dO
    float2 *sSt = reinterpret_cast<float2 *>(sY2 + kRowsStaged * LD);   // cols passes: statistics of the staged queries

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m4 = lane >> 3, r8 = lane & 7;
    const int hh = blockIdx.x, b = blockIdx.z, r0 = blockIdx.y * kT;
    const int back = COLS ? a.right : a.left, fwd = COLS ? a.left : a.right;   // row r sees columns r - back .. r + fwd
    const int col_lo = max(0, r0 - back);
    const int col_hi = min(a.S - 1, min(r0 + kT, a.S) - 1 + fwd);
    const int base_w = max(col_lo, r0 + 16 * warp - back);   // (NS > 0) the warp's first column
    int n_chunks = 0;                                        // chunks, or passes of the warp with the longest walk
    if (col_hi >= col_lo) {
        if constexpr (DIAG) {
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) {
                const int cols_w = min(col_hi, r0 + 16 * w + 15 + fwd) - max(col_lo, r0 + 16 * w - back) + 1;
                n_chunks = max(n_chunks, (cols_w + 16 * NS - 1) / (16 * NS));
            }
            n_chunks = min(n_chunks, (col_hi - col_lo) / (16 * NS) + 1);
        } else {
            n_chunks = (col_hi - col_lo) / kT + 1;
        }
    }
    const int64_t tok = (int64_t)a.HH * D;
    const int64_t head = ((int64_t)b * a.S * a.HH + hh) * D;
    const T *x1 = (const T *)(COLS ? a.k : a.q) + head, *x2 = (const T *)(COLS ? a.v : a.go) + head;
    const T *y1 = (const T *)(COLS ? a.q : a.k) + head, *y2 = (const T *)(COLS ? a.go : a.v) + head;
    const float2 *st_in = a.stats + ((int64_t)b * a.HH + hh) * a.S;

    // chunk c into buffer buf (NS = 0), or the rows of pass c (warp 0's base is col_lo) into the one buffer
    auto load_chunk = [&](int c, int buf) {
        constexpr int kPieces = D / 8;
        constexpr int kStage = DIAG ? kRowsStaged : kT;
        const int base = col_lo + c * (DIAG ? 16 * NS : kT);
        for (int i = threadIdx.x; i < kStage * kPieces; i += kThreads) {
            const int r = i / kPieces, pc = i % kPieces;
            const int j = base + r;
            const bool in = j < a.S;   // rows past the end are zero-filled
            const int64_t src = (int64_t)(in ? j : 0) * tok + pc * 8;
            cp_async16(sY1 + (buf * kT + r) * LD + pc * 8, y1 + src, in ? 16 : 0);
            cp_async16(sY2 + (buf * kT + r) * LD + pc * 8, y2 + src, in ? 16 : 0);
        }
        static_assert(kStage <= kThreads, "one thread per staged row's statistics");
        if (COLS && threadIdx.x < kStage) {
            const int j = base + threadIdx.x;
            sSt[buf * kT + threadIdx.x] = j < a.S ? st_in[j] : make_float2(0.f, 0.f);
        }
    };
    if (!DIAG && n_chunks > 0) load_chunk(0, 0);
    cp_async_commit();

    // the warp's 16 tile rows as A fragments: rows g and g + 8, columns 2t, 2t+1 (+8) of each 16
    const int row_a = r0 + 16 * warp + g, row_b = row_a + 8;
    uint32_t xf1[KS][4], xf2[PASS == kColsV ? 1 : KS][4];
    {
        const T *pa = x1 + (int64_t)row_a * tok, *pb = x1 + (int64_t)row_b * tok;
        const T *qa = x2 + (int64_t)row_a * tok, *qb = x2 + (int64_t)row_b * tok;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 16 + 2 * t;
            xf1[ks][0] = row_a < a.S ? *reinterpret_cast<const uint32_t *>(pa + c) : 0u;
            xf1[ks][1] = row_b < a.S ? *reinterpret_cast<const uint32_t *>(pb + c) : 0u;
            xf1[ks][2] = row_a < a.S ? *reinterpret_cast<const uint32_t *>(pa + c + 8) : 0u;
            xf1[ks][3] = row_b < a.S ? *reinterpret_cast<const uint32_t *>(pb + c + 8) : 0u;
            if constexpr (PASS != kColsV) {
                xf2[ks][0] = row_a < a.S ? *reinterpret_cast<const uint32_t *>(qa + c) : 0u;
                xf2[ks][1] = row_b < a.S ? *reinterpret_cast<const uint32_t *>(qb + c) : 0u;
                xf2[ks][2] = row_a < a.S ? *reinterpret_cast<const uint32_t *>(qa + c + 8) : 0u;
                xf2[ks][3] = row_b < a.S ? *reinterpret_cast<const uint32_t *>(qb + c + 8) : 0u;
            }
        }
    }
    const float sl = a.scale * 1.4426950408889634f;
    const int rows[2] = {row_a, row_b};
    // column j of row r counts iff -back <= j - r <= fwd and j exists
    auto seen = [&](int j, int r) { return (unsigned)(j - r + back) <= (unsigned)(back + fwd) && j < a.S; };

    float acc[2 * KS][4];   // dQ, dV or dK of the warp's rows
#pragma unroll
    for (int n = 0; n < 2 * KS; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f}, dr[2] = {0.f, 0.f}, lse[2] = {0.f, 0.f}, dsc[2] = {0.f, 0.f};

    // the tile's product with 16 of the chunk's rows: (out0 | out1) (16 x 16) = X (16 x D) . Y[n2*16 .. n2*16+15]^T
    auto product = [&](float (&out0)[4], float (&out1)[4], const uint32_t (&xf)[KS][4], uint32_t y_addr, int n2) {
        out0[0] = out0[1] = out0[2] = out0[3] = 0.f;
        out1[0] = out1[1] = out1[2] = out1[3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            // matrices: (columns n2*16 + 0..7, dims +0), (same columns, dims +8), (columns +8, dims +0), (columns +8, dims +8)
            uint32_t yf[4];
            ptx::ldmatrix_x4(yf, y_addr + (uint32_t)(((n2 * 16 + r8 + (m4 >> 1) * 8) * LD + ks * 16 + (m4 & 1) * 8) * 2));
            M::run(out0, xf[ks], yf[0], yf[1]);
            M::run(out1, xf[ks], yf[2], yf[3]);
        }
    };
    // acc += W (16 x 16: two accumulator tiles, rounded to the input type) . Y[n2*16 .. n2*16+15] (16 x D)
    auto accumulate = [&](const float (&w0)[4], const float (&w1)[4], uint32_t y_addr, int n2) {
        const uint32_t wa[4] = {M::pack(w0[0], w0[1]), M::pack(w0[2], w0[3]), M::pack(w1[0], w1[1]), M::pack(w1[2], w1[3])};
#pragma unroll
        for (int d2 = 0; d2 < KS; ++d2) {
            // matrices (transposed on load): (columns n2*16 + 0..7, dims d2*16 + 0..7), (columns +8, same dims),
            // (columns + 0, dims + 8), (columns + 8, dims + 8)
            uint32_t yf[4];
            ptx::ldmatrix_x4_trans(yf, y_addr + (uint32_t)(((n2 * 16 + r8 + (m4 & 1) * 8) * LD + d2 * 16 + (m4 >> 1) * 8) * 2));
            M::run(acc[2 * d2], wa, yf[0], yf[1]);
            M::run(acc[2 * d2 + 1], wa, yf[2], yf[3]);
        }
    };

    const int total = PASS == kRows ? 2 * n_chunks : n_chunks;   // the rows pass walks the keys twice
    for (int n = 0; n < total; ++n) {
        const int c = n_chunks ? n % n_chunks : 0, buf = DIAG ? 0 : n & 1;
        if constexpr (DIAG) {
            if (n == 0 || n_chunks > 1) {   // a one-pass walk keeps its rows for the second sweep
                if (n) __syncthreads();     // the previous pass has been read
                load_chunk(c, 0);
                cp_async_commit();
                cp_async_wait<0>();
                __syncthreads();
            }
        } else {
            if (n + 1 < total) {
                load_chunk((n + 1) % n_chunks, buf ^ 1);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
        }
        const int cb = DIAG ? base_w + c * 16 * NS : col_lo + c * kT;       // the first column of the warp's steps
        const int st_off = DIAG ? cb - (col_lo + c * 16 * NS) : buf * kT;   // its row in shared memory
        const uint32_t cy1 = ptx::smem_u32(sY1 + st_off * LD), cy2 = ptx::smem_u32(sY2 + st_off * LD);

        if (PASS == kRows && n == n_chunks) {   // between the sweeps: the statistics are complete
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                sum[i] = quad_sum(sum[i]);
                dr[i] = quad_sum(dr[i]);
                const bool live = sum[i] > 0.f;
                lse[i] = live ? mx[i] * sl + log2f(sum[i]) : 0.f;
                dsc[i] = live ? dr[i] / sum[i] * a.scale : 0.f;
                if (t == 0 && rows[i] < a.S) a.stats[((int64_t)b * a.HH + hh) * a.S + rows[i]] = make_float2(lse[i], dsc[i]);
            }
        }
        bool sweep_one = false;
        if constexpr (PASS == kRows) sweep_one = n < n_chunks;
        if (sweep_one) {
          if constexpr (PASS == kRows) {
            // ---- sweep one: running maximum, sum of exponentials, sum of exponentials x dP ----
            float s[2 * STEPS][4];
            float cm[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n2 = 0; n2 < STEPS; ++n2) {
                product(s[2 * n2], s[2 * n2 + 1], xf1, cy1, n2);
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int nt = 2 * n2 + h2;
                        if (!seen(cb + nt * 8 + 2 * t + (e & 1), rows[e >> 1])) s[nt][e] = -INFINITY;
                        cm[e >> 1] = fmaxf(cm[e >> 1], s[nt][e]);
                    }
            }
            float msl[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float m_new = fmaxf(mx[i], quad_max(cm[i]));
                const float alpha = mx[i] == -INFINITY ? 0.f : ptx::ex2((mx[i] - m_new) * sl);
                sum[i] *= alpha;
                dr[i] *= alpha;
                mx[i] = m_new;
                msl[i] = m_new == -INFINITY ? 0.f : m_new * sl;
            }
#pragma unroll
            for (int n2 = 0; n2 < STEPS; ++n2) {
                float dp[2][4];
                product(dp[0], dp[1], xf2, cy2, n2);
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float ex = ptx::ex2(fmaf(s[2 * n2 + h2][e], sl, -msl[e >> 1]));
                        sum[e >> 1] += ex;
                        dr[e >> 1] = fmaf(ex, dp[h2][e], dr[e >> 1]);
                    }
            }
          }
        } else {
            // ---- rows pass, sweep two: dS, dQ += dS K.  cols passes: P^T (and dS^T), dV += P^T dO / dK += dS^T Q ----
#pragma unroll
            for (int n2 = 0; n2 < STEPS; ++n2) {
                float s[2][4], w[2][4];
                product(s[0], s[1], xf1, cy1, n2);
                float dp[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                if constexpr (PASS != kColsV) product(dp[0], dp[1], xf2, cy2, n2);
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int col = (2 * n2 + h2) * 8 + 2 * t + (e & 1);
                        // the query's statistics: the row's own (rows pass) or the column's (cols passes)
                        const float2 sq = COLS ? sSt[st_off + col] : make_float2(lse[e >> 1], dsc[e >> 1]);
                        float p = ptx::ex2(fmaf(s[h2][e], sl, -sq.x));
                        if (!seen(cb + col, rows[e >> 1])) p = 0.f;
                        w[h2][e] = PASS == kColsV ? p : p * fmaf(dp[h2][e], a.scale, -sq.y);
                    }
                accumulate(w[0], w[1], PASS == kColsV ? cy2 : cy1, n2);
            }
        }
        if (!DIAG) __syncthreads();   // the buffer is free for the chunk after the next
    }
    if (PASS == kRows && n_chunks == 0 && t == 0) {   // rows that see no key
#pragma unroll
        for (int i = 0; i < 2; ++i)
            if (rows[i] < a.S) a.stats[((int64_t)b * a.HH + hh) * a.S + rows[i]] = make_float2(0.f, 0.f);
    }
    T *out = (T *)(PASS == kRows ? a.dq : PASS == kColsV ? a.dv : a.dk) + head;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (rows[i] < a.S) {
            T *dst = out + (int64_t)rows[i] * tok + 2 * t;
#pragma unroll
            for (int d = 0; d < 2 * KS; ++d)
                *reinterpret_cast<uint32_t *>(dst + d * 8) = M::pack(acc[d][2 * i], acc[d][2 * i + 1]);
        }
    }
}

// Wide heads (D = 128, 192, ... 512) with narrow windows.  The same three passes and per-warp column ranges (passes
// of five 16-column steps from the warp's own first column), with the head dimension taken 64 columns at a time:
// the two score-shaped products of a pass (S and dP, or their transposes) accumulate in registers over the slices
// of their operands, staged one slice at a time; the weights (P^T or dS, rounded to the input type) are formed once,
// and every 64-column slice of the output is their product with one more staged slice, written out - added to what
// the first pass of the same rows wrote when the walk has a second one (a row of dQ, dK or dV belongs to one thread
// pair of one CTA: no atomics).  Walks of more passes keep the sums in fp32 copies of the outputs' shape (the
// caller's workspace) until a row's last pass rounds them: 16-bit values cannot carry fifty partial sums.  Registers hold one pass's two score tiles and one slice's fragments whatever D is.
// A one-pass walk (windows of at most 64 taps) keeps S and dP from the statistics sweep instead of recomputing them.
template <typename T, int PASS, int NS>
__global__ void __launch_bounds__(kThreads)
bwd_d_wide_kernel(const BwdDArgs a) {
    using M = ptx::Mma<T>;
    constexpr int LD = 64 + 8, KS = 4;
    constexpr int kStage = 48 + 16 * NS;
    constexpr bool COLS = PASS != kRows;
    constexpr bool kTwo = PASS != kColsV;   // two score-shaped products (S and dP); the dV pass needs only S^T
    extern __shared__ __align__(16) uint8_t smem_raw[];
    T *sY1 = reinterpret_cast<T *>(smem_raw);   // a slice of: rows pass K, cols passes Q
    T *sY2 = sY1 + kStage * LD;                 // a slice of: rows pass V, cols passes dO
    float2 *sSt = reinterpret_cast<float2 *>(sY2 + kStage * LD);   // cols passes: statistics of the staged queries

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m4 = lane >> 3, r8 = lane & 7;
    const int hh = blockIdx.x, b = blockIdx.z, r0 = blockIdx.y * kT;
    const int D = a.D, n_slices = (D + 63) >> 6;   // (the last slice may be partly beyond D: zeros in, nothing out)
    const int back = COLS ? a.right : a.left, fwd = COLS ? a.left : a.right;   // row r sees columns r - back .. r + fwd
    const int col_lo = max(0, r0 - back);
    const int col_hi = min(a.S - 1, min(r0 + kT, a.S) - 1 + fwd);
    const int base_w = max(col_lo, r0 + 16 * warp - back);   // the warp's first column
    int n_pass = 0;
    if (col_hi >= col_lo) {
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) {
            const int cols_w = min(col_hi, r0 + 16 * w + 15 + fwd) - max(col_lo, r0 + 16 * w - back) + 1;
            n_pass = max(n_pass, (cols_w + 16 * NS - 1) / (16 * NS));
        }
        n_pass = min(n_pass, (col_hi - col_lo) / (16 * NS) + 1);
    }
    const int64_t tok = (int64_t)a.HH * D;
    const int64_t head = ((int64_t)b * a.S * a.HH + hh) * D;
    const T *x1 = (const T *)(COLS ? a.k : a.q) + head, *x2 = (const T *)(COLS ? a.v : a.go) + head;
    const T *y1 = (const T *)(COLS ? a.q : a.k) + head, *y2 = (const T *)(COLS ? a.go : a.v) + head;
    const float2 *st_in = a.stats + ((int64_t)b * a.HH + hh) * a.S;
    const int row_a = r0 + 16 * warp + g, row_b = row_a + 8;
    const int rows[2] = {row_a, row_b};
    const float sl = a.scale * 1.4426950408889634f;
    auto seen = [&](int j, int r) { return (unsigned)(j - r + back) <= (unsigned)(back + fwd) && j < a.S; };

    // 64 columns (slice) of the kStage rows from `first` on, of one operand, into one buffer; rows past the end are zeros
    auto stage = [&](T *dst, const T *src, int first, int slice) {
        for (int x = threadIdx.x; x < kStage * 8; x += kThreads) {
            const int r = x >> 3, pc = x & 7;
            const int j = first + r;
            const bool in = j < a.S && slice * 64 + pc * 8 < D;
            cp_async16(dst + r * LD + pc * 8, src + (int64_t)(in ? j : 0) * tok + slice * 64 + pc * 8, in ? 16 : 0);
        }
    };
    // the warp's 16 rows of a slice as A fragments: rows g and g + 8, columns 2t, 2t+1 (+8) of each 16
    auto load_x = [&](uint32_t (&xf)[KS][4], const T *x, int slice) {
        const T *pa = x + (int64_t)row_a * tok + slice * 64, *pb = x + (int64_t)row_b * tok + slice * 64;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 16 + 2 * t, col = slice * 64 + c;   // (D is a multiple of 8: each half of a 16-column step is inside D or beyond it)
            xf[ks][0] = row_a < a.S && col < D ? *reinterpret_cast<const uint32_t *>(pa + c) : 0u;
            xf[ks][1] = row_b < a.S && col < D ? *reinterpret_cast<const uint32_t *>(pb + c) : 0u;
            xf[ks][2] = row_a < a.S && col + 8 < D ? *reinterpret_cast<const uint32_t *>(pa + c + 8) : 0u;
            xf[ks][3] = row_b < a.S && col + 8 < D ? *reinterpret_cast<const uint32_t *>(pb + c + 8) : 0u;
        }
    };
    // pass c: s (and dp) = the warp's rows against its NS steps of 16 columns, summed over the slices
    auto scores = [&](int c, float (&s)[2 * NS][4], float (&dp)[2 * NS][4], int st_off) {
#pragma unroll
        for (int n = 0; n < 2 * NS; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = dp[n][e] = 0.f;
        const int first = col_lo + c * 16 * NS;
        for (int slice = 0; slice < n_slices; ++slice) {
            uint32_t xf1[KS][4], xf2[kTwo ? KS : 1][4];
            load_x(xf1, x1, slice);
            if constexpr (kTwo) load_x(xf2, x2, slice);
            __syncthreads();   // whoever still read the buffers is done
            stage(sY1, y1, first, slice);
            if constexpr (kTwo) stage(sY2, y2, first, slice);
            if (COLS && slice == 0) {
                for (int x = threadIdx.x; x < kStage; x += kThreads) {
                    const int j = first + x;
                    sSt[x] = j < a.S ? st_in[j] : make_float2(0.f, 0.f);
                }
            }
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
            const uint32_t cy1 = ptx::smem_u32(sY1 + st_off * LD), cy2 = ptx::smem_u32(sY2 + st_off * LD);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                for (int n2 = 0; n2 < NS; ++n2) {
                    // matrices: (columns n2*16 + 0..7, dims +0), (same columns, dims +8), (columns +8, dims +0), (columns +8, dims +8)
                    const uint32_t off = (uint32_t)(((n2 * 16 + r8 + (m4 >> 1) * 8) * LD + ks * 16 + (m4 & 1) * 8) * 2);
                    uint32_t yf[4];
                    ptx::ldmatrix_x4(yf, cy1 + off);
                    M::run(s[2 * n2], xf1[ks], yf[0], yf[1]);
                    M::run(s[2 * n2 + 1], xf1[ks], yf[2], yf[3]);
                    if constexpr (kTwo) {
                        ptx::ldmatrix_x4(yf, cy2 + off);
                        M::run(dp[2 * n2], xf2[ks], yf[0], yf[1]);
                        M::run(dp[2 * n2 + 1], xf2[ks], yf[2], yf[3]);
                    }
                }
        }
    };
    // out rows (+)= W (the pass's weights as A fragments) . Y, 64 columns of Y at a time
    float *const out32 = (PASS == kRows ? a.scr_dq : PASS == kColsV ? a.scr_dv : a.scr_dk) == nullptr
                             ? nullptr : (PASS == kRows ? a.scr_dq : PASS == kColsV ? a.scr_dv : a.scr_dk) + head;
    auto emit = [&](int c, const uint32_t (&wa)[NS][4], const T *y, T *out, int st_off) {
        const int first = col_lo + c * 16 * NS;
        for (int slice = 0; slice < n_slices; ++slice) {
            __syncthreads();
            stage(sY1, y, first, slice);
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
            const uint32_t cy = ptx::smem_u32(sY1 + st_off * LD);
            float acc[2 * KS][4];
#pragma unroll
            for (int n = 0; n < 2 * KS; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll
            for (int n2 = 0; n2 < NS; ++n2)
#pragma unroll
                for (int d2 = 0; d2 < KS; ++d2) {
                    // matrices (transposed on load): (columns n2*16 + 0..7, dims d2*16 + 0..7), (columns +8, same dims),
                    // (columns + 0, dims + 8), (columns + 8, dims + 8)
                    uint32_t yf[4];
                    ptx::ldmatrix_x4_trans(yf, cy + (uint32_t)(((n2 * 16 + r8 + (m4 & 1) * 8) * LD + d2 * 16 + (m4 >> 1) * 8) * 2));
                    M::run(acc[2 * d2], wa[n2], yf[0], yf[1]);
                    M::run(acc[2 * d2 + 1], wa[n2], yf[2], yf[3]);
                }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (rows[i] >= a.S) continue;
                T *dst = out + (int64_t)rows[i] * tok + slice * 64 + 2 * t;
#pragma unroll
                for (int n = 0; n < 2 * KS; ++n) {
                    if (slice * 64 + n * 8 + 2 * t >= D) continue;
                    float vx = acc[n][2 * i], vy = acc[n][2 * i + 1];
                    if (out32) {   // many passes: the sums stay in fp32 until the row's last pass rounds them
                        float2 *sc = reinterpret_cast<float2 *>(out32 + (int64_t)rows[i] * tok + slice * 64 + 2 * t + n * 8);
                        if (c > 0) { const float2 old = *sc; vx += old.x; vy += old.y; }
                        if (c + 1 < n_pass) { *sc = make_float2(vx, vy); continue; }
                    } else if (c > 0) {   // the first pass of these rows wrote here
                        const uint32_t old = *reinterpret_cast<const uint32_t *>(dst + n * 8);
                        vx += M::lo(old);
                        vy += M::hi(old);
                    }
                    *reinterpret_cast<uint32_t *>(dst + n * 8) = M::pack(vx, vy);
                }
            }
        }
    };
    T *out = (T *)(PASS == kRows ? a.dq : PASS == kColsV ? a.dv : a.dk) + head;
    if (n_pass == 0) {   // rows that meet no column: zero gradient (and zero statistics)
        for (int i = 0; i < 2; ++i) {
            if (rows[i] >= a.S) continue;
            for (int c = 2 * t; c < D; c += 8) *reinterpret_cast<uint32_t *>(out + (int64_t)rows[i] * tok + c) = 0u;
            if (PASS == kRows && t == 0) a.stats[((int64_t)b * a.HH + hh) * a.S + rows[i]] = make_float2(0.f, 0.f);
        }
        return;
    }

    float s[2 * NS][4], dp[2 * NS][4];
    uint32_t wa[NS][4];
    const int st_off = base_w - col_lo;
    if constexpr (PASS == kRows) {
        float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f}, dr[2] = {0.f, 0.f}, lse[2], dsc[2];
        // sweep one: running maximum, sum of exponentials, sum of exponentials x dP
        for (int c = 0; c < n_pass; ++c) {
            const int cb = base_w + c * 16 * NS;
            scores(c, s, dp, st_off);
            float cm[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 2 * NS; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (!seen(cb + n * 8 + 2 * t + (e & 1), rows[e >> 1])) s[n][e] = -INFINITY;
                    cm[e >> 1] = fmaxf(cm[e >> 1], s[n][e]);
                }
            float msl[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float m_new = fmaxf(mx[i], quad_max(cm[i]));
                const float alpha = mx[i] == -INFINITY ? 0.f : ptx::ex2((mx[i] - m_new) * sl);
                sum[i] *= alpha;
                dr[i] *= alpha;
                mx[i] = m_new;
                msl[i] = m_new == -INFINITY ? 0.f : m_new * sl;
            }
#pragma unroll
            for (int n = 0; n < 2 * NS; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float ex = ptx::ex2(fmaf(s[n][e], sl, -msl[e >> 1]));
                    sum[e >> 1] += ex;
                    dr[e >> 1] = fmaf(ex, dp[n][e], dr[e >> 1]);
                }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            sum[i] = quad_sum(sum[i]);
            dr[i] = quad_sum(dr[i]);
            const bool live = sum[i] > 0.f;
            lse[i] = live ? mx[i] * sl + log2f(sum[i]) : 0.f;
            dsc[i] = live ? dr[i] / sum[i] * a.scale : 0.f;
            if (t == 0 && rows[i] < a.S) a.stats[((int64_t)b * a.HH + hh) * a.S + rows[i]] = make_float2(lse[i], dsc[i]);
        }
        // sweep two: dS, dQ (+)= dS K; a one-pass walk still holds S (masked) and dP
        for (int c = 0; c < n_pass; ++c) {
            const int cb = base_w + c * 16 * NS;
            if (n_pass > 1) scores(c, s, dp, st_off);
#pragma unroll
            for (int n = 0; n < 2 * NS; ++n) {
                float w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float p = ptx::ex2(fmaf(s[n][e], sl, -lse[e >> 1]));
                    if (!seen(cb + n * 8 + 2 * t + (e & 1), rows[e >> 1])) p = 0.f;
                    w[e] = p * fmaf(dp[n][e], a.scale, -dsc[e >> 1]);
                }
                wa[n >> 1][(n & 1) * 2] = M::pack(w[0], w[1]);
                wa[n >> 1][(n & 1) * 2 + 1] = M::pack(w[2], w[3]);
            }
            emit(c, wa, y1, out, st_off);
        }
    } else {
        for (int c = 0; c < n_pass; ++c) {
            const int cb = base_w + c * 16 * NS;
            scores(c, s, dp, st_off);
#pragma unroll
            for (int n = 0; n < 2 * NS; ++n) {
                float w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = n * 8 + 2 * t + (e & 1);
                    const float2 sq = sSt[st_off + col];   // the query's statistics
                    float p = ptx::ex2(fmaf(s[n][e], sl, -sq.x));
                    if (!seen(cb + col, rows[e >> 1])) p = 0.f;
                    w[e] = PASS == kColsV ? p : p * fmaf(dp[n][e], a.scale, -sq.y);
                }
                wa[n >> 1][(n & 1) * 2] = M::pack(w[0], w[1]);
                wa[n >> 1][(n & 1) * 2 + 1] = M::pack(w[2], w[3]);
            }
            emit(c, wa, PASS == kColsV ? y2 : y1, out, st_off);
        }
    }
}

template <typename T, int NS>
int launch_wide(const BwdDArgs &a, int64_t B, cudaStream_t stream) {
    constexpr int kStaged = 48 + 16 * NS;
    constexpr size_t smem = (size_t)2 * kStaged * 72 * sizeof(T) + kStaged * sizeof(float2);
    int rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_d_wide_kernel<T, kRows, NS>, smem, "bwd_d wide rows")) != MAT_OK) return rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_d_wide_kernel<T, kColsV, NS>, smem, "bwd_d wide dV")) != MAT_OK) return rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_d_wide_kernel<T, kColsK, NS>, smem, "bwd_d wide dK")) != MAT_OK) return rc;
    const dim3 grid((unsigned)a.HH, (unsigned)((a.S + kT - 1) / kT), (unsigned)B);
    bwd_d_wide_kernel<T, kRows, NS><<<grid, kThreads, smem, stream>>>(a);
    bwd_d_wide_kernel<T, kColsV, NS><<<grid, kThreads, smem, stream>>>(a);
    bwd_d_wide_kernel<T, kColsK, NS><<<grid, kThreads, smem, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "16-bit backward (wide heads) launch");
    note_kernel("bwd_d_mma");
    return MAT_OK;
}

template <typename T, int D, int NS>
int launch_d(const BwdDArgs &a, int64_t B, cudaStream_t stream) {
    constexpr int kStaged = NS > 0 ? 48 + 16 * NS : 2 * kT;
    constexpr size_t smem = (size_t)2 * kStaged * (D + 8) * sizeof(T) + kStaged * sizeof(float2);
    int rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_d_kernel<T, D, kRows, NS>, smem, "bwd_d rows")) != MAT_OK) return rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_d_kernel<T, D, kColsV, NS>, smem, "bwd_d dV")) != MAT_OK) return rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_d_kernel<T, D, kColsK, NS>, smem, "bwd_d dK")) != MAT_OK) return rc;
    const dim3 grid((unsigned)a.HH, (unsigned)((a.S + kT - 1) / kT), (unsigned)B);
    bwd_d_kernel<T, D, kRows, NS><<<grid, kThreads, smem, stream>>>(a);
    bwd_d_kernel<T, D, kColsV, NS><<<grid, kThreads, smem, stream>>>(a);
    bwd_d_kernel<T, D, kColsK, NS><<<grid, kThreads, smem, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "16-bit backward (other head widths) launch");
    note_kernel("bwd_d_mma");
    return MAT_OK;
}

// columns a warp's 16 rows meet: up to 160 the warp walks its own range in passes of 5 steps (one pass at 64 causal
// taps); wider windows walk the 64-column chunks.  MAT_BWD_D_WALK=chunks forces those (a measurement aid).
template <typename T, int D>
int launch_walk(const BwdDArgs &a, int64_t B, cudaStream_t stream) {
    const char *walk = std::getenv("MAT_BWD_D_WALK");
    const bool own = a.left + a.right + 16 <= 160 && !(walk && std::strcmp(walk, "chunks") == 0);
    return own ? launch_d<T, D, 5>(a, B, stream) : launch_d<T, D, 0>(a, B, stream);
}

template <typename T>
int launch_any_d(const BwdDArgs &a, int64_t B, int64_t D, cudaStream_t stream) {
    switch (D) {
        case 16: return launch_walk<T, 16>(a, B, stream);
        case 32: return launch_walk<T, 32>(a, B, stream);
        case 48: return launch_walk<T, 48>(a, B, stream);
        case 80: return launch_walk<T, 80>(a, B, stream);
        case 96: return launch_walk<T, 96>(a, B, stream);
        case 112: return launch_walk<T, 112>(a, B, stream);
        case 128: return launch_walk<T, 128>(a, B, stream);
    }
    return fail(MAT_ERR_UNSUPPORTED, "head width %lld has no instantiation of the warp-level backward", (long long)D);
}

}  // namespace

// 16-bit window patterns with a head width that is a multiple of 16 up to 128 other than 64, and windows of at most
// 144 taps with a head width of 192, 256, ... 512 (two passes of a warp's walk at most: the second pass adds to 16-bit
// values the first one wrote); lengths a multiple of the dilation, 16-byte aligned tensors.  MAT_BWD_KERNEL=warp
// keeps the one-warp-per-row kernels.
size_t bwd_d_mma_scratch_bytes(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t dil, int64_t left, int64_t right) {
    if (dtype != MAT_BF16 && dtype != MAT_F16) return 0;
    if (D % 8 || D < 8 || D > 512 || D == 64 || !(D > 128 || D % 16) || dil < 1 || S % dil != 0) return 0;
    const int64_t Sv1 = S / dil;
    if (std::min(left, Sv1) + std::min(right, Sv1) + 16 <= 160) return 0;
    return 3 * (((size_t)B * S * H * D * sizeof(float) + 255) & ~(size_t)255);
}

bool bwd_d_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t dil, int64_t left, int64_t right,
                        bool have_scratch) {
    if (dtype != MAT_BF16 && dtype != MAT_F16) return false;
    if (D % 8 || D < 8 || D == 64 || dil < 1 || S % dil != 0) return false;   // (rows stay 16-byte aligned)
    if (D > 128 || D % 16) {
        const int64_t Sv1 = S / dil;
        if (D > 512 || (std::min(left, Sv1) + std::min(right, Sv1) + 16 > 160 && !have_scratch)) return false;
    }
    const char *env = std::getenv("MAT_BWD_KERNEL");
    if (env && std::strcmp(env, "warp") == 0) return false;
    const int64_t Sv = S / dil;
    return Sv < (1LL << 30) && H * dil < (1LL << 31) && (Sv + kT - 1) / kT <= 65535 && B <= 65535;
}

int launch_bwd_d_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
                     float2 *stats, int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t left, int64_t right,
                     int64_t dil, float scale, float *scratch, cudaStream_t stream) {
    BwdDArgs a;
    a.scr_dq = a.scr_dk = a.scr_dv = nullptr;
    if (scratch && bwd_d_mma_scratch_bytes(B, S, H, D, dtype, dil, left, right)) {
        const size_t one = bwd_d_mma_scratch_bytes(B, S, H, D, dtype, dil, left, right) / 3 / sizeof(float);
        a.scr_dq = scratch; a.scr_dk = scratch + one; a.scr_dv = scratch + 2 * one;
    }
    a.q = q; a.k = k; a.v = v; a.go = dout;
    a.dq = dq; a.dk = dk; a.dv = dv;
    a.stats = stats;
    a.S = (int32_t)(S / dil);
    a.HH = (int32_t)(H * dil);
    a.left = (int32_t)std::min<int64_t>(left, a.S);
    a.right = (int32_t)std::min<int64_t>(right, a.S);
    a.scale = scale;
    a.D = (int32_t)D;
    // heads wider than 128 columns go 64 columns at a time.  A head of 128 does so where that makes its walk one pass
    // instead of two (81 to 144 columns: the rows pass then keeps S and dP); with 64 taps it gains nothing from it
    // (0.353 against 0.339 ms at 65536 tokens x 4 heads; MAT_BWD_D_WALK=sliced sends those there too, chunks or whole
    // keeps every window on the kernels above: measurement aids)
    const char *walk = std::getenv("MAT_BWD_D_WALK");
    const bool sliced128 = D == 128 && (walk ? std::strcmp(walk, "sliced") == 0 && a.left + a.right + 16 <= 144
                                             : a.left + a.right + 16 > 80 && a.left + a.right + 16 <= 144);
    if (D > 128 || D % 16 || sliced128)
    {
        // (a walk of 81 to 144 columns - the reference's default window of 64 either side - in one pass of 9 steps)
        if (a.left + a.right + 16 > 80 && a.left + a.right + 16 <= 144)
            return dtype == MAT_BF16 ? launch_wide<__nv_bfloat16, 9>(a, B, stream) : launch_wide<__half, 9>(a, B, stream);
        return dtype == MAT_BF16 ? launch_wide<__nv_bfloat16, 5>(a, B, stream) : launch_wide<__half, 5>(a, B, stream);
    }
    return dtype == MAT_BF16 ? launch_any_d<__nv_bfloat16>(a, B, D, stream) : launch_any_d<__half>(a, B, D, stream);
}

}  // namespace mat
