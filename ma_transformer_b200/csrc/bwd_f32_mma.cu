// fp32 backward of window attention on the tensor cores at fp32 accuracy.
//
// The reference computes its backward in fp32 (sparse_attention_backward_kernel,
// src/cuda/sparse_attention_kernel.cu:265-346; dense: 104-208), and fp32 is what an unmodified caller of
// its module trains in.  The warp-level kernels of backward.cu hold that accuracy but run one warp per row
// (55 ms at 65536 tokens x 8 heads x 64 taps); the 16-bit tensor-core kernels of bwd_mma.cu do not take
// fp32.  Here every product is three TF32 products of error-compensated halves, as in the forward
// (mma_window_f32.cu), with the same shape: 64-row tiles, four warps of 16 rows, the band walked in 64-column
// chunks through two cp.async buffers, scalar fragment loads from rows padded by four floats, and the
// accumulator layout of one product reused as the A operand of the next by ordering the 8 columns of a step
// as (0, 2, 4, 6, 1, 3, 5, 7).  An accumulating chain of MMAs ends with each chunk (the tensor core's fp32
// sums are not rounded to nearest); chunks are combined by ordinary additions.
//
// Three launches, no atomics, deterministic:
//   rows pass   one CTA per 64 queries, two sweeps over the keys they see: S = Q K^T and dP = dO V^T give the
//               row statistics (log2-sum-exp, delta * scale; left in the workspace), then dS and dQ = dS K.
//   dV pass     one CTA per 64 keys over the queries that see them: P^T from the statistics, dV = P^T dO.
//   dK pass     the same walk with dP^T = V dO^T: dS^T, dK = dS^T Q.
// (dK and dV in one launch would need both accumulators, their per-chunk partials and both operand tiles in
// registers at once.)
#include <algorithm>
#include <cstring>

#include "mat_common.cuh"
#include "ptx.cuh"

namespace mat {
namespace {

constexpr int kT = 64, kThreads = 128;

struct BwdFArgs {
    const float *q, *k, *v, *go;
    float *dq, *dk, *dv;
    float2 *stats;             // [B, HH, S]: (log2-sum-exp of the scaled scores, delta * scale)
    int32_t S, HH;             // rows and heads of the (possibly dilated) view
    int32_t left, right;
    float scale;
    int32_t D;                 // head width (read by the kernel for wide heads only)
};

__device__ __forceinline__ void cp_async16(void *dst, const void *src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(ptx::smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// x = hi + lo, hi = x rounded to TF32 (half a TF32 ulp added to the bit pattern, then cut), lo exact
__device__ __forceinline__ void split_tf32(uint32_t x, uint32_t &hi, uint32_t &lo) {
    hi = (x + 0x1000u) & 0xffffe000u;
    lo = __float_as_uint(__uint_as_float(x) - __uint_as_float(hi));
}
// d += a b at fp32 accuracy from the halves of a and the raw b
__device__ __forceinline__ void mma_3x(float (&d)[4], const uint32_t (&a_hi)[4], const uint32_t (&a_lo)[4], uint32_t b0,
                                       uint32_t b1) {
    uint32_t h0, l0, h1, l1;
    split_tf32(b0, h0, l0);
    split_tf32(b1, h1, l1);
    mma_tf32(d, a_lo, h0, h1);
    mma_tf32(d, a_hi, l0, l1);
    mma_tf32(d, a_hi, h0, h1);
}
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
// NT = 0: the band is walked in 64-column chunks shared by the four warps (two buffers).  NT > 0, for narrow windows:
// every warp walks the columns from a base of its own, the first column its first row meets, in passes of NT 8-column
// tiles, so that no tile is without a visible column but the last of the walk (10 tiles instead of 16 at 64 causal
// taps); the CTA stages the 48 + 8 NT rows the four warps' passes span, in one buffer.
template <int D, int PASS, int NT>
__global__ void __launch_bounds__(kThreads)
bwd_f32_kernel(const BwdFArgs a) {
    constexpr int LD = D + 4, KS = D / 8;
    constexpr bool COLS = PASS != kRows, DIAG = NT > 0;
    constexpr int TILES = DIAG ? NT : 8;                       // 8-column tiles a warp takes per chunk or pass
    constexpr int kRowsStaged = DIAG ? 48 + 8 * NT : 2 * kT;   // rows of each operand in shared memory
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float *sY1 = reinterpret_cast<float *>(smem_raw);   // rows pass K, cols passes Q
    float *sY2 = sY1 + kRowsStaged * LD;                // rows pass V, cols passes dO
    float2 *sSt = reinterpret_cast<float2 *>(sY2 + kRowsStaged * LD);   // cols passes: statistics of the staged queries

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int hh = blockIdx.x, b = blockIdx.z, r0 = blockIdx.y * kT;
    const int back = COLS ? a.right : a.left, fwd = COLS ? a.left : a.right;   // row r sees columns r - back .. r + fwd
    const int col_lo = max(0, r0 - back);
    const int col_hi = min(a.S - 1, min(r0 + kT, a.S) - 1 + fwd);
    const int base_w = max(col_lo, r0 + 16 * warp - back);   // (NT > 0) the warp's first column
    int n_chunks = 0;                                        // chunks, or passes of the warp with the longest walk
    if (col_hi >= col_lo) {
        if constexpr (DIAG) {
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) {
                const int cols_w = min(col_hi, r0 + 16 * w + 15 + fwd) - max(col_lo, r0 + 16 * w - back) + 1;
                n_chunks = max(n_chunks, (cols_w + 8 * NT - 1) / (8 * NT));
            }
            n_chunks = min(n_chunks, (col_hi - col_lo) / (8 * NT) + 1);
        } else {
            n_chunks = (col_hi - col_lo) / kT + 1;
        }
    }
    const int64_t tok = (int64_t)a.HH * D;
    const int64_t head = ((int64_t)b * a.S * a.HH + hh) * D;
    const float *x1 = (COLS ? a.k : a.q) + head, *x2 = (COLS ? a.v : a.go) + head;
    const float *y1 = (COLS ? a.q : a.k) + head, *y2 = (COLS ? a.go : a.v) + head;
    const float2 *st_in = a.stats + ((int64_t)b * a.HH + hh) * a.S;

    // chunk c into buffer buf (NT = 0), or the rows of pass c (warp 0's base is col_lo) into the one buffer
    auto load_chunk = [&](int c, int buf) {
        constexpr int kPieces = D / 4;
        constexpr int kStage = DIAG ? kRowsStaged : kT;
        const int base = col_lo + c * (DIAG ? 8 * NT : kT);
        for (int i = threadIdx.x; i < kStage * kPieces; i += kThreads) {
            const int r = i / kPieces, pc = i % kPieces;
            const int j = base + r;
            const bool in = j < a.S;   // rows past the end are zero-filled
            const int64_t src = (int64_t)(in ? j : 0) * tok + pc * 4;
            cp_async16(sY1 + (buf * kT + r) * LD + pc * 4, y1 + src, in ? 16 : 0);
            cp_async16(sY2 + (buf * kT + r) * LD + pc * 4, y2 + src, in ? 16 : 0);
        }
        static_assert(kStage <= kThreads, "one thread per staged row's statistics");
        if (COLS && threadIdx.x < kStage) {
            const int j = base + threadIdx.x;
            sSt[buf * kT + threadIdx.x] = j < a.S ? st_in[j] : make_float2(0.f, 0.f);
        }
    };
    if (!DIAG && n_chunks > 0) load_chunk(0, 0);
    cp_async_commit();

    // the warp's 16 tile rows as A fragments (rows g and g + 8, columns t and t + 4 of each 8)
    const int row_a = r0 + 16 * warp + g, row_b = row_a + 8;
    uint32_t xf1[KS][4], xf2[PASS == kColsV ? 1 : KS][4];
    {
        const float *pa = x1 + (int64_t)row_a * tok, *pb = x1 + (int64_t)row_b * tok;
        const float *qa = x2 + (int64_t)row_a * tok, *qb = x2 + (int64_t)row_b * tok;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 8 + t;
            xf1[ks][0] = row_a < a.S ? __float_as_uint(pa[c]) : 0u;
            xf1[ks][1] = row_b < a.S ? __float_as_uint(pb[c]) : 0u;
            xf1[ks][2] = row_a < a.S ? __float_as_uint(pa[c + 4]) : 0u;
            xf1[ks][3] = row_b < a.S ? __float_as_uint(pb[c + 4]) : 0u;
            if constexpr (PASS != kColsV) {
                xf2[ks][0] = row_a < a.S ? __float_as_uint(qa[c]) : 0u;
                xf2[ks][1] = row_b < a.S ? __float_as_uint(qb[c]) : 0u;
                xf2[ks][2] = row_a < a.S ? __float_as_uint(qa[c + 4]) : 0u;
                xf2[ks][3] = row_b < a.S ? __float_as_uint(qb[c + 4]) : 0u;
            }
        }
    }
    const float sl = a.scale * 1.4426950408889634f;
    const int rows[2] = {row_a, row_b};
    // column j of row r counts iff -back <= j - r <= fwd and j exists
    auto seen = [&](int j, int r) { return (unsigned)(j - r + back) <= (unsigned)(back + fwd) && j < a.S; };

    float acc[KS][4];   // dQ, dV or dK of the warp's rows
#pragma unroll
    for (int n = 0; n < KS; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f}, dr[2] = {0.f, 0.f}, lse[2] = {0.f, 0.f}, dsc[2] = {0.f, 0.f};

    // the tile's product with the chunk's rows: out[n] (16 x 8) = X (16 x D) . Y[n*8 .. n*8+7]^T
    auto product = [&](float (&out)[4], const uint32_t (&xf)[KS][4], const uint32_t *y, int n) {
        out[0] = out[1] = out[2] = out[3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t x_hi[4], x_lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_tf32(xf[ks][e], x_hi[e], x_lo[e]);
            const uint32_t *yr = y + (n * 8 + g) * LD + ks * 8 + t;   // B: (k = dim, n = column)
            mma_3x(out, x_hi, x_lo, yr[0], yr[4]);
        }
    };
    // part[d] += W (16 x 8, held as an accumulator tile: columns 2t, 2t+1 of rows g, g+8) . Y[n*8 .. n*8+7] (8 x D);
    // the step's columns are taken in the order the accumulator holds them, so W is its own A fragment
    auto accumulate = [&](float (&part)[KS][4], const float (&w)[4], const uint32_t *y, int n) {
        const uint32_t wa[4] = {__float_as_uint(w[0]), __float_as_uint(w[2]), __float_as_uint(w[1]), __float_as_uint(w[3])};
        uint32_t w_hi[4], w_lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) split_tf32(wa[e], w_hi[e], w_lo[e]);
        const uint32_t *yr = y + (n * 8 + 2 * t) * LD + g;   // B: (k = column 2t / 2t + 1, n = dim)
#pragma unroll
        for (int d = 0; d < KS; ++d) mma_3x(part[d], w_hi, w_lo, yr[d * 8], yr[LD + d * 8]);
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
        const int cb = DIAG ? base_w + c * 8 * NT : col_lo + c * kT;       // the first column of the warp's tiles
        const int st_off = DIAG ? cb - (col_lo + c * 8 * NT) : buf * kT;   // its row in shared memory
        const uint32_t *cy1 = reinterpret_cast<const uint32_t *>(sY1 + st_off * LD);
        const uint32_t *cy2 = reinterpret_cast<const uint32_t *>(sY2 + st_off * LD);

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
        float part[KS][4];
#pragma unroll
        for (int d = 0; d < KS; ++d) part[d][0] = part[d][1] = part[d][2] = part[d][3] = 0.f;

        bool sweep_one = false;
        if constexpr (PASS == kRows) sweep_one = n < n_chunks;
        if (sweep_one) {
          if constexpr (PASS == kRows) {
            // ---- sweep one: running maximum, sum of exponentials, sum of exponentials x dP ----
            float s[TILES][4];
            float cm[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < TILES; ++nt) {
                product(s[nt], xf1, cy1, nt);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
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
            for (int nt = 0; nt < TILES; ++nt) {
                float dp[4];
                product(dp, xf2, cy2, nt);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float ex = ptx::ex2(fmaf(s[nt][e], sl, -msl[e >> 1]));
                    sum[e >> 1] += ex;
                    dr[e >> 1] = fmaf(ex, dp[e], dr[e >> 1]);
                }
            }
          }
        } else {
            // ---- rows pass, sweep two: dS, dQ += dS K.  cols passes: P^T (and dS^T), dV += P^T dO / dK += dS^T Q ----
#pragma unroll
            for (int nt = 0; nt < TILES; ++nt) {
                float s[4], w[4];
                product(s, xf1, cy1, nt);
                float dp[4] = {0.f, 0.f, 0.f, 0.f};
                if constexpr (PASS != kColsV) product(dp, xf2, cy2, nt);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = nt * 8 + 2 * t + (e & 1);
                    // the query's statistics: the row's own (rows pass) or the column's (cols passes)
                    const float2 sq = COLS ? sSt[st_off + col] : make_float2(lse[e >> 1], dsc[e >> 1]);
                    float p = ptx::ex2(fmaf(s[e], sl, -sq.x));
                    if (!seen(cb + col, rows[e >> 1])) p = 0.f;
                    w[e] = PASS == kColsV ? p : p * fmaf(dp[e], a.scale, -sq.y);
                }
                accumulate(part, w, PASS == kColsV ? cy2 : cy1, nt);
            }
#pragma unroll
            for (int d = 0; d < KS; ++d)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[d][e] += part[d][e];
        }
        if (!DIAG) __syncthreads();   // the buffer is free for the chunk after the next
    }
    if (PASS == kRows && n_chunks == 0 && t == 0) {   // rows that see no key
#pragma unroll
        for (int i = 0; i < 2; ++i)
            if (rows[i] < a.S) a.stats[((int64_t)b * a.HH + hh) * a.S + rows[i]] = make_float2(0.f, 0.f);
    }
    float *out = (PASS == kRows ? a.dq : PASS == kColsV ? a.dv : a.dk) + head;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (rows[i] < a.S) {
            float *dst = out + (int64_t)rows[i] * tok + 2 * t;
#pragma unroll
            for (int d = 0; d < KS; ++d) *reinterpret_cast<float2 *>(dst + d * 8) = make_float2(acc[d][2 * i], acc[d][2 * i + 1]);
        }
    }
}

// Wide heads (D = 128, 192, ... 512: the reference's layer passes one head of width model_dim,
// src/layers/sparse_attention.py:71-78).  The same three passes and the same per-warp column ranges (passes of ten
// 8-column tiles from the warp's own first column), with the head dimension taken 64 columns at a time: the two
// score-shaped products of a pass (S and dP, or their transposes) accumulate in registers over the slices of their
// operands, which are staged one slice at a time; the weights (P^T or dS) are formed once, and every 64-column slice
// of the output is their product with one more staged slice, written out - added to what an earlier pass of the
// same rows wrote, which needs no atomics: a row of dQ, dK or dV belongs to one thread pair of one CTA.  Registers
// hold one pass's two score tiles and one slice's fragments whatever D is.  When the walk is a single pass (windows
// of at most 64 taps) the rows pass keeps S and dP from its first sweep instead of recomputing them.
template <int PASS, int NT>
__global__ void __launch_bounds__(kThreads, NT <= 10 ? 3 : 2)
bwd_f32_wide_kernel(const BwdFArgs a) {
    constexpr int LD = 64 + 4, KS = 8;
    constexpr int kStage = 48 + 8 * NT;
    constexpr bool COLS = PASS != kRows;
    constexpr bool kTwo = PASS != kColsV;   // two score-shaped products (S and dP); the dV pass needs only S^T
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float *sY1 = reinterpret_cast<float *>(smem_raw);   // a slice of: rows pass K, cols passes Q
    float *sY2 = sY1 + kStage * LD;                     // a slice of: rows pass V, cols passes dO
    float2 *sSt = reinterpret_cast<float2 *>(sY2 + kStage * LD);   // cols passes: statistics of the staged queries

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
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
            n_pass = max(n_pass, (cols_w + 8 * NT - 1) / (8 * NT));
        }
        n_pass = min(n_pass, (col_hi - col_lo) / (8 * NT) + 1);
    }
    const int64_t tok = (int64_t)a.HH * D;
    const int64_t head = ((int64_t)b * a.S * a.HH + hh) * D;
    const float *x1 = (COLS ? a.k : a.q) + head, *x2 = (COLS ? a.v : a.go) + head;
    const float *y1 = (COLS ? a.q : a.k) + head, *y2 = (COLS ? a.go : a.v) + head;
    const float2 *st_in = a.stats + ((int64_t)b * a.HH + hh) * a.S;
    const int row_a = r0 + 16 * warp + g, row_b = row_a + 8;
    const int rows[2] = {row_a, row_b};
    const float sl = a.scale * 1.4426950408889634f;
    auto seen = [&](int j, int r) { return (unsigned)(j - r + back) <= (unsigned)(back + fwd) && j < a.S; };

    // 64 columns (slice) of the kStage rows from `first` on, of one operand, into one buffer; rows past the end are zeros
    auto stage = [&](float *dst, const float *src, int first, int slice) {
        for (int x = threadIdx.x; x < kStage * 16; x += kThreads) {
            const int r = x >> 4, pc = x & 15;
            const int j = first + r;
            const bool in = j < a.S && slice * 64 + pc * 4 < D;
            cp_async16(dst + r * LD + pc * 4, src + (int64_t)(in ? j : 0) * tok + slice * 64 + pc * 4, in ? 16 : 0);
        }
    };
    // the warp's 16 rows of a slice as A fragments (rows g and g + 8, columns t and t + 4 of each 8)
    auto load_x = [&](uint32_t (&xf)[KS][4], const float *x, int slice) {
        const float *pa = x + (int64_t)row_a * tok + slice * 64, *pb = x + (int64_t)row_b * tok + slice * 64;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 8 + t;
            const int col = slice * 64 + c;   // (D is a multiple of 4: each half of an 8-column step is inside D or beyond it)
            xf[ks][0] = row_a < a.S && col < D ? __float_as_uint(pa[c]) : 0u;
            xf[ks][1] = row_b < a.S && col < D ? __float_as_uint(pb[c]) : 0u;
            xf[ks][2] = row_a < a.S && col + 4 < D ? __float_as_uint(pa[c + 4]) : 0u;
            xf[ks][3] = row_b < a.S && col + 4 < D ? __float_as_uint(pb[c + 4]) : 0u;
        }
    };
    // one 8-column step of those fragments
    auto load_x8 = [&](uint32_t (&xf)[4], const float *x, int slice, int ks) {
        const float *pa = x + (int64_t)row_a * tok + slice * 64 + ks * 8 + t, *pb = x + (int64_t)row_b * tok + slice * 64 + ks * 8 + t;
        const int col = slice * 64 + ks * 8 + t;
        xf[0] = row_a < a.S && col < D ? __float_as_uint(pa[0]) : 0u;
        xf[1] = row_b < a.S && col < D ? __float_as_uint(pb[0]) : 0u;
        xf[2] = row_a < a.S && col + 4 < D ? __float_as_uint(pa[4]) : 0u;
        xf[3] = row_b < a.S && col + 4 < D ? __float_as_uint(pb[4]) : 0u;
    };
    // pass c: s[nt] (and dp[nt]) = the warp's rows against its NT tiles of columns, summed over the slices
    auto scores = [&](int c, float (&s)[NT][4], float (&dp)[NT][4], int st_off) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = dp[nt][e] = 0.f;
        const int first = col_lo + c * 8 * NT;
        for (int slice = 0; slice < n_slices; ++slice) {
            // the rows' fragments: the whole slice in registers, or (the rows pass with its two score tiles: no room)
            // one 8-column step at a time, the next step's loads in flight under the current step's products
            constexpr bool kStream = PASS == kRows;
            uint32_t xf1[kStream ? 1 : KS][4], xf2[kTwo && !kStream ? KS : 1][4];
            uint32_t xa[4], xb[4];
            if constexpr (kStream) {
                load_x8(xa, x1, slice, 0);
                load_x8(xb, x2, slice, 0);
            } else {
                load_x(xf1, x1, slice);
                if constexpr (kTwo) load_x(xf2, x2, slice);
            }
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
            const uint32_t *cy1 = reinterpret_cast<const uint32_t *>(sY1 + st_off * LD);
            const uint32_t *cy2 = reinterpret_cast<const uint32_t *>(sY2 + st_off * LD);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t h1[4], l1[4], h2[4], l2[4];
                uint32_t na[4], nb[4];
                if constexpr (kStream) {
                    if (ks + 1 < KS) {
                        load_x8(na, x1, slice, ks + 1);
                        load_x8(nb, x2, slice, ks + 1);
                    }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    split_tf32(kStream ? xa[e] : xf1[ks][e], h1[e], l1[e]);
                    if constexpr (kTwo) split_tf32(kStream ? xb[e] : xf2[ks][e], h2[e], l2[e]);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int off = (nt * 8 + g) * LD + ks * 8 + t;   // B: (k = dim, n = column)
                    mma_3x(s[nt], h1, l1, cy1[off], cy1[off + 4]);
                    if constexpr (kTwo) mma_3x(dp[nt], h2, l2, cy2[off], cy2[off + 4]);
                }
                if constexpr (kStream) {
                    if (ks + 1 < KS) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) { xa[e] = na[e]; xb[e] = nb[e]; }
                    }
                }
            }
        }
    };
    // out rows (+)= W (the pass's weights, held as accumulator tiles) . Y, 64 columns of Y at a time
    auto emit = [&](int c, const float (&w)[NT][4], const float *y, float *out, int st_off) {
        const int first = col_lo + c * 8 * NT;
        for (int slice = 0; slice < n_slices; ++slice) {
            __syncthreads();
            stage(sY1, y, first, slice);
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
            const uint32_t *cy = reinterpret_cast<const uint32_t *>(sY1 + st_off * LD);
            float part[KS][4];
#pragma unroll
            for (int d = 0; d < KS; ++d) part[d][0] = part[d][1] = part[d][2] = part[d][3] = 0.f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                // the tile's columns in the order the accumulator holds them, so W is its own A fragment
                const uint32_t wa[4] = {__float_as_uint(w[nt][0]), __float_as_uint(w[nt][2]), __float_as_uint(w[nt][1]),
                                        __float_as_uint(w[nt][3])};
                uint32_t w_hi[4], w_lo[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) split_tf32(wa[e], w_hi[e], w_lo[e]);
                const uint32_t *yr = cy + (nt * 8 + 2 * t) * LD + g;   // B: (k = column 2t / 2t + 1, n = dim)
#pragma unroll
                for (int d = 0; d < KS; ++d) mma_3x(part[d], w_hi, w_lo, yr[d * 8], yr[LD + d * 8]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (rows[i] >= a.S) continue;
                float *dst = out + (int64_t)rows[i] * tok + slice * 64 + 2 * t;
#pragma unroll
                for (int d = 0; d < KS; ++d) {
                    if (slice * 64 + d * 8 + 2 * t >= D) continue;
                    float2 val = make_float2(part[d][2 * i], part[d][2 * i + 1]);
                    if (c > 0) {   // an earlier pass of these rows wrote here
                        const float2 old = *reinterpret_cast<const float2 *>(dst + d * 8);
                        val.x += old.x;
                        val.y += old.y;
                    }
                    *reinterpret_cast<float2 *>(dst + d * 8) = val;
                }
            }
        }
    };
    float *out = (PASS == kRows ? a.dq : PASS == kColsV ? a.dv : a.dk) + head;
    if (n_pass == 0) {   // rows that meet no column: zero gradient (and zero statistics)
        for (int i = 0; i < 2; ++i) {
            if (rows[i] >= a.S) continue;
            for (int c = 2 * t; c < D; c += 8) *reinterpret_cast<float2 *>(out + (int64_t)rows[i] * tok + c) = make_float2(0.f, 0.f);
            if (PASS == kRows && t == 0) a.stats[((int64_t)b * a.HH + hh) * a.S + rows[i]] = make_float2(0.f, 0.f);
        }
        return;
    }

    float s[NT][4], dp[NT][4];
    if constexpr (PASS == kRows) {
        float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f}, dr[2] = {0.f, 0.f}, lse[2], dsc[2];
        // sweep one: running maximum, sum of exponentials, sum of exponentials x dP
        for (int c = 0; c < n_pass; ++c) {
            const int cb = base_w + c * 8 * NT;
            scores(c, s, dp, base_w - col_lo);
            float cm[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (!seen(cb + nt * 8 + 2 * t + (e & 1), rows[e >> 1])) s[nt][e] = -INFINITY;
                    cm[e >> 1] = fmaxf(cm[e >> 1], s[nt][e]);
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
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float ex = ptx::ex2(fmaf(s[nt][e], sl, -msl[e >> 1]));
                    sum[e >> 1] += ex;
                    dr[e >> 1] = fmaf(ex, dp[nt][e], dr[e >> 1]);
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
            const int cb = base_w + c * 8 * NT;
            if (n_pass > 1) scores(c, s, dp, base_w - col_lo);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float p = ptx::ex2(fmaf(s[nt][e], sl, -lse[e >> 1]));
                    if (!seen(cb + nt * 8 + 2 * t + (e & 1), rows[e >> 1])) p = 0.f;
                    s[nt][e] = p * fmaf(dp[nt][e], a.scale, -dsc[e >> 1]);
                }
            emit(c, s, y1, out, base_w - col_lo);
        }
    } else {
        for (int c = 0; c < n_pass; ++c) {
            const int cb = base_w + c * 8 * NT, st_off = base_w - col_lo;
            scores(c, s, dp, st_off);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = nt * 8 + 2 * t + (e & 1);
                    const float2 sq = sSt[st_off + col];   // the query's statistics
                    float p = ptx::ex2(fmaf(s[nt][e], sl, -sq.x));
                    if (!seen(cb + col, rows[e >> 1])) p = 0.f;
                    s[nt][e] = PASS == kColsV ? p : p * fmaf(dp[nt][e], a.scale, -sq.y);
                }
            emit(c, s, PASS == kColsV ? y2 : y1, out, st_off);
        }
    }
}

template <int NT>
int launch_wide(const BwdFArgs &a, int64_t B, cudaStream_t stream) {
    constexpr int kStaged = 48 + 8 * NT;
    constexpr size_t smem = (size_t)2 * kStaged * 68 * sizeof(float) + kStaged * sizeof(float2);
    int rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_f32_wide_kernel<kRows, NT>, smem, "bwd_f32 wide rows")) != MAT_OK) return rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_f32_wide_kernel<kColsV, NT>, smem, "bwd_f32 wide dV")) != MAT_OK) return rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_f32_wide_kernel<kColsK, NT>, smem, "bwd_f32 wide dK")) != MAT_OK) return rc;
    const dim3 grid((unsigned)a.HH, (unsigned)((a.S + kT - 1) / kT), (unsigned)B);
    bwd_f32_wide_kernel<kRows, NT><<<grid, kThreads, smem, stream>>>(a);
    bwd_f32_wide_kernel<kColsV, NT><<<grid, kThreads, smem, stream>>>(a);
    bwd_f32_wide_kernel<kColsK, NT><<<grid, kThreads, smem, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "fp32 tensor-core backward (wide heads) launch");
    note_kernel("bwd_f32_mma");
    return MAT_OK;
}

template <int D, int NT>
int launch_f(const BwdFArgs &a, int64_t B, cudaStream_t stream) {
    constexpr int kStaged = NT > 0 ? 48 + 8 * NT : 2 * kT;
    constexpr size_t smem = (size_t)2 * kStaged * (D + 4) * sizeof(float) + kStaged * sizeof(float2);
    int rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_f32_kernel<D, kRows, NT>, smem, "bwd_f32 rows")) != MAT_OK) return rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_f32_kernel<D, kColsV, NT>, smem, "bwd_f32 dV")) != MAT_OK) return rc;
    if ((rc = ensure_dynamic_smem((const void *)bwd_f32_kernel<D, kColsK, NT>, smem, "bwd_f32 dK")) != MAT_OK) return rc;
    const dim3 grid((unsigned)a.HH, (unsigned)((a.S + kT - 1) / kT), (unsigned)B);
    bwd_f32_kernel<D, kRows, NT><<<grid, kThreads, smem, stream>>>(a);
    bwd_f32_kernel<D, kColsV, NT><<<grid, kThreads, smem, stream>>>(a);
    bwd_f32_kernel<D, kColsK, NT><<<grid, kThreads, smem, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "fp32 tensor-core backward launch");
    note_kernel("bwd_f32_mma");
    return MAT_OK;
}

}  // namespace

// fp32 window patterns with a head width that is a multiple of 4 up to 512, lengths a multiple of the dilation,
// 16-byte aligned tensors.
// MAT_BWD_KERNEL=warp keeps the warp-level kernels.
bool bwd_f32_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t dil) {
    const bool wide_head = D >= 4 && D <= 512 && D % 4 == 0;   // 64 columns at a time (rows stay 16-byte aligned)
    const bool narrow_head = D == 16 || D == 32 || D == 48 || D == 64;
    if (dtype != MAT_F32 || (!narrow_head && !wide_head) || dil < 1 || S % dil != 0) return false;
    const char *env = std::getenv("MAT_BWD_KERNEL");
    if (env && std::strcmp(env, "warp") == 0) return false;
    const int64_t Sv = S / dil;
    return Sv < (1LL << 30) && H * dil < (1LL << 31) && (Sv + kT - 1) / kT <= 65535 && B <= 65535;
}

int launch_bwd_f32_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
                       float2 *stats, int64_t B, int64_t S, int64_t H, int64_t D, int64_t left, int64_t right,
                       int64_t dil, float scale, cudaStream_t stream) {
    BwdFArgs a;
    a.q = (const float *)q; a.k = (const float *)k; a.v = (const float *)v; a.go = (const float *)dout;
    a.dq = (float *)dq; a.dk = (float *)dk; a.dv = (float *)dv;
    a.stats = stats;
    a.S = (int32_t)(S / dil);
    a.HH = (int32_t)(H * dil);
    a.left = (int32_t)std::min<int64_t>(left, a.S);
    a.right = (int32_t)std::min<int64_t>(right, a.S);
    a.scale = scale;
    a.D = (int32_t)D;
    // (a walk of 81 to 144 columns - the reference's default window of 64 either side - in one pass of 18 tiles)
    const bool one18 = a.left + a.right + 16 > 80 && a.left + a.right + 16 <= 144;
    if (D != 16 && D != 32 && D != 48 && D != 64) return one18 ? launch_wide<18>(a, B, stream) : launch_wide<10>(a, B, stream);
    const char *walk = std::getenv("MAT_BWD_F32_WALK");
    // (a 64-wide head whose walk is one pass takes that kernel too: its rows pass keeps S and dP instead of
    // recomputing them; MAT_BWD_F32_WALK=recompute or chunks keeps it on the kernels below)
    if (D == 64 && a.left + a.right + 16 <= 80 && !walk) return launch_wide<10>(a, B, stream);
    if (D == 64 && one18 && !walk) return launch_wide<18>(a, B, stream);
    // columns a warp's 16 rows meet: up to 160 the warp walks its own range in passes of 10 tiles (one pass at 64
    // causal taps); wider windows walk the 64-column chunks.  MAT_BWD_F32_WALK=chunks forces those (a measurement aid).
    const bool own = a.left + a.right + 16 <= 160 && !(walk && std::strcmp(walk, "chunks") == 0);
    switch (D) {
    case 16: return own ? launch_f<16, 10>(a, B, stream) : launch_f<16, 0>(a, B, stream);
    case 32: return own ? launch_f<32, 10>(a, B, stream) : launch_f<32, 0>(a, B, stream);
    case 48: return own ? launch_f<48, 10>(a, B, stream) : launch_f<48, 0>(a, B, stream);
    default: return own ? launch_f<64, 10>(a, B, stream) : launch_f<64, 0>(a, B, stream);
    }
}

}  // namespace mat
