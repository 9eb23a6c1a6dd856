// Tensor-core backward of window attention for bf16 / fp16 with head width 64: causal,
// two-sided, dilated (through a view) and dense (the window that covers the sequence).
// Windows with left + right <= 128 taps keep their whole band in shared memory
// (bwd_window_mma_kernel); wider ones stream it in 64-column chunks (bwd_stream_mma_kernel,
// described above that kernel).
//
// Replaces sparse_attention_backward_kernel (src/cuda/sparse_attention_kernel.cu:265-346),
// which runs one thread per query row and scatters dK / dV with fp32 atomicAdd (:322, :343).
// Nothing here is atomic; the result is deterministic.  Two launches of one kernel template:
//
//   rows pass (COLS = false)  one CTA per (batch, head, 64 queries): S = Q K^T on the band of
//       keys the tile can see, softmax statistics, dP = dO V^T, delta_i = sum_j P_ij dP_ij,
//       dS = P (dP - delta) scale, dQ = dS K.  Leaves (log2-sum-exp, delta scale) per row in the
//       workspace.
//   cols pass (COLS = true)   one CTA per (batch, head, 64 keys): the same band walk with the
//       roles mirrored (rows are keys, the band holds the queries that attend to them):
//       P^T from the stored statistics, dV = P^T dO, dK = dS^T Q.
//
// Both passes share the structure "16 rows per warp against a band of at most 80 columns"
// (144 for windows of more than 64 taps, where the rows pass keeps only the scores in registers
// and recomputes dP):
// one thread stages the tile's rows and the band by TMA (64-row boxes, 128-byte swizzle, zeros
// outside the sequence; the wait for them is bounded), the row operands are A fragments held in
// registers, the band operands stay in shared memory (every ldmatrix conflict-free) and feed mma.sync.m16n8k16 as B fragments, plain for the score-shaped
// products and transposed for the output-shaped ones.  A dilated window over [B,S,H,64] is a
// plain window over the same bytes viewed as [B, S/dil, dil*H, 64], so the kernel never sees
// a dilation.
#include "mat_common.cuh"
#include "ptx.cuh"

#include <math.h>
#include <mutex>
#include <stdlib.h>
#include <string.h>

namespace mat {
namespace {

constexpr int kTile = 64;       // rows per CTA (4 warps x 16)
constexpr int kThreads = 128;
// NP = 16-column groups one warp's rows can reach: 5 (16 + 64 = 80 columns) for windows of at most 64 taps
// between the two sides, 9 (16 + 128 = 144 columns) for up to 128 (the reference's default +-64)
constexpr int band_rows_max(int NP) { return 48 + 16 * NP; }
constexpr int smem_bytes(int NP) { return 2 * 8192 + band_rows_max(NP) * (2 * 128 + (int)sizeof(float2)) + 16; }

struct BwdArgs {
    const void *q, *k, *v, *go;
    void *dq, *dk, *dv;
    float2 *stats;            // per (batch, head, row), row fastest: (log2-sum-exp of the scaled scores, delta * scale)
    int64_t B, S, HH;         // sequence length and head count of the (possibly dilated) view
    int left, right;
    float scale;
    int prefetch_ahead;       // resident-band kernels: L2-prefetch the tile this many CTAs ahead (0 = off)
    // Block layouts (streamed kernel only): a 64-row tile walks the 64-column chunks of its layout row's blocks
    // (rows pass: query block -> key blocks; cols pass: the transposed layout, key block -> query blocks)
    int block_mode = 0, causal = 0;
    int per_blk = 1;          // 64-column chunks per layout block
    const int32_t *rowptr = nullptr, *colidx = nullptr, *t_rowptr = nullptr, *t_colidx = nullptr;
    // Longformer (streamed kernel only; at most 64 global positions, whose Q, K, V, dO rows the launcher gathers
    // into [B, n_global, HH, 64] tensors).  lf_mode 1, every tile: the window band plus one chunk that holds the
    // gathered rows (the global keys in the rows pass, the global queries in the cols pass), less the positions
    // the window already holds.  lf_mode 2, one tile per (batch, head): the gathered rows themselves against
    // every chunk of the sequence (a global query attends every key, a global key is attended by every query);
    // its results overwrite what the lf_mode 1 passes left for those positions.
    int lf_mode = 0, n_global = 0;
    const int64_t *gidx = nullptr;
    float2 *stats_g = nullptr;   // [B, HH, 64]: the statistics of the global rows in gathered order
};

// the gathered counterparts of the four tensors
struct LfMaps {
    CUtensorMap q, k, v, go;
};

__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}
// a kernel whose bounded wait for its tile copies ran out leaves 1 here and returns (read by mat_device_status)
__device__ int g_bwd_status = 0;

__device__ __forceinline__ float quad_max(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    return fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x + __shfl_xor_sync(0xffffffffu, x, 2);
}

// a warp's 16 x 64 fp32 accumulator tile -> its own 16 rows of a swizzled shared tile -> global, 16 bytes per lane
template <typename T>
__device__ __forceinline__ void store_tile(uint8_t *smem, uint32_t tile_off, const float (&o)[8][4], T *head,
                                           int64_t row0, int64_t S, int64_t stride, int warp, int lane,
                                           const int32_t *scatter = nullptr) {
    const int g = lane >> 2, t = lane & 3;
    __syncwarp();
#pragma unroll
    for (int dt = 0; dt < 8; ++dt) {
        *(uint32_t *)(smem + tile_off + swz(16 * warp + g, dt) + 4 * t) = ptx::Mma<T>::pack(o[dt][0], o[dt][1]);
        *(uint32_t *)(smem + tile_off + swz(16 * warp + g + 8, dt) + 4 * t) = ptx::Mma<T>::pack(o[dt][2], o[dt][3]);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = lane + 32 * i, row = idx >> 3, chunk = idx & 7;
        // scatter: row i of the tile belongs at sequence position scatter[i] (negative: no such row)
        const int64_t gr = scatter ? (int64_t)scatter[16 * warp + row] : row0 + 16 * warp + row;
        if (gr >= 0 && gr < S) {
            const uint4 val = *(const uint4 *)(smem + tile_off + swz(16 * warp + row, chunk));
            *(uint4 *)(head + gr * stride + chunk * 8) = val;
        }
    }
}

template <typename T, bool COLS, int NP>
__global__ void __launch_bounds__(kThreads, NP == 5 ? 4 : 3)
bwd_window_mma_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                      const __grid_constant__ CUtensorMap mv, const __grid_constant__ CUtensorMap mgo, BwdArgs a) {
    constexpr int kPairs = NP;
    extern __shared__ __align__(1024) uint8_t smem[];
    using M = ptx::Mma<T>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int64_t r0 = (int64_t)blockIdx.y * kTile;   // heads vary fastest over the grid: neighbouring CTAs read neighbouring bytes
    const int64_t h = blockIdx.x, b = blockIdx.z;
    const int W = a.left + a.right;
    const int back = COLS ? a.right : a.left;       // how far the band starts before the tile's first row
    const int64_t c0 = r0 - back;                   // global index of band row 0
    const int np = min(kPairs, (15 + W) / 16 + 1);  // 16-column groups a warp walks
    const int64_t stride = a.HH * 64;
    const int64_t head_off = (b * a.S * a.HH + h) * 64;
    const CUtensorMap *x1 = COLS ? &mk : &mq, *x2 = COLS ? &mv : &mgo;   // row operands: one A fragment set each
    const CUtensorMap *y1 = COLS ? &mq : &mk, *y2 = COLS ? &mgo : &mv;   // band operands
    constexpr uint32_t oX1 = 0, oX2 = 8192, oY1 = 16384, oY2 = oY1 + band_rows_max(NP) * 128,
                       oSt = oY2 + band_rows_max(NP) * 128, oBar = oSt + band_rows_max(NP) * 8;
    const uint32_t sbase = ptx::smem_u32(smem);
    float2 *sst = (float2 *)(smem + oSt);
    uint64_t *bar = (uint64_t *)(smem + oBar);

    // One thread stages everything by TMA: 64-row boxes, 128-byte swizzle (chunk ^ (row & 7), the pattern swz()
    // addresses), rows outside [0, S) arrive as zeros.  Band boxes beyond the groups the warps walk are skipped.
    const int band_rows = 48 + 16 * np;
    const int boxes = (band_rows + 63) / 64;
    if (tid == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_barrier_init();
    }
    __syncthreads();
    if (tid == 0) {
        ptx::mbar_expect_tx(bar, (uint32_t)((2 + 2 * boxes) * 8192));
        ptx::tma_load_4d(smem + oX1, x1, bar, 0, (int)h, (int)r0, (int)b);
        ptx::tma_load_4d(smem + oX2, x2, bar, 0, (int)h, (int)r0, (int)b);
        for (int i = 0; i < boxes; ++i) {
            ptx::tma_load_4d(smem + oY1 + i * 8192, y1, bar, 0, (int)h, (int)c0 + 64 * i, (int)b);
            ptx::tma_load_4d(smem + oY2 + i * 8192, y2, bar, 0, (int)h, (int)c0 + 64 * i, (int)b);
        }
    }
    if (tid == 32 && a.prefetch_ahead > 0) {
        // Pull the tile that will run in this CTA's slot a generation from now into L2 (same boxes as the real
        // copies, nothing lands in shared memory), so that its own copies find their rows there.
        const uint32_t gx = gridDim.x, gy = gridDim.y;
        const uint32_t lin = (blockIdx.z * gy + blockIdx.y) * gx + blockIdx.x + (uint32_t)a.prefetch_ahead;
        const int h2 = (int)(lin % gx), t2 = (int)((lin / gx) % gy), b2 = (int)(lin / (gx * gy));
        if (b2 < (int)gridDim.z) {
            const int64_t r2 = (int64_t)t2 * kTile, c2 = r2 - back;
            if (r2 + kTile <= a.S) {
                ptx::tma_prefetch_4d(x1, 0, h2, (int)r2, b2);
                ptx::tma_prefetch_4d(x2, 0, h2, (int)r2, b2);
            }
            for (int i = 0; i < boxes; ++i) {
                const int64_t cr = c2 + 64 * i;
                if (cr >= 0 && cr + 64 <= a.S && (cr < r2 || cr >= r2 + kTile)) {   // the tile's own rows are on their way already
                    ptx::tma_prefetch_4d(y1, 0, h2, (int)cr, b2);
                    ptx::tma_prefetch_4d(y2, 0, h2, (int)cr, b2);
                }
            }
        }
    }
    if (COLS) {
        const float2 *st = a.stats + (b * a.HH + h) * a.S;
        for (int i = tid; i < band_rows; i += kThreads) {
            const int64_t gi = c0 + i;
            sst[i] = (gi >= 0 && gi < a.S) ? st[gi] : make_float2(0.f, 0.f);
        }
    }
    if (!ptx::mbar_wait(bar, 0)) {
        atomicExch(&g_bwd_status, 1);
        return;
    }
    __syncthreads();

    // A fragments of the warp's 16 rows, four k-steps over the head width
    uint32_t a1[4][4], a2[4][4];
    {
        const int row = 16 * warp + (lane & 15), cadd = lane >> 4;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            ptx::ldmatrix_x4(a1[ks], sbase + oX1 + swz(row, 2 * ks + cadd));
            ptx::ldmatrix_x4(a2[ks], sbase + oX2 + swz(row, 2 * ks + cadd));
        }
    }
    const int mi = lane >> 3, rr = lane & 7;
    const int brow_n = 16 * warp + (mi >> 1) * 8 + rr;   // + 16p: band row a lane addresses, plain B fragments
    const int bchk_n = mi & 1;                           // + 2ks
    const int brow_t = 16 * warp + (mi & 1) * 8 + rr;    // transposed B fragments
    const int bchk_t = mi >> 1;                          // + 2dn
    const float sl = a.scale * 1.4426950408889634f;
    const int64_t colbase = c0 + 16 * warp;              // global index of the warp's column 0
    // Column c (0..16 NP - 1, relative to the warp) is seen by row r (0..15) iff 0 <= c - r <= W and the column
    // exists.  Existence only matters in CTAs whose band crosses an end of the sequence (clo, chi clip it);
    // the diagonal test only in the first group and in groups that reach past W - 15.
    const int clo = colbase < 0 ? (int)-colbase : 0;
    const int chi = a.S - colbase < 16 * NP ? (int)(a.S - colbase) - 1 : 16 * NP - 1;
    const bool clipped = clo > 0 || chi < 16 * NP - 1;
    auto seen = [&](int c, int r) -> bool {
        return (unsigned)(c - r) <= (unsigned)W && c >= clo && c <= chi;
    };
    auto group_masked = [&](int p) -> bool { return clipped || p == 0 || 16 * p + 15 > W; };

    if constexpr (!COLS) {
        // The scores of the whole band stay in registers.  dP stays too when the band is narrow (NP <= 5);
        // a wide band recomputes it, once for delta and once for dS, which is cheaper than a second sweep
        // over both products.
        constexpr bool KEEP_DP = NP <= 5;
        float s[kPairs][2][4], dp[KEEP_DP ? kPairs : 1][2][4];
#pragma unroll
        for (int p = 0; p < kPairs; ++p)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[p][nt][e] = 0.f;
                    if (KEEP_DP) dp[KEEP_DP ? p : 0][nt][e] = 0.f;
                }
#pragma unroll
        for (int p = 0; p < kPairs; ++p) {
            if (p < np) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    uint32_t bf[4];
                    ptx::ldmatrix_x4(bf, sbase + oY1 + swz(brow_n + 16 * p, 2 * ks + bchk_n));
                    M::run(s[p][0], a1[ks], bf[0], bf[1]);
                    M::run(s[p][1], a1[ks], bf[2], bf[3]);
                    if (KEEP_DP) {
                        ptx::ldmatrix_x4(bf, sbase + oY2 + swz(brow_n + 16 * p, 2 * ks + bchk_n));
                        M::run(dp[KEEP_DP ? p : 0][0], a2[ks], bf[0], bf[1]);
                        M::run(dp[KEEP_DP ? p : 0][1], a2[ks], bf[2], bf[3]);
                    }
                }
            }
        }
        auto dp_group = [&](int p, float (&d)[2][4]) {   // dP of one group, for bands whose dP is not kept
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) d[nt][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t bf[4];
                ptx::ldmatrix_x4(bf, sbase + oY2 + swz(brow_n + 16 * p, 2 * ks + bchk_n));
                M::run(d[0], a2[ks], bf[0], bf[1]);
                M::run(d[1], a2[ks], bf[2], bf[3]);
            }
        };
        // softmax statistics of rows g and g + 8 (maximum of the raw scores: the scale is positive)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int p = 0; p < kPairs; ++p) {
            if (p < np) {
                if (group_masked(p)) {
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (!seen(16 * p + 8 * nt + 2 * t + (e & 1), g + (e >> 1) * 8)) s[p][nt][e] = -INFINITY;
                }
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[p][nt][e]);
            }
        }
        float sum[2] = {0.f, 0.f}, delta[2] = {0.f, 0.f}, msl[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            mx[hh] = quad_max(mx[hh]);
            if (mx[hh] == -INFINITY) mx[hh] = 0.f;   // a row past the end of the sequence
            msl[hh] = mx[hh] * sl;
        }
        // e = exp2(s sl - max sl); row sums of e and of e dP
#pragma unroll
        for (int p = 0; p < kPairs; ++p) {
            if (p < np) {
                float dl[2][4];
                if (!KEEP_DP) dp_group(p, dl);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float ex = ptx::ex2(fmaf(s[p][nt][e], sl, -msl[e >> 1]));
                        s[p][nt][e] = ex;
                        sum[e >> 1] += ex;
                        delta[e >> 1] = fmaf(ex, KEEP_DP ? dp[KEEP_DP ? p : 0][nt][e] : dl[nt][e], delta[e >> 1]);
                    }
            }
        }
        float cs[2], dcs[2];   // scale / sum and delta scale / sum: dS = e (dP cs - dcs)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            sum[hh] = quad_sum(sum[hh]);
            const float inv = sum[hh] > 0.f ? 1.f / sum[hh] : 0.f;
            delta[hh] = quad_sum(delta[hh]) * inv;
            cs[hh] = inv * a.scale;
            dcs[hh] = delta[hh] * cs[hh];
        }
        if (t == 0) {
            float2 *st = a.stats + (b * a.HH + h) * a.S;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int64_t gr = r0 + 16 * warp + g + 8 * hh;
                if (gr < a.S) st[gr] = make_float2(msl[hh] + log2f(sum[hh]), delta[hh] * a.scale);
            }
        }
        // dQ = dS K over the band, dS = P (dP - delta) scale
        float o[8][4];
#pragma unroll
        for (int dt = 0; dt < 8; ++dt)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[dt][e] = 0.f;
#pragma unroll
        for (int p = 0; p < kPairs; ++p) {
            if (p < np) {
                uint32_t af[4];
                float dl[2][4];
                if (!KEEP_DP) dp_group(p, dl);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    float ds[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        ds[e] = s[p][nt][e] * fmaf(KEEP_DP ? dp[KEEP_DP ? p : 0][nt][e] : dl[nt][e], cs[e >> 1], -dcs[e >> 1]);
                    af[2 * nt] = M::pack(ds[0], ds[1]);
                    af[2 * nt + 1] = M::pack(ds[2], ds[3]);
                }
#pragma unroll
                for (int dn = 0; dn < 4; ++dn) {
                    uint32_t bf[4];
                    ptx::ldmatrix_x4_trans(bf, sbase + oY1 + swz(brow_t + 16 * p, 2 * dn + bchk_t));
                    M::run(o[2 * dn], af, bf[0], bf[1]);
                    M::run(o[2 * dn + 1], af, bf[2], bf[3]);
                }
            }
        }
        store_tile<T>(smem, oX1, o, (T *)a.dq + head_off, r0, a.S, stride, warp, lane);
    } else {
        float ok_[8][4], ov[8][4];   // dK and dV of the warp's 16 keys
#pragma unroll
        for (int dt = 0; dt < 8; ++dt)
#pragma unroll
            for (int e = 0; e < 4; ++e) ok_[dt][e] = ov[dt][e] = 0.f;
#pragma unroll
        for (int p = 0; p < kPairs; ++p) {
            if (p < np) {
                float st[2][4], dpt[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) st[nt][e] = dpt[nt][e] = 0.f;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    uint32_t bf[4];
                    ptx::ldmatrix_x4(bf, sbase + oY1 + swz(brow_n + 16 * p, 2 * ks + bchk_n));
                    M::run(st[0], a1[ks], bf[0], bf[1]);
                    M::run(st[1], a1[ks], bf[2], bf[3]);
                    ptx::ldmatrix_x4(bf, sbase + oY2 + swz(brow_n + 16 * p, 2 * ks + bchk_n));
                    M::run(dpt[0], a2[ks], bf[0], bf[1]);
                    M::run(dpt[1], a2[ks], bf[2], bf[3]);
                }
                uint32_t ap[4], as[4];
                const bool masked = group_masked(p);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int cb = 16 * p + 8 * nt + 2 * t;
                    const float4 sd = *(const float4 *)&sst[16 * warp + cb];   // (lse, delta scale) of two queries
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float lse = (e & 1) ? sd.z : sd.x, dl = (e & 1) ? sd.w : sd.y;
                        float pp = ptx::ex2(fmaf(st[nt][e], sl, -lse));
                        if (masked && !seen(cb + (e & 1), g + (e >> 1) * 8)) pp = 0.f;
                        st[nt][e] = pp;
                        dpt[nt][e] = pp * fmaf(dpt[nt][e], a.scale, -dl);
                    }
                    ap[2 * nt] = M::pack(st[nt][0], st[nt][1]);
                    ap[2 * nt + 1] = M::pack(st[nt][2], st[nt][3]);
                    as[2 * nt] = M::pack(dpt[nt][0], dpt[nt][1]);
                    as[2 * nt + 1] = M::pack(dpt[nt][2], dpt[nt][3]);
                }
#pragma unroll
                for (int dn = 0; dn < 4; ++dn) {
                    uint32_t bf[4];
                    ptx::ldmatrix_x4_trans(bf, sbase + oY2 + swz(brow_t + 16 * p, 2 * dn + bchk_t));
                    M::run(ov[2 * dn], ap, bf[0], bf[1]);
                    M::run(ov[2 * dn + 1], ap, bf[2], bf[3]);
                    ptx::ldmatrix_x4_trans(bf, sbase + oY1 + swz(brow_t + 16 * p, 2 * dn + bchk_t));
                    M::run(ok_[2 * dn], as, bf[0], bf[1]);
                    M::run(ok_[2 * dn + 1], as, bf[2], bf[3]);
                }
            }
        }
        store_tile<T>(smem, oX1, ok_, (T *)a.dk + head_off, r0, a.S, stride, warp, lane);
        store_tile<T>(smem, oX2, ov, (T *)a.dv + head_off, r0, a.S, stride, warp, lane);
    }
}

template <typename T, int NP>
int launch_bwd(const BwdArgs &a, int dtype, cudaStream_t stream) {
    int rc = ensure_dynamic_smem((const void *)bwd_window_mma_kernel<T, false, NP>, smem_bytes(NP), "bwd_window_mma rows");
    if (rc != MAT_OK) return rc;
    rc = ensure_dynamic_smem((const void *)bwd_window_mma_kernel<T, true, NP>, smem_bytes(NP), "bwd_window_mma cols");
    if (rc != MAT_OK) return rc;
    CUtensorMap mq, mk, mv, mgo;
    if ((rc = make_row_tensor_map(&mq, a.q, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&mk, a.k, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&mv, a.v, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&mgo, a.go, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    const dim3 grid((unsigned)a.HH, (unsigned)((a.S + kTile - 1) / kTile), (unsigned)a.B);
    bwd_window_mma_kernel<T, false, NP><<<grid, kThreads, smem_bytes(NP), stream>>>(mq, mk, mv, mgo, a);
    bwd_window_mma_kernel<T, true, NP><<<grid, kThreads, smem_bytes(NP), stream>>>(mq, mk, mv, mgo, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "tensor-core backward launch");
    note_kernel("bwd_window_mma");
    return MAT_OK;
}

// ---- any window wider than 128 taps, dense included: the band streamed through shared memory ----------------
//
// Same two passes, same roles, but the band no longer fits in shared memory: it is walked in 64-column chunks
// aligned to the sequence (one TMA box of each band operand per chunk, two stages: a chunk's copies are issued
// while the previous chunk is being computed).  The rows pass walks it twice, once for the row statistics with a running maximum and once for
// dQ; the cols pass walks it once.  A warp skips the 16-column groups none of its rows can see and masks only
// the groups that straddle an edge of the window or the end of the sequence.
constexpr int kStreamSmemBytes = 2 * 8192 + 2 * 16384 + 2 * 64 * (int)sizeof(float2) + 16 + 64 * (int)sizeof(int32_t);

template <typename T, bool COLS>
__global__ void __launch_bounds__(kThreads, COLS ? 3 : 4)
bwd_stream_mma_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                      const __grid_constant__ CUtensorMap mv, const __grid_constant__ CUtensorMap mgo,
                      const __grid_constant__ LfMaps lf, BwdArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    using M = ptx::Mma<T>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int64_t r0 = (int64_t)blockIdx.y * kTile;   // heads vary fastest over the grid
    const int64_t h = blockIdx.x, b = blockIdx.z;
    const int64_t back = COLS ? a.right : a.left, fwd = COLS ? a.left : a.right;   // row r sees columns r - back .. r + fwd
    const unsigned W = (unsigned)(back + fwd);
    const int64_t stride = a.HH * 64;
    const int64_t head_off = (b * a.S * a.HH + h) * 64;
    const bool lf_tile = a.lf_mode == 2;   // the tile is the gathered global rows (queries) or keys
    const CUtensorMap *x1 = lf_tile ? (COLS ? &lf.k : &lf.q) : (COLS ? &mk : &mq);
    const CUtensorMap *x2 = lf_tile ? (COLS ? &lf.v : &lf.go) : (COLS ? &mv : &mgo);
    const CUtensorMap *y1 = COLS ? &mq : &mk, *y2 = COLS ? &mgo : &mv;
    const CUtensorMap *y1g = COLS ? &lf.q : &lf.k, *y2g = COLS ? &lf.go : &lf.v;   // lf_mode 1: the gathered chunk
    // tile rows | two stages of (band operand 1, band operand 2) | two stages of statistics | two barriers | global positions
    constexpr uint32_t oX1 = 0, oX2 = 8192, oY = 16384, oSt = oY + 2 * 16384, oBar = oSt + 2 * 512, oG = oBar + 16;
    const uint32_t sbase = ptx::smem_u32(smem);
    uint64_t *bar = (uint64_t *)(smem + oBar);
    int32_t *sG = (int32_t *)(smem + oG);   // Longformer: the global positions (slots past the list: -1)
    if (a.lf_mode != 0 && tid < 64) sG[tid] = tid < a.n_global ? (int32_t)a.gidx[tid] : -1;
    const int64_t lo = r0 - back > 0 ? r0 - back : 0;
    const int64_t hi = r0 + 63 + fwd < a.S - 1 ? r0 + 63 + fwd : a.S - 1;
    const int64_t k_first = lo / 64;
    const bool blk = a.block_mode != 0;
    const int32_t *blk_idx = COLS ? a.t_colidx : a.colidx;
    int64_t e0 = 0;
    int nch = (int)(hi / 64 - k_first) + 1;              // chunks per walk of the band
    if (blk) {
        const int32_t *ptr = COLS ? a.t_rowptr : a.rowptr;
        const int64_t lr = r0 / (64 * a.per_blk);        // the tile's layout row
        e0 = ptr[lr];
        nch = (ptr[lr + 1] - (int)e0) * a.per_blk;
    }
    const int nch_band = nch;
    if (a.lf_mode == 1 && a.n_global > 0) ++nch;         // + the chunk of gathered rows
    // chunk m of the walk: 64 columns starting at 64 * chunk_at(m); -1: the gathered chunk
    auto chunk_at = [&](int m) -> int64_t {
        if (a.lf_mode == 1 && m >= nch_band) return -1;
        return blk ? (int64_t)blk_idx[e0 + m / a.per_blk] * a.per_blk + m % a.per_blk : k_first + m;
    };
    const int total = COLS ? nch : 2 * nch;              // the rows pass walks it twice
    const int64_t wrow = r0 + 16 * warp;                 // the warp's first row
    if (nch == 0) {
        // a layout row without a block: no gradient flows through these rows
        float zero[8][4];
#pragma unroll
        for (int dt = 0; dt < 8; ++dt) zero[dt][0] = zero[dt][1] = zero[dt][2] = zero[dt][3] = 0.f;
        if constexpr (!COLS) {
            if (tid < 64 && r0 + tid < a.S) a.stats[(b * a.HH + h) * a.S + r0 + tid] = make_float2(0.f, 0.f);
            store_tile<T>(smem, oX1, zero, (T *)a.dq + head_off, r0, a.S, stride, warp, lane);
        } else {
            store_tile<T>(smem, oX1, zero, (T *)a.dk + head_off, r0, a.S, stride, warp, lane);
            store_tile<T>(smem, oX2, zero, (T *)a.dv + head_off, r0, a.S, stride, warp, lane);
        }
        return;
    }

    if (tid == 0) {
        ptx::mbar_init(bar, 1);
        ptx::mbar_init(bar + 1, 1);
        ptx::fence_barrier_init();
    }
    __syncthreads();
    // Step n of the flat walk (chunk k_first + n % nch) goes to stage n & 1.  It is issued while step n - 1 is
    // being computed, after the barrier that says every warp has left step n - 2, the stage's previous tenant.
    auto issue = [&](int n) {
        const int64_t k = chunk_at(n % nch);
        const int st = n & 1;
        if (tid == 0) {
            ptx::mbar_expect_tx(bar + st, n == 0 ? 32768u : 16384u);
            if (n == 0) {
                ptx::tma_load_4d(smem + oX1, x1, bar, 0, (int)h, (int)r0, (int)b);
                ptx::tma_load_4d(smem + oX2, x2, bar, 0, (int)h, (int)r0, (int)b);
            }
            ptx::tma_load_4d(smem + oY + st * 16384, k < 0 ? y1g : y1, bar + st, 0, (int)h, k < 0 ? 0 : (int)(64 * k), (int)b);
            ptx::tma_load_4d(smem + oY + st * 16384 + 8192, k < 0 ? y2g : y2, bar + st, 0, (int)h, k < 0 ? 0 : (int)(64 * k), (int)b);
        }
        if (COLS && tid < 64) {
            const int64_t gi = 64 * k + tid;
            float2 sv = make_float2(0.f, 0.f);
            if (k < 0) sv = a.stats_g[(b * a.HH + h) * 64 + tid];
            else if (gi < a.S) sv = a.stats[(b * a.HH + h) * a.S + gi];
            ((float2 *)(smem + oSt + st * 512))[tid] = sv;
        }
    };
    issue(0);

    const int mi = lane >> 3, rr = lane & 7;
    const int brow_n = (mi >> 1) * 8 + rr, bchk_n = mi & 1;   // + 16p / + 2ks: plain B fragments
    const int brow_t = (mi & 1) * 8 + rr, bchk_t = mi >> 1;   // + 16p / + 2dn: transposed B fragments
    const float sl = a.scale * 1.4426950408889634f;
    uint32_t a1[4][4], a2[4][4];
    // group p of chunk k: 0 = none of the warp's rows sees it, 1 = every (row, column) pair is seen, 2 = mask it
    auto group_kind = [&](int64_t k, int p) -> int {
        if (k < 0) return 16 * p < a.n_global ? 2 : 0;   // the gathered chunk: always masked (window positions, unused slots)
        const int64_t c = 64 * k + 16 * p;      // the group's first column
        if (blk) {
            // every (row, column) pair of a block counts, except past the causal diagonal (a key after its query:
            // the rows pass has queries as rows, the cols pass keys) and past the end of the sequence
            if (c >= a.S) return 0;
            bool full = c + 15 < a.S;
            if (a.causal) {
                if (COLS ? c + 15 < wrow : c > wrow + 15) return 0;
                full = full && (COLS ? c >= wrow + 15 : c + 15 <= wrow);
            }
            return full ? 1 : 2;
        }
        if (c + 15 < wrow - back || c > wrow + 15 + fwd || c >= a.S) return 0;
        return (c - (wrow + 15) >= -back && c + 15 - wrow <= fwd && c + 15 < a.S) ? 1 : 2;
    };
    // column 64k + 16p + cc of row wrow + r is seen iff -back <= column - row <= fwd and the column exists
    auto seen = [&](int64_t k, int p, int cc, int r) -> bool {
        if (k < 0) {
            // slot 16p + cc of the gathered chunk: a global position counts unless the row's window holds it already
            const int pos = sG[16 * p + cc];
            const int d = pos - (int)(wrow + r);
            return pos >= 0 && (unsigned)(d + (int)back) > W;
        }
        const int64_t c = 64 * k + 16 * p;
        const int d = (int)(c - wrow) + cc - r;     // column - row
        if (blk) return c + cc < a.S && (!a.causal || (COLS ? d >= 0 : d <= 0));
        return (unsigned)(d + (int)back) <= W && c + cc < a.S;
    };
    auto group_products = [&](uint32_t y, int p, float (&s)[2][4], float (&dp)[2][4]) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = dp[nt][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t bf[4];
            ptx::ldmatrix_x4(bf, y + swz(brow_n + 16 * p, 2 * ks + bchk_n));
            M::run(s[0], a1[ks], bf[0], bf[1]);
            M::run(s[1], a1[ks], bf[2], bf[3]);
            ptx::ldmatrix_x4(bf, y + 8192 + swz(brow_n + 16 * p, 2 * ks + bchk_n));
            M::run(dp[0], a2[ks], bf[0], bf[1]);
            M::run(dp[1], a2[ks], bf[2], bf[3]);
        }
    };

    // rows pass: running statistics of sweep one, then what sweep two needs; cols pass: the two outputs
    float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f}, dr[2] = {0.f, 0.f}, lse[2] = {0.f, 0.f}, dsc[2] = {0.f, 0.f};
    float o[8][4], ov[COLS ? 8 : 1][4];   // rows: dQ; cols: dK in o, dV in ov
#pragma unroll
    for (int dt = 0; dt < 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            o[dt][e] = 0.f;
            if (COLS) ov[dt][e] = 0.f;
        }

    for (int n = 0; n < total; ++n) {
        __syncthreads();   // every warp has left step n - 1; the statistics written for step n are visible
        if (n + 1 < total) issue(n + 1);
        if (!ptx::mbar_wait(bar + (n & 1), (n >> 1) & 1)) {
            atomicExch(&g_bwd_status, 1);
            return;
        }
        if (n == 0) {
            const int row = 16 * warp + (lane & 15), cadd = lane >> 4;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                ptx::ldmatrix_x4(a1[ks], sbase + oX1 + swz(row, 2 * ks + cadd));
                ptx::ldmatrix_x4(a2[ks], sbase + oX2 + swz(row, 2 * ks + cadd));
            }
        }
        const int64_t k = chunk_at(n % nch);
        const uint32_t y = sbase + oY + (n & 1) * 16384;
        if constexpr (!COLS) {
            if (n == nch) {   // between the sweeps: the statistics are complete
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    sum[hh] = quad_sum(sum[hh]);
                    dr[hh] = quad_sum(dr[hh]);            // every lane takes part in the shuffles, live row or not
                    const bool live = sum[hh] > 0.f;
                    lse[hh] = live ? mx[hh] * sl + log2f(sum[hh]) : 0.f;
                    dsc[hh] = live ? dr[hh] / sum[hh] * a.scale : 0.f;
                }
                if (t == 0) {
                    float2 *st = a.stats + (b * a.HH + h) * a.S;
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int64_t gr = wrow + g + 8 * hh;
                        if (lf_tile) {
                            // the gathered rows: their statistics go to their positions and, in gathered order, to
                            // where the cols pass reads its chunk of global queries from
                            const int pos = sG[gr];
                            const float2 sv = pos >= 0 ? make_float2(lse[hh], dsc[hh]) : make_float2(0.f, 0.f);
                            a.stats_g[(b * a.HH + h) * 64 + gr] = sv;
                            if (pos >= 0) st[pos] = sv;
                        } else if (gr < a.S) {
                            st[gr] = make_float2(lse[hh], dsc[hh]);
                        }
                    }
                }
            }
#pragma unroll 1
            for (int p = 0; p < 4; ++p) {
                const int kind = group_kind(k, p);
                if (kind == 0) continue;
                float s[2][4], dp[2][4];
                group_products(y, p, s, dp);
                if (n < nch) {
                    if (kind == 2) {
#pragma unroll
                        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (!seen(k, p, 8 * nt + 2 * t + (e & 1), g + (e >> 1) * 8)) s[nt][e] = -INFINITY;
                    }
                    float gm[2] = {-INFINITY, -INFINITY}, msl[2];
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) gm[e >> 1] = fmaxf(gm[e >> 1], s[nt][e]);
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const float m_new = fmaxf(mx[hh], quad_max(gm[hh]));
                        const float alpha = mx[hh] == -INFINITY ? 0.f : ptx::ex2((mx[hh] - m_new) * sl);
                        sum[hh] *= alpha;
                        dr[hh] *= alpha;
                        mx[hh] = m_new;
                        msl[hh] = m_new == -INFINITY ? 0.f : m_new * sl;
                    }
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float ex = ptx::ex2(fmaf(s[nt][e], sl, -msl[e >> 1]));
                            sum[e >> 1] += ex;
                            dr[e >> 1] = fmaf(ex, dp[nt][e], dr[e >> 1]);
                        }
                } else {
                    uint32_t af[4];
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        float ds[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float pp = ptx::ex2(fmaf(s[nt][e], sl, -lse[e >> 1]));
                            if (kind == 2 && !seen(k, p, 8 * nt + 2 * t + (e & 1), g + (e >> 1) * 8)) pp = 0.f;
                            ds[e] = pp * fmaf(dp[nt][e], a.scale, -dsc[e >> 1]);
                        }
                        af[2 * nt] = M::pack(ds[0], ds[1]);
                        af[2 * nt + 1] = M::pack(ds[2], ds[3]);
                    }
#pragma unroll
                    for (int dn = 0; dn < 4; ++dn) {
                        uint32_t bf[4];
                        ptx::ldmatrix_x4_trans(bf, y + swz(brow_t + 16 * p, 2 * dn + bchk_t));
                        M::run(o[2 * dn], af, bf[0], bf[1]);
                        M::run(o[2 * dn + 1], af, bf[2], bf[3]);
                    }
                }
            }
        } else {
            const float2 *sst = (const float2 *)(smem + oSt + (n & 1) * 512);
#pragma unroll 1
            for (int p = 0; p < 4; ++p) {
                const int kind = group_kind(k, p);
                if (kind == 0) continue;
                float st[2][4], dpt[2][4];
                group_products(y, p, st, dpt);
                uint32_t ap[4], as[4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int cb = 8 * nt + 2 * t;
                    const float4 sd = *(const float4 *)&sst[16 * p + cb];   // (lse, delta scale) of two queries
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float ls = (e & 1) ? sd.z : sd.x, dl = (e & 1) ? sd.w : sd.y;
                        float pp = ptx::ex2(fmaf(st[nt][e], sl, -ls));
                        if (kind == 2 && !seen(k, p, cb + (e & 1), g + (e >> 1) * 8)) pp = 0.f;
                        st[nt][e] = pp;
                        dpt[nt][e] = pp * fmaf(dpt[nt][e], a.scale, -dl);
                    }
                    ap[2 * nt] = M::pack(st[nt][0], st[nt][1]);
                    ap[2 * nt + 1] = M::pack(st[nt][2], st[nt][3]);
                    as[2 * nt] = M::pack(dpt[nt][0], dpt[nt][1]);
                    as[2 * nt + 1] = M::pack(dpt[nt][2], dpt[nt][3]);
                }
#pragma unroll
                for (int dn = 0; dn < 4; ++dn) {
                    uint32_t bf[4];
                    ptx::ldmatrix_x4_trans(bf, y + 8192 + swz(brow_t + 16 * p, 2 * dn + bchk_t));
                    M::run(ov[2 * dn], ap, bf[0], bf[1]);
                    M::run(ov[2 * dn + 1], ap, bf[2], bf[3]);
                    ptx::ldmatrix_x4_trans(bf, y + swz(brow_t + 16 * p, 2 * dn + bchk_t));
                    M::run(o[2 * dn], as, bf[0], bf[1]);
                    M::run(o[2 * dn + 1], as, bf[2], bf[3]);
                }
            }
        }
    }
    const int32_t *scatter = lf_tile ? sG : nullptr;   // the gathered tile's rows go to their positions
    if constexpr (!COLS) {
        store_tile<T>(smem, oX1, o, (T *)a.dq + head_off, r0, a.S, stride, warp, lane, scatter);
    } else {
        store_tile<T>(smem, oX1, o, (T *)a.dk + head_off, r0, a.S, stride, warp, lane, scatter);
        store_tile<T>(smem, oX2, ov, (T *)a.dv + head_off, r0, a.S, stride, warp, lane, scatter);
    }
}

template <typename T>
int launch_bwd_stream(const BwdArgs &a, int dtype, cudaStream_t stream) {
    int rc = ensure_dynamic_smem((const void *)bwd_stream_mma_kernel<T, false>, kStreamSmemBytes, "bwd_stream_mma rows");
    if (rc != MAT_OK) return rc;
    rc = ensure_dynamic_smem((const void *)bwd_stream_mma_kernel<T, true>, kStreamSmemBytes, "bwd_stream_mma cols");
    if (rc != MAT_OK) return rc;
    CUtensorMap mq, mk, mv, mgo;
    if ((rc = make_row_tensor_map(&mq, a.q, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&mk, a.k, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&mv, a.v, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&mgo, a.go, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    const dim3 grid((unsigned)a.HH, (unsigned)((a.S + kTile - 1) / kTile), (unsigned)a.B);
    LfMaps lf;
    lf.q = mq; lf.k = mk; lf.v = mv; lf.go = mgo;   // unused outside the Longformer modes
    bwd_stream_mma_kernel<T, false><<<grid, kThreads, kStreamSmemBytes, stream>>>(mq, mk, mv, mgo, lf, a);
    bwd_stream_mma_kernel<T, true><<<grid, kThreads, kStreamSmemBytes, stream>>>(mq, mk, mv, mgo, lf, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "tensor-core backward launch");
    note_kernel(a.block_mode ? "bwd_block_mma" : "bwd_stream_mma");
    return MAT_OK;
}

// rows of four [B, S, HH, 64] tensors at the global positions -> four [B, n_global, HH, 64] tensors;
// grid = (global position, batch), threads stride over the HH * 8 16-byte pieces of a row set
__global__ void gather4_kernel(const uint4 *__restrict__ s0, const uint4 *__restrict__ s1, const uint4 *__restrict__ s2,
                               const uint4 *__restrict__ s3, uint4 *__restrict__ d0, uint4 *__restrict__ d1,
                               uint4 *__restrict__ d2, uint4 *__restrict__ d3, const int64_t *__restrict__ gidx,
                               int n_global, int64_t S, int64_t HH) {
    const int e = blockIdx.x, b = blockIdx.y;
    const int64_t row = gidx[e];
    const bool in = row >= 0 && row < S;   // a position outside the sequence gathers zeros, never memory
    const int64_t src = ((int64_t)b * S + (in ? row : 0)) * HH * 8, dst = ((int64_t)b * n_global + e) * HH * 8;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int64_t i = threadIdx.x; i < HH * 8; i += blockDim.x) {
        d0[dst + i] = in ? s0[src + i] : zero;
        d1[dst + i] = in ? s1[src + i] : zero;
        d2[dst + i] = in ? s2[src + i] : zero;
        d3[dst + i] = in ? s3[src + i] : zero;
    }
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// Longformer on the streamed kernels: gather, rows pass over every tile (window band + the chunk of global keys),
// rows pass over the gathered global queries (every key), cols pass over every tile (mirrored band + the chunk of
// global queries), cols pass over the gathered global keys (every query).  The two gathered passes overwrite what
// the tile passes left at the global positions.
template <typename T>
int launch_bwd_longformer(BwdArgs a, int dtype, void *extra_ws, cudaStream_t stream) {
    int rc = ensure_dynamic_smem((const void *)bwd_stream_mma_kernel<T, false>, kStreamSmemBytes, "bwd_stream_mma rows");
    if (rc != MAT_OK) return rc;
    rc = ensure_dynamic_smem((const void *)bwd_stream_mma_kernel<T, true>, kStreamSmemBytes, "bwd_stream_mma cols");
    if (rc != MAT_OK) return rc;
    const size_t gbytes = align256((size_t)a.B * a.n_global * a.HH * 128);
    uint8_t *w = (uint8_t *)extra_ws;
    a.stats_g = (float2 *)w;
    w += align256((size_t)a.B * a.HH * 64 * sizeof(float2));
    void *qg = w, *kg = w + gbytes, *vg = w + 2 * gbytes, *gog = w + 3 * gbytes;
    gather4_kernel<<<dim3((unsigned)a.n_global, (unsigned)a.B), 128, 0, stream>>>(
        (const uint4 *)a.q, (const uint4 *)a.k, (const uint4 *)a.v, (const uint4 *)a.go, (uint4 *)qg, (uint4 *)kg,
        (uint4 *)vg, (uint4 *)gog, a.gidx, a.n_global, a.S, a.HH);
    CUtensorMap mq, mk, mv, mgo;
    LfMaps lf;
    if ((rc = make_row_tensor_map(&mq, a.q, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&mk, a.k, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&mv, a.v, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&mgo, a.go, dtype, a.HH, a.S, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&lf.q, qg, dtype, a.HH, a.n_global, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&lf.k, kg, dtype, a.HH, a.n_global, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&lf.v, vg, dtype, a.HH, a.n_global, a.B, kTile)) != MAT_OK) return rc;
    if ((rc = make_row_tensor_map(&lf.go, gog, dtype, a.HH, a.n_global, a.B, kTile)) != MAT_OK) return rc;
    const dim3 grid((unsigned)a.HH, (unsigned)((a.S + kTile - 1) / kTile), (unsigned)a.B);
    const dim3 grid_g((unsigned)a.HH, 1, (unsigned)a.B);
    BwdArgs tiles = a, rows_g = a;
    tiles.lf_mode = 1;
    rows_g.lf_mode = 2;
    rows_g.left = rows_g.right = (int)a.S;   // the gathered rows against every chunk
    bwd_stream_mma_kernel<T, false><<<grid, kThreads, kStreamSmemBytes, stream>>>(mq, mk, mv, mgo, lf, tiles);
    bwd_stream_mma_kernel<T, false><<<grid_g, kThreads, kStreamSmemBytes, stream>>>(mq, mk, mv, mgo, lf, rows_g);
    bwd_stream_mma_kernel<T, true><<<grid, kThreads, kStreamSmemBytes, stream>>>(mq, mk, mv, mgo, lf, tiles);
    bwd_stream_mma_kernel<T, true><<<grid_g, kThreads, kStreamSmemBytes, stream>>>(mq, mk, mv, mgo, lf, rows_g);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "tensor-core Longformer backward launch");
    note_kernel("bwd_longformer_mma");
    return MAT_OK;
}

}  // namespace

int bwd_status_read_and_clear(int *out) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(out, g_bwd_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_bwd_status, &zero, sizeof(int));
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, "reading the backward kernels' status word");
}

bool bwd_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t left, int64_t right,
                      int64_t dil) {
    if (dtype != MAT_BF16 && dtype != MAT_F16) return false;
    if (D != 64 || dil < 1 || S % dil != 0) return false;
    const char *env = getenv("MAT_BWD_KERNEL");
    if (env && strcmp(env, "warp") == 0) return false;
    const int64_t Sv = S / dil;
    const int64_t l = left < Sv - 1 ? left : Sv - 1, r = right < Sv - 1 ? right : Sv - 1;
    return H * dil < (1LL << 31) && (Sv + kTile - 1) / kTile <= 65535 && B <= 65535;
}

int launch_bwd_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
                   float2 *stats, int64_t B, int64_t S, int64_t H, int dtype, int64_t left, int64_t right,
                   int64_t dil, float scale, cudaStream_t stream) {
    BwdArgs a;
    a.q = q; a.k = k; a.v = v; a.go = dout;
    a.dq = dq; a.dk = dk; a.dv = dv;
    a.stats = stats;
    a.B = B; a.S = S / dil; a.HH = H * dil;
    a.left = (int)(left < a.S - 1 ? left : a.S - 1);
    a.right = (int)(right < a.S - 1 ? right : a.S - 1);
    if (a.left < 0) a.left = 0;     // a one-row sequence
    if (a.right < 0) a.right = 0;
    a.scale = scale;
    {   // prefetch distance: half of the CTAs resident on the GPU (4 per SM); MAT_BWD_PREFETCH_AHEAD overrides, 0 = off
        static int dist = -1;
        static std::once_flag once;
        std::call_once(once, [] {
            const char *env = getenv("MAT_BWD_PREFETCH_AHEAD");
            if (env) { dist = atoi(env); return; }
            int dev = 0, sms = 148;
            if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            dist = 2 * sms;
        });
        a.prefetch_ahead = dist;
    }
    if (a.left + a.right <= 64)
        return dtype == MAT_BF16 ? launch_bwd<__nv_bfloat16, 5>(a, dtype, stream) : launch_bwd<__half, 5>(a, dtype, stream);
    if (a.left + a.right <= 128)
        return dtype == MAT_BF16 ? launch_bwd<__nv_bfloat16, 9>(a, dtype, stream) : launch_bwd<__half, 9>(a, dtype, stream);
    return dtype == MAT_BF16 ? launch_bwd_stream<__nv_bfloat16>(a, dtype, stream) : launch_bwd_stream<__half>(a, dtype, stream);
}

// The Longformer pattern on the streamed tensor-core kernels: 16-bit, D = 64, 1 to 64 global positions.
bool bwd_longformer_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t n_global) {
    if (dtype != MAT_BF16 && dtype != MAT_F16) return false;
    if (D != 64 || n_global < 1 || n_global > 64 || S >= (1LL << 30)) return false;
    const char *env = getenv("MAT_BWD_KERNEL");
    if (env && strcmp(env, "warp") == 0) return false;
    return H < (1LL << 31) && (S + kTile - 1) / kTile <= 65535 && B <= 65535;
}

// bytes behind the per-row statistics: the global rows' statistics and the four gathered tensors
size_t bwd_longformer_mma_extra_bytes(int64_t B, int64_t H, int64_t n_global) {
    return align256((size_t)B * H * 64 * sizeof(float2)) + 4 * align256((size_t)B * n_global * H * 128);
}

int launch_bwd_longformer_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk,
                              void *dv, float2 *stats, void *extra_ws, int64_t B, int64_t S, int64_t H, int dtype,
                              int64_t left, int64_t right, int64_t n_global, const int64_t *gidx, float scale,
                              cudaStream_t stream) {
    BwdArgs a;
    a.q = q; a.k = k; a.v = v; a.go = dout;
    a.dq = dq; a.dk = dk; a.dv = dv;
    a.stats = stats;
    a.B = B; a.S = S; a.HH = H;
    a.left = (int)(left < S - 1 ? left : S - 1);
    a.right = (int)(right < S - 1 ? right : S - 1);
    if (a.left < 0) a.left = 0;
    if (a.right < 0) a.right = 0;
    a.scale = scale;
    a.prefetch_ahead = 0;
    a.n_global = (int)n_global;
    a.gidx = gidx;
    return dtype == MAT_BF16 ? launch_bwd_longformer<__nv_bfloat16>(a, dtype, extra_ws, stream)
                             : launch_bwd_longformer<__half>(a, dtype, extra_ws, stream);
}

// Block layouts on the streamed tensor-core kernels: 16-bit, D = 64, block a multiple of 64, both the layout and
// its transpose on the device.
bool bwd_block_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t block) {
    if (dtype != MAT_BF16 && dtype != MAT_F16) return false;
    if (D != 64 || block < 64 || block % 64 != 0 || block / 64 > 0x7fffffffLL) return false;
    const char *env = getenv("MAT_BWD_KERNEL");
    if (env && strcmp(env, "warp") == 0) return false;
    return H < (1LL << 31) && (S + kTile - 1) / kTile <= 65535 && B <= 65535;
}

int launch_bwd_block_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
                         float2 *stats, int64_t B, int64_t S, int64_t H, int dtype, int64_t block, int causal,
                         const int32_t *rowptr, const int32_t *colidx, const int32_t *t_rowptr, const int32_t *t_colidx,
                         float scale, cudaStream_t stream) {
    BwdArgs a;
    a.q = q; a.k = k; a.v = v; a.go = dout;
    a.dq = dq; a.dk = dk; a.dv = dv;
    a.stats = stats;
    a.B = B; a.S = S; a.HH = H;
    a.left = a.right = 0;
    a.scale = scale;
    a.prefetch_ahead = 0;
    a.block_mode = 1;
    a.causal = causal;
    a.per_blk = (int)(block / 64);
    a.rowptr = rowptr; a.colidx = colidx; a.t_rowptr = t_rowptr; a.t_colidx = t_colidx;
    return dtype == MAT_BF16 ? launch_bwd_stream<__nv_bfloat16>(a, dtype, stream) : launch_bwd_stream<__half>(a, dtype, stream);
}

}  // namespace mat
