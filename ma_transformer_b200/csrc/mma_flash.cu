// Tiled forward for 16-bit inputs with head width 64: per query tile, fused
// Q*K^T -> softmax -> P*V on the warp-level tensor-core path, with Q and the
// K/V window (halo included) staged in shared memory by TMA.
//
// This is the kernel for the narrow-window patterns, which are bound by HBM
// traffic: every Q/K/V row is one 128-byte line, fetched once per tile by a
// tiled bulk-tensor copy (128-byte swizzle, so ldmatrix reads are free of bank
// conflicts), and the output tile leaves through a bulk-tensor store.  Replaces
// sparse_attention_forward_warp (src/cuda/sparse_attention_kernel.cu:211-263),
// which re-reads K/V per query row from global memory with 4-byte loads.
//
// Work decomposition
//   - A dilated window over [B,S,H,64] is a plain window over the same memory
//     viewed as [B, S/dil, dil*H, 64]: query p = m*dil + r attends keys
//     (m+t)*dil + r, so residue r behaves as dil*H independent heads.  The
//     kernel only ever sees dil = 1.
//   - One CTA per (batch, head, tile of TQ queries); TQ/16 consumer warps own
//     16 query rows each, one extra warp issues the TMA loads through a ring of
//     TK-key K/V stages guarded by full/empty mbarriers.
//   - A warp walks only the 16-key column pairs that intersect its rows' key
//     set, NP pairs per softmax step, and masks only the pairs that straddle the
//     edge of the set.  When the whole window of a tile fits one stage and NP
//     pairs per warp (SINGLE, the case of 64 causal taps), there is exactly one
//     step: no running max / rescale, and the output accumulators are not live
//     while the scores are computed.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "mat_common.cuh"
#include "ptx.cuh"

namespace mat {
namespace {

constexpr int kRowBytes = 128;  // 64 elements of 2 bytes
constexpr int kBig = 1 << 29;   // "no limit" for a mask edge

// status words a kernel can leave in g_flash_status (0 = fine)
constexpr int kStatusWaitTimeout = 1;
__device__ int g_flash_status = 0;

struct FlashParams {
    int32_t Sq1, Skv1, off1;      // query rows, key rows and q_offset of one sub-sequence
    // Keys live in a virtual coordinate line: [0, Skv1) is this GPU's own K/V, [key_lo, 0) the tail
    // of the previous sequence shard and [Skv1, key_hi) the head of the next one, both read in
    // place from the neighbour GPU's memory.  Without neighbours key_lo = 0 and key_hi = Skv1.
    int32_t key_lo, key_hi;
    int32_t prev_rows, next_rows;  // rows per sub-sequence of the neighbours' K/V tensors
    int32_t left, right;          // window taps (clamped to Skv1); chunk enumeration
    int32_t mask_left, mask_right;  // a key j is attended by row p iff -mask_left <= j-p <= mask_right
    int32_t n_tiles;              // query tiles per (batch, head)
    int32_t prefetch_ahead;       // single-step window kernel: L2-prefetch the tile this many CTAs ahead (0 = off)
    int32_t HH;                   // heads seen by the kernel (dil * H)
    float sl2;                    // scale * log2(e)
    // block layout
    int32_t block, per_blk;
    int64_t n_qblocks;
    const int32_t *rowptr;
    const int32_t *colidx;
    // Longformer: sorted global positions.  Every row attends them besides its window
    // (MAT_LONGFORMER); the rows AT those positions attend every key (kGlobalRows pass).
    int32_t n_global;
    const int64_t *gidx;
    // kGlobalRows: the key axis is cut into n_splits ranges of split_len keys; each CTA leaves
    // (max, sum, unnormalised output) per row in `partial`, merged by merge_global_rows_kernel
    int32_t split_len, n_splits, ng_pad;
    float *partial;  // [B, HH, n_splits, ng_pad, kPartialStride]
    // MAT_LONGFORMER: the K/V rows at the global positions, gathered once into [B, n_global, HH, 64]
    // buffers by gather_global_rows_kernel (NULL: every tile gathers them itself, row by row)
    const void *kg, *vg;
};

constexpr int kGlobalRows = 3;       // kernel kind beside the MAT_* pattern kinds

__device__ __forceinline__ uint32_t swz(uint32_t base, int row, int chunk16) {
    return base + row * kRowBytes + ((chunk16 ^ (row & 7)) << 4);
}

// The staged key chunks of one query tile: chunk c starts at key base(c).
template <int KIND, int TQ, int TK>
struct Chunks {
    int n;
    int n_seq;  // chunks that are contiguous key ranges (the rest gather global keys)
    int start;  // first key of chunk 0 (window kinds, global-row pass)
    int e0;     // block: first CSR entry of the tile's layout row
    // key_lo / key_hi: the keys this CTA may touch
    __device__ __forceinline__ Chunks(const FlashParams &P, int q0, int key_lo, int key_hi) {
        n = 0; n_seq = 0; start = 0; e0 = 0;
        if (KIND == MAT_WINDOW || KIND == MAT_LONGFORMER) {
            int lo = q0 + P.off1 - P.left;
            if (lo < key_lo) lo = key_lo;
            lo &= ~15;
            int hi = q0 + TQ - 1 + P.off1 + P.right;
            if (hi > key_hi - 1) hi = key_hi - 1;
            start = lo;
            n_seq = hi >= lo ? (hi - lo) / TK + 1 : 0;
            n = n_seq + (KIND == MAT_LONGFORMER ? (P.n_global + TK - 1) / TK : 0);
        } else if (KIND == kGlobalRows) {
            start = key_lo;
            n = n_seq = key_hi > key_lo ? (key_hi - key_lo + TK - 1) / TK : 0;
        } else {
            const uint32_t r = (uint32_t)(q0 + P.off1) / (uint32_t)P.block;
            if ((int64_t)r < P.n_qblocks) {
                e0 = P.rowptr[r];
                n = n_seq = (P.rowptr[r + 1] - e0) * P.per_blk;
            }
        }
    }
    __device__ __forceinline__ int base(const FlashParams &P, int c) const {
        if (KIND != MAT_BLOCK) return start + c * TK;
        return P.colidx[e0 + c / P.per_blk] * P.block + (c % P.per_blk) * TK;
    }
};

// 16-row views of K and V used where a stage straddles the edge of this GPU's shard: own rows,
// the previous shard's rows and the next shard's rows (the neighbours' live in peer memory and
// are read by ordinary tiled TMA loads).
// q_row / k_row / v_row are one-row views used to gather the rows at the global positions.
struct PeerMaps {
    CUtensorMap k_own, v_own, k_prev, v_prev, k_next, v_next, q_row, k_row, v_row;
};

constexpr int kSideRows = 64;  // one-stage Longformer kernel: rows of the side region for the gathered keys

template <int TQ, int TK, int STAGES, bool SIDE = false>
constexpr size_t flash_smem_bytes() {
    // Q tile, K/V stages, [side region for gathered keys], barriers, then per stage the global
    // positions of a gathered chunk
    return 1024 + (size_t)TQ * kRowBytes + (size_t)STAGES * 2 * TK * kRowBytes +
           (SIDE ? 2 * kSideRows * kRowBytes : 0) + 8 * (1 + 2 * STAGES) + 8 + (size_t)STAGES * TK * 4;
}

constexpr int kNoKey = INT32_MIN;  // marks an unused slot of a gathered chunk

// Kernels whose tile needs at most one K/V stage (STAGES == 1, which includes every SINGLE
// kernel) issue all their loads up front, so they carry no producer warp: lane 0 of warp 0 issues
// the copies and then computes like every other lane.
template <int TQ, bool UPFRONT> constexpr int flash_threads() { return (TQ / 16 + (UPFRONT ? 0 : 1)) * 32; }

template <typename T, int KIND, int TQ, int TK, int NP, int STAGES, bool SINGLE, int MINB>
__global__ void __launch_bounds__(flash_threads<TQ, SINGLE || STAGES == 1>(), MINB)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                 const __grid_constant__ PeerMaps peer, const FlashParams P) {
    constexpr int NW = TQ / 16;  // consumer warps
    constexpr bool UPFRONT = SINGLE || STAGES == 1;  // no producer warp
    // Longformer with one stage: the window is the stage, the gathered keys (at most kSideRows of
    // them, pre-gathered by the host side) sit in a side region with a barrier of their own
    constexpr bool SIDE = KIND == MAT_LONGFORMER && STAGES == 1;
    constexpr int kStageBytes = 2 * TK * kRowBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem;
    uint8_t *sKV = smem + TQ * kRowBytes;
    uint8_t *sSide = sKV + STAGES * kStageBytes;
    uint64_t *bar_q = (uint64_t *)(sSide + (SIDE ? 2 * kSideRows * kRowBytes : 0));
    uint64_t *bar_full = bar_q + 1;
    uint64_t *bar_empty = bar_full + STAGES;
    uint64_t *bar_side = bar_empty + STAGES;            // completion of the side region's copies
    int32_t *sG = (int32_t *)(bar_empty + STAGES + 1);  // [STAGES][TK] positions of gathered keys

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // grid = (heads, query tiles, batch): the heads of one tile are scheduled together, so the
    // 128-byte rows they fetch from the same token range share DRAM pages
    const int hh = blockIdx.x;
    const int b = blockIdx.z;
    // kGlobalRows: blockIdx.y = (tile of the global-position list) * n_splits + key split
    const int split = KIND == kGlobalRows ? blockIdx.y % P.n_splits : 0;
    const int q0 = (KIND == kGlobalRows ? blockIdx.y / P.n_splits : blockIdx.y) * TQ;
    const int key_lo = KIND == kGlobalRows ? split * P.split_len : P.key_lo;
    const int key_hi = KIND == kGlobalRows ? min(key_lo + P.split_len, P.Skv1) : P.key_hi;

    if (threadIdx.x == 0) {
        ptx::mbar_init(bar_q, 1);
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full + s, 1);
            ptx::mbar_init(bar_empty + s, NW);
        }
        ptx::mbar_init(bar_side, 1);
        ptx::fence_barrier_init();
    }
    __syncthreads();

    const Chunks<KIND, TQ, TK> chunks(P, q0, key_lo, key_hi);

    if (UPFRONT ? warp == 0 : warp == NW) {  // ---- producer: one lane feeds the ring ----
        if (lane == 0) {
            ptx::mbar_expect_tx(bar_q, TQ * kRowBytes);
            if (KIND == kGlobalRows) {
                // the query tile is gathered: row r of the tile is the query at global position
                // gidx[q0 + r]; slots past the list read out of bounds, i.e. zeros
                for (int r = 0; r < TQ; ++r) {
                    const int e = q0 + r;
                    const int row = e < P.n_global ? (int)P.gidx[e] : P.Sq1;
                    ptx::tma_load_4d(sQ + r * kRowBytes, &peer.q_row, bar_q, 0, hh, row, b);
                }
            } else {
                ptx::tma_load_4d(sQ, &map_q, bar_q, 0, hh, q0, b);
            }
            for (int c = 0; c < chunks.n; ++c) {
                const int s = c % STAGES, use = c / STAGES;
                if (SIDE && c >= chunks.n_seq) {
                    // the (single) gathered chunk goes to the side region
                    const int n_in = min(kSideRows, P.n_global);
                    for (int i = 0; i < kSideRows; ++i) sG[i] = i < n_in ? (int)P.gidx[i] : kNoKey;
                    ptx::mbar_expect_tx(bar_side, 2 * kSideRows * kRowBytes);
                    ptx::tma_load_4d(sSide, &peer.k_row, bar_side, 0, hh, 0, b);
                    ptx::tma_load_4d(sSide + kSideRows * kRowBytes, &peer.v_row, bar_side, 0, hh, 0, b);
                    continue;
                }
                if (use > 0 && !ptx::mbar_wait(bar_empty + s, (use - 1) & 1)) {
                    atomicExch(&g_flash_status, kStatusWaitTimeout);
                    break;
                }
                uint8_t *dst = sKV + s * kStageBytes;
                if (KIND == MAT_LONGFORMER && c >= chunks.n_seq) {
                    // gathered chunk: the K/V rows at the next TK global positions, whole 16-key
                    // pairs only (slots past the list read out of bounds: zeros, so that a zero
                    // weight never meets a non-finite value)
                    const int e0 = (c - chunks.n_seq) * TK;
                    const int n_in = min(TK, P.n_global - e0);
                    const int rows = (n_in + 15) & ~15;
                    for (int i = 0; i < rows; ++i) sG[s * TK + i] = i < n_in ? (int)P.gidx[e0 + i] : kNoKey;
                    if (P.kg) {   // pre-gathered: one box per tensor; rows past the list are out of bounds = zeros
                        ptx::mbar_expect_tx(bar_full + s, kStageBytes);
                        ptx::tma_load_4d(dst, &peer.k_row, bar_full + s, 0, hh, e0, b);
                        ptx::tma_load_4d(dst + TK * kRowBytes, &peer.v_row, bar_full + s, 0, hh, e0, b);
                        continue;
                    }
                    ptx::mbar_expect_tx(bar_full + s, rows * 2 * kRowBytes);
                    for (int i = 0; i < rows; ++i) {
                        const int row = i < n_in ? sG[s * TK + i] : P.Skv1;
                        ptx::tma_load_4d(dst + i * kRowBytes, &peer.k_row, bar_full + s, 0, hh, row, b);
                        ptx::tma_load_4d(dst + (TK + i) * kRowBytes, &peer.v_row, bar_full + s, 0, hh, row, b);
                    }
                    continue;
                }
                const int kb = chunks.base(P, c);
                ptx::mbar_expect_tx(bar_full + s, kStageBytes);
                if (kb >= 0 && kb + TK <= P.Skv1 || P.key_lo == 0 && P.key_hi == P.Skv1) {
                    ptx::tma_load_4d(dst, &map_k, bar_full + s, 0, hh, kb, b);
                    ptx::tma_load_4d(dst + TK * kRowBytes, &map_v, bar_full + s, 0, hh, kb, b);
                } else {
                    // the stage crosses into a neighbour's rows: fetch it 16 rows at a time, each
                    // piece from the tensor that owns it
                    for (int i = 0; i < TK / 16; ++i) {
                        const int a = kb + 16 * i;
                        const CUtensorMap *mk = &peer.k_own, *mv = &peer.v_own;
                        int row = a;
                        if (a < 0 && P.key_lo < 0) {
                            mk = &peer.k_prev; mv = &peer.v_prev; row = P.prev_rows + a;
                        } else if (a >= P.Skv1 && P.key_hi > P.Skv1) {
                            mk = &peer.k_next; mv = &peer.v_next; row = a - P.Skv1;
                        }
                        ptx::tma_load_4d(dst + i * 16 * kRowBytes, mk, bar_full + s, 0, hh, row, b);
                        ptx::tma_load_4d(dst + (TK + i * 16) * kRowBytes, mv, bar_full + s, 0, hh, row, b);
                    }
                }
            }
        }
        if (SINGLE && KIND == MAT_WINDOW && lane == 0 && P.prefetch_ahead > 0) {
            // Pull the tile that will run in this CTA's slot a few generations from now into L2,
            // so that its own copies find their rows there: the wait for a tile's copies is the
            // largest stall of this kernel.  Same boxes as the real loads, nothing lands in
            // shared memory, every byte still leaves DRAM once.
            const uint32_t gx = gridDim.x, gy = gridDim.y;
            const uint32_t lin = (blockIdx.z * gy + blockIdx.y) * gx + blockIdx.x + (uint32_t)P.prefetch_ahead;
            const uint32_t hh2 = lin % gx, t2 = (lin / gx) % gy, b2 = lin / (gx * gy);
            if (b2 < gridDim.z) {
                const Chunks<KIND, TQ, TK> next(P, (int)t2 * TQ, key_lo, key_hi);
                ptx::tma_prefetch_4d(&map_q, 0, hh2, t2 * TQ, b2);
                if (next.n > 0 && next.start >= 0 && next.start + TK <= P.Skv1) {
                    ptx::tma_prefetch_4d(&map_k, 0, hh2, next.start, b2);
                    ptx::tma_prefetch_4d(&map_v, 0, hh2, next.start, b2);
                }
            }
        }
        if (!UPFRONT) return;
        __syncwarp();
    }

    // ---- consumer warps ----
    const int g = lane >> 2;   // row within the 8-row group
    const int tq = lane & 3;   // column pair within an 8-wide tile
    const int row0 = warp * 16;                 // first row of this warp inside the tile
    // key-coordinate position of that row (the global-row pass has no band: every key counts)
    const int p_min = KIND == kGlobalRows ? 0 : q0 + row0 + P.off1;
    const int p_max = p_min + 15;
    const uint32_t mask_span = (uint32_t)(P.mask_left + P.mask_right);

    // key range this warp's rows can attend
    const int k_lo = max(p_min - P.mask_left, key_lo);
    const int k_hi = min(p_max + P.mask_right, key_hi - 1);
    // a 16-key pair starting at key a needs no mask iff w_lo <= a <= w_hi
    const int w_lo = max(p_max - P.mask_left, key_lo);
    const int w_hi = min(p_min + P.mask_right, key_hi - 1) - 15;

    if (!ptx::mbar_wait(bar_q, 0)) {
        atomicExch(&g_flash_status, kStatusWaitTimeout);
        return;
    }
    const uint32_t q_base = ptx::smem_u32(sQ);
    const int q_row = row0 + (lane & 7) + ((lane >> 3) & 1) * 8;

    float o[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float lsum[4] = {0.f, 0.f, 0.f, 0.f};  // P * ones: [0] = row g, [2] = row g + 8 (every column alike)

    for (int c = 0; c < chunks.n; ++c) {
        const bool gathered = KIND == MAT_LONGFORMER && c >= chunks.n_seq;  // keys at global positions
        const bool side = SIDE && gathered;
        const int s = side ? 0 : c % STAGES, use = side ? 0 : c / STAGES;
        if (!ptx::mbar_wait(side ? bar_side : bar_full + s, use & 1)) {
            atomicExch(&g_flash_status, kStatusWaitTimeout);
            return;
        }
        const int kb = chunks.base(P, c);
        const uint32_t k_base = ptx::smem_u32(side ? sSide : sKV + s * kStageBytes);
        const uint32_t v_base = k_base + (side ? kSideRows : TK) * kRowBytes;
        // pairs of this chunk that intersect [k_lo, k_hi]
        int first = max(0, (k_lo - kb) >> 4);  // k_lo - kb may be negative: >> floors
        int last = k_hi >= kb ? min(TK / 16 - 1, (k_hi - kb) >> 4) : -1;
        if (gathered) {
            first = 0;
            last = (min(TK, P.n_global - (c - chunks.n_seq) * TK) - 1) >> 4;
        }
        const bool edge = kb < key_lo || kb + TK > key_hi;  // chunk reaches outside the key line

        // SINGLE: one step of exactly NP pairs (pairs past the key set are masked away, which
        // only costs work on the sequence's first and last tiles), so the step is straight-line code
        for (int pp = SINGLE ? min(first, TK / 16 - NP) : first; pp <= last; pp += SINGLE ? TK : NP) {
            const int npairs = SINGLE ? NP : min(NP, last - pp + 1);
            float sc[2 * NP][4];

            // ---- S = Q K^T over the step's pairs ----
            const int kr = 16 * pp + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t qa[4];
                ptx::ldmatrix_x4(qa, swz(q_base, q_row, 2 * ks + (lane >> 4)));
                const uint32_t k_addr = swz(k_base, kr, 2 * ks + ((lane >> 3) & 1));
#pragma unroll
                for (int j = 0; j < NP; ++j) {
                    if (j < npairs) {
                        uint32_t kf[4];
                        ptx::ldmatrix_x4(kf, k_addr + j * 16 * kRowBytes);
                        if (ks == 0) {
                            ptx::Mma<T>::run0(sc[2 * j], qa, kf[0], kf[1]);
                            ptx::Mma<T>::run0(sc[2 * j + 1], qa, kf[2], kf[3]);
                        } else {
                            ptx::Mma<T>::run(sc[2 * j], qa, kf[0], kf[1]);
                            ptx::Mma<T>::run(sc[2 * j + 1], qa, kf[2], kf[3]);
                        }
                    }
                }
            }

            // ---- mask the pairs that straddle the edge of the key set; row max ----
            float mloc[2] = {-INFINITY, -INFINITY};
            // d = j - p for element (pair 0, half 0, e = 0) of this lane, shifted so that 0 <= d + mask_left
            const int u0 = kb + 16 * pp + 2 * tq - (p_min + g) + P.mask_left;
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                if (j < npairs) {
                    const int a = kb + 16 * (pp + j);
                    if (KIND == MAT_LONGFORMER && gathered) {
                        // a gathered key counts unless the slot is unused or the row's window
                        // already holds that position
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const int2 gp = *reinterpret_cast<const int2 *>(
                                sG + s * TK + 16 * (pp + j) + 8 * half + 2 * tq);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int gk = (e & 1) ? gp.y : gp.x;
                                const int p = p_min + g + 8 * (e >> 1);
                                const bool in_window =
                                    (uint32_t)gk - (uint32_t)p + (uint32_t)P.mask_left <= mask_span;
                                if (gk == kNoKey || in_window) sc[2 * j + half][e] = -INFINITY;
                            }
                        }
                    } else if (a < w_lo || a > w_hi) {
#pragma unroll
                        for (int half = 0; half < 2; ++half)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int du = u0 + 16 * j + 8 * half + (e & 1) - 8 * (e >> 1);
                                bool ok = (uint32_t)du <= mask_span;
                                if (edge) {
                                    const int key = a + 8 * half + 2 * tq + (e & 1);
                                    ok = ok && key >= key_lo && key < key_hi;
                                }
                                if (!ok) sc[2 * j + half][e] = -INFINITY;
                            }
                    }
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        mloc[0] = fmaxf(mloc[0], fmaxf(sc[2 * j + half][0], sc[2 * j + half][1]));
                        mloc[1] = fmaxf(mloc[1], fmaxf(sc[2 * j + half][2], sc[2 * j + half][3]));
                    }
                }
            }
            float m_use[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mloc[i] = fmaxf(mloc[i], __shfl_xor_sync(0xffffffffu, mloc[i], 1));
                mloc[i] = fmaxf(mloc[i], __shfl_xor_sync(0xffffffffu, mloc[i], 2));
                if (SINGLE) {
                    m_use[i] = mloc[i] == -INFINITY ? 0.f : mloc[i] * P.sl2;
                } else {
                    const float m_new = fmaxf(m_run[i], mloc[i]);
                    const float mu = m_new == -INFINITY ? 0.f : m_new;
                    const float alpha = ptx::ex2((m_run[i] - mu) * P.sl2);
                    m_run[i] = m_new;
                    lsum[2 * i] *= alpha;
#pragma unroll
                    for (int n = 0; n < 8; ++n) {
                        o[n][2 * i] *= alpha;
                        o[n][2 * i + 1] *= alpha;
                    }
                    m_use[i] = mu * P.sl2;
                }
            }

            // ---- P = exp2(S*sl2 - m), O += P V ----
            const int vr = 16 * pp + (lane & 7) + ((lane >> 3) & 1) * 8;
            const uint32_t v_addr0 = swz(v_base, vr, lane >> 4);
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                if (j < npairs) {
                    // exp2 on packed 16-bit pairs: the argument is rounded to the operand type first
                    // (error in a weight <= |x| * 2^x * 2^-9, i.e. < 1e-3 of the row maximum), and the
                    // row sums come out of the tensor core as P times a column of ones, so the
                    // normaliser is the sum of exactly the weights that multiply V.
                    uint32_t pa[4];
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const float x0 = fmaf(sc[2 * j + half][0], P.sl2, -m_use[0]);
                        const float x1 = fmaf(sc[2 * j + half][1], P.sl2, -m_use[0]);
                        const float x2 = fmaf(sc[2 * j + half][2], P.sl2, -m_use[1]);
                        const float x3 = fmaf(sc[2 * j + half][3], P.sl2, -m_use[1]);
                        pa[2 * half] = ptx::Mma<T>::ex2_packed(ptx::Mma<T>::pack(x0, x1));
                        pa[2 * half + 1] = ptx::Mma<T>::ex2_packed(ptx::Mma<T>::pack(x2, x3));
                    }
                    if (SINGLE && j == 0) ptx::Mma<T>::run0(lsum, pa, ptx::Mma<T>::kOnes, ptx::Mma<T>::kOnes);
                    else ptx::Mma<T>::run(lsum, pa, ptx::Mma<T>::kOnes, ptx::Mma<T>::kOnes);
#pragma unroll
                    for (int dp = 0; dp < 4; ++dp) {
                        uint32_t vf[4];
                        // the 16-byte column index 2*dp + (lane>>4) xor (row&7): xor distributes over the even part
                        ptx::ldmatrix_x4_trans(vf, (v_addr0 ^ (uint32_t)(dp << 5)) + j * 16 * kRowBytes);
                        if (SINGLE && j == 0) {
                            ptx::Mma<T>::run0(o[2 * dp], pa, vf[0], vf[1]);
                            ptx::Mma<T>::run0(o[2 * dp + 1], pa, vf[2], vf[3]);
                        } else {
                            ptx::Mma<T>::run(o[2 * dp], pa, vf[0], vf[1]);
                            ptx::Mma<T>::run(o[2 * dp + 1], pa, vf[2], vf[3]);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0 && !side) ptx::mbar_arrive(bar_empty + s);
    }

    if (KIND == kGlobalRows) {
        // ---- epilogue of the global-row pass: leave (max, sum, unnormalised output) per row ----
        float *part = P.partial +
                      ((((int64_t)b * P.HH + hh) * P.n_splits + split) * P.ng_pad + q0 + row0) * kPartialStride;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = g + 8 * i;
            if (q0 + row0 + r >= P.n_global) continue;
            float *pr = part + r * kPartialStride;
            if (tq == 0) {
                pr[0] = m_run[i];
                pr[1] = lsum[2 * i];
            }
#pragma unroll
            for (int n = 0; n < 8; ++n)
                *reinterpret_cast<float2 *>(pr + 2 + 8 * n + 2 * tq) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
        }
        return;
    }

    // ---- epilogue: normalise, stage the warp's 16 rows in its own Q rows, bulk store ----
    float l_run[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) l_run[i] = lsum[2 * i] > 0.f ? __frcp_rn(lsum[2 * i]) : 0.f;
    __syncwarp();  // every lane has finished reading Q before the rows are overwritten
    {
        uint8_t *so = sQ + row0 * kRowBytes;
        // element (row g + 8i, columns 8n + 2tq..) sits in 16-byte column n ^ g of its row
        const uint32_t so_lane = ptx::smem_u32(so) + g * kRowBytes + (g << 4) + tq * 4;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t v = ptx::Mma<T>::pack(o[n][2 * i] * l_run[i], o[n][2 * i + 1] * l_run[i]);
                asm volatile("st.shared.b32 [%0], %1;" ::"r"((so_lane ^ (uint32_t)(n << 4)) + i * 8 * kRowBytes), "r"(v)
                             : "memory");
            }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && q0 + row0 < P.Sq1) {
            ptx::tma_store_4d(&map_o, so, 0, hh, q0 + row0, b);
            ptx::tma_store_commit();
            ptx::tma_store_wait_read();
        }
    }
}

// Copies the K and V rows at the global positions into dense [B, n_global, HH, 64] buffers, once per
// forward, so that the tiles of the first pass fetch them with one bulk copy each.
// grid = (global position, batch), threads stride over the HH * 8 16-byte pieces of a row set.
__global__ void gather_global_rows_kernel(const uint4 *__restrict__ k, const uint4 *__restrict__ v,
                                          uint4 *__restrict__ kg, uint4 *__restrict__ vg,
                                          const int64_t *__restrict__ gidx, int n_global, int64_t S, int HH,
                                          const uint4 *__restrict__ q = nullptr, uint4 *__restrict__ qg = nullptr) {
    const int e = blockIdx.x, b = blockIdx.y;
    const int64_t row = gidx[e];
    const bool in_range = row >= 0 && row < S;   // a position outside the sequence gathers zeros, never memory
    const int64_t src = ((int64_t)b * S + (in_range ? row : 0)) * HH * 8, dst = ((int64_t)b * n_global + e) * HH * 8;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < HH * 8; i += blockDim.x) {
        kg[dst + i] = in_range ? k[src + i] : zero;
        vg[dst + i] = in_range ? v[src + i] : zero;
        if (qg) qg[dst + i] = in_range ? q[src + i] : zero;   // (callers pass q only when it has as many rows as k)
    }
}

// Combines the partials of the global-row pass and writes the rows at the global positions:
// out = sum w * acc / sum w * l with w = exp2((m - max m) * sl2), over n_outer groups (one per
// sequence shard when the key axis is spread over GPUs, else 1) of n_splits partials each.
// grid = (global position index - e_first, head, batch), 64 threads = one per output column;
// gidx[e] is the output row of global position e.
template <typename T>
__global__ void __launch_bounds__(64)
merge_global_rows_kernel(const float *__restrict__ partial, T *__restrict__ out, const int64_t *__restrict__ gidx,
                         int n_splits, int ng_pad, int HH, int64_t Sq1, float sl2, int n_outer,
                         int64_t outer_stride, int e_first) {
    const int e = e_first + blockIdx.x, hh = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
    const int64_t row = gidx[e];
    if (row < 0 || row >= Sq1) return;   // a position outside the sequence owns no output row
    const float *base = partial + (((int64_t)b * HH + hh) * n_splits * ng_pad + e) * kPartialStride;
    const int64_t split_stride = (int64_t)ng_pad * kPartialStride;
    float m = -INFINITY;
    for (int g = 0; g < n_outer; ++g)
        for (int s = 0; s < n_splits; ++s) m = fmaxf(m, base[g * outer_stride + s * split_stride]);
    float l = 0.f, acc = 0.f;
    if (m != -INFINITY)
        for (int g = 0; g < n_outer; ++g)
            for (int s = 0; s < n_splits; ++s) {
                const float *pr = base + g * outer_stride + s * split_stride;
                const float w = ptx::ex2((pr[0] - m) * sl2);
                l = fmaf(w, pr[1], l);
                acc = fmaf(w, pr[2 + d], acc);
            }
    out[((b * Sq1 + row) * HH + hh) * 64 + d] = Elem<T>::from_f(l > 0.f ? acc / l : 0.f);
}

// ---- host side ------------------------------------------------------------

PFN_cuTensorMapEncodeTiled encode_fn() {
    static PFN_cuTensorMapEncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (PFN_cuTensorMapEncodeTiled)p;
    });
    return fn;
}

// [B, S1*HH, 64] 16-bit rows seen as dims {64, HH, S1, B}; box = {64, 1, box_rows, 1}.
int make_map(CUtensorMap *m, const void *base, int dtype, int64_t HH, int64_t S1, int64_t B,
             int box_rows) {
    PFN_cuTensorMapEncodeTiled enc = encode_fn();
    if (!enc) return fail(MAT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[4] = {64, (cuuint64_t)HH, (cuuint64_t)S1, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)kRowBytes, (cuuint64_t)HH * kRowBytes,
                                   (cuuint64_t)S1 * HH * kRowBytes};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, dtype == MAT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MAT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return MAT_OK;
}

template <typename T, int KIND, int TQ, int TK, int NP, int STAGES, bool SINGLE, int MINB>
int launch_kind(const Problem &p, const FlashParams &fp_in, int64_t dil, const char *name, int64_t grid_y = -1) {
    FlashParams fp = fp_in;
    fp.n_tiles = (fp.Sq1 + TQ - 1) / TQ;   // query tiles of this instantiation's height
    CUtensorMap mq, mk, mv, mo;
    const int64_t HH = fp.HH;
    if (int rc = make_map(&mq, p.q, p.dtype, HH, p.Sq / dil, p.B, TQ)) return rc;
    if (int rc = make_map(&mk, p.k, p.dtype, HH, p.Skv / dil, p.B, TK)) return rc;
    if (int rc = make_map(&mv, p.v, p.dtype, HH, p.Skv / dil, p.B, TK)) return rc;
    if (int rc = make_map(&mo, p.o, p.dtype, HH, p.Sq / dil, p.B, 16)) return rc;
    PeerMaps pm;
    if (int rc = make_map(&pm.k_own, p.k, p.dtype, HH, p.Skv / dil, p.B, 16)) return rc;
    if (int rc = make_map(&pm.v_own, p.v, p.dtype, HH, p.Skv / dil, p.B, 16)) return rc;
    pm.k_prev = pm.k_next = pm.k_own;
    pm.v_prev = pm.v_next = pm.v_own;
    if (p.k_prev) {
        if (int rc = make_map(&pm.k_prev, p.k_prev, p.dtype, HH, p.S_prev / dil, p.B, 16)) return rc;
        if (int rc = make_map(&pm.v_prev, p.v_prev, p.dtype, HH, p.S_prev / dil, p.B, 16)) return rc;
    }
    if (p.k_next) {
        if (int rc = make_map(&pm.k_next, p.k_next, p.dtype, HH, p.S_next / dil, p.B, 16)) return rc;
        if (int rc = make_map(&pm.v_next, p.v_next, p.dtype, HH, p.S_next / dil, p.B, 16)) return rc;
    }
    pm.q_row = pm.k_row = pm.k_own;
    pm.v_row = pm.v_own;
    constexpr bool SIDE = KIND == MAT_LONGFORMER && STAGES == 1;
    if (KIND == MAT_LONGFORMER && fp.kg) {
        if (int rc = make_map(&pm.k_row, fp.kg, p.dtype, HH, fp.n_global, p.B, SIDE ? kSideRows : TK)) return rc;
        if (int rc = make_map(&pm.v_row, fp.vg, p.dtype, HH, fp.n_global, p.B, SIDE ? kSideRows : TK)) return rc;
    } else if (KIND == MAT_LONGFORMER || KIND == kGlobalRows) {
        if (int rc = make_map(&pm.q_row, p.q, p.dtype, HH, p.Sq / dil, p.B, 1)) return rc;
        if (int rc = make_map(&pm.k_row, p.k, p.dtype, HH, p.Skv / dil, p.B, 1)) return rc;
        if (int rc = make_map(&pm.v_row, p.v, p.dtype, HH, p.Skv / dil, p.B, 1)) return rc;
    }
    auto kern = flash_fwd_kernel<T, KIND, TQ, TK, NP, STAGES, SINGLE, MINB>;
    constexpr size_t smem = flash_smem_bytes<TQ, TK, STAGES, KIND == MAT_LONGFORMER && STAGES == 1>();
    if (int rc = ensure_dynamic_smem((const void *)kern, smem, "cudaFuncSetAttribute(flash_fwd_kernel)")) return rc;
    const dim3 grid((unsigned)HH, (unsigned)(grid_y >= 0 ? grid_y : fp.n_tiles), (unsigned)p.B);
    kern<<<grid, flash_threads<TQ, SINGLE || STAGES == 1>(), smem, p.stream>>>(mq, mk, mv, mo, pm, fp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "flash_fwd_kernel launch");
    note_kernel(name);
    return MAT_OK;
}

// How the global-row pass cuts the key axis: enough CTAs to fill the GPU a few times over,
// splits a multiple of the 128-key stage, at least 512 keys each.
struct GlobalRowPlan {
    int tiles;      // 64-row tiles of the global-position list
    int n_splits, split_len;
    size_t bytes;   // partial buffer
};

GlobalRowPlan plan_global_rows(const Problem &p) {
    GlobalRowPlan g;
    g.tiles = (int)((p.pat.n_global + 63) / 64);
    const int64_t units = std::max<int64_t>(1, p.B * p.H * g.tiles);
    int64_t want = std::max<int64_t>(1, 2048 / units);
    int64_t len = (p.Skv + want - 1) / want;
    len = std::max<int64_t>(512, (len + 127) / 128 * 128);
    g.split_len = (int)len;
    g.n_splits = (int)((p.Skv + len - 1) / len);
    g.bytes = (size_t)p.B * p.H * g.n_splits * g.tiles * 64 * kPartialStride * sizeof(float);
    return g;
}

// CTAs between a tile and the one prefetched for it: half of the CTAs resident on the whole GPU
// (5 per SM).  Measured on the 64K-token window workload: 49.1 us without prefetch, 46.1 us for
// any distance from 1.5 to 3.5 CTAs per SM, slower again beyond 5 per SM (the lines are evicted
// or arrive too early).  MAT_PREFETCH_AHEAD overrides it (0 switches the prefetch off).
int prefetch_distance() {
    static int dist = -1;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *env = std::getenv("MAT_PREFETCH_AHEAD");
        if (env) { dist = std::atoi(env); return; }
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        dist = 5 * sms / 2;
    });
    return dist;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
// workspace layout of a Longformer forward: [partials of the global rows][K at globals][V at globals][Q at globals]
size_t partial_region_bytes(const Problem &p) {
    return align256(std::max({plan_global_rows(p).bytes, plan_umma_global_rows(p).bytes,
                              umma_band_longformer_partial_bytes(p)}));
}
size_t gathered_region_bytes(const Problem &p) { return align256((size_t)p.B * p.pat.n_global * p.H * kRowBytes); }

bool use_mma_global_rows() {
    const char *force = std::getenv("MAT_GLOBAL_ROWS_KERNEL");
    return force && force[0] == 'm';
}

template <typename T>
int launch_t(const Problem &p) {
    constexpr int TQ = 64;
    const int64_t dil = p.pat.kind == MAT_WINDOW ? p.pat.dilation : 1;
    FlashParams fp;
    fp.Sq1 = (int32_t)(p.Sq / dil);
    fp.Skv1 = (int32_t)(p.Skv / dil);
    fp.off1 = (int32_t)(p.pat.q_offset / dil);
    fp.n_tiles = (fp.Sq1 + TQ - 1) / TQ;
    fp.prefetch_ahead = prefetch_distance();
    fp.prev_rows = p.k_prev ? (int32_t)(p.S_prev / dil) : 0;
    fp.next_rows = p.k_next ? (int32_t)(p.S_next / dil) : 0;
    fp.key_lo = -fp.prev_rows;
    fp.key_hi = fp.Skv1 + fp.next_rows;
    fp.HH = (int32_t)(p.H * dil);
    fp.sl2 = p.scale * 1.4426950408889634f;
    fp.block = (int32_t)p.pat.block;
    fp.per_blk = fp.block / 64;
    fp.n_qblocks = p.pat.n_qblocks;
    fp.rowptr = p.pat.rowptr;
    fp.colidx = p.pat.colidx;
    fp.n_global = 0;
    fp.gidx = nullptr;
    fp.split_len = fp.n_splits = fp.ng_pad = 0;
    fp.partial = nullptr;
    fp.kg = fp.vg = nullptr;
    if (p.pat.kind == MAT_WINDOW) {
        fp.left = fp.mask_left = (int32_t)std::min<int64_t>(p.pat.left, fp.Skv1 + fp.prev_rows);
        fp.right = fp.mask_right = (int32_t)std::min<int64_t>(p.pat.right, fp.Skv1 + fp.next_rows);
        // one stage holds the tile's whole window when TQ + left (rounded up to 16, plus the
        // misalignment of the shard offset) + right fits TQ + 64 keys
        const int mis = fp.off1 & 15;
        // chunk 0 starts at the tile's first key rounded down to 16: that slack adds to the span
        const int slack = (((mis - fp.left) % 16) + 16) % 16;
        const int pairs = (fp.left + 15) / 16 + (15 + fp.right) / 16 + 1 + (mis ? 1 : 0);
        if (fp.left + slack + fp.right <= 64 && pairs <= 3)
            return launch_kind<T, MAT_WINDOW, TQ, TQ + 64, 3, 1, true, 5>(p, fp, dil, "mma_window");
        if (fp.left + slack + fp.right <= 64 && pairs <= 5)
            return launch_kind<T, MAT_WINDOW, TQ, TQ + 64, 5, 1, true, 5>(p, fp, dil, "mma_window");
        // up to 128 keys of reach (the reference's default window of +-64): still one softmax step per
        // warp over nine pairs of a 192-key stage (86 us at the 64K-token shape, 156 registers, 3 CTAs/SM)
        if (fp.left + slack + fp.right <= 128 && pairs <= 9)
            return launch_kind<T, MAT_WINDOW, TQ, TQ + 128, 9, 1, true, 3>(p, fp, dil, "mma_window");
        // the same reach on a shard offset that costs a tenth pair: 128-row tiles whose 256-key window
        // is one stage, two softmax steps per warp, no producer warp (102 us; 125 us on the ring path)
        if (fp.left + slack + fp.right <= 128 && (p.Sq / dil + 127) / 128 <= 65535)
            return launch_kind<T, MAT_WINDOW, 128, 256, 5, 1, false, 2>(p, fp, dil, "mma_window");
        return launch_kind<T, MAT_WINDOW, TQ, 128, 4, 2, false, 3>(p, fp, dil, "mma_window");
    }
    if (p.pat.kind == MAT_LONGFORMER) {
        fp.left = fp.mask_left = (int32_t)std::min<int64_t>(p.pat.left, fp.Skv1 + fp.prev_rows);
        fp.right = fp.mask_right = (int32_t)std::min<int64_t>(p.pat.right, fp.Skv1 + fp.next_rows);
        fp.n_global = (int32_t)p.pat.n_global;
        fp.gidx = p.pat.gidx;
        bool fold = false;       // the band kernel's first pass also accumulates the rows AT the global positions
        uint8_t *qg = nullptr;   // the Q rows there
        if (p.shard_kg) {
            // one shard of a sequence spread over GPUs: the caller gathered the K/V rows at ALL global
            // positions (gidx holds their positions relative to this shard's first row); only the first
            // pass runs here, the rows at global positions are finished by the partial / merge calls
            fp.kg = p.shard_kg;
            fp.vg = p.shard_vg;
        } else if (fp.n_global > 0) {
            // pass 0: the K/V rows at the global positions, gathered once behind the partials
            const size_t part = partial_region_bytes(p);
            const size_t gbytes = gathered_region_bytes(p);
            uint8_t *kg = (uint8_t *)p.workspace + part, *vg = kg + gbytes;
            fold = umma_band_longformer_supports(p) && umma_band_longformer_lanes(p) > 0;
            qg = fold ? vg + gbytes : nullptr;
            gather_global_rows_kernel<<<dim3((unsigned)fp.n_global, (unsigned)p.B), 128, 0, p.stream>>>(
                (const uint4 *)p.k, (const uint4 *)p.v, (uint4 *)kg, (uint4 *)vg, fp.gidx, fp.n_global, p.Skv,
                fp.HH, fold ? (const uint4 *)p.q : nullptr, (uint4 *)qg);
            cudaError_t e0 = cudaGetLastError();
            if (e0 != cudaSuccess) return cuda_fail(e0, "gather_global_rows_kernel launch");
            fp.kg = kg;
            fp.vg = vg;
        }
        // pass 1: every row over its window plus the keys at the global positions.  Windows that
        // reach at most 128 keys with at most 64 global positions (the +-64 / 32-token configuration):
        // 128-row tiles, the whole window in one stage, the gathered keys in a side region, no
        // producer warp; otherwise the ring of stages
        const bool one_stage = fp.left + ((16 - fp.left % 16) % 16) + fp.right <= 128 && fp.n_global <= kSideRows &&
                               (fp.n_global == 0 || fp.kg) && (fp.Sq1 + 127) / 128 <= 65535;
        if (fp.kg && !p.shard_kg && umma_band_longformer_supports(p)) {
            // at most 32 global positions and a window of at most 128 taps: the persistent tcgen05 band kernel,
            // 96 query rows per item against 224 window keys and the gathered keys
            // (fold: rows 96..127 of every query tile are the queries at the global positions; their partials, one
            // per lane of CTAs, go through the merge kernel like the splits of the separate pass)
            if (int rc = launch_umma_band_longformer(p, fp.kg, fp.vg, qg, fold ? (float *)p.workspace : nullptr)) return rc;
            if (fold) {
                const dim3 grid_m((unsigned)fp.n_global, (unsigned)fp.HH, (unsigned)p.B);
                merge_global_rows_kernel<T><<<grid_m, 64, 0, p.stream>>>((const float *)p.workspace, (T *)p.o, fp.gidx,
                                                                        umma_band_longformer_lanes(p), 32, fp.HH, fp.Sq1,
                                                                        fp.sl2, 1, 0, 0);
                cudaError_t e2 = cudaGetLastError();
                return e2 == cudaSuccess ? MAT_OK : cuda_fail(e2, "merge_global_rows_kernel launch");
            }
        } else if (one_stage) {
            if (int rc = launch_kind<T, MAT_LONGFORMER, 128, 256, 5, 1, false, 2>(p, fp, dil, "mma_longformer")) return rc;
        } else if (int rc = launch_kind<T, MAT_LONGFORMER, TQ, 128, 4, 2, false, 3>(p, fp, dil, "mma_longformer")) return rc;
        if (fp.n_global == 0 || p.shard_kg) return MAT_OK;
        // pass 2: the rows AT the global positions over every key, split along the key axis:
        // on tcgen05 (128 gathered rows per CTA) unless MAT_GLOBAL_ROWS_KERNEL=mma asks for the
        // warp-level kernel (debugging aid)
        if (!use_mma_global_rows()) {
            const GlobalRowSplit u = plan_umma_global_rows(p);
            if (int rc = launch_umma_global_rows(p, u, (float *)p.workspace)) return rc;
            const dim3 grid_m((unsigned)fp.n_global, (unsigned)fp.HH, (unsigned)p.B);
            merge_global_rows_kernel<T><<<grid_m, 64, 0, p.stream>>>((const float *)p.workspace, (T *)p.o, fp.gidx,
                                                                    u.n_splits, u.ng_pad, fp.HH, fp.Sq1, fp.sl2, 1, 0, 0);
            cudaError_t e2 = cudaGetLastError();
            return e2 == cudaSuccess ? MAT_OK : cuda_fail(e2, "merge_global_rows_kernel launch");
        }
        const GlobalRowPlan g = plan_global_rows(p);
        fp.left = fp.right = 0;
        fp.mask_left = fp.mask_right = kBig;
        fp.n_splits = g.n_splits;
        fp.split_len = g.split_len;
        fp.ng_pad = g.tiles * 64;
        fp.partial = (float *)p.workspace;
        if (int rc = launch_kind<T, kGlobalRows, TQ, 128, 4, 2, false, 3>(p, fp, dil, "mma_longformer",
                                                                         (int64_t)g.tiles * g.n_splits))
            return rc;
        // pass 3: merge the splits and overwrite those rows of the output
        const dim3 grid((unsigned)fp.n_global, (unsigned)fp.HH, (unsigned)p.B);
        merge_global_rows_kernel<T><<<grid, 64, 0, p.stream>>>(fp.partial, (T *)p.o, fp.gidx, fp.n_splits,
                                                              fp.ng_pad, fp.HH, fp.Sq1, fp.sl2, 1, 0, 0);
        cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? MAT_OK : cuda_fail(e, "merge_global_rows_kernel launch");
    }
    fp.left = fp.right = 0;
    fp.mask_left = kBig;
    fp.mask_right = p.pat.causal ? 0 : kBig;
    return launch_kind<T, MAT_BLOCK, TQ, 64, 4, 3, false, 3>(p, fp, dil, "mma_block");
}

}  // namespace

bool mma_flash_supports(const Problem &p) {
    if (p.dtype != MAT_BF16 && p.dtype != MAT_F16) return false;
    if (p.D != 64) return false;
    const uintptr_t al = (uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o;
    if (al % 16) return false;
    if (p.Skv >= (1LL << 28) || p.B > 65535) return false;
    {   // grid.y carries the query tiles
        const int64_t dil = p.pat.kind == MAT_WINDOW ? p.pat.dilation : 1;
        if ((p.Sq / dil + 63) / 64 > 65535) return false;
    }
    if (p.pat.kind == MAT_WINDOW) {
        const int64_t dil = p.pat.dilation;
        if (p.Sq % dil || p.Skv % dil || p.pat.q_offset % dil) return false;
        if (p.H * dil >= (1LL << 31)) return false;
        return true;
    }
    if (p.pat.kind == MAT_BLOCK) {
        // query tiles of 64 rows must not straddle a layout row
        return p.pat.block % 64 == 0 && p.pat.q_offset % 64 == 0 && p.pat.block < (1 << 24);
    }
    if (p.pat.kind == MAT_LONGFORMER) {
        // whole sequences only (the global rows need every key); the list of global positions
        // must fit the grid of the merge kernel
        return p.pat.q_offset == 0 && p.Sq == p.Skv && p.pat.n_global <= 65535 * 64 && p.H <= 65535;
    }
    return false;
}

size_t mma_flash_workspace_bytes(const Problem &p) {
    if (p.pat.kind != MAT_LONGFORMER || p.pat.n_global == 0) return 0;
    return partial_region_bytes(p) + 3 * gathered_region_bytes(p);
}

int launch_mma_flash(const Problem &p) {
    return p.dtype == MAT_BF16 ? launch_t<__nv_bfloat16>(p) : launch_t<__half>(p);
}

// ---- Longformer forward for callers that cannot allocate device memory ----------------------
//
// Some hosts of this library may never call cudaMalloc once they are running: an inference
// server that hands all of HBM to its own arena at start-up, or a latency-critical loop where
// the implicit device synchronisation of an allocation is not acceptable.  They cannot provide
// the workspace mat_sparse_attn_fwd asks for either, if every byte they own is already spoken
// for.  For them the per-split partials of the global-row pass live in this fixed array, which
// every GPU that loads the library holds until the process exits.
constexpr size_t kStaticScratchBytes = (size_t)4 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {

// In host code g_static_scratch is only a stand-in for the symbol, not a device address: the
// address on the current device comes from cudaGetSymbolAddress, looked up once per device.
int static_scratch_on_current_device(float **out) {
    static std::mutex mu;
    static void *ptrs[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(MAT_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        ptrs[dev] = p;
    }
    *out = (float *)ptrs[dev];
    return MAT_OK;
}

// Same three passes as the MAT_LONGFORMER branch of launch_t, with the key axis cut into as
// many splits as the fixed array can hold partials for.
template <typename T>
int launch_longformer_static(const Problem &p, float *scratch) {
    constexpr int TQ = 64;
    // every refusal comes before the first launch: a call that is turned away has enqueued nothing
    // and leaves the caller's output untouched
    const int tiles = (int)((p.pat.n_global + 63) / 64);
    const size_t per_split = (size_t)p.B * p.H * tiles * 64 * kPartialStride * sizeof(float);
    if (per_split > kStaticScratchBytes)
        return fail(MAT_ERR_UNSUPPORTED,
                    "B*H*global rows = %lld*%lld*%d needs %zu bytes of partials even unsplit; the built-in "
                    "scratch holds %zu: use mat_sparse_attn_fwd with a workspace",
                    (long long)p.B, (long long)p.H, tiles * 64, per_split, kStaticScratchBytes);
    FlashParams fp;
    fp.Sq1 = (int32_t)p.Sq;
    fp.Skv1 = (int32_t)p.Skv;
    fp.off1 = 0;
    fp.n_tiles = (fp.Sq1 + TQ - 1) / TQ;
    fp.prefetch_ahead = 0;
    fp.prev_rows = fp.next_rows = 0;
    fp.key_lo = 0;
    fp.key_hi = fp.Skv1;
    fp.HH = (int32_t)p.H;
    fp.sl2 = p.scale * 1.4426950408889634f;
    fp.block = fp.per_blk = 0;
    fp.n_qblocks = 0;
    fp.rowptr = fp.colidx = nullptr;
    fp.left = fp.mask_left = (int32_t)std::min<int64_t>(p.pat.left, fp.Skv1);
    fp.right = fp.mask_right = (int32_t)std::min<int64_t>(p.pat.right, fp.Skv1);
    fp.n_global = (int32_t)p.pat.n_global;
    fp.gidx = p.pat.gidx;
    fp.split_len = fp.n_splits = fp.ng_pad = 0;
    fp.partial = nullptr;
    fp.kg = fp.vg = nullptr;   // no workspace here: every tile gathers the global rows itself
    if (int rc = launch_kind<T, MAT_LONGFORMER, TQ, 128, 4, 2, false, 3>(p, fp, 1, "mma_longformer_static")) return rc;
    if (fp.n_global == 0) return MAT_OK;

    const GlobalRowPlan want = plan_global_rows(p);
    int64_t n_splits = std::min<int64_t>(want.n_splits, (int64_t)(kStaticScratchBytes / per_split));
    int64_t len = (p.Skv + n_splits - 1) / n_splits;
    len = std::max<int64_t>(512, (len + 127) / 128 * 128);
    fp.split_len = (int32_t)len;
    fp.n_splits = (int32_t)((p.Skv + len - 1) / len);
    fp.ng_pad = tiles * 64;
    fp.partial = scratch;
    fp.left = fp.right = 0;
    fp.mask_left = fp.mask_right = kBig;
    if (int rc = launch_kind<T, kGlobalRows, TQ, 128, 4, 2, false, 3>(p, fp, 1, "mma_longformer_static",
                                                                     (int64_t)tiles * fp.n_splits))
        return rc;
    const dim3 grid((unsigned)fp.n_global, (unsigned)fp.HH, (unsigned)p.B);
    merge_global_rows_kernel<T><<<grid, 64, 0, p.stream>>>(fp.partial, (T *)p.o, fp.gidx, fp.n_splits, fp.ng_pad,
                                                          fp.HH, fp.Sq1, fp.sl2, 1, 0, 0);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, "merge_global_rows_kernel launch");
}

}  // namespace

int launch_longformer_noalloc(const Problem &p) {
    if (p.pat.kind != MAT_LONGFORMER)
        return fail(MAT_ERR_UNSUPPORTED, "the allocation-free entry point serves MAT_LONGFORMER patterns only");
    if (!mma_flash_supports(p))
        return fail(MAT_ERR_UNSUPPORTED,
                    "the allocation-free entry point needs 16-bit inputs, head width 64, q_offset 0 and S_q = S_kv");
    float *scratch = nullptr;
    if (int rc = static_scratch_on_current_device(&scratch)) return rc;
    return p.dtype == MAT_BF16 ? launch_longformer_static<__nv_bfloat16>(p, scratch)
                               : launch_longformer_static<__half>(p, scratch);
}

int make_row_tensor_map(CUtensorMap *m, const void *base, int dtype, int64_t HH, int64_t S1, int64_t B,
                        int box_rows) {
    return make_map(m, base, dtype, HH, S1, B, box_rows);
}

int make_row_tensor_map5(CUtensorMap *m, const void *base, int dtype, int64_t H, int64_t dil, int64_t S1, int64_t B,
                         int box_rows, int64_t token_stride_bytes) {
    PFN_cuTensorMapEncodeTiled enc = encode_fn();
    if (!enc) return fail(MAT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t ts = (cuuint64_t)token_stride_bytes;
    const cuuint64_t dims[5] = {64, (cuuint64_t)H, (cuuint64_t)dil, (cuuint64_t)S1, (cuuint64_t)B};
    const cuuint64_t strides[4] = {(cuuint64_t)kRowBytes, ts, (cuuint64_t)dil * ts, (cuuint64_t)S1 * dil * ts};
    const cuuint32_t box[5] = {64, 1, 1, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = enc(m, dtype == MAT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     5, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MAT_ERR_CUDA, "cuTensorMapEncodeTiled (5-D) failed with code %d", (int)r);
    return MAT_OK;
}

int flash_status_read_and_clear(int *out) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(out, g_flash_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_flash_status, &zero, sizeof(int));
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, "reading the kernel status word");
}

}  // namespace mat

// Allocation-free Longformer forward (declared in include/mat_sparse_attn.h).  Neither this
// function nor anything it calls allocates or frees device memory.
extern "C" int mat_sparse_attn_fwd_longformer_noalloc(const void *q, const void *k, const void *v, void *o,
                                                      int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                                                      const mat_pattern_spec *spec, float scale, void *stream) {
    mat::Problem p;
    if (int rc = mat::make_problem(p, q, k, v, o, B, S, S, H, D, dtype, spec, scale, nullptr, 0, stream)) return rc;
    return mat::launch_longformer_noalloc(p);
}

// ---- Longformer over a sequence spread across GPUs: the three building blocks ----------------------

// Pass 1 of one shard: every local row over its window (halo rows read in place from the neighbour
// shards) plus the keys at all global positions (kg / vg: [B, n_global, H, 64], gathered by the
// caller across the shards).  g_pos: device array, position of each global token relative to this
// shard's first row (negative / beyond S for tokens owned by other shards).
extern "C" int mat_longformer_shard_fwd(const void *q, const void *k, const void *v, void *o, const void *k_prev,
                                        const void *v_prev, int64_t S_prev, const void *k_next,
                                        const void *v_next, int64_t S_next, const void *kg, const void *vg,
                                        const int64_t *g_pos, int64_t n_global, int64_t B, int64_t S, int64_t H,
                                        int64_t D, int dtype, int64_t left, int64_t right, float scale,
                                        void *stream) {
    using namespace mat;
    mat_pattern_spec spec = {};
    spec.kind = MAT_LONGFORMER;
    spec.left = left;
    spec.right = right;
    spec.dilation = 1;
    spec.n_global = n_global;
    spec.global_idx = g_pos;
    Problem p;
    if (int rc = make_problem(p, q, k, v, o, B, S, S, H, D, dtype, &spec, scale, nullptr, 0, stream)) return rc;
    if (n_global > 0 && (!kg || !vg || !g_pos)) return fail(MAT_ERR_INVALID, "gathered global rows missing");
    if (!mma_flash_supports(p))
        return fail(MAT_ERR_UNSUPPORTED, "the sharded Longformer pass needs 16-bit inputs and head width 64");
    if ((k_prev == nullptr) != (v_prev == nullptr) || (k_next == nullptr) != (v_next == nullptr))
        return fail(MAT_ERR_INVALID, "a neighbour needs both its K and its V");
    if (k_prev && (S_prev % 16 || left > S_prev)) return fail(MAT_ERR_INVALID, "S_prev must be a multiple of 16 covering the window");
    if (k_next && (S % 16 || right > S_next)) return fail(MAT_ERR_INVALID, "S must be a multiple of 16 and S_next cover the window");
    p.k_prev = k_prev; p.v_prev = v_prev; p.S_prev = k_prev ? S_prev : 0;
    p.k_next = k_next; p.v_next = v_next; p.S_next = k_next ? S_next : 0;
    p.shard_kg = n_global > 0 ? kg : nullptr;   // without global tokens only the window pass exists anyway
    p.shard_vg = n_global > 0 ? vg : nullptr;
    return launch_mma_flash(p);
}

// Partials of the global queries qg [B, n_global, H, 64] against one shard's keys k, v [B, S_kv, H, 64]:
// per key split and row (max, sum, unnormalised output).  The layout is reported by
// mat_global_rows_partial_layout; partial must hold that many bytes.
extern "C" size_t mat_global_rows_partial_layout(int64_t B, int64_t n_global, int64_t S_kv, int64_t H,
                                                 int32_t *n_splits_out, int32_t *ng_pad_out) {
    using namespace mat;
    Problem p;
    p.B = B; p.Sq = n_global; p.Skv = S_kv; p.H = H; p.D = 64;
    p.pat = DevPattern{};
    p.pat.n_global = n_global;
    const GlobalRowSplit g = plan_umma_global_rows(p);
    if (n_splits_out) *n_splits_out = g.n_splits;
    if (ng_pad_out) *ng_pad_out = g.ng_pad;
    return g.bytes;
}

extern "C" int mat_global_rows_partial(const void *qg, const void *k, const void *v, void *partial, int64_t B,
                                       int64_t n_global, int64_t S_kv, int64_t H, int64_t D, int dtype,
                                       float scale, void *stream) {
    using namespace mat;
    if (D != 64 || (dtype != MAT_BF16 && dtype != MAT_F16))
        return fail(MAT_ERR_UNSUPPORTED, "the global-row pass needs 16-bit inputs and head width 64");
    if (!qg || !k || !v || !partial || B <= 0 || n_global <= 0 || S_kv <= 0 || H <= 0)
        return fail(MAT_ERR_INVALID, "bad argument");
    Problem p;
    p.q = qg; p.k = k; p.v = v; p.o = nullptr;
    p.B = B; p.Sq = n_global; p.Skv = S_kv; p.H = H; p.D = D;
    p.dtype = dtype;
    p.scale = scale > 0.f ? scale : 0.125f;
    p.pat = DevPattern{};
    p.pat.kind = MAT_LONGFORMER;
    p.pat.n_global = n_global;
    p.pat.gidx = nullptr;   // the queries are already gathered: row e of qg is global token e
    p.workspace = nullptr; p.workspace_bytes = 0;
    p.stream = (cudaStream_t)stream;
    return launch_umma_global_rows(p, plan_umma_global_rows(p), (float *)partial);
}

// Merges n_parts partial buffers (one per shard, part_stride_floats apart) for the global tokens
// [e_first, e_first + n_rows) and writes their rows of o [B, S, H, 64] at g_pos[e] (positions
// relative to this shard: the caller passes the range of tokens the shard owns).
extern "C" int mat_global_rows_merge(const void *partials, int64_t n_parts, int64_t part_stride_floats, void *o,
                                     const int64_t *g_pos, int64_t e_first, int64_t n_rows, int64_t B, int64_t S,
                                     int64_t H, int32_t n_splits, int32_t ng_pad, int dtype, float scale,
                                     void *stream) {
    using namespace mat;
    if (n_rows <= 0) return MAT_OK;
    if (!partials || !o || !g_pos || n_parts <= 0 || B <= 0 || H <= 0 || H > 65535 || B > 65535)
        return fail(MAT_ERR_INVALID, "bad argument");
    const float sl2 = (scale > 0.f ? scale : 0.125f) * 1.4426950408889634f;
    const dim3 grid((unsigned)n_rows, (unsigned)H, (unsigned)B);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == MAT_BF16)
        merge_global_rows_kernel<__nv_bfloat16><<<grid, 64, 0, st>>>((const float *)partials, (__nv_bfloat16 *)o, g_pos,
                                                                   n_splits, ng_pad, (int)H, S, sl2, (int)n_parts,
                                                                   part_stride_floats, (int)e_first);
    else if (dtype == MAT_F16)
        merge_global_rows_kernel<__half><<<grid, 64, 0, st>>>((const float *)partials, (__half *)o, g_pos, n_splits,
                                                            ng_pad, (int)H, S, sl2, (int)n_parts, part_stride_floats,
                                                            (int)e_first);
    else
        return fail(MAT_ERR_UNSUPPORTED, "16-bit outputs only");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, "merge_global_rows_kernel launch");
}
