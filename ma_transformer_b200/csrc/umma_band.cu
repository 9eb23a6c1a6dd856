// Narrow-window forward on the 5th-generation tensor cores: a persistent kernel that runs
// both contractions of every 128-query tile as single tcgen05.mma sweeps over the tile's whole
// key band, with the accumulators in tensor memory and the operands staged by TMA.
//
// Replaces sparse_attention_forward_warp (src/cuda/sparse_attention_kernel.cu:211-263) for
// 16-bit inputs with head width 64 and windows that reach at most 128 keys
// (left + right <= 128 taps, the reference's default window_size = 64 included).
//
// Why tcgen05 for a band that is mostly mask: the warp-level mma path feeds its operands through
// ldmatrix, and at 64 taps per row the shared-memory traffic of those fragment loads (every warp
// re-reads the K/V rows its neighbours read too) is what bounds it, not HBM.  tcgen05.mma reads
// K and V from shared memory once per tile; P never touches shared memory at all (it is stored in
// tensor memory and read from there as the A operand); the scores outside the band cost tensor
// work, of which there is plenty to spare, and no memory traffic.
//
// Work decomposition
//   - A dilated window over [B,S,H,64] is a plain window over the same memory viewed as
//     [B, S/dil, dil*H, 64]; the kernel only ever sees dilation 1 and HH = dil*H heads.
//   - Work item = (batch, 128-query tile, head), heads running fastest, so the CTAs resident at
//     one time work on a short range of tokens across all heads (the 128-byte rows of a token's
//     heads leave DRAM together).  One CTA per SM; CTA c takes items c, c + G, c + 2G, ...
//   - Keys of an item: KT = 192 or 256 consecutive rows starting at the first key of the tile's
//     first row, rounded down to a multiple of 16.  Row r of the tile attends the columns
//     [r + cl, r + cl + left + right] of that range (cl = the rounding, 0..15).
//   - Warp roles: one TMA lane fills two rings of stages ({Q, K} and V, separately released);
//     one MMA lane issues S = Q K^T (4 instructions of N = KT) and [O | l] = P [V | 1]
//     (KT/16 instructions of N = 80: V widened by a block of ones, so the row sums come out of
//     the tensor core); eight softmax warps, four per TMEM slot, thread r owning query row r:
//     read the row's band of scores from TMEM, mask, maximum, exponentials, store P (16-bit
//     pairs) over the first KT/2 columns of the slot with zeros outside the band, then read the
//     finished O row and the row sum, normalise and write the output row.
//   - Two TMEM slots of 256 columns alternate between items, so the tensor core computes the
//     scores of item i + 1 and the P V product of item i - 1 while the softmax warps of the other
//     slot work on item i.  Inside a slot S (KT columns), then P (columns [0, KT/2)) and
//     [O | l] (columns [KT/2, KT/2 + 80)) reuse the same columns in turn.
//
// Every wait is bounded; a wait that runs out sets the library's status word, every role leaves
// its loop, and the CTA frees its tensor memory and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "mat_common.cuh"
#include "ptx.cuh"
#include "umma.cuh"

namespace mat {
namespace {

using namespace umma;

constexpr int kRowBytes = 128;
constexpr int kTQ = 128;          // query rows per item
constexpr int kSumN = 16;         // extra B columns of the P V product: a block of ones
constexpr int kSlotCols = 256;    // TMEM columns per slot
constexpr int kSoftmaxWarps = 8;  // four per slot
constexpr int kEpilogueWarp0 = kSoftmaxWarps + 3;   // warps 11..14: warp w reads the TMEM lanes of quarter w % 4
constexpr int kThreads = (kSoftmaxWarps + 3 + 4) * 32;   // + one MMA warp per slot + the TMA warp + four epilogue warps

__device__ int g_band_status = 0;

// Timeline of the first items of CTA 0 (build with -DMAT_BAND_TRACE; read with mat_debug_band_trace):
// slot [role][item][event] = %globaltimer at that point.  Compiled out otherwise.
#ifdef MAT_BAND_TRACE
__device__ unsigned long long g_trace[3 * 24 * 8];
#define TR(role, item, ev) do { if (blockIdx.x == 0 && (item) < 24) g_trace[((role) * 24 + (item)) * 8 + (ev)] = ptx::global_ns(); } while (0)
#else
#define TR(role, item, ev) do { } while (0)
#endif

struct BandParams {
    int32_t Sq1, Skv1, off1;       // query rows, key rows and q_offset of one sub-sequence
    int32_t key_lo, key_hi;        // keys the kernel may touch: [key_lo, 0) previous shard, [Skv1, key_hi) next shard
    int32_t prev_rows;
    int32_t left, right;
    int32_t cl;                    // column of row 0's first key inside an item's key range
    int32_t HH, n_tiles;
    int32_t H;                     // heads of the tensor itself: head hh of the kernel's view is head hh % H, residue hh / H
    uint32_t n_items;
    float sl2;                     // scale * log2(e)
    // Longformer variant: the sorted global positions; every row attends them besides its window
    int32_t n_global;
    const int64_t *gidx;
    // Longformer variant with the rows AT the global positions folded in (lanes > 0): CTA c works on head
    // c % HH only and on every lanes-th tile of it, starting at tile c / HH, batches following one another;
    // rows 96..127 of its query tile are the queries at the global positions, whose scores against the keys
    // an item owns are accumulated over the CTA's items and left in `partial`
    // ([B, HH, lanes, 32, kPartialStride]: maximum, sum, 64 unnormalised outputs) for the merge kernel.
    int32_t lanes, B;
    float *partial;
};

struct BandMaps {
    CUtensorMap q, k, v, o;                                  // boxes of 128 (q, o) and KT rows
    CUtensorMap k_own, v_own, k_prev, v_prev, k_next, v_next;   // 16-row boxes for stages that cross a shard edge
    CUtensorMap kg, vg;   // Longformer variant: the K/V rows at the global positions, [B, n_global, HH, 64], 32-row boxes
    CUtensorMap qg;       // and, with the global rows folded in, the Q rows there (q then has 96-row boxes)
};

// Longformer variant: an item is 96 query rows, its key range 224 window keys followed by the (at most 32)
// keys at the global positions, so that scores, weights and output still fit one 256-column slot and one
// tcgen05.mma of N = 256 per slice.  The tile's rows 96..127 are the queries AT the global positions (which attend
// every key): each item adds their scores against the 96 keys its own rows sit on, the epilogue warp of that
// quarter keeps the running maximum, sum and output of the 32 rows over the CTA's items in registers (a CTA stays
// on one head), and the per-CTA partials are merged by merge_global_rows_kernel.  The whole Longformer forward is
// then gather (Q, K, V at the global positions) -> this kernel -> merge, and K and V leave DRAM once.
// (Without the fold - more heads than half the SMs - rows 96..127 are the next item's and computed for nothing.)
constexpr int kLfRows = 96, kLfBand = 224, kLfGlobals = 32;
constexpr int kNoGlobal = INT32_MIN;   // unused slot of the global-position list

template <int KT> struct BandCfg {
    static constexpr int kNQK = 2;                   // {Q, K} stages
    static constexpr int kNV = KT == 192 ? 3 : 2;    // V stages (released later than K: after the P V product)
    static constexpr int kQKBytes = kTQ * kRowBytes + KT * kRowBytes;
    static constexpr int kVBytes = KT * kRowBytes;
    static constexpr int kNCH = (KT - 96) / 32;      // 32-column chunks of a warp's band: 3 or 5 (Longformer: 5 and the globals)
    // (behind the barriers: the global-position list, then per slot the 32 item maxima of the global rows)
    static constexpr int kBars = 2 * kNQK + 2 * kNV + 12 + kLfGlobals / 2 + kLfGlobals;
    static constexpr int kOutBytes = kTQ * kRowBytes;   // one output tile per slot, staged for its bulk store
    static constexpr size_t kSmemBytes = 1024 + (size_t)kNQK * kQKBytes + (size_t)kNV * kVBytes + 2 * kOutBytes +
                                         kSumN * kRowBytes + kBars * 8 + 16;
};

template <typename T, int KT, bool LF>
__global__ void __launch_bounds__(kThreads, 1)
umma_band_kernel(const __grid_constant__ BandMaps maps, const BandParams P) {
    using C = BandCfg<KT>;
    constexpr int NQK = C::kNQK, NV = C::kNV, NCH = C::kNCH;
    static_assert(!LF || KT == 256, "the Longformer variant uses the 256-column slot");
    constexpr int kRows = LF ? kLfRows : kTQ;       // query rows an item really owns
    constexpr int kBandKT = LF ? kLfBand : KT;      // key rows of the window part of a stage
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQK = smem;                                  // stage s: Q at +0 (16 KB), K behind it
    uint8_t *sV = sQK + NQK * C::kQKBytes;
    uint8_t *sOut = sV + NV * C::kVBytes;                 // slot s: its output tile, 128-byte swizzled rows
    uint8_t *sOnes = sOut + 2 * C::kOutBytes;             // 16 rows of ones
    uint64_t *bars = (uint64_t *)(sOnes + kSumN * kRowBytes);
    uint64_t *qk_full = bars, *qk_empty = qk_full + NQK, *v_full = qk_empty + NQK, *v_empty = v_full + NV;
    uint64_t *s_ready = v_empty + NV, *p_ready = s_ready + 2, *o_ready = p_ready + 2, *slot_free = o_ready + 2;
    uint64_t *out_full = slot_free + 2, *out_free = out_full + 2;   // the staged output tile of a slot
    int32_t *sG = (int32_t *)(out_free + 2);             // Longformer variant: the global positions (kNoGlobal: unused)
    float *sM = (float *)(sG + kLfGlobals);              // [slot][global row]: maximum of the row's scores in the slot's item
    uint32_t *tmem_slot = (uint32_t *)(sM + 2 * kLfGlobals);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- the TMA lane's work for item `it` of this CTA: {Q, K} and V into their rings ----
    const uint32_t G = gridDim.x, HHu = (uint32_t)P.HH, n_tiles = (uint32_t)P.n_tiles;
    const bool fold = LF && P.lanes > 0;   // the rows at the global positions ride along (see BandParams)
    const uint32_t my_lane = blockIdx.x / HHu, n_slots = (uint32_t)P.B * n_tiles;
    const uint32_t n_mine = fold ? (my_lane < (uint32_t)P.lanes && my_lane < n_slots ? (n_slots - my_lane + P.lanes - 1) / P.lanes : 0)
                                 : (blockIdx.x < P.n_items ? (P.n_items - blockIdx.x + G - 1) / G : 0);   // items of this CTA
    // item `it` of this CTA: head of the kernel's view, batch, first query row
    auto item_at = [&](uint32_t it, int &hh, int &b, int &q0) {
        if (fold) {
            const uint32_t t = my_lane + it * (uint32_t)P.lanes;
            hh = blockIdx.x % HHu;
            b = t / n_tiles;
            q0 = (int)(t % n_tiles) * kRows;
        } else {
            const uint32_t L = blockIdx.x + it * G;
            hh = L % HHu;
            b = L / (HHu * n_tiles);
            q0 = (int)((L / HHu) % n_tiles) * kRows;
        }
    };
    auto produce = [&](uint32_t it) -> bool {
        int hh, b, q0;
        item_at(it, hh, b, q0);
        const int hd = hh % P.H, rs = hh / P.H;
        const int start = (q0 + P.off1 - P.left) - P.cl;   // first key row of the item (a multiple of 16)
        const int sq = it % NQK, sv = it % NV;
        // a stage that crosses into a neighbour shard's rows is fetched 16 rows at a time, each
        // piece from the tensor that owns it
        const bool pieces = !LF && ((start < 0 && P.key_lo < 0) || (start + KT > P.Skv1 && P.key_hi > P.Skv1));
        auto load_rows = [&](uint8_t *dst, uint64_t *bar, const CUtensorMap *whole, const CUtensorMap *own,
                             const CUtensorMap *prev, const CUtensorMap *next) {
            if (!pieces) {
                ptx::tma_load_5d(dst, whole, bar, 0, hd, rs, start, b);   // (Longformer variant: a box of 224 rows)
                return;
            }
            for (int i = 0; i < KT / 16; ++i) {
                const int a = start + 16 * i;
                const CUtensorMap *m = own;
                int row = a;
                if (a < 0 && P.key_lo < 0) { m = prev; row = P.prev_rows + a; }
                else if (a >= P.Skv1 && P.key_hi > P.Skv1) { m = next; row = a - P.Skv1; }
                ptx::tma_load_5d(dst + i * 16 * kRowBytes, m, bar, 0, hd, rs, row, b);
            }
        };
        if (it >= (uint32_t)NQK && !ptx::mbar_wait(qk_empty + sq, (it / NQK - 1) & 1)) {
            atomicExch(&g_band_status, 1);
            return false;
        }
        TR(0, it, 0);
        uint8_t *dq = sQK + sq * C::kQKBytes;
        ptx::mbar_expect_tx(qk_full + sq, C::kQKBytes);
        ptx::tma_load_5d(dq, &maps.q, qk_full + sq, 0, hd, rs, q0, b);   // (fold: a box of 96 rows)
        if (fold) ptx::tma_load_5d(dq + kLfRows * kRowBytes, &maps.qg, qk_full + sq, 0, hd, rs, 0, b);
        load_rows(dq + kTQ * kRowBytes, qk_full + sq, &maps.k, &maps.k_own, &maps.k_prev, &maps.k_next);
        if (LF)   // the keys at the global positions behind the window keys (slots past the list: zeros)
            ptx::tma_load_5d(dq + (kTQ + kBandKT) * kRowBytes, &maps.kg, qk_full + sq, 0, hd, rs, 0, b);
        if (it >= (uint32_t)NV && !ptx::mbar_wait(v_empty + sv, (it / NV - 1) & 1)) {
            atomicExch(&g_band_status, 1);
            return false;
        }
        TR(0, it, 1);
        ptx::mbar_expect_tx(v_full + sv, C::kVBytes);
        load_rows(sV + sv * C::kVBytes, v_full + sv, &maps.v, &maps.v_own, &maps.v_prev, &maps.v_next);
        if (LF) ptx::tma_load_5d(sV + sv * C::kVBytes + kBandKT * kRowBytes, &maps.vg, v_full + sv, 0, hd, rs, 0, b);
        return true;
    };
    constexpr uint32_t kEarly = NQK < NV ? NQK : NV;   // items whose copies need no stage to be handed back first

    if (warp == kSoftmaxWarps + 2 && lane == 0) {
        // The TMA lane sets the barriers up itself and starts the copies of its first items at once: they are in
        // flight while the rest of the CTA allocates tensor memory and meets at the barrier below.
        for (int i = 0; i < NQK; ++i) { ptx::mbar_init(qk_full + i, 1); ptx::mbar_init(qk_empty + i, 1); }
        for (int i = 0; i < NV; ++i) { ptx::mbar_init(v_full + i, 1); ptx::mbar_init(v_empty + i, 1); }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(s_ready + i, 1);
            ptx::mbar_init(p_ready + i, 4);
            ptx::mbar_init(o_ready + i, 1);
            ptx::mbar_init(slot_free + i, 4);
            ptx::mbar_init(out_full + i, fold ? 3 : 4);   // (fold: quarter 3 stages no rows)
            ptx::mbar_init(out_free + i, 1);
        }
        ptx::fence_barrier_init();
        for (uint32_t it = 0; it < kEarly && it < n_mine; ++it) produce(it);
    }
    if (LF && threadIdx.x < kLfGlobals)
        sG[threadIdx.x] = (int)threadIdx.x < P.n_global ? (int32_t)P.gidx[threadIdx.x] : kNoGlobal;
    if (threadIdx.x < kSumN * kRowBytes / 16) {
        const uint32_t one2 = ptx::Mma<T>::kOnes;
        reinterpret_cast<uint4 *>(sOnes)[threadIdx.x] = make_uint4(one2, one2, one2, one2);
        ptx::fence_proxy_async_smem();
    }
    if (warp == kSoftmaxWarps) {
        tmem_alloc(tmem_slot, 2 * kSlotCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == kSoftmaxWarps + 2) {
        // ================= TMA lane: the items after the ones it started before the CTA was set up =================
        if (lane == 0) {
            for (uint32_t it = kEarly; it < n_mine; ++it)
                if (!produce(it)) break;
        }
    } else if (warp >= kEpilogueWarp0) {
        // ================= epilogue warps: the finished rows of every item, both slots in turn =================
        // (their own warps, so that the softmax warps of a slot go straight on to the slot's next item)
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        bool ok = true;
        if (fold && quad == 3) {
            // fold, quarter 3: lane e carries the row at global position e of the head this CTA works on: the
            // running maximum, sum and unnormalised output over the keys of the CTA's items so far in the batch
            float g_m = -INFINITY, g_l = 0.f, g_acc[64];
#pragma unroll
            for (int c = 0; c < 64; ++c) g_acc[c] = 0.f;
            int g_b = 0;   // batch the running values belong to
            auto flush_rows = [&](int b_end) {   // leaves the partial of batch g_b, and empty ones up to b_end
                for (; g_b < b_end; ++g_b) {
                    float *pr = P.partial + ((((int64_t)g_b * P.HH + blockIdx.x % HHu) * P.lanes + my_lane) * kLfGlobals + lane) * kPartialStride;
                    pr[0] = g_m;
                    pr[1] = g_l;
#pragma unroll
                    for (int c = 0; c < 64; c += 2) *reinterpret_cast<float2 *>(pr + 2 + c) = make_float2(g_acc[c], g_acc[c + 1]);
                    g_m = -INFINITY;
                    g_l = 0.f;
#pragma unroll
                    for (int c = 0; c < 64; ++c) g_acc[c] = 0.f;
                }
            };
            for (uint32_t i = 0; ok && i < n_mine; ++i) {
                const int slot = i & 1;
                int hh, b, q0;
                item_at(i, hh, b, q0);
                const uint32_t t_lane = tmem_base + slot * kSlotCols + ((uint32_t)(quad * 32) << 16);
                if (!(ok = ptx::mbar_wait(o_ready + slot, (i >> 1) & 1))) break;
                tc_fence_after();
                if (b != g_b) flush_rows(b);
                const float m_it = sM[slot * kLfGlobals + lane];   // maximum of the row's scores in this item
                const float m_new = fmaxf(g_m, m_it);
                // (an item none of whose keys the row may use: maximum -inf, weights and sum zero)
                const float a = m_new == -INFINITY ? 0.f : ptx::ex2((g_m - m_new) * P.sl2);
                const float w = m_new == -INFINITY ? 0.f : ptx::ex2((m_it - m_new) * P.sl2);
                uint32_t part[32];
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    tmem_ld32(t_lane + KT / 2 + 32 * hf, part);
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        g_acc[32 * hf + c] = fmaf(g_acc[32 * hf + c], a, w * __uint_as_float(part[c]));
                }
                tmem_ld32(t_lane + KT / 2 + 64, part);   // its first column: the row sum
                g_l = fmaf(g_l, a, w * __uint_as_float(part[0]));
                g_m = m_new;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(slot_free + slot);
            }
            if (ok) flush_rows(P.B);
            if (!ok) atomicExch(&g_band_status, 1);
        } else {
            for (uint32_t i = 0; ok && i < n_mine; ++i) {
                const int slot = i & 1;
                const uint32_t u = i >> 1;
                int hh, b, q0;
                item_at(i, hh, b, q0);
                const int hd = hh % P.H, rs = hh / P.H;
                const uint32_t t_lane = tmem_base + slot * kSlotCols + ((uint32_t)(quad * 32) << 16);
                // ---- the finished row: O and its sum ----
                if (!(ok = ptx::mbar_wait(o_ready + slot, u & 1))) break;
                tc_fence_after();
                if (r == 0) TR(2, i, 3);
                float o[64], l_run;
                tmem_ld64_and_1(t_lane + KT / 2, o, t_lane + KT / 2 + 64, l_run);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(slot_free + slot);   // the slot may take the scores of item i + 2
                // normalise, stage the tile (128-byte swizzled rows, as the bulk store expects), store it
                {
                    const float inv = l_run > 0.f ? __frcp_rn(l_run) : 0.f;
                    uint8_t *so = sOut + slot * C::kOutBytes;
                    // the bulk store of this slot's previous tile has finished reading the staging rows
                    // (every hand-over is an mbarrier with a bounded wait, never a bar.sync: a warp that gave
                    // up on a wait must not leave the others stuck)
                    if (u >= 1) {
                        if (quad == 0 && lane == 0) {
                            ptx::tma_store_wait_read();
                            ptx::mbar_arrive(out_free + slot);
                        }
                        if (!(ok = ptx::mbar_wait(out_free + slot, (u - 1) & 1))) break;
                    }
                    if (r == 0) TR(2, i, 4);
                    uint8_t *row = so + r * kRowBytes;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        uint4 v;
                        v.x = ptx::Mma<T>::pack(o[8 * q] * inv, o[8 * q + 1] * inv);
                        v.y = ptx::Mma<T>::pack(o[8 * q + 2] * inv, o[8 * q + 3] * inv);
                        v.z = ptx::Mma<T>::pack(o[8 * q + 4] * inv, o[8 * q + 5] * inv);
                        v.w = ptx::Mma<T>::pack(o[8 * q + 6] * inv, o[8 * q + 7] * inv);
                        *reinterpret_cast<uint4 *>(row + ((q ^ (r & 7)) << 4)) = v;
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(out_full + slot);
                    if (quad == 0 && lane == 0) {
                        if (!ptx::mbar_wait(out_full + slot, u & 1)) {
                            ok = false;
                        } else {
                            ptx::tma_store_5d(&maps.o, so, 0, hd, rs, q0, b);   // rows past the sequence end are clipped
                            ptx::tma_store_commit();
                        }
                        TR(2, i, 5);
                    }
                }
            }
            if (quad == 0 && lane == 0) ptx::tma_store_wait_all();
            if (!ok) atomicExch(&g_band_status, 1);
        }
    } else if (warp >= kSoftmaxWarps) {
        // ================= MMA lanes, one per slot: S(i), then [O | l](i) once the weights are stored =================
        // (two issuing lanes: an instruction costs its issuer about 125 cycles whatever its shape, and a slot's
        // 4 + KT/16 instructions per item would otherwise sit on the other slot's critical path)
        if (lane == 0) {
            const int slot = warp - kSoftmaxWarps;
            const uint32_t idesc_s = instr_desc<T>(false, KT), idesc_pv = instr_desc<T>(true, 64 + kSumN);
            const uint32_t qk_addr = ptx::smem_u32(sQK), v_addr0 = ptx::smem_u32(sV), ones_addr = ptx::smem_u32(sOnes);
            const uint32_t ts = tmem_base + slot * kSlotCols;      // S, then P in its columns [0, KT/2)
            const uint32_t td = ts + KT / 2;                       // [O | l]: 80 columns behind P
            bool ok = true;
            for (uint32_t i = slot; ok && i < n_mine; i += 2) {
                const int sq = i % NQK, sv = i % NV;
                TR(1, i, 0);
                if (!(ok = ptx::mbar_wait(qk_full + sq, (i / NQK) & 1))) break;
                TR(1, i, 1);
                // the slot's previous item (i - 2) has been read out by its softmax warps
                if (i >= 2 && !(ok = ptx::mbar_wait(slot_free + slot, ((i >> 1) - 1) & 1))) break;
                tc_fence_after();
                TR(1, i, 2);
                const uint64_t dq = smem_desc(qk_addr + sq * C::kQKBytes);
                const uint64_t dk = smem_desc(qk_addr + sq * C::kQKBytes + kTQ * kRowBytes);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   // 16 of the 64 head columns per instruction (32 bytes along a row)
                    umma_f16_ss(ts, dq + ks * 2, dk + ks * 2, idesc_s, ks > 0);
                umma_commit(s_ready + slot);
                umma_commit(qk_empty + sq);
                TR(1, i, 3);
                if (!(ok = ptx::mbar_wait(v_full + sv, (i / NV) & 1))) break;
                TR(1, i, 4);
                if (!(ok = ptx::mbar_wait(p_ready + slot, (i >> 1) & 1))) break;   // P(i) is in TMEM
                tc_fence_after();
                TR(1, i, 5);
                const uint32_t v_addr = v_addr0 + sv * C::kVBytes;
#pragma unroll
                for (int ks = 0; ks < KT / 16; ++ks) {
                    // B = 16 keys x 80 columns: the 64 head columns from the V stage, then a second 64-wide
                    // block (16 of it used) that the leading-dimension offset points at the ones
                    const uint32_t vk = v_addr + ks * 16 * kRowBytes;
                    umma_f16_ta(td, ts + ks * 8, smem_desc(vk, (ones_addr - vk) >> 4), idesc_pv, ks > 0);
                }
                umma_commit(o_ready + slot);
                umma_commit(v_empty + sv);
                TR(1, i, 6);
            }
            if (!ok) atomicExch(&g_band_status, 1);
        }
    } else {
        // ================= softmax warps: thread r owns query row r of its slot's item =================
        const int slot = warp >> 2, quad = warp & 3;
        const int r = quad * 32 + lane;
        const uint32_t t_lane = tmem_base + slot * kSlotCols + ((uint32_t)(quad * 32) << 16);
        const uint32_t span = (uint32_t)(P.left + P.right);
        // fold: quarter 3 holds the rows at the global positions, which take the keys the item's own 96 rows sit
        // on (every key belongs to exactly one item): columns left + cl ... + 95, inside the five chunks that
        // start at the chunk of column left + cl (at the third chunk when that would reach past the window keys)
        const bool grow = fold && quad == 3;
        const int pq = grow ? min(2, (P.left + P.cl) >> 5) : quad;   // first 32-column chunk of this warp's band
        const int c0 = pq * 32;
        bool ok = true;
        for (uint32_t i = slot; ok && i < n_mine; i += 2) {
            const uint32_t u = i >> 1;
            int hh_, b_, q0;
            item_at(i, hh_, b_, q0);
            const int start = (q0 + P.off1 - P.left) - P.cl;
            const bool edge = start < P.key_lo || start + kBandKT > P.key_hi;   // some columns lie outside the key line
            if (r == 0) TR(2, i, 0);
            if (!(ok = ptx::mbar_wait(s_ready + slot, u & 1))) break;
            tc_fence_after();
            if (r == 0) TR(2, i, 1);
            if (LF && quad == 3 && !fold) {
                // rows 96..127 of the tile belong to the next item: nothing to compute, their rows of P stay
                // whatever the scores left there and their output rows are never stored
                tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(p_ready + slot);
                continue;
            }
            // Columns of this row that count: its band, cut to the keys that exist.  n_ok = 0: none.
            int lo = r + P.cl, hi = r + P.cl + (int)span;
            if (grow) {
                lo = P.left + P.cl;
                hi = lo + kLfRows - 1;
            }
            if (edge || grow) {
                lo = max(lo, P.key_lo - start);
                hi = min(hi, P.key_hi - 1 - start);
            }
            const uint32_t n_ok = (uint32_t)max(0, hi - lo + 1);
            // chunk ch (columns c0 + 32 ch ...) lies inside the band of every row of this warp iff
            // 32 ch >= cl + 31 and 32 ch + 31 <= cl + span; such a chunk needs no mask
            const int ch_free_lo = (P.cl + 31 + 31) >> 5, ch_free_hi = edge || grow ? -1 : ((P.cl + (int)span - 31) >> 5);
            // mask of one 32-column chunk (skipped when the chunk lies inside every row's band), its share of
            // the row maximum, and its weights: packed two to a column and stored as P over columns [0, KT/2)
            // of this lane.  P column j holds keys 2j, 2j + 1 of the item, so the pairs of chunk ch go to the
            // 16 columns at 16 (pq + ch): always below the scores this thread has still to read.
            auto mask_chunk = [&](uint32_t (&sr)[32], int ch) {
                const int d = c0 + 32 * ch - lo;
                // (the rows at the global positions all take the same columns: a chunk inside them needs no mask either)
                if (grow ? (d < 0 || d + 31 >= (int)n_ok) : (ch < ch_free_lo || ch > ch_free_hi)) {
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if ((uint32_t)(d + e) >= n_ok) sr[e] = 0xff800000u;   // -inf
                }
            };
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            auto max_chunk = [&](const uint32_t (&sr)[32]) {
#pragma unroll
                for (int e = 0; e < 32; e += 8) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        mx[q] = max3(mx[q], __uint_as_float(sr[e + 2 * q]), __uint_as_float(sr[e + 2 * q + 1]));
                }
            };
            float mus = 0.f, m_row = -INFINITY;
            // Longformer variant: chunk NCH is the scores against the keys at the global positions (columns
            // 224..255); a slot counts unless it is unused or the row's window already holds that position
            auto mask_globals = [&](uint32_t (&sr)[32]) {
                const int p = q0 + r + P.off1;
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int gk = sG[e];
                    if (gk == kNoGlobal || (uint32_t)(gk - p + P.left) <= span || grow) sr[e] = 0xff800000u;
                }
            };
            auto weights_chunk = [&](const uint32_t (&sr)[32], int piece) {
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    float x0, x1;
                    ffma2(x0, x1, __uint_as_float(sr[2 * e]), __uint_as_float(sr[2 * e + 1]), P.sl2, -mus);
                    pk[e] = ptx::Mma<T>::ex2_packed(ptx::Mma<T>::pack(x0, x1));
                }
                tmem_st16(t_lane + 16 * piece, pk);
            };
            if constexpr (NCH == 3) {
                // the whole band of a row fits the registers: one read of the scores
                uint32_t s0[32], s1[32], s2[32];
                tmem_ld32_issue(t_lane + c0, s0);
                tmem_ld32_issue(t_lane + c0 + 32, s1);
                tmem_ld32_issue(t_lane + c0 + 64, s2);
                tmem_ld32_wait(s0);
                mask_chunk(s0, 0);
                max_chunk(s0);
                tmem_ld32_wait(s1);
                mask_chunk(s1, 1);
                max_chunk(s1);
                tmem_ld32_wait(s2);
                if (r == 0) TR(0, i, 2);
                mask_chunk(s2, 2);
                max_chunk(s2);
                m_row = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                mus = (m_row == -INFINITY ? 0.f : m_row) * P.sl2;
                if (r == 0) TR(0, i, 3);
                weights_chunk(s0, pq);
                weights_chunk(s1, pq + 1);
                weights_chunk(s2, pq + 2);
                if (r == 0) TR(0, i, 4);
            } else {
                // Two passes over the scores with three register buffers.  Every tcgen05.wait::ld covers all
                // loads in flight, so the chunks are fetched in groups whose latency is paid once per group:
                // pass 1 takes the high chunks first and ends on the low ones, which then stay in registers
                // (masked) for pass 2; pass 2 goes upward, as the P stores must (a chunk's weights land on
                // columns below every score still to be read), and re-reads only the high chunks.
                constexpr int NC = LF ? NCH + 1 : NCH;   // the Longformer variant's last chunk: the global keys
                constexpr int NL = NC - 3;               // low chunks 0..NL-1, high chunks NL..NC-1 (three of them)
                static_assert(NL >= 1 && NL <= 3, "three buffers hold either group");
                auto ccol = [&](int ch) { return LF && ch == NCH ? kLfBand : c0 + 32 * ch; };
                auto piece_of = [&](int ch) { return LF && ch == NCH ? kLfBand / 32 : pq + ch; };
                auto mask_any = [&](uint32_t (&sr)[32], int ch) {
                    if (LF && ch == NCH) mask_globals(sr);
                    else mask_chunk(sr, ch);
                };
                uint32_t b0[32], b1[32], b2[32];
                tmem_ld32_issue(t_lane + ccol(NL), b0);
                tmem_ld32_issue(t_lane + ccol(NL + 1), b1);
                tmem_ld32_issue(t_lane + ccol(NL + 2), b2);
                tmem_ld32_wait(b0);
                tmem_ld32_wait(b1);
                tmem_ld32_wait(b2);
                if (r == 0) TR(0, i, 2);
                mask_any(b0, NL);
                max_chunk(b0);
                tmem_ld32_issue(t_lane + ccol(0), b0);
                mask_any(b1, NL + 1);
                max_chunk(b1);
                if (NL > 1) tmem_ld32_issue(t_lane + ccol(1), b1);
                mask_any(b2, NL + 2);
                max_chunk(b2);
                if (NL > 2) tmem_ld32_issue(t_lane + ccol(2), b2);
                tmem_ld32_wait(b0);
                mask_any(b0, 0);
                max_chunk(b0);
                if (NL > 1) {
                    tmem_ld32_wait(b1);
                    mask_any(b1, 1);
                    max_chunk(b1);
                }
                if (NL > 2) {
                    tmem_ld32_wait(b2);
                    mask_any(b2, 2);
                    max_chunk(b2);
                }
                m_row = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                mus = (m_row == -INFINITY ? 0.f : m_row) * P.sl2;
                if (r == 0) TR(0, i, 3);
                // pass 2: the low chunks from the registers, each buffer refilled with a high chunk as it frees
                weights_chunk(b0, piece_of(0));
                tmem_ld32_issue(t_lane + ccol(NL), b0);
                if (NL > 1) {
                    weights_chunk(b1, piece_of(1));
                    tmem_ld32_issue(t_lane + ccol(NL + 1), b1);
                }
                if (NL > 2) {
                    weights_chunk(b2, piece_of(2));
                    tmem_ld32_issue(t_lane + ccol(NL + 2), b2);
                }
                tmem_ld32_wait(b0);
                if (r == 0) TR(0, i, 4);
                mask_any(b0, NL);
                weights_chunk(b0, piece_of(NL));
                if (NL > 1) {
                    tmem_ld32_wait(b1);
                    mask_any(b1, NL + 1);
                    weights_chunk(b1, piece_of(NL + 1));
                    if (NL > 2) {
                        tmem_ld32_wait(b2);
                        mask_any(b2, NL + 2);
                    }
                    weights_chunk(b2, piece_of(NL + 2));   // NL == 2: still in its register from pass 1, masked
                } else {
                    // NL == 1 does not occur (NC is 5 or 6); kept so that every NL compiles
                    weights_chunk(b1, piece_of(NL + 1));
                    weights_chunk(b2, piece_of(NL + 2));
                }
            }
            // zeros in the P columns outside the band (the scores there belong to other rows' bands)
            if (r == 0) TR(0, i, 7);
            {
                uint32_t z[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) z[e] = 0u;
#pragma unroll
                for (int piece = 0; piece < KT / 32; ++piece)
                    if ((piece < pq || piece >= pq + NCH) && !(LF && piece == kLfBand / 32))
                        tmem_st16(t_lane + 16 * piece, z);
            }
            if (grow) sM[slot * kLfGlobals + lane] = m_row;   // read by the epilogue warp once the P V product is done
            if (r == 0) TR(0, i, 5);
            tmem_wait_st();
            if (r == 0) TR(0, i, 6);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_ready + slot);
            if (r == 0) TR(2, i, 2);

        }
        if (!ok) atomicExch(&g_band_status, 1);
    }
    // every role has left its loop (each of its waits is bounded): free the tensor memory
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == kSoftmaxWarps) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * kSlotCols);
    }
}

// ---- host side --------------------------------------------------------------------------------

template <typename T, int KT, bool LF>
int launch_band(const Problem &p, const BandParams &bp_in, int64_t dil, const void *kg, const void *vg,
                const void *qg = nullptr) {
    BandParams bp = bp_in;
    BandMaps m;
    constexpr int kBandKT = LF ? kLfBand : KT;
    // token strides in bytes: the caller's, or contiguous heads
    const int64_t contiguous = p.H * 64 * 2;
    const int64_t TS_q = p.q_ts ? p.q_ts * 2 : contiguous, TS_k = p.k_ts ? p.k_ts * 2 : contiguous;
    const int64_t TS_v = p.v_ts ? p.v_ts * 2 : contiguous, TS_o = p.o_ts ? p.o_ts * 2 : contiguous;
    const int64_t TS_k_own = TS_k, TS_v_own = TS_v;
    const int64_t TS_k_prev = contiguous, TS_v_prev = contiguous, TS_k_next = contiguous, TS_v_next = contiguous;
    const bool fold = LF && bp.lanes > 0;
    if (int rc = make_row_tensor_map5(&m.q, p.q, p.dtype, p.H, dil, p.Sq / dil, p.B, fold ? kLfRows : kTQ, TS_q)) return rc;
    if (int rc = make_row_tensor_map5(&m.k, p.k, p.dtype, p.H, dil, p.Skv / dil, p.B, kBandKT, TS_k)) return rc;
    if (int rc = make_row_tensor_map5(&m.v, p.v, p.dtype, p.H, dil, p.Skv / dil, p.B, kBandKT, TS_v)) return rc;
    if (int rc = make_row_tensor_map5(&m.o, p.o, p.dtype, p.H, dil, p.Sq / dil, p.B, LF ? kLfRows : kTQ, TS_o)) return rc;
    if (int rc = make_row_tensor_map5(&m.k_own, p.k, p.dtype, p.H, dil, p.Skv / dil, p.B, 16, TS_k_own)) return rc;
    if (int rc = make_row_tensor_map5(&m.v_own, p.v, p.dtype, p.H, dil, p.Skv / dil, p.B, 16, TS_v_own)) return rc;
    m.k_prev = m.k_next = m.k_own;
    m.v_prev = m.v_next = m.v_own;
    if (p.k_prev) {
        if (int rc = make_row_tensor_map5(&m.k_prev, p.k_prev, p.dtype, p.H, dil, p.S_prev / dil, p.B, 16, TS_k_prev)) return rc;
        if (int rc = make_row_tensor_map5(&m.v_prev, p.v_prev, p.dtype, p.H, dil, p.S_prev / dil, p.B, 16, TS_v_prev)) return rc;
    }
    if (p.k_next) {
        if (int rc = make_row_tensor_map5(&m.k_next, p.k_next, p.dtype, p.H, dil, p.S_next / dil, p.B, 16, TS_k_next)) return rc;
        if (int rc = make_row_tensor_map5(&m.v_next, p.v_next, p.dtype, p.H, dil, p.S_next / dil, p.B, 16, TS_v_next)) return rc;
    }
    m.kg = m.k_own;
    m.vg = m.v_own;
    if (LF) {
        if (int rc = make_row_tensor_map5(&m.kg, kg, p.dtype, p.H, 1, bp.n_global, p.B, kLfGlobals, contiguous)) return rc;
        if (int rc = make_row_tensor_map5(&m.vg, vg, p.dtype, p.H, 1, bp.n_global, p.B, kLfGlobals, contiguous)) return rc;
    }
    m.qg = m.kg;
    if (fold)
        if (int rc = make_row_tensor_map5(&m.qg, qg, p.dtype, p.H, 1, bp.n_global, p.B, kLfGlobals, contiguous)) return rc;
    auto kern = umma_band_kernel<T, KT, LF>;
    constexpr size_t smem = BandCfg<KT>::kSmemBytes;
    if (int rc = ensure_dynamic_smem((const void *)kern, smem, "cudaFuncSetAttribute(umma_band_kernel)")) return rc;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e, "sizing the persistent grid");
    // one CTA per SM: it owns the SM's tensor memory (fold: one per head and lane, see BandParams)
    const unsigned grid = fold ? (unsigned)(bp.HH * bp.lanes) : (unsigned)std::min<uint64_t>(bp.n_items, (uint64_t)sms);
    if (fold && (int)grid > sms) return fail(MAT_ERR_INVALID, "more lanes than the device has SMs");
    kern<<<grid, kThreads, smem, p.stream>>>(m, bp);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "umma_band_kernel launch");
    note_kernel(LF ? "umma_longformer" : "umma_band");
    return MAT_OK;
}

// Fills bp and returns the key-range width (192 or 256), or 0 when the window does not fit.
// rows = query rows per item, band_cols = columns available to the window part of an item's key range.
int plan_band(const Problem &p, BandParams &bp, bool longformer) {
    const int64_t dil = longformer ? 1 : p.pat.dilation;
    const int rows = longformer ? kLfRows : kTQ;
    bp.Sq1 = (int32_t)(p.Sq / dil);
    bp.Skv1 = (int32_t)(p.Skv / dil);
    bp.off1 = (int32_t)(p.pat.q_offset / dil);
    bp.prev_rows = p.k_prev ? (int32_t)(p.S_prev / dil) : 0;
    const int32_t next_rows = p.k_next ? (int32_t)(p.S_next / dil) : 0;
    bp.key_lo = -bp.prev_rows;
    bp.key_hi = bp.Skv1 + next_rows;
    bp.left = (int32_t)std::min<int64_t>(p.pat.left, bp.Skv1 + bp.prev_rows);
    bp.right = (int32_t)std::min<int64_t>(p.pat.right, bp.Skv1 + next_rows);
    bp.cl = (((bp.off1 - bp.left) % 16) + 16) % 16;
    bp.HH = (int32_t)(p.H * dil);
    bp.H = (int32_t)p.H;
    bp.n_tiles = (bp.Sq1 + rows - 1) / rows;
    bp.sl2 = p.scale * 1.4426950408889634f;
    bp.n_global = longformer ? (int32_t)p.pat.n_global : 0;
    bp.gidx = longformer ? p.pat.gidx : nullptr;
    bp.lanes = 0;
    bp.B = (int32_t)p.B;
    bp.partial = nullptr;
    const uint64_t items = (uint64_t)p.B * bp.n_tiles * bp.HH;
    if (items >= (1ull << 31)) return 0;
    bp.n_items = (uint32_t)items;
    const int need = bp.cl + bp.left + bp.right + rows;   // columns from the first row's first key to the last row's last
    if (longformer) return need <= kLfBand ? 256 : 0;
    return need <= 192 ? 192 : need <= 256 ? 256 : 0;
}

}  // namespace

// Whether the band kernel can run the problem at all (shape, dtype, alignment, window width), leaving aside
// which kernel is the faster one for its size.
bool umma_band_fits(const Problem &p) {
    if (p.pat.kind != MAT_WINDOW) return false;
    if (p.dtype != MAT_BF16 && p.dtype != MAT_F16) return false;
    if (p.D != 64) return false;
    const uintptr_t al = (uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o;
    if (al % 16) return false;
    const int64_t dil = p.pat.dilation;
    if (p.Sq % dil || p.Skv % dil || p.pat.q_offset % dil) return false;
    if (p.Skv / dil >= (1LL << 28) || p.H * dil >= (1LL << 24) || p.B > 65535) return false;
    BandParams bp;
    return plan_band(p, bp, false) != 0;
}

// Windows of at most 128 taps between their two sides on 16-bit inputs with head width 64.
// MAT_WINDOW_KERNEL=mma keeps them on the warp-level kernels, MAT_WINDOW_KERNEL=band sends every window
// the band kernel can take to it whatever the size (debugging and measurement aids).
bool umma_band_supports(const Problem &p) {
    if (!umma_band_fits(p)) return false;
    const char *force = std::getenv("MAT_WINDOW_KERNEL");
    if (force && std::strcmp(force, "mma") == 0) return false;
    BandParams bp;
    const int kt = plan_band(p, bp, false);
    if (kt == 0) return false;
    if (force && std::strcmp(force, "band") == 0) return true;
    // Small problems: a persistent CTA pays about 4.5 us of start-up and drain and works in 128-row items of
    // about 1.4 us, so with few items per SM the one-tile-per-CTA warp-level kernel finishes sooner (a shard
    // of 8192 tokens x 8 heads: 7.0 against 9.6 us; 16384 tokens: 12.6 against 14.4 us; 32768 tokens: 24.6
    // against 23.3 us).  Windows of more than 64 taps always come here: there the warp-level kernel is
    // bound by its shared-memory traffic and loses at every size.
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return kt == 256 || bp.n_items >= 10u * (uint32_t)sms;
}

int launch_umma_band(const Problem &p) {
    BandParams bp;
    const int kt = plan_band(p, bp, false);
    if (kt == 0) return fail(MAT_ERR_UNSUPPORTED, "window too wide for the band kernel");
    const int64_t dil = p.pat.dilation;
    if (p.dtype == MAT_BF16)
        return kt == 192 ? launch_band<__nv_bfloat16, 192, false>(p, bp, dil, nullptr, nullptr)
                         : launch_band<__nv_bfloat16, 256, false>(p, bp, dil, nullptr, nullptr);
    return kt == 192 ? launch_band<__half, 192, false>(p, bp, dil, nullptr, nullptr)
                     : launch_band<__half, 256, false>(p, bp, dil, nullptr, nullptr);
}

// First pass of a Longformer forward (every row over its window plus the keys at the global positions) on
// the band kernel: whole sequences, 1 to 32 global positions whose K/V rows the caller has gathered into
// [B, n_global, H, 64] buffers, a window of at most 128 taps whose first tap sits on a multiple of 16.
// MAT_WINDOW_KERNEL=mma keeps the warp-level kernel.
bool umma_band_longformer_supports(const Problem &p) {
    if (p.pat.kind != MAT_LONGFORMER) return false;
    if (p.dtype != MAT_BF16 && p.dtype != MAT_F16) return false;
    if (p.D != 64 || p.pat.q_offset != 0 || p.Sq != p.Skv) return false;
    if (p.pat.n_global < 1 || p.pat.n_global > kLfGlobals) return false;
    if (p.k_prev || p.k_next) return false;
    const uintptr_t al = (uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o;
    if (al % 16) return false;
    if (p.Skv >= (1LL << 28) || p.H >= (1LL << 24) || p.B > 65535) return false;
    const char *force = std::getenv("MAT_WINDOW_KERNEL");
    if (force && std::strcmp(force, "mma") == 0) return false;
    BandParams bp;
    return plan_band(p, bp, true) != 0;
}

// Lanes per head when the rows at the global positions are folded into the first pass: as many as the SMs
// hold with one CTA per (head, lane); 0 = not folded (more heads than half the SMs would leave too many SMs
// without a CTA, and MAT_LONGFORMER_FOLD=0 keeps the separate global-row pass: a measurement aid).
int umma_band_longformer_lanes(const Problem &p) {
    const char *e = std::getenv("MAT_LONGFORMER_FOLD");
    if (e && e[0] == '0') return 0;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (p.H > sms / 2) return 0;
    return (int)(sms / p.H);
}

size_t umma_band_longformer_partial_bytes(const Problem &p) {
    return (size_t)p.B * p.H * umma_band_longformer_lanes(p) * kLfGlobals * kPartialStride * sizeof(float);
}

// qg and partial given: the rows at the global positions are folded in (lanes from umma_band_longformer_lanes),
// and the caller merges `partial` as lanes splits of 32 rows
int launch_umma_band_longformer(const Problem &p, const void *kg, const void *vg, const void *qg, float *partial) {
    BandParams bp;
    if (plan_band(p, bp, true) == 0) return fail(MAT_ERR_UNSUPPORTED, "window too wide for the band kernel");
    if (((uintptr_t)kg | (uintptr_t)vg | (uintptr_t)qg) % 16) return fail(MAT_ERR_INVALID, "gathered rows must be 16-byte aligned");
    if (qg && partial) {
        bp.lanes = umma_band_longformer_lanes(p);
        bp.partial = partial;
    }
    return p.dtype == MAT_BF16 ? launch_band<__nv_bfloat16, 256, true>(p, bp, 1, kg, vg, qg)
                               : launch_band<__half, 256, true>(p, bp, 1, kg, vg, qg);
}

}  // namespace mat
#ifdef MAT_BAND_TRACE
extern "C" int mat_debug_band_trace(unsigned long long *out) {
    return (int)cudaMemcpyFromSymbol(out, mat::g_trace, sizeof(mat::g_trace));
}
#endif
namespace mat {
int band_status_read_and_clear(int *out) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(out, g_band_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_band_status, &zero, sizeof(int));
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, "reading the kernel status word");
}

}  // namespace mat
