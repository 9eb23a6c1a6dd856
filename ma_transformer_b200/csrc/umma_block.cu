// Block-sparse forward on the 5th-generation tensor cores: tcgen05.mma with the
// accumulators in tensor memory (TMEM), operands staged by TMA.
//
// Block layouts with 64-wide (or wider) blocks make both contractions dense
// 128 x 64 x 64 tiles, which is what tcgen05 is built for; the narrow-window
// kernel stays on the warp-level mma path because its tiles are mostly mask.
// Replaces, for MAT_BLOCK patterns, the intent of the reference's
// BlockSparseAttention (src/csrc/sparse_attention.cpp:203-231 builds the layout,
// :43-152 would walk it entry by entry in COO form).
//
// One CTA = 128 query rows of one (batch, head) = two 64-row halves that may
// belong to different rows of the block layout.  The CTA walks the union of the
// two rows' key blocks in ascending order (column ids are ascending within a
// layout row, so the union is a two-pointer merge, done identically by every
// thread that needs it), 64 keys per step:
//
//   softmax warps (0-3 of a tile):    thread r owns query row r: copies it once from the TMA tile
//                                     into TMEM, then per step tcgen05.ld its 64 scores, masks, takes
//                                     the row maximum and stores P = 2^(s - m) as 16-bit pairs over
//                                     the first 32 columns of the score buffer (tcgen05.st).
//   MMA warp (one lane per tile):     S = Q K^T      tcgen05.mma 128x64x16 x4, A = Q from TMEM, B = K
//                                     from smem, into one of two TMEM S buffers
//                                     [O | l] += P [V | 1]   tcgen05.mma 128x80x16 x4, A = P from TMEM,
//                                     B = V from smem widened to 80 columns whose last 16 read a block
//                                     of ones, so the row sums land in the 16 TMEM columns after O
//   load warp (one lane):             TMA K and V chunks -> smem stages, each released by a commit
//
// A CTA holds one such tile (two CTAs per SM) or, as an option, two tiles sharing the K/V stages.
// The output and the row sums stay in TMEM for the whole walk.  The reference maximum m of a row
// moves only when the chunk's maximum exceeds it by more than a factor 2 (weights then stay <= 2:
// the exponent, rounded to the 16-bit operand type before ex2, keeps an absolute error <= 2^-9
// for the large weights, as with an exact running maximum); only then are the row's O and l read
// back, scaled and stored again (tcgen05.ld / tcgen05.st), which after the first chunks of a
// long row is rare.
//
// A half whose layout row does not hold the step's key block writes a zero row of P for that
// step.  Everything that waits does so on an mbarrier with a bounded wait; a wait that runs out
// sets the library's status word and the CTA drains, frees its TMEM and leaves.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <mutex>

#include "mat_common.cuh"
#include "ptx.cuh"
#include "umma.cuh"

namespace mat {
namespace {

constexpr int kRowBytes = 128;
constexpr int kTileQ = 128;     // query rows per CTA (UMMA M)
constexpr int kTileK = 64;      // keys per step (UMMA N for S, K extent for P V)
// TMEM columns of one tile (256 allocated): S buffers in [0,128), O in [128,192), row sums in [192,208), Q in [208,240)
constexpr int kColO = 128, kColSum = 192, kColQ = 208;   // Q: 64 values of a row in 32 columns
constexpr int kSumN = 16;       // N grows in steps of 16 for M = 128; column 0 of the extra 16 is read
// A row's reference maximum moves (and O and l are rescaled) only when the scores outgrow it by 2^8: until then
// the weights are at most 256, well inside both 16-bit formats, and the sums are fp32.  With a threshold of 2 nearly
// every early step of a walk rescaled (some row of the warp always grew), which cost a wait for the previous P V
// product and a round trip of O through the registers per step.
constexpr float kLazyLog2 = 8.f;

__device__ int g_umma_status = 0;

// Timeline of the first steps of CTA 0 (build with -DMAT_BLOCK_TRACE; read with mat_debug_block_trace):
// slot [role][step][event] = %globaltimer at that point.  Compiled out otherwise.
#ifdef MAT_BLOCK_TRACE
__device__ unsigned long long g_btrace[2 * 48 * 8];
#define BTR(role, step, ev) do { if (blockIdx.x == 0 && (step) < 48) g_btrace[((role) * 48 + (step)) * 8 + (ev)] = ptx::global_ns(); } while (0)
#else
#define BTR(role, step, ev) do { } while (0)
#endif

struct UmmaParams {
    int32_t Sq, Skv, off;  // query rows, key rows, q_offset
    int32_t H;
    int32_t block, per_blk;  // layout block edge, 64-key chunks per block
    int32_t causal;
    int32_t win_left, win_right;   // kModeDense: row p uses keys p - win_left .. p + win_right (clamped to the sequence by the host)
    int64_t n_qblocks;
    const int32_t *rowptr;
    const int32_t *colidx;
    float sl2;
    // global-row pass (kModeGlobalRows): the query tile is the rows at the Longformer global
    // positions, the keys are one split of the whole sequence, the result is a partial
    int32_t n_global;
    const int64_t *gidx;
    int32_t split_len, n_splits, ng_pad;
    float *partial;   // [B, H, n_splits, ng_pad, kPartialStride]: max, sum, unnormalised output
    // work items of the persistent grid: (head, y, batch) with heads running fastest; y = 128-row tile
    // (global-row pass: tile of the global-position list x key split)
    uint32_t n_work, grid_y;
};

constexpr int kModeBlock = 0, kModeGlobalRows = 1, kModeDense = 2;   // kModeDense: every key (up to the query when causal)

using namespace umma;

// Ascending merge of the key blocks of the layout rows a CTA covers (one per 64-row half of each
// 128-row tile), 64 keys per step.  Column ids ascend within a layout row, so the union is a merge
// that every thread needing it performs identically.
template <int NH>
struct ChunkWalk {
    const int32_t *colidx;
    int it[NH], en[NH];  // cursor / end of each half's layout row (empty for a half that shares the row of an earlier half)
    int rep[NH];         // the first half that lies in the same layout row
    int sub, per_blk, block;
    int cur;             // current key block, -1 when exhausted
    int hit;             // bit i: half i's own cursor stands on the current block
    int flags;           // bit i: half i holds the current block
    // rowptr / colidx: the layout, in global memory or the CTA's copy of it in shared memory
    __device__ __forceinline__ void init(const UmmaParams &P, const int32_t *rowptr, const int32_t *colidx_, int q0) {
        colidx = colidx_;
        per_blk = P.per_blk;
        block = P.block;
        int64_t prev_row = -1;
        int prev_i = 0;
#pragma unroll
        for (int i = 0; i < NH; ++i) {
            it[i] = en[i] = 0;
            rep[i] = i;
            const int64_t row = (int64_t)((uint32_t)(q0 + 64 * i + P.off) / (uint32_t)P.block);
            if (i > 0 && row == prev_row) { rep[i] = prev_i; continue; }
            if (q0 + 64 * i < P.Sq && row < P.n_qblocks) { it[i] = rowptr[row]; en[i] = rowptr[row + 1]; }
            prev_row = row;
            prev_i = i;
        }
        sub = 0;
        load();
    }
    __device__ __forceinline__ void load() {
        int col[NH];
        int c = INT32_MAX;
#pragma unroll
        for (int i = 0; i < NH; ++i) {
            col[i] = it[i] < en[i] ? colidx[it[i]] : INT32_MAX;
            c = min(c, col[i]);
        }
        if (c == INT32_MAX) { cur = -1; hit = flags = 0; return; }
        cur = c;
        hit = flags = 0;
#pragma unroll
        for (int i = 0; i < NH; ++i) hit |= (col[i] == c ? 1 : 0) << i;
#pragma unroll
        for (int i = 0; i < NH; ++i) flags |= ((hit >> rep[i]) & 1) << i;
    }
    // a plain key range [lo, hi) instead of a layout: 64-key steps, every half takes part
    __device__ __forceinline__ void init_range(int lo, int hi) {
        colidx = nullptr;
        block = kTileK; per_blk = 1; sub = 0;
#pragma unroll
        for (int i = 0; i < NH; ++i) { it[i] = en[i] = 0; rep[i] = 0; }
        it[0] = lo / kTileK;                    // lo is a multiple of 64
        en[0] = (hi + kTileK - 1) / kTileK;
        cur = it[0] < en[0] ? it[0] : -1;
        hit = 1;
        flags = (1 << NH) - 1;
    }
    __device__ __forceinline__ bool done() const { return cur < 0; }
    __device__ __forceinline__ int key_base() const { return cur * block + sub * kTileK; }
    __device__ __forceinline__ void next() {
        if (colidx == nullptr) { cur = ++it[0] < en[0] ? it[0] : -1; return; }
        if (++sub < per_blk) return;
        sub = 0;
#pragma unroll
        for (int i = 0; i < NH; ++i) it[i] += (hit >> i) & 1;
        load();
    }
};

// NT = 128-row query tiles per CTA.  One tile: 256 TMEM columns, two CTAs per SM.  Two tiles: all 512
// columns, one CTA per SM, and every K/V chunk fetched from L2 serves 256 query rows instead of 128.
constexpr int kSoftmaxWarpsPerTile = 4;
// QS = query tiles held in shared memory: 1 when the softmax warps copy Q into TMEM (the A operand of the S
// products comes from there), 2 when the S products read Q from shared memory, double-buffered over items.
template <int NT, int QS> struct Cfg {
    static constexpr int kSoftmaxWarps = kSoftmaxWarpsPerTile * NT;
    // softmax warps, one MMA warp per tile, load warp; with Q in shared memory a second issuing warp (the P V products)
    static constexpr int kThreads = (kSoftmaxWarps + NT + 1 + (QS == 2 ? 1 : 0)) * 32;
    static constexpr int kKvStages = NT == 1 ? (QS == 2 ? 4 : 5) : 8;   // (two CTAs of one tile share an SM's shared memory)
    static constexpr int kTmemCols = 256 * NT;
    static constexpr int kBars = 2 + NT * 9 + 4 * kKvStages + 2;
    // block layouts: the CTA's copy of the layout (row pointers, then column ids) when it fits
    static constexpr int kLayoutInts = QS == 2 ? 3072 : 0;
    static constexpr size_t kSmemBytes = 1024 + (size_t)QS * NT * kTileQ * kRowBytes /*Q*/ +
                                         (size_t)kKvStages * 2 * kTileK * kRowBytes + kSumN * kRowBytes +
                                         kBars * 8 + 16 /*tmem address*/ + kLayoutInts * 4;
};
// Block layouts only.  (The dense walk on the same path - Q from shared memory, two issuing lanes - was measured
// slower than with Q in TMEM and one lane: 423.7 against 411.1 us at 2 x 8192 x 8 heads.)
__host__ __device__ constexpr int qs_of(int mode, int nt) { return mode == 0 /* kModeBlock */ && nt == 1 ? 2 : 1; }
constexpr int kStage = 2 * kTileK * kRowBytes;  // one K/V stage: K then V
constexpr int kOnesBytes = kSumN * kRowBytes;   // the second 64-wide block of the P V product's B operand: ones

// The step pipeline (t = index of the 64-key chunk), per tile:
//   load warp: K(t) as soon as S(t - kKvStages) has left its stage (in every tile), V(t) once P V(t - kKvStages) has.
//   MMA warp:  S(t+1) is issued before P V(t), so the tensor core computes the next scores while
//              the softmax warps work on the current ones; S is double-buffered in TMEM.  Q and P
//              are A operands read from TMEM: Q is copied there once per tile, P(t) is stored by
//              the softmax warps over the first 32 columns of the S buffer it was computed from
//              (S(t+2), which overwrites them, is issued after P V(t) and so runs after it).
//              Shared memory then carries only K and V (its bandwidth, not the tensor pipe, bounded
//              the variant that kept Q and P there).  P V(t) accumulates into O and l in TMEM (the
//              first chunk overwrites).
//   softmax:   softmax(t) -> store P(t) -> (rarely: wait for P V(t-1), rescale O and l) -> publish.
template <typename T, int MODE, int NT>
__global__ void __launch_bounds__(Cfg<NT, qs_of(MODE, NT)>::kThreads)
umma_block_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, T *__restrict__ out, const UmmaParams P) {
    // Block layouts (short walks, so what happens between two items counts): the S products read Q from shared
    // memory, where the next item's tile lands while this one's is in use, and nothing of the hand-over from
    // one item to the next runs through the softmax warps.  The long walks (dense, wide windows, global rows)
    // keep Q in TMEM: there the shared-memory reads per step are what matters.
    constexpr int QS = qs_of(MODE, NT);
    constexpr bool kQsmem = QS == 2;
    static_assert(!kQsmem || NT == 1, "the shared-memory Q path is written for one tile per CTA");
    using C = Cfg<NT, QS>;
    constexpr int kSoftmaxWarps = C::kSoftmaxWarps, kKvStages = C::kKvStages, NH = 2 * NT;
    constexpr int kQBytes = NT * kTileQ * kRowBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem;                                // QS buffers of NT tiles of 128 rows
    uint8_t *sKV = sQ + QS * kQBytes;                  // stage s: K at +0, V at +8 KB
    uint8_t *sOnes = sKV + kKvStages * kStage;         // 16 rows of ones
    uint64_t *bars = (uint64_t *)(sOnes + kOnesBytes);
    // shared by the tiles: Q arrival, K/V arrival and release per stage
    uint64_t *bar_q = bars, *bar_k = bars + 2, *bar_v = bar_k + kKvStages, *bar_kfree = bar_v + kKvStages,
             *bar_vfree = bar_kfree + kKvStages;
    // per tile (9 each): Q in TMEM, end of walk, TMEM reads done, S ready [2], P ready [2], P V done [2]
    uint64_t *tile_bars = bar_vfree + kKvStages;
    uint64_t *bar_qfree = tile_bars + 9 * NT;   // [2]: the S products of an item have left its Q buffer
    uint32_t *tmem_slot = (uint32_t *)(bar_qfree + 2);
    int32_t *sLayout = (int32_t *)(tmem_slot + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Persistent: CTA c works on items c, c + G, c + 2G, ...; every barrier's phase runs on across items
    // (per-item barriers flip once per item, per-step barriers count the steps of all items so far).
    const uint32_t G = gridDim.x;
    const uint32_t n_mine = blockIdx.x < P.n_work ? (P.n_work - blockIdx.x + G - 1) / G : 0;
    struct Item {
        int h, b, q0, split;
        int lo, hi;   // key range: a split of the sequence (global rows), or what the tile's rows can see (dense, windows)
    };
    auto item_at = [&](uint32_t n) {
        const uint32_t L = blockIdx.x + n * G, H = (uint32_t)P.H;
        Item I;
        I.h = (int)(L % H);
        uint32_t y = (L / H) % P.grid_y;
        I.b = (int)(L / (H * P.grid_y));
        // causal walks grow with the tile index: the long ones first, so that the CTAs finish together
        if (MODE == kModeDense) y = P.grid_y - 1 - y;
        // global-row pass: y = (128-row tile of the global-position list) * n_splits + key split
        I.split = MODE == kModeGlobalRows ? (int)(y % (uint32_t)P.n_splits) : 0;
        I.q0 = (int)(MODE == kModeGlobalRows ? y / (uint32_t)P.n_splits : y) * (NT * kTileQ);
        // (a window: from the 64-key chunk that holds the first row's first key to the last row's last key)
        I.lo = MODE == kModeGlobalRows ? I.split * P.split_len
             : MODE == kModeDense ? (max(0, I.q0 + P.off - P.win_left) & ~(kTileK - 1)) : 0;
        I.hi = MODE == kModeGlobalRows ? min(I.lo + P.split_len, P.Skv)
             : MODE == kModeDense ? min(P.Skv, I.q0 + P.off + NT * kTileQ + P.win_right)
             : P.Skv;
        return I;
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(bar_q + i, 1);
            ptx::mbar_init(bar_qfree + i, NT);
        }
        for (int i = 0; i < kKvStages; ++i) {
            ptx::mbar_init(bar_k + i, 1);
            ptx::mbar_init(bar_v + i, 1);
            ptx::mbar_init(bar_kfree + i, NT);
            ptx::mbar_init(bar_vfree + i, NT);
        }
        for (int tl = 0; tl < NT; ++tl) {
            uint64_t *tb = tile_bars + 9 * tl;
            ptx::mbar_init(tb + 0, kSoftmaxWarpsPerTile);   // Q in TMEM
            ptx::mbar_init(tb + 1, 1);                      // end of walk
            ptx::mbar_init(tb + 2, kSoftmaxWarpsPerTile);   // TMEM reads done
            for (int i = 0; i < 2; ++i) {
                ptx::mbar_init(tb + 3 + i, 1);                      // S ready
                ptx::mbar_init(tb + 5 + i, kSoftmaxWarpsPerTile);   // P ready
                ptx::mbar_init(tb + 7 + i, 1);                      // P V done
            }
        }
        ptx::fence_barrier_init();
    }
    // Block layouts: every role walks the layout rows of its items, and the walk's reads sit on its critical
    // path (each is a row pointer, then a column id per step).  A persistent CTA sees many rows, so it copies
    // the whole layout into shared memory once when that fits; a larger layout is read from global memory.
    const int32_t *rowptr = P.rowptr, *colidx = P.colidx;
    if (MODE == kModeBlock && P.n_qblocks + 1 <= C::kLayoutInts) {
        const int n_row = (int)P.n_qblocks + 1;
        const int nnz = P.rowptr[P.n_qblocks];
        if (nnz >= 0 && n_row + nnz <= C::kLayoutInts) {
            for (int i = threadIdx.x; i < n_row; i += blockDim.x) sLayout[i] = P.rowptr[i];
            for (int i = threadIdx.x; i < nnz; i += blockDim.x) sLayout[n_row + i] = P.colidx[i];
            rowptr = sLayout;
            colidx = sLayout + n_row;
        }
    }
    if (threadIdx.x < kOnesBytes / 16) {
        const uint32_t one2 = ptx::Mma<T>::kOnes;
        reinterpret_cast<uint4 *>(sOnes)[threadIdx.x] = make_uint4(one2, one2, one2, one2);
        ptx::fence_proxy_async_smem();
    }
    if (warp == kSoftmaxWarps) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // TMEM columns of tile i start at 256 i: S buffer j at 64 j (P(t) over its first 32), O at kColO,
    // row sums at kColSum, Q at kColQ

    if (warp == kSoftmaxWarps + NT) {
        // ================= load warp: per item Q, then K and V chunk by chunk =================
        if (lane == 0) {
            bool ok = true;
            int c_k = 0, c_v = 0;   // K and V chunks fetched so far, all items: they name the stage and its phase
            for (uint32_t n = 0; ok && n < n_mine; ++n) {
                const Item I = item_at(n);
                ChunkWalk<NH> w_k, w_v;   // K runs one chunk ahead of V: its stage is free earlier (after S, not after P V)
                if (MODE != kModeBlock) w_k.init_range(I.lo, I.hi);
                else w_k.init(P, rowptr, colidx, I.q0);
                w_v = w_k;
                if (kQsmem) {
                    // buffer n & 1, once the S products of item n - 2 have left it
                    const int qb = n & 1;
                    if (n >= 2 && !(ok = ptx::mbar_wait(bar_qfree + qb, ((n >> 1) - 1) & 1))) break;
                    ptx::mbar_expect_tx(bar_q + qb, kQBytes);
                    ptx::tma_load_4d(sQ + qb * kQBytes, &map_q, bar_q + qb, 0, I.h, I.q0, I.b);
                } else {
                    // the softmax warps have copied the previous item's Q out of shared memory
                    for (int tl = 0; n >= 1 && tl < NT; ++tl) ok = ok && ptx::mbar_wait(tile_bars + 9 * tl, (n - 1) & 1);
                    if (!ok) break;
                    ptx::mbar_expect_tx(bar_q, kQBytes);
                    if (MODE == kModeGlobalRows) {
                        // map_q is a one-row view here: row r of the tile is the query at global position
                        // gidx[q0 + r]; slots past the list read out of bounds, i.e. zeros
                        for (int r = 0; r < NT * kTileQ; ++r) {
                            const int e = I.q0 + r;
                            const int row = e < P.n_global ? (P.gidx ? (int)P.gidx[e] : e) : P.Sq;   // no list: already gathered
                            ptx::tma_load_4d(sQ + r * kRowBytes, &map_q, bar_q, 0, I.h, row, I.b);
                        }
                    } else {
                        for (int tl = 0; tl < NT; ++tl)
                            ptx::tma_load_4d(sQ + tl * kTileQ * kRowBytes, &map_q, bar_q, 0, I.h, I.q0 + tl * kTileQ, I.b);
                    }
                }
                auto load_k = [&]() -> bool {   // the next K chunk once the S product kKvStages chunks back has left the stage
                    const int s = c_k % kKvStages;
                    if (c_k >= kKvStages && !ptx::mbar_wait(bar_kfree + s, (c_k / kKvStages - 1) & 1)) return false;
                    ptx::mbar_expect_tx(bar_k + s, kTileK * kRowBytes);
                    ptx::tma_load_4d(sKV + s * kStage, &map_k, bar_k + s, 0, I.h, w_k.key_base(), I.b);
                    ++c_k;
                    w_k.next();
                    return true;
                };
                if (!w_k.done()) ok = load_k();
                for (; ok && !w_v.done(); ++c_v, w_v.next()) {
                    if (!w_k.done() && !(ok = load_k())) break;
                    const int s = c_v % kKvStages;   // V once the P V product kKvStages chunks back has left the stage
                    if (c_v >= kKvStages && !(ok = ptx::mbar_wait(bar_vfree + s, (c_v / kKvStages - 1) & 1))) break;
                    ptx::mbar_expect_tx(bar_v + s, kTileK * kRowBytes);
                    ptx::tma_load_4d(sKV + s * kStage + kTileK * kRowBytes, &map_v, bar_v + s, 0, I.h, w_v.key_base(), I.b);
                }
            }
            if (!ok) atomicExch(&g_umma_status, 1);
        }
        return;
    }
    if (kQsmem && warp == kSoftmaxWarps + NT + 1) {
        // ================= second issuing warp (Q in shared memory): the P V products =================
        // Block layouts have short walks, and one lane that issues both products of every step (4 + 4
        // tcgen05.mma, four commits, three or four barrier waits and the layout walk: about 0.9 us per step)
        // was what bounded them.  Here one lane issues the S products, running ahead over item boundaries, and
        // this one the P V products; what used to be program order between them is explicit: S(g) waits for
        // P V(g - 2), whose weights sit in the score buffer it overwrites.
        if (lane == 0) {
            bool ok = true;
            const uint32_t tmem = tmem_base;
            uint64_t *tb = tile_bars;
            uint64_t *bar_fin = tb + 1, *bar_done = tb + 2, *bar_p = tb + 5, *bar_o = tb + 7;
            const uint32_t idesc_pv = instr_desc<T>(true, kTileK + kSumN);
            const uint32_t kv_addr = ptx::smem_u32(sKV), ones_addr = ptx::smem_u32(sOnes);
            int g = 0;   // step, counted over all items
            for (uint32_t n = 0; ok && n < n_mine; ++n) {
                ChunkWalk<NH> w_p;   // counts the item's steps
                {
                    const Item I = item_at(n);
                    if (MODE != kModeBlock) w_p.init_range(I.lo, I.hi);
                    else w_p.init(P, rowptr, colidx, I.q0);
                }
                for (bool first = true; ok && !w_p.done(); w_p.next(), first = false, ++g) {
                    const int s = g % kKvStages;
                    BTR(1, g, 3);
                    if (!(ok = ptx::mbar_wait(bar_v + s, (g / kKvStages) & 1))) break;
                    BTR(1, g, 4);
                    if (!(ok = ptx::mbar_wait(bar_p + (g & 1), (g >> 1) & 1))) break;   // P is in TMEM
                    BTR(1, g, 5);
                    // the item's first product overwrites O: the previous item's rows have been read out of it
                    if (first && n >= 1 && !(ok = ptx::mbar_wait(bar_done, (n - 1) & 1))) break;
                    tc_fence_after();
                    const uint32_t v_addr = kv_addr + s * kStage + kTileK * kRowBytes;
                    const uint32_t tp = tmem + (g & 1) * kTileK;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint32_t vk = v_addr + ks * 16 * kRowBytes;
                        umma_f16_ta(tmem + kColO, tp + ks * 8, smem_desc(vk, (ones_addr - vk) >> 4), idesc_pv, !first || ks > 0);
                    }
                    umma_commit(bar_o + (g & 1));
                    umma_commit(bar_vfree + s);
                    BTR(1, g, 6);
                }
                if (ok) umma_commit(bar_fin);
            }
            if (!ok) atomicExch(&g_umma_status, 1);
        }
        return;
    }
    // everything below belongs to one tile
    const int tile = warp >= kSoftmaxWarps ? warp - kSoftmaxWarps : warp / kSoftmaxWarpsPerTile;
    const uint32_t tmem = tmem_base + 256 * tile;
    uint64_t *tb = tile_bars + 9 * tile;
    uint64_t *bar_qt = tb, *bar_fin = tb + 1, *bar_done = tb + 2, *bar_s = tb + 3, *bar_p = tb + 5, *bar_o = tb + 7;

    if (warp >= kSoftmaxWarps) {
        // ================= MMA warp of the tile: one lane issues every tcgen05.mma =================
        if (lane == 0) {
            bool ok = true;
            const uint32_t idesc_s = instr_desc<T>(false, kTileK), idesc_pv = instr_desc<T>(true, kTileK + kSumN);
            // descriptors differ from step to step only in the start address field (16-byte units)
            const uint32_t kv_addr = ptx::smem_u32(sKV), ones_addr = ptx::smem_u32(sOnes);
            const uint64_t dkv = smem_desc(kv_addr);
            if constexpr (kQsmem) {
                // the S products of every item, as far ahead as the K ring and the two score buffers allow
                int g = 0;
                for (uint32_t n = 0; ok && n < n_mine; ++n) {
                    ChunkWalk<NH> w_s;
                    {
                        const Item I = item_at(n);
                        if (MODE != kModeBlock) w_s.init_range(I.lo, I.hi);
                        else w_s.init(P, rowptr, colidx, I.q0);
                    }
                    if (!(ok = ptx::mbar_wait(bar_q + (n & 1), (n >> 1) & 1))) break;   // Q has landed in its buffer
                    const uint64_t dq = smem_desc(ptx::smem_u32(sQ) + (n & 1) * kQBytes);
                    for (; ok && !w_s.done(); w_s.next(), ++g) {
                        const int s = g % kKvStages;
                        BTR(1, g, 0);
                        if (!(ok = ptx::mbar_wait(bar_k + s, (g / kKvStages) & 1))) break;
                        // the weights of step g - 2 have been read out of this score buffer by their P V product
                        if (g >= 2 && !(ok = ptx::mbar_wait(bar_o + (g & 1), ((g - 2) >> 1) & 1))) break;
                        tc_fence_after();
                        BTR(1, g, 1);
                        const uint64_t dk = dkv + (uint64_t)(s * (kStage >> 4));
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks)
                            umma_f16_ss(tmem + (g & 1) * kTileK, dq + ks * 2, dk + ks * 2, idesc_s, ks > 0);
                        umma_commit(bar_s + (g & 1));
                        umma_commit(bar_kfree + s);
                        BTR(1, g, 2);
                    }
                    if (ok) umma_commit(bar_qfree + (n & 1));
                }
            }
            int base = 0;   // steps of the items before this one: step t of the item is step base + t of the barriers
            for (uint32_t n = 0; !kQsmem && ok && n < n_mine; ++n) {
                const Item I = item_at(n);
                ChunkWalk<NH> w_s;     // only counts the chunks here
                if (MODE != kModeBlock) w_s.init_range(I.lo, I.hi);
                else w_s.init(P, rowptr, colidx, I.q0);
                int t_s = 0;   // S products issued for this item
                const uint64_t dq = smem_desc(ptx::smem_u32(sQ) + (n & 1) * (kQsmem ? kQBytes : 0));   // (Q in shared memory)
                auto issue_s = [&]() -> bool {   // the next S = Q K^T, into S buffer (base + t_s) & 1
                    const int g = base + t_s, s = g % kKvStages;
                    BTR(1, g, 0);
                    if (!ptx::mbar_wait(bar_k + s, (g / kKvStages) & 1)) return false;
                    tc_fence_after();
                    BTR(1, g, 1);
                    const uint64_t dk = dkv + (uint64_t)(s * (kStage >> 4));
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {   // 16 of the 64 head columns per instruction (8 TMEM columns, or 32 bytes of a row, of Q)
                        if (kQsmem) umma_f16_ss(tmem + (g & 1) * kTileK, dq + ks * 2, dk + ks * 2, idesc_s, ks > 0);
                        else umma_f16_ta(tmem + (g & 1) * kTileK, tmem + kColQ + ks * 8, dk + ks * 2, idesc_s, ks > 0);
                    }
                    umma_commit(bar_s + (g & 1));
                    umma_commit(bar_kfree + s);
                    BTR(1, g, 2);
                    ++t_s;
                    w_s.next();
                    return true;
                };
                if (kQsmem) {
                    if (!(ok = ptx::mbar_wait(bar_q + (n & 1), (n >> 1) & 1))) break;   // Q has landed in its buffer
                } else {
                    // Q is in TMEM.  (A softmax warp stores it after reading the previous item's O, so the first
                    // P V product below, which overwrites O, cannot run ahead of that read either.)
                    if (!(ok = ptx::mbar_wait(bar_qt, n & 1))) break;
                }
                tc_fence_after();
                if (!w_s.done()) ok = issue_s();
                for (int t = 0; ok && t < t_s; ++t) {
                    // the next scores first: their S buffer was released by the P V product two steps back,
                    // issued before this point (the tensor core runs them in order)
                    if (!w_s.done() && !(ok = issue_s())) break;
                    const int g = base + t, s = g % kKvStages;
                    BTR(1, g, 3);
                    if (!(ok = ptx::mbar_wait(bar_v + s, (g / kKvStages) & 1))) break;
                    BTR(1, g, 4);
                    if (!(ok = ptx::mbar_wait(bar_p + (g & 1), (g >> 1) & 1))) break;   // P(t) is in TMEM
                    BTR(1, g, 5);
                    // the item's first product overwrites O: the previous item's rows have been read out of it
                    if (kQsmem && t == 0 && n >= 1 && !(ok = ptx::mbar_wait(bar_done, (n - 1) & 1))) break;
                    tc_fence_after();
                    const uint32_t v_addr = kv_addr + s * kStage + kTileK * kRowBytes;
                    const uint32_t tp = tmem + (g & 1) * kTileK;   // P(t): 64 weights of a row in 32 columns
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {   // [O | l] += P [V | 1], 16 of the 64 keys per instruction
                        // B is 16 keys x 80 columns: the 64 head columns from the V stage, then a second
                        // 64-wide block (16 of it used) that the leading-dimension offset points at the ones
                        const uint32_t vk = v_addr + ks * 16 * kRowBytes;
                        umma_f16_ta(tmem + kColO, tp + ks * 8, smem_desc(vk, (ones_addr - vk) >> 4), idesc_pv, t > 0 || ks > 0);
                    }
                    umma_commit(bar_o + (g & 1));
                    umma_commit(bar_vfree + s);
                    BTR(1, g, 6);
                }
                // each bar_o barrier sees every other product, so its parity names one product for a
                // waiter that is at most one product behind; the end of an item's walk gets a barrier of its own
                if (ok) umma_commit(bar_fin);
                if (ok && kQsmem) umma_commit(bar_qfree + (n & 1));
                base += t_s;
            }
            if (!ok) atomicExch(&g_umma_status, 1);
            // every softmax warp of every tile has read its last TMEM values before the columns are freed
            for (int tl = 0; n_mine >= 1 && tl < NT; ++tl)
                if (warp == kSoftmaxWarps && !ptx::mbar_wait(tile_bars + 9 * tl + 2, (n_mine - 1) & 1)) atomicExch(&g_umma_status, 1);
        }
        __syncwarp();
        if (warp == kSoftmaxWarps) {   // the allocating warp frees
            tc_fence_after();
            tmem_dealloc(tmem_base, C::kTmemCols);
        }
        return;
    }

    // ================= softmax warps: thread r owns query row r of its tile =================
    const int quad = warp % kSoftmaxWarpsPerTile;   // == warp % 4: the TMEM lanes this warp may access
    const int r = quad * 32 + lane;        // row of the tile == TMEM lane
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
    bool ok = true;
    // the query row, from the swizzled tile the TMA wrote, into TMEM: the A operand of every S product of item n
    auto stage_q = [&](uint32_t n) {
        if (!(ok = ptx::mbar_wait(bar_q, n & 1))) return;
        const uint8_t *q_row = sQ + (tile * kTileQ + r) * kRowBytes;
        uint32_t qv[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint4 v = *reinterpret_cast<const uint4 *>(q_row + ((c ^ (r & 7)) << 4));
            qv[4 * c] = v.x; qv[4 * c + 1] = v.y; qv[4 * c + 2] = v.z; qv[4 * c + 3] = v.w;
        }
        tmem_st32(t_lane + kColQ, qv);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_qt);
    };
    if (!kQsmem && n_mine >= 1) stage_q(0);
    // what the read-out of an item needs once its walk is over
    struct Finished {
        Item I;
        uint32_t n;
        int steps;
        float m_run;
    };
    // The accumulated row and its sum, once the item's last P V product has completed; then the row is written out.
    // Q in TMEM: the next item's queries go there before the rows are written, so that the tensor core starts
    // on its scores while the stores are under way.
    auto read_out = [&](const Finished &f) {
        const int tq0 = f.I.q0 + tile * kTileQ;
        float o[64];
        float l_run = 0.f;
        if (!(ok = ptx::mbar_wait(bar_fin, f.n & 1))) return;
        tc_fence_after();
        if (f.steps >= 1) {
            tmem_ld64_and_1(t_lane + kColO, o, t_lane + kColSum, l_run);
        } else {
#pragma unroll
            for (int i = 0; i < 64; ++i) o[i] = 0.f;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_done);
        if (!kQsmem && f.n + 1 < n_mine) {
            stage_q(f.n + 1);
            if (!ok) return;
        }
        if (MODE == kModeGlobalRows) {
            if (tq0 + r < P.n_global) {
                float *pr = P.partial +
                            ((((int64_t)f.I.b * P.H + f.I.h) * P.n_splits + f.I.split) * P.ng_pad + tq0 + r) * kPartialStride;
                pr[0] = f.m_run;
                pr[1] = l_run;
#pragma unroll
                for (int i = 0; i < 64; i += 2) *reinterpret_cast<float2 *>(pr + 2 + i) = make_float2(o[i], o[i + 1]);
            }
        } else if (tq0 + r < P.Sq) {
            const float inv = l_run > 0.f ? __frcp_rn(l_run) : 0.f;
            T *dst = out + (((int64_t)f.I.b * P.Sq + tq0 + r) * P.H + f.I.h) * 64;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                uint4 v;
                v.x = ptx::Mma<T>::pack(o[8 * q] * inv, o[8 * q + 1] * inv);
                v.y = ptx::Mma<T>::pack(o[8 * q + 2] * inv, o[8 * q + 3] * inv);
                v.z = ptx::Mma<T>::pack(o[8 * q + 4] * inv, o[8 * q + 5] * inv);
                v.w = ptx::Mma<T>::pack(o[8 * q + 6] * inv, o[8 * q + 7] * inv);
                *reinterpret_cast<uint4 *>(dst + 8 * q) = v;
            }
        }
    };
    int base = 0;   // steps of the items before this one (see the MMA warp)
    // Q in shared memory: an item's read-out waits until the weights of the NEXT item's first step are stored (its
    // scores were computed while this item's last steps ran, and that step never touches O), so the wait for the
    // last P V product and the read of O sit behind useful work instead of between two items.
    bool pending = false;
    Finished fin;
    for (uint32_t n = 0; ok && n < n_mine; ++n) {
        const Item I = item_at(n);
        const int tq0 = I.q0 + tile * kTileQ;    // first row of the tile
        const int half = tile * 2 + (r >> 6);
        const int p = tq0 + r + P.off;         // key-coordinate position of this row
        float m_run = -INFINITY;   // reference maximum of the row's weights (raw score units); -inf: no key yet
        ChunkWalk<NH> w;
        if (MODE != kModeBlock) w.init_range(I.lo, I.hi);
        else w.init(P, rowptr, colidx, I.q0);
        // global-row pass: a warp takes part iff any of its 32 rows is a real global position
        const bool warp_has_rows = MODE != kModeGlobalRows || tq0 + quad * 32 < P.n_global;
        int t = 0;
        for (; ok && !w.done(); ++t) {
            const int g = base + t;
            const int kb = w.key_base();
            const bool mine = MODE == kModeGlobalRows ? warp_has_rows : (w.flags >> half) & 1;   // uniform within a warp (dense: always)
            w.next();   // the layout reads for the next step are in flight during this one
            if (threadIdx.x == 0) BTR(0, g, 0);
            if (!(ok = ptx::mbar_wait(bar_s + (g & 1), (g >> 1) & 1))) break;
            tc_fence_after();
            if (threadIdx.x == 0) BTR(0, g, 1);
            const uint32_t s_addr = t_lane + (g & 1) * kTileK;   // S(t), and P(t) over its first 32 columns
            if (mine) {
                // keys this row may use in the chunk: j < j_end
                int j_end = min(kTileK, (MODE == kModeGlobalRows ? I.hi : P.Skv) - kb);
                if (MODE == kModeBlock && P.causal) j_end = min(j_end, p - kb + 1);
                int j_begin = 0;   // and j >= j_begin (a window's left edge)
                if (MODE == kModeDense) {
                    j_end = min(j_end, p + P.win_right - kb + 1);
                    j_begin = p - P.win_left - kb;
                }
                float s[64];
                tmem_ld64(s_addr, s);
                if (threadIdx.x == 0) BTR(0, g, 2);
                if (j_end < kTileK || j_begin > 0) {   // only the chunks on an edge of the window or at the sequence end
#pragma unroll
                    for (int i = 0; i < 64; ++i) if (i >= j_end || i < j_begin) s[i] = -INFINITY;
                }
                float mq[4];   // four independent chains of three-input maxima
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    mq[q] = max3(s[16 * q], s[16 * q + 1], s[16 * q + 2]);
#pragma unroll
                    for (int i = 3; i < 15; i += 2) mq[q] = max3(mq[q], s[16 * q + i], s[16 * q + i + 1]);
                    mq[q] = fmaxf(mq[q], s[16 * q + 15]);
                }
                const float mx = fmaxf(max3(mq[0], mq[1], mq[2]), mq[3]);
                if (threadIdx.x == 0) BTR(0, g, 3);
                // move the reference maximum only when the scores outgrow it by 2^kLazyLog2
                const bool seen = m_run != -INFINITY;
                const bool grow = seen ? (mx - m_run) * P.sl2 > kLazyLog2 : mx != -INFINITY;
                const bool rescale = seen && grow;
                const float alpha = rescale ? ptx::ex2((m_run - mx) * P.sl2) : 1.f;
                if (grow) m_run = mx;
                const float mus = (m_run == -INFINITY ? 0.f : m_run) * P.sl2;
                // weights, packed to the operand type two at a time: column i of P holds keys 2i and 2i+1.
                // (The exponentials bound the step: the special-function unit gives 16 results per clock and SM,
                // packed 16-bit forms included, so the 8192 of a step take 512 clocks against about 290 of tensor
                // work.  Moving a share of them to the FMA pipe as a cubic - rounding trick, three packed FMAs,
                // an integer add into the exponent - was measured slower at every share: about 23 issue clocks
                // per pair against 16 on the unit.)
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float x0, x1;
                    ffma2(x0, x1, s[2 * i], s[2 * i + 1], P.sl2, -mus);
                    pk[i] = ptx::Mma<T>::ex2_packed(ptx::Mma<T>::pack(x0, x1));
                }
                tmem_st32(s_addr, pk);
                if (threadIdx.x == 0) BTR(0, g, 4);
                if (__any_sync(0xffffffffu, rescale)) {
                    // O and l hold the chunks up to t-1: wait for P V(t-1), then scale this row in place
                    if (!(ok = ptx::mbar_wait(bar_o + ((g - 1) & 1), ((g - 1) >> 1) & 1))) break;
                    tc_fence_after();
                    float part[64], l_part;
                    tmem_ld64_and_1(t_lane + kColO, part, t_lane + kColSum, l_part);
#pragma unroll
                    for (int i = 0; i < 64; i += 2) fmul2(part[i], part[i + 1], part[i], part[i + 1], alpha);
                    tmem_st64(t_lane + kColO, part);
                    tmem_st1(t_lane + kColSum, l_part * alpha);
                }
                tmem_wait_st();
            } else {
                // this half sits the chunk out: its rows of P (scores at this point) must add nothing to O and l
                uint32_t z[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) z[i] = 0u;
                tmem_st32(s_addr, z);
                tmem_wait_st();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_p + (g & 1));
            if (threadIdx.x == 0) BTR(0, g, 5);
            if (pending) {   // (only with Q in shared memory, and only at an item's first step)
                pending = false;
                read_out(fin);
            }
        }
        if (ok && pending) {   // an item without a step
            pending = false;
            read_out(fin);
        }
        if (!ok) break;
        base += t;
        fin.I = I;
        fin.n = n;
        fin.steps = t;
        fin.m_run = m_run;
        if (kQsmem) pending = true;
        else read_out(fin);
    }
    if (ok && pending) read_out(fin);
    if (!ok) atomicExch(&g_umma_status, 1);
}

// ---- host side --------------------------------------------------------------------------------

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

// [B, S, H, 64] 16-bit rows as dims {64, H, S, B}, box {64, 1, rows, 1}, 128-byte swizzle
int make_map(CUtensorMap *m, const void *base, int dtype, int64_t H, int64_t S, int64_t B, int rows) {
    PFN_cuTensorMapEncodeTiled enc = encode_fn();
    if (!enc) return fail(MAT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[4] = {64, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
    const cuuint64_t strides[3] = {128, (cuuint64_t)H * 128, (cuuint64_t)S * H * 128};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)rows, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, dtype == MAT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                     const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MAT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return MAT_OK;
}

// One 128-row tile per CTA (two CTAs per SM) is the measured optimum: two tiles per CTA sharing the
// K/V stages fetch every chunk from L2 half as often but came out slower (dense 16K tokens x 8 heads:
// 0.91 ms against 0.83 ms; the 16K block-sparse workload 267 us against 193 us), so the L2 -> shared
// memory traffic is not what bounds the walk.  MAT_UMMA_TILES=2 selects the two-tile variant for the dense
// walks (a measurement aid; block layouts always run one tile per CTA).
int tiles_per_cta() {
    const char *e = std::getenv("MAT_UMMA_TILES");
    return e && e[0] == '2' ? 2 : 1;
}

// grid = (heads, y, batch) of work items; the launch is a persistent grid of at most as many CTAs as are
// resident at one time (the tensor memory holds two one-tile CTAs or one two-tile CTA per SM)
template <typename T, int MODE, int NT>
int launch_mode(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, T *out, const UmmaParams &up_in,
                dim3 grid, cudaStream_t stream, const char *what) {
    auto kern = umma_block_fwd_kernel<T, MODE, NT>;
    using C = Cfg<NT, qs_of(MODE, NT)>;
    if (int rc = ensure_dynamic_smem((const void *)kern, C::kSmemBytes, what)) return rc;
    const uint64_t n_work = (uint64_t)grid.x * grid.y * grid.z;
    if (n_work == 0) return MAT_OK;
    if (n_work >= (1ull << 31)) return fail(MAT_ERR_UNSUPPORTED, "%s: too many tiles", what);
    UmmaParams up = up_in;
    up.n_work = (uint32_t)n_work;
    up.grid_y = grid.y;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const unsigned ctas = (unsigned)std::min<uint64_t>(n_work, (uint64_t)sms * (NT == 1 ? 2 : 1));
    kern<<<ctas, C::kThreads, C::kSmemBytes, stream>>>(mq, mk, mv, out, up);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, what);
}

template <typename T>
int launch_t(const Problem &p) {
    CUtensorMap mq, mk, mv;
    if (int rc = make_map(&mq, p.q, p.dtype, p.H, p.Sq, p.B, kTileQ)) return rc;
    if (int rc = make_map(&mk, p.k, p.dtype, p.H, p.Skv, p.B, kTileK)) return rc;
    if (int rc = make_map(&mv, p.v, p.dtype, p.H, p.Skv, p.B, kTileK)) return rc;
    UmmaParams up;
    up.Sq = (int32_t)p.Sq;
    up.Skv = (int32_t)p.Skv;
    up.off = (int32_t)p.pat.q_offset;
    up.H = (int32_t)p.H;
    up.block = (int32_t)p.pat.block;
    up.per_blk = up.block / kTileK;
    up.causal = p.pat.causal;
    up.win_left = up.win_right = 0;
    up.n_qblocks = p.pat.n_qblocks;
    up.rowptr = p.pat.rowptr;
    up.colidx = p.pat.colidx;
    up.sl2 = p.scale * 1.4426950408889634f;
    up.n_global = 0; up.gidx = nullptr; up.split_len = up.n_splits = up.ng_pad = 0; up.partial = nullptr;
    const dim3 grid((unsigned)p.H, (unsigned)((p.Sq + kTileQ - 1) / kTileQ), (unsigned)p.B);
    const int rc = launch_mode<T, kModeBlock, 1>(mq, mk, mv, (T *)p.o, up, grid, p.stream, "umma block kernel");
    if (rc == MAT_OK) note_kernel("umma_block");
    return rc;
}

template <typename T>
int launch_dense_t(const Problem &p) {
    CUtensorMap mq, mk, mv;
    if (int rc = make_map(&mq, p.q, p.dtype, p.H, p.Sq, p.B, kTileQ)) return rc;
    if (int rc = make_map(&mk, p.k, p.dtype, p.H, p.Skv, p.B, kTileK)) return rc;
    if (int rc = make_map(&mv, p.v, p.dtype, p.H, p.Skv, p.B, kTileK)) return rc;
    UmmaParams up;
    up.Sq = (int32_t)p.Sq; up.Skv = (int32_t)p.Skv; up.off = (int32_t)p.pat.q_offset; up.H = (int32_t)p.H;
    up.block = kTileK; up.per_blk = 1; up.causal = 0; up.n_qblocks = 0; up.rowptr = up.colidx = nullptr;
    up.win_left = (int32_t)std::min<int64_t>(p.pat.left, p.Skv); up.win_right = (int32_t)std::min<int64_t>(p.pat.right, p.Skv);
    up.sl2 = p.scale * 1.4426950408889634f;
    up.n_global = 0; up.gidx = nullptr; up.split_len = up.n_splits = up.ng_pad = 0; up.partial = nullptr;
    const int nt = tiles_per_cta();
    const dim3 grid((unsigned)p.H, (unsigned)((p.Sq + nt * kTileQ - 1) / (nt * kTileQ)), (unsigned)p.B);
    const int rc = nt == 2 ? launch_mode<T, kModeDense, 2>(mq, mk, mv, (T *)p.o, up, grid, p.stream, "umma dense kernel")
                           : launch_mode<T, kModeDense, 1>(mq, mk, mv, (T *)p.o, up, grid, p.stream, "umma dense kernel");
    if (rc == MAT_OK) note_kernel(up.win_left >= p.Skv - 1 && (up.win_right >= p.Skv - 1 || up.win_right == 0) ? "umma_dense" : "umma_window");
    return rc;
}

template <typename T>
int launch_global_rows_t(const Problem &p, const GlobalRowSplit &g, float *partial) {
    CUtensorMap mq, mk, mv;
    if (int rc = make_map(&mq, p.q, p.dtype, p.H, p.Sq, p.B, 1)) return rc;   // one-row view: gathered tile
    if (int rc = make_map(&mk, p.k, p.dtype, p.H, p.Skv, p.B, kTileK)) return rc;
    if (int rc = make_map(&mv, p.v, p.dtype, p.H, p.Skv, p.B, kTileK)) return rc;
    UmmaParams up;
    up.Sq = (int32_t)p.Sq; up.Skv = (int32_t)p.Skv; up.off = 0; up.H = (int32_t)p.H;
    up.block = kTileK; up.per_blk = 1; up.causal = 0; up.n_qblocks = 0; up.rowptr = up.colidx = nullptr;
    up.win_left = up.win_right = 0;
    up.sl2 = p.scale * 1.4426950408889634f;
    up.n_global = (int32_t)p.pat.n_global;
    up.gidx = p.pat.gidx;
    up.split_len = g.split_len; up.n_splits = g.n_splits; up.ng_pad = g.ng_pad;
    up.partial = partial;
    const dim3 grid((unsigned)p.H, (unsigned)(g.tiles * g.n_splits), (unsigned)p.B);
    return launch_mode<T, kModeGlobalRows, 1>(mq, mk, mv, (T *)nullptr, up, grid, p.stream, "umma global-row kernel");
}

}  // namespace

// The rows at the Longformer global positions over every key, on tcgen05: 128 gathered query rows
// per CTA, the key axis cut into splits (64 a multiple), partials left for the merge kernel.
GlobalRowSplit plan_umma_global_rows(const Problem &p) {
    GlobalRowSplit g;
    g.tile_rows = kTileQ;
    g.tiles = (int)((p.pat.n_global + kTileQ - 1) / kTileQ);
    g.ng_pad = (int)((p.pat.n_global + 31) / 32 * 32);
    // Splits of the key axis: as many CTAs as fill whole waves of the resident slots (2 per SM); a
    // wave that is nearly empty costs as much as a full one.  Cost model: waves x (steps + 4), the
    // 4 standing for a CTA's start and read-out; at least 8 steps per split.
    const int64_t units = std::max<int64_t>(1, p.B * p.H * g.tiles);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t slots = 2 * (int64_t)sms, n_chunks = (p.Skv + kTileK - 1) / kTileK;
    int64_t best_steps = n_chunks, best_cost = INT64_MAX;
    for (int64_t w = 1; w <= 4; ++w) {
        int64_t splits = std::max<int64_t>(1, slots * w / units);
        splits = std::min(splits, std::max<int64_t>(1, n_chunks / 8));
        const int64_t steps = (n_chunks + splits - 1) / splits;
        const int64_t real_splits = (n_chunks + steps - 1) / steps;
        const int64_t waves = (units * real_splits + slots - 1) / slots;
        const int64_t cost = waves * (steps + 4);
        if (cost < best_cost) { best_cost = cost; best_steps = steps; }
    }
    const int64_t len = best_steps * kTileK;
    g.split_len = (int)len;
    g.n_splits = (int)((p.Skv + len - 1) / len);
    g.bytes = (size_t)p.B * p.H * g.n_splits * g.ng_pad * kPartialStride * sizeof(float);
    return g;
}

int launch_umma_global_rows(const Problem &p, const GlobalRowSplit &g, float *partial) {
    return p.dtype == MAT_BF16 ? launch_global_rows_t<__nv_bfloat16>(p, g, partial)
                               : launch_global_rows_t<__half>(p, g, partial);
}

// Column ids must ascend within each layout row (the merge of the two rows a CTA covers relies
// on it); the python front end sorts them, C callers are told so in the header.
bool umma_block_supports(const Problem &p) {
    if (p.pat.kind != MAT_BLOCK) return false;
    if (p.dtype != MAT_BF16 && p.dtype != MAT_F16) return false;
    if (p.D != 64 || p.pat.block % 64 != 0 || p.pat.q_offset % 64 != 0) return false;
    const uintptr_t al = (uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o;
    if (al % 16) return false;
    if (p.Skv >= (1LL << 28) || p.B > 65535 || p.H > 0x7fffffffLL || (p.Sq + kTileQ - 1) / kTileQ > 65535) return false;
    if (p.pat.block >= (1 << 24)) return false;
    const char *force = std::getenv("MAT_BLOCK_KERNEL");  // debugging aid: "mma" keeps the warp-level kernel
    return !(force && force[0] == 'm');
}

// Dense and causal-dense attention (the window that covers the whole sequence, the reference's
// dense_forward, src/cuda/sparse_attention_kernel.cu:348-382) and windows of more than 128 taps between
// their two sides on the same tcgen05 pipeline: every 128-row tile walks the keys its rows can see 64 at
// a time; the chunks on an edge of the window are masked.  Narrower windows stay on the warp-level
// kernels: a walk of four steps does not amortise the pipeline's start and read-out.  MAT_WINDOW_KERNEL=mma keeps
// every window that is not dense on the warp-level kernels (debugging and measurement aid).
bool umma_dense_supports(const Problem &p) {
    if (p.pat.kind != MAT_WINDOW || p.pat.dilation != 1) return false;
    if (p.dtype != MAT_BF16 && p.dtype != MAT_F16) return false;
    if (p.D != 64 || p.pat.q_offset % 64 != 0) return false;
    if (p.k_prev || p.k_next) return false;   // neighbour shards are read by the warp-level kernel only
    const int64_t left = std::min<int64_t>(p.pat.left, p.Skv - 1), right = std::min<int64_t>(p.pat.right, p.Skv - 1);
    const bool dense = left >= p.Skv - 1 && (right >= p.Skv - 1 || right == 0);
    if (!dense) {
        if (left + right <= 128) return false;   // measured: the warp-level tiles win up to 128 taps (86 against 117 us at 64K x 8)
        const char *force = std::getenv("MAT_WINDOW_KERNEL");
        if (force && std::strcmp(force, "mma") == 0) return false;
    }
    if (p.Skv < 256) return false;   // short sequences: the window kernels are as good and need no TMEM
    const uintptr_t al = (uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o;
    if (al % 16) return false;
    return p.Skv < (1LL << 28) && p.B <= 65535 && (p.Sq + kTileQ - 1) / kTileQ <= 65535;
}

int launch_umma_dense(const Problem &p) {
    return p.dtype == MAT_BF16 ? launch_dense_t<__nv_bfloat16>(p) : launch_dense_t<__half>(p);
}

int launch_umma_block(const Problem &p) {
    return p.dtype == MAT_BF16 ? launch_t<__nv_bfloat16>(p) : launch_t<__half>(p);
}

}  // namespace mat
#ifdef MAT_BLOCK_TRACE
extern "C" int mat_debug_block_trace(unsigned long long *out) {
    return (int)cudaMemcpyFromSymbol(out, mat::g_btrace, sizeof(mat::g_btrace));
}
#endif
namespace mat {
int umma_status_read_and_clear(int *out) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(out, g_umma_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(int));
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, "reading the kernel status word");
}

}  // namespace mat
