// Tiled forward for fp32 inputs, the reference's own precision
// (src/csrc/attention_types.hpp:10): window patterns of at most 128 taps between
// their two sides, head width 32, 64 or 128.
//
// Replaces sparse_attention_forward_warp (src/cuda/sparse_attention_kernel.cu:211-263),
// which fetches every K/V row from global memory once per query row that sees it
// and rewrites the output row in global memory once per key.  Here one CTA owns
// 64 consecutive query rows of one head; TMA stages the tile's Q rows and the
// K/V rows its windows reach (64 + left + right of them) in shared memory once,
// and all 64 rows read them from there.  The arithmetic stays on the fp32 FMA
// pipe (no TF32: the parity bar is 1e-5 relative): the tensor cores cannot hold
// that bar, so this path is bounded by FMA issue, not by HBM.
//
//   - 8 warps x 8 query rows.  A warp's rows see keys kw .. kw + 7 + left + right;
//     for Q K^T lane l scores keys kw + l, kw + l + 32, ... (NS per lane) for all 8 rows
//     at once: per 4 head columns one 16-byte shared-memory load per key and one
//     (broadcast) per row feed 8 x NS x 4 FMAs.
//   - Row maximum and sum by warp shuffles; the weights go to shared memory (over the K
//     tile, which every warp has finished with by then).
//   - For P V lane l owns D/32 output columns of all 8 rows: per 4 keys one broadcast
//     16-byte load of weights per row and one load of V per key feed 8 x 4 x D/32 FMAs.
//   - TMA boxes are 32 floats (128 bytes) wide with the 128-byte swizzle, so a tile is
//     stored as D/32 sub-tiles and both access patterns above (32 lanes on 32 different
//     rows, or 32 lanes along one row) are free of bank conflicts.
//   - A dilated window is the plain window over the [B, S/dil, dil*H, D] view, as in the
//     16-bit kernels.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <mutex>

#include "mat_common.cuh"
#include "ptx.cuh"

namespace mat {
namespace {

constexpr int kSubBytes = 128; // bytes of a row inside one sub-tile (32 floats)

__device__ int g_tiled_status = 0;

struct TiledParams {
    int32_t Sq1, Skv1, off1;   // rows of one sub-sequence (dilation view) and q_offset in it
    int32_t left, right;
    int32_t HH;
    float sl2;                 // scale * log2(e)
};

// Two fp32 FMAs in one instruction on a pair of registers: d = a * b + d, lane-wise on (lo, hi).
// Half the issue slots of scalar FMAs; this kernel is bound by instruction issue.
typedef unsigned long long f32x2;
__device__ __forceinline__ void fma2(f32x2 &d, f32x2 a, f32x2 b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ f32x2 dup2(float x) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float2 unpack2(f32x2 v) {
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
    return r;
}

// byte offset of float f (0..31) of row r inside a 128-byte-swizzled sub-tile
__device__ __forceinline__ uint32_t swz_f(int r, int f) {
    return (uint32_t)(r * kSubBytes + (((f >> 2) ^ (r & 7)) << 4) + ((f & 3) << 2));
}

// The weights of all warps (8 rows x 32 NS floats each) go over the Q and K tiles when they fit there,
// else behind the V tile.
template <int D, int TQ, int NS, int KBOX>
constexpr bool weights_alias() { return TQ * NS * 32 * 4 <= (D / 32) * (TQ + KBOX) * kSubBytes; }
template <int D, int TQ, int NS, int KBOX>
constexpr size_t tiled_smem_bytes() {
    return 1024 + (size_t)(D / 32) * (TQ + 2 * KBOX) * kSubBytes +
           (weights_alias<D, TQ, NS, KBOX>() ? 0 : (size_t)TQ * NS * 32 * 4) + 16;
}

// D: head width; TQ: query rows per CTA; R: rows per warp; NS: keys per lane in the score phase
// (32 NS >= R + left + right); KBOX: key rows staged per tile (>= TQ + left + right)
template <int D, int TQ, int R, int NS, int KBOX>
__global__ void __launch_bounds__(TQ / R * 32, TQ == 64 ? 2 : 1)
tiled_f32_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, float *__restrict__ out, const TiledParams P) {
    constexpr int NSUB = D / 32;          // sub-tiles (32 head columns each)
    constexpr int DPL = D / 32;           // output columns per lane
    constexpr int kTQ = TQ;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem;                                   // [NSUB][64 rows][128 B]
    uint8_t *sK = sQ + NSUB * kTQ * kSubBytes;            // [NSUB][KBOX rows][128 B]
    uint8_t *sV = sK + NSUB * KBOX * kSubBytes;
    uint64_t *bar = (uint64_t *)(sV + NSUB * KBOX * kSubBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hh = blockIdx.x, b = blockIdx.z;
    const int q0 = blockIdx.y * kTQ;
    const int ks0 = q0 + P.off1 - P.left;     // key position of staged row 0 (may be negative: zero rows)

    if (threadIdx.x == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        ptx::mbar_expect_tx(bar, NSUB * (kTQ + 2 * KBOX) * kSubBytes);
#pragma unroll
        for (int s = 0; s < NSUB; ++s) {
            ptx::tma_load_4d(sQ + s * kTQ * kSubBytes, &map_q, bar, 32 * s, hh, q0, b);
            ptx::tma_load_4d(sK + s * KBOX * kSubBytes, &map_k, bar, 32 * s, hh, ks0, b);
            ptx::tma_load_4d(sV + s * KBOX * kSubBytes, &map_v, bar, 32 * s, hh, ks0, b);
        }
    }
    // a wait that runs out is recorded and the CTA carries on with whatever it has (the output is then wrong,
    // which the status word says): nobody is left behind at the barrier below
    if (!ptx::mbar_wait(bar, 0)) atomicExch(&g_tiled_status, 1);

    const int row0 = warp * R;                // first row of this warp inside the tile
    // the warp's rows see staged key rows row0 .. row0 + 7 + left + right; lane l takes row0 + l + 32 s
    const int span = P.left + P.right;
    int kr[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) kr[s] = min(row0 + lane + 32 * s, KBOX - 1);   // beyond the tile: masked below

    // ---- scores: acc[r][s] = q_(row0 + r) . k_(kr[s]); even and odd head columns are summed apart (packed
    // FMAs on the (x, y) and (z, w) halves of every 16-byte load) and joined at the end ----
    float acc[R][NS];
    {
        f32x2 acc2[R][NS];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int s = 0; s < NS; ++s) acc2[r][s] = 0ull;
        // row kr[s] of sub-tile `sub`, 16-byte chunk c: base + c * 16 xor (kr & 7) * 16
        const uint8_t *kbase[NS];
        uint32_t kx[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            kbase[s] = sK + kr[s] * kSubBytes;
            kx[s] = (uint32_t)(kr[s] & 7) << 4;
        }
        // (the sub-tile loop stays rolled and the key loop below is unrolled by 8 only: the loop bodies must stay
        // well inside the instruction cache)
#pragma unroll 1
        for (int sub = 0; sub < NSUB; ++sub) {
            const uint8_t *qq = sQ + sub * kTQ * kSubBytes + row0 * kSubBytes;
#pragma unroll
            for (int c = 0; c < 8; ++c) {          // 4 head columns per step
                ulonglong2 kf[NS];
#pragma unroll
                for (int s = 0; s < NS; ++s)
                    kf[s] = *reinterpret_cast<const ulonglong2 *>(kbase[s] + sub * KBOX * kSubBytes + (((uint32_t)c << 4) ^ kx[s]));
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    // row0 is a multiple of 8, so (row0 + r) & 7 == r & 7; every lane reads the same 16 bytes (a broadcast)
                    const ulonglong2 qf = *reinterpret_cast<const ulonglong2 *>(qq + r * kSubBytes + ((c ^ (r & 7)) << 4));
#pragma unroll
                    for (int s = 0; s < NS; ++s) {
                        fma2(acc2[r][s], qf.x, kf[s].x);
                        fma2(acc2[r][s], qf.y, kf[s].y);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                const float2 h = unpack2(acc2[r][s]);
                acc[r][s] = h.x + h.y;
            }
    }

    // ---- mask, softmax statistics; the weights replace the scores ----
    float inv_l[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        // staged row j holds key ks0 + j; row (row0 + r) attends staged rows row0 + r .. row0 + r + span
        // whose keys exist
        float m = -INFINITY;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            const int j = row0 + lane + 32 * s;
            const int key = ks0 + j;
            const bool ok = (uint32_t)(j - row0 - r) <= (uint32_t)span && key >= 0 && key < P.Skv1 && j < KBOX;
            acc[r][s] = ok ? acc[r][s] : -INFINITY;
            m = fmaxf(m, acc[r][s]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float mu = m == -INFINITY ? 0.f : m;
        float l = 0.f;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            // the difference first: exact for scores near the maximum, whatever their magnitude
            acc[r][s] = ptx::ex2((acc[r][s] - mu) * P.sl2);
            l += acc[r][s];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        inv_l[r] = l > 0.f ? 1.f / l : 0.f;
    }

    // ---- the weights to shared memory (over the Q and K tiles where they fit), key-major: pw[32 s + lane][r],
    // so that one 16-byte load brings one key's weights for four rows, already paired for the packed FMAs ----
    static_assert(R == 8, "the weight layout below is written for 8 rows per warp");
    __syncthreads();   // every warp has read its last Q and K row
    float *pw = reinterpret_cast<float *>(weights_alias<D, TQ, NS, KBOX>() ? sQ : (uint8_t *)(bar + 2)) +
                warp * (R * NS * 32);
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        float4 *dst = reinterpret_cast<float4 *>(pw + (32 * s + lane) * R);
        dst[0] = make_float4(acc[0][s], acc[1][s], acc[2][s], acc[3][s]);
        dst[1] = make_float4(acc[4][s], acc[5][s], acc[6][s], acc[7][s]);
    }
    __syncwarp();

    // ---- output: o[r][.] = sum_j w[j][r] v_(row0 + j); lane l owns columns DPL l .. DPL l + DPL - 1 of all 8
    // rows, held as pairs of rows ----
    f32x2 o2[R / 2][DPL];
#pragma unroll
    for (int rp = 0; rp < R / 2; ++rp)
#pragma unroll
        for (int e = 0; e < DPL; ++e) o2[rp][e] = 0ull;
    const int d0 = lane * DPL;
    const int f0 = d0 & 31;
    // staged row row0 + j of the lane's sub-tile: vrow + j * 128 + (chunk xor (j & 7)) * 16, row0 a multiple of 8
    const uint8_t *vrow = sV + (d0 >> 5) * KBOX * kSubBytes + row0 * kSubBytes + ((f0 & 3) << 2);
    uint32_t vx[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) vx[t] = (uint32_t)(((f0 >> 2) ^ t) << 4);
    const int n_keys = R + span;      // staged rows this warp's rows can see (never past the tile: KBOX >= TQ + span)
#pragma unroll 1
    for (int j8 = 0; j8 < n_keys; j8 += 8) {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const int j = j8 + t;                        // (j & 7) == t; keys past the window carry zero weights
        const float *src = reinterpret_cast<const float *>(vrow + j * kSubBytes + vx[t]);
        f32x2 vv[DPL];
        if constexpr (DPL == 1) {
            vv[0] = dup2(src[0]);
        } else if constexpr (DPL == 2) {
            const float2 x = *reinterpret_cast<const float2 *>(src);
            vv[0] = dup2(x.x); vv[1] = dup2(x.y);
        } else {
            const float4 x = *reinterpret_cast<const float4 *>(src);
            vv[0] = dup2(x.x); vv[1] = dup2(x.y); vv[2] = dup2(x.z); vv[3] = dup2(x.w);
        }
        const ulonglong2 wa = *reinterpret_cast<const ulonglong2 *>(pw + j * R);       // rows 0..3 (broadcast)
        const ulonglong2 wb = *reinterpret_cast<const ulonglong2 *>(pw + j * R + 4);   // rows 4..7
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            fma2(o2[0][e], wa.x, vv[e]);
            fma2(o2[1][e], wa.y, vv[e]);
            fma2(o2[2][e], wb.x, vv[e]);
            fma2(o2[3][e], wb.y, vv[e]);
        }
      }
    }
    float o[R][DPL];
#pragma unroll
    for (int rp = 0; rp < R / 2; ++rp)
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            const float2 h = unpack2(o2[rp][e]);
            o[2 * rp][e] = h.x;
            o[2 * rp + 1][e] = h.y;
        }

    // ---- normalise and store: a row is D contiguous floats, the warp writes it whole ----
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = q0 + row0 + r;
        if (row >= P.Sq1) break;
        float *dst = out + (((int64_t)b * P.Sq1 + row) * P.HH + hh) * D + d0;
        if constexpr (DPL == 1) {
            dst[0] = o[r][0] * inv_l[r];
        } else if constexpr (DPL == 2) {
            *reinterpret_cast<float2 *>(dst) = make_float2(o[r][0] * inv_l[r], o[r][1] * inv_l[r]);
        } else {
            *reinterpret_cast<float4 *>(dst) = make_float4(o[r][0] * inv_l[r], o[r][1] * inv_l[r], o[r][2] * inv_l[r],
                                                           o[r][3] * inv_l[r]);
        }
    }
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

// fp32 [B, S1, HH, D] rows as dims {D, HH, S1, B}; box {32, 1, rows, 1}: 128 bytes wide, 128-byte swizzle,
// zeros for rows outside the tensor
int make_map_f32(CUtensorMap *m, const void *base, int64_t D, int64_t HH, int64_t S1, int64_t B, int rows) {
    PFN_cuTensorMapEncodeTiled enc = encode_fn();
    if (!enc) return fail(MAT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)HH, (cuuint64_t)S1, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 4, (cuuint64_t)HH * D * 4, (cuuint64_t)S1 * HH * D * 4};
    const cuuint32_t box[4] = {32, 1, (cuuint32_t)rows, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MAT_ERR_CUDA, "cuTensorMapEncodeTiled (fp32) failed with code %d", (int)r);
    return MAT_OK;
}

template <int D, int TQ, int R, int NS, int KBOX>
int launch_tiled(const Problem &p, const TiledParams &tp, int64_t dil) {
    constexpr int kTQ = TQ;
    CUtensorMap mq, mk, mv;
    if (int rc = make_map_f32(&mq, p.q, D, tp.HH, p.Sq / dil, p.B, kTQ)) return rc;
    if (int rc = make_map_f32(&mk, p.k, D, tp.HH, p.Skv / dil, p.B, KBOX)) return rc;
    if (int rc = make_map_f32(&mv, p.v, D, tp.HH, p.Skv / dil, p.B, KBOX)) return rc;
    auto kern = tiled_f32_kernel<D, TQ, R, NS, KBOX>;
    constexpr size_t smem = tiled_smem_bytes<D, TQ, NS, KBOX>();
    if (int rc = ensure_dynamic_smem((const void *)kern, smem, "cudaFuncSetAttribute(tiled_f32_kernel)")) return rc;
    const dim3 grid((unsigned)tp.HH, (unsigned)((tp.Sq1 + kTQ - 1) / kTQ), (unsigned)p.B);
    kern<<<grid, TQ / R * 32, smem, p.stream>>>(mq, mk, mv, (float *)p.o, tp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "tiled_f32_kernel launch");
    note_kernel("tiled_f32");
    return MAT_OK;
}

template <int D>
int launch_tiled_d(const Problem &p, const TiledParams &tp, int64_t dil) {
    // up to 64 taps between the sides: 64-row tiles, 8 + 64 <= 96 keys per warp, 128 rows staged, two CTAs per SM;
    // up to 128: 128-row tiles (16 warps, one CTA per SM), 8 + 128 <= 160 keys per warp, 256 rows staged
    // (16 rows per warp, i.e. half the shared-memory loads per FMA at half the warps, measured slower:
    // 513 against 481 us at 65536 tokens x 8 heads)
    if (tp.left + tp.right <= 64) return launch_tiled<D, 64, 8, 3, 128>(p, tp, dil);
    return launch_tiled<D, 128, 8, 5, 256>(p, tp, dil);
}

}  // namespace

bool tiled_f32_supports(const Problem &p) {
    if (p.dtype != MAT_F32 || p.pat.kind != MAT_WINDOW) return false;
    if (p.D != 32 && p.D != 64 && p.D != 128) return false;
    const uintptr_t al = (uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o;
    if (al % 16) return false;
    const int64_t dil = p.pat.dilation;
    if (p.Sq % dil || p.Skv % dil || p.pat.q_offset % dil) return false;
    if (p.Skv / dil >= (1LL << 28) || p.H * dil >= (1LL << 31) || p.B > 65535) return false;
    if ((p.Sq / dil + 63) / 64 > 65535) return false;
    const int64_t left = std::min<int64_t>(p.pat.left, p.Skv / dil), right = std::min<int64_t>(p.pat.right, p.Skv / dil);
    if (left + right > 128) return false;
    if (p.D == 128 && left + right > 64) return false;    // Q + K + V of the wider tile would not fit two CTAs per SM
    return true;
}

int launch_tiled_f32(const Problem &p) {
    const int64_t dil = p.pat.dilation;
    TiledParams tp;
    tp.Sq1 = (int32_t)(p.Sq / dil);
    tp.Skv1 = (int32_t)(p.Skv / dil);
    tp.off1 = (int32_t)(p.pat.q_offset / dil);
    tp.left = (int32_t)std::min<int64_t>(p.pat.left, tp.Skv1);
    tp.right = (int32_t)std::min<int64_t>(p.pat.right, tp.Skv1);
    tp.HH = (int32_t)(p.H * dil);
    tp.sl2 = p.scale * 1.4426950408889634f;
    if (p.D == 32) return launch_tiled_d<32>(p, tp, dil);
    if (p.D == 64) return launch_tiled_d<64>(p, tp, dil);
    return launch_tiled<128, 64, 8, 3, 128>(p, tp, dil);
}

int tiled_status_read_and_clear(int *out) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(out, g_tiled_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_tiled_status, &zero, sizeof(int));
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, "reading the kernel status word");
}

}  // namespace mat
