// Backward of window attention (sliding, causal, dilated, and dense as the window
// that covers the sequence): dQ, dK, dV from Q, K, V and dO.
//
// Replaces sparse_attention_backward_kernel / dense_attention_backward_kernel
// (src/cuda/sparse_attention_kernel.cu:265-346, 104-208), which run one THREAD per
// query row, recompute the probabilities three times and scatter dK/dV with fp32
// atomicAdd (:322, :343).  Here nothing is atomic and the result is deterministic:
//
//   bwd_rows_kernel  one warp per (b, h, query i): log-sum-exp of the row, then
//                    delta_i = sum_j p_ij (dO_i . v_j), then
//                    dQ_i = scale * sum_j p_ij (dO_i . v_j - delta_i) k_j;
//                    leaves (lse_i, delta_i) in the workspace.
//   bwd_cols_kernel  one warp per (b, h, key j): walks the queries that attend to j
//                    (the window mirrored), recomputes p_ij from lse_i and gathers
//                    dK_j = scale * sum_i p_ij (dO_i . v_j - delta_i) q_i,
//                    dV_j = sum_i p_ij dO_i.
//
// Written for clarity and exactness (fp32 math for every dtype), any head width up
// to 512.  16-bit inputs with head width 64 go to the tensor-core kernels of bwd_mma.cu instead.
//
// The same two kernels run block-sparse layouts and the Longformer pattern (the reference has no
// backward for those: src/csrc/attention_interface.hpp:14-52 throws): a row's keys and a key's queries
// are enumerated by PartnerSet below instead of by window arithmetic.  The queries of a key need the
// transposed block layout, which the caller passes in (mat_sparse_attn_bwd_general).
#include "mat_common.cuh"

namespace mat {
namespace {

constexpr int kWarps = 8;

__device__ __forceinline__ float wmax(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float wsum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

template <typename T>
__device__ __forceinline__ float dot_row(const float *a, const T *b, int D) {
    float s = 0.f;
    for (int d = 0; d < D; ++d) s = fmaf(a[d], Elem<T>::to_f(b[d]), s);
    return s;
}

struct WindowArgs {
    int64_t B, S, H;
    int D;
    int64_t left, right, dil;
    float scale;
    // other patterns (kind != MAT_WINDOW)
    int kind = MAT_WINDOW;
    int causal = 0;
    int64_t block = 0, n_blocks = 0;          // block layouts: block edge, blocks along the sequence
    const int32_t *rowptr = nullptr, *colidx = nullptr;      // query block -> its key blocks (ascending)
    const int32_t *t_rowptr = nullptr, *t_colidx = nullptr;  // key block -> the query blocks that hold it
    int64_t n_global = 0;
    const int64_t *gidx = nullptr;            // Longformer: sorted global positions
};

// The partners of position x: the keys of query x (COLS = false) or the queries of key x (COLS = true), as a
// count n and at(idx) for idx in [0, n), which returns the partner's position or -1 for a slot that holds none
// (a key past the causal diagonal of a block, a global position the window already covers).
template <bool COLS>
struct PartnerSet {
    int64_t n, first, dil;       // window part: first + idx * dil for idx < n_win
    int64_t n_win;
    int64_t x;
    const WindowArgs *a;
    int64_t e0;                  // block layouts: first entry of x's layout row
    int64_t w_lo, w_hi;          // Longformer: the window part as a closed range, for the de-duplication
    bool all;                    // Longformer: x is a global position, every position is a partner

    __device__ bool is_global(int64_t p) const {
        int64_t lo = 0, hi = a->n_global;
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if (a->gidx[mid] < p) lo = mid + 1; else hi = mid;
        }
        return lo < a->n_global && a->gidx[lo] == p;
    }
    __device__ void init(const WindowArgs &args, int64_t pos) {
        a = &args;
        x = pos;
        all = false;
        e0 = 0;
        dil = args.dil;
        if (args.kind == MAT_BLOCK) {
            const int64_t r = x / args.block;
            const int32_t *ptr = COLS ? args.t_rowptr : args.rowptr;
            e0 = r < args.n_blocks ? ptr[r] : 0;
            n_win = 0;
            first = 0;
            n = r < args.n_blocks ? (int64_t)(ptr[r + 1] - e0) * args.block : 0;
            return;
        }
        // window part: query x sees keys x + t*dil, -left <= t <= right; key x is seen by queries x - t*dil
        int64_t lo = COLS ? -args.right : -args.left, hi = COLS ? args.left : args.right;
        if (x + lo * dil < 0) lo = -(x / dil);
        if (x + hi * dil >= args.S) hi = (args.S - 1 - x) / dil;
        n_win = hi >= lo ? hi - lo + 1 : 0;
        first = x + lo * dil;
        n = n_win;
        if (args.kind == MAT_LONGFORMER) {
            w_lo = first;
            w_hi = first + (n_win - 1);
            // a global query attends every key, and every query attends a global key
            if (is_global(x)) {
                all = true;
                n = args.S;
            } else {
                n = n_win + args.n_global;   // keys: the global keys; queries: the global rows
            }
        }
    }
    __device__ int64_t at(int64_t idx) const {
        if (a->kind == MAT_BLOCK) {
            const int32_t *ci = COLS ? a->t_colidx : a->colidx;
            const int64_t p = (int64_t)ci[e0 + idx / a->block] * a->block + idx % a->block;
            if (p >= a->S) return -1;
            if (a->causal && (COLS ? p < x : p > x)) return -1;   // key <= query
            return p;
        }
        if (all) return idx;
        if (idx < n_win) return first + idx * dil;
        const int64_t g = a->gidx[idx - n_win];
        return (g < 0 || g >= a->S || (g >= w_lo && g <= w_hi)) ? -1 : g;
    }
};

template <typename T, int MAXR>
__global__ void __launch_bounds__(kWarps * 32)
bwd_rows_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                const T *__restrict__ dout, T *__restrict__ dq, float2 *__restrict__ stats, WindowArgs a) {
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float *qs = sm + (size_t)warp * 2 * a.D, *gs = qs + a.D;   // q row, dO row
    const int64_t row = (int64_t)blockIdx.x * kWarps + warp;
    if (row >= a.B * a.S * a.H) return;
    const int64_t i = row % a.S, h = (row / a.S) % a.H, b = row / (a.S * a.H);
    const int64_t base = ((b * a.S + i) * a.H + h) * a.D;
    for (int d = lane; d < a.D; d += 32) {
        qs[d] = Elem<T>::to_f(q[base + d]);
        gs[d] = Elem<T>::to_f(dout[base + d]);
    }
    __syncwarp();
    const int64_t stride = a.H * (int64_t)a.D;
    const T *kb = k + (b * a.S * a.H + h) * (int64_t)a.D;
    const T *vb = v + (b * a.S * a.H + h) * (int64_t)a.D;
    PartnerSet<false> keys;
    keys.init(a, i);
    const int64_t n = keys.n;

    // pass A: log-sum-exp of the scaled scores
    float m = -INFINITY, l = 0.f;
    for (int64_t c = 0; c < n; c += 32) {
        const int64_t idx = c + lane;
        const int64_t j = idx < n ? keys.at(idx) : -1;
        const float s = j >= 0 ? dot_row(qs, kb + j * stride, a.D) * a.scale : -INFINITY;
        const float m_new = fmaxf(m, wmax(s));
        if (m_new != -INFINITY) {   // (a chunk of empty slots before the first key leaves the sums untouched)
            l = l * expf(m - m_new) + wsum(j >= 0 ? expf(s - m_new) : 0.f);
            m = m_new;
        }
    }
    const float lse = m != -INFINITY ? m + logf(l) : 0.f;
    // pass B: delta = sum_j p_j (dO . v_j)
    float delta = 0.f;
    for (int64_t c = 0; c < n; c += 32) {
        const int64_t idx = c + lane;
        const int64_t j = idx < n ? keys.at(idx) : -1;
        if (j >= 0) {
            const float p = expf(dot_row(qs, kb + j * stride, a.D) * a.scale - lse);
            delta += p * dot_row(gs, vb + j * stride, a.D);
        }
    }
    delta = wsum(delta);
    if (lane == 0) stats[row] = make_float2(lse, delta);
    // pass C: dQ = scale * sum_j p_j (dO . v_j - delta) k_j
    float acc[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;
    for (int64_t c = 0; c < n; c += 32) {
        const int64_t idx = c + lane;
        float ds = 0.f;
        const int64_t j = idx < n ? keys.at(idx) : -1;
        if (j >= 0) {
            const float p = expf(dot_row(qs, kb + j * stride, a.D) * a.scale - lse);
            ds = p * (dot_row(gs, vb + j * stride, a.D) - delta) * a.scale;
        }
        const int steps = n - c < 32 ? (int)(n - c) : 32;
        for (int t = 0; t < steps; ++t) {
            const int64_t jt = __shfl_sync(0xffffffffu, j, t);
            const float dst = __shfl_sync(0xffffffffu, ds, t);
            if (jt < 0) continue;   // an empty slot (the same for every lane)
            const T *kr = kb + jt * stride;
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                const int d = lane + 32 * r;
                if (d < a.D) acc[r] = fmaf(dst, Elem<T>::to_f(kr[d]), acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        const int d = lane + 32 * r;
        if (d < a.D) dq[base + d] = Elem<T>::from_f(acc[r]);
    }
}

template <typename T, int MAXR>
__global__ void __launch_bounds__(kWarps * 32)
bwd_cols_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                const T *__restrict__ dout, T *__restrict__ dk, T *__restrict__ dv,
                const float2 *__restrict__ stats, WindowArgs a) {
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float *ks = sm + (size_t)warp * 2 * a.D, *vs = ks + a.D;   // k row, v row
    const int64_t row = (int64_t)blockIdx.x * kWarps + warp;
    if (row >= a.B * a.S * a.H) return;
    const int64_t j = row % a.S, h = (row / a.S) % a.H, b = row / (a.S * a.H);
    const int64_t base = ((b * a.S + j) * a.H + h) * a.D;
    for (int d = lane; d < a.D; d += 32) {
        ks[d] = Elem<T>::to_f(k[base + d]);
        vs[d] = Elem<T>::to_f(v[base + d]);
    }
    __syncwarp();
    const int64_t stride = a.H * (int64_t)a.D;
    const T *qb = q + (b * a.S * a.H + h) * (int64_t)a.D;
    const T *gb = dout + (b * a.S * a.H + h) * (int64_t)a.D;
    const float2 *st = stats + (b * a.H + h) * a.S;   // stats are stored per (b, h, i) with i fastest
    // the queries that attend key j (a window: i = j - t*dil with -left <= t <= right)
    PartnerSet<true> rows;
    rows.init(a, j);
    const int64_t n = rows.n;

    float ak[MAXR], av[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) ak[r] = av[r] = 0.f;
    for (int64_t c = 0; c < n; c += 32) {
        const int64_t idx = c + lane;
        float p = 0.f, ds = 0.f;
        const int64_t i = idx < n ? rows.at(idx) : -1;
        if (i >= 0) {
            const float2 s2 = st[i];
            p = expf(dot_row(ks, qb + i * stride, a.D) * a.scale - s2.x);
            ds = p * (dot_row(vs, gb + i * stride, a.D) - s2.y) * a.scale;
        }
        const int steps = n - c < 32 ? (int)(n - c) : 32;
        for (int t = 0; t < steps; ++t) {
            const int64_t it = __shfl_sync(0xffffffffu, i, t);
            const float pt = __shfl_sync(0xffffffffu, p, t);
            const float dst = __shfl_sync(0xffffffffu, ds, t);
            if (it < 0) continue;
            const T *qr = qb + it * stride;
            const T *gr = gb + it * stride;
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                const int d = lane + 32 * r;
                if (d < a.D) {
                    ak[r] = fmaf(dst, Elem<T>::to_f(qr[d]), ak[r]);
                    av[r] = fmaf(pt, Elem<T>::to_f(gr[d]), av[r]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        const int d = lane + 32 * r;
        if (d < a.D) {
            dk[base + d] = Elem<T>::from_f(ak[r]);
            dv[base + d] = Elem<T>::from_f(av[r]);
        }
    }
}

template <typename T, int MAXR>
int launch_r(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
             float2 *stats, const WindowArgs &a, cudaStream_t stream) {
    const int64_t rows = a.B * a.S * a.H;
    const int64_t ctas = (rows + kWarps - 1) / kWarps;
    if (ctas > 0x7fffffffLL) return fail(MAT_ERR_UNSUPPORTED, "too many rows for one launch");
    const size_t smem = (size_t)kWarps * 2 * a.D * sizeof(float);
    bwd_rows_kernel<T, MAXR><<<(unsigned)ctas, kWarps * 32, smem, stream>>>(
        (const T *)q, (const T *)k, (const T *)v, (const T *)dout, (T *)dq, stats, a);
    bwd_cols_kernel<T, MAXR><<<(unsigned)ctas, kWarps * 32, smem, stream>>>(
        (const T *)q, (const T *)k, (const T *)v, (const T *)dout, (T *)dk, (T *)dv, stats, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "backward launch");
    note_kernel(a.kind == MAT_WINDOW ? "bwd_window" : "bwd_general");
    return MAT_OK;
}

template <typename T>
int launch_t(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
             float2 *stats, const WindowArgs &a, cudaStream_t stream) {
    if (a.D <= 64) return launch_r<T, 2>(q, k, v, dout, dq, dk, dv, stats, a, stream);
    if (a.D <= 128) return launch_r<T, 4>(q, k, v, dout, dq, dk, dv, stats, a, stream);
    if (a.D <= 256) return launch_r<T, 8>(q, k, v, dout, dq, dk, dv, stats, a, stream);
    if (a.D <= 512) return launch_r<T, 16>(q, k, v, dout, dq, dk, dv, stats, a, stream);
    return fail(MAT_ERR_UNSUPPORTED, "head width D=%d exceeds the supported maximum of 512", a.D);
}

}  // namespace
}  // namespace mat

using namespace mat;

extern "C" {

size_t mat_sparse_attn_bwd_workspace_bytes(int64_t B, int64_t S, int64_t H) {
    return B > 0 && S > 0 && H > 0 ? (size_t)B * S * H * sizeof(float2) : 0;
}

size_t mat_sparse_attn_bwd_general_workspace_bytes(int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                                                   const mat_pattern_spec *spec) {
    size_t n = mat_sparse_attn_bwd_workspace_bytes(B, S, H);
    if (n == 0 || !spec) return n;
    n = (n + 255) & ~(size_t)255;
    if (spec->kind == MAT_LONGFORMER && bwd_longformer_mma_supports(B, S, H, D, dtype, spec->n_global))
        n += bwd_longformer_mma_extra_bytes(B, H, spec->n_global);
    // (16-bit heads that go 64 columns at a time, windows of many passes: fp32 copies of the three outputs' shape;
    // a call that brings only the statistics' bytes runs those on the warp-level kernels instead)
    if (spec->kind == MAT_WINDOW && spec->dilation >= 1)
        n += bwd_d_mma_scratch_bytes(B, S, H, D, dtype, spec->dilation, std::min<int64_t>(spec->left, S), std::min<int64_t>(spec->right, S));
    return n;
}

int mat_sparse_attn_bwd(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk,
                        void *dv, int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                        const mat_pattern_spec *spec, float scale, void *workspace, size_t workspace_bytes,
                        void *stream) {
    if (spec && spec->kind == MAT_BLOCK)
        return fail(MAT_ERR_UNSUPPORTED, "the backward of a block layout needs the transposed layout: mat_sparse_attn_bwd_general");
    return mat_sparse_attn_bwd_general(q, k, v, dout, dq, dk, dv, B, S, H, D, dtype, spec, nullptr, nullptr, scale,
                                       workspace, workspace_bytes, stream);
}

int mat_sparse_attn_bwd_general(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk,
                                void *dv, int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                                const mat_pattern_spec *spec, const int32_t *t_rowptr, const int32_t *t_colidx,
                                float scale, void *workspace, size_t workspace_bytes, void *stream) {
    if (!spec) return fail(MAT_ERR_INVALID, "pattern description is NULL");
    if (spec->kind != MAT_WINDOW && spec->kind != MAT_BLOCK && spec->kind != MAT_LONGFORMER)
        return fail(MAT_ERR_INVALID, "unknown pattern kind %d", spec->kind);
    if (spec->q_offset != 0) return fail(MAT_ERR_INVALID, "q_offset must be 0 for the backward pass");
    if (spec->kind != MAT_BLOCK && (spec->left < 0 || spec->right < 0 || spec->dilation < 1))
        return fail(MAT_ERR_INVALID, "bad window description for the backward pass");
    if (spec->kind == MAT_LONGFORMER && (spec->dilation != 1 || spec->n_global < 0 || (spec->n_global > 0 && !spec->global_idx)))
        return fail(MAT_ERR_INVALID, "bad Longformer description for the backward pass");
    if (spec->kind == MAT_BLOCK) {
        if (spec->block < 1 || spec->n_qblocks < 1 || !spec->blk_rowptr || !spec->blk_colidx || !t_rowptr || !t_colidx)
            return fail(MAT_ERR_INVALID, "block layout and its transpose (device pointers) are required");
        if (spec->n_qblocks * spec->block < S) return fail(MAT_ERR_INVALID, "the block layout does not cover the sequence");
    }
    if (!q || !k || !v || !dout || !dq || !dk || !dv) return fail(MAT_ERR_INVALID, "tensor pointers must be non-NULL");
    if (B <= 0 || S <= 0 || H <= 0 || D <= 0) return fail(MAT_ERR_INVALID, "all tensor dimensions must be > 0");
    const size_t full = mat_sparse_attn_bwd_general_workspace_bytes(B, S, H, D, dtype, spec);
    const size_t scratch_bytes = spec->kind == MAT_WINDOW
        ? bwd_d_mma_scratch_bytes(B, S, H, D, dtype, spec->dilation, std::min<int64_t>(spec->left, S), std::min<int64_t>(spec->right, S)) : 0;
    const size_t need = full - scratch_bytes;   // the scratch is optional: without it those problems take the warp-level kernels
    const bool have_scratch = scratch_bytes > 0 && workspace && workspace_bytes >= full;
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace % 256) != 0)
        return fail(MAT_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) required, got %zu", need,
                    workspace ? workspace_bytes : (size_t)0);
    WindowArgs a;
    a.B = B; a.S = S; a.H = H; a.D = (int)D;
    a.left = spec->left > S ? S : spec->left;
    a.right = spec->right > S ? S : spec->right;
    a.dil = spec->kind == MAT_BLOCK ? 1 : spec->dilation;
    a.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)D);
    a.kind = spec->kind;
    a.causal = spec->causal;
    a.block = spec->block;
    a.n_blocks = spec->n_qblocks;
    a.rowptr = spec->blk_rowptr;
    a.colidx = spec->blk_colidx;
    a.t_rowptr = t_rowptr;
    a.t_colidx = t_colidx;
    a.n_global = spec->kind == MAT_LONGFORMER ? spec->n_global : 0;
    a.gidx = spec->global_idx;
    float2 *stats = (float2 *)workspace;
    cudaStream_t st = (cudaStream_t)stream;
    // the tensor-core kernels move 16-byte vectors and TMA boxes: unaligned tensors stay on the warp-level kernels
    const uintptr_t al = (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)dout | (uintptr_t)dq | (uintptr_t)dk |
                         (uintptr_t)dv;
    if (spec->kind == MAT_LONGFORMER && al % 16 == 0 && bwd_longformer_mma_supports(B, S, H, D, dtype, spec->n_global)) {
        const size_t stats_bytes = (mat_sparse_attn_bwd_workspace_bytes(B, S, H) + 255) & ~(size_t)255;
        return launch_bwd_longformer_mma(q, k, v, dout, dq, dk, dv, stats, (uint8_t *)workspace + stats_bytes, B, S, H, dtype,
                                         a.left, a.right, spec->n_global, spec->global_idx, a.scale, st);
    }
    if (spec->kind == MAT_LONGFORMER && spec->n_global == 0 && al % 16 == 0 &&
        bwd_mma_supports(B, S, H, D, dtype, a.left, a.right, 1))   // no global position: a plain window
        return launch_bwd_mma(q, k, v, dout, dq, dk, dv, stats, B, S, H, dtype, a.left, a.right, 1, a.scale, st);
    if (spec->kind == MAT_BLOCK && al % 16 == 0 && bwd_block_mma_supports(B, S, H, D, dtype, spec->block))
        return launch_bwd_block_mma(q, k, v, dout, dq, dk, dv, stats, B, S, H, dtype, spec->block, spec->causal,
                                    spec->blk_rowptr, spec->blk_colidx, t_rowptr, t_colidx, a.scale, st);
    if (spec->kind == MAT_WINDOW && al % 16 == 0 && bwd_d_mma_supports(B, S, H, D, dtype, a.dil, a.left, a.right, have_scratch))
        return launch_bwd_d_mma(q, k, v, dout, dq, dk, dv, stats, B, S, H, D, dtype, a.left, a.right, a.dil, a.scale,
                                have_scratch ? (float *)((uint8_t *)workspace + (full - scratch_bytes)) : nullptr, st);
    if (spec->kind == MAT_WINDOW && al % 16 == 0 && bwd_f32_mma_supports(B, S, H, D, dtype, a.dil))
        return launch_bwd_f32_mma(q, k, v, dout, dq, dk, dv, stats, B, S, H, D, a.left, a.right, a.dil, a.scale, st);
    if (spec->kind == MAT_WINDOW && al % 16 == 0 && bwd_mma_supports(B, S, H, D, dtype, a.left, a.right, a.dil))
        return launch_bwd_mma(q, k, v, dout, dq, dk, dv, stats, B, S, H, dtype, a.left, a.right, a.dil, a.scale, st);
    switch (dtype) {
        case MAT_F32: return launch_t<float>(q, k, v, dout, dq, dk, dv, stats, a, st);
        case MAT_BF16: return launch_t<__nv_bfloat16>(q, k, v, dout, dq, dk, dv, stats, a, st);
        case MAT_F16: return launch_t<__half>(q, k, v, dout, dq, dk, dv, stats, a, st);
    }
    return fail(MAT_ERR_INVALID, "unknown dtype %d", dtype);
}

}  // extern "C"
