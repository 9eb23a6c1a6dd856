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
};

// first tap index and tap count of row p (keys p + t*dil, t in [t_lo, t_lo + n))
__device__ __forceinline__ void taps_of(const WindowArgs &a, int64_t p, int64_t &t_lo, int64_t &n) {
    int64_t lo = -a.left, hi = a.right;
    if (p + lo * a.dil < 0) lo = -(p / a.dil);
    if (p + hi * a.dil >= a.S) hi = (a.S - 1 - p) / a.dil;
    t_lo = lo;
    n = hi >= lo ? hi - lo + 1 : 0;
}

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
    int64_t t_lo, n;
    taps_of(a, i, t_lo, n);
    const int64_t first = i + t_lo * a.dil;

    // pass A: log-sum-exp of the scaled scores
    float m = -INFINITY, l = 0.f;
    for (int64_t c = 0; c < n; c += 32) {
        const int64_t idx = c + lane;
        const float s = idx < n ? dot_row(qs, kb + (first + idx * a.dil) * stride, a.D) * a.scale : -INFINITY;
        const float m_new = fmaxf(m, wmax(s));
        l = l * expf(m - m_new) + wsum(idx < n ? expf(s - m_new) : 0.f);
        m = m_new;
    }
    const float lse = n > 0 ? m + logf(l) : 0.f;
    // pass B: delta = sum_j p_j (dO . v_j)
    float delta = 0.f;
    for (int64_t c = 0; c < n; c += 32) {
        const int64_t idx = c + lane;
        if (idx < n) {
            const int64_t j = first + idx * a.dil;
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
        int64_t j = -1;
        if (idx < n) {
            j = first + idx * a.dil;
            const float p = expf(dot_row(qs, kb + j * stride, a.D) * a.scale - lse);
            ds = p * (dot_row(gs, vb + j * stride, a.D) - delta) * a.scale;
        }
        const int steps = n - c < 32 ? (int)(n - c) : 32;
        for (int t = 0; t < steps; ++t) {
            const int64_t jt = __shfl_sync(0xffffffffu, j, t);
            const float dst = __shfl_sync(0xffffffffu, ds, t);
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
    // query i attends key j iff j = i + t*dil with -left <= t <= right, i.e. i = j - t*dil
    int64_t u_lo = -a.right, u_hi = a.left;           // i = j + u*dil
    if (j + u_lo * a.dil < 0) u_lo = -(j / a.dil);
    if (j + u_hi * a.dil >= a.S) u_hi = (a.S - 1 - j) / a.dil;
    const int64_t n = u_hi >= u_lo ? u_hi - u_lo + 1 : 0;
    const int64_t first = j + u_lo * a.dil;

    float ak[MAXR], av[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) ak[r] = av[r] = 0.f;
    for (int64_t c = 0; c < n; c += 32) {
        const int64_t idx = c + lane;
        float p = 0.f, ds = 0.f;
        int64_t i = -1;
        if (idx < n) {
            i = first + idx * a.dil;
            const float2 s2 = st[i];
            p = expf(dot_row(ks, qb + i * stride, a.D) * a.scale - s2.x);
            ds = p * (dot_row(vs, gb + i * stride, a.D) - s2.y) * a.scale;
        }
        const int steps = n - c < 32 ? (int)(n - c) : 32;
        for (int t = 0; t < steps; ++t) {
            const int64_t it = __shfl_sync(0xffffffffu, i, t);
            const float pt = __shfl_sync(0xffffffffu, p, t);
            const float dst = __shfl_sync(0xffffffffu, ds, t);
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
    note_kernel("bwd_window");
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

int mat_sparse_attn_bwd(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk,
                        void *dv, int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                        const mat_pattern_spec *spec, float scale, void *workspace, size_t workspace_bytes,
                        void *stream) {
    if (!spec) return fail(MAT_ERR_INVALID, "pattern description is NULL");
    if (spec->kind != MAT_WINDOW) return fail(MAT_ERR_UNSUPPORTED, "backward is defined for window patterns");
    if (spec->left < 0 || spec->right < 0 || spec->dilation < 1 || spec->q_offset != 0)
        return fail(MAT_ERR_INVALID, "bad window description for the backward pass");
    if (!q || !k || !v || !dout || !dq || !dk || !dv) return fail(MAT_ERR_INVALID, "tensor pointers must be non-NULL");
    if (B <= 0 || S <= 0 || H <= 0 || D <= 0) return fail(MAT_ERR_INVALID, "all tensor dimensions must be > 0");
    const size_t need = mat_sparse_attn_bwd_workspace_bytes(B, S, H);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace % 256) != 0)
        return fail(MAT_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) required, got %zu", need,
                    workspace ? workspace_bytes : (size_t)0);
    WindowArgs a;
    a.B = B; a.S = S; a.H = H; a.D = (int)D;
    a.left = spec->left > S ? S : spec->left;
    a.right = spec->right > S ? S : spec->right;
    a.dil = spec->dilation;
    a.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)D);
    float2 *stats = (float2 *)workspace;
    cudaStream_t st = (cudaStream_t)stream;
    // the tensor-core kernels move 16-byte vectors and TMA boxes: unaligned tensors stay on the warp-level kernels
    const uintptr_t al = (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)dout | (uintptr_t)dq | (uintptr_t)dk |
                         (uintptr_t)dv;
    if (al % 16 == 0 && bwd_mma_supports(B, S, H, D, dtype, a.left, a.right, a.dil))
        return launch_bwd_mma(q, k, v, dout, dq, dk, dv, stats, B, S, H, dtype, a.left, a.right, a.dil, a.scale, st);
    switch (dtype) {
        case MAT_F32: return launch_t<float>(q, k, v, dout, dq, dk, dv, stats, a, st);
        case MAT_BF16: return launch_t<__nv_bfloat16>(q, k, v, dout, dq, dk, dv, stats, a, st);
        case MAT_F16: return launch_t<__half>(q, k, v, dout, dq, dk, dv, stats, a, st);
    }
    return fail(MAT_ERR_INVALID, "unknown dtype %d", dtype);
}

}  // extern "C"
