// Pattern-general forward: one warp per (batch, head, query row).
//
// Covers every pattern kind, every element type and any head width up to 512,
// so it is the path for fp32 (the reference's precision,
// src/csrc/attention_types.hpp:10) and for shapes the tensor-core kernels do not
// take (odd D, ragged dilation).  Replaces sparse_attention_forward_warp
// (src/cuda/sparse_attention_kernel.cu:211-263), which rewrites the output row
// in global memory once per key; here the row lives in registers and is stored
// once.
//
// Per 32-key step each lane scores one key (sequential fp32 dot over d, then
// * scale, the order of src/csrc/ma_core.cpp:202-209), the step's max and sum
// are warp shuffles, and the lanes then split the head width for P*V.
#include "mat_common.cuh"

namespace mat {
namespace {

constexpr int kWarpsPerCta = 8;

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Flat enumeration of one row's candidate keys: idx in [0, n) -> key position,
// or -1 where the candidate is masked (outside the tensor, behind the causal
// edge, or a global key the window already holds).
struct RowKeys {
    int64_t n;
    int64_t p;        // query position in key coordinates
    int64_t first;    // window: first tap's key position
    int64_t n_win;    // longformer: number of window keys
    int64_t e0;       // block: first CSR entry of the row
    int kind;         // MAT_* or 3 = every key (longformer global row)
};

__device__ __forceinline__ bool is_global_pos(const DevPattern &pat, int64_t p) {
    int64_t lo = 0, hi = pat.n_global;
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        int64_t g = pat.gidx[mid];
        if (g == p) return true;
        if (g < p) lo = mid + 1; else hi = mid;
    }
    return false;
}

__device__ __forceinline__ RowKeys row_keys(const DevPattern &pat, int64_t i, int64_t Skv) {
    RowKeys r;
    r.p = i + pat.q_offset;
    r.kind = pat.kind;
    r.n = 0; r.first = 0; r.n_win = 0; r.e0 = 0;
    if (pat.kind == MAT_WINDOW || pat.kind == MAT_LONGFORMER) {
        const int64_t dil = pat.kind == MAT_WINDOW ? pat.dilation : 1;
        if (pat.kind == MAT_LONGFORMER && is_global_pos(pat, r.p)) {
            r.kind = 3;
            r.n = Skv;
            return r;
        }
        int64_t t_lo = -pat.left, t_hi = pat.right;
        if (r.p + t_lo * dil < 0) t_lo = -(r.p / dil);
        if (r.p + t_hi * dil >= Skv) t_hi = (Skv - 1 - r.p) / dil;
        r.first = r.p + t_lo * dil;
        r.n_win = t_hi >= t_lo ? t_hi - t_lo + 1 : 0;
        r.n = r.n_win + (pat.kind == MAT_LONGFORMER ? pat.n_global : 0);
    } else {  // MAT_BLOCK
        const int64_t qb = r.p / pat.block;
        if (qb < pat.n_qblocks) {
            r.e0 = pat.rowptr[qb];
            r.n = (int64_t)(pat.rowptr[qb + 1] - pat.rowptr[qb]) * pat.block;
        }
    }
    return r;
}

__device__ __forceinline__ int64_t key_at(const DevPattern &pat, const RowKeys &r, int64_t idx,
                                          int64_t Skv) {
    switch (r.kind) {
        case MAT_WINDOW:
            return r.first + idx * pat.dilation;
        case 3:
            return idx;
        case MAT_LONGFORMER: {
            if (idx < r.n_win) return r.first + idx;
            const int64_t g = pat.gidx[idx - r.n_win];
            if (g < 0 || g >= Skv) return -1;
            if (g >= r.p - pat.left && g <= r.p + pat.right) return -1;  // already in the window
            return g;
        }
        default: {  // MAT_BLOCK
            const int64_t c = pat.colidx[r.e0 + idx / pat.block];
            const int64_t j = c * pat.block + idx % pat.block;
            if (j >= Skv || (pat.causal && j > r.p)) return -1;
            return j;
        }
    }
}

template <typename T, bool VEC> struct RowDot;

// scalar path: any alignment, any D
template <typename T> struct RowDot<T, false> {
    static __device__ __forceinline__ float run(const float *qs, const T *kr, int D) {
        float s = 0.f;
        for (int d = 0; d < D; ++d) s = fmaf(qs[d], Elem<T>::to_f(kr[d]), s);
        return s;
    }
};
// 16-byte loads: rows are 16-byte aligned and D*sizeof(T) is a multiple of 16
template <> struct RowDot<float, true> {
    static __device__ __forceinline__ float run(const float *qs, const float *kr, int D) {
        float s = 0.f;
        const float4 *k4 = reinterpret_cast<const float4 *>(kr);
        for (int d = 0; d < D; d += 4) {
            float4 x = __ldg(k4 + (d >> 2));
            s = fmaf(qs[d], x.x, s); s = fmaf(qs[d + 1], x.y, s);
            s = fmaf(qs[d + 2], x.z, s); s = fmaf(qs[d + 3], x.w, s);
        }
        return s;
    }
};
template <typename T> struct RowDot16 {
    static __device__ __forceinline__ float run(const float *qs, const T *kr, int D) {
        float s = 0.f;
        const uint4 *k4 = reinterpret_cast<const uint4 *>(kr);
        for (int d = 0; d < D; d += 8) {
            uint4 x = __ldg(k4 + (d >> 3));
            const T *e = reinterpret_cast<const T *>(&x);
#pragma unroll
            for (int t = 0; t < 8; ++t) s = fmaf(qs[d + t], Elem<T>::to_f(e[t]), s);
        }
        return s;
    }
};
template <> struct RowDot<__nv_bfloat16, true> : RowDot16<__nv_bfloat16> {};
template <> struct RowDot<__half, true> : RowDot16<__half> {};

template <typename T, int MAXR, bool VEC>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
attn_fwd_rowwarp(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                 T *__restrict__ o, int64_t B, int64_t Sq, int64_t Skv, int64_t H, int D,
                 DevPattern pat, float scale) {
    extern __shared__ float q_smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float *qs = q_smem + (size_t)warp * D;

    const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + warp;
    if (row >= B * Sq * H) return;  // whole warp leaves together
    const int64_t i = row % Sq;
    const int64_t h = (row / Sq) % H;
    const int64_t b = row / (Sq * H);

    const T *qr = q + ((b * Sq + i) * H + h) * D;
    for (int d = lane; d < D; d += 32) qs[d] = Elem<T>::to_f(qr[d]);
    __syncwarp();

    const RowKeys rk = row_keys(pat, i, Skv);
    const int64_t kv_row_stride = H * (int64_t)D;
    const T *kb = k + (b * Skv * H + h) * (int64_t)D;
    const T *vb = v + (b * Skv * H + h) * (int64_t)D;

    float m = -INFINITY, l = 0.f;
    float acc[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;

    for (int64_t base = 0; base < rk.n; base += 32) {
        const int64_t idx = base + lane;
        const int64_t j = idx < rk.n ? key_at(pat, rk, idx, Skv) : -1;
        float s = -INFINITY;
        if (j >= 0) s = RowDot<T, VEC>::run(qs, kb + j * kv_row_stride, D) * scale;
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;  // every candidate of this step is masked
        const float pj = j >= 0 ? expf(s - m_new) : 0.f;
        const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
        l = l * alpha + warp_sum(pj);
#pragma unroll
        for (int r = 0; r < MAXR; ++r) acc[r] *= alpha;
        const int steps = rk.n - base < 32 ? (int)(rk.n - base) : 32;
        for (int t = 0; t < steps; ++t) {
            const int64_t jt = __shfl_sync(0xffffffffu, j, t);
            const float pt = __shfl_sync(0xffffffffu, pj, t);
            if (jt < 0) continue;  // uniform across the warp
            const T *vr = vb + jt * kv_row_stride;
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                const int d = lane + 32 * r;
                if (d < D) acc[r] = fmaf(pt, Elem<T>::to_f(vr[d]), acc[r]);
            }
        }
        m = m_new;
    }

    const float inv = l > 0.f ? 1.f / l : 0.f;
    T *orow = o + ((b * Sq + i) * H + h) * D;
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        const int d = lane + 32 * r;
        if (d < D) orow[d] = Elem<T>::from_f(acc[r] * inv);
    }
}

template <typename T, int MAXR>
int launch_t(const Problem &p) {
    const int64_t rows = p.B * p.Sq * p.H;
    const int64_t ctas = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
    if (ctas > 0x7fffffffLL) return fail(MAT_ERR_UNSUPPORTED, "rowwarp: too many rows for one launch");
    const size_t smem = (size_t)kWarpsPerCta * p.D * sizeof(float);
    const size_t row_bytes = (size_t)p.D * sizeof(T);
    const bool vec = row_bytes % 16 == 0 && ((uintptr_t)p.k % 16) == 0;
    const T *q = (const T *)p.q, *k = (const T *)p.k, *v = (const T *)p.v;
    T *o = (T *)p.o;
    if (vec)
        attn_fwd_rowwarp<T, MAXR, true><<<(unsigned)ctas, kWarpsPerCta * 32, smem, p.stream>>>(
            q, k, v, o, p.B, p.Sq, p.Skv, p.H, (int)p.D, p.pat, p.scale);
    else
        attn_fwd_rowwarp<T, MAXR, false><<<(unsigned)ctas, kWarpsPerCta * 32, smem, p.stream>>>(
            q, k, v, o, p.B, p.Sq, p.Skv, p.H, (int)p.D, p.pat, p.scale);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "rowwarp launch");
    note_kernel("rowwarp");
    return MAT_OK;
}

template <typename T>
int launch_d(const Problem &p) {
    if (p.D <= 64) return launch_t<T, 2>(p);
    if (p.D <= 128) return launch_t<T, 4>(p);
    if (p.D <= 256) return launch_t<T, 8>(p);
    if (p.D <= 512) return launch_t<T, 16>(p);
    return fail(MAT_ERR_UNSUPPORTED, "head width D=%lld exceeds the supported maximum of 512",
                (long long)p.D);
}

}  // namespace

int launch_rowwarp(const Problem &p) {
    switch (p.dtype) {
        case MAT_F32: return launch_d<float>(p);
        case MAT_BF16: return launch_d<__nv_bfloat16>(p);
        case MAT_F16: return launch_d<__half>(p);
    }
    return fail(MAT_ERR_INVALID, "unknown dtype %d", p.dtype);
}

}  // namespace mat
