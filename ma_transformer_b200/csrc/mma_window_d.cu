// 16-bit window attention for head widths other than 64 (the multiples of 16 up to 128) on the warp-level
// tensor-core instructions.
//
// The reference kernel takes any head width (sparse_attention_forward_warp,
// src/cuda/sparse_attention_kernel.cu:238-262: `d = lane; d < D; d += 32`), and its layer calls it with
// D = model_dim (src/layers/sparse_attention.py:71-78).  The TMA / tcgen05 kernels of this library are
// laid out for 128-byte rows (D = 64); this kernel covers the other common widths so that they do not fall
// to the one-warp-per-row kernel.
//
// One CTA = 64 query rows of one (batch, head), four warps of 16 rows.  The keys the tile can see
// (first row's first tap to last row's last tap) are walked 64 at a time: K and V chunks arrive in shared
// memory by cp.async (two buffers, rows padded by 16 bytes so that ldmatrix is conflict-free; rows past the
// sequence end are zero-filled, so a masked weight never multiplies stale shared memory), S = Q K^T by
// mma.sync m16n8k16 with Q held in registers, masks, an online softmax in registers, P re-used in place
// as the A fragments of O += P V.  A dilated window is a plain window over the tensor viewed as
// [B, S/dil, dil*H, D], as everywhere in this library.  (Skipping, per warp, the 16-key groups none of its rows
// can use by a branch per group was measured slower - 117 against 93 us at 64K tokens x 4 heads of 128: the branches
// inside the unrolled products cost more than the masked work they save.  Narrow windows take the second kernel
// below, which gets rid of those groups without a branch.)
#include <algorithm>
#include <cstring>

#include "mat_common.cuh"
#include "ptx.cuh"

namespace mat {
namespace {

constexpr int kTQ = 64, kTK = 64, kThreads = 128;

struct WinDParams {
    int32_t Sq1, Skv1, off1;   // query rows, key rows, q_offset of one sub-sequence
    int32_t HH;                // heads of the view
    int32_t left, right;
    float sl2;                 // scale * log2(e)
    int32_t D;                 // head width (read by the kernel for wide heads only)
};

__device__ __forceinline__ void cp_async16(void *dst, const void *src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(ptx::smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
window_d_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, T *__restrict__ o,
                const WinDParams P) {
    constexpr int LD = D + 8;          // padded row, elements
    constexpr int KS = D / 16;         // k-steps of S = Q K^T; pairs of 8-wide output tiles of O
    extern __shared__ __align__(16) uint8_t smem_raw[];
    T *sK = reinterpret_cast<T *>(smem_raw);          // [2][kTK][LD]
    T *sV = sK + 2 * kTK * LD;                        // [2][kTK][LD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int hh = blockIdx.x, b = blockIdx.z, q0 = blockIdx.y * kTQ;
    const int p_first = q0 + P.off1;   // key-coordinate position of the tile's first row
    const int last_row = min(q0 + kTQ, P.Sq1) - 1;
    const int key_lo = max(0, p_first - P.left);
    const int key_hi = min(P.Skv1 - 1, last_row + P.off1 + P.right);
    const int n_chunks = key_hi >= key_lo ? (key_hi - key_lo) / kTK + 1 : 0;
    const int64_t tok = (int64_t)P.HH * D;   // elements per token
    const T *kb_ptr = k + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const T *vb_ptr = v + ((int64_t)b * P.Skv1 * P.HH + hh) * D;

    auto load_chunk = [&](int c, int buf) {
        constexpr int kPieces = D / 8;   // 16-byte pieces per row
        const int base = key_lo + c * kTK;
        for (int i = threadIdx.x; i < kTK * kPieces; i += kThreads) {
            const int r = i / kPieces, pc = i % kPieces;
            const int j = base + r;
            const bool in = j < P.Skv1;
            const int64_t src = (int64_t)(in ? j : 0) * tok + pc * 8;
            cp_async16(sK + (buf * kTK + r) * LD + pc * 8, kb_ptr + src, in ? 16 : 0);
            cp_async16(sV + (buf * kTK + r) * LD + pc * 8, vb_ptr + src, in ? 16 : 0);
        }
    };
    if (n_chunks > 0) load_chunk(0, 0);
    cp_async_commit();

    // the warp's 16 query rows as A fragments: thread (g, t) holds rows g and g + 8, columns 2t, 2t+1 (+8)
    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    uint32_t qf[KS][4];
    {
        const T *qa = q + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D;
        const T *qb = q + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 16 + 2 * t;
            qf[ks][0] = row_a < P.Sq1 ? *reinterpret_cast<const uint32_t *>(qa + c) : 0u;
            qf[ks][1] = row_b < P.Sq1 ? *reinterpret_cast<const uint32_t *>(qb + c) : 0u;
            qf[ks][2] = row_a < P.Sq1 ? *reinterpret_cast<const uint32_t *>(qa + c + 8) : 0u;
            qf[ks][3] = row_b < P.Sq1 ? *reinterpret_cast<const uint32_t *>(qb + c + 8) : 0u;
        }
    }
    const int pos[2] = {row_a + P.off1, row_b + P.off1};
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[2 * KS][4];
#pragma unroll
    for (int n = 0; n < 2 * KS; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

    for (int c = 0; c < n_chunks; ++c) {
        const int buf = c & 1;
        if (c + 1 < n_chunks) {
            load_chunk(c + 1, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int kb = key_lo + c * kTK;
        const uint32_t k_addr = ptx::smem_u32(sK + buf * kTK * LD), v_addr = ptx::smem_u32(sV + buf * kTK * LD);
        const int m4 = lane >> 3, r8 = lane & 7;

        // ---- S = Q K^T: eight 8-key tiles per warp ----
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int n2 = 0; n2 < 4; ++n2) {
                // matrices: (keys n2*16 + 0..7, dims +0), (same keys, dims +8), (keys +8, dims +0), (keys +8, dims +8)
                uint32_t kf[4];
                ptx::ldmatrix_x4(kf, k_addr + (uint32_t)(((n2 * 16 + r8 + (m4 >> 1) * 8) * LD + ks * 16 + (m4 & 1) * 8) * 2));
                ptx::Mma<T>::run(s[2 * n2], qf[ks], kf[0], kf[1]);
                ptx::Mma<T>::run(s[2 * n2 + 1], qf[ks], kf[2], kf[3]);
            }
        }
        // ---- mask, online softmax (raw scores; the scale enters the exponent) ----
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = kb + n * 8 + 2 * t + (e & 1), p = pos[e >> 1];
                const bool ok = j >= p - P.left && j <= p + P.right && j < P.Skv1;
                s[n][e] = ok ? s[n][e] : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
            }
        float alpha[2], mus[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float m_new = fmaxf(m_run[i], mx[i]);
            alpha[i] = m_new == -INFINITY ? 1.f : ptx::ex2((m_run[i] - m_new) * P.sl2);
            m_run[i] = m_new;
            mus[i] = m_new == -INFINITY ? 0.f : m_new * P.sl2;
            l_run[i] *= alpha[i];
        }
#pragma unroll
        for (int n = 0; n < 2 * KS; ++n) {
            acc[n][0] *= alpha[0]; acc[n][1] *= alpha[0];
            acc[n][2] *= alpha[1]; acc[n][3] *= alpha[1];
        }
        uint32_t pa[4][4];   // the weights as A fragments of the 16-key steps of P V
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                w[e] = ptx::ex2(fmaf(s[n][e], P.sl2, -mus[e >> 1]));
                l_run[e >> 1] += w[e];
            }
            pa[n >> 1][(n & 1) * 2] = ptx::Mma<T>::pack(w[0], w[1]);
            pa[n >> 1][(n & 1) * 2 + 1] = ptx::Mma<T>::pack(w[2], w[3]);
        }
        // ---- O += P V ----
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int d2 = 0; d2 < KS; ++d2) {
                // matrices (transposed on load): (keys kk*16 + 0..7, dims d2*16 + 0..7), (keys +8, same dims),
                // (keys + 0, dims + 8), (keys + 8, dims + 8)
                uint32_t vf[4];
                ptx::ldmatrix_x4_trans(vf, v_addr + (uint32_t)(((kk * 16 + r8 + (m4 & 1) * 8) * LD + d2 * 16 + (m4 >> 1) * 8) * 2));
                ptx::Mma<T>::run(acc[2 * d2], pa[kk], vf[0], vf[1]);
                ptx::Mma<T>::run(acc[2 * d2 + 1], pa[kk], vf[2], vf[3]);
            }
        }
        __syncthreads();   // the buffer is free for the chunk after the next
    }

    // ---- normalise and write the two rows of this thread ----
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float l = l_run[i];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int row = i == 0 ? row_a : row_b;
        if (row < P.Sq1) {
            T *dst = o + (((int64_t)b * P.Sq1 + row) * P.HH + hh) * D + 2 * t;
#pragma unroll
            for (int n = 0; n < 2 * KS; ++n)
                *reinterpret_cast<uint32_t *>(dst + n * 8) = ptx::Mma<T>::pack(acc[n][2 * i] * inv, acc[n][2 * i + 1] * inv);
        }
    }
}

// Narrow windows: every warp walks the keys from a base of its own, the first key its first row can see, in passes
// of NS 16-key steps, so that no step is without a visible key but the last of the walk (at 64 causal taps 5 steps
// instead of the 8 of two chunks), and the code is the same straight line for every warp.  The CTA stages the
// 48 + 16 NS rows the four warps' passes span.
template <typename T, int D, int NS>
__global__ void __launch_bounds__(kThreads, NS <= 5 ? 3 : 2)
window_d_diag_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, T *__restrict__ o,
                     const WinDParams P) {
    constexpr int LD = D + 8, KS = D / 16;
    constexpr int kStage = 48 + 16 * NS;   // rows of K and of V in shared memory
    extern __shared__ __align__(16) uint8_t smem_raw[];
    T *sK = reinterpret_cast<T *>(smem_raw);   // [kStage][LD]
    T *sV = sK + kStage * LD;                  // [kStage][LD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int hh = blockIdx.x, b = blockIdx.z, q0 = blockIdx.y * kTQ;
    const int p_first = q0 + P.off1;
    const int key_lo = max(0, p_first - P.left);
    const int key_hi = min(P.Skv1 - 1, min(q0 + kTQ, P.Sq1) - 1 + P.off1 + P.right);
    const int base_w = max(key_lo, p_first + 16 * warp - P.left);   // the warp's first key
    int n_pass = 0;   // passes of the warp with the longest walk
    if (key_hi >= key_lo) {
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) {
            const int keys_w = min(key_hi, p_first + 16 * w + 15 + P.right) - max(key_lo, p_first + 16 * w - P.left) + 1;
            n_pass = max(n_pass, (keys_w + 16 * NS - 1) / (16 * NS));
        }
    }
    const int64_t tok = (int64_t)P.HH * D;
    const T *kb_ptr = k + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const T *vb_ptr = v + ((int64_t)b * P.Skv1 * P.HH + hh) * D;

    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    uint32_t qf[KS][4];
    {
        const T *qa = q + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D;
        const T *qb = q + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 16 + 2 * t;
            qf[ks][0] = row_a < P.Sq1 ? *reinterpret_cast<const uint32_t *>(qa + c) : 0u;
            qf[ks][1] = row_b < P.Sq1 ? *reinterpret_cast<const uint32_t *>(qb + c) : 0u;
            qf[ks][2] = row_a < P.Sq1 ? *reinterpret_cast<const uint32_t *>(qa + c + 8) : 0u;
            qf[ks][3] = row_b < P.Sq1 ? *reinterpret_cast<const uint32_t *>(qb + c + 8) : 0u;
        }
    }
    const int pos[2] = {row_a + P.off1, row_b + P.off1};
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[2 * KS][4];
#pragma unroll
    for (int n = 0; n < 2 * KS; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    const int m4 = lane >> 3, r8 = lane & 7;

    for (int c = 0; c < n_pass; ++c) {
        const int stage_lo = key_lo + c * 16 * NS;   // warp 0's base is key_lo
        if (stage_lo > key_hi) break;
        if (c) __syncthreads();   // the previous pass has been read
        {
            constexpr int kPieces = D / 8;
            for (int i = threadIdx.x; i < kStage * kPieces; i += kThreads) {
                const int r = i / kPieces, pc = i % kPieces;
                const int j = stage_lo + r;
                const bool in = j <= key_hi;   // rows past the tile's last key are zero-filled
                const int64_t src = (int64_t)(in ? j : 0) * tok + pc * 8;
                cp_async16(sK + r * LD + pc * 8, kb_ptr + src, in ? 16 : 0);
                cp_async16(sV + r * LD + pc * 8, vb_ptr + src, in ? 16 : 0);
            }
            cp_async_commit();
            cp_async_wait<0>();
        }
        __syncthreads();
        const int kb = base_w + c * 16 * NS;   // the warp's first key of the pass
        const uint32_t k_addr = ptx::smem_u32(sK + (kb - stage_lo) * LD), v_addr = ptx::smem_u32(sV + (kb - stage_lo) * LD);

        float s[2 * NS][4];
#pragma unroll
        for (int n = 0; n < 2 * NS; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int n2 = 0; n2 < NS; ++n2) {
                uint32_t kf[4];
                ptx::ldmatrix_x4(kf, k_addr + (uint32_t)(((n2 * 16 + r8 + (m4 >> 1) * 8) * LD + ks * 16 + (m4 & 1) * 8) * 2));
                ptx::Mma<T>::run(s[2 * n2], qf[ks], kf[0], kf[1]);
                ptx::Mma<T>::run(s[2 * n2 + 1], qf[ks], kf[2], kf[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2 * NS; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = kb + n * 8 + 2 * t + (e & 1), p = pos[e >> 1];
                const bool ok = j >= p - P.left && j <= p + P.right && j < P.Skv1;
                s[n][e] = ok ? s[n][e] : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
            }
        float alpha[2], mus[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float m_new = fmaxf(m_run[i], mx[i]);
            alpha[i] = m_new == -INFINITY ? 1.f : ptx::ex2((m_run[i] - m_new) * P.sl2);
            m_run[i] = m_new;
            mus[i] = m_new == -INFINITY ? 0.f : m_new * P.sl2;
            l_run[i] *= alpha[i];
        }
        if (c) {
#pragma unroll
            for (int n = 0; n < 2 * KS; ++n) {
                acc[n][0] *= alpha[0]; acc[n][1] *= alpha[0];
                acc[n][2] *= alpha[1]; acc[n][3] *= alpha[1];
            }
        }
        uint32_t pa[NS][4];
#pragma unroll
        for (int n = 0; n < 2 * NS; ++n) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                w[e] = ptx::ex2(fmaf(s[n][e], P.sl2, -mus[e >> 1]));
                l_run[e >> 1] += w[e];
            }
            pa[n >> 1][(n & 1) * 2] = ptx::Mma<T>::pack(w[0], w[1]);
            pa[n >> 1][(n & 1) * 2 + 1] = ptx::Mma<T>::pack(w[2], w[3]);
        }
#pragma unroll
        for (int kk = 0; kk < NS; ++kk) {
#pragma unroll
            for (int d2 = 0; d2 < KS; ++d2) {
                uint32_t vf[4];
                ptx::ldmatrix_x4_trans(vf, v_addr + (uint32_t)(((kk * 16 + r8 + (m4 & 1) * 8) * LD + d2 * 16 + (m4 >> 1) * 8) * 2));
                ptx::Mma<T>::run(acc[2 * d2], pa[kk], vf[0], vf[1]);
                ptx::Mma<T>::run(acc[2 * d2 + 1], pa[kk], vf[2], vf[3]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float l = l_run[i];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int row = i == 0 ? row_a : row_b;
        if (row < P.Sq1) {
            T *dst = o + (((int64_t)b * P.Sq1 + row) * P.HH + hh) * D + 2 * t;
#pragma unroll
            for (int n = 0; n < 2 * KS; ++n)
                *reinterpret_cast<uint32_t *>(dst + n * 8) = ptx::Mma<T>::pack(acc[n][2 * i] * inv, acc[n][2 * i + 1] * inv);
        }
    }
}

// Wide heads (D = 192, 256, ... 512) with narrow windows: the per-warp walk of the kernel above in a single pass, the
// head dimension taken 64 columns at a time.  The K slices stream through two buffers while the scores accumulate,
// then the V slices while each 64-column slice of the output is formed from the finished weights, normalised and
// written; the copy of the next slice is in flight during the products of the current one.  Registers hold the
// scores / weights of the pass and one slice's operands, whatever D is.
template <typename T, int NS>
__global__ void __launch_bounds__(kThreads)
window_d_wide_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, T *__restrict__ o,
                     const WinDParams P) {
    constexpr int LD = 64 + 8, KS = 4;
    constexpr int kStage = 48 + 16 * NS;   // rows of a slice in shared memory
    extern __shared__ __align__(16) uint8_t smem_raw[];
    T *sBuf = reinterpret_cast<T *>(smem_raw);   // [2][kStage][LD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m4 = lane >> 3, r8 = lane & 7;
    const int hh = blockIdx.x, b = blockIdx.z, q0 = blockIdx.y * kTQ;
    const int D = P.D, n_slices = (D + 63) >> 6;   // (the last slice may be partly beyond D: zeros in, nothing out)
    const int p_first = q0 + P.off1;
    const int key_lo = max(0, p_first - P.left);
    const int key_hi = min(P.Skv1 - 1, min(q0 + kTQ, P.Sq1) - 1 + P.off1 + P.right);
    const int base_w = max(key_lo, p_first + 16 * warp - P.left);   // the warp's first key
    const int64_t tok = (int64_t)P.HH * D;
    const T *kb_ptr = k + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const T *vb_ptr = v + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    const T *qa = q + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D;
    const T *qb = q + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D;
    T *oa = o + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D + 2 * t;
    T *ob = o + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D + 2 * t;

    if (key_hi < key_lo) {   // a tile whose rows see no key (the whole CTA alike): zeros
        for (int c = 0; c + 2 * t < D; c += 8) {
            if (row_a < P.Sq1) *reinterpret_cast<uint32_t *>(oa + c) = 0u;
            if (row_b < P.Sq1) *reinterpret_cast<uint32_t *>(ob + c) = 0u;
        }
        return;
    }
    // copy i of the pass: K slice i, then V slice i - n_slices, into buffer i & 1
    auto issue = [&](int i) {
        const int col0 = (i < n_slices ? i : i - n_slices) * 64;
        const T *src_base = (i < n_slices ? kb_ptr : vb_ptr) + col0;
        T *dst = sBuf + (i & 1) * kStage * LD;
        for (int x = threadIdx.x; x < kStage * 8; x += kThreads) {
            const int r = x >> 3, pc = x & 7;
            const int j = key_lo + r;
            const bool in = j <= key_hi && col0 + pc * 8 < D;   // rows past the tile's last key and columns past D are zero-filled
            cp_async16(dst + r * LD + pc * 8, src_base + (int64_t)(in ? j : 0) * tok + pc * 8, in ? 16 : 0);
        }
        cp_async_commit();
    };
    issue(0);
    const int row_off = (base_w - key_lo) * LD;   // the warp's first key inside a buffer

    float s[2 * NS][4];
#pragma unroll
    for (int n = 0; n < 2 * NS; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    for (int sl = 0; sl < n_slices; ++sl) {
        uint32_t qf[KS][4];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = sl * 64 + ks * 16 + 2 * t;   // (D is a multiple of 8: each half of a 16-column step is inside D or beyond it)
            qf[ks][0] = row_a < P.Sq1 && c < D ? *reinterpret_cast<const uint32_t *>(qa + c) : 0u;
            qf[ks][1] = row_b < P.Sq1 && c < D ? *reinterpret_cast<const uint32_t *>(qb + c) : 0u;
            qf[ks][2] = row_a < P.Sq1 && c + 8 < D ? *reinterpret_cast<const uint32_t *>(qa + c + 8) : 0u;
            qf[ks][3] = row_b < P.Sq1 && c + 8 < D ? *reinterpret_cast<const uint32_t *>(qb + c + 8) : 0u;
        }
        issue(sl + 1);   // the next K slice, or the first V slice
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t k_addr = ptx::smem_u32(sBuf + (sl & 1) * kStage * LD + row_off);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int n2 = 0; n2 < NS; ++n2) {
                uint32_t kf[4];
                ptx::ldmatrix_x4(kf, k_addr + (uint32_t)(((n2 * 16 + r8 + (m4 >> 1) * 8) * LD + ks * 16 + (m4 & 1) * 8) * 2));
                ptx::Mma<T>::run(s[2 * n2], qf[ks], kf[0], kf[1]);
                ptx::Mma<T>::run(s[2 * n2 + 1], qf[ks], kf[2], kf[3]);
            }
        }
        __syncthreads();   // the buffer is free for the copy after the next
    }
    // ---- mask and softmax of the whole row (one pass: no running maximum) ----
    const int pos[2] = {row_a + P.off1, row_b + P.off1};
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2 * NS; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = base_w + n * 8 + 2 * t + (e & 1), p = pos[e >> 1];
            const bool ok = j >= p - P.left && j <= p + P.right && j < P.Skv1;
            s[n][e] = ok ? s[n][e] : -INFINITY;
            mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
        }
    float l[2] = {0.f, 0.f}, mus[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        mus[i] = mx[i] == -INFINITY ? 0.f : mx[i] * P.sl2;
    }
    uint32_t pa[NS][4];   // the weights as A fragments of the 16-key steps of P V
#pragma unroll
    for (int n = 0; n < 2 * NS; ++n) {
        float w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            w[e] = ptx::ex2(fmaf(s[n][e], P.sl2, -mus[e >> 1]));
            l[e >> 1] += w[e];
        }
        pa[n >> 1][(n & 1) * 2] = ptx::Mma<T>::pack(w[0], w[1]);
        pa[n >> 1][(n & 1) * 2 + 1] = ptx::Mma<T>::pack(w[2], w[3]);
    }
    float inv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        inv[i] = l[i] > 0.f ? 1.f / l[i] : 0.f;
    }
    // ---- the output, 64 columns at a time ----
    for (int sl = 0; sl < n_slices; ++sl) {
        const int i = n_slices + sl;
        if (sl + 1 < n_slices) {
            issue(i + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t v_addr = ptx::smem_u32(sBuf + (i & 1) * kStage * LD + row_off);
        float acc[2 * KS][4];
#pragma unroll
        for (int n = 0; n < 2 * KS; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < NS; ++kk) {
#pragma unroll
            for (int d2 = 0; d2 < KS; ++d2) {
                uint32_t vf[4];
                ptx::ldmatrix_x4_trans(vf, v_addr + (uint32_t)(((kk * 16 + r8 + (m4 & 1) * 8) * LD + d2 * 16 + (m4 >> 1) * 8) * 2));
                ptx::Mma<T>::run(acc[2 * d2], pa[kk], vf[0], vf[1]);
                ptx::Mma<T>::run(acc[2 * d2 + 1], pa[kk], vf[2], vf[3]);
            }
        }
#pragma unroll
        for (int n = 0; n < 2 * KS; ++n) {
            if (sl * 64 + n * 8 + 2 * t >= D) continue;
            if (row_a < P.Sq1)
                *reinterpret_cast<uint32_t *>(oa + sl * 64 + n * 8) = ptx::Mma<T>::pack(acc[n][0] * inv[0], acc[n][1] * inv[0]);
            if (row_b < P.Sq1)
                *reinterpret_cast<uint32_t *>(ob + sl * 64 + n * 8) = ptx::Mma<T>::pack(acc[n][2] * inv[1], acc[n][3] * inv[1]);
        }
        __syncthreads();   // the buffer is free for the copy after the next
    }
}

template <typename T, int NS>
int launch_wide(const Problem &p) {
    const int64_t dil = p.pat.dilation;
    WinDParams wp;
    wp.Sq1 = (int32_t)(p.Sq / dil);
    wp.Skv1 = (int32_t)(p.Skv / dil);
    wp.off1 = (int32_t)(p.pat.q_offset / dil);
    wp.HH = (int32_t)(p.H * dil);
    wp.left = (int32_t)std::min<int64_t>(p.pat.left, wp.Skv1);
    wp.right = (int32_t)std::min<int64_t>(p.pat.right, wp.Skv1);
    wp.sl2 = p.scale * 1.4426950408889634f;
    wp.D = (int32_t)p.D;
    auto kern = window_d_wide_kernel<T, NS>;
    constexpr size_t smem = (size_t)2 * (48 + 16 * NS) * 72 * sizeof(T);
    if (int rc = ensure_dynamic_smem((const void *)kern, smem, "cudaFuncSetAttribute(window_d_wide_kernel)")) return rc;
    const dim3 grid((unsigned)wp.HH, (unsigned)((wp.Sq1 + kTQ - 1) / kTQ), (unsigned)p.B);
    kern<<<grid, kThreads, smem, p.stream>>>((const T *)p.q, (const T *)p.k, (const T *)p.v, (T *)p.o, wp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "window_d_wide_kernel launch");
    note_kernel("mma_window_d");
    return MAT_OK;
}

// Wide or odd heads with windows that take a warp more than one pass (up to dense).  Two sweeps over the passes, the
// head dimension 64 columns at a time in both: sweep one accumulates each pass's scores over the K slices and keeps the
// rows' running maximum and sum; sweep two forms the scores again, turns them into normalised weights (rounded to the
// input type, as everywhere) and multiplies them with every V slice.  The output rows are sums over the passes, and
// 16-bit values cannot carry fifty partial sums, so they are kept in fp32 in a scratch tensor of the output's shape
// (the caller's workspace): a row's first pass writes it, later passes add to it, the last pass adds, rounds and writes
// the output itself (a row belongs to one thread pair of one CTA: no atomics, and nothing else reads the scratch).
template <typename T>
__global__ void __launch_bounds__(kThreads)
window_d_wide_passes_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, T *__restrict__ o,
                            float *__restrict__ scratch, const WinDParams P) {
    constexpr int NS = 5, LD = 64 + 8, KS = 4;
    constexpr int kStage = 48 + 16 * NS;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    T *sBuf = reinterpret_cast<T *>(smem_raw);   // [kStage][LD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m4 = lane >> 3, r8 = lane & 7;
    const int hh = blockIdx.x, b = blockIdx.z, q0 = blockIdx.y * kTQ;
    const int D = P.D, n_slices = (D + 63) >> 6;
    const int p_first = q0 + P.off1;
    const int key_lo = max(0, p_first - P.left);
    const int key_hi = min(P.Skv1 - 1, min(q0 + kTQ, P.Sq1) - 1 + P.off1 + P.right);
    const int base_w = max(key_lo, p_first + 16 * warp - P.left);   // the warp's first key
    const int st_off = (base_w - key_lo) * LD;
    int n_pass = 0;
    if (key_hi >= key_lo) {
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) {
            const int keys_w = min(key_hi, p_first + 16 * w + 15 + P.right) - max(key_lo, p_first + 16 * w - P.left) + 1;
            n_pass = max(n_pass, (keys_w + 16 * NS - 1) / (16 * NS));
        }
        n_pass = min(n_pass, (key_hi - key_lo) / (16 * NS) + 1);
    }
    const int64_t tok = (int64_t)P.HH * D;
    const T *kb_ptr = k + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const T *vb_ptr = v + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    const int64_t off_a = (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D, off_b = (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D;
    const T *qa = q + off_a, *qb = q + off_b;
    const int pos[2] = {row_a + P.off1, row_b + P.off1};

    if (n_pass == 0) {   // a tile whose rows see no key (the whole CTA alike): zeros
        for (int c = 2 * t; c < D; c += 8) {
            if (row_a < P.Sq1) *reinterpret_cast<uint32_t *>(o + off_a + c) = 0u;
            if (row_b < P.Sq1) *reinterpret_cast<uint32_t *>(o + off_b + c) = 0u;
        }
        return;
    }
    // one 64-column slice of the kStage rows of pass c, of K or V; rows past the tile's last key and columns past D are zeros
    auto stage = [&](const T *src, int c, int slice) {
        const int first = key_lo + c * 16 * NS;
        __syncthreads();   // whoever still read the buffer is done
        for (int x = threadIdx.x; x < kStage * 8; x += kThreads) {
            const int r = x >> 3, pc = x & 7;
            const int j = first + r;
            const bool in = j <= key_hi && slice * 64 + pc * 8 < D;
            cp_async16(sBuf + r * LD + pc * 8, src + (int64_t)(in ? j : 0) * tok + slice * 64 + pc * 8, in ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
    };
    // the masked scores of pass c
    auto scores = [&](int c, float (&s)[2 * NS][4]) {
#pragma unroll
        for (int n = 0; n < 2 * NS; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        for (int sl = 0; sl < n_slices; ++sl) {
            uint32_t qf[KS][4];
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int col = sl * 64 + ks * 16 + 2 * t;
                qf[ks][0] = row_a < P.Sq1 && col < D ? *reinterpret_cast<const uint32_t *>(qa + col) : 0u;
                qf[ks][1] = row_b < P.Sq1 && col < D ? *reinterpret_cast<const uint32_t *>(qb + col) : 0u;
                qf[ks][2] = row_a < P.Sq1 && col + 8 < D ? *reinterpret_cast<const uint32_t *>(qa + col + 8) : 0u;
                qf[ks][3] = row_b < P.Sq1 && col + 8 < D ? *reinterpret_cast<const uint32_t *>(qb + col + 8) : 0u;
            }
            stage(kb_ptr, c, sl);
            const uint32_t k_addr = ptx::smem_u32(sBuf + st_off);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                for (int n2 = 0; n2 < NS; ++n2) {
                    uint32_t kf[4];
                    ptx::ldmatrix_x4(kf, k_addr + (uint32_t)(((n2 * 16 + r8 + (m4 >> 1) * 8) * LD + ks * 16 + (m4 & 1) * 8) * 2));
                    ptx::Mma<T>::run(s[2 * n2], qf[ks], kf[0], kf[1]);
                    ptx::Mma<T>::run(s[2 * n2 + 1], qf[ks], kf[2], kf[3]);
                }
        }
        const int kb = base_w + c * 16 * NS;
#pragma unroll
        for (int n = 0; n < 2 * NS; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = kb + n * 8 + 2 * t + (e & 1), p = pos[e >> 1];
                const bool ok = j >= p - P.left && j <= p + P.right && j < P.Skv1;
                s[n][e] = ok ? s[n][e] : -INFINITY;
            }
    };
    float s[2 * NS][4];
    // ---- sweep one: the rows' maximum and sum ----
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    for (int c = 0; c < n_pass; ++c) {
        scores(c, s);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2 * NS; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
        float mus[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float m_new = fmaxf(m_run[i], mx[i]);
            l_run[i] *= m_new == -INFINITY ? 1.f : ptx::ex2((m_run[i] - m_new) * P.sl2);
            m_run[i] = m_new;
            mus[i] = m_new == -INFINITY ? 0.f : m_new * P.sl2;
        }
#pragma unroll
        for (int n = 0; n < 2 * NS; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) l_run[e >> 1] += ptx::ex2(fmaf(s[n][e], P.sl2, -mus[e >> 1]));
    }
    float inv[2], mus[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float l = l_run[i];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        inv[i] = l > 0.f ? 1.f / l : 0.f;
        mus[i] = m_run[i] == -INFINITY ? 0.f : m_run[i] * P.sl2;
    }
    // ---- sweep two: normalised weights, rows (+)= W V, 64 columns at a time ----
    for (int c = 0; c < n_pass; ++c) {
        scores(c, s);
        uint32_t pa[NS][4];   // the weights as A fragments of the 16-key steps
#pragma unroll
        for (int n = 0; n < 2 * NS; ++n) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) w[e] = ptx::ex2(fmaf(s[n][e], P.sl2, -mus[e >> 1])) * inv[e >> 1];
            pa[n >> 1][(n & 1) * 2] = ptx::Mma<T>::pack(w[0], w[1]);
            pa[n >> 1][(n & 1) * 2 + 1] = ptx::Mma<T>::pack(w[2], w[3]);
        }
        const bool last = c + 1 == n_pass;
        for (int sl = 0; sl < n_slices; ++sl) {
            stage(vb_ptr, c, sl);
            const uint32_t v_addr = ptx::smem_u32(sBuf + st_off);
            float acc[2 * KS][4];
#pragma unroll
            for (int n = 0; n < 2 * KS; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < NS; ++kk)
#pragma unroll
                for (int d2 = 0; d2 < KS; ++d2) {
                    uint32_t vf[4];
                    ptx::ldmatrix_x4_trans(vf, v_addr + (uint32_t)(((kk * 16 + r8 + (m4 & 1) * 8) * LD + d2 * 16 + (m4 >> 1) * 8) * 2));
                    ptx::Mma<T>::run(acc[2 * d2], pa[kk], vf[0], vf[1]);
                    ptx::Mma<T>::run(acc[2 * d2 + 1], pa[kk], vf[2], vf[3]);
                }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if ((i == 0 ? row_a : row_b) >= P.Sq1) continue;
                const int64_t off = (i == 0 ? off_a : off_b) + sl * 64 + 2 * t;
#pragma unroll
                for (int n = 0; n < 2 * KS; ++n) {
                    if (sl * 64 + n * 8 + 2 * t >= D) continue;
                    float2 val = make_float2(acc[n][2 * i], acc[n][2 * i + 1]);
                    float2 *sc = reinterpret_cast<float2 *>(scratch + off + n * 8);
                    if (c > 0) { const float2 old = *sc; val.x += old.x; val.y += old.y; }
                    if (last) *reinterpret_cast<uint32_t *>(o + off + n * 8) = ptx::Mma<T>::pack(val.x, val.y);
                    else *sc = val;
                }
            }
        }
    }
}

template <typename T>
int launch_wide_passes(const Problem &p) {
    const int64_t dil = p.pat.dilation;
    WinDParams wp;
    wp.Sq1 = (int32_t)(p.Sq / dil);
    wp.Skv1 = (int32_t)(p.Skv / dil);
    wp.off1 = (int32_t)(p.pat.q_offset / dil);
    wp.HH = (int32_t)(p.H * dil);
    wp.left = (int32_t)std::min<int64_t>(p.pat.left, wp.Skv1);
    wp.right = (int32_t)std::min<int64_t>(p.pat.right, wp.Skv1);
    wp.sl2 = p.scale * 1.4426950408889634f;
    wp.D = (int32_t)p.D;
    auto kern = window_d_wide_passes_kernel<T>;
    constexpr size_t smem = (size_t)(48 + 16 * 5) * 72 * sizeof(T);
    if (int rc = ensure_dynamic_smem((const void *)kern, smem, "cudaFuncSetAttribute(window_d_wide_passes_kernel)")) return rc;
    const dim3 grid((unsigned)wp.HH, (unsigned)((wp.Sq1 + kTQ - 1) / kTQ), (unsigned)p.B);
    kern<<<grid, kThreads, smem, p.stream>>>((const T *)p.q, (const T *)p.k, (const T *)p.v, (T *)p.o, (float *)p.workspace, wp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "window_d_wide_passes_kernel launch");
    note_kernel("mma_window_d");
    return MAT_OK;
}

// NS = 0: the 64-key chunks; otherwise the per-warp walk in passes of NS 16-key steps
template <typename T, int D, int NS>
int launch_d(const Problem &p) {
    const int64_t dil = p.pat.dilation;
    WinDParams wp;
    wp.Sq1 = (int32_t)(p.Sq / dil);
    wp.Skv1 = (int32_t)(p.Skv / dil);
    wp.off1 = (int32_t)(p.pat.q_offset / dil);
    wp.HH = (int32_t)(p.H * dil);
    wp.left = (int32_t)std::min<int64_t>(p.pat.left, wp.Skv1);
    wp.right = (int32_t)std::min<int64_t>(p.pat.right, wp.Skv1);
    wp.sl2 = p.scale * 1.4426950408889634f;
    wp.D = (int32_t)p.D;
    void (*kern)(const T *, const T *, const T *, T *, WinDParams);
    if constexpr (NS > 0) kern = window_d_diag_kernel<T, D, (NS > 0 ? NS : 1)>;
    else kern = window_d_kernel<T, D>;
    constexpr size_t smem = (size_t)(NS > 0 ? 2 * (48 + 16 * NS) : 4 * kTK) * (D + 8) * sizeof(T);
    if (int rc = ensure_dynamic_smem((const void *)kern, smem, "cudaFuncSetAttribute(window_d_kernel)")) return rc;
    const dim3 grid((unsigned)wp.HH, (unsigned)((wp.Sq1 + kTQ - 1) / kTQ), (unsigned)p.B);
    kern<<<grid, kThreads, smem, p.stream>>>((const T *)p.q, (const T *)p.k, (const T *)p.v, (T *)p.o, wp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "window_d_kernel launch");
    note_kernel("mma_window_d");
    return MAT_OK;
}

}  // namespace

// 16-bit window patterns (any taps, any dilation that divides the lengths) with head width 16, 32, 48, 80, 96, 112
// or 128, whole
// tensors (no neighbour shards), 16-byte aligned.  MAT_WINDOW_D_KERNEL=rowwarp keeps the one-warp-per-row
// kernel (a measurement aid).
// fp32 scratch (a copy of the output's shape) for heads that go 64 columns at a time when the window takes a warp
// more than one pass; 0 otherwise
size_t mma_window_d_scratch_bytes(const Problem &p) {
    if (p.pat.kind != MAT_WINDOW || (p.dtype != MAT_BF16 && p.dtype != MAT_F16)) return 0;
    if (p.D % 8 || p.D < 8 || p.D > 512 || p.D == 64 || !(p.D > 128 || p.D % 16) || p.pat.dilation < 1) return 0;
    const int64_t skv1 = p.Skv / p.pat.dilation;
    if (std::min<int64_t>(p.pat.left, skv1) + std::min<int64_t>(p.pat.right, skv1) + 16 <= 144) return 0;
    return (size_t)p.B * p.Sq * p.H * p.D * sizeof(float);
}

bool mma_window_d_supports(const Problem &p) {
    if (p.pat.kind != MAT_WINDOW) return false;
    if (p.dtype != MAT_BF16 && p.dtype != MAT_F16) return false;
    if (p.D % 8 || p.D < 8 || p.D == 64) return false;   // (64: the TMA / tcgen05 kernels; rows stay 16-byte aligned)
    if (p.D > 128 || p.D % 16) {   // 64 columns at a time: windows one pass of a warp covers, or an fp32 scratch copy of the output
        if (p.D > 512 || p.pat.dilation < 1) return false;
        if (mma_window_d_scratch_bytes(p) > 0 && (!p.workspace || p.workspace_bytes < mma_window_d_scratch_bytes(p) ||
                                                  (uintptr_t)p.workspace % 16))
            return false;
    }
    if (p.k_prev || p.k_next || p.q_ts || p.k_ts || p.v_ts || p.o_ts) return false;
    const uintptr_t al = (uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o;
    if (al % 16) return false;
    const int64_t dil = p.pat.dilation;
    if (dil < 1 || p.Sq % dil || p.Skv % dil || p.pat.q_offset % dil) return false;
    if (p.Skv / dil >= (1LL << 30) || p.Sq / dil >= (1LL << 30) || p.H * dil > 0x7fffffffLL || p.B > 65535) return false;
    if ((p.Sq / dil + kTQ - 1) / kTQ > 65535) return false;
    const char *force = std::getenv("MAT_WINDOW_D_KERNEL");
    return !(force && std::strcmp(force, "rowwarp") == 0);
}

template <typename T, int D>
int launch_span(const Problem &p) {
    // Keys a warp's 16 rows can see: up to 80 (64 causal taps) the warp walks its own range in 5 steps of 16, up to
    // 144 (the reference's default window of 64 either side) in 9; wider windows keep the double-buffered chunks.
    // MAT_WINDOW_D_KERNEL=chunks forces those (a measurement aid).
    const int64_t skv1 = p.Skv / p.pat.dilation;
    const int64_t span = std::min<int64_t>(p.pat.left, skv1) + std::min<int64_t>(p.pat.right, skv1) + 16;
    const char *force = std::getenv("MAT_WINDOW_D_KERNEL");
    if (force && std::strcmp(force, "chunks") == 0) return launch_d<T, D, 0>(p);
    if (span <= 80) return launch_d<T, D, 5>(p);
    if (span <= 144) return launch_d<T, D, 9>(p);
    return launch_d<T, D, 0>(p);
}

template <typename T>
int launch_any_d(const Problem &p) {
    switch (p.D) {
        case 16: return launch_span<T, 16>(p);
        case 32: return launch_span<T, 32>(p);
        case 48: return launch_span<T, 48>(p);
        case 80: return launch_span<T, 80>(p);
        case 96: return launch_span<T, 96>(p);
        case 112: return launch_span<T, 112>(p);
        case 128: return launch_span<T, 128>(p);
    }
    return fail(MAT_ERR_UNSUPPORTED, "head width %lld has no instantiation of the warp-level window kernel", (long long)p.D);
}

int launch_mma_window_d(const Problem &p) {
    // a head of 128 columns with a narrow window also goes 64 columns at a time: 79 against 86 us at 65536 tokens x 4
    // heads, 64 causal taps (124 registers instead of 168); MAT_WINDOW_D_KERNEL=whole or chunks keeps it in one piece
    const char *force = std::getenv("MAT_WINDOW_D_KERNEL");
    const bool sliced128 = p.D == 128 && !(force && (std::strcmp(force, "whole") == 0 || std::strcmp(force, "chunks") == 0)) &&
                           std::min<int64_t>(p.pat.left, p.Skv / p.pat.dilation) +
                               std::min<int64_t>(p.pat.right, p.Skv / p.pat.dilation) + 16 <= 144;
    if ((p.D > 128 || p.D % 16) && mma_window_d_scratch_bytes(p) > 0)
        return p.dtype == MAT_BF16 ? launch_wide_passes<__nv_bfloat16>(p) : launch_wide_passes<__half>(p);
    if (p.D > 128 || p.D % 16 || sliced128) {
        const int64_t skv1 = p.Skv / p.pat.dilation;
        const bool five = std::min<int64_t>(p.pat.left, skv1) + std::min<int64_t>(p.pat.right, skv1) + 16 <= 80;
        if (p.dtype == MAT_BF16) return five ? launch_wide<__nv_bfloat16, 5>(p) : launch_wide<__nv_bfloat16, 9>(p);
        return five ? launch_wide<__half, 5>(p) : launch_wide<__half, 9>(p);
    }
    return p.dtype == MAT_BF16 ? launch_any_d<__nv_bfloat16>(p) : launch_any_d<__half>(p);
}

}  // namespace mat
