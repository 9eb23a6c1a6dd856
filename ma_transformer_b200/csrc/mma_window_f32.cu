// fp32 window attention on the tensor cores at fp32 accuracy: every product is evaluated as three TF32
// products of error-compensated halves (x = hi + lo with hi = x rounded to TF32 and lo = x - hi, exact in fp32;
// a * b ~ a_lo b_hi + a_hi b_lo + a_hi b_hi, the missing a_lo b_lo being 2^-22 of the product), accumulated in
// fp32 by mma.sync.m16n8k8.  The reference computes in fp32 (src/csrc/ma_core.cpp:195-240 and the CUDA
// kernel src/cuda/sparse_attention_kernel.cu:211-263), and fp32 is what an unmodified caller of its module
// passes; the parity bar for it (max |gpu - oracle| / max |oracle| <= 1e-5) rules out plain TF32 or 16-bit
// operands but not this.  The FMA-pipe kernel (tiled_f32.cu) needs one FMA per multiply-add of the band; here
// the tensor pipe does three m16n8k8 per 1024 of them.
//
// Same shape as the 16-bit kernel for other head widths (mma_window_d.cu): one CTA = 64 query rows of one
// (batch, head), four warps of 16 rows, the keys the tile can see walked 64 at a time through two cp.async
// buffers, online softmax in registers.  Operands are read from shared memory as scalars (rows padded by four
// floats, which makes both the K and the V fragment loads conflict-free).  The key order inside an 8-key step of
// P V is chosen so that a thread's A fragment is exactly the four weights it already holds (virtual key t is
// key 2t of the step, virtual key t + 4 is key 2t + 1): no shuffles between the two products.
#include <algorithm>
#include <cstring>

#include "mat_common.cuh"
#include "ptx.cuh"

namespace mat {
namespace {

constexpr int kTQ = 64, kTK = 64, kThreads = 128;

struct WinFParams {
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

// d += a b, TF32 operands (the low 13 mantissa bits of the 32-bit operands are not used), fp32 accumulation
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// x = hi + lo.  ROUND = true: hi is x rounded to TF32 (to nearest, by adding half a TF32 ulp to the bit pattern
// and cutting), lo the rest (exact).  A cut hi leaves a lo of x's own sign, and the tensor core cuts lo in turn,
// so every product errs the same way.
// ROUND = false: hi is x itself (the tensor core cuts the low 13 bits) and lo = x - cut(x): two operations instead
// of three per element and no register for hi, 15 % faster, errors up to 5e-6 on a 1000-key row against 2.5e-6;
// used for windows of at most 512 taps, where the sums are short.
template <bool ROUND>
__device__ __forceinline__ void split_tf32(uint32_t x, uint32_t &hi, uint32_t &lo) {
    if (ROUND) {
        hi = (x + 0x1000u) & 0xffffe000u;
        lo = __float_as_uint(__uint_as_float(x) - __uint_as_float(hi));
    } else {
        hi = x;
        lo = __float_as_uint(__uint_as_float(x) - __uint_as_float(x & 0xffffe000u));
    }
}
// d += a b at fp32 accuracy from the halves of a and the raw b
template <bool ROUND>
__device__ __forceinline__ void mma_3x(float (&d)[4], const uint32_t (&a_hi)[4], const uint32_t (&a_lo)[4], uint32_t b0,
                                       uint32_t b1) {
    uint32_t h0, l0, h1, l1;
    split_tf32<ROUND>(b0, h0, l0);
    split_tf32<ROUND>(b1, h1, l1);
    mma_tf32(d, a_lo, h0, h1);
    mma_tf32(d, a_hi, l0, l1);
    mma_tf32(d, a_hi, h0, h1);
}

template <int D, bool ROUND>
__global__ void __launch_bounds__(kThreads)
window_f32_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                  float *__restrict__ o, const WinFParams P) {
    constexpr int LD = D + 4;          // padded row, floats
    constexpr int KS = D / 8;          // k-steps of S = Q K^T; 8-wide output tiles of O
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float *sK = reinterpret_cast<float *>(smem_raw);   // [2][kTK][LD]
    float *sV = sK + 2 * kTK * LD;                     // [2][kTK][LD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int hh = blockIdx.x, b = blockIdx.z, q0 = blockIdx.y * kTQ;
    const int p_first = q0 + P.off1;   // key-coordinate position of the tile's first row
    const int last_row = min(q0 + kTQ, P.Sq1) - 1;
    const int key_lo = max(0, p_first - P.left);
    const int key_hi = min(P.Skv1 - 1, last_row + P.off1 + P.right);
    const int n_chunks = key_hi >= key_lo ? (key_hi - key_lo) / kTK + 1 : 0;
    const int64_t tok = (int64_t)P.HH * D;   // elements per token
    const float *kb_ptr = k + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const float *vb_ptr = v + ((int64_t)b * P.Skv1 * P.HH + hh) * D;

    auto load_chunk = [&](int c, int buf) {
        constexpr int kPieces = D / 4;   // 16-byte pieces per row
        const int base = key_lo + c * kTK;
        for (int i = threadIdx.x; i < kTK * kPieces; i += kThreads) {
            const int r = i / kPieces, pc = i % kPieces;
            const int j = base + r;
            const bool in = j < P.Skv1;   // rows past the sequence end are zero-filled: a masked weight never meets stale memory
            const int64_t src = (int64_t)(in ? j : 0) * tok + pc * 4;
            cp_async16(sK + (buf * kTK + r) * LD + pc * 4, kb_ptr + src, in ? 16 : 0);
            cp_async16(sV + (buf * kTK + r) * LD + pc * 4, vb_ptr + src, in ? 16 : 0);
        }
    };
    if (n_chunks > 0) load_chunk(0, 0);
    cp_async_commit();

    // the warp's 16 query rows as A fragments: thread (g, t) holds rows g and g + 8, columns t and t + 4 of each 8
    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    uint32_t qf[KS][4];
    {
        const float *qa = q + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D;
        const float *qb = q + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 8 + t;
            qf[ks][0] = row_a < P.Sq1 ? __float_as_uint(qa[c]) : 0u;
            qf[ks][1] = row_b < P.Sq1 ? __float_as_uint(qb[c]) : 0u;
            qf[ks][2] = row_a < P.Sq1 ? __float_as_uint(qa[c + 4]) : 0u;
            qf[ks][3] = row_b < P.Sq1 ? __float_as_uint(qb[c + 4]) : 0u;
        }
    }
    const int pos[2] = {row_a + P.off1, row_b + P.off1};
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[KS][4];
#pragma unroll
    for (int n = 0; n < KS; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

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
        const uint32_t *ck = reinterpret_cast<const uint32_t *>(sK + buf * kTK * LD);
        const uint32_t *cv = reinterpret_cast<const uint32_t *>(sV + buf * kTK * LD);

        // ---- S = Q K^T: eight 8-key tiles per warp ----
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t q_hi[4], q_lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_tf32<ROUND>(qf[ks][e], q_hi[e], q_lo[e]);
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                // B = K^T: element (k = dim, n = key): b0 = K[key g][dim t], b1 = K[key g][dim t + 4] of the step
                const uint32_t *kr = ck + (n * 8 + g) * LD + ks * 8 + t;
                mma_3x<ROUND>(s[n], q_hi, q_lo, kr[0], kr[4]);
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
        // ---- the chunk's P V, one 8-key step per score tile, into accumulators of its own ----
        // (The tensor core does not round its fp32 sums to nearest, so a long chain of accumulating MMAs drifts:
        // 9e-6 relative on a 1000-key row with one chain per output tile.  The chains end with the chunk; the
        // chunks are combined by ordinary FMAs, which is also where the running maximum's rescale goes.)
        float part[KS][4];
#pragma unroll
        for (int n = 0; n < KS; ++n) part[n][0] = part[n][1] = part[n][2] = part[n][3] = 0.f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                w[e] = ptx::ex2(fmaf(s[n][e], P.sl2, -mus[e >> 1]));
                l_run[e >> 1] += w[e];
            }
            // A fragment in the step's own key order (virtual key t = key 2t, virtual key t + 4 = key 2t + 1):
            // rows g and g + 8 at virtual keys t and t + 4 are the four weights this thread holds
            const uint32_t pa[4] = {__float_as_uint(w[0]), __float_as_uint(w[2]), __float_as_uint(w[1]), __float_as_uint(w[3])};
            uint32_t p_hi[4], p_lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_tf32<ROUND>(pa[e], p_hi[e], p_lo[e]);
            const uint32_t *vr = cv + (n * 8 + 2 * t) * LD + g;
#pragma unroll
            for (int d = 0; d < KS; ++d)   // B: element (k = virtual key, n = dim): rows 2t and 2t + 1 of the step
                mma_3x<ROUND>(part[d], p_hi, p_lo, vr[d * 8], vr[LD + d * 8]);
        }
#pragma unroll
        for (int n = 0; n < KS; ++n) {
            acc[n][0] = fmaf(acc[n][0], alpha[0], part[n][0]);
            acc[n][1] = fmaf(acc[n][1], alpha[0], part[n][1]);
            acc[n][2] = fmaf(acc[n][2], alpha[1], part[n][2]);
            acc[n][3] = fmaf(acc[n][3], alpha[1], part[n][3]);
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
            float *dst = o + (((int64_t)b * P.Sq1 + row) * P.HH + hh) * D + 2 * t;
#pragma unroll
            for (int n = 0; n < KS; ++n)
                *reinterpret_cast<float2 *>(dst + n * 8) = make_float2(acc[n][2 * i] * inv, acc[n][2 * i + 1] * inv);
        }
    }
}

// Narrow windows.  In the kernel above a warp multiplies its 16 rows with all 64 keys of every chunk, although the
// band crosses the tile as a parallelogram: at 64 causal taps a warp needs 79 of the 127 keys the tile sees, 10 of
// the 16 score tiles it computes.  Skipping the others by a branch per tile was measured slower (the branches keep
// the compiler from overlapping the tiles).  Here every warp walks keys from a base of its own, the first key its
// first row can see, in passes of NT 8-key tiles: the same straight-line code for every warp, no tile without a
// visible key but the last of the walk.  The CTA stages the 48 + 8 NT rows the four warps' passes span.
template <int D, bool ROUND, int NT>
__global__ void __launch_bounds__(kThreads)
window_f32_diag_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                       float *__restrict__ o, const WinFParams P) {
    constexpr int LD = D + 4, KS = D / 8;
    constexpr int kStage = 48 + 8 * NT;   // rows of K and of V in shared memory
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float *sK = reinterpret_cast<float *>(smem_raw);   // [kStage][LD]
    float *sV = sK + kStage * LD;                      // [kStage][LD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int hh = blockIdx.x, b = blockIdx.z, q0 = blockIdx.y * kTQ;
    const int p_first = q0 + P.off1;
    const int key_lo = max(0, p_first - P.left);
    const int key_hi = min(P.Skv1 - 1, min(q0 + kTQ, P.Sq1) - 1 + P.off1 + P.right);
    const int base_w = max(key_lo, p_first + 16 * warp - P.left);   // the warp's first key
    int n_pass = 0;   // passes of the warp with the longest walk (the bases of a sequence's first tiles are clamped)
    if (key_hi >= key_lo) {
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) {
            const int keys_w = min(key_hi, p_first + 16 * w + 15 + P.right) - max(key_lo, p_first + 16 * w - P.left) + 1;
            n_pass = max(n_pass, (keys_w + 8 * NT - 1) / (8 * NT));
        }
    }
    const int64_t tok = (int64_t)P.HH * D;
    const float *kb_ptr = k + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const float *vb_ptr = v + ((int64_t)b * P.Skv1 * P.HH + hh) * D;

    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    uint32_t qf[KS][4];
    {
        const float *qa = q + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D;
        const float *qb = q + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 8 + t;
            qf[ks][0] = row_a < P.Sq1 ? __float_as_uint(qa[c]) : 0u;
            qf[ks][1] = row_b < P.Sq1 ? __float_as_uint(qb[c]) : 0u;
            qf[ks][2] = row_a < P.Sq1 ? __float_as_uint(qa[c + 4]) : 0u;
            qf[ks][3] = row_b < P.Sq1 ? __float_as_uint(qb[c + 4]) : 0u;
        }
    }
    const int pos[2] = {row_a + P.off1, row_b + P.off1};
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[KS][4];
#pragma unroll
    for (int n = 0; n < KS; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

    for (int c = 0; c < n_pass; ++c) {
        const int stage_lo = key_lo + c * 8 * NT;   // warp 0's base is key_lo
        if (stage_lo > key_hi) break;
        if (c) __syncthreads();   // the previous pass has been read
        {
            constexpr int kPieces = D / 4;
            for (int i = threadIdx.x; i < kStage * kPieces; i += kThreads) {
                const int r = i / kPieces, pc = i % kPieces;
                const int j = stage_lo + r;
                const bool in = j <= key_hi;   // rows past the tile's last key are zero-filled
                const int64_t src = (int64_t)(in ? j : 0) * tok + pc * 4;
                cp_async16(sK + r * LD + pc * 4, kb_ptr + src, in ? 16 : 0);
                cp_async16(sV + r * LD + pc * 4, vb_ptr + src, in ? 16 : 0);
            }
            cp_async_commit();
            cp_async_wait<0>();
        }
        __syncthreads();
        const int kb = base_w + c * 8 * NT;   // the warp's first key of the pass
        const uint32_t *ck = reinterpret_cast<const uint32_t *>(sK + (kb - stage_lo) * LD);
        const uint32_t *cv = reinterpret_cast<const uint32_t *>(sV + (kb - stage_lo) * LD);

        float s[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t q_hi[4], q_lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_tf32<ROUND>(qf[ks][e], q_hi[e], q_lo[e]);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const uint32_t *kr = ck + (n * 8 + g) * LD + ks * 8 + t;
                mma_3x<ROUND>(s[n], q_hi, q_lo, kr[0], kr[4]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < NT; ++n)
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
        float part[KS][4];   // the pass's P V in accumulators of its own (short chains, see above)
#pragma unroll
        for (int n = 0; n < KS; ++n) part[n][0] = part[n][1] = part[n][2] = part[n][3] = 0.f;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                w[e] = ptx::ex2(fmaf(s[n][e], P.sl2, -mus[e >> 1]));
                l_run[e >> 1] += w[e];
            }
            const uint32_t pa[4] = {__float_as_uint(w[0]), __float_as_uint(w[2]), __float_as_uint(w[1]), __float_as_uint(w[3])};
            uint32_t p_hi[4], p_lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_tf32<ROUND>(pa[e], p_hi[e], p_lo[e]);
            const uint32_t *vr = cv + (n * 8 + 2 * t) * LD + g;
#pragma unroll
            for (int d = 0; d < KS; ++d) mma_3x<ROUND>(part[d], p_hi, p_lo, vr[d * 8], vr[LD + d * 8]);
            if (NT > 10 && n == NT / 2 - 1) {   // a long pass ends its accumulation chains half way, like a chunk
#pragma unroll
                for (int d = 0; d < KS; ++d) {
                    acc[d][0] = fmaf(acc[d][0], alpha[0], part[d][0]);
                    acc[d][1] = fmaf(acc[d][1], alpha[0], part[d][1]);
                    acc[d][2] = fmaf(acc[d][2], alpha[1], part[d][2]);
                    acc[d][3] = fmaf(acc[d][3], alpha[1], part[d][3]);
                    part[d][0] = part[d][1] = part[d][2] = part[d][3] = 0.f;
                }
                alpha[0] = alpha[1] = 1.f;
            }
        }
#pragma unroll
        for (int n = 0; n < KS; ++n) {
            acc[n][0] = fmaf(acc[n][0], alpha[0], part[n][0]);
            acc[n][1] = fmaf(acc[n][1], alpha[0], part[n][1]);
            acc[n][2] = fmaf(acc[n][2], alpha[1], part[n][2]);
            acc[n][3] = fmaf(acc[n][3], alpha[1], part[n][3]);
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
            float *dst = o + (((int64_t)b * P.Sq1 + row) * P.HH + hh) * D + 2 * t;
#pragma unroll
            for (int n = 0; n < KS; ++n)
                *reinterpret_cast<float2 *>(dst + n * 8) = make_float2(acc[n][2 * i] * inv, acc[n][2 * i + 1] * inv);
        }
    }
}

// Wide heads (D = 128, 192, ... 512: the reference's layer passes one head of width model_dim,
// src/layers/sparse_attention.py:71-78) with narrow windows: the per-warp walk of the kernel above in a single pass,
// the head dimension taken 64 columns at a time.  The K slices stream through two buffers while the scores
// accumulate, then the V slices while each 64-column slice of the output is formed from the finished weights,
// normalised and written; the copy of the next slice is in flight during the products of the current one.
// Registers hold the scores / weights of the pass (NT tiles) and one slice's operands, whatever D is.
// (ROUND: rounded high halves, for heads of 256 columns and more, whose long dot products need them)
template <int NT, bool ROUND>
__global__ void __launch_bounds__(kThreads)
window_f32_wide_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                       float *__restrict__ o, const WinFParams P) {
    constexpr int LD = 64 + 4, KS = 8;
    constexpr int kStage = 48 + 8 * NT;   // rows of a slice in shared memory
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float *sBuf = reinterpret_cast<float *>(smem_raw);   // [2][kStage][LD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int hh = blockIdx.x, b = blockIdx.z, q0 = blockIdx.y * kTQ;
    const int D = P.D, n_slices = (D + 63) >> 6;   // (the last slice may be partly beyond D: zeros in, nothing out)
    const int p_first = q0 + P.off1;
    const int key_lo = max(0, p_first - P.left);
    const int key_hi = min(P.Skv1 - 1, min(q0 + kTQ, P.Sq1) - 1 + P.off1 + P.right);
    const int base_w = max(key_lo, p_first + 16 * warp - P.left);   // the warp's first key
    const int64_t tok = (int64_t)P.HH * D;
    const float *kb_ptr = k + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const float *vb_ptr = v + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    const float *qa = q + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D;
    const float *qb = q + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D;
    float *oa = o + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D + 2 * t;
    float *ob = o + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D + 2 * t;

    if (key_hi < key_lo) {   // a tile whose rows see no key (the whole CTA alike): zeros
        for (int c = 0; c + 2 * t < D; c += 8) {
            if (row_a < P.Sq1) *reinterpret_cast<float2 *>(oa + c) = make_float2(0.f, 0.f);
            if (row_b < P.Sq1) *reinterpret_cast<float2 *>(ob + c) = make_float2(0.f, 0.f);
        }
        return;
    }
    // copy i of the pass: K slice i, then V slice i - n_slices, into buffer i & 1
    auto issue = [&](int i) {
        const int col0 = (i < n_slices ? i : i - n_slices) * 64;
        const float *src_base = (i < n_slices ? kb_ptr : vb_ptr) + col0;
        float *dst = sBuf + (i & 1) * kStage * LD;
        for (int x = threadIdx.x; x < kStage * 16; x += kThreads) {
            const int r = x >> 4, pc = x & 15;
            const int j = key_lo + r;
            const bool in = j <= key_hi && col0 + pc * 4 < D;   // rows past the tile's last key and columns past D are zero-filled
            cp_async16(dst + r * LD + pc * 4, src_base + (int64_t)(in ? j : 0) * tok + pc * 4, in ? 16 : 0);
        }
        cp_async_commit();
    };
    issue(0);
    const int row_off = (base_w - key_lo) * LD;   // the warp's first key inside a buffer

    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    for (int sl = 0; sl < n_slices; ++sl) {
        uint32_t qf[KS][4];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = sl * 64 + ks * 8 + t;   // (D is a multiple of 4: each half of an 8-column step is inside D or beyond it)
            qf[ks][0] = row_a < P.Sq1 && c < D ? __float_as_uint(qa[c]) : 0u;
            qf[ks][1] = row_b < P.Sq1 && c < D ? __float_as_uint(qb[c]) : 0u;
            qf[ks][2] = row_a < P.Sq1 && c + 4 < D ? __float_as_uint(qa[c + 4]) : 0u;
            qf[ks][3] = row_b < P.Sq1 && c + 4 < D ? __float_as_uint(qb[c + 4]) : 0u;
        }
        issue(sl + 1);   // the next K slice, or the first V slice
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t *ck = reinterpret_cast<const uint32_t *>(sBuf + (sl & 1) * kStage * LD + row_off);
        // (ten tiles: a slice's share of the scores in accumulators of its own, added by ordinary additions - the
        // tensor core's fp32 sums are not rounded to nearest, and a chain over several hundred columns drifts;
        // eighteen tiles leave no registers for that)
        constexpr bool kOwn = NT <= 10;
        float ss[kOwn ? NT : 1][4];
        if constexpr (kOwn) {
#pragma unroll
            for (int n = 0; n < NT; ++n) ss[n][0] = ss[n][1] = ss[n][2] = ss[n][3] = 0.f;
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t q_hi[4], q_lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_tf32<ROUND>(qf[ks][e], q_hi[e], q_lo[e]);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const uint32_t *kr = ck + (n * 8 + g) * LD + ks * 8 + t;
                if constexpr (kOwn) mma_3x<ROUND>(ss[n], q_hi, q_lo, kr[0], kr[4]);
                else mma_3x<ROUND>(s[n], q_hi, q_lo, kr[0], kr[4]);
            }
        }
        if constexpr (kOwn) {
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[n][e] += ss[n][e];
        }
        __syncthreads();   // the buffer is free for the copy after the next
    }
    // ---- mask and softmax of the whole row (one pass: no running maximum) ----
    const int pos[2] = {row_a + P.off1, row_b + P.off1};
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n)
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
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            s[n][e] = ptx::ex2(fmaf(s[n][e], P.sl2, -mus[e >> 1]));
            l[e >> 1] += s[n][e];
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
        const uint32_t *cv = reinterpret_cast<const uint32_t *>(sBuf + (i & 1) * kStage * LD + row_off);
        // two accumulation chains per output tile (the tensor core's fp32 sums are not rounded to nearest: chains
        // stay at most 72 keys long), added at the end
        float part[2][KS][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int d = 0; d < KS; ++d) part[h][d][0] = part[h][d][1] = part[h][d][2] = part[h][d][3] = 0.f;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const uint32_t pa[4] = {__float_as_uint(s[n][0]), __float_as_uint(s[n][2]), __float_as_uint(s[n][1]),
                                    __float_as_uint(s[n][3])};
            uint32_t p_hi[4], p_lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_tf32<ROUND>(pa[e], p_hi[e], p_lo[e]);
            const uint32_t *vr = cv + (n * 8 + 2 * t) * LD + g;
#pragma unroll
            for (int d = 0; d < KS; ++d) mma_3x<ROUND>(part[n < NT / 2 ? 0 : 1][d], p_hi, p_lo, vr[d * 8], vr[LD + d * 8]);
        }
#pragma unroll
        for (int d = 0; d < KS; ++d) {
            if (sl * 64 + d * 8 + 2 * t >= D) continue;
            if (row_a < P.Sq1)
                *reinterpret_cast<float2 *>(oa + sl * 64 + d * 8) =
                    make_float2((part[0][d][0] + part[1][d][0]) * inv[0], (part[0][d][1] + part[1][d][1]) * inv[0]);
            if (row_b < P.Sq1)
                *reinterpret_cast<float2 *>(ob + sl * 64 + d * 8) =
                    make_float2((part[0][d][2] + part[1][d][2]) * inv[1], (part[0][d][3] + part[1][d][3]) * inv[1]);
        }
        __syncthreads();   // the buffer is free for the copy after the next
    }
}

// Wide heads with windows that take a warp more than one pass (up to dense): two sweeps over the passes, the head
// dimension 64 columns at a time in both.  Sweep one accumulates each pass's scores over the K slices and keeps the
// running maximum and sum of the rows; sweep two forms the scores again, turns them into normalised weights, and adds
// their product with every V slice to the output rows, which the first pass of a row wrote (a row of the output
// belongs to one thread pair of one CTA, so the read-modify-write needs no atomics).  One buffer per operand: the
// three CTAs of an SM cover each other's copies.
template <int NT>
__global__ void __launch_bounds__(kThreads)
window_f32_wide_passes_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                              float *__restrict__ o, const WinFParams P) {
    constexpr int LD = 64 + 4, KS = 8;
    constexpr int kStage = 48 + 8 * NT;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float *sBuf = reinterpret_cast<float *>(smem_raw);   // [kStage][LD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int hh = blockIdx.x, b = blockIdx.z, q0 = blockIdx.y * kTQ;
    const int D = P.D, n_slices = (D + 63) >> 6;   // (the last slice may be partly beyond D: zeros in, nothing out)
    const int p_first = q0 + P.off1;
    const int key_lo = max(0, p_first - P.left);
    const int key_hi = min(P.Skv1 - 1, min(q0 + kTQ, P.Sq1) - 1 + P.off1 + P.right);
    const int base_w = max(key_lo, p_first + 16 * warp - P.left);   // the warp's first key
    const int st_off = (base_w - key_lo) * LD;                      // its row inside the staged range of a pass
    int n_pass = 0;
    if (key_hi >= key_lo) {
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) {
            const int keys_w = min(key_hi, p_first + 16 * w + 15 + P.right) - max(key_lo, p_first + 16 * w - P.left) + 1;
            n_pass = max(n_pass, (keys_w + 8 * NT - 1) / (8 * NT));
        }
        n_pass = min(n_pass, (key_hi - key_lo) / (8 * NT) + 1);
    }
    const int64_t tok = (int64_t)P.HH * D;
    const float *kb_ptr = k + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const float *vb_ptr = v + ((int64_t)b * P.Skv1 * P.HH + hh) * D;
    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    const float *qa = q + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D;
    const float *qb = q + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D;
    float *oa = o + (((int64_t)b * P.Sq1 + row_a) * P.HH + hh) * D + 2 * t;
    float *ob = o + (((int64_t)b * P.Sq1 + row_b) * P.HH + hh) * D + 2 * t;
    const int pos[2] = {row_a + P.off1, row_b + P.off1};

    if (n_pass == 0) {   // a tile whose rows see no key (the whole CTA alike): zeros
        for (int c = 0; c + 2 * t < D; c += 8) {
            if (row_a < P.Sq1) *reinterpret_cast<float2 *>(oa + c) = make_float2(0.f, 0.f);
            if (row_b < P.Sq1) *reinterpret_cast<float2 *>(ob + c) = make_float2(0.f, 0.f);
        }
        return;
    }
    // one 64-column slice of the kStage rows of pass c, of K or V; rows past the tile's last key are zeros
    auto stage = [&](const float *src, int c, int slice) {
        const int first = key_lo + c * 8 * NT;
        __syncthreads();   // whoever still read the buffer is done
        for (int x = threadIdx.x; x < kStage * 16; x += kThreads) {
            const int r = x >> 4, pc = x & 15;
            const int j = first + r;
            const bool in = j <= key_hi && slice * 64 + pc * 4 < D;
            cp_async16(sBuf + r * LD + pc * 4, src + (int64_t)(in ? j : 0) * tok + slice * 64 + pc * 4, in ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
    };
    // the masked scores of pass c
    auto scores = [&](int c, float (&s)[NT][4]) {
#pragma unroll
        for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        for (int sl = 0; sl < n_slices; ++sl) {
            uint32_t qf[KS][4];
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int col = sl * 64 + ks * 8 + t;
                qf[ks][0] = row_a < P.Sq1 && col < D ? __float_as_uint(qa[col]) : 0u;
                qf[ks][1] = row_b < P.Sq1 && col < D ? __float_as_uint(qb[col]) : 0u;
                qf[ks][2] = row_a < P.Sq1 && col + 4 < D ? __float_as_uint(qa[col + 4]) : 0u;
                qf[ks][3] = row_b < P.Sq1 && col + 4 < D ? __float_as_uint(qb[col + 4]) : 0u;
            }
            stage(kb_ptr, c, sl);
            const uint32_t *ck = reinterpret_cast<const uint32_t *>(sBuf + st_off);
            // a slice's share of the scores in accumulators of its own, added by ordinary additions: the tensor
            // core's fp32 sums are not rounded to nearest, and a chain over 256 or 512 columns drifts (1.04e-5 on
            // dense rows of 4096 keys at D = 256 with one chain)
            float ss[NT][4];
#pragma unroll
            for (int n = 0; n < NT; ++n) ss[n][0] = ss[n][1] = ss[n][2] = ss[n][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t q_hi[4], q_lo[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) split_tf32<true>(qf[ks][e], q_hi[e], q_lo[e]);
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const uint32_t *kr = ck + (n * 8 + g) * LD + ks * 8 + t;
                    mma_3x<true>(ss[n], q_hi, q_lo, kr[0], kr[4]);
                }
            }
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[n][e] += ss[n][e];
        }
        const int kb = base_w + c * 8 * NT;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = kb + n * 8 + 2 * t + (e & 1), p = pos[e >> 1];
                const bool ok = j >= p - P.left && j <= p + P.right && j < P.Skv1;
                s[n][e] = ok ? s[n][e] : -INFINITY;
            }
    };
    float s[NT][4];
    // ---- sweep one: the rows' maximum and sum ----
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    for (int c = 0; c < n_pass; ++c) {
        scores(c, s);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < NT; ++n)
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
        for (int n = 0; n < NT; ++n)
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
    // ---- sweep two: normalised weights, output rows (+)= W V, 64 columns at a time ----
    for (int c = 0; c < n_pass; ++c) {
        scores(c, s);
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = ptx::ex2(fmaf(s[n][e], P.sl2, -mus[e >> 1])) * inv[e >> 1];
        for (int sl = 0; sl < n_slices; ++sl) {
            stage(vb_ptr, c, sl);
            const uint32_t *cv = reinterpret_cast<const uint32_t *>(sBuf + st_off);
            float part[KS][4];
#pragma unroll
            for (int d = 0; d < KS; ++d) part[d][0] = part[d][1] = part[d][2] = part[d][3] = 0.f;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const uint32_t pa[4] = {__float_as_uint(s[n][0]), __float_as_uint(s[n][2]), __float_as_uint(s[n][1]),
                                        __float_as_uint(s[n][3])};
                uint32_t p_hi[4], p_lo[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) split_tf32<true>(pa[e], p_hi[e], p_lo[e]);
                const uint32_t *vr = cv + (n * 8 + 2 * t) * LD + g;
#pragma unroll
                for (int d = 0; d < KS; ++d) mma_3x<true>(part[d], p_hi, p_lo, vr[d * 8], vr[LD + d * 8]);
            }
#pragma unroll
            for (int d = 0; d < KS; ++d) {
                if (sl * 64 + d * 8 + 2 * t >= D) continue;
                if (row_a < P.Sq1) {
                    float2 val = make_float2(part[d][0], part[d][1]);
                    float2 *dst = reinterpret_cast<float2 *>(oa + sl * 64 + d * 8);
                    if (c > 0) { const float2 old = *dst; val.x += old.x; val.y += old.y; }
                    *dst = val;
                }
                if (row_b < P.Sq1) {
                    float2 val = make_float2(part[d][2], part[d][3]);
                    float2 *dst = reinterpret_cast<float2 *>(ob + sl * 64 + d * 8);
                    if (c > 0) { const float2 old = *dst; val.x += old.x; val.y += old.y; }
                    *dst = val;
                }
            }
        }
    }
}

template <int NT, bool PASSES, bool ROUND>
int launch_wide(const Problem &p) {
    const int64_t dil = p.pat.dilation;
    WinFParams wp;
    wp.Sq1 = (int32_t)(p.Sq / dil);
    wp.Skv1 = (int32_t)(p.Skv / dil);
    wp.off1 = (int32_t)(p.pat.q_offset / dil);
    wp.HH = (int32_t)(p.H * dil);
    wp.left = (int32_t)std::min<int64_t>(p.pat.left, wp.Skv1);
    wp.right = (int32_t)std::min<int64_t>(p.pat.right, wp.Skv1);
    wp.sl2 = p.scale * 1.4426950408889634f;
    wp.D = (int32_t)p.D;
    auto kern = PASSES ? window_f32_wide_passes_kernel<NT> : window_f32_wide_kernel<NT, ROUND>;
    constexpr size_t smem = (size_t)(PASSES ? 1 : 2) * (48 + 8 * NT) * 68 * sizeof(float);
    if (int rc = ensure_dynamic_smem((const void *)kern, smem, "cudaFuncSetAttribute(window_f32_wide_kernel)")) return rc;
    const dim3 grid((unsigned)wp.HH, (unsigned)((wp.Sq1 + kTQ - 1) / kTQ), (unsigned)p.B);
    kern<<<grid, kThreads, smem, p.stream>>>((const float *)p.q, (const float *)p.k, (const float *)p.v, (float *)p.o, wp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "window_f32_wide_kernel launch");
    note_kernel("mma_window_f32");
    return MAT_OK;
}

// NT = 0: the 64-key chunks; otherwise the per-warp walk in passes of NT tiles
template <int D, bool ROUND, int NT>
int launch_f(const Problem &p) {
    constexpr bool DIAG = NT > 0;
    const int64_t dil = p.pat.dilation;
    WinFParams wp;
    wp.Sq1 = (int32_t)(p.Sq / dil);
    wp.Skv1 = (int32_t)(p.Skv / dil);
    wp.off1 = (int32_t)(p.pat.q_offset / dil);
    wp.HH = (int32_t)(p.H * dil);
    wp.left = (int32_t)std::min<int64_t>(p.pat.left, wp.Skv1);
    wp.right = (int32_t)std::min<int64_t>(p.pat.right, wp.Skv1);
    wp.sl2 = p.scale * 1.4426950408889634f;
    wp.D = (int32_t)p.D;
    void (*kern)(const float *, const float *, const float *, float *, WinFParams);
    if constexpr (DIAG) kern = window_f32_diag_kernel<D, ROUND, DIAG ? NT : 1>;
    else kern = window_f32_kernel<D, ROUND>;
    constexpr size_t smem = (size_t)(DIAG ? 2 * (48 + 8 * NT) : 4 * kTK) * (D + 4) * sizeof(float);
    if (int rc = ensure_dynamic_smem((const void *)kern, smem, "cudaFuncSetAttribute(window_f32_kernel)")) return rc;
    const dim3 grid((unsigned)wp.HH, (unsigned)((wp.Sq1 + kTQ - 1) / kTQ), (unsigned)p.B);
    kern<<<grid, kThreads, smem, p.stream>>>((const float *)p.q, (const float *)p.k, (const float *)p.v, (float *)p.o, wp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "window_f32_kernel launch");
    note_kernel("mma_window_f32");
    return MAT_OK;
}

}  // namespace

// the instantiation for the problem's head width (16, 32, 48, 64 or 96 columns)
template <bool ROUND, int NT>
static int launch_head(const Problem &p) {
    switch (p.D) {
    case 16: return launch_f<16, ROUND, NT>(p);
    case 32: return launch_f<32, ROUND, NT>(p);
    case 48: return launch_f<48, ROUND, NT>(p);
    case 96: return launch_f<96, ROUND, (NT == 18 ? 10 : NT)>(p);
    default: return launch_f<64, ROUND, NT>(p);
    }
}

// keys a warp's 16 rows can see
static int64_t warp_span(const Problem &p) {
    const int64_t skv1 = p.Skv / p.pat.dilation;
    return std::min<int64_t>(p.pat.left, skv1) + std::min<int64_t>(p.pat.right, skv1) + 16;
}

// fp32 window patterns (any taps, any dilation that divides the lengths) with a head width that is a multiple of 4
// up to 512 (16, 32, 48, 64 and 96 columns have instantiations of their own, the others go 64 columns at a time);
// whole tensors, 16-byte aligned.
// MAT_F32_KERNEL=tiled keeps them on the FMA-pipe kernels (a measurement aid).
bool mma_window_f32_supports(const Problem &p) {
    if (p.pat.kind != MAT_WINDOW || p.dtype != MAT_F32) return false;
    const bool narrow_head = p.D == 16 || p.D == 32 || p.D == 48 || p.D == 64 || p.D == 96;   // (96: 768 columns in 8 heads)
    const bool wide_head = !narrow_head && p.D >= 4 && p.D <= 512 && p.D % 4 == 0;   // 64 columns at a time (rows stay 16-byte aligned)
    if (!narrow_head && !wide_head) return false;
    if (wide_head && p.pat.dilation < 1) return false;
    if (p.k_prev || p.k_next || p.q_ts || p.k_ts || p.v_ts || p.o_ts) return false;
    const uintptr_t al = (uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o;
    if (al % 16) return false;
    const int64_t dil = p.pat.dilation;
    if (dil < 1 || p.Sq % dil || p.Skv % dil || p.pat.q_offset % dil) return false;
    if (p.Skv / dil >= (1LL << 30) || p.Sq / dil >= (1LL << 30) || p.H * dil > 0x7fffffffLL || p.B > 65535) return false;
    if ((p.Sq / dil + kTQ - 1) / kTQ > 65535) return false;
    const char *force = std::getenv("MAT_F32_KERNEL");
    return !(force && std::strcmp(force, "tiled") == 0);
}

int launch_mma_window_f32(const Problem &p) {
    if (p.D != 16 && p.D != 32 && p.D != 48 && p.D != 64 && p.D != 96) {   // 64 columns at a time: one pass of 10 or 18 tiles per warp; wider windows, up to dense: passes of 10
        if (warp_span(p) > 144) return launch_wide<10, true, true>(p);
        // 18 tiles on a head of 512 columns stayed at 1.2e-5 with cut halves and one chain per score: two passes of 10
        if (warp_span(p) > 80 && p.D > 256) return launch_wide<10, true, true>(p);
        if (p.D >= 256) return warp_span(p) <= 80 ? launch_wide<10, false, true>(p) : launch_wide<18, false, true>(p);
        return warp_span(p) <= 80 ? launch_wide<10, false, false>(p) : launch_wide<18, false, false>(p);
    }
    if (const char *f = std::getenv("MAT_F32_KERNEL"); f && std::strcmp(f, "sliced") == 0 && p.D == 64 && warp_span(p) <= 144)
        return warp_span(p) <= 80 ? launch_wide<10, false, false>(p) : launch_wide<18, false, false>(p);   // (a measurement aid)
    const int64_t dil = p.pat.dilation, skv1 = p.Skv / dil;
    const bool wide = std::min<int64_t>(p.pat.left, skv1) + std::min<int64_t>(p.pat.right, skv1) > 512;
    if (wide) return launch_head<true, 0>(p);
    // Keys a warp's 16 rows can see.  Up to 144 the warp walks its own range in one pass (6, 10 or 18 tiles: 32
    // causal taps, 64 causal taps, the reference's default window of 64 either side), up to 160 in two passes of 10;
    // wider windows keep the double-buffered chunks.  MAT_F32_KERNEL=chunks forces those (a measurement aid),
    // MAT_F32_TILES=6|10|18 the pass length.
    const int64_t span = std::min<int64_t>(p.pat.left, skv1) + std::min<int64_t>(p.pat.right, skv1) + 16;
    const char *force = std::getenv("MAT_F32_KERNEL");
    int nt = span <= 48 ? 6 : span <= 80 ? 10 : span <= 144 ? 18 : span <= 160 ? 10 : 0;
    if (force && std::strcmp(force, "chunks") == 0) nt = 0;
    if (const char *t = std::getenv("MAT_F32_TILES"); t && nt) nt = std::atoi(t);
    if (nt == 18 && p.D == 96) nt = span <= 160 ? 10 : 0;   // (18 tiles of a 96-wide head do not fit the registers: two passes of 10)
    switch (nt) {
    case 6: return launch_head<false, 6>(p);
    case 10: return launch_head<false, 10>(p);
    case 18: return launch_head<false, 18>(p);
    default: return launch_head<false, 0>(p);
    }
}

}  // namespace mat
