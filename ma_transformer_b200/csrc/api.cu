// extern "C" surface of libmat_sparse_attn: argument validation, kernel
// selection and the host-side index sets.  Declarations and the reference
// interfaces they stand in for are in include/mat_sparse_attn.h.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "mat_common.cuh"

namespace mat {

static thread_local std::string g_last_error;
static thread_local const char *g_last_kernel = "";

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int cuda_fail(cudaError_t e, const char *what) {
    return fail(MAT_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

void note_kernel(const char *name) { g_last_kernel = name; }

int ensure_dynamic_smem(const void *kernel, size_t bytes, const char *what) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, size_t> done;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    std::lock_guard<std::mutex> lock(mu);
    size_t &have = done[{kernel, dev}];
    if (have >= bytes) return MAT_OK;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return cuda_fail(e, what);
    have = bytes;
    return MAT_OK;
}

static int check_spec(const mat_pattern_spec *s) {
    if (!s) return fail(MAT_ERR_INVALID, "pattern description is NULL");
    if (s->q_offset < 0) return fail(MAT_ERR_INVALID, "q_offset must be >= 0");
    switch (s->kind) {
        case MAT_WINDOW:
            if (s->left < 0 || s->right < 0)
                return fail(MAT_ERR_INVALID, "window taps must be >= 0 (left=%lld right=%lld)",
                            (long long)s->left, (long long)s->right);
            if (s->dilation < 1) return fail(MAT_ERR_INVALID, "dilation must be >= 1");
            return MAT_OK;
        case MAT_BLOCK:
            if (s->block < 1) return fail(MAT_ERR_INVALID, "block size must be >= 1");
            if (s->n_qblocks < 0 || (s->n_qblocks > 0 && (!s->blk_rowptr || !s->blk_colidx)))
                return fail(MAT_ERR_INVALID, "block layout needs row pointers and column ids");
            return MAT_OK;
        case MAT_LONGFORMER:
            if (s->left < 0 || s->right < 0)
                return fail(MAT_ERR_INVALID, "window taps must be >= 0");
            if (s->n_global < 0 || (s->n_global > 0 && !s->global_idx))
                return fail(MAT_ERR_INVALID, "global positions missing");
            return MAT_OK;
    }
    return fail(MAT_ERR_INVALID, "unknown pattern kind %d", s->kind);
}

static DevPattern to_dev(const mat_pattern_spec *s) {
    DevPattern d;
    d.kind = s->kind;
    d.causal = s->causal;
    d.left = s->left;
    d.right = s->right;
    d.dilation = s->kind == MAT_WINDOW ? s->dilation : 1;
    d.block = s->block;
    d.n_qblocks = s->n_qblocks;
    d.rowptr = s->blk_rowptr;
    d.colidx = s->blk_colidx;
    d.n_global = s->kind == MAT_LONGFORMER ? s->n_global : 0;
    d.gidx = s->global_idx;
    d.q_offset = s->q_offset;
    return d;
}

int make_problem(Problem &p, const void *q, const void *k, const void *v, void *o,
                        int64_t B, int64_t S_q, int64_t S_kv, int64_t H, int64_t D, int dtype,
                        const mat_pattern_spec *spec, float scale, void *ws, size_t ws_bytes,
                        void *stream) {
    if (int rc = check_spec(spec)) return rc;
    if (dtype != MAT_F32 && dtype != MAT_BF16 && dtype != MAT_F16)
        return fail(MAT_ERR_INVALID, "unknown dtype %d", dtype);
    if (B <= 0 || S_q <= 0 || S_kv <= 0 || H <= 0 || D <= 0)
        return fail(MAT_ERR_INVALID, "all tensor dimensions must be > 0 (B=%lld S_q=%lld S_kv=%lld H=%lld D=%lld)",
                    (long long)B, (long long)S_q, (long long)S_kv, (long long)H, (long long)D);
    if (S_q + spec->q_offset > S_kv)
        return fail(MAT_ERR_INVALID, "sequence length mismatch: S_q + q_offset = %lld exceeds S_kv = %lld",
                    (long long)(S_q + spec->q_offset), (long long)S_kv);
    if (!q || !k || !v || !o) return fail(MAT_ERR_INVALID, "q, k, v and o must be non-NULL");
    p.q = q; p.k = k; p.v = v; p.o = o;
    p.B = B; p.Sq = S_q; p.Skv = S_kv; p.H = H; p.D = D;
    p.dtype = dtype;
    p.scale = scale > 0.f ? scale : 1.0f / std::sqrt((float)D);
    p.pat = to_dev(spec);
    p.workspace = ws;
    p.workspace_bytes = ws_bytes;
    p.stream = (cudaStream_t)stream;
    return MAT_OK;
}

int run_problem(const Problem &p) {
    if (umma_block_supports(p)) return launch_umma_block(p);
    if (umma_dense_supports(p)) return launch_umma_dense(p);
    if (umma_band_supports(p)) return launch_umma_band(p);
    if (mma_flash_supports(p)) {
        const size_t need = mma_flash_workspace_bytes(p);
        if (need > 0) {
            if (!p.workspace || p.workspace_bytes < need || ((uintptr_t)p.workspace % 256) != 0)
                return fail(MAT_ERR_WORKSPACE,
                            "workspace of %zu bytes (256-byte aligned) required, got %zu",
                            need, p.workspace ? p.workspace_bytes : (size_t)0);
        }
        return launch_mma_flash(p);
    }
    if (mma_window_d_supports(p)) return launch_mma_window_d(p);
    if (mma_window_f32_supports(p)) return launch_mma_window_f32(p);
    if (tiled_f32_supports(p)) return launch_tiled_f32(p);
    return launch_rowwarp(p);
}

// ---- host index sets ----------------------------------------------------

static bool host_is_global(const mat_pattern_spec *s, int64_t p) {
    return std::binary_search(s->global_idx, s->global_idx + s->n_global, p);
}

static void host_rowset(const mat_pattern_spec *s, int64_t S_kv, int64_t i, std::vector<int64_t> &out) {
    out.clear();
    const int64_t p = i + s->q_offset;
    if (s->kind == MAT_BLOCK) {
        const int64_t r = p / s->block;
        if (r >= s->n_qblocks) return;
        for (int32_t e = s->blk_rowptr[r]; e < s->blk_rowptr[r + 1]; ++e) {
            const int64_t j0 = (int64_t)s->blk_colidx[e] * s->block;
            const int64_t j1 = std::min(j0 + s->block, S_kv);
            for (int64_t j = j0; j < j1; ++j)
                if (!s->causal || j <= p) out.push_back(j);
        }
    } else if (s->kind == MAT_LONGFORMER && host_is_global(s, p)) {
        out.resize((size_t)S_kv);
        for (int64_t j = 0; j < S_kv; ++j) out[(size_t)j] = j;
        return;
    } else {
        const int64_t dil = s->kind == MAT_WINDOW ? s->dilation : 1;
        int64_t t_lo = -s->left, t_hi = s->right;
        if (p + t_lo * dil < 0) t_lo = -(p / dil);
        if (p + t_hi * dil >= S_kv) t_hi = (S_kv - 1 - p) / dil;
        for (int64_t t = t_lo; t <= t_hi; ++t) out.push_back(p + t * dil);
        if (s->kind == MAT_LONGFORMER)
            for (int64_t g = 0; g < s->n_global; ++g)
                if (s->global_idx[g] >= 0 && s->global_idx[g] < S_kv) out.push_back(s->global_idx[g]);
    }
    std::sort(out.begin(), out.end());
    out.erase(std::unique(out.begin(), out.end()), out.end());
}

}  // namespace mat

using namespace mat;

extern "C" {

int mat_version(void) { return 100; }

const char *mat_last_error(void) { return g_last_error.c_str(); }

const char *mat_last_kernel(void) { return g_last_kernel; }

int mat_device_status(int *status_out) {
    if (!status_out) return fail(MAT_ERR_INVALID, "status_out is NULL");
    int a = 0, b = 0, c = 0, d = 0;
    if (int rc = flash_status_read_and_clear(&a)) return rc;
    if (int rc = umma_status_read_and_clear(&b)) return rc;
    if (int rc = bwd_status_read_and_clear(&c)) return rc;
    if (int rc = band_status_read_and_clear(&d)) return rc;
    int e = 0;
    if (int rc = tiled_status_read_and_clear(&e)) return rc;
    d |= e;
    *status_out = a | b | c | d;
    return MAT_OK;
}

int mat_sparse_attn_fwd(const void *q, const void *k, const void *v, void *o, int64_t B,
                        int64_t S_q, int64_t S_kv, int64_t H, int64_t D, int dtype,
                        const mat_pattern_spec *spec, float scale, void *workspace,
                        size_t workspace_bytes, void *stream) {
    Problem p;
    if (int rc = make_problem(p, q, k, v, o, B, S_q, S_kv, H, D, dtype, spec, scale, workspace,
                              workspace_bytes, stream))
        return rc;
    return run_problem(p);
}

int mat_sparse_attn_fwd_strided(const void *q, const void *k, const void *v, void *o, int64_t B,
                                int64_t S_q, int64_t S_kv, int64_t H, int64_t D, int dtype,
                                const mat_pattern_spec *spec, float scale, int64_t q_token_stride,
                                int64_t k_token_stride, int64_t v_token_stride, int64_t o_token_stride,
                                void *stream) {
    Problem p;
    if (int rc = make_problem(p, q, k, v, o, B, S_q, S_kv, H, D, dtype, spec, scale, nullptr, 0, stream))
        return rc;
    const int64_t row = H * D;
    const int64_t ts[4] = {q_token_stride, k_token_stride, v_token_stride, o_token_stride};
    bool strided = false;
    for (int64_t t : ts) {
        if (t != 0 && t < row) return fail(MAT_ERR_INVALID, "a token stride of %lld elements is shorter than a token (%lld)", (long long)t, (long long)row);
        if (t % 8) return fail(MAT_ERR_INVALID, "token strides must be multiples of 8 elements (16 bytes)");
        strided = strided || (t != 0 && t != row);
    }
    if (!strided) return run_problem(p);
    p.q_ts = q_token_stride; p.k_ts = k_token_stride; p.v_ts = v_token_stride; p.o_ts = o_token_stride;
    // strided tensors are read by the band kernel only (whatever the problem's size)
    if (spec->kind != MAT_WINDOW || (dtype != MAT_BF16 && dtype != MAT_F16) || D != 64 || !umma_band_fits(p))
        return fail(MAT_ERR_UNSUPPORTED,
                    "token-strided tensors are supported for window patterns of at most 128 taps on 16-bit inputs "
                    "with head width 64 (sequence lengths divisible by the dilation): pass contiguous tensors");
    return launch_umma_band(p);
}

size_t mat_sparse_attn_workspace_bytes(int64_t B, int64_t S_q, int64_t S_kv, int64_t H, int64_t D,
                                       int dtype, const mat_pattern_spec *spec) {
    Problem p;
    alignas(256) static char dummy[256];  // stands in for the tensors: kernel selection looks at alignment
    if (make_problem(p, dummy, dummy, dummy, dummy, B, S_q, S_kv, H, D, dtype, spec,
                     0.f, nullptr, 0, nullptr))
        return 0;
    if (mma_flash_supports(p)) return mma_flash_workspace_bytes(p);
    return mma_window_d_scratch_bytes(p);
}

int mat_sparse_attn_fwd_window(const void *q, const void *k, const void *v, void *o, int64_t B,
                               int64_t S, int64_t H, int64_t D, int dtype, int64_t window_size,
                               void *stream) {
    if (window_size < 0) return fail(MAT_ERR_INVALID, "window_size must be >= 0");
    mat_pattern_spec s;
    memset(&s, 0, sizeof s);
    s.kind = MAT_WINDOW;
    s.left = s.right = std::min<int64_t>(window_size, S);  // beyond S every key is already in
    s.dilation = 1;
    return mat_sparse_attn_fwd(q, k, v, o, B, S, S, H, D, dtype, &s, 0.f, nullptr, 0, stream);
}

int mat_sparse_attn_fwd_sharded(const void *q, const void *k, const void *v, void *o,
                                const void *k_prev, const void *v_prev, int64_t S_prev,
                                const void *k_next, const void *v_next, int64_t S_next, int64_t B,
                                int64_t S, int64_t H, int64_t D, int dtype,
                                const mat_pattern_spec *spec, float scale, void *stream) {
    Problem p;
    if (int rc = make_problem(p, q, k, v, o, B, S, S, H, D, dtype, spec, scale, nullptr, 0, stream))
        return rc;
    if (spec->kind != MAT_WINDOW)
        return fail(MAT_ERR_UNSUPPORTED, "sequence shards apply to window patterns only");
    if (spec->q_offset != 0) return fail(MAT_ERR_INVALID, "q_offset must be 0: the shard holds no halo rows");
    if ((k_prev == nullptr) != (v_prev == nullptr) || (k_next == nullptr) != (v_next == nullptr))
        return fail(MAT_ERR_INVALID, "a neighbour needs both its K and its V");
    const int64_t dil = spec->dilation, unit = 16 * dil;
    if (!mma_flash_supports(p))
        return fail(MAT_ERR_UNSUPPORTED,
                    "in-place neighbour reads need 16-bit inputs, head width 64 and S divisible by the dilation");
    if (k_prev) {
        if (S_prev <= 0 || S_prev % unit) return fail(MAT_ERR_INVALID, "S_prev must be a positive multiple of 16*dilation");
        if (spec->left * dil > S_prev) return fail(MAT_ERR_UNSUPPORTED, "window reaches past the previous shard");
        if (((uintptr_t)k_prev | (uintptr_t)v_prev) % 16) return fail(MAT_ERR_INVALID, "neighbour tensors must be 16-byte aligned");
    } else {
        S_prev = 0;
    }
    if (k_next) {
        if (S_next <= 0 || S_next % dil || S % unit)
            return fail(MAT_ERR_INVALID, "with a next shard, S must be a multiple of 16*dilation and S_next of the dilation");
        if (spec->right * dil > S_next) return fail(MAT_ERR_UNSUPPORTED, "window reaches past the next shard");
        if (((uintptr_t)k_next | (uintptr_t)v_next) % 16) return fail(MAT_ERR_INVALID, "neighbour tensors must be 16-byte aligned");
    } else {
        S_next = 0;
    }
    p.k_prev = k_prev; p.v_prev = v_prev; p.S_prev = S_prev;
    p.k_next = k_next; p.v_next = v_next; p.S_next = S_next;
    if (umma_band_supports(p)) return launch_umma_band(p);
    return launch_mma_flash(p);
}

int mat_enable_peer_access(int device, int peer_device) {
    if (device == peer_device) return MAT_OK;
    int can = 0;
    cudaError_t e = cudaDeviceCanAccessPeer(&can, device, peer_device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceCanAccessPeer");
    if (!can) return fail(MAT_ERR_UNSUPPORTED, "device %d cannot map memory of device %d", device, peer_device);
    int prev = 0;
    if ((e = cudaGetDevice(&prev)) != cudaSuccess || (e = cudaSetDevice(device)) != cudaSuccess)
        return cuda_fail(e, "selecting the device");
    e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();  // clear the sticky-free error state
        e = cudaSuccess;
    }
    cudaSetDevice(prev);
    return e == cudaSuccess ? MAT_OK : cuda_fail(e, "cudaDeviceEnablePeerAccess");
}

int mat_pattern_rowset(const mat_pattern_spec *spec, int64_t S_kv, int64_t i, int64_t *out,
                       int64_t cap, int64_t *n_out) {
    if (int rc = check_spec(spec)) return rc;
    if (S_kv <= 0 || i < 0 || !n_out) return fail(MAT_ERR_INVALID, "bad row query");
    std::vector<int64_t> row;
    host_rowset(spec, S_kv, i, row);
    *n_out = (int64_t)row.size();
    if ((int64_t)row.size() > cap || (!out && !row.empty()))
        return fail(MAT_ERR_INVALID, "row holds %zu keys, buffer holds %lld", row.size(), (long long)cap);
    if (!row.empty()) memcpy(out, row.data(), row.size() * sizeof(int64_t));
    return MAT_OK;
}

int mat_pattern_nnz(const mat_pattern_spec *spec, int64_t S_q, int64_t S_kv, int64_t *nnz_out) {
    if (int rc = check_spec(spec)) return rc;
    if (S_q <= 0 || S_kv <= 0 || !nnz_out) return fail(MAT_ERR_INVALID, "bad nnz query");
    std::vector<int64_t> row;
    int64_t total = 0;
    for (int64_t i = 0; i < S_q; ++i) {
        host_rowset(spec, S_kv, i, row);
        total += (int64_t)row.size();
    }
    *nnz_out = total;
    return MAT_OK;
}

}  // extern "C"
