// Forward pass on host buffers: the counterpart of handing CPU tensors to the
// reference's CPU engine (src/layers/ma_core_bridge.py:102-112 marshals torch ->
// numpy -> ma_core::Tensor -> compute_sparse_attention -> numpy -> torch).
//
// The sequence is cut into chunks of query rows.  Four internal streams (two for the
// input copies, which alternate between them) run a pipeline: copy chunk c of q, k, v to the device; run the forward for the
// queries of chunk c as soon as the last key chunk they can see has landed
// (window patterns need at most the next chunk, causal block layouts only their
// own, everything else the whole sequence); copy chunk c of the output back.
// PCIe is full duplex, so the output copies hide under the input copies.
#include <cstdlib>
#include <mutex>
#include <vector>

#include "mat_common.cuh"

namespace mat {
namespace {

struct Pipe {
    cudaStream_t h2d = nullptr, h2d_b = nullptr, comp = nullptr, d2h = nullptr;
    std::vector<cudaEvent_t> ev_in, ev_out;
};

// one pipeline (and one lock) per device: calls for different GPUs run side by side, calls for the
// same GPU take turns, since they share its three streams
std::mutex g_mus[64];
Pipe g_pipes[64];

int get_pipe(int device, size_t n_events, Pipe **out) {
    if (device < 0 || device >= 64) return fail(MAT_ERR_INVALID, "device ordinal %d out of range", device);
    Pipe &p = g_pipes[device];
    cudaError_t e;
    if (!p.h2d) {
        if ((e = cudaStreamCreateWithFlags(&p.h2d, cudaStreamNonBlocking)) != cudaSuccess ||
            (e = cudaStreamCreateWithFlags(&p.h2d_b, cudaStreamNonBlocking)) != cudaSuccess ||
            (e = cudaStreamCreateWithFlags(&p.comp, cudaStreamNonBlocking)) != cudaSuccess ||
            (e = cudaStreamCreateWithFlags(&p.d2h, cudaStreamNonBlocking)) != cudaSuccess)
            return cuda_fail(e, "creating the pipeline streams");
    }
    while (p.ev_in.size() < n_events) {
        cudaEvent_t a, b;
        if ((e = cudaEventCreateWithFlags(&a, cudaEventDisableTiming)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&b, cudaEventDisableTiming)) != cudaSuccess)
            return cuda_fail(e, "creating the pipeline events");
        p.ev_in.push_back(a);
        p.ev_out.push_back(b);
    }
    *out = &p;
    return MAT_OK;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

int64_t chunk_rows(int64_t S, int64_t H, int64_t D, int dtype, const mat_pattern_spec *spec) {
    const int64_t row_bytes = H * D * (int64_t)dtype_size(dtype);
    const int64_t dil = spec->kind == MAT_WINDOW ? spec->dilation : 1;
    int64_t unit = 64 * dil;  // keeps every chunk eligible for the tiled kernels
    if (spec->kind == MAT_BLOCK && spec->block > 0) {
        // a chunk boundary must not split a layout row
        int64_t a = unit, b = spec->block;
        while (b) { int64_t t = a % b; a = b; b = t; }
        unit = unit / a * spec->block;
    }
    // An eighth of the sequence per chunk, between 2 and 8 MiB per tensor.  Every copy costs a fixed few
    // microseconds of set-up on top of its bytes (measured at 64 MiB per tensor: 5.52 ms per forward with 1 MiB
    // chunks, 4.91 with 2, 4.40 with 4, 4.23 with 8, 4.22 with 16), while the first chunk's copy and the last
    // chunk's forward and output copy are not overlapped with anything, which is what larger chunks cost.
    // MAT_HOST_CHUNK_KB overrides the size (a measurement aid).
    int64_t chunk_bytes = S * row_bytes / 8;
    chunk_bytes = chunk_bytes > (8 << 20) ? (8 << 20) : (chunk_bytes < (2 << 20) ? (2 << 20) : chunk_bytes);
    if (const char *e = std::getenv("MAT_HOST_CHUNK_KB")) chunk_bytes = std::max<int64_t>(64, atoi(e)) << 10;
    const int64_t target = chunk_bytes / row_bytes;
    int64_t c = target / unit * unit;
    if (c < unit) c = unit;
    return c >= S ? S : c;
}

}  // namespace
}  // namespace mat

using namespace mat;

extern "C" {

size_t mat_sparse_attn_host_staging_bytes(int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                                          const mat_pattern_spec *spec) {
    if (B <= 0 || S <= 0 || H <= 0 || D <= 0 || !spec) return 0;
    const size_t t = align256((size_t)B * S * H * D * dtype_size(dtype));
    const int64_t C = chunk_rows(S, H, D, dtype, spec);
    mat_pattern_spec s = *spec;
    s.q_offset = 0;
    // the largest workspace any chunk launch can ask for
    const size_t ws = mat_sparse_attn_workspace_bytes(1, C, S, H, D, dtype, &s);
    return 4 * t + align256(ws);
}

int mat_sparse_attn_fwd_host(const void *q_host, const void *k_host, const void *v_host,
                             void *o_host, int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                             const mat_pattern_spec *spec, float scale, void *staging,
                             size_t staging_bytes, int device) {
    if (!spec) return fail(MAT_ERR_INVALID, "pattern description is NULL");
    if (spec->q_offset != 0) return fail(MAT_ERR_INVALID, "q_offset must be 0 for the host entry point");
    if (!q_host || !k_host || !v_host || !o_host) return fail(MAT_ERR_INVALID, "host buffers must be non-NULL");
    if (B <= 0 || S <= 0 || H <= 0 || D <= 0)
        return fail(MAT_ERR_INVALID, "all tensor dimensions must be > 0");
    if (dtype != MAT_F32 && dtype != MAT_BF16 && dtype != MAT_F16)
        return fail(MAT_ERR_INVALID, "unknown dtype %d", dtype);
    const size_t need = mat_sparse_attn_host_staging_bytes(B, S, H, D, dtype, spec);
    if (!staging || staging_bytes < need || ((uintptr_t)staging % 256) != 0)
        return fail(MAT_ERR_WORKSPACE, "device staging of %zu bytes (256-byte aligned) required, got %zu",
                    need, staging ? staging_bytes : (size_t)0);

    if (device < 0 || device >= 64) return fail(MAT_ERR_INVALID, "device ordinal %d out of range", device);
    std::lock_guard<std::mutex> lock(g_mus[device]);
    int prev = 0;
    cudaError_t e = cudaGetDevice(&prev);
    if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
    if (e != cudaSuccess) return cuda_fail(e, "selecting the device");

    const size_t row_bytes = (size_t)H * D * dtype_size(dtype);
    const size_t t = align256((size_t)B * S * row_bytes);
    uint8_t *dq = (uint8_t *)staging, *dk = dq + t, *dv = dk + t, *dout = dv + t;
    void *ws = dout + t;
    const size_t ws_bytes = staging_bytes - 4 * t;

    const int64_t C = chunk_rows(S, H, D, dtype, spec);
    const int64_t nch = (S + C - 1) / C;
    Pipe *pipe = nullptr;
    int rc = get_pipe(device, (size_t)(B * nch), &pipe);

    // 1. inputs, chunk by chunk, each followed by an event
    // (the chunks alternate between two copy streams: the next chunk's copies are queued on the other
    // engine while this chunk's drain, 4.23 -> 4.15 ms per forward at 64 MiB per tensor)
    const bool two = true;
    for (int64_t b = 0; rc == MAT_OK && b < B; ++b)
        for (int64_t c = 0; c < nch; ++c) {
            const size_t off = ((size_t)b * S + (size_t)c * C) * row_bytes;
            const size_t n = (size_t)std::min<int64_t>(C, S - c * C) * row_bytes;
            cudaStream_t hs = two && ((b * nch + c) & 1) ? pipe->h2d_b : pipe->h2d;
            if ((e = cudaMemcpyAsync(dq + off, (const uint8_t *)q_host + off, n, cudaMemcpyHostToDevice, hs)) != cudaSuccess ||
                (e = cudaMemcpyAsync(dk + off, (const uint8_t *)k_host + off, n, cudaMemcpyHostToDevice, hs)) != cudaSuccess ||
                (e = cudaMemcpyAsync(dv + off, (const uint8_t *)v_host + off, n, cudaMemcpyHostToDevice, hs)) != cudaSuccess ||
                (e = cudaEventRecord(pipe->ev_in[(size_t)(b * nch + c)], hs)) != cudaSuccess) {
                rc = cuda_fail(e, "host-to-device copy");
                break;
            }
        }

    // 2. forward per chunk, 3. output copy per chunk
    const int64_t dil = spec->kind == MAT_WINDOW ? spec->dilation : 1;
    for (int64_t b = 0; rc == MAT_OK && b < B; ++b)
        for (int64_t c = 0; c < nch; ++c) {
            const int64_t c0 = c * C, c1 = std::min(S, c0 + C);
            int64_t last = nch - 1;  // last key chunk the queries of this chunk can see
            if (spec->kind == MAT_WINDOW) {
                const int64_t reach = spec->right > S ? S : spec->right * dil;
                last = std::min(nch - 1, (c1 - 1 + reach) / C);
            } else if (spec->kind == MAT_BLOCK && spec->causal) {
                last = c;
            }
            if (two && b * nch + last >= 1) cudaStreamWaitEvent(pipe->comp, pipe->ev_in[(size_t)(b * nch + last - 1)], 0);
            if ((e = cudaStreamWaitEvent(pipe->comp, pipe->ev_in[(size_t)(b * nch + last)], 0)) != cudaSuccess) {
                rc = cuda_fail(e, "cudaStreamWaitEvent");
                break;
            }
            mat_pattern_spec s = *spec;
            s.q_offset = c0;
            const size_t qoff = ((size_t)b * S + (size_t)c0) * row_bytes;
            const size_t koff = (size_t)b * S * row_bytes;
            // The launch sees only the key rows whose copies it waited for.  The tiled kernels stage
            // whole groups of keys, and a staged row that lies past the last landed chunk would be
            // multiplied by a zero weight; whatever the staging memory held there (possibly a NaN
            // pattern) must not reach that product, so those rows are outside the tensor and read as zeros.
            const int64_t skv = std::min(S, (last + 1) * C);
            Problem p;
            rc = make_problem(p, dq + qoff, dk + koff, dv + koff, dout + qoff, 1, c1 - c0, skv, H, D,
                              dtype, &s, scale, ws, ws_bytes, pipe->comp);
            if (rc == MAT_OK) rc = run_problem(p);
            if (rc != MAT_OK) break;
            const size_t slot = (size_t)(b * nch + c);
            if ((e = cudaEventRecord(pipe->ev_out[slot], pipe->comp)) != cudaSuccess ||
                (e = cudaStreamWaitEvent(pipe->d2h, pipe->ev_out[slot], 0)) != cudaSuccess ||
                (e = cudaMemcpyAsync((uint8_t *)o_host + qoff, dout + qoff, (size_t)(c1 - c0) * row_bytes,
                                     cudaMemcpyDeviceToHost, pipe->d2h)) != cudaSuccess) {
                rc = cuda_fail(e, "device-to-host copy");
                break;
            }
        }

    // drain every stream, also after an error, so the staging buffer is quiescent on return
    if (pipe) {
        cudaStreamSynchronize(pipe->h2d_b);
        cudaError_t e1 = cudaStreamSynchronize(pipe->h2d);
        cudaError_t e2 = cudaStreamSynchronize(pipe->comp);
        cudaError_t e3 = cudaStreamSynchronize(pipe->d2h);
        if (rc == MAT_OK && (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess))
            rc = cuda_fail(e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3), "draining the pipeline");
    }
    if (prev != device) cudaSetDevice(prev);
    return rc;
}

}  // extern "C"
