/*
 * C ABI of libmat_sparse_attn: the sparse-attention forward of ma-transformer,
 * written for NVIDIA B200 (sm_100a).  Plain pointers and sizes only; no torch
 * or pybind types.  Every tensor is row-major [B, S, H, D] with D contiguous,
 * the layout of the reference's tensors (src/csrc/tensor.cpp:104-110,
 * src/cuda/sparse_attention_kernel.cu:28-32).
 *
 * All entry points return MAT_OK (0) or a MAT_ERR_* code; mat_last_error()
 * gives the text of the calling thread's last failure.  Device entry points
 * enqueue work on the given stream and return without synchronising, as the
 * reference's extension does (sparse_attention_kernel.cu:450-456).
 */
#ifndef MAT_SPARSE_ATTN_H
#define MAT_SPARSE_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MAT_OK 0
#define MAT_ERR_INVALID 1      /* malformed argument (shape, pointer, pattern) */
#define MAT_ERR_UNSUPPORTED 2  /* valid request outside what the kernels cover */
#define MAT_ERR_CUDA 3         /* a CUDA call failed; text holds its message */
#define MAT_ERR_WORKSPACE 4    /* workspace missing, misaligned or too small */

/* element types of q, k, v, o (the reference computes in fp32 only,
 * src/csrc/attention_types.hpp:10; bf16/fp16 accumulate in fp32) */
#define MAT_F32 0
#define MAT_BF16 1
#define MAT_F16 2

/* pattern kinds, after AttentionPattern (src/csrc/attention_types.hpp:26-38) */
#define MAT_WINDOW 0      /* SLIDING_WINDOW, causal or two-sided, optionally dilated */
#define MAT_BLOCK 1       /* BLOCK_SPARSE over an explicit block-CSR layout */
#define MAT_LONGFORMER 2  /* LONGFORMER: window plus global tokens */

/*
 * Key set of one query row.  With p = i + q_offset the position of query row
 * i in key coordinates and S_kv the number of key rows:
 *   MAT_WINDOW      { p + t*dilation : -left <= t <= right } within [0, S_kv)
 *                   (src/csrc/sparse_attention.cpp:190-197 with left = right =
 *                   window_size; dilation per doc/sparse_attention_whitepaper.md:102-105)
 *   MAT_BLOCK       all keys of the key blocks listed in row floor(p/block) of
 *                   the block-CSR layout, minus keys j > p when causal != 0
 *                   (src/csrc/sparse_attention.cpp:209-227 is the layout
 *                   |row - col| <= 1, causal = 0).  Column ids within a row
 *                   must be distinct and ascending.
 *   MAT_LONGFORMER  [p-left, p+right] united with the global positions; a query
 *                   at a global position takes every key
 *                   (src/csrc/sparse_attention.cpp:241-256, de-duplicated).
 *                   global_idx must be sorted ascending without repeats, every
 *                   entry in [0, S_kv): the list lives on the device, so the
 *                   library cannot refuse a bad entry; the kernels never touch
 *                   memory through one (such a position contributes a zero key
 *                   and owns no output row), the result is then unspecified.
 * A row whose set is empty produces zeros.
 * blk_rowptr, blk_colidx and global_idx are DEVICE pointers for
 * mat_sparse_attn_fwd and HOST pointers for mat_pattern_rowset / mat_pattern_nnz.
 */
typedef struct mat_pattern_spec {
    int32_t kind;
    int32_t causal;
    int64_t left;
    int64_t right;
    int64_t dilation;
    int64_t block;
    int64_t n_qblocks;
    const int32_t *blk_rowptr; /* [n_qblocks + 1] */
    const int32_t *blk_colidx;
    int64_t n_global;
    const int64_t *global_idx;
    int64_t q_offset;
} mat_pattern_spec;

/* Library version, major*10000 + minor*100 + patch. */
int mat_version(void);

/* Text of the calling thread's most recent error ("" when none). */
const char *mat_last_error(void);

/*
 * Forward pass on device buffers.  Replaces sparse_forward_cuda and its kernel
 * (src/cuda/sparse_attention_kernel.cu:423-458, 211-263) and, for the general
 * patterns, the intent of SparseAttention::forward
 * (src/csrc/sparse_attention.cpp:11-41).
 *   q, o: [B, S_q, H, D]; k, v: [B, S_kv, H, D]; S_kv >= S_q + q_offset lets a
 *   sequence shard carry halo rows in front of (and behind) its own keys.
 *   scale <= 0 selects 1/sqrt(D) (sparse_attention_kernel.cu:442).
 *   workspace: device scratch of at least mat_sparse_attn_workspace_bytes()
 *   bytes, 256-byte aligned; may be NULL when that size is 0.
 */
int mat_sparse_attn_fwd(const void *q, const void *k, const void *v, void *o,
                        int64_t B, int64_t S_q, int64_t S_kv, int64_t H, int64_t D,
                        int dtype, const mat_pattern_spec *spec, float scale,
                        void *workspace, size_t workspace_bytes, void *stream);

/*
 * Forward pass on device tensors whose tokens are not packed: q, k, v and o keep D contiguous and the H heads
 * of a token contiguous, but consecutive tokens lie *_token_stride ELEMENTS apart (0 = packed, H*D), and
 * batch item b starts b * S * stride elements after item 0.  This is how q, k and v sit inside the output
 * [B, S, 3, H, D] of one fused projection: the caller passes three views of it (stride 3*H*D) and no copy is
 * made.  The reference's integration example projects q, k and v separately and reshapes each
 * (examples/pytorch_integration_example.py:65-107), and its extension refuses anything but packed tensors
 * (src/cuda/sparse_attention_kernel.cu:430); this entry point is the additive relaxation.
 * MAT_WINDOW patterns of at most 128 taps between their two sides, 16-bit dtypes, D = 64, strides multiples
 * of 8 elements; other requests with real strides get MAT_ERR_UNSUPPORTED.  Packed strides behave exactly as
 * mat_sparse_attn_fwd (without a workspace).
 */
int mat_sparse_attn_fwd_strided(const void *q, const void *k, const void *v, void *o,
                                int64_t B, int64_t S_q, int64_t S_kv, int64_t H, int64_t D,
                                int dtype, const mat_pattern_spec *spec, float scale,
                                int64_t q_token_stride, int64_t k_token_stride,
                                int64_t v_token_stride, int64_t o_token_stride, void *stream);

/* Scratch bytes mat_sparse_attn_fwd needs for this problem (0 for most: the Longformer pattern needs its partial
 * results, 16-bit heads of more than 128 columns or of a width that is not a multiple of 16 need an fp32 copy of the
 * output's shape when the window has more than 128 taps between its sides). */
size_t mat_sparse_attn_workspace_bytes(int64_t B, int64_t S_q, int64_t S_kv, int64_t H,
                                       int64_t D, int dtype, const mat_pattern_spec *spec);

/*
 * The reference extension's call, unchanged in meaning: keys [i-w, i+w],
 * w >= 0 (0 = the query itself), w beyond S clamps
 * (sparse_attention_kernel.cu:423-458: forward(query, key, value, window_size)).
 */
int mat_sparse_attn_fwd_window(const void *q, const void *k, const void *v, void *o,
                               int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                               int64_t window_size, void *stream);

/*
 * Forward pass of one SEQUENCE SHARD whose window reaches into its neighbours:
 * one process per GPU owns a contiguous chunk [B, S, H, D] of a longer sequence,
 * and the query tiles at the chunk's edges read the halo rows they need straight
 * from the neighbouring GPUs' K/V tensors (peer-mapped device pointers, fetched
 * by ordinary tiled TMA loads inside the same kernel): no separate exchange step,
 * no halo copy.  k_prev/v_prev: the previous shard's [B, S_prev, H, D] tensors or
 * NULL on the first shard; k_next/v_next likewise for two-sided windows.
 * MAT_WINDOW patterns with 16-bit inputs and D = 64; S_prev (and S when a next
 * shard is given) must be multiples of 16*dilation and cover the window's reach.
 * The caller guarantees that the neighbours' tensors are complete before the
 * launch and stay unchanged until it finishes.  The reference has no distributed
 * path (no counterpart); the single-GPU call it extends is sparse_forward_cuda
 * (src/cuda/sparse_attention_kernel.cu:423-458).
 */
int mat_sparse_attn_fwd_sharded(const void *q, const void *k, const void *v, void *o,
                                const void *k_prev, const void *v_prev, int64_t S_prev,
                                const void *k_next, const void *v_next, int64_t S_next,
                                int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                                const mat_pattern_spec *spec, float scale, void *stream);

/*
 * Backward of window attention: dQ, dK, dV from Q, K, V and the output gradient,
 * all [B, S, H, D].  Replaces sparse_backward_cuda / dense_backward_cuda and their
 * kernels (src/cuda/sparse_attention_kernel.cu:460-497, 384-421, 265-346, 104-208):
 * the reference's window is left = right = window_size, its dense call is the
 * window that covers S (right = 0 when causal).  MAT_WINDOW (and MAT_LONGFORMER, see
 * mat_sparse_attn_bwd_general) patterns, q_offset = 0.
 * Deterministic (no atomics).  workspace: mat_sparse_attn_bwd_workspace_bytes()
 * bytes of device scratch, 256-byte aligned (per-row log-sum-exp and delta).
 * 16-bit inputs with D = 64 and S a multiple of the dilation run on tensor-core
 * kernels (probabilities rounded to the input type for the second products; the
 * band of a window with at most 128 taps between its two sides stays in shared
 * memory, wider windows and dense stream it).  So do 16-bit inputs with any other
 * D that is a multiple of 8 up to 512, and fp32 inputs with a D that is a multiple
 * of 4 up to 512 (every product as three TF32 products of error-compensated
 * halves: fp32 accuracy).  Everything else (other head widths, tensors off a
 * 16-byte boundary, lengths the dilation does not divide) runs on warp-level
 * kernels with fp32 math throughout.
 */
int mat_sparse_attn_bwd(const void *q, const void *k, const void *v, const void *dout,
                        void *dq, void *dk, void *dv, int64_t B, int64_t S, int64_t H, int64_t D,
                        int dtype, const mat_pattern_spec *spec, float scale,
                        void *workspace, size_t workspace_bytes, void *stream);
size_t mat_sparse_attn_bwd_workspace_bytes(int64_t B, int64_t S, int64_t H);

/*
 * The same backward for every pattern kind.  The reference has no backward for
 * its generic masked patterns (src/csrc/attention_interface.hpp:14-52: backward
 * throws); this one exists so that block layouts and the Longformer pattern can
 * be trained through the same module.  MAT_WINDOW: as mat_sparse_attn_bwd (which
 * forwards here; t_rowptr / t_colidx unused).  MAT_LONGFORMER: dilation 1,
 * global_idx sorted and unique (device pointer); also accepted by
 * mat_sparse_attn_bwd.  MAT_BLOCK: blk_rowptr / blk_colidx as for the forward,
 * plus the TRANSPOSED layout t_rowptr [n_qblocks + 1] / t_colidx (device
 * pointers): for every key block the ascending list of query blocks whose
 * layout row holds it; n_qblocks * block must cover S.  16-bit block layouts
 * with D = 64 and block a multiple of 64 run on the streamed tensor-core kernels
 * (a tile walks the chunks of its layout row's blocks), and so does the
 * Longformer pattern with 1 to 64 global positions (window band plus a chunk of
 * gathered global rows per tile, then the gathered global rows and keys against
 * the whole sequence); other shapes on the warp-level kernels (fp32 math, any
 * D <= 512).  Deterministic.  workspace: mat_sparse_attn_bwd_general_workspace_bytes()
 * bytes (what mat_sparse_attn_bwd wants, plus the gathered rows of a Longformer
 * call, plus fp32 copies of the three outputs for a 16-bit window of more than 144
 * taps on a head of more than 128 columns or of a width off the multiples of 16;
 * a window call that brings only mat_sparse_attn_bwd_workspace_bytes() is served
 * too, that case then on the warp-level kernels), 256-byte aligned.
 */
size_t mat_sparse_attn_bwd_general_workspace_bytes(int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                                                   const mat_pattern_spec *spec);
int mat_sparse_attn_bwd_general(const void *q, const void *k, const void *v, const void *dout,
                                void *dq, void *dk, void *dv, int64_t B, int64_t S, int64_t H, int64_t D,
                                int dtype, const mat_pattern_spec *spec, const int32_t *t_rowptr,
                                const int32_t *t_colidx, float scale, void *workspace,
                                size_t workspace_bytes, void *stream);

/*
 * Longformer forward that allocates nothing and takes no workspace.  It has no
 * counterpart in the reference.  It is for hosts that may not obtain device
 * memory while they run: a server that gave all of HBM to its own arena at
 * start-up has nothing left to lend as a workspace, and a latency-critical loop
 * cannot afford the device-wide synchronisation an allocation implies.  The
 * per-split partial results of the global-row pass (the only scratch the forward
 * uses) go to an array built into the library, 4 MiB per GPU, which a GPU holds
 * from the moment the library's device code is loaded onto it (with CUDA's
 * default lazy loading: at the library's first use on that GPU) until the
 * process ends.
 *   - MAT_LONGFORMER patterns, 16-bit dtypes, D = 64, whole sequences
 *     (q, k, v, o all [B, S, H, D]; q_offset = 0).  The caller still owns inputs
 *     and output.  Same results as mat_sparse_attn_fwd up to summation order.
 *   - Limit: B * H * (global positions rounded up to 64) * 264 bytes must fit in
 *     4 MiB; larger problems get MAT_ERR_UNSUPPORTED and should use
 *     mat_sparse_attn_fwd with a caller workspace.  Within the limit the key axis
 *     is cut into as many splits as fit, so very large B*H runs with less
 *     parallelism in the global-row pass than the workspace version.
 *   - The first call on each device looks up the array's device address (once)
 *     and may be the moment the driver loads the library's device code: treat
 *     it as a warm-up and make it outside any stream capture.  The library
 *     itself calls no cudaMalloc, cudaFree or other allocating routine, on the
 *     first call or later.
 *   - Every refusal happens before anything is launched: a call that returns
 *     an error has not touched o.
 *   - global_idx entries must lie in [0, S) (as for mat_sparse_attn_fwd).
 *   - All calls on a device share the one array and nothing in it needs
 *     clearing (every slot that is read is written first by the same call), but
 *     two calls that overlap on the GPU, e.g. on different streams, race on it:
 *     keep them on one stream or order them with events.
 */
int mat_sparse_attn_fwd_longformer_noalloc(const void *q, const void *k, const void *v, void *o,
                                           int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                                           const mat_pattern_spec *spec, float scale, void *stream);

/*
 * Longformer over a sequence spread across GPUs (one shard [B, S, H, 64] per process): three
 * building blocks around two small collectives the caller runs (all-gather of the Q/K/V rows at
 * the global positions, all-gather of the partials).  No counterpart in the reference, whose
 * LongformerAttention (src/csrc/sparse_attention.cpp:234-259) is single-process.
 *   mat_longformer_shard_fwd       pass 1 of a shard: every local row over its window (halo rows
 *                                  read in place from the neighbour shards, as in
 *                                  mat_sparse_attn_fwd_sharded) plus the keys at ALL global
 *                                  positions (kg, vg: [B, n_global, H, 64]).  g_pos[e] = position of
 *                                  global token e relative to this shard's first row (device
 *                                  array, ascending; negative or >= S for other shards' tokens).
 *   mat_global_rows_partial        (max, sum, unnormalised output) of the global queries
 *                                  qg [B, n_global, H, 64] against this shard's keys, per key
 *                                  split; layout and size from mat_global_rows_partial_layout.
 *   mat_global_rows_merge          merges n_parts such buffers (one per shard,
 *                                  part_stride_floats apart) for the global tokens
 *                                  [e_first, e_first + n_rows) this shard owns and writes their
 *                                  rows of o.
 * 16-bit dtypes, D = 64.
 */
int mat_longformer_shard_fwd(const void *q, const void *k, const void *v, void *o,
                             const void *k_prev, const void *v_prev, int64_t S_prev,
                             const void *k_next, const void *v_next, int64_t S_next,
                             const void *kg, const void *vg, const int64_t *g_pos, int64_t n_global,
                             int64_t B, int64_t S, int64_t H, int64_t D, int dtype,
                             int64_t left, int64_t right, float scale, void *stream);
size_t mat_global_rows_partial_layout(int64_t B, int64_t n_global, int64_t S_kv, int64_t H,
                                      int32_t *n_splits_out, int32_t *ng_pad_out);
int mat_global_rows_partial(const void *qg, const void *k, const void *v, void *partial,
                            int64_t B, int64_t n_global, int64_t S_kv, int64_t H, int64_t D,
                            int dtype, float scale, void *stream);
int mat_global_rows_merge(const void *partials, int64_t n_parts, int64_t part_stride_floats, void *o,
                          const int64_t *g_pos, int64_t e_first, int64_t n_rows, int64_t B, int64_t S,
                          int64_t H, int32_t n_splits, int32_t ng_pad, int dtype, float scale,
                          void *stream);

/*
 * Lets kernels running on `device` read memory that lives on `peer_device`
 * (cudaDeviceEnablePeerAccess; already-enabled is not an error).  Call once per
 * neighbour before mat_sparse_attn_fwd_sharded.  No counterpart in the reference.
 */
int mat_enable_peer_access(int device, int peer_device);

/*
 * Sharing a shard's K/V with the process that drives the neighbouring GPU (one
 * process per GPU).  No counterpart in the reference (it is single-process).
 *   mat_ipc_export  fills a MAT_IPC_HANDLE_BYTES handle naming the device
 *                   allocation that contains dev_ptr, and dev_ptr's byte offset
 *                   inside it; send both to the neighbour by any host channel.
 *   mat_ipc_open    in the neighbour's process: maps that allocation for kernels
 *                   running on `device` (peer access over NVLink) and returns its
 *                   base; the tensor is at base + offset.  Open each handle once
 *                   per process and reuse the base.
 *   mat_ipc_close   unmaps it.
 */
#define MAT_IPC_HANDLE_BYTES 64
int mat_ipc_export(const void *dev_ptr, void *handle_out, int64_t *offset_out);
int mat_ipc_open(const void *handle, int device, void **base_out);
int mat_ipc_close(void *base, int device);

/*
 * Forward pass on HOST buffers: the counterpart of the CPU engine's call
 * ma_core.compute_sparse_attention and the marshalling around it
 * (src/csrc/ma_core.cpp:160-246, src/layers/ma_core_bridge.py:102-112,157-181).
 * Copies q, k, v to the device in sequence chunks, runs the forward and copies
 * o back, overlapping the three on internal streams; returns after o is
 * complete in host memory.  staging is caller-owned DEVICE scratch of at least
 * mat_sparse_attn_host_staging_bytes() bytes (256-byte aligned).  Pinned host
 * buffers make the copies asynchronous; pageable ones work but serialise.
 * spec pointers are device pointers, as for mat_sparse_attn_fwd.
 */
int mat_sparse_attn_fwd_host(const void *q_host, const void *k_host, const void *v_host,
                             void *o_host, int64_t B, int64_t S, int64_t H, int64_t D,
                             int dtype, const mat_pattern_spec *spec, float scale,
                             void *staging, size_t staging_bytes, int device);

size_t mat_sparse_attn_host_staging_bytes(int64_t B, int64_t S, int64_t H, int64_t D,
                                          int dtype, const mat_pattern_spec *spec);

/*
 * Host-side index sets: the sorted, duplicate-free key positions of query row
 * i, the single source the kernels' masks are checked against.  Counterpart of
 * the COO generators (src/csrc/ma_core.cpp:34-48,
 * src/csrc/sparse_attention.cpp:181-259).  Returns the count in *n_out; when
 * cap is too small nothing is written and MAT_ERR_INVALID is returned with the
 * needed count in *n_out.
 */
int mat_pattern_rowset(const mat_pattern_spec *spec, int64_t S_kv, int64_t i,
                       int64_t *out, int64_t cap, int64_t *n_out);

/* Number of (query, key) pairs over query rows [0, S_q): the pattern's nnz. */
int mat_pattern_nnz(const mat_pattern_spec *spec, int64_t S_q, int64_t S_kv, int64_t *nnz_out);

/* Name of the kernel family the last mat_sparse_attn_fwd call on this thread
 * selected ("rowwarp", "mma_window", ...): lets tests assert which path ran. */
const char *mat_last_kernel(void);

/*
 * Reads and clears the device status word of the current device (synchronises
 * with it).  0 = every kernel ran to completion; 1 = a kernel gave up on a
 * bounded wait for a staged tile and left its outputs incomplete.  No
 * counterpart in the reference, whose kernel never waits.
 */
int mat_device_status(int *status_out);

#ifdef __cplusplus
}
#endif
#endif /* MAT_SPARSE_ATTN_H */
