// Shared declarations of libmat_sparse_attn's translation units: element-type
// helpers, the device-side copy of the pattern description, error plumbing and
// the launchers each kernel file exports to the C-ABI layer.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mat_sparse_attn.h"

namespace mat {

// Pattern description as the kernels see it (pointers are device pointers).
struct DevPattern {
    int32_t kind;
    int32_t causal;
    int64_t left, right, dilation;
    int64_t block, n_qblocks;
    const int32_t *rowptr;
    const int32_t *colidx;
    int64_t n_global;
    const int64_t *gidx;
    int64_t q_offset;
};

struct Problem {
    const void *q, *k, *v;
    void *o;
    int64_t B, Sq, Skv, H, D;
    int dtype;
    float scale;
    DevPattern pat;
    void *workspace;
    size_t workspace_bytes;
    cudaStream_t stream;
    // neighbouring sequence shards read in place (peer memory); NULL when absent
    const void *k_prev = nullptr, *v_prev = nullptr, *k_next = nullptr, *v_next = nullptr;
    int64_t S_prev = 0, S_next = 0;
    // Token strides of q, k, v, o in elements (0: contiguous, i.e. H * D).  Heads of a token stay contiguous and
    // a batch item is S tokens of that stride: the layout of q, k, v inside a fused projection output
    // [B, S, 3, H, D].  Only the band kernel reads strided tensors.
    int64_t q_ts = 0, k_ts = 0, v_ts = 0, o_ts = 0;
    // Longformer shard of a sequence spread over GPUs: K/V rows at all global positions, gathered by the caller
    const void *shard_kg = nullptr, *shard_vg = nullptr;
};

// error plumbing (api.cu)
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);
void note_kernel(const char *name);
// Raises a kernel's dynamic shared-memory limit, once per (kernel, device): the attribute belongs
// to the function on one device, so a process that drives several GPUs needs it on each.
int ensure_dynamic_smem(const void *kernel, size_t bytes, const char *what);
// validation + kernel selection shared by the device and host entry points (api.cu)
int make_problem(Problem &p, const void *q, const void *k, const void *v, void *o, int64_t B,
                 int64_t S_q, int64_t S_kv, int64_t H, int64_t D, int dtype,
                 const mat_pattern_spec *spec, float scale, void *ws, size_t ws_bytes, void *stream);
int run_problem(const Problem &p);

// kernel families; each returns MAT_OK or a MAT_ERR_* after recording the text
int launch_rowwarp(const Problem &p);        // rowwarp.cu: any pattern, any D <= 512
bool mma_window_f32_supports(const Problem &p);   // mma_window_f32.cu: fp32 windows as three TF32 products, D = 16, 32, 48, 64, 96, 128, 192, ... 512
int launch_mma_window_f32(const Problem &p);
bool tiled_f32_supports(const Problem &p);   // tiled_f32.cu: fp32 windows of at most 128 taps, D = 32, 64 or 128
int launch_tiled_f32(const Problem &p);
int tiled_status_read_and_clear(int *out);
bool mma_window_d_supports(const Problem &p);   // mma_window_d.cu: 16-bit windows, head widths 16..128 in steps of 16 other than 64
int launch_mma_window_d(const Problem &p);
size_t mma_window_d_scratch_bytes(const Problem &p);   // fp32 scratch of the sliced kernel for windows of several passes
bool mma_flash_supports(const Problem &p);   // mma_flash.cu
int launch_mma_flash(const Problem &p);
size_t mma_flash_workspace_bytes(const Problem &p);
int flash_status_read_and_clear(int *out);   // status word left by a kernel whose bounded wait ran out
bool umma_block_supports(const Problem &p);  // umma_block.cu: block layouts on tcgen05 / TMEM
int launch_umma_block(const Problem &p);
bool umma_dense_supports(const Problem &p);  // dense / causal dense on the same tcgen05 pipeline
int launch_umma_dense(const Problem &p);
int umma_status_read_and_clear(int *out);
bool umma_band_supports(const Problem &p);   // umma_band.cu: windows of at most 128 taps, persistent, on tcgen05 / TMEM
bool umma_band_fits(const Problem &p);       // can run it at all (umma_band_supports also weighs the problem's size)
int launch_umma_band(const Problem &p);
int band_status_read_and_clear(int *out);
// first pass of a Longformer forward on the band kernel; kg, vg: the K/V rows at the global positions, gathered
bool umma_band_longformer_supports(const Problem &p);
int launch_umma_band_longformer(const Problem &p, const void *kg, const void *vg, const void *qg, float *partial);
// lanes per head when that pass also accumulates the rows AT the global positions (0: it does not), and the
// bytes of the partials it then leaves: [B, H, lanes, 32, kPartialStride] floats
int umma_band_longformer_lanes(const Problem &p);
size_t umma_band_longformer_partial_bytes(const Problem &p);
// Longformer global-row pass on tcgen05 (umma_block.cu): how the key axis is split, and the launch
constexpr int kPartialStride = 66;   // floats per row of a partial: max, sum, 64 outputs
struct GlobalRowSplit {
    int tiles, tile_rows;   // tiles of the global-position list, rows per tile
    int n_splits, split_len;
    int ng_pad;             // rows per split in the partial buffer
    size_t bytes;           // partial buffer size
};
GlobalRowSplit plan_umma_global_rows(const Problem &p);
int launch_umma_global_rows(const Problem &p, const GlobalRowSplit &g, float *partial);

// Tiled tensor map over 16-bit [B, S1, HH, 64] rows (mma_flash.cu): dims {64, HH, S1, B}, box {64, 1, box_rows, 1},
// 128-byte swizzle, zeros for rows outside the tensor.
int make_row_tensor_map(CUtensorMap *m, const void *base, int dtype, int64_t HH, int64_t S1, int64_t B,
                        int box_rows);
// The same rows as a 5-D map {64, H, dil, S/dil, B} with an explicit token stride (bytes): box {64, 1, 1, box_rows, 1}.
int make_row_tensor_map5(CUtensorMap *m, const void *base, int dtype, int64_t H, int64_t dil, int64_t S1, int64_t B,
                         int box_rows, int64_t token_stride_bytes);
int bwd_status_read_and_clear(int *out);     // bwd_mma.cu
// tensor-core backward of window patterns, dense included (bwd_mma.cu): 16-bit types, D = 64, S a multiple of the dilation
bool bwd_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t left, int64_t right,
                      int64_t dil);
int launch_bwd_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
                   float2 *stats, int64_t B, int64_t S, int64_t H, int dtype, int64_t left, int64_t right,
                   int64_t dil, float scale, cudaStream_t stream);
bool bwd_d_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t dil, int64_t left, int64_t right,
                        bool have_scratch);   // bwd_d_mma.cu
size_t bwd_d_mma_scratch_bytes(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t dil, int64_t left, int64_t right);
int launch_bwd_d_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
                     float2 *stats, int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t left, int64_t right,
                     int64_t dil, float scale, float *scratch, cudaStream_t stream);
bool bwd_f32_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t dil);   // bwd_f32_mma.cu
int launch_bwd_f32_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
                       float2 *stats, int64_t B, int64_t S, int64_t H, int64_t D, int64_t left, int64_t right,
                       int64_t dil, float scale, cudaStream_t stream);
bool bwd_longformer_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t n_global);
size_t bwd_longformer_mma_extra_bytes(int64_t B, int64_t H, int64_t n_global);
int launch_bwd_longformer_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk,
                              void *dv, float2 *stats, void *extra_ws, int64_t B, int64_t S, int64_t H, int dtype,
                              int64_t left, int64_t right, int64_t n_global, const int64_t *gidx, float scale,
                              cudaStream_t stream);
bool bwd_block_mma_supports(int64_t B, int64_t S, int64_t H, int64_t D, int dtype, int64_t block);
int launch_bwd_block_mma(const void *q, const void *k, const void *v, const void *dout, void *dq, void *dk, void *dv,
                         float2 *stats, int64_t B, int64_t S, int64_t H, int dtype, int64_t block, int causal,
                         const int32_t *rowptr, const int32_t *colidx, const int32_t *t_rowptr, const int32_t *t_colidx,
                         float scale, cudaStream_t stream);

template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float to_f(float x) { return x; }
    static __device__ __forceinline__ float from_f(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};

static inline size_t dtype_size(int dtype) { return dtype == MAT_F32 ? 4 : 2; }

}  // namespace mat
