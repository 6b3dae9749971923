// Shared definitions for the sparse-MLA kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/smla.h"

namespace smla {

constexpr int D_NOPE = SMLA_D_NOPE;
constexpr int D_ROPE = SMLA_D_ROPE;
constexpr int D_QK = SMLA_D_QK;
constexpr int D_V = SMLA_D_V;
constexpr int ROW_BYTES = SMLA_ROW_BYTES;
constexpr int SCALE_OFF = 512;   // byte offset of the 4 fp32 scales inside a row
constexpr int ROPE_OFF = 528;    // byte offset of the 64 bf16 RoPE values inside a row
constexpr int BLOCK_N = SMLA_BLOCK_N;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_BIG = -1e30f;  // "no entry" logit / LSE sentinel, as in the reference kernels

// One partition record of the split-KV scheduler (8 x int32).
struct SchedMeta {
    int begin_req, end_req, begin_block, end_block, begin_split, first_split, last_split, pad;
};
static_assert(sizeof(SchedMeta) == 32, "scheduler record is 8 int32");

// Arguments common to the attention kernels.
struct AttnParams {
    const __nv_bfloat16* q;      // [T, H, 576]
    const uint8_t* kv;           // packed rows
    const int32_t* indices;      // [T, topk]
    float* o_accum;              // [splits, H, 512] (decode only)
    float* lse_accum;            // [splits, H]
    __nv_bfloat16* out;          // [T, H, 512]
    float* out_lse;              // [T, H]
    float* out_max_logits;       // [T, H] or null (prefill only)
    const SchedMeta* sched;      // [parts] or null => one partition per token, never split
    const int32_t* num_splits;   // [T+1] or null
    const float* attn_sink;      // [H] or null
    const int32_t* topk_length;  // [T] or null
    int32_t* status;             // device int32[4] or null
    int num_tokens, num_heads, topk, num_parts;
    int force_partial;           // 1: every request writes an fp32 partial record, none writes `out`
    int uniform_k;               // > 1 (no scheduler, all requests topk long): every request is cut into uniform_k equal
                                 // partitions, partition j of request r writes partial record j * num_tokens + r
    int page_block_size;
    int64_t block_stride;        // bytes between pages
    float sm_scale;
    // The cache layout and the second ("extra") cache.
    int layout;                       // SMLA_LAYOUT_*
    const uint8_t* extra_kv;          // null = none
    const int32_t* extra_indices;     // [T, extra_topk]
    const int32_t* extra_topk_length; // [T] or null
    int extra_topk;
    int extra_page_block_size;
    int64_t extra_block_stride;
};

__device__ __forceinline__ const uint8_t* kv_row_ptr(const uint8_t* kv, int idx, int page_block_size,
                                                     int64_t block_stride) {
    const unsigned u = (unsigned)idx;
    const unsigned blk = u / (unsigned)page_block_size;
    const unsigned in = u - blk * (unsigned)page_block_size;
    return kv + (int64_t)blk * block_stride + (int64_t)in * ROW_BYTES;
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
    __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(__half(hr));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Programmatic dependent launch: a kernel launched with launch_dependent() may start (and run everything that comes
// before its grid_dep_wait()) while the kernel before it on the stream is still running; grid_dep_wait() returns
// when that kernel has completed and its writes are visible.  A kernel that calls grid_dep_launch() lets the next
// one start early.  Both are no-ops in a kernel that was launched the ordinary way.  The reference uses the same
// mechanism between its scheduler, decode and combine kernels (csrc/kernel/decode/decode_launch.cu:46-49).
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Host-side error plumbing (api.cu).
int set_error(int code, const char* fmt, ...);
int check_launch(const char* what);
// Argument checks shared by the attention entry points (nothing is launched when it fails).
int check_attn_common(const char* fn, const void* q, const void* kv, const int32_t* indices, const void* out,
                      const float* out_lse, int num_tokens, int num_heads, int topk, int page_block_size, int64_t stride,
                      int impl);

// Launchers (one per translation unit).
int launch_sched_meta(int b, int topk, int extra_topk, int num_sm_parts, int fixed_overhead,
                      const int32_t* topk_length, const int32_t* extra_topk_length,
                      int32_t* sched_meta, int32_t* num_splits, cudaStream_t stream);
int launch_combine(const float* o_accum, const float* lse_accum, __nv_bfloat16* out, float* out_lse,
                   const int32_t* num_splits, int batch, int num_heads, int max_nsplits,
                   const float* attn_sink, cudaStream_t stream);
int launch_combine_f32(const float* o_accum, const float* lse_accum, float* out, float* out_lse,
                       const int32_t* num_splits, int batch, int num_heads, int out_slices, int64_t out_slice_stride,
                       cudaStream_t stream);
int launch_cp_unslice(const void* gathered, __nv_bfloat16* out, float* lse, int slices, int num_tokens, int hs,
                      int64_t chunk_bytes, cudaStream_t stream);
int launch_combine_parts(const float* o_parts, const float* lse_parts, __nv_bfloat16* out, float* out_lse,
                         int parts, int batch, int num_heads, int64_t part_stride_o, int64_t part_stride_l,
                         const float* attn_sink, cudaStream_t stream);
int launch_combine_parts_f16(const void* o_parts, const float* lse_parts, __nv_bfloat16* out, float* out_lse,
                             int parts, int batch, int num_heads, const float* attn_sink, cudaStream_t stream);
int launch_attn_scalar(const AttnParams& p, cudaStream_t stream);
int launch_attn_pair(const AttnParams& p, cudaStream_t stream);
bool attn_pair_takes(const AttnParams& p);   // alignment of the caches that the tensor-core kernel's bulk copies need
int launch_pack_kv(const __nv_bfloat16* kv, uint8_t* packed, int64_t num_rows, cudaStream_t stream);
int launch_mqa_logits_scalar(const uint8_t* q, const uint8_t* k, const float* k_scale, const float* weights,
                             const int32_t* ks, const int32_t* ke, float* logits, int s_q, int num_heads,
                             int s_k, int64_t logits_stride, cudaStream_t stream);
int launch_mqa_logits_tc(const uint8_t* q, const uint8_t* k, const float* k_scale, const float* weights,
                         const int32_t* ks, const int32_t* ke, float* logits, int s_q, int num_heads,
                         int s_k, int64_t logits_stride, int32_t* status, cudaStream_t stream);
int launch_topk(const float* logits, const int32_t* ks, const int32_t* ke, int32_t* out, int num_rows,
                int num_cols, int64_t logits_stride, int k, cudaStream_t stream);
int launch_cp_partition(const int32_t* indices, int32_t* local_indices, int32_t* local_length,
                        int num_tokens, int topk, int lo, int hi, cudaStream_t stream);

int launch_cp_window(const int32_t* ks, const int32_t* ke, int32_t* ks_local, int32_t* ke_local, int num_tokens,
                     int lo, int hi, cudaStream_t stream);
int launch_cp_candidates(const float* logits, int64_t logits_stride, const int32_t* picked, float* values,
                         int32_t* positions, int num_tokens, int k, int lo, cudaStream_t stream);
int launch_cp_interleave(const int32_t* gathered, int32_t* values, int32_t* positions, int world, int num_tokens, int k,
                         cudaStream_t stream);
int launch_cp_pick(const int32_t* positions, const int32_t* pick, int32_t* out, int num_tokens, int k, int num_candidates,
                   cudaStream_t stream);

}  // namespace smla
