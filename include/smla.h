/*
 * C ABI of the B200 sparse-MLA kernel library (libsmla_b200.so).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (cudaStream_t passed
 * as void*; NULL = the legacy default stream).  Nothing here allocates, synchronises with the
 * host or reads device memory on the host unless its comment says so, so the calls can be
 * recorded into CUDA graphs.  All functions return 0 on success, a negative SMLA_E_* code for
 * an argument error (nothing was launched) or a positive cudaError_t value when a launch
 * failed.  smla_last_error() returns the message of the last failure on the calling thread.
 *
 * Each declaration names the interface of the reference project (path:line in that project)
 * that it stands in for.
 */
#ifndef SMLA_H_
#define SMLA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMLA_D_NOPE 512
#define SMLA_D_ROPE 64
#define SMLA_D_QK 576
#define SMLA_D_V 512
#define SMLA_ROW_BYTES 656   /* 512 e4m3 | 4 fp32 scales | 64 bf16 */
#define SMLA_BLOCK_N 64      /* tokens per scheduling block */
#define SMLA_SCHED_META_INTS 8

enum {
    SMLA_OK = 0,
    SMLA_E_NULL = -1,        /* a required pointer is NULL */
    SMLA_E_SHAPE = -2,       /* unsupported size (heads, topk, d_qk, ...) */
    SMLA_E_ALIGN = -3,       /* pointer or stride not 16-byte aligned */
    SMLA_E_UNSUPPORTED = -4, /* feature of the reference interface that is not built */
    SMLA_E_WORKSPACE = -5,   /* scratch too small for the request */
    SMLA_E_DEVICE = -6       /* the kernel reported a device-side status (see smla_device_status) */
};

/*
 * Device-side status.  The tcgen05 kernels bound every wait; a wait that gives up writes its code to
 * status[0] (first one wins), counts the CTAs that gave up in status[1] and names one of them in status[2].
 * smla_device_status copies the four words to the host (it synchronises the stream: not for the hot
 * path), clears status[0..3] on the device when a code was set, and returns 0 or SMLA_E_DEVICE with the
 * wait's name in smla_last_error().  smla_status_string names a code ("" for 0, "unknown" otherwise).
 */
int smla_device_status(int32_t* status, int32_t host_out[4], void* stream);
const char* smla_status_string(int code);

/* Kernel selection for the attention entry points. */
enum {
    SMLA_IMPL_AUTO = 0,    /* tcgen05 kernel */
    SMLA_IMPL_SCALAR = 1,  /* fp32 CUDA-core kernel: slow, exact; a second opinion in tests */
    SMLA_IMPL_TC = 2       /* tcgen05/TMEM kernel on a pair of SMs (cta_group::2), FP8 QK^T and PV */
};

/*
 * Cache layouts (csrc/model/kv_cache_traits.cuh:16-59 and :61-111).
 *   V32     656 bytes per token, scales inline: 512 e4m3 | 4 fp32 scales | 64 bf16; q has 576 dims,
 *           V is the 512 dequantised values.
 *   MODEL1  584 bytes per token, scales in a footer: a page of `page_block_size` tokens is
 *           page_block_size x 576 data bytes (448 e4m3 | 64 bf16 per token) followed by
 *           page_block_size x 8 footer bytes (7 UE8M0 scales, one per 64 values, + 1 pad);
 *           q has 512 dims, V is the whole dequantised row (448 values + the 64 bf16).
 */
enum {
    SMLA_LAYOUT_V32 = 0,
    SMLA_LAYOUT_MODEL1 = 1
};
#define SMLA_M1_D_QK 512
#define SMLA_M1_ROW_BYTES 584
#define SMLA_M1_DATA_BYTES 576

const char* smla_last_error(void);
int smla_version(void);

/* Number of SMs of the current device (cached per device).  Host query only. */
int smla_num_sms(void);

/*
 * Split-KV scheduler.  Replaces get_decode_metadata (csrc/binding.cpp:281-286,
 * csrc/kernel/sched/get_sched_meta.cu:148-165).  Writes num_sm_parts records of 8 int32
 * {begin_req, end_req, begin_block, end_block, begin_split_idx, first_is_split, last_is_split, 0}
 * (layout of csrc/kernel/sched/sched_params.h:8-18) and the prefix sum num_splits[b+1].
 * topk_length / extra_topk_length may be NULL.  One 32-thread CTA; b <= 8192.
 */
int smla_sched_meta(int b, int topk, int extra_topk, int num_sm_parts, int fixed_overhead,
                    const int32_t* topk_length, const int32_t* extra_topk_length,
                    int32_t* sched_meta, int32_t* num_splits, void* stream);

/*
 * Scheduler-driven split-KV decode.  Replaces sparse_mla_splitkv_v2_fwd
 * (csrc/binding.cpp:96-164, kernel csrc/kernel/decode/decode_v2_kernel.cuh:54-657).
 *   q          [num_tokens, num_heads, 576] bf16, contiguous
 *   kv         packed rows of 656 bytes; row r lives at
 *              kv + (r / page_block_size) * kv_block_stride_bytes + (r % page_block_size) * 656
 *   indices    [num_tokens, topk] int32, physical row numbers, -1 = no entry
 *   o_accum    [>= num_tokens + num_sm_parts, 1, num_heads, 512] fp32 partial outputs
 *   lse_accum  [>= num_tokens + num_sm_parts, 1, num_heads]      fp32 base-2 partial LSE
 *   out        [num_tokens, num_heads, 512] bf16 (written directly for unsplit requests)
 *   out_lse    [num_tokens, num_heads] fp32, base-2 LSE of the scaled logits, -1e30 when empty
 *   attn_sink  [num_heads] fp32 natural-log sink logit or NULL; topk_length [num_tokens] or NULL
 * num_heads in 1..128; topk >= 1 (a last block that is partly filled is masked).  status (device
 * int32[4], may be NULL) receives a non-zero code when a bounded wait inside the tcgen05 kernel gave up.
 */
int smla_decode_splitkv(const void* q, const void* kv, const int32_t* indices,
                        float* o_accum, float* lse_accum, void* out, float* out_lse,
                        const int32_t* sched_meta, const int32_t* num_splits,
                        int num_tokens, int num_heads, int topk, float sm_scale,
                        int page_block_size, int64_t kv_block_stride_bytes, int num_sm_parts,
                        const float* attn_sink, const int32_t* topk_length,
                        int impl, int32_t* status, void* stream);

/*
 * Split-KV decode of requests that all have `topk` entries (no topk_length), every request cut into
 * parts_per_request equal partitions (a divisor of ceil(topk / 64)): what smla_sched_meta would lay out for
 * parts_per_request * num_tokens partitions and a fixed overhead of 0, derived inside the attention kernel, so that
 * the step is two launches (attention, combine) instead of three.  o_accum / lse_accum are scratch for
 * parts_per_request * num_tokens records (partition j of request r is record j * num_tokens + r; the call keeps
 * the partial outputs in fp16 there, so o_accum needs half of what its type says, its contents are private).  tcgen05 kernel
 * only.  No counterpart in the reference (its scheduler kernel runs every step, flash_mla_sm120/ops.py:78-99).
 */
int smla_decode_uniform(const void* q, const void* kv, const int32_t* indices,
                        float* o_accum, float* lse_accum, void* out, float* out_lse,
                        int num_tokens, int num_heads, int topk, float sm_scale,
                        int page_block_size, int64_t kv_block_stride_bytes, int parts_per_request,
                        const float* attn_sink, int impl, int32_t* status, void* stream);

/*
 * LSE-weighted merge of the split partials.  Replaces sparse_mla_combine_v2_fwd
 * (csrc/binding.cpp:166-183, kernel csrc/kernel/combine/combine_kernel.cu:39-159).
 * Requests with <= 1 split are left untouched.  max_nsplits <= 1024.
 */
int smla_combine(const float* o_accum, const float* lse_accum, void* out, float* out_lse,
                 const int32_t* num_splits, int batch, int num_heads, int max_nsplits,
                 const float* attn_sink, void* stream);

/*
 * Single-pass sparse attention for many query tokens.  Replaces sparse_mla_prefill_fwd
 * (csrc/binding.cpp:185-247, kernels csrc/kernel/prefill/prefill_kernel.cuh:48-553,570-1134).
 * out_max_logits [num_tokens, num_heads] fp32 (running maximum of the scaled base-2 logits)
 * may be NULL.
 */
int smla_prefill(const void* q, const void* kv, const int32_t* indices,
                 void* out, float* out_lse, float* out_max_logits,
                 int num_tokens, int num_heads, int topk, float sm_scale,
                 int page_block_size, int64_t kv_block_stride_bytes,
                 const float* attn_sink, const int32_t* topk_length,
                 int impl, int32_t* status, void* stream);

/*
 * The two calls above with everything the reference's entry points take besides
 * (csrc/binding.cpp:96-164 and :185-247, kernel arguments csrc/kernel/decode/decode_v2_kernel.cuh:40-66):
 * the cache layout, and a second ("extra") cache with its own page size, index array
 * [num_tokens, extra_topk] and lengths.  A request walks max(ceil(topk_length/64), 1) blocks of the main
 * cache, then ceil(extra_topk_length/64) blocks of the extra cache (decode_v2_kernel.cuh:109-115); one
 * softmax runs over both.  For SMLA_LAYOUT_MODEL1 q is [num_tokens, num_heads, 512].  extra_kv NULL and
 * extra_topk 0 = no second cache; the scheduler must have been given the same extra_topk and
 * extra_topk_length.  impl as above, with two differences.  SMLA_IMPL_TC refuses caches whose base address or
 * page stride is not a multiple of 16 bytes (what the kernel's bulk copies need) with SMLA_E_ALIGN; SMLA_IMPL_AUTO
 * runs the fp32 kernel for them.  And SMLA_IMPL_AUTO runs the fp32 kernel for SMLA_LAYOUT_MODEL1: V includes the
 * row's RoPE there, which the tcgen05 kernel rounds to e4m3 with the rest of V (the reference multiplies it in
 * bf16, csrc/kernel/common/xv_rope_mma.cuh:23-93), so results of rows with few entries differ from the
 * reference's by up to about 2e-3 on its own test data; callers that accept this ask for SMLA_IMPL_TC.
 */
int smla_decode_splitkv_ext(const void* q, const void* kv, const int32_t* indices,
                            const void* extra_kv, const int32_t* extra_indices,
                            float* o_accum, float* lse_accum, void* out, float* out_lse,
                            const int32_t* sched_meta, const int32_t* num_splits,
                            int num_tokens, int num_heads, int topk, int extra_topk, float sm_scale, int layout,
                            int page_block_size, int64_t kv_block_stride_bytes,
                            int extra_page_block_size, int64_t extra_block_stride_bytes, int num_sm_parts,
                            const float* attn_sink, const int32_t* topk_length, const int32_t* extra_topk_length,
                            int impl, int32_t* status, void* stream);
int smla_prefill_ext(const void* q, const void* kv, const int32_t* indices,
                     const void* extra_kv, const int32_t* extra_indices,
                     void* out, float* out_lse, float* out_max_logits,
                     int num_tokens, int num_heads, int topk, int extra_topk, float sm_scale, int layout,
                     int page_block_size, int64_t kv_block_stride_bytes,
                     int extra_page_block_size, int64_t extra_block_stride_bytes,
                     const float* attn_sink, const int32_t* topk_length, const int32_t* extra_topk_length,
                     int impl, int32_t* status, void* stream);

/*
 * bf16 -> packed 656-byte rows (the writer of the cache format).  No kernel of the reference
 * does this; the format is specified by tests/test_decode.py:33-57 (quantize_kv_v32).
 *   kv_bf16 [num_rows, 576] bf16, packed [num_rows, 656] uint8.
 */
int smla_pack_kv(const void* kv_bf16, void* packed, int64_t num_rows, void* stream);

/*
 * FP8 MQA-logits indexer.  No counterpart in the reference (the indices it consumes come from
 * an external indexer, flash_mla_sm120/interface.py:39-58).
 *   logits[i, j] = k_scale[j] * sum_h weights[i, h] * relu(q[i, h, :] . k[j, :]),
 *   -inf for j outside [ks[i], ke[i]).
 *   q [s_q, num_heads, 128] e4m3, k [s_k, 128] e4m3, k_scale [s_k] fp32,
 *   weights [s_q, num_heads] fp32, ks/ke [s_q] int32, logits [s_q, logits_stride] fp32.
 */
int smla_mqa_logits(const void* q, const void* k, const float* k_scale, const float* weights,
                    const int32_t* ks, const int32_t* ke, float* logits,
                    int s_q, int num_heads, int s_k, int64_t logits_stride,
                    int impl, int32_t* status, void* stream);

/*
 * Per-row top-k selection over logits[row, ks[row]:ke[row]) (ks/ke may be NULL = whole row).
 * Writes k int32 indices per row, unordered, padded with -1 when fewer than k candidates are
 * finite.  Ties at the threshold are broken towards the lower index.  No counterpart in the
 * reference.
 */
int smla_topk(const float* logits, const int32_t* ks, const int32_t* ke, int32_t* out_indices,
              int num_rows, int num_cols, int64_t logits_stride, int k, void* stream);

/*
 * Context-parallel index partition: keeps, in order, the entries of each row that fall in
 * [lo, hi), rebases them to lo, pads with -1 and writes the count to local_length.  No
 * counterpart in the reference (it has no multi-GPU path).
 */
int smla_cp_partition_indices(const int32_t* indices, int32_t* local_indices, int32_t* local_length,
                              int num_tokens, int topk, int lo, int hi, void* stream);

/*
 * Distributed top-k of the indexer under context parallelism (rank g holds the keys of positions
 * [lo, hi)); four small steps around smla_mqa_logits / smla_topk.  No counterpart in the
 * reference.
 *   smla_cp_local_window          ks/ke [num_tokens] (global positions) clipped to the shard and
 *                                 rebased to lo.
 *   smla_cp_candidates            picked [num_tokens, k] (columns of the shard's logits, -1 =
 *                                 none) -> values [num_tokens, k] (the logits, -inf for none) and
 *                                 positions [num_tokens, k] (picked + lo, -1 for none).
 *   smla_cp_interleave_candidates gathered [world][2][num_tokens][k] (every rank's values, then
 *                                 positions, as all-gathered) -> values / positions
 *                                 [num_tokens][world * k], the candidates of a token side by side.
 *   smla_cp_pick_positions        out[t][i] = positions[t][pick[t][i]] (pick: the columns
 *                                 smla_topk chose among the world * k candidates; -1 stays -1).
 */
int smla_cp_local_window(const int32_t* ks, const int32_t* ke, int32_t* ks_local, int32_t* ke_local, int num_tokens,
                         int lo, int hi, void* stream);
int smla_cp_candidates(const float* logits, int64_t logits_stride, const int32_t* picked, float* values,
                       int32_t* positions, int num_tokens, int k, int lo, void* stream);
int smla_cp_interleave_candidates(const int32_t* gathered, float* values, int32_t* positions, int world, int num_tokens,
                                  int k, void* stream);
int smla_cp_pick_positions(const int32_t* positions, const int32_t* pick, int32_t* out, int num_tokens, int k,
                           int num_candidates, void* stream);

/*
 * Context-parallel local step: split-KV decode over this GPU's shard followed by the local
 * merge, giving ONE fp32 partial per token (normalised by its own sum) and its base-2 LSE, ready
 * to be exchanged.  Same arguments as smla_decode_splitkv; o_part [num_tokens, num_heads, 512]
 * fp32 and lse_part [num_tokens, num_heads] fp32 replace out / out_lse, and no sink is applied
 * (the sink belongs to the final merge).  No counterpart in the reference.
 */
int smla_decode_partial(const void* q, const void* kv, const int32_t* indices,
                        float* o_accum, float* lse_accum, float* o_part, float* lse_part,
                        const int32_t* sched_meta, const int32_t* num_splits,
                        int num_tokens, int num_heads, int topk, float sm_scale,
                        int page_block_size, int64_t kv_block_stride_bytes, int num_sm_parts,
                        const int32_t* topk_length, int impl, int32_t* status, void* stream);

/*
 * The same local step with the result cut into head slices for an all-to-all: slice d (the heads
 * [d * num_heads / slices, (d + 1) * num_heads / slices), destined for rank d) starts slice_stride
 * floats after slice d - 1 and holds [num_tokens, num_heads / slices, 512] partials followed by the
 * slice's [num_tokens, num_heads / slices] LSEs.  slice_stride must be a multiple of 512 floats and
 * at least num_tokens * (num_heads / slices) * 513.  No counterpart in the reference.
 */
int smla_decode_partial_sliced(const void* q, const void* kv, const int32_t* indices,
                               float* o_accum, float* lse_accum, float* send, int slices, int64_t slice_stride,
                               const int32_t* sched_meta, const int32_t* num_splits,
                               int num_tokens, int num_heads, int topk, float sm_scale,
                               int page_block_size, int64_t kv_block_stride_bytes, int num_sm_parts,
                               const int32_t* topk_length, int impl, int32_t* status, void* stream);

/*
 * Reassembles the all-gathered head slices of the merged output: chunk g of `gathered` (chunk_bytes
 * apart, a multiple of 16) holds [num_tokens, heads_per_slice, 512] bf16 followed by
 * [num_tokens, heads_per_slice] fp32 LSEs -> out [num_tokens, slices * heads_per_slice, 512] bf16 and
 * lse [num_tokens, slices * heads_per_slice].  No counterpart in the reference.
 */
int smla_cp_unslice(const void* gathered, void* out, float* lse, int slices, int num_tokens, int heads_per_slice,
                    int64_t chunk_bytes, void* stream);

/*
 * Final merge of the context-parallel exchange: o_parts [parts, num_tokens, num_heads, 512] fp32
 * and lse_parts [parts, num_tokens, num_heads] fp32 (the layout an all-gather of the per-GPU
 * partials produces) -> out bf16 and base-2 LSE, sink applied if given.  Same arithmetic as
 * smla_combine (csrc/kernel/combine/combine_kernel.cu:39-159); the strided layout has no
 * counterpart in the reference.
 */
int smla_combine_parts(const float* o_parts, const float* lse_parts, void* out, float* out_lse,
                       int parts, int num_tokens, int num_heads, const float* attn_sink, void* stream);

/*
 * The same merge when the partials of rank g start o_part_stride floats after those of rank
 * g - 1 (and the LSEs lse_part_stride floats), e.g. one buffer per rank holding
 * [num_tokens * num_heads * 512 partials | num_tokens * num_heads LSEs], which ONE all-gather
 * fills: o_part_stride = lse_part_stride = num_tokens * num_heads * 513 and lse_parts =
 * o_parts + num_tokens * num_heads * 512.  o_part_stride must be a multiple of 4 floats.
 */
int smla_combine_parts_strided(const float* o_parts, const float* lse_parts, void* out, float* out_lse,
                               int parts, int num_tokens, int num_heads, int64_t o_part_stride,
                               int64_t lse_part_stride, const float* attn_sink, void* stream);

/*
 * Split-KV decode (scheduler + attention + combine in one call) that allocates nothing and takes
 * no scratch from the caller.  It has no counterpart in the reference.  It is for hosts that
 * cannot give this library device memory at call time: a process whose own pool already owns the
 * whole device, or a call site that must stay out of the CUDA allocator because cudaMalloc can
 * synchronise the device.  The scratch is an array of SMLA_NOALLOC_SCRATCH_BYTES built into the
 * library (held on every GPU that loads it until the process exits), so requests are limited to
 * smla_noalloc_scratch_need(num_tokens, num_heads, num_sm_parts) <= SMLA_NOALLOC_SCRATCH_BYTES
 * (at 128 heads: num_tokens + num_sm_parts <= 63); larger ones return SMLA_E_WORKSPACE and a
 * message.  The first call on a device looks up the array's device address and should be made
 * before any stream capture.  All calls share the array: calls that overlap on the GPU race.
 * Arguments as smla_decode_splitkv, fixed_overhead of the scheduler is 5.
 */
#define SMLA_NOALLOC_SCRATCH_BYTES (16u << 20)
size_t smla_noalloc_scratch_need(int num_tokens, int num_heads, int num_sm_parts);
int smla_decode_splitkv_noalloc(const void* q, const void* kv, const int32_t* indices,
                                void* out, float* out_lse,
                                int num_tokens, int num_heads, int topk, float sm_scale,
                                int page_block_size, int64_t kv_block_stride_bytes, int num_sm_parts,
                                const float* attn_sink, const int32_t* topk_length,
                                int impl, int32_t* status, void* stream);

/* Bytes of o_accum + lse_accum scratch that smla_decode_splitkv needs. */
size_t smla_workspace_bytes(int num_tokens, int num_heads, int num_sm_parts);

#ifdef __cplusplus
}
#endif
#endif /* SMLA_H_ */
