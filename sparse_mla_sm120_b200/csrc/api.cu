// extern "C" entry points of libsmla_b200.so: argument checks, error strings, dispatch.
// No torch types, no allocation, no host synchronisation.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace smla {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return 0;
    return set_error((int)e, "%s: launch failed: %s", what, cudaGetErrorString(e));
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_attn_common(const char* fn, const void* q, const void* kv, const int32_t* indices,
                             const void* out, const float* out_lse, int num_tokens, int num_heads, int topk,
                             int page_block_size, int64_t stride, int impl) {
    if (!q || !kv || !indices || !out || !out_lse) return set_error(SMLA_E_NULL, "%s: null pointer argument", fn);
    if (num_tokens < 0) return set_error(SMLA_E_SHAPE, "%s: num_tokens=%d", fn, num_tokens);
    if (num_heads < 1 || num_heads > 128)
        return set_error(SMLA_E_SHAPE, "%s: num_heads=%d, supported 1..128", fn, num_heads);
    if (topk < 1) return set_error(SMLA_E_SHAPE, "%s: topk=%d", fn, topk);
    if (page_block_size < 1) return set_error(SMLA_E_SHAPE, "%s: page_block_size=%d", fn, page_block_size);
    if (!aligned16(q) || !aligned16(kv) || !aligned16(out) || (stride & 15))
        return set_error(SMLA_E_ALIGN, "%s: q, kv, out and the page stride must be 16-byte aligned", fn);
    if (stride < (int64_t)page_block_size * ROW_BYTES)
        return set_error(SMLA_E_SHAPE, "%s: page stride %lld smaller than %d rows of %d bytes", fn,
                         (long long)stride, page_block_size, ROW_BYTES);
    if (impl != SMLA_IMPL_AUTO && impl != SMLA_IMPL_SCALAR && impl != SMLA_IMPL_TC)
        return set_error(SMLA_E_SHAPE, "%s: unknown impl %d", fn, impl);
    return 0;
}

}  // namespace smla

using namespace smla;

extern "C" {

const char* smla_last_error(void) { return g_err; }

const char* smla_status_string(int code) {
    switch (code) {
        case 0: return "";
        case 11: return "indexer q_full"; case 12: return "indexer k_full"; case 13: return "indexer k_empty";
        case 14: return "indexer d_full"; case 15: return "indexer d_empty"; case 16: return "indexer q_empty";
        case 17: return "indexer tmem";
        case 21: return "attention k_empty"; case 22: return "attention k_stored"; case 23: return "attention k_full";
        case 24: return "attention half-tile record"; case 25: return "attention v_empty"; case 26: return "attention v_full (one CTA)";
        case 27: return "attention v_full"; case 28: return "attention s_ready"; case 29: return "attention s_free";
        case 30: return "attention p_ready"; case 31: return "attention pv_done"; case 32: return "attention q_ready";
        case 33: return "attention q_staged"; case 34: return "attention q_free"; case 35: return "attention raw_empty";
        case 36: return "attention raw_full";
        default: return "unknown";
    }
}

int smla_device_status(int32_t* status, int32_t host_out[4], void* stream) {
    if (!status || !host_out) return set_error(SMLA_E_NULL, "smla_device_status: null pointer argument");
    cudaError_t e = cudaMemcpyAsync(host_out, status, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return set_error((int)e, "smla_device_status: %s", cudaGetErrorString(e));
    if (host_out[0] == 0) return 0;
    cudaMemsetAsync(status, 0, 4 * sizeof(int32_t), (cudaStream_t)stream);
    return set_error(SMLA_E_DEVICE, "kernel wait gave up: %s (code %d), %d CTAs, one of them CTA %d", smla_status_string(host_out[0]),
                     host_out[0], host_out[1], host_out[2]);
}
int smla_version(void) { return 100; }

int smla_num_sms(void) {
    static int cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return set_error(SMLA_E_DEVICE, "smla_num_sms: no CUDA device");
    if (dev < 64 && cache[dev]) return cache[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return set_error(SMLA_E_DEVICE, "smla_num_sms: attribute query failed");
    if (dev < 64) cache[dev] = n;
    return n;
}

size_t smla_workspace_bytes(int num_tokens, int num_heads, int num_sm_parts) {
    const size_t splits = (size_t)num_tokens + (size_t)num_sm_parts;
    return splits * num_heads * (D_V + 1) * sizeof(float);
}

int smla_sched_meta(int b, int topk, int extra_topk, int num_sm_parts, int fixed_overhead,
                    const int32_t* topk_length, const int32_t* extra_topk_length,
                    int32_t* sched_meta, int32_t* num_splits, void* stream) {
    if (!sched_meta || !num_splits) return set_error(SMLA_E_NULL, "smla_sched_meta: null output");
    if (b < 1 || b > 8192) return set_error(SMLA_E_SHAPE, "smla_sched_meta: b=%d, supported 1..8192", b);
    if (num_sm_parts < 1) return set_error(SMLA_E_SHAPE, "smla_sched_meta: num_sm_parts=%d", num_sm_parts);
    if (topk < 0 || extra_topk < 0 || fixed_overhead < 0)
        return set_error(SMLA_E_SHAPE, "smla_sched_meta: negative size");
    return launch_sched_meta(b, topk, extra_topk, num_sm_parts, fixed_overhead, topk_length,
                             extra_topk_length, sched_meta, num_splits, (cudaStream_t)stream);
}

int smla_decode_splitkv(const void* q, const void* kv, const int32_t* indices,
                        float* o_accum, float* lse_accum, void* out, float* out_lse,
                        const int32_t* sched_meta, const int32_t* num_splits,
                        int num_tokens, int num_heads, int topk, float sm_scale,
                        int page_block_size, int64_t kv_block_stride_bytes, int num_sm_parts,
                        const float* attn_sink, const int32_t* topk_length,
                        int impl, int32_t* status, void* stream) {
    if (int e = check_attn_common("smla_decode_splitkv", q, kv, indices, out, out_lse, num_tokens, num_heads,
                                  topk, page_block_size, kv_block_stride_bytes, impl)) return e;
    if (!o_accum || !lse_accum || !sched_meta || !num_splits)
        return set_error(SMLA_E_NULL, "smla_decode_splitkv: null scratch or scheduler pointer");
    if (!aligned16(o_accum)) return set_error(SMLA_E_ALIGN, "smla_decode_splitkv: o_accum not 16-byte aligned");
    if (num_sm_parts < 1) return set_error(SMLA_E_SHAPE, "smla_decode_splitkv: num_sm_parts=%d", num_sm_parts);
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.kv = (const uint8_t*)kv; p.indices = indices;
    p.o_accum = o_accum; p.lse_accum = lse_accum; p.out = (__nv_bfloat16*)out; p.out_lse = out_lse;
    p.out_max_logits = nullptr; p.sched = (const SchedMeta*)sched_meta; p.num_splits = num_splits;
    p.attn_sink = attn_sink; p.topk_length = topk_length; p.status = status;
    p.num_tokens = num_tokens; p.num_heads = num_heads; p.topk = topk; p.num_parts = num_sm_parts;
    p.page_block_size = page_block_size; p.block_stride = kv_block_stride_bytes; p.sm_scale = sm_scale;
    if (impl == SMLA_IMPL_SCALAR) return launch_attn_scalar(p, (cudaStream_t)stream);
    return launch_attn_pair(p, (cudaStream_t)stream);
}

int smla_decode_uniform(const void* q, const void* kv, const int32_t* indices,
                        float* o_accum, float* lse_accum, void* out, float* out_lse,
                        int num_tokens, int num_heads, int topk, float sm_scale,
                        int page_block_size, int64_t kv_block_stride_bytes, int parts_per_request,
                        const float* attn_sink, int impl, int32_t* status, void* stream) {
    if (int e = check_attn_common("smla_decode_uniform", q, kv, indices, out, out_lse, num_tokens, num_heads,
                                  topk, page_block_size, kv_block_stride_bytes, impl)) return e;
    if (impl == SMLA_IMPL_SCALAR)
        return set_error(SMLA_E_SHAPE, "smla_decode_uniform: the fp32 kernel needs the scheduler's records (use smla_decode_splitkv)");
    if (!o_accum || !lse_accum) return set_error(SMLA_E_NULL, "smla_decode_uniform: null scratch pointer");
    if (!aligned16(o_accum)) return set_error(SMLA_E_ALIGN, "smla_decode_uniform: o_accum not 16-byte aligned");
    const int blocks = (topk + BLOCK_N - 1) / BLOCK_N;
    if (parts_per_request < 2 || blocks % parts_per_request != 0)
        return set_error(SMLA_E_SHAPE, "smla_decode_uniform: %d blocks per request do not divide into %d partitions", blocks,
                         parts_per_request);
    if (num_tokens == 0) return SMLA_OK;
    if ((int64_t)num_tokens * parts_per_request > (1 << 20))
        return set_error(SMLA_E_SHAPE, "smla_decode_uniform: %d x %d partitions", num_tokens, parts_per_request);
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.kv = (const uint8_t*)kv; p.indices = indices;
    p.o_accum = o_accum; p.lse_accum = lse_accum; p.out = (__nv_bfloat16*)out; p.out_lse = out_lse;
    p.attn_sink = attn_sink; p.status = status;
    p.num_tokens = num_tokens; p.num_heads = num_heads; p.topk = topk; p.num_parts = num_tokens * parts_per_request;
    p.page_block_size = page_block_size; p.block_stride = kv_block_stride_bytes; p.sm_scale = sm_scale;
    p.uniform_k = parts_per_request;
    if (int e = launch_attn_pair(p, (cudaStream_t)stream)) return e;
    return launch_combine_parts_f16(o_accum, lse_accum, (__nv_bfloat16*)out, out_lse, parts_per_request, num_tokens,
                                    num_heads, attn_sink, (cudaStream_t)stream);
}

int smla_combine(const float* o_accum, const float* lse_accum, void* out, float* out_lse,
                 const int32_t* num_splits, int batch, int num_heads, int max_nsplits,
                 const float* attn_sink, void* stream) {
    if (!o_accum || !lse_accum || !out || !out_lse || !num_splits)
        return set_error(SMLA_E_NULL, "smla_combine: null pointer argument");
    if (batch < 0 || num_heads < 1) return set_error(SMLA_E_SHAPE, "smla_combine: batch=%d heads=%d", batch, num_heads);
    if (max_nsplits > 1024) return set_error(SMLA_E_SHAPE, "smla_combine: max_nsplits=%d exceeds 1024", max_nsplits);
    if (!aligned16(o_accum) || !aligned16(out)) return set_error(SMLA_E_ALIGN, "smla_combine: unaligned buffer");
    return launch_combine(o_accum, lse_accum, (__nv_bfloat16*)out, out_lse, num_splits, batch, num_heads,
                          max_nsplits, attn_sink, (cudaStream_t)stream);
}

static int decode_partial_common(const char* fn, const void* q, const void* kv, const int32_t* indices,
                                 float* o_accum, float* lse_accum, float* o_part, float* lse_part,
                                 const int32_t* sched_meta, const int32_t* num_splits,
                                 int num_tokens, int num_heads, int topk, float sm_scale,
                                 int page_block_size, int64_t kv_block_stride_bytes, int num_sm_parts,
                                 const int32_t* topk_length, int impl, int32_t* status, int slices, int64_t slice_stride,
                                 void* stream) {
    if (int e = check_attn_common(fn, q, kv, indices, o_part, lse_part, num_tokens, num_heads,
                                  topk, page_block_size, kv_block_stride_bytes, impl)) return e;
    if (!o_accum || !lse_accum || !sched_meta || !num_splits)
        return set_error(SMLA_E_NULL, "%s: null scratch or scheduler pointer", fn);
    if (!aligned16(o_accum)) return set_error(SMLA_E_ALIGN, "%s: o_accum not 16-byte aligned", fn);
    if (num_sm_parts < 1) return set_error(SMLA_E_SHAPE, "%s: num_sm_parts=%d", fn, num_sm_parts);
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.kv = (const uint8_t*)kv; p.indices = indices;
    p.o_accum = o_accum; p.lse_accum = lse_accum; p.out = nullptr; p.out_lse = nullptr;
    p.sched = (const SchedMeta*)sched_meta; p.num_splits = num_splits;
    p.topk_length = topk_length; p.status = status;
    p.num_tokens = num_tokens; p.num_heads = num_heads; p.topk = topk; p.num_parts = num_sm_parts;
    p.force_partial = 1;
    p.page_block_size = page_block_size; p.block_stride = kv_block_stride_bytes; p.sm_scale = sm_scale;
    const int e = (impl == SMLA_IMPL_SCALAR) ? launch_attn_scalar(p, (cudaStream_t)stream) : launch_attn_pair(p, (cudaStream_t)stream);
    if (e) return e;
    return launch_combine_f32(o_accum, lse_accum, o_part, lse_part, num_splits, num_tokens, num_heads, slices, slice_stride,
                              (cudaStream_t)stream);
}

int smla_decode_partial(const void* q, const void* kv, const int32_t* indices,
                        float* o_accum, float* lse_accum, float* o_part, float* lse_part,
                        const int32_t* sched_meta, const int32_t* num_splits,
                        int num_tokens, int num_heads, int topk, float sm_scale,
                        int page_block_size, int64_t kv_block_stride_bytes, int num_sm_parts,
                        const int32_t* topk_length, int impl, int32_t* status, void* stream) {
    return decode_partial_common("smla_decode_partial", q, kv, indices, o_accum, lse_accum, o_part, lse_part, sched_meta,
                                 num_splits, num_tokens, num_heads, topk, sm_scale, page_block_size, kv_block_stride_bytes,
                                 num_sm_parts, topk_length, impl, status, 1, 0, stream);
}

int smla_decode_partial_sliced(const void* q, const void* kv, const int32_t* indices,
                               float* o_accum, float* lse_accum, float* send, int slices, int64_t slice_stride,
                               const int32_t* sched_meta, const int32_t* num_splits,
                               int num_tokens, int num_heads, int topk, float sm_scale,
                               int page_block_size, int64_t kv_block_stride_bytes, int num_sm_parts,
                               const int32_t* topk_length, int impl, int32_t* status, void* stream) {
    if (slices < 1 || num_heads % (slices < 1 ? 1 : slices) != 0)
        return set_error(SMLA_E_SHAPE, "smla_decode_partial_sliced: %d heads do not divide into %d slices", num_heads, slices);
    const int64_t need = (int64_t)num_tokens * (num_heads / slices) * (D_V + 1);
    if (slice_stride < need || slice_stride % D_V != 0 || !aligned16(send))
        return set_error(SMLA_E_SHAPE, "smla_decode_partial_sliced: slice stride %lld must be a multiple of %d floats and hold %lld",
                         (long long)slice_stride, D_V, (long long)need);
    return decode_partial_common("smla_decode_partial_sliced", q, kv, indices, o_accum, lse_accum, send, send, sched_meta,
                                 num_splits, num_tokens, num_heads, topk, sm_scale, page_block_size, kv_block_stride_bytes,
                                 num_sm_parts, topk_length, impl, status, slices, slice_stride, stream);
}

int smla_cp_unslice(const void* gathered, void* out, float* lse, int slices, int num_tokens, int heads_per_slice,
                    int64_t chunk_bytes, void* stream) {
    if (!gathered || !out || !lse) return set_error(SMLA_E_NULL, "smla_cp_unslice: null pointer argument");
    if (slices < 1 || num_tokens < 0 || heads_per_slice < 1 ||
        chunk_bytes < (int64_t)num_tokens * heads_per_slice * (D_V * 2 + 4) || (chunk_bytes & 15))
        return set_error(SMLA_E_SHAPE, "smla_cp_unslice: slices=%d tokens=%d heads=%d chunk=%lld", slices, num_tokens,
                         heads_per_slice, (long long)chunk_bytes);
    if (!aligned16(gathered) || !aligned16(out)) return set_error(SMLA_E_ALIGN, "smla_cp_unslice: unaligned buffer");
    return launch_cp_unslice(gathered, (__nv_bfloat16*)out, lse, slices, num_tokens, heads_per_slice, chunk_bytes, (cudaStream_t)stream);
}

int smla_combine_parts(const float* o_parts, const float* lse_parts, void* out, float* out_lse,
                       int parts, int num_tokens, int num_heads, const float* attn_sink, void* stream) {
    if (!o_parts || !lse_parts || !out || !out_lse)
        return set_error(SMLA_E_NULL, "smla_combine_parts: null pointer argument");
    if (parts < 1 || num_tokens < 0 || num_heads < 1)
        return set_error(SMLA_E_SHAPE, "smla_combine_parts: parts=%d tokens=%d heads=%d", parts, num_tokens, num_heads);
    if (!aligned16(o_parts) || !aligned16(out)) return set_error(SMLA_E_ALIGN, "smla_combine_parts: unaligned buffer");
    return launch_combine_parts(o_parts, lse_parts, (__nv_bfloat16*)out, out_lse, parts, num_tokens, num_heads, 0, 0,
                                attn_sink, (cudaStream_t)stream);
}

int smla_combine_parts_strided(const float* o_parts, const float* lse_parts, void* out, float* out_lse,
                               int parts, int num_tokens, int num_heads, int64_t o_part_stride,
                               int64_t lse_part_stride, const float* attn_sink, void* stream) {
    if (!o_parts || !lse_parts || !out || !out_lse)
        return set_error(SMLA_E_NULL, "smla_combine_parts_strided: null pointer argument");
    if (parts < 1 || num_tokens < 0 || num_heads < 1 || o_part_stride < (int64_t)num_tokens * num_heads * 512 ||
        lse_part_stride < (int64_t)num_tokens * num_heads)
        return set_error(SMLA_E_SHAPE, "smla_combine_parts_strided: parts=%d tokens=%d heads=%d strides=%lld,%lld", parts,
                         num_tokens, num_heads, (long long)o_part_stride, (long long)lse_part_stride);
    if (!aligned16(o_parts) || !aligned16(out) || (o_part_stride % 4) != 0)
        return set_error(SMLA_E_ALIGN, "smla_combine_parts_strided: unaligned buffer or stride");
    return launch_combine_parts(o_parts, lse_parts, (__nv_bfloat16*)out, out_lse, parts, num_tokens, num_heads,
                                o_part_stride, lse_part_stride, attn_sink, (cudaStream_t)stream);
}

int smla_prefill(const void* q, const void* kv, const int32_t* indices,
                 void* out, float* out_lse, float* out_max_logits,
                 int num_tokens, int num_heads, int topk, float sm_scale,
                 int page_block_size, int64_t kv_block_stride_bytes,
                 const float* attn_sink, const int32_t* topk_length,
                 int impl, int32_t* status, void* stream) {
    if (int e = check_attn_common("smla_prefill", q, kv, indices, out, out_lse, num_tokens, num_heads, topk,
                                  page_block_size, kv_block_stride_bytes, impl)) return e;
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.kv = (const uint8_t*)kv; p.indices = indices;
    p.out = (__nv_bfloat16*)out; p.out_lse = out_lse; p.out_max_logits = out_max_logits;
    p.attn_sink = attn_sink; p.topk_length = topk_length; p.status = status;
    p.num_tokens = num_tokens; p.num_heads = num_heads; p.topk = topk; p.num_parts = num_tokens;
    p.page_block_size = page_block_size; p.block_stride = kv_block_stride_bytes; p.sm_scale = sm_scale;
    if (impl == SMLA_IMPL_SCALAR) return launch_attn_scalar(p, (cudaStream_t)stream);
    return launch_attn_pair(p, (cudaStream_t)stream);
}

static int check_ext(const char* fn, const void* q, const void* kv, const int32_t* indices, const void* extra_kv,
                     const int32_t* extra_indices, const void* out, const float* out_lse, int num_tokens, int num_heads,
                     int topk, int extra_topk, int layout, int page_block_size, int64_t stride,
                     int extra_page_block_size, int64_t extra_stride) {
    if (layout != SMLA_LAYOUT_V32 && layout != SMLA_LAYOUT_MODEL1)
        return set_error(SMLA_E_SHAPE, "%s: unknown cache layout %d", fn, layout);
    const int row = (layout == SMLA_LAYOUT_MODEL1) ? SMLA_M1_ROW_BYTES : ROW_BYTES;
    if (!q || !kv || !indices || !out || !out_lse) return set_error(SMLA_E_NULL, "%s: null pointer argument", fn);
    if (num_tokens < 0) return set_error(SMLA_E_SHAPE, "%s: num_tokens=%d", fn, num_tokens);
    if (num_heads < 1 || num_heads > 128)
        return set_error(SMLA_E_SHAPE, "%s: num_heads=%d, supported 1..128", fn, num_heads);
    if (topk < 1 || extra_topk < 0) return set_error(SMLA_E_SHAPE, "%s: topk=%d extra_topk=%d", fn, topk, extra_topk);
    if (page_block_size < 1) return set_error(SMLA_E_SHAPE, "%s: page_block_size=%d", fn, page_block_size);
    if (!aligned16(q) || !aligned16(out)) return set_error(SMLA_E_ALIGN, "%s: q and out must be 16-byte aligned", fn);
    if ((reinterpret_cast<uintptr_t>(kv) & 3u) || (stride & 3))
        return set_error(SMLA_E_ALIGN, "%s: kv and the page stride must be 4-byte aligned", fn);
    if (stride < (int64_t)page_block_size * row)
        return set_error(SMLA_E_SHAPE, "%s: page stride %lld smaller than %d rows of %d bytes", fn, (long long)stride,
                         page_block_size, row);
    if (extra_topk > 0) {
        if (!extra_kv || !extra_indices) return set_error(SMLA_E_NULL, "%s: extra_topk=%d without an extra cache or indices", fn, extra_topk);
        if (extra_page_block_size < 1 || extra_stride < (int64_t)extra_page_block_size * row)
            return set_error(SMLA_E_SHAPE, "%s: extra page of %d rows with stride %lld", fn, extra_page_block_size,
                             (long long)extra_stride);
        if ((reinterpret_cast<uintptr_t>(extra_kv) & 3u) || (extra_stride & 3))
            return set_error(SMLA_E_ALIGN, "%s: extra_kv and its page stride must be 4-byte aligned", fn);
    }
    return 0;
}

// impl AUTO: V32 (with a second cache) runs the tensor-core kernel when the caches are aligned for its bulk copies,
// else the fp32 kernel.  MODEL1 runs the fp32 kernel unless the tensor-core kernel is asked for by name: there V
// includes the row's RoPE, which the tensor-core kernel rounds to e4m3 like the rest of V, while the reference keeps
// it in bf16 (csrc/kernel/common/xv_rope_mma.cuh:23-93) and bounds the error of short rows in its own tests
// (tests/test_prefill.py:95-107, tests/test_v4_features.py:28-47) below what that rounding costs.
static int launch_ext(const char* fn, const AttnParams& p, int impl, cudaStream_t stream) {
    if (impl != SMLA_IMPL_AUTO && impl != SMLA_IMPL_SCALAR && impl != SMLA_IMPL_TC)
        return set_error(SMLA_E_SHAPE, "%s: unknown impl %d", fn, impl);
    if (impl == SMLA_IMPL_SCALAR || (impl == SMLA_IMPL_AUTO && p.layout == SMLA_LAYOUT_MODEL1))
        return launch_attn_scalar(p, stream);
    if (attn_pair_takes(p)) return launch_attn_pair(p, stream);
    if (impl == SMLA_IMPL_TC)
        return set_error(SMLA_E_ALIGN, "%s: the tensor-core kernel needs 16-byte aligned caches and page strides", fn);
    return launch_attn_scalar(p, stream);
}

int smla_decode_splitkv_ext(const void* q, const void* kv, const int32_t* indices,
                            const void* extra_kv, const int32_t* extra_indices,
                            float* o_accum, float* lse_accum, void* out, float* out_lse,
                            const int32_t* sched_meta, const int32_t* num_splits,
                            int num_tokens, int num_heads, int topk, int extra_topk, float sm_scale, int layout,
                            int page_block_size, int64_t kv_block_stride_bytes,
                            int extra_page_block_size, int64_t extra_block_stride_bytes, int num_sm_parts,
                            const float* attn_sink, const int32_t* topk_length, const int32_t* extra_topk_length,
                            int impl, int32_t* status, void* stream) {
    if (int e = check_ext("smla_decode_splitkv_ext", q, kv, indices, extra_kv, extra_indices, out, out_lse, num_tokens,
                          num_heads, topk, extra_topk, layout, page_block_size, kv_block_stride_bytes,
                          extra_page_block_size, extra_block_stride_bytes)) return e;
    if (!o_accum || !lse_accum || !sched_meta || !num_splits)
        return set_error(SMLA_E_NULL, "smla_decode_splitkv_ext: null scratch or scheduler pointer");
    if (num_sm_parts < 1) return set_error(SMLA_E_SHAPE, "smla_decode_splitkv_ext: num_sm_parts=%d", num_sm_parts);
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.kv = (const uint8_t*)kv; p.indices = indices;
    p.o_accum = o_accum; p.lse_accum = lse_accum; p.out = (__nv_bfloat16*)out; p.out_lse = out_lse;
    p.sched = (const SchedMeta*)sched_meta; p.num_splits = num_splits;
    p.attn_sink = attn_sink; p.topk_length = topk_length; p.status = status;
    p.num_tokens = num_tokens; p.num_heads = num_heads; p.topk = topk; p.num_parts = num_sm_parts;
    p.page_block_size = page_block_size; p.block_stride = kv_block_stride_bytes; p.sm_scale = sm_scale;
    p.layout = layout;
    if (extra_topk > 0) {
        p.extra_kv = (const uint8_t*)extra_kv; p.extra_indices = extra_indices; p.extra_topk_length = extra_topk_length;
        p.extra_topk = extra_topk; p.extra_page_block_size = extra_page_block_size;
        p.extra_block_stride = extra_block_stride_bytes;
    }
    return launch_ext("smla_decode_splitkv_ext", p, impl, (cudaStream_t)stream);
}

int smla_prefill_ext(const void* q, const void* kv, const int32_t* indices,
                     const void* extra_kv, const int32_t* extra_indices,
                     void* out, float* out_lse, float* out_max_logits,
                     int num_tokens, int num_heads, int topk, int extra_topk, float sm_scale, int layout,
                     int page_block_size, int64_t kv_block_stride_bytes,
                     int extra_page_block_size, int64_t extra_block_stride_bytes,
                     const float* attn_sink, const int32_t* topk_length, const int32_t* extra_topk_length,
                     int impl, int32_t* status, void* stream) {
    if (int e = check_ext("smla_prefill_ext", q, kv, indices, extra_kv, extra_indices, out, out_lse, num_tokens,
                          num_heads, topk, extra_topk, layout, page_block_size, kv_block_stride_bytes,
                          extra_page_block_size, extra_block_stride_bytes)) return e;
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.kv = (const uint8_t*)kv; p.indices = indices;
    p.out = (__nv_bfloat16*)out; p.out_lse = out_lse; p.out_max_logits = out_max_logits;
    p.attn_sink = attn_sink; p.topk_length = topk_length; p.status = status;
    p.num_tokens = num_tokens; p.num_heads = num_heads; p.topk = topk; p.num_parts = num_tokens;
    p.page_block_size = page_block_size; p.block_stride = kv_block_stride_bytes; p.sm_scale = sm_scale;
    p.layout = layout;
    if (extra_topk > 0) {
        p.extra_kv = (const uint8_t*)extra_kv; p.extra_indices = extra_indices; p.extra_topk_length = extra_topk_length;
        p.extra_topk = extra_topk; p.extra_page_block_size = extra_page_block_size;
        p.extra_block_stride = extra_block_stride_bytes;
    }
    return launch_ext("smla_prefill_ext", p, impl, (cudaStream_t)stream);
}

int smla_pack_kv(const void* kv_bf16, void* packed, int64_t num_rows, void* stream) {
    if (!kv_bf16 || !packed) return set_error(SMLA_E_NULL, "smla_pack_kv: null pointer argument");
    if (num_rows < 0) return set_error(SMLA_E_SHAPE, "smla_pack_kv: num_rows=%lld", (long long)num_rows);
    if (!aligned16(kv_bf16) || !aligned16(packed)) return set_error(SMLA_E_ALIGN, "smla_pack_kv: unaligned buffer");
    return launch_pack_kv((const __nv_bfloat16*)kv_bf16, (uint8_t*)packed, num_rows, (cudaStream_t)stream);
}

int smla_mqa_logits(const void* q, const void* k, const float* k_scale, const float* weights,
                    const int32_t* ks, const int32_t* ke, float* logits,
                    int s_q, int num_heads, int s_k, int64_t logits_stride,
                    int impl, int32_t* status, void* stream) {
    if (!q || !k || !k_scale || !weights || !ks || !ke || !logits)
        return set_error(SMLA_E_NULL, "smla_mqa_logits: null pointer argument");
    if (s_q < 0 || s_k < 0 || num_heads < 1 || num_heads > 64)
        return set_error(SMLA_E_SHAPE, "smla_mqa_logits: s_q=%d s_k=%d heads=%d (heads 1..64)", s_q, s_k, num_heads);
    if (logits_stride < s_k) return set_error(SMLA_E_SHAPE, "smla_mqa_logits: logits_stride < s_k");
    if (!aligned16(q) || !aligned16(k)) return set_error(SMLA_E_ALIGN, "smla_mqa_logits: q and k must be 16-byte aligned");
    if (impl == SMLA_IMPL_SCALAR)
        return launch_mqa_logits_scalar((const uint8_t*)q, (const uint8_t*)k, k_scale, weights, ks, ke, logits,
                                        s_q, num_heads, s_k, logits_stride, (cudaStream_t)stream);
    return launch_mqa_logits_tc((const uint8_t*)q, (const uint8_t*)k, k_scale, weights, ks, ke, logits, s_q,
                                num_heads, s_k, logits_stride, status, (cudaStream_t)stream);
}

int smla_topk(const float* logits, const int32_t* ks, const int32_t* ke, int32_t* out_indices,
              int num_rows, int num_cols, int64_t logits_stride, int k, void* stream) {
    if (!logits || !out_indices) return set_error(SMLA_E_NULL, "smla_topk: null pointer argument");
    if (num_rows < 0 || num_cols < 0 || k < 0 || logits_stride < num_cols)
        return set_error(SMLA_E_SHAPE, "smla_topk: rows=%d cols=%d k=%d stride=%lld", num_rows, num_cols, k,
                         (long long)logits_stride);
    return launch_topk(logits, ks, ke, out_indices, num_rows, num_cols, logits_stride, k, (cudaStream_t)stream);
}

int smla_cp_partition_indices(const int32_t* indices, int32_t* local_indices, int32_t* local_length,
                              int num_tokens, int topk, int lo, int hi, void* stream) {
    if (!indices || !local_indices || !local_length)
        return set_error(SMLA_E_NULL, "smla_cp_partition_indices: null pointer argument");
    if (num_tokens < 0 || topk < 0 || hi < lo)
        return set_error(SMLA_E_SHAPE, "smla_cp_partition_indices: tokens=%d topk=%d range=[%d,%d)", num_tokens,
                         topk, lo, hi);
    return launch_cp_partition(indices, local_indices, local_length, num_tokens, topk, lo, hi,
                               (cudaStream_t)stream);
}

int smla_cp_local_window(const int32_t* ks, const int32_t* ke, int32_t* ks_local, int32_t* ke_local, int num_tokens,
                         int lo, int hi, void* stream) {
    if (!ks || !ke || !ks_local || !ke_local) return set_error(SMLA_E_NULL, "smla_cp_local_window: null pointer argument");
    if (num_tokens < 0 || hi < lo) return set_error(SMLA_E_SHAPE, "smla_cp_local_window: tokens=%d range=[%d,%d)", num_tokens, lo, hi);
    return launch_cp_window(ks, ke, ks_local, ke_local, num_tokens, lo, hi, (cudaStream_t)stream);
}

int smla_cp_candidates(const float* logits, int64_t logits_stride, const int32_t* picked, float* values,
                       int32_t* positions, int num_tokens, int k, int lo, void* stream) {
    if (!logits || !picked || !values || !positions) return set_error(SMLA_E_NULL, "smla_cp_candidates: null pointer argument");
    if (num_tokens < 0 || k < 0) return set_error(SMLA_E_SHAPE, "smla_cp_candidates: tokens=%d k=%d", num_tokens, k);
    return launch_cp_candidates(logits, logits_stride, picked, values, positions, num_tokens, k, lo, (cudaStream_t)stream);
}

int smla_cp_interleave_candidates(const int32_t* gathered, float* values, int32_t* positions, int world, int num_tokens,
                                  int k, void* stream) {
    if (!gathered || !values || !positions) return set_error(SMLA_E_NULL, "smla_cp_interleave_candidates: null pointer argument");
    if (world < 1 || num_tokens < 0 || k < 0)
        return set_error(SMLA_E_SHAPE, "smla_cp_interleave_candidates: world=%d tokens=%d k=%d", world, num_tokens, k);
    return launch_cp_interleave(gathered, reinterpret_cast<int32_t*>(values), positions, world, num_tokens, k, (cudaStream_t)stream);
}

int smla_cp_pick_positions(const int32_t* positions, const int32_t* pick, int32_t* out, int num_tokens, int k,
                           int num_candidates, void* stream) {
    if (!positions || !pick || !out) return set_error(SMLA_E_NULL, "smla_cp_pick_positions: null pointer argument");
    if (num_tokens < 0 || k < 0 || num_candidates < 0)
        return set_error(SMLA_E_SHAPE, "smla_cp_pick_positions: tokens=%d k=%d candidates=%d", num_tokens, k, num_candidates);
    return launch_cp_pick(positions, pick, out, num_tokens, k, num_candidates, (cudaStream_t)stream);
}

}  // extern "C"
