// Split-KV decode for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand it scratch memory: a serving process that gave
// every byte of the device to its own memory pool at start-up, or a call site in which entering
// the CUDA allocator is off limits because cudaMalloc may synchronise the whole device.  For
// them this entry point keeps the scratch of the split-KV decode (partial outputs, partial LSEs,
// scheduler records, split prefix sums) in a fixed array that is part of the library image: every
// GPU that loads the library holds SMLA_NOALLOC_SCRATCH_BYTES of it until the process exits.
//
// The array's name is only a stand-in on the host; the device address is looked up with
// cudaGetSymbolAddress once per device, on the first call made with that device current.  That
// first call does the lookup and should therefore be made before any stream capture starts.
// All calls share the one array and it keeps the last call's contents: nothing in it needs to
// start at zero (the scheduler rewrites its records and the decode kernel writes every partial
// the combine reads), but two calls that overlap on the GPU race on it.
#include "common.cuh"

namespace smla {

namespace {

constexpr size_t SCRATCH_BYTES = SMLA_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[SCRATCH_BYTES];

// Device address of the array, per device (0 = not looked up yet).
unsigned char* g_scratch_ptr[64] = {};

int scratch_for_current_device(unsigned char** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error((int)e, "smla_decode_splitkv_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return set_error(SMLA_E_SHAPE, "smla_decode_splitkv_noalloc: device ordinal %d not supported", dev);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return set_error(e == cudaSuccess ? SMLA_E_DEVICE : (int)e,
                             "smla_decode_splitkv_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_ptr[dev];
    return 0;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

}  // namespace smla

using namespace smla;

extern "C" size_t smla_noalloc_scratch_need(int num_tokens, int num_heads, int num_sm_parts) {
    const size_t records = (size_t)num_tokens + (size_t)num_sm_parts;
    return align_up(records * num_heads * D_V * sizeof(float), 256) + align_up(records * num_heads * sizeof(float), 256) +
           align_up((size_t)num_sm_parts * sizeof(SchedMeta), 256) + align_up(((size_t)num_tokens + 1) * sizeof(int32_t), 256);
}

extern "C" int smla_decode_splitkv_noalloc(const void* q, const void* kv, const int32_t* indices,
                                           void* out, float* out_lse,
                                           int num_tokens, int num_heads, int topk, float sm_scale,
                                           int page_block_size, int64_t kv_block_stride_bytes, int num_sm_parts,
                                           const float* attn_sink, const int32_t* topk_length,
                                           int impl, int32_t* status, void* stream) {
    // every check of the attention call comes first: a refused call launches nothing, the scheduler included
    if (int e = check_attn_common("smla_decode_splitkv_noalloc", q, kv, indices, out, out_lse, num_tokens, num_heads, topk,
                                  page_block_size, kv_block_stride_bytes, impl)) return e;
    if (num_tokens < 1 || num_tokens > 8192 || num_heads < 1 || num_heads > 128 || topk < 1 || num_sm_parts < 1 ||
        page_block_size < 1)
        return set_error(SMLA_E_SHAPE, "smla_decode_splitkv_noalloc: tokens=%d heads=%d topk=%d parts=%d page=%d",
                         num_tokens, num_heads, topk, num_sm_parts, page_block_size);
    const size_t need = smla_noalloc_scratch_need(num_tokens, num_heads, num_sm_parts);
    if (need > SCRATCH_BYTES)
        return set_error(SMLA_E_WORKSPACE,
                         "smla_decode_splitkv_noalloc: %d tokens + %d partitions x %d heads need %zu bytes of scratch, the "
                         "built-in array has %zu; use smla_decode_splitkv with caller-owned scratch",
                         num_tokens, num_sm_parts, num_heads, need, SCRATCH_BYTES);
    unsigned char* base = nullptr;
    if (int e = scratch_for_current_device(&base)) return e;

    const size_t records = (size_t)num_tokens + (size_t)num_sm_parts;
    float* o_accum = reinterpret_cast<float*>(base);
    size_t off = align_up(records * num_heads * D_V * sizeof(float), 256);
    float* lse_accum = reinterpret_cast<float*>(base + off);
    off += align_up(records * num_heads * sizeof(float), 256);
    int32_t* sched_meta = reinterpret_cast<int32_t*>(base + off);
    off += align_up((size_t)num_sm_parts * sizeof(SchedMeta), 256);
    int32_t* num_splits = reinterpret_cast<int32_t*>(base + off);

    if (int e = smla_sched_meta(num_tokens, topk, 0, num_sm_parts, 5, topk_length, nullptr, sched_meta, num_splits, stream))
        return e;
    if (int e = smla_decode_splitkv(q, kv, indices, o_accum, lse_accum, out, out_lse, sched_meta, num_splits, num_tokens,
                                    num_heads, topk, sm_scale, page_block_size, kv_block_stride_bytes, num_sm_parts,
                                    attn_sink, topk_length, impl, status, stream))
        return e;
    const int max_nsplits = (topk + BLOCK_N - 1) / BLOCK_N < num_sm_parts ? (topk + BLOCK_N - 1) / BLOCK_N : num_sm_parts;
    return smla_combine(o_accum, lse_accum, out, out_lse, num_splits, num_tokens, num_heads, max_nsplits, attn_sink, stream);
}
