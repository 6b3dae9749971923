// LSE-weighted merge of split-KV (or context-parallel) partial outputs.
//
// Semantics follow the reference combine kernel (csrc/kernel/combine/combine_kernel.cu:39-159):
// base-2 LSE, partials already normalised by their own row sum, requests with <= 1 split are
// left untouched (the decode kernel wrote their bf16 output directly), optional per-head sink
// folded into the merged LSE.  The kernel is HBM-bound: it reads splits * 2 KB per (token, head)
// and writes 1 KB.  One warp owns one (token, head) row, 16 floats per lane per split as four
// 16-byte loads, two splits in flight per iteration.
#include "common.cuh"

namespace smla {

namespace {

constexpr int WARPS = 8;

// Two addressing modes.  Packed (num_splits != null): the splits of token t are the consecutive
// records [num_splits[t], num_splits[t+1]) of o_accum [S, H, 512]; tokens with <= 1 split are
// skipped unless OutT is float (then the single record is passed through).  Strided
// (num_splits == null): every token has fixed_ns parts and part g of token t is record
// g * batch + t, the layout an all-gather of per-GPU [T, H, 512] partials produces.
// Four consecutive values of a partial record as fp32 (records are fp32, or fp16 where the attention kernel wrote them so).
__device__ __forceinline__ float4 load4(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4(const __half* p) {
    const uint2 v = __ldcs(reinterpret_cast<const uint2*>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename OutT, typename InT = float>
__global__ void __launch_bounds__(WARPS * 32)
combine_kernel(const InT* __restrict__ o_accum, const float* __restrict__ lse_accum,
               OutT* __restrict__ out, float* __restrict__ out_lse,
               const int32_t* __restrict__ num_splits, const float* __restrict__ attn_sink,
               int batch, int num_heads, int fixed_ns, int64_t part_stride_o, int64_t part_stride_l,
               int out_slices, int64_t out_slice_stride) {
    constexpr bool F32 = sizeof(OutT) == 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * WARPS + warp;   // (token, head)
    grid_dep_wait();      // the partials of the attention kernel before this one are complete
    if (row >= (int64_t)batch * num_heads) return;
    const int tok = (int)(row / num_heads), h = (int)(row % num_heads);
    int s0, ns;
    size_t rec_stride;   // records between consecutive splits of one token
    if (num_splits != nullptr) {
        s0 = num_splits[tok];
        ns = num_splits[tok + 1] - s0;
        rec_stride = 1;
        if (ns <= (F32 ? 0 : 1)) return;
    } else {
        s0 = tok; ns = fixed_ns; rec_stride = (size_t)batch;
    }

    // strided mode may give the distance (in floats) between the parts explicitly: partials and
    // LSEs of a rank then share one buffer, as one all-gather leaves them
    const size_t o_stride = (num_splits == nullptr && part_stride_o > 0) ? (size_t)part_stride_o : rec_stride * num_heads * D_V;
    const size_t l_stride = (num_splits == nullptr && part_stride_l > 0) ? (size_t)part_stride_l : rec_stride * num_heads;
    const float* lse_p = lse_accum + (size_t)s0 * num_heads + h;
    const InT* o_p = o_accum + (size_t)s0 * num_heads * D_V + (size_t)h * D_V + lane * 4;

    float mx = NEG_BIG;
    for (int s = lane; s < ns; s += 32) mx = fmaxf(mx, lse_p[(size_t)s * l_stride]);
    mx = warp_max(mx);
    if (mx == NEG_BIG) mx = 0.f;
    float sum = 0.f;
    for (int s = lane; s < ns; s += 32) sum += exp2f(lse_p[(size_t)s * l_stride] - mx);
    sum = warp_sum(sum);
    float lse = (sum > 0.f) ? (log2f(sum) + mx) : NEG_BIG;
    // Weights are taken against the sink-free LSE; the sink then only scales the result.
    const float lse_w = lse;
    float sink_scale = 1.f;
    if (attn_sink != nullptr) {
        const float sink2 = attn_sink[h] * LOG2E;
        if (lse != NEG_BIG) {
            const float t = exp2f(sink2 - lse);
            sink_scale = 1.f / (1.f + t);
            lse += log2f(1.f + t);
        } else {
            lse = sink2;
        }
    }
    // fp32 output cut into head slices (one per destination rank of an all-to-all): slice d holds
    // [batch, num_heads / out_slices, 512] partials followed by its [batch, num_heads / out_slices] LSEs
    size_t out_row = (size_t)row;
    float* lse_dst = out_lse + row;
    if (F32 && out_slices > 1) {
        const int hs = num_heads / out_slices, d = h / hs;
        out_row = (size_t)tok * hs + (h - d * hs);
        lse_dst = reinterpret_cast<float*>(out) + (size_t)d * out_slice_stride + (size_t)batch * hs * D_V + out_row;
        out_row += (size_t)d * out_slice_stride / D_V;      // out_slice_stride is a multiple of D_V floats
    }
    if (lane == 0) *lse_dst = lse;

    float4 acc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    int s = 0;
    for (; s + 1 < ns; s += 2) {
        float4 a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            a[i] = load4(o_p + (size_t)s * o_stride + i * 128);
            b[i] = load4(o_p + (size_t)(s + 1) * o_stride + i * 128);
        }
        const float wa = exp2f(lse_p[(size_t)s * l_stride] - lse_w) * sink_scale;
        const float wb = exp2f(lse_p[(size_t)(s + 1) * l_stride] - lse_w) * sink_scale;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[i].x += wa * a[i].x + wb * b[i].x;
            acc[i].y += wa * a[i].y + wb * b[i].y;
            acc[i].z += wa * a[i].z + wb * b[i].z;
            acc[i].w += wa * a[i].w + wb * b[i].w;
        }
    }
    if (s < ns) {
        const float wa = exp2f(lse_p[(size_t)s * l_stride] - lse_w) * sink_scale;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 a = load4(o_p + (size_t)s * o_stride + i * 128);
            acc[i].x += wa * a.x; acc[i].y += wa * a.y; acc[i].z += wa * a.z; acc[i].w += wa * a.w;
        }
    }
    if constexpr (F32) {
        float* o_out = reinterpret_cast<float*>(out) + out_row * D_V + lane * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(o_out + i * 128) = acc[i];
        return;
    }
    __nv_bfloat16* o_out = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * D_V + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i].x, acc[i].y);
        __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i].z, acc[i].w);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t*>(&lo);
        v.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(o_out + i * 128) = v;
    }
}

}  // namespace

int launch_combine(const float* o_accum, const float* lse_accum, __nv_bfloat16* out, float* out_lse,
                   const int32_t* num_splits, int batch, int num_heads, int max_nsplits,
                   const float* attn_sink, cudaStream_t stream) {
    (void)max_nsplits;
    const int64_t rows = (int64_t)batch * num_heads;
    if (rows == 0) return 0;
    const unsigned grid = (unsigned)((rows + WARPS - 1) / WARPS);
    launch_dependent(combine_kernel<__nv_bfloat16>, dim3(grid), dim3(WARPS * 32), 0, stream, o_accum, lse_accum, out, out_lse, num_splits,
                                                                    attn_sink, batch, num_heads, 0, 0, 0, 1, 0);
    return check_launch("combine_kernel");
}

// Local merge for the context-parallel path: every token (also those with one split) to fp32.
// With out_slices > 1 the result is written as `out_slices` head slices, slice d at out + d * out_slice_stride
// floats: [batch, num_heads / out_slices, 512] partials, then the slice's LSEs (out_lse is not used).
int launch_combine_f32(const float* o_accum, const float* lse_accum, float* out, float* out_lse,
                       const int32_t* num_splits, int batch, int num_heads, int out_slices, int64_t out_slice_stride,
                       cudaStream_t stream) {
    const int64_t rows = (int64_t)batch * num_heads;
    if (rows == 0) return 0;
    const unsigned grid = (unsigned)((rows + WARPS - 1) / WARPS);
    launch_dependent(combine_kernel<float>, dim3(grid), dim3(WARPS * 32), 0, stream, o_accum, lse_accum, out, out_lse, num_splits, nullptr,
                                                            batch, num_heads, 0, 0, 0, out_slices, out_slice_stride);
    return check_launch("combine_kernel<f32>");
}

// Merge of `parts` per-GPU partials laid out [parts, batch, H, 512] / [parts, batch, H]; non-zero
// part strides (in floats) give the distance between two ranks' partials / LSEs explicitly.
int launch_combine_parts(const float* o_parts, const float* lse_parts, __nv_bfloat16* out, float* out_lse,
                         int parts, int batch, int num_heads, int64_t part_stride_o, int64_t part_stride_l,
                         const float* attn_sink, cudaStream_t stream) {
    const int64_t rows = (int64_t)batch * num_heads;
    if (rows == 0) return 0;
    const unsigned grid = (unsigned)((rows + WARPS - 1) / WARPS);
    launch_dependent(combine_kernel<__nv_bfloat16>, dim3(grid), dim3(WARPS * 32), 0, stream, o_parts, lse_parts, out, out_lse, nullptr,
                                                                    attn_sink, batch, num_heads, parts, part_stride_o,
                                                                    part_stride_l, 1, 0);
    return check_launch("combine_kernel<parts>");
}

// The same merge over fp16 records (what the attention kernel writes when it derives a uniform split itself).
int launch_combine_parts_f16(const void* o_parts, const float* lse_parts, __nv_bfloat16* out, float* out_lse,
                             int parts, int batch, int num_heads, const float* attn_sink, cudaStream_t stream) {
    const int64_t rows = (int64_t)batch * num_heads;
    if (rows == 0) return 0;
    const unsigned grid = (unsigned)((rows + WARPS - 1) / WARPS);
    launch_dependent(combine_kernel<__nv_bfloat16, __half>, dim3(grid), dim3(WARPS * 32), 0, stream,
                     reinterpret_cast<const __half*>(o_parts), lse_parts, out, out_lse, nullptr, attn_sink, batch, num_heads, parts,
                     0, 0, 1, 0);
    return check_launch("combine_kernel<parts, f16>");
}

namespace {
// gathered: `slices` chunks of `chunk_bytes`, chunk g = [num_tokens, hs, 512] bf16 followed by [num_tokens, hs] fp32
// (the merged output of head slice g and its LSEs) -> out [num_tokens, slices * hs, 512] bf16, lse [num_tokens, slices * hs].
__global__ void cp_unslice_kernel(const uint8_t* __restrict__ gathered, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                                  int slices, int num_tokens, int hs, int64_t chunk_bytes) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;      // one 16-byte piece of the output
    const int64_t pieces = (int64_t)num_tokens * slices * hs * (D_V / 8);
    if (i < pieces) {
        const int c = (int)(i % (D_V / 8));
        const int64_t row = i / (D_V / 8);                                 // (token, head)
        const int h = (int)(row % ((int64_t)slices * hs)), t = (int)(row / ((int64_t)slices * hs));
        const int g = h / hs, hh = h - g * hs;
        const uint4 v = *reinterpret_cast<const uint4*>(gathered + (size_t)g * chunk_bytes + ((size_t)t * hs + hh) * (D_V * 2) + c * 16);
        *reinterpret_cast<uint4*>(out + (size_t)row * D_V + c * 8) = v;
        if (c == 0)
            lse[row] = *reinterpret_cast<const float*>(gathered + (size_t)g * chunk_bytes + (size_t)num_tokens * hs * (D_V * 2) +
                                                       ((size_t)t * hs + hh) * 4);
    }
}
}  // namespace

int launch_cp_unslice(const void* gathered, __nv_bfloat16* out, float* lse, int slices, int num_tokens, int hs,
                      int64_t chunk_bytes, cudaStream_t stream) {
    const int64_t pieces = (int64_t)num_tokens * slices * hs * (D_V / 8);
    if (pieces == 0) return 0;
    cp_unslice_kernel<<<(unsigned)((pieces + 255) / 256), 256, 0, stream>>>((const uint8_t*)gathered, out, lse, slices, num_tokens, hs,
                                                                           chunk_bytes);
    return check_launch("cp_unslice_kernel");
}

}  // namespace smla
