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
template <typename OutT>
__global__ void __launch_bounds__(WARPS * 32)
combine_kernel(const float* __restrict__ o_accum, const float* __restrict__ lse_accum,
               OutT* __restrict__ out, float* __restrict__ out_lse,
               const int32_t* __restrict__ num_splits, const float* __restrict__ attn_sink,
               int batch, int num_heads, int fixed_ns, int64_t part_stride_o, int64_t part_stride_l) {
    constexpr bool F32 = sizeof(OutT) == 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * WARPS + warp;   // (token, head)
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
    const float* o_p = o_accum + (size_t)s0 * num_heads * D_V + (size_t)h * D_V + lane * 4;

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
    if (lane == 0) out_lse[row] = lse;

    float4 acc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    int s = 0;
    for (; s + 1 < ns; s += 2) {
        float4 a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            a[i] = __ldcs(reinterpret_cast<const float4*>(o_p + (size_t)s * o_stride + i * 128));
            b[i] = __ldcs(reinterpret_cast<const float4*>(o_p + (size_t)(s + 1) * o_stride + i * 128));
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
            const float4 a = __ldcs(reinterpret_cast<const float4*>(o_p + (size_t)s * o_stride + i * 128));
            acc[i].x += wa * a.x; acc[i].y += wa * a.y; acc[i].z += wa * a.z; acc[i].w += wa * a.w;
        }
    }
    if constexpr (F32) {
        float* o_out = reinterpret_cast<float*>(out) + (size_t)row * D_V + lane * 4;
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
    combine_kernel<__nv_bfloat16><<<grid, WARPS * 32, 0, stream>>>(o_accum, lse_accum, out, out_lse, num_splits,
                                                                    attn_sink, batch, num_heads, 0, 0, 0);
    return check_launch("combine_kernel");
}

// Local merge for the context-parallel path: every token (also those with one split) to fp32.
int launch_combine_f32(const float* o_accum, const float* lse_accum, float* out, float* out_lse,
                       const int32_t* num_splits, int batch, int num_heads, cudaStream_t stream) {
    const int64_t rows = (int64_t)batch * num_heads;
    if (rows == 0) return 0;
    const unsigned grid = (unsigned)((rows + WARPS - 1) / WARPS);
    combine_kernel<float><<<grid, WARPS * 32, 0, stream>>>(o_accum, lse_accum, out, out_lse, num_splits, nullptr,
                                                            batch, num_heads, 0, 0, 0);
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
    combine_kernel<__nv_bfloat16><<<grid, WARPS * 32, 0, stream>>>(o_parts, lse_parts, out, out_lse, nullptr,
                                                                    attn_sink, batch, num_heads, parts, part_stride_o,
                                                                    part_stride_l);
    return check_launch("combine_kernel<parts>");
}

}  // namespace smla
