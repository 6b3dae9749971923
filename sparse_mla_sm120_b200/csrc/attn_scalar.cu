// fp32 CUDA-core sparse-MLA attention (decode with split-KV, and prefill).
//
// This kernel is the slow, exact member of the family: it dequantises every gathered row to
// fp32 (fp8 * power-of-two scale is exact), takes fp32 dot products and keeps fp32 softmax
// state.  It exists as an on-device second opinion for the tensor-core kernel and serves head
// counts or top-k sizes the tensor-core kernel does not take.  Work decomposition, masking and
// the split / no-split epilogue follow the reference decode kernel
// (csrc/kernel/decode/decode_v2_kernel.cuh:104-133 for the partition walk, :346-362 for
// masking, :529-648 for the two epilogues).
//
// One CTA = (8 heads, one scheduler partition).  Per 64-token block it walks 8 sub-tiles of
// 8 tokens: dequantise 8 rows to shared memory, 64 dot products of length 576 (4 threads each),
// online softmax per head, then P.V with one thread per (head, 16 output dims).
//
// It is also the kernel that serves the second cache layout and the second ("extra") cache:
//  * layout MODEL1 (csrc/model/kv_cache_traits.cuh:61-111): a page of `block` tokens is
//    block x 576 data bytes (448 e4m3 + 64 bf16 RoPE per token) followed by a footer of
//    block x 8 bytes (7 UE8M0 scales, one per 64 values, + 1 pad); q has 512 dims and V is the
//    whole dequantised row, RoPE included.
//  * extra cache (decode_v2_kernel.cuh:109-115, 147-160, 351-361): after the
//    max(ceil(topk_length/64),1) blocks of the main cache a request walks
//    ceil(extra_topk_length/64) blocks whose rows come from a second cache through a second
//    index array; the softmax runs over both.
#include "common.cuh"

namespace smla {

namespace {

constexpr int HT = 8;        // heads per CTA
constexpr int ST = 8;        // tokens per sub-tile
constexpr int THREADS = 256;
constexpr int KPAD = D_QK + 1;

constexpr int M1_NOPE = 448;       // MODEL1: e4m3 values per row
constexpr int M1_DATA = 576;       // MODEL1: data bytes per token (448 + 64 bf16)
constexpr int M1_SCALE_BYTES = 8;  // MODEL1: footer bytes per token

// Dequantise one gathered row into `dst` (fp32), one warp per row.  The reference rounds the
// dequantised value to bf16 (tests/test_decode.py:66-69, :139-141), exact for power-of-two scales.
template <int LAYOUT>
__device__ __forceinline__ void load_row(float* dst, const uint8_t* kv, int idx, int page_block_size,
                                         int64_t block_stride, int lane) {
    if (LAYOUT == SMLA_LAYOUT_V32) {
        const uint8_t* row = kv_row_ptr(kv, idx, page_block_size, block_stride);
        const float* sc = reinterpret_cast<const float*>(row + SCALE_OFF);
        for (int d = lane; d < D_NOPE; d += 32)
            dst[d] = __bfloat162float(__float2bfloat16(e4m3_to_float(row[d]) * sc[d >> 7]));
        const __nv_bfloat16* rope = reinterpret_cast<const __nv_bfloat16*>(row + ROPE_OFF);
        for (int d = lane; d < D_ROPE; d += 32) dst[D_NOPE + d] = __bfloat162float(rope[d]);
    } else {
        const unsigned u = (unsigned)idx;
        const unsigned blk = u / (unsigned)page_block_size;
        const unsigned in = u - blk * (unsigned)page_block_size;
        const uint8_t* page = kv + (int64_t)blk * block_stride;
        const uint8_t* row = page + (int64_t)in * M1_DATA;
        const uint8_t* sc = page + (int64_t)page_block_size * M1_DATA + (int64_t)in * M1_SCALE_BYTES;
        for (int d = lane; d < M1_NOPE; d += 32) {
            const uint32_t e = sc[d >> 6];                       // UE8M0: 2^(e-127)
            const float scale = __uint_as_float(e ? (e << 23) : 0x00400000u);
            dst[d] = __bfloat162float(__float2bfloat16(e4m3_to_float(row[d]) * scale));
        }
        const __nv_bfloat16* rope = reinterpret_cast<const __nv_bfloat16*>(row + M1_NOPE);
        for (int d = lane; d < D_ROPE; d += 32) dst[M1_NOPE + d] = __bfloat162float(rope[d]);
    }
}

template <int LAYOUT>
__global__ void __launch_bounds__(THREADS) attn_scalar_kernel(const AttnParams p) {
    constexpr int DQ = (LAYOUT == SMLA_LAYOUT_V32) ? D_QK : 512;   // q / K row length
    __shared__ float qs[HT][D_QK];
    __shared__ float ks[ST][KPAD];
    __shared__ float ps[HT][ST];
    __shared__ float m_s[HT], l_s[HT], alpha_s[HT];
    __shared__ int valid_s[ST];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h0 = blockIdx.y * HT;
    const int part = blockIdx.x;
    const float scale2 = p.sm_scale * LOG2E;

    SchedMeta meta;
    if (p.sched != nullptr) {
        grid_dep_wait();
        meta = p.sched[part];
    } else {  // one partition per token, whole request, never split
        meta.begin_req = meta.end_req = part;
        meta.begin_block = 0; meta.end_block = 0x7fffffff;
        meta.begin_split = 0; meta.first_split = meta.last_split = 0;
    }

    for (int req = meta.begin_req; req <= meta.end_req && req < p.num_tokens; ++req) {
        int len = p.topk_length ? p.topk_length[req] : p.topk;
        len = min(len, p.topk);
        const int main_blocks = max((len + BLOCK_N - 1) / BLOCK_N, 1);
        int extra_len = 0;
        if (p.extra_topk > 0) {
            extra_len = p.extra_topk_length ? p.extra_topk_length[req] : p.extra_topk;
            extra_len = max(min(extra_len, p.extra_topk), 0);
        }
        const int total_blocks = main_blocks + (extra_len + BLOCK_N - 1) / BLOCK_N;
        const int blk0 = (req == meta.begin_req) ? meta.begin_block : 0;
        const int blk1 = min((req == meta.end_req) ? meta.end_block : total_blocks, total_blocks);
        if (blk1 - blk0 <= 0) continue;
        const bool no_split = !p.force_partial && ((req == meta.begin_req) ? !meta.first_split
                              : ((req == meta.end_req) ? !meta.last_split : true));
        const int split_idx = p.num_splits ? p.num_splits[req] + ((req == meta.begin_req) ? meta.begin_split : 0) : 0;

        __syncthreads();  // previous request's epilogue has finished with shared state
        for (int i = tid; i < HT * DQ; i += THREADS) {
            const int h = i / DQ, d = i - h * DQ;
            qs[h][d] = (h0 + h < p.num_heads)
                           ? __bfloat162float(p.q[((size_t)req * p.num_heads + h0 + h) * DQ + d]) : 0.f;
        }
        if (tid < HT) { m_s[tid] = NEG_BIG; l_s[tid] = 0.f; }
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
        const int32_t* idx_row = p.indices + (size_t)req * p.topk;
        const int32_t* extra_idx_row = p.extra_topk > 0 ? p.extra_indices + (size_t)req * p.extra_topk : nullptr;
        const int main_end = main_blocks * BLOCK_N;   // positions from here on belong to the extra cache

        for (int pos0 = blk0 * BLOCK_N; pos0 < blk1 * BLOCK_N; pos0 += ST) {
            __syncthreads();
            // gather + dequantise ST rows: 32 threads per row
            {
                const int r = warp;  // THREADS/32 == ST
                const int pos = pos0 + r;
                int idx = -1;
                const bool from_extra = pos >= main_end;
                if (!from_extra) {
                    if (pos < len) idx = idx_row[pos];
                } else if (pos - main_end < extra_len) {
                    idx = extra_idx_row[pos - main_end];
                }
                if (lane == 0) valid_s[r] = (idx >= 0);
                if (idx >= 0) {
                    if (!from_extra) load_row<LAYOUT>(ks[r], p.kv, idx, p.page_block_size, p.block_stride, lane);
                    else load_row<LAYOUT>(ks[r], p.extra_kv, idx, p.extra_page_block_size, p.extra_block_stride, lane);
                } else {
                    for (int d = lane; d < DQ; d += 32) ks[r][d] = 0.f;  // exact zero: no 0*NaN in P.V
                }
            }
            __syncthreads();
            // 64 dot products, 4 threads each (interleaved so that the 4 partners share a quad)
            {
                const int pair = tid >> 2, part4 = tid & 3;
                const int h = pair / ST, t = pair % ST;
                float s = 0.f;
                for (int d = part4; d < DQ; d += 4) s += qs[h][d] * ks[t][d];
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if (part4 == 0) ps[h][t] = valid_s[t] ? s * scale2 : NEG_BIG;
            }
            __syncthreads();
            if (tid < HT) {
                const int h = tid;
                float mx = m_s[h];
                for (int t = 0; t < ST; ++t) if (valid_s[t]) mx = fmaxf(mx, ps[h][t]);
                const float alpha = exp2f(m_s[h] - mx);   // 1 when nothing changed (also -1e30 - -1e30)
                float sum = 0.f;
                for (int t = 0; t < ST; ++t) {
                    const float w = valid_s[t] ? exp2f(ps[h][t] - mx) : 0.f;
                    ps[h][t] = w;
                    sum += w;
                }
                m_s[h] = mx;
                l_s[h] = l_s[h] * alpha + sum;
                alpha_s[h] = alpha;
            }
            __syncthreads();
            {
                const int h = warp;  // HT == 8 warps
                const float alpha = alpha_s[h];
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] *= alpha;
                for (int t = 0; t < ST; ++t) {
                    const float w = ps[h][t];
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[j] += w * ks[t][lane + 32 * j];
                }
            }
        }
        __syncthreads();
        // epilogue
        const int h = warp;
        if (h0 + h < p.num_heads) {
            const float m = m_s[h], l = l_s[h];
            float lse = (l > 0.f) ? (log2f(l) + m) : NEG_BIG;
            if (no_split) {
                float denom = l;
                if (p.attn_sink != nullptr) {
                    const float sink2 = p.attn_sink[h0 + h] * LOG2E;
                    denom = l + exp2f(sink2 - m);
                    if (lse != NEG_BIG) lse += log2f(1.f + exp2f(sink2 - lse));
                    else lse = sink2;
                }
                const float inv = (denom > 0.f) ? 1.f / denom : 0.f;
                __nv_bfloat16* o = p.out + ((size_t)req * p.num_heads + h0 + h) * D_V;
#pragma unroll
                for (int j = 0; j < 16; ++j) o[lane + 32 * j] = __float2bfloat16(acc[j] * inv);
                if (lane == 0) {
                    p.out_lse[(size_t)req * p.num_heads + h0 + h] = lse;
                    if (p.out_max_logits) p.out_max_logits[(size_t)req * p.num_heads + h0 + h] = m;
                }
            } else {
                const float inv = (l > 0.f) ? 1.f / l : 0.f;
                float* o = p.o_accum + ((size_t)split_idx * p.num_heads + h0 + h) * D_V;
#pragma unroll
                for (int j = 0; j < 16; ++j) o[lane + 32 * j] = acc[j] * inv;
                if (lane == 0) p.lse_accum[(size_t)split_idx * p.num_heads + h0 + h] = lse;
            }
        }
    }
}

}  // namespace

int launch_attn_scalar(const AttnParams& p, cudaStream_t stream) {
    if (p.num_tokens == 0) return 0;
    const int parts = p.sched ? p.num_parts : p.num_tokens;
    dim3 grid(parts, (p.num_heads + HT - 1) / HT);
    if (p.layout == SMLA_LAYOUT_MODEL1) attn_scalar_kernel<SMLA_LAYOUT_MODEL1><<<grid, THREADS, 0, stream>>>(p);
    else attn_scalar_kernel<SMLA_LAYOUT_V32><<<grid, THREADS, 0, stream>>>(p);
    return check_launch("attn_scalar_kernel");
}

}  // namespace smla
