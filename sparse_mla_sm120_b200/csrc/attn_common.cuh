// Device helpers shared by the tensor-core attention kernels: a partition's work list, power-of-two
// scale arithmetic and e4m3 / bf16 packing.
#pragma once

#include "common.cuh"

namespace smla {
namespace attn {

struct Work {   // one request's share of a partition
    int req, blk0, nblk, len, split_idx;
    int main_blocks, extra_len;   // blocks [0, main_blocks) of a request walk the main cache, the rest the second ("extra") cache
    bool no_split;
};

__device__ __forceinline__ SchedMeta load_meta(const AttnParams& p, int part) {
    SchedMeta m;
    if (p.sched != nullptr) {
        m = p.sched[part];
    } else if (p.uniform_k > 1) {
        // no scheduler, requests of equal length: pair `part` owns partition part % k of request part / k, which is
        // what the scheduler would say for k * num_tokens partitions and no fixed overhead
        const int k = p.uniform_k, req = part / k, j = part - req * k;
        const int per = max((p.topk + BLOCK_N - 1) / BLOCK_N, 1) / k;
        m.begin_req = m.end_req = req;
        m.begin_block = j * per; m.end_block = (j + 1) * per;
        m.begin_split = j * p.num_tokens + req; m.first_split = m.last_split = 1; m.pad = 0;
    } else {
        // no scheduler: the CTA pairs of the grid share the requests as contiguous, whole ranges
        // (one request each when there are at least as many pairs as requests)
        const unsigned pairs = gridDim.x >> 1;
        if ((unsigned long long)pairs * (unsigned)p.num_tokens < 0x100000000ull) {      // 32-bit divisions: every warp of the CTA does this
            m.begin_req = (int)((unsigned)part * (unsigned)p.num_tokens / pairs);
            m.end_req = (int)((unsigned)(part + 1) * (unsigned)p.num_tokens / pairs) - 1;
        } else {
            m.begin_req = (int)((long long)part * p.num_tokens / pairs);
            m.end_req = (int)((long long)(part + 1) * p.num_tokens / pairs) - 1;
        }
        m.begin_block = 0; m.end_block = 0x7fffffff;
        m.begin_split = 0; m.first_split = m.last_split = 0; m.pad = 0;
    }
    return m;
}

__device__ __forceinline__ bool get_work(const AttnParams& p, const SchedMeta& m, int req, Work& w) {
    int len = p.topk_length ? p.topk_length[req] : p.topk;
    len = min(len, p.topk);
    // A request walks max(ceil(len / 64), 1) blocks of the main cache, then ceil(extra_len / 64) blocks of the
    // second cache when there is one (csrc/kernel/decode/decode_v2_kernel.cuh:109-115).
    w.main_blocks = max((len + BLOCK_N - 1) / BLOCK_N, 1);
    w.extra_len = 0;
    if (p.extra_topk > 0) {
        const int el = p.extra_topk_length ? p.extra_topk_length[req] : p.extra_topk;
        w.extra_len = max(min(el, p.extra_topk), 0);
    }
    const int total = w.main_blocks + (w.extra_len + BLOCK_N - 1) / BLOCK_N;
    const int b0 = (req == m.begin_req) ? m.begin_block : 0;
    const int b1 = min((req == m.end_req) ? m.end_block : total, total);
    w.req = req; w.blk0 = b0; w.nblk = b1 - b0; w.len = len;
    w.no_split = !p.force_partial &&
                 ((req == m.begin_req) ? !m.first_split : ((req == m.end_req) ? !m.last_split : true));
    w.split_idx = (p.num_splits ? p.num_splits[req] : 0) + ((req == m.begin_req) ? m.begin_split : 0);
    return w.nblk > 0;
}

// Entry r of 64-token block b of the request: its index in the cache that block walks, or -1 when there is no
// entry (past the request's length, past the partition's share, or a -1 in the index array).
__device__ __forceinline__ int fetch_entry(const AttnParams& p, const Work& w, int b, int r) {
    if (b >= w.blk0 + w.nblk) return -1;
    if (b < w.main_blocks) {
        const int pos = b * BLOCK_N + r;
        return pos < w.len ? __ldg(p.indices + (size_t)w.req * p.topk + pos) : -1;
    }
    const int pos = (b - w.main_blocks) * BLOCK_N + r;
    return pos < w.extra_len ? __ldg(p.extra_indices + (size_t)w.req * p.extra_topk + pos) : -1;
}

__device__ __forceinline__ float pow2_ceil(float x) {
    uint32_t b = __float_as_uint(x);
    if (b & 0x007fffffu) b = (b + 0x00800000u) & 0x7f800000u;
    return __uint_as_float(b);
}

__device__ __forceinline__ float ex2(float x) {   // 2^x, ex2(-inf) = +0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return (uint32_t)lo | ((uint32_t)hi << 16);
}

// Multiplies four packed e4m3 values by a power of two (given as half2) with rounding.
__device__ __forceinline__ uint32_t rescale_e4m3x4(uint32_t w, __half2 ratio) {
    uint32_t lo, hi;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"((uint16_t)(w & 0xffffu)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"((uint16_t)(w >> 16)));
    __half2 a = __hmul2(*reinterpret_cast<__half2*>(&lo), ratio);
    __half2 b = __hmul2(*reinterpret_cast<__half2*>(&hi), ratio);
    uint16_t ra, rb;
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(ra) : "r"(*reinterpret_cast<uint32_t*>(&a)));
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(rb) : "r"(*reinterpret_cast<uint32_t*>(&b)));
    return (uint32_t)ra | ((uint32_t)rb << 16);
}

// Divides four packed e4m3 values by 2^d with integer arithmetic: the exponent field of every byte drops
// by d (`sub` = d * 8 in every byte, d <= 15).  Exact while the result stays a normal number; a result
// below 2^-6 is cut to the subnormal grid or to zero (off by at most 2^-7, i.e. 2^-15 of the largest
// e4m3 value), which is far below the rounding step of the values that dominate a row.
__device__ __forceinline__ uint32_t shift_down_e4m3x4(uint32_t w, uint32_t sub) {
    const uint32_t t = ((w & 0x7f7f7f7fu) | 0x80808080u) - sub;   // bit 7 of a byte survives iff its magnitude >= sub
    uint32_t keep;                                                 // every byte's bit 7 spread over the byte: 0xff where no underflow
    asm("prmt.b32 %0, %1, %1, 0xba98;" : "=r"(keep) : "r"(t));     // (selector bit 3 = replicate the sign of the chosen byte)
    return (t & 0x7f7f7f7fu & keep) | (w & 0x80808080u);
}
// d * 8 in every byte for a ratio 2^-d (a power of two <= 1).
__device__ __forceinline__ uint32_t shift_bytes_of_ratio(float ratio) {
    const int d = min(127 - (int)(__float_as_uint(ratio) >> 23), 15);
    return (uint32_t)(d * 8) * 0x01010101u;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t w, __nv_bfloat162 f) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&w), f);
    return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

}  // namespace attn
}  // namespace smla
