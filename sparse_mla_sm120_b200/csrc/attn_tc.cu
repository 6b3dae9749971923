// Sparse-MLA attention on tcgen05 tensor cores (sm_100a): split-KV decode and prefill.
//
// Work unit.  One CTA owns one scheduler partition (a run of 64-token blocks of consecutive
// requests, see sched.cu; for prefill: one query token) and ONE HALF of the 512 output
// dimensions, for all (<= 128) query heads at once: heads are the M = 128 rows of every MMA.
// The fp32 output accumulator for 128 heads x 256 dims takes 256 of the 512 tensor-memory
// columns; two 64-column score buffers take 128 more.  The two CTAs of a partition both compute
// the scores (the score MMA is the cheaper part once everything is FP8) and are launched next
// to each other so that the second gather of a row is served by L2.
//
// Numerics (the FP8 class of the reference's V32 kernels, which quantise Q and P to e4m3:
// csrc/kernel/common/fp8_quant.cuh:44-103, csrc/kernel/decode/decode_v2_kernel.cuh:414-493):
//   * Q no-PE is quantised to e4m3 with one power-of-two scale per head; Q RoPE stays bf16 and
//     is pre-divided by that scale.
//   * K/V bytes are consumed as stored.  A row whose four 128-value tiles carry different
//     scales is re-expressed against its largest scale (a power-of-two shift, exact until the
//     e4m3 subnormal range); K RoPE is pre-divided by the row scale s_t.  One accumulator then
//     holds  S = (q . k) / (sq_h * s_t)  for no-PE (FP8 MMA) and RoPE (BF16 MMA) together.
//   * The row scale of V is folded into the exponent: z = S*sq_h*s_t*sm_scale*log2e + log2(s_t),
//     P' = 2^(z - m) with m the (lazily updated) running maximum of z, so that
//     O_acc = sum_t P'_t * Vfp8_t needs no per-tile scale; the denominator is tracked apart as
//     l = sum_t P'_t / s_t in fp32.  O = O_acc / l, LSE = log2(l) + m (base 2, as the reference).
//   * P' is rounded to e4m3 (times 2^P_SHIFT); the accumulator is rescaled only when a row
//     maximum grows by more than 2^RESCALE_TAU, which is exact because l and O share m.
//   * Invalid entries (index < 0, position >= topk_length) are never loaded: their shared-memory
//     rows are zero-filled and their weight is exactly 0 (NaN-safe, decode_v2_kernel.cuh:262-278).
//
// Warp roles (288 threads): warps 0-3 softmax + epilogue (thread = head row = TMEM lane),
// warps 4-7 gather producers (cp.async 16 B into 128B-swizzled tiles, three stages),
// warp 8 MMA issue (one lane) and TMEM allocation.  Every wait is bounded; a wait that gives up
// records a code in status[] and the CTA drains and exits.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace smla {

namespace {

using namespace ptx;

constexpr int TC_THREADS = 288;
constexpr int NSTAGE = 3;
constexpr int PREFETCH = 2;            // tiles in flight per producer thread
constexpr int P_SHIFT = 5;             // P' is stored as e4m3(P' * 2^P_SHIFT)
constexpr float RESCALE_TAU = 3.0f;    // lazy-rescale threshold (log2 units); P' <= 2^TAU

// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t QN_OFF = 0;                       // Q no-PE e4m3: 4 k-chunks x [128 rows x 128 B]
constexpr uint32_t QN_CHUNK = 128 * 128;
constexpr uint32_t QR_OFF = QN_OFF + 4 * QN_CHUNK;   // Q RoPE bf16: [128 rows x 128 B]
constexpr uint32_t ST_OFF = QR_OFF + 128 * 128;      // KV stages
constexpr uint32_t KV_CHUNK = 64 * 128;              // one 128-dim chunk of a 64-token tile
constexpr uint32_t ST_ROPE = 4 * KV_CHUNK;           // offset of the RoPE tile inside a stage
constexpr uint32_t ST_BYTES = ST_ROPE + 64 * 128;
constexpr uint32_t P_OFF = ST_OFF + NSTAGE * ST_BYTES;   // P' e4m3: 2 buffers x [4 k-chunks x 16 groups x 128 B]
constexpr uint32_t P_BYTES = 128 * 64;
constexpr uint32_t TOK_OFF = P_OFF + 2 * P_BYTES;    // per stage: s_t[64], log2 s_t[64], 1/s_t[64]
constexpr uint32_t TOK_BYTES = 3 * 64 * 4;
constexpr uint32_t SQC_OFF = TOK_OFF + NSTAGE * TOK_BYTES;  // sq_h * sm_scale * log2e, [128]
constexpr uint32_t BAR_OFF = SQC_OFF + 128 * 4;
// barriers (8 B each): full[3] empty[3] s_ready[2] p_ready[2] pv_done[2] q_ready
constexpr int BAR_FULL = 0, BAR_EMPTY = 3, BAR_SREADY = 6, BAR_PREADY = 8, BAR_PVDONE = 10, BAR_QREADY = 12, NBAR = 13;
constexpr uint32_t MISC_OFF = BAR_OFF + NBAR * 8;    // tmem base (4 B), abort flag (4 B)
constexpr uint32_t SMEM_BYTES = MISC_OFF + 16;
constexpr uint32_t SMEM_ALLOC = SMEM_BYTES + 1024;   // slack for the 1024-byte alignment
static_assert(SMEM_ALLOC <= 227 * 1024, "shared memory budget");

constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_O = 0, TM_S = 256;             // O: 256 columns; S buffer b at 256 + 64 b

constexpr uint32_t IDESC_QK_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, false, 128, 64);
constexpr uint32_t IDESC_QK_BF16 = instr_desc(FMT_BF16, FMT_BF16, false, false, 128, 64);
constexpr uint32_t IDESC_PV_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, true, 128, 256);

// give-up codes reported through status[0]
enum { W_EMPTY = 1, W_FULL = 2, W_SREADY = 3, W_PREADY = 4, W_PVDONE = 5, W_QREADY = 6 };

// Optional timeline of CTA 0 (debugging aid): records (tag, tile, clock) triples when a trace
// buffer has been registered with smla_debug_set_trace.
struct Trace {
    long long* buf;
    int cap;
};
__device__ __forceinline__ void trace(const Trace& t, int tag, int tile) {
    if (t.buf != nullptr && blockIdx.x == 0 && (threadIdx.x & 31) == 0) {
        const int slot = atomicAdd(reinterpret_cast<int*>(t.buf), 1);
        if (slot < t.cap) {
            long long c;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(c));
            t.buf[1 + 2 * slot] = ((long long)tag << 32) | (unsigned)tile;
            t.buf[2 + 2 * slot] = c;
        }
    }
}

struct Work {   // one request's share of a partition
    int req, blk0, nblk, len, split_idx;
    bool no_split;
};

__device__ __forceinline__ SchedMeta load_meta(const AttnParams& p, int part) {
    SchedMeta m;
    if (p.sched != nullptr) {
        m = p.sched[part];
    } else {
        m.begin_req = m.end_req = part;
        m.begin_block = 0; m.end_block = 0x7fffffff;
        m.begin_split = 0; m.first_split = m.last_split = 0; m.pad = 0;
    }
    return m;
}

__device__ __forceinline__ bool get_work(const AttnParams& p, const SchedMeta& m, int req, Work& w) {
    int len = p.topk_length ? p.topk_length[req] : p.topk;
    len = min(len, p.topk);
    const int total = max((len + BLOCK_N - 1) / BLOCK_N, 1);
    const int b0 = (req == m.begin_req) ? m.begin_block : 0;
    const int b1 = min((req == m.end_req) ? m.end_block : total, total);
    w.req = req; w.blk0 = b0; w.nblk = b1 - b0; w.len = len;
    w.no_split = !p.force_partial &&
                 ((req == m.begin_req) ? !m.first_split : ((req == m.end_req) ? !m.last_split : true));
    w.split_idx = p.num_splits ? p.num_splits[req] + ((req == m.begin_req) ? m.begin_split : 0) : 0;
    return w.nblk > 0;
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

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t w, __nv_bfloat162 f) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&w), f);
    return *reinterpret_cast<uint32_t*>(&r);
}

// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(TC_THREADS, 1) attn_tc_kernel(const AttnParams p, const Trace tr) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    float* sqc = reinterpret_cast<float*>(sm + SQC_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + MISC_OFF + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + MISC_OFF);
    auto bar = [&](int i) -> uint32_t { return base + BAR_OFF + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int part = blockIdx.x >> 1, half = blockIdx.x & 1;
    const SchedMeta meta = load_meta(p, part);

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar(BAR_FULL + s), 128); mbar_init(bar(BAR_EMPTY + s), 1); }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(BAR_SREADY + b), 1); mbar_init(bar(BAR_PREADY + b), 128); mbar_init(bar(BAR_PVDONE + b), 1);
        }
        mbar_init(bar(BAR_QREADY), 128);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 8) {
        tmem_alloc(base + MISC_OFF, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int last_req = min(meta.end_req, p.num_tokens - 1);

    if (warp < 4) {
        // =================================================================== softmax + epilogue
        const int row = tid;                      // head index == TMEM lane
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
        uint32_t it = 0, rq = 0;                  // running tile / request counters of this CTA
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            // ---- Q: load, quantise, store in the 128B-swizzled K-major layout ----------------
            for (int r0 = warp * 32; r0 < warp * 32 + 32; r0 += 4) {
                uint4 a[4], b[4], c[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int h = r0 + u;
                    a[u] = b[u] = c[u] = make_uint4(0, 0, 0, 0);
                    if (h < p.num_heads) {
                        const __nv_bfloat16* src = p.q + ((size_t)req * p.num_heads + h) * D_QK;
                        a[u] = __ldg(reinterpret_cast<const uint4*>(src + lane * 16));
                        b[u] = __ldg(reinterpret_cast<const uint4*>(src + lane * 16 + 8));
                        if (lane < 8) c[u] = __ldg(reinterpret_cast<const uint4*>(src + D_NOPE + lane * 8));
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int h = r0 + u;
                    const uint32_t wd[8] = {a[u].x, a[u].y, a[u].z, a[u].w, b[u].x, b[u].y, b[u].z, b[u].w};
                    float v[16];
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        v[2 * i] = __uint_as_float(wd[i] << 16);
                        v[2 * i + 1] = __uint_as_float(wd[i] & 0xffff0000u);
                        amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
                    }
                    amax = warp_max(amax);
                    const float sq = pow2_ceil(fmaxf(amax, 1e-4f) * (1.f / 448.f));
                    const float inv = 1.f / sq;
                    uint4 o;
                    o.x = pack_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
                    o.y = pack_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
                    o.z = pack_e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv);
                    o.w = pack_e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv);
                    const uint32_t sw = (uint32_t)(h & 7);
                    *reinterpret_cast<uint4*>(sm + QN_OFF + (lane >> 3) * QN_CHUNK + h * 128 + (((lane & 7) ^ sw) << 4)) = o;
                    if (lane < 8) {
                        const __nv_bfloat162 f = __float2bfloat162_rn(inv);
                        uint4 r;
                        r.x = mul_bf16x2(c[u].x, f); r.y = mul_bf16x2(c[u].y, f);
                        r.z = mul_bf16x2(c[u].z, f); r.w = mul_bf16x2(c[u].w, f);
                        *reinterpret_cast<uint4*>(sm + QR_OFF + h * 128 + ((lane ^ sw) << 4)) = r;
                    }
                    if (lane == 0) sqc[h] = (h < p.num_heads) ? sq * p.sm_scale * LOG2E : 0.f;
                }
            }
            fence_proxy_async();
            tc_fence_before();     // orders the previous epilogue's TMEM reads before the next MMAs
            mbar_arrive(bar(BAR_QREADY));
            __syncwarp();
            const float my_sqc = sqc[row];

            float m_run = -INFINITY;   // running maximum of z (lags by at most RESCALE_TAU)
            float l_run = 0.f;         // sum of P'/s_t
            float x_max = -INFINITY;   // running maximum of the scaled logits (max_logits output)
            for (int j = 0; j < w.nblk && ok; ++j, ++it) {
                const uint32_t b = it & 1u, st = it % NSTAGE;
                ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_SREADY + b), (it >> 1) & 1u, abort_flag, W_SREADY));
                if (!ok) break;
                trace(tr, 10 + warp, it);
                // the per-token scale arrays of this stage were published with the tile itself
                ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_FULL + st), (it / NSTAGE) & 1u, abort_flag, W_FULL));
                if (!ok) break;
                tc_fence_after();
                uint32_t sv[2][32];
                tmem_ld32(lane_addr + TM_S + 64 * b, sv[0]);
                tmem_ld32(lane_addr + TM_S + 64 * b + 32, sv[1]);
                tmem_wait_ld();
                const float* tok = reinterpret_cast<const float*>(sm + TOK_OFF + st * TOK_BYTES);
                float z[64];
                float mx = -INFINITY;
#pragma unroll
                for (int t = 0; t < 64; t += 4) {
                    const float4 s4 = *reinterpret_cast<const float4*>(tok + t);
                    const float4 g4 = *reinterpret_cast<const float4*>(tok + 64 + t);
                    z[t + 0] = fmaf(__uint_as_float(sv[t >> 5][(t + 0) & 31]) * s4.x, my_sqc, g4.x);
                    z[t + 1] = fmaf(__uint_as_float(sv[t >> 5][(t + 1) & 31]) * s4.y, my_sqc, g4.y);
                    z[t + 2] = fmaf(__uint_as_float(sv[t >> 5][(t + 2) & 31]) * s4.z, my_sqc, g4.z);
                    z[t + 3] = fmaf(__uint_as_float(sv[t >> 5][(t + 3) & 31]) * s4.w, my_sqc, g4.w);
                    mx = fmaxf(mx, fmaxf(fmaxf(z[t], z[t + 1]), fmaxf(z[t + 2], z[t + 3])));
                }
                if (p.out_max_logits != nullptr) {
#pragma unroll
                    for (int t = 0; t < 64; t += 4) {
                        const float4 g4 = *reinterpret_cast<const float4*>(tok + 64 + t);
                        x_max = fmaxf(x_max, fmaxf(fmaxf(z[t] - g4.x, z[t + 1] - g4.y), fmaxf(z[t + 2] - g4.z, z[t + 3] - g4.w)));
                    }
                }
                trace(tr, 15 + warp, it);
                const bool grow = mx > m_run + RESCALE_TAU;   // false while the row has seen no valid entry
                if (__any_sync(0xffffffffu, grow)) {
                    if (j > 0) {   // the accumulator holds earlier tiles: wait for the last P.V, then scale it
                        ok = __all_sync(0xffffffffu,
                                        mbar_wait(bar(BAR_PVDONE + ((it - 1) & 1u)), ((it - 1) >> 1) & 1u, abort_flag, W_PVDONE));
                        if (!ok) break;
                        tc_fence_after();
                    }
                    const float alpha = grow ? exp2f(m_run - mx) : 1.f;   // exp2(-inf) = 0 for the first tile
                    if (grow) { m_run = mx; l_run *= alpha; }
                    if (j > 0) {
#pragma unroll 1
                        for (int c = 0; c < 256; c += 32) {
                            uint32_t o[32];
                            tmem_ld32(lane_addr + TM_O + c, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(lane_addr + TM_O + c, o);
                        }
                        tmem_wait_st();
                    }
                }
                const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
                // the P' buffer of tile it was last read by the P.V of tile it-2
                if (it >= 2) {
                    ok = __all_sync(0xffffffffu,
                                    mbar_wait(bar(BAR_PVDONE + b), ((it - 2) >> 1) & 1u, abort_flag, W_PVDONE));
                    if (!ok) break;
                }
                uint8_t* pbuf = sm + P_OFF + b * P_BYTES + (row >> 3) * 128 + (row & 7) * 16;
                float lsum = 0.f;
#pragma unroll
                for (int t = 0; t < 64; t += 16) {
                    float pv[16];
#pragma unroll
                    for (int i = 0; i < 16; i += 4) {
                        const float4 i4 = *reinterpret_cast<const float4*>(tok + 128 + t + i);
                        pv[i + 0] = ex2(z[t + i + 0] - m_use);
                        pv[i + 1] = ex2(z[t + i + 1] - m_use);
                        pv[i + 2] = ex2(z[t + i + 2] - m_use);
                        pv[i + 3] = ex2(z[t + i + 3] - m_use);
                        lsum = fmaf(pv[i + 0], i4.x, lsum);
                        lsum = fmaf(pv[i + 1], i4.y, lsum);
                        lsum = fmaf(pv[i + 2], i4.z, lsum);
                        lsum = fmaf(pv[i + 3], i4.w, lsum);
                    }
                    constexpr float PS = (float)(1 << P_SHIFT);
                    uint4 o;
                    o.x = pack_e4m3x4(pv[0] * PS, pv[1] * PS, pv[2] * PS, pv[3] * PS);
                    o.y = pack_e4m3x4(pv[4] * PS, pv[5] * PS, pv[6] * PS, pv[7] * PS);
                    o.z = pack_e4m3x4(pv[8] * PS, pv[9] * PS, pv[10] * PS, pv[11] * PS);
                    o.w = pack_e4m3x4(pv[12] * PS, pv[13] * PS, pv[14] * PS, pv[15] * PS);
                    *reinterpret_cast<uint4*>(pbuf + (t >> 4) * 2048) = o;   // k-chunk t/16, 16 tokens = 16 B
                }
                l_run += lsum;
                fence_proxy_async();
                tc_fence_before();
                mbar_arrive(bar(BAR_PREADY + b));
                trace(tr, 20 + warp, it);
            }
            if (!ok) break;
            // ---- epilogue ---------------------------------------------------------------------
            {
                const uint32_t last = it - 1;
                ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_PVDONE + (last & 1u)), (last >> 1) & 1u, abort_flag, W_PVDONE));
                if (!ok) break;
                tc_fence_after();
                const bool live = row < p.num_heads;
                float lse = (l_run > 0.f) ? (log2f(l_run) + m_run) : NEG_BIG;
                float denom = l_run;
                if (w.no_split && p.attn_sink != nullptr && live) {
                    const float sink2 = p.attn_sink[row] * LOG2E;
                    denom = l_run + ((m_run == -INFINITY) ? INFINITY : exp2f(sink2 - m_run));
                    if (lse != NEG_BIG) lse += log2f(1.f + exp2f(sink2 - lse));
                    else lse = sink2;
                }
                const float inv = (denom > 0.f) ? 1.f / (denom * (float)(1 << P_SHIFT)) : 0.f;
                if (w.no_split) {
                    __nv_bfloat16* dst = p.out + ((size_t)req * p.num_heads + row) * D_V + half * 256;
#pragma unroll 1
                    for (int c = 0; c < 256; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + TM_O + c, o);
                        tmem_wait_ld();
                        if (live) {
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                uint4 v;
                                __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(o[i + 0]) * inv, __uint_as_float(o[i + 1]) * inv);
                                __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                                __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                                __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                                v.x = *reinterpret_cast<uint32_t*>(&t0); v.y = *reinterpret_cast<uint32_t*>(&t1);
                                v.z = *reinterpret_cast<uint32_t*>(&t2); v.w = *reinterpret_cast<uint32_t*>(&t3);
                                *reinterpret_cast<uint4*>(dst + c + i) = v;
                            }
                        }
                    }
                    if (live && half == 0) {
                        p.out_lse[(size_t)req * p.num_heads + row] = lse;
                        if (p.out_max_logits) p.out_max_logits[(size_t)req * p.num_heads + row] = (x_max == -INFINITY) ? NEG_BIG : x_max;
                    }
                } else {
                    float* dst = p.o_accum + ((size_t)w.split_idx * p.num_heads + row) * D_V + half * 256;
#pragma unroll 1
                    for (int c = 0; c < 256; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + TM_O + c, o);
                        tmem_wait_ld();
                        if (live) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                float4 v = make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv,
                                                       __uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                                *reinterpret_cast<float4*>(dst + c + i) = v;
                            }
                        }
                    }
                    if (live && half == 0) p.lse_accum[(size_t)w.split_idx * p.num_heads + row] = lse;
                }
            }
            ++rq;
        }
        (void)rq;
    } else if (warp < 8) {
        // =================================================================== gather producers
        const int ptid = tid - 128;
        const int r = ptid >> 1, hf = ptid & 1;    // token row inside the tile, half of the row
        const uint32_t sw = (uint32_t)(r & 7);
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int32_t* idx_row = p.indices + (size_t)req * p.topk;
            static_assert(PREFETCH == 2, "the in-flight bookkeeping below is written for two tiles");
            float4 sc_a = make_float4(0.f, 0.f, 0.f, 0.f), sc_b = sc_a, sc_c = sc_a;   // scales of tiles k-2, k-1, k
            int idx_a = -1, idx_b = -1, idx_c = -1;
            auto fetch_idx = [&](int j) -> int {
                const int pos = (w.blk0 + j) * BLOCK_N + r;
                return (j < w.nblk && pos < w.len) ? __ldg(idx_row + pos) : -1;
            };
            int idx_next = fetch_idx(0);
#pragma unroll 1
            for (int k = 0; k < w.nblk + PREFETCH && ok; ++k) {
                // Finishing tile k-2 comes first: the MMA warp needs it (score MMA of tile k-2) before it
                // can retire the P.V of tile k-3, which is what frees the stage tile k goes into.
                if (k >= PREFETCH) {
                    // -------- finish tile k - PREFETCH
                    const int kk = k - PREFETCH;
                    cp_async_wait<PREFETCH - 1>();
                    const uint32_t t_it = it + kk, st = t_it % NSTAGE;
                    trace(tr, 30 + warp, t_it);
                    uint8_t* sp = sm + ST_OFF + st * ST_BYTES;
                    float* tok = reinterpret_cast<float*>(sm + TOK_OFF + st * TOK_BYTES);
                    const float4 sc = sc_a;
                    const bool valid = idx_a >= 0;
                    const float smax = fmaxf(fmaxf(sc.x, sc.y), fmaxf(sc.z, sc.w));
                    if (valid) {
                        const float inv_s = 1.f / smax;
                        // no-PE tiles whose scale is below the row scale: shift them onto the row scale
                        const float mine[2] = {hf ? sc.z : sc.x, hf ? sc.w : sc.y};
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            if (mine[q] != smax) {
                                const __half2 ratio = __float2half2_rn(mine[q] * inv_s);
                                uint8_t* rowp = sp + (hf * 2 + q) * KV_CHUNK + r * 128;
#pragma unroll
                                for (int c = 0; c < 8; ++c) {
                                    uint4 v = *reinterpret_cast<uint4*>(rowp + c * 16);
                                    v.x = rescale_e4m3x4(v.x, ratio); v.y = rescale_e4m3x4(v.y, ratio);
                                    v.z = rescale_e4m3x4(v.z, ratio); v.w = rescale_e4m3x4(v.w, ratio);
                                    *reinterpret_cast<uint4*>(rowp + c * 16) = v;
                                }
                            }
                        }
                        // RoPE part of K, pre-divided by the row scale
                        const __nv_bfloat162 f = __float2bfloat162_rn(inv_s);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int ch = hf * 4 + c;
                            uint4* q4 = reinterpret_cast<uint4*>(sp + ST_ROPE + r * 128 + (((uint32_t)ch ^ sw) << 4));
                            uint4 v = *q4;
                            v.x = mul_bf16x2(v.x, f); v.y = mul_bf16x2(v.y, f);
                            v.z = mul_bf16x2(v.z, f); v.w = mul_bf16x2(v.w, f);
                            *q4 = v;
                        }
                        if (hf == 0) { tok[r] = smax; tok[64 + r] = log2f(smax); tok[128 + r] = inv_s; }
                    } else if (hf == 0) {
                        tok[r] = 0.f; tok[64 + r] = -INFINITY; tok[128 + r] = 0.f;
                    }
                    fence_proxy_async();
                    mbar_arrive(bar(BAR_FULL + st));
                    trace(tr, 40 + warp, t_it);
                }
                if (k < w.nblk) {
                    // -------- issue tile k
                    const uint32_t t_it = it + k, st = t_it % NSTAGE;
                    const int idx = idx_next;
                    idx_next = fetch_idx(k + 1);
                    if (t_it >= NSTAGE) {
                        ok = __all_sync(0xffffffffu,
                                        mbar_wait(bar(BAR_EMPTY + st), ((t_it / NSTAGE) - 1) & 1u, abort_flag, W_EMPTY));
                        if (!ok) break;
                    }
                    trace(tr, 50 + warp, t_it);
                    const uint32_t sbase = base + ST_OFF + st * ST_BYTES;
                    float4 sc = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (idx >= 0) {
                        const uint8_t* src = kv_row_ptr(p.kv, idx, p.page_block_size, p.block_stride);
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int ch = hf * 16 + c;        // 16-byte chunk of the 512 no-PE bytes
                            cp_async16(sbase + (ch >> 3) * KV_CHUNK + r * 128 + ((((uint32_t)ch & 7u) ^ sw) << 4), src + ch * 16);
                        }
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int ch = hf * 4 + c;
                            cp_async16(sbase + ST_ROPE + r * 128 + (((uint32_t)ch ^ sw) << 4), src + ROPE_OFF + ch * 16);
                        }
                        sc = __ldg(reinterpret_cast<const float4*>(src + SCALE_OFF));
                    } else {
                        uint8_t* sp = sm + ST_OFF + st * ST_BYTES;
                        const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int ch = hf * 16 + c;
                            *reinterpret_cast<uint4*>(sp + (ch >> 3) * KV_CHUNK + r * 128 + ((((uint32_t)ch & 7u) ^ sw) << 4)) = zero;
                        }
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int ch = hf * 4 + c;
                            *reinterpret_cast<uint4*>(sp + ST_ROPE + r * 128 + (((uint32_t)ch ^ sw) << 4)) = zero;
                        }
                    }
                    sc_c = sc;
                    idx_c = idx;
                    trace(tr, 60 + warp, t_it);
                }
                cp_async_commit();
                sc_a = sc_b; idx_a = idx_b;
                sc_b = sc_c; idx_b = idx_c;
            }
            it += w.nblk;
        }
        cp_async_wait<0>();
    } else {
        // =================================================================== MMA issue
        uint32_t it = 0, rq = 0;
        bool ok = true;
        const uint32_t qn = base + QN_OFF, qr = base + QR_OFF;
        auto issue_qk = [&](uint32_t t_it) {
            const uint32_t st = t_it % NSTAGE, b = t_it & 1u;
            const uint32_t kb = base + ST_OFF + st * ST_BYTES;
            const uint32_t d = tmem + TM_S + 64 * b;
#pragma unroll
            for (int kc = 0; kc < 4; ++kc) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    mma_f8(d, smem_desc(qn + kc * QN_CHUNK + ks * 32, 16, 1024, SWIZZLE_128B),
                           smem_desc(kb + kc * KV_CHUNK + ks * 32, 16, 1024, SWIZZLE_128B), IDESC_QK_F8, (kc | ks) != 0);
                }
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                mma_f16(d, smem_desc(qr + ks * 32, 16, 1024, SWIZZLE_128B),
                        smem_desc(kb + ST_ROPE + ks * 32, 16, 1024, SWIZZLE_128B), IDESC_QK_BF16, true);
            }
            tc_commit(bar(BAR_SREADY + b));
        };
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_QREADY), rq & 1u, abort_flag, W_QREADY));
            if (!ok) break;
            ++rq;
            ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_FULL + it % NSTAGE), (it / NSTAGE) & 1u, abort_flag, W_FULL));
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) issue_qk(it);
            __syncwarp();
            for (int j = 0; j < w.nblk && ok; ++j, ++it) {
                if (j + 1 < w.nblk) {
                    const uint32_t nx = it + 1;
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_FULL + nx % NSTAGE), (nx / NSTAGE) & 1u, abort_flag, W_FULL));
                    if (!ok) break;
                    tc_fence_after();
                    trace(tr, 70, nx);
                    if (lane == 0) issue_qk(nx);
                    __syncwarp();
                    trace(tr, 71, nx);
                }
                const uint32_t b = it & 1u, st = it % NSTAGE;
                ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_PREADY + b), (it >> 1) & 1u, abort_flag, W_PREADY));
                if (!ok) break;
                tc_fence_after();
                trace(tr, 72, it);
                if (lane == 0) {
                    const uint32_t pb = base + P_OFF + b * P_BYTES;
                    const uint32_t vb = base + ST_OFF + st * ST_BYTES + (uint32_t)half * 2 * KV_CHUNK;
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) {
                        mma_f8(tmem + TM_O, smem_desc(pb + ks * 4096, 2048, 128, SWIZZLE_NONE),
                               smem_desc(vb + ks * 4096, KV_CHUNK, 1024, SWIZZLE_128B), IDESC_PV_F8, (j | ks) != 0);
                    }
                    tc_commit(bar(BAR_EMPTY + st));
                    tc_commit(bar(BAR_PVDONE + b));
                }
                __syncwarp();
                trace(tr, 73, it);
            }
        }
    }

    // ------------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) {
        atomicCAS(p.status, 0, *abort_flag);
        atomicAdd(p.status + 1, 1);
        p.status[2] = blockIdx.x;
    }
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace

static Trace g_trace = {nullptr, 0};
void set_attn_trace(long long* buf, int cap) { g_trace.buf = buf; g_trace.cap = cap; }

int launch_attn_tc(const AttnParams& p, cudaStream_t stream) {
    if (p.num_tokens == 0) return 0;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_ALLOC);
        if (e != cudaSuccess) return set_error((int)e, "attn_tc_kernel: cannot reserve %u bytes of shared memory: %s",
                                               SMEM_ALLOC, cudaGetErrorString(e));
        attr_set[dev] = true;
    }
    const int parts = p.sched ? p.num_parts : p.num_tokens;
    attn_tc_kernel<<<2 * parts, TC_THREADS, SMEM_ALLOC, stream>>>(p, g_trace);
    return check_launch("attn_tc_kernel");
}

int launch_mqa_logits_tc(const uint8_t* q, const uint8_t* k, const float* k_scale, const float* weights,
                         const int32_t* ks, const int32_t* ke, float* logits, int s_q, int num_heads,
                         int s_k, int64_t logits_stride, int32_t* status, cudaStream_t stream) {
    (void)status;
    return launch_mqa_logits_scalar(q, k, k_scale, weights, ks, ke, logits, s_q, num_heads, s_k, logits_stride, stream);
}

}  // namespace smla
