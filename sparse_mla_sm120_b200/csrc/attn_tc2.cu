// Sparse-MLA attention on tcgen05 tensor cores (sm_100a), pair-split variant: the two CTAs of a
// partition form a thread-block cluster and share the score work instead of repeating it.
//
// Work split.  As in attn_tc.cu a partition is served by two CTAs, CTA c holding the fp32
// accumulator of output dims [256c, 256c+256) for all (<= 128) heads.  The 64-token tiles of the
// partition alternate between the two: the OWNER of a tile gathers its full 656-byte rows,
// computes the scores (Q . K^T), the softmax weights P' and its own P' . V; it also writes P'
// (8 KB of e4m3) and the reference exponent it used (one float per head) into the other CTA's
// shared memory.  The other CTA gathers only its 256-byte half of the tile's V bytes (plus the
// 16 scale bytes) and adds P' . V for its dims.  Per tile a CTA therefore takes in 34 KB instead
// of 42 KB and does half of the score MMAs and half of the softmax.
//
// Consistency of the two accumulators.  P' of a tile is 2^(z - m) for a reference m chosen by the
// tile's owner.  Every CTA keeps one reference per head row for its accumulator (and for its
// partial denominator l, which sums the tiles it owns).  Before the P' . V of a tile is released,
// the row's accumulator is brought to the reference that tile's P' was computed with: a no-op in
// the steady state.  References are whole numbers and only move up: a tile that arrives with a
// higher reference makes the accumulator follow (a rescale after the P' . V issued so far have
// completed), a tile with a lower one has its P' row shifted down by the difference, an exact
// exponent change (zeroed when nothing representable is left).  Because an owner starts from its
// accumulator's current reference, both CTAs settle on the same running maximum.  At the end of a request the CTAs exchange (l, reference, max logit) per
// row, so that both normalise with the full denominator.
//
// Numerics, tensor-memory map, the per-tile pipeline inside a CTA and the bounded-wait protocol
// are those of attn_tc.cu (see its header).  Nothing here loads with cluster multicast; the only
// cross-CTA traffic is plain st.shared::cluster stores and mbarrier arrives.
#include <cstdlib>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace smla {

namespace {

using namespace ptx;

constexpr int N_SM_WARPS = 8, N_PR_WARPS = 4, N_FX_WARPS = 8;
constexpr int FX_ROWS = 8;
constexpr int FX_WARP0 = N_SM_WARPS + N_PR_WARPS;
constexpr int MMA_WARP = FX_WARP0 + N_FX_WARPS;       // score MMAs; +1: P.V MMAs (and slot credits); +2: P' sender; +3: receipt relay
constexpr int TC_THREADS = (MMA_WARP + 4) * 32;
constexpr int REGS_LAUNCH = 80, REGS_SOFTMAX = 128, REGS_OTHER = 48;
static_assert(N_SM_WARPS * 32 * REGS_SOFTMAX + (N_PR_WARPS + N_FX_WARPS) * 32 * REGS_OTHER + 128 * REGS_LAUNCH
                  <= TC_THREADS * REGS_LAUNCH, "register budgets exceed what the CTA owns");
static_assert(65536 / TC_THREADS / 8 * 8 == REGS_LAUNCH, "launch-time registers per thread");
constexpr int NS = 3;                  // stages of the ring of owned tiles and of the ring of the other CTA's tiles
constexpr int NP = 3;                  // P' slots (tiles of the other CTA whose weights may be waiting here)
constexpr int NDONE = 8;               // ring of "the n-th issued P.V has completed" barriers
constexpr int P_SHIFT = 5;
constexpr float RESCALE_TAU = 3.0f;

// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t QR_OFF = 0;                        // Q RoPE bf16, K-major 128B swizzle
constexpr uint32_t KV_CHUNK = 64 * 128;
constexpr uint32_t ST_ROPE = 4 * KV_CHUNK;
constexpr uint32_t ST_SCALE = ST_ROPE + 64 * 128;
constexpr uint32_t ST_BYTES = ST_SCALE + 64 * 16;     // 41984: a full tile (owned)
constexpr uint32_t HS_SCALE = 2 * KV_CHUNK;
constexpr uint32_t HS_BYTES = HS_SCALE + 64 * 16;     // 17408: two no-PE chunks + the rows' scales (other CTA's tile)
constexpr uint32_t FS_OFF = QR_OFF + 128 * 128;
constexpr uint32_t HS_OFF = FS_OFF + NS * ST_BYTES;
// P' of the other CTA's tiles as the A operand of P.V: NP slots of [128 rows x 64 B], K-major
// 64B swizzle (chunk c of row r at 16 * (c ^ ((r >> 1) & 3))).  The owner builds the same image
// in the RoPE region of the tile's own stage (dead once the scores exist) and bulk-copies it.
constexpr uint32_t PS_OFF = HS_OFF + NS * HS_BYTES;
constexpr uint32_t PS_BYTES = 128 * 64;
constexpr uint32_t PM_OFF = PS_OFF + NP * PS_BYTES;   // [NP][128] reference exponents that came with the P' slots
constexpr uint32_t XCH_OFF = PM_OFF + NP * 128 * 4;   // pair exchange inside the CTA [2][2][128] fp32
constexpr uint32_t EPI_OFF = XCH_OFF + 2 * 2 * 128 * 4;   // [2 request parities][3][128]: l, reference, max logit from the other CTA
constexpr uint32_t BAR_OFF = EPI_OFF + 2 * 3 * 128 * 4;
constexpr int BAR_FULL = 0, BAR_EMPTY = NS, BAR_LOADED = 2 * NS, BAR_HLOADED = 3 * NS, BAR_HFULL = 4 * NS, BAR_HEMPTY = 5 * NS,
              BAR_SREADY = 6 * NS, BAR_PREADY = BAR_SREADY + 2, BAR_PVOWN = BAR_PREADY + 2, BAR_QREADY = BAR_PVOWN + 2,
              BAR_PFULL = BAR_QREADY + 1, BAR_PFREE = BAR_PFULL + NP, BAR_PDONE = BAR_PFREE + NP, BAR_ADOPTED = BAR_PDONE + NP,
              BAR_DONE = BAR_ADOPTED + NP, BAR_EPI = BAR_DONE + NDONE, BAR_STAGED = BAR_EPI + 2, NBAR = BAR_STAGED + NS;
constexpr uint32_t MISC_OFF = BAR_OFF + NBAR * 8;
constexpr uint32_t SMEM_BYTES = MISC_OFF + 16;
constexpr uint32_t SMEM_ALLOC = SMEM_BYTES + 1024;
static_assert(SMEM_ALLOC <= 227 * 1024, "shared memory budget");
static_assert(FS_OFF % 1024 == 0 && ST_BYTES % 1024 == 0 && HS_OFF % 1024 == 0 && HS_BYTES % 1024 == 0 && PS_OFF % 1024 == 0 && PS_BYTES % 1024 == 0,
              "swizzled tiles need 1024-byte alignment");

constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_O = 0, TM_S = 256, TM_Q = 384;

constexpr uint32_t IDESC_QK_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, false, 128, 64);
constexpr uint32_t IDESC_QK_BF16 = instr_desc(FMT_BF16, FMT_BF16, false, false, 128, 64);
constexpr uint32_t IDESC_PV_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, true, 128, 256);
constexpr uint32_t DESC_HI_SW128 = desc_hi(1024, (uint32_t)SWIZZLE_128B);
constexpr uint32_t DESC_HI_SW64 = desc_hi(512, (uint32_t)SWIZZLE_64B);

enum { W_EMPTY = 21, W_FULL = 22, W_SREADY = 23, W_PREADY = 24, W_PVOWN = 25, W_QREADY = 26, W_LOADED = 27, W_HEMPTY = 28,
       W_HLOADED = 29, W_HFULL = 30, W_PFULL = 31, W_PFREE = 32, W_PDONE = 33, W_ADOPTED = 34, W_DONE = 35, W_EPI = 36, W_PVPOLL = 37 };

struct Work {
    int req, blk0, nblk, len, split_idx;
    bool no_split;
};

// Optional timeline of CTA 0 (debugging aid, see attn_tc.cu).
struct Trace {
    long long* buf;
    int cap;
    int block;    // the CTA that records
};
struct TraceCursor {
    int n = 0;
};
__device__ __forceinline__ void trace(const Trace& t, TraceCursor& c, int tag, int tile) {
    if (t.buf != nullptr && blockIdx.x == t.block && (threadIdx.x & 31) == 0 && c.n < t.cap) {
        long long* slot = t.buf + ((size_t)(threadIdx.x >> 5) * t.cap + c.n) * 2;
        slot[0] = ((long long)tag << 32) | (unsigned)tile;
        slot[1] = clock64();
        ++c.n;
    }
}

__device__ __forceinline__ SchedMeta load_meta(const AttnParams& p, int part) {
    SchedMeta m;
    if (p.sched != nullptr) {
        m = p.sched[part];
    } else {
        const long long pairs = gridDim.x >> 1;
        m.begin_req = (int)((long long)part * p.num_tokens / pairs);
        m.end_req = (int)((long long)(part + 1) * p.num_tokens / pairs) - 1;
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
__device__ __forceinline__ float ex2(float x) {
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
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Order in which a CTA consumes the n tiles of a request that starts at running tile t0: its own
// tiles in order, and each tile of the other CTA three tiles after the own tile that precedes it
// (so that the other CTA's P' has normally arrived, and neither softmax waits for the other).
// Gathers, fix-up, softmax and P.V issue all walk this order; fo(t) / fp(t) return false to stop.
template <typename FO, typename FP>
__device__ __forceinline__ bool run_sequence(uint32_t t0, uint32_t n, uint32_t rank, FO fo, FP fp) {
    const uint32_t first_own = ((t0 & 1u) == rank) ? 0u : 1u, first_oth = 1u - first_own;
    const uint32_t n_own = (n > first_own) ? (n - first_own + 1) / 2 : 0, n_oth = (n > first_oth) ? (n - first_oth + 1) / 2 : 0;
    const uint32_t lead = (first_own == 0u) ? 2u : 1u;      // how many own tiles the own side runs ahead
    uint32_t io = 0, ip = 0;
#pragma unroll 1
    while (io < n_own || ip < n_oth) {
        if (io < n_own && (ip >= n_oth || io <= ip + lead)) { if (!fo(t0 + first_own + 2 * io)) return false; ++io; }
        else { if (!fp(t0 + first_oth + 2 * ip)) return false; ++ip; }
    }
    return true;
}

// The same walk for callers that want to look one tile ahead: f(tile, is_own, next_tile), with
// next_tile = 0xffffffff after the last one.  `first` receives the first tile of the order.
template <typename F>
__device__ __forceinline__ bool run_sequence_ahead(uint32_t t0, uint32_t n, uint32_t rank, F f) {
    const uint32_t first_own = ((t0 & 1u) == rank) ? 0u : 1u, first_oth = 1u - first_own;
    const uint32_t n_own = (n > first_own) ? (n - first_own + 1) / 2 : 0, n_oth = (n > first_oth) ? (n - first_oth + 1) / 2 : 0;
    const uint32_t lead = (first_own == 0u) ? 2u : 1u;
    uint32_t io = 0, ip = 0;
    auto pick = [&](uint32_t a, uint32_t b, bool& own) -> uint32_t {
        if (a >= n_own && b >= n_oth) { own = false; return 0xffffffffu; }
        own = a < n_own && (b >= n_oth || a <= b + lead);
        return own ? t0 + first_own + 2 * a : t0 + first_oth + 2 * b;
    };
    bool own;
    uint32_t cur = pick(io, ip, own);
#pragma unroll 1
    while (cur != 0xffffffffu) {
        if (own) ++io; else ++ip;
        bool own_next;
        const uint32_t nxt = pick(io, ip, own_next);
        if (!f(cur, own, nxt)) return false;
        cur = nxt; own = own_next;
    }
    return true;
}
__device__ __forceinline__ uint32_t first_in_sequence(uint32_t t0, uint32_t n, uint32_t rank) {
    // an owned tile comes first whenever the request has one; otherwise its only tile is the other CTA's
    const uint32_t first_own = ((t0 & 1u) == rank) ? 0u : 1u;
    return (n > first_own) ? t0 + first_own : t0;
}

// ---------------------------------------------------------------------------------------------
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1) attn_tc2_kernel(const AttnParams p, const Trace tr) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + MISC_OFF + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + MISC_OFF);
    auto bar = [&](int i) -> uint32_t { return base + BAR_OFF + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int part = blockIdx.x >> 1;
    const uint32_t rank = cluster_ctarank(), peer = rank ^ 1u;
    const int half = (int)rank;                       // this CTA's half of the output dims
    auto remote = [&](uint32_t local_addr) -> uint32_t { return mapa_shared(local_addr, peer); };
    const SchedMeta meta = load_meta(p, part);
    TraceCursor tc;
    trace(tr, tc, 1, 0);

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar(BAR_FULL + s), N_FX_WARPS * 32);
            mbar_init(bar(BAR_EMPTY + s), 2);                    // own P.V done + the other CTA has received P' (staged in this stage)
            mbar_init(bar(BAR_LOADED + s), N_PR_WARPS * 32);
            mbar_init(bar(BAR_HLOADED + s), N_PR_WARPS * 32);
            mbar_init(bar(BAR_HFULL + s), N_FX_WARPS * 32);
            mbar_init(bar(BAR_HEMPTY + s), 1);
            mbar_init(bar(BAR_STAGED + s), N_SM_WARPS * 32);     // P' image of the owned tile in this stage is complete
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(BAR_SREADY + b), 1);
            mbar_init(bar(BAR_PREADY + b), N_SM_WARPS * 32);
            mbar_init(bar(BAR_PVOWN + b), 1);
            mbar_init(bar(BAR_EPI + b), N_SM_WARPS * 16);        // the hh = 0 threads of the other CTA
        }
        for (int s = 0; s < NP; ++s) {
            mbar_init(bar(BAR_PFULL + s), 1);                    // armed by this CTA, filled by the other CTA's bulk copies of P' and references
            mbar_init(bar(BAR_PFREE + s), 1);                    // arrived by the other CTA's relay thread
            mbar_init(bar(BAR_PDONE + s), 1);
            mbar_init(bar(BAR_ADOPTED + s), N_SM_WARPS * 32);
        }
        for (int s = 0; s < NDONE; ++s) mbar_init(bar(BAR_DONE + s), 1);
        mbar_init(bar(BAR_QREADY), N_SM_WARPS * 32);
        *abort_flag = 0;
        mbar_init_fence();
        // every use of a P' slot is armed here, by the receiver: the sender only copies
        for (int s = 0; s < NP; ++s) mbar_arrive_expect_tx(bar(BAR_PFULL + s), PS_BYTES + 128 * 4);
    }
    if (warp == MMA_WARP) {
        tmem_alloc(base + MISC_OFF, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // both CTAs' barriers exist before anything arrives on them remotely
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int last_req = min(meta.end_req, p.num_tokens - 1);

    if (warp < N_SM_WARPS) setmaxnreg_inc<REGS_SOFTMAX>();
    else if (warp < MMA_WARP) setmaxnreg_dec<REGS_OTHER>();

    // Tile t of the partition (running count over its requests) is owned by CTA (t & 1); both rings
    // and the P' slots advance once per two tiles, so tile t uses ring position t >> 1 in either.
    auto owned = [&](uint32_t t) -> bool { return (t & 1u) == rank; };

    if (warp < N_SM_WARPS) {
        // =================================================================== softmax + epilogue
        const int quarter = warp & 3, hh = warp >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        float* xch = reinterpret_cast<float*>(sm + XCH_OFF);
        const bool live = row < p.num_heads;
        uint32_t it = 0;            // running tile counter of the partition
        uint32_t n_rel = 0;         // P.V products released to the issuing thread so far (all requests)
        uint32_t n_req = 0;         // requests handled so far
        bool ok = true;

        // Waits until every P.V released so far has completed (they complete in issue order and the
        // issuing thread cannot have issued more than were released).
        auto wait_released = [&]() -> bool {
            if (n_rel == 0) return true;
            const uint32_t k = n_rel - 1;
            const bool r = mbar_wait_hot(bar(BAR_DONE + (int)(k % NDONE)), (k / NDONE) & 1u, abort_flag, W_DONE);
            tc_fence_after();
            return r;
        };
        // Multiplies this thread's row of the accumulator (its 128 columns) by alpha.
        auto scale_acc = [&](float alpha) {
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
                uint32_t o[32];
                tmem_ld32(lane_addr + TM_O + 128 * hh + c, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st32(lane_addr + TM_O + 128 * hh + c, o);
            }
            tmem_wait_st();
        };

        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            // ---- Q: this warp owns rows [32*quarter, +32) x no-PE dims [256*hh, +256), read once ----
            {
                const int g = lane >> 2, c4 = lane & 3;
#pragma unroll 1
                for (int hf = 0; hf < 2; ++hf) {
                    const int r_a = quarter * 32 + 16 * hf + g, r_b = r_a + 8;
                    const __nv_bfloat16* src_a = p.q + ((size_t)req * p.num_heads + r_a) * D_QK + hh * 256 + c4 * 8;
                    const __nv_bfloat16* src_b = src_a + (size_t)8 * D_QK;
                    const bool v_a = r_a < p.num_heads, v_b = r_b < p.num_heads;
                    uint4 xa[8], xb[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        xa[i] = v_a ? __ldg(reinterpret_cast<const uint4*>(src_a + 32 * i)) : make_uint4(0, 0, 0, 0);
                        xb[i] = v_b ? __ldg(reinterpret_cast<const uint4*>(src_b + 32 * i)) : make_uint4(0, 0, 0, 0);
                    }
                    auto absmax8 = [](const uint4& a) {
                        return fmaxf(fmaxf(fmaxf(fabsf(bf16lo(a.x)), fabsf(bf16hi(a.x))), fmaxf(fabsf(bf16lo(a.y)), fabsf(bf16hi(a.y)))),
                                     fmaxf(fmaxf(fabsf(bf16lo(a.z)), fabsf(bf16hi(a.z))), fmaxf(fabsf(bf16lo(a.w)), fabsf(bf16hi(a.w)))));
                    };
                    float am_a = 0.f, am_b = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) { am_a = fmaxf(am_a, absmax8(xa[i])); am_b = fmaxf(am_b, absmax8(xb[i])); }
                    am_a = fmaxf(am_a, __shfl_xor_sync(0xffffffffu, am_a, 1)); am_b = fmaxf(am_b, __shfl_xor_sync(0xffffffffu, am_b, 1));
                    am_a = fmaxf(am_a, __shfl_xor_sync(0xffffffffu, am_a, 2)); am_b = fmaxf(am_b, __shfl_xor_sync(0xffffffffu, am_b, 2));
                    if (c4 == 0) { xch[hh * 128 + r_a] = am_a; xch[hh * 128 + r_b] = am_b; }
                    named_bar_sync(1 + quarter, 64);
                    am_a = fmaxf(am_a, xch[(1 - hh) * 128 + r_a]);
                    am_b = fmaxf(am_b, xch[(1 - hh) * 128 + r_b]);
                    const float sq_a = pow2_ceil(fmaxf(am_a, 1e-4f) * (1.f / 448.f)), sq_b = pow2_ceil(fmaxf(am_b, 1e-4f) * (1.f / 448.f));
                    const float ia = __uint_as_float(0x7f000000u - __float_as_uint(sq_a));
                    const float ib = __uint_as_float(0x7f000000u - __float_as_uint(sq_b));
                    if (c4 == 0) { xch[256 + r_a] = sq_a; xch[256 + r_b] = sq_b; }
#pragma unroll
                    for (int h4 = 0; h4 < 2; ++h4) {
                        uint32_t wq[16];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint4 a = xa[4 * h4 + k], b4 = xb[4 * h4 + k];
                            wq[4 * k + 0] = pack_e4m3x4(bf16lo(a.x) * ia, bf16hi(a.x) * ia, bf16lo(a.y) * ia, bf16hi(a.y) * ia);
                            wq[4 * k + 1] = pack_e4m3x4(bf16lo(a.z) * ia, bf16hi(a.z) * ia, bf16lo(a.w) * ia, bf16hi(a.w) * ia);
                            wq[4 * k + 2] = pack_e4m3x4(bf16lo(b4.x) * ib, bf16hi(b4.x) * ib, bf16lo(b4.y) * ib, bf16hi(b4.y) * ib);
                            wq[4 * k + 3] = pack_e4m3x4(bf16lo(b4.z) * ib, bf16hi(b4.z) * ib, bf16lo(b4.w) * ib, bf16hi(b4.w) * ib);
                        }
                        tmem_st_16x256b_x4(tmem + ((uint32_t)(quarter * 32 + 16 * hf) << 16) + TM_Q + hh * 64 + h4 * 32, wq);
                    }
                }
                __syncwarp();
            }
            const float sq = xch[256 + row];
            const float my_sqc = live ? sq * p.sm_scale * LOG2E : 0.f;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int rl = hh * 16 + g * 4 + (lane >> 3);
                const int h = quarter * 32 + rl;
                uint4 c = make_uint4(0, 0, 0, 0);
                if (h < p.num_heads)
                    c = __ldg(reinterpret_cast<const uint4*>(p.q + ((size_t)req * p.num_heads + h) * D_QK + D_NOPE + (lane & 7) * 8));
                const __nv_bfloat162 f = __float2bfloat162_rn(__uint_as_float(0x7f000000u - __float_as_uint(xch[256 + h])));
                c.x = mul_bf16x2(c.x, f); c.y = mul_bf16x2(c.y, f); c.z = mul_bf16x2(c.z, f); c.w = mul_bf16x2(c.w, f);
                *reinterpret_cast<uint4*>(sm + QR_OFF + h * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)h & 7u)) << 4)) = c;
            }
            tmem_wait_st();
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(bar(BAR_QREADY));

            float m_run = -INFINITY;   // reference exponent of this row's accumulator (and of l_run)
            float l_run = 0.f;         // sum of P'/s_t over the owned tiles, this thread's 32 columns
            float x_max = -INFINITY;
            uint32_t rel_req = 0;      // products released for this request (0: the accumulator holds nothing yet)

            // ---- an owned tile: scores -> P', to this CTA's tensor memory and to the other CTA ----
            auto own_tile = [&](uint32_t t) -> bool {
                const uint32_t r = t >> 1, b = r & 1u, st = r % NS;
                trace(tr, tc, 5, t);
                if (!mbar_wait_hot(bar(BAR_SREADY + b), (r >> 1) & 1u, abort_flag, W_SREADY)) return false;
                if (!mbar_wait(bar(BAR_FULL + st), (r / NS) & 1u, abort_flag, W_FULL)) return false;
                tc_fence_after();
                trace(tr, tc, 10 + warp, t);
                uint32_t sv[32];
                tmem_ld32(lane_addr + TM_S + 64 * b + 32 * hh, sv);
                const float4* tok = reinterpret_cast<const float4*>(sm + FS_OFF + st * ST_BYTES + ST_SCALE) + 32 * hh;
                tmem_wait_ld();
                float z[32];
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int u = 0; u < 32; u += 4) {
                    const float2 a0 = *reinterpret_cast<const float2*>(tok + u), a1 = *reinterpret_cast<const float2*>(tok + u + 1);
                    const float2 a2 = *reinterpret_cast<const float2*>(tok + u + 2), a3 = *reinterpret_cast<const float2*>(tok + u + 3);
                    z[u + 0] = fmaf(__uint_as_float(sv[u + 0]) * a0.x, my_sqc, a0.y);
                    z[u + 1] = fmaf(__uint_as_float(sv[u + 1]) * a1.x, my_sqc, a1.y);
                    z[u + 2] = fmaf(__uint_as_float(sv[u + 2]) * a2.x, my_sqc, a2.y);
                    z[u + 3] = fmaf(__uint_as_float(sv[u + 3]) * a3.x, my_sqc, a3.y);
                    mx0 = fmaxf(mx0, fmaxf(z[u], z[u + 1]));
                    mx1 = fmaxf(mx1, fmaxf(z[u + 2], z[u + 3]));
                    if (p.out_max_logits != nullptr)
                        x_max = fmaxf(x_max, fmaxf(fmaxf(z[u] - a0.y, z[u + 1] - a1.y), fmaxf(z[u + 2] - a2.y, z[u + 3] - a3.y)));
                }
                xch[b * 256 + hh * 128 + row] = fmaxf(mx0, mx1);
                named_bar_sync(1 + quarter, 64);
                const float mx = fmaxf(fmaxf(mx0, mx1), xch[b * 256 + (1 - hh) * 128 + row]);
                const bool grow = mx > m_run + RESCALE_TAU;
                if (__any_sync(0xffffffffu, grow)) {
                    if (rel_req > 0) { if (!wait_released()) return false; }
                    // references are whole numbers, so that two references always differ by a power of two
                    const float m_new = ceilf(mx);
                    const float alpha = grow ? ex2(m_run - m_new) : 1.f;
                    if (grow) { m_run = m_new; l_run *= alpha; }
                    if (rel_req > 0) scale_acc(alpha);
                }
                const float m_off = ((m_run == -INFINITY) ? 0.f : m_run) - (float)P_SHIFT;
                uint32_t pw[8];
                float l0 = 0.f, l1 = 0.f;
#pragma unroll
                for (int u = 0; u < 32; u += 4) {
                    const float p0 = ex2(z[u + 0] - m_off), p1 = ex2(z[u + 1] - m_off);
                    const float p2 = ex2(z[u + 2] - m_off), p3 = ex2(z[u + 3] - m_off);
                    l0 = fmaf(p0, tok[u].z, l0); l1 = fmaf(p1, tok[u + 1].z, l1);
                    l0 = fmaf(p2, tok[u + 2].z, l0); l1 = fmaf(p3, tok[u + 3].z, l1);
                    pw[u >> 2] = pack_e4m3x4(p0, p1, p2, p3);
                }
                l_run += l0 + l1;
                {
                    // image of the other CTA's P' slot in the (dead) RoPE region of this tile's stage, the
                    // references in the first bytes of a no-PE chunk of the other CTA's dims (dead as well);
                    // the sender thread copies both once every softmax thread has arrived on PREADY
                    uint8_t* stg = sm + FS_OFF + st * ST_BYTES + ST_ROPE + row * 64;
                    const uint32_t sw = ((uint32_t)row >> 1) & 3u;
                    *reinterpret_cast<uint4*>(stg + (((2u * (uint32_t)hh) ^ sw) << 4)) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
                    *reinterpret_cast<uint4*>(stg + (((2u * (uint32_t)hh + 1u) ^ sw) << 4)) = make_uint4(pw[4], pw[5], pw[6], pw[7]);
                    if (hh == 0) reinterpret_cast<float*>(sm + FS_OFF + st * ST_BYTES + 2u * (1u - (uint32_t)half) * KV_CHUNK)[row] = m_run;
                    fence_proxy_async();
                }
                tmem_st8(lane_addr + TM_S + 64 * b + 8 * hh, pw);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar(BAR_PREADY + b));
                mbar_arrive(bar(BAR_STAGED + (int)st));
                trace(tr, tc, 30 + warp, t);
                ++n_rel; ++rel_req;
                return true;
            };
            // ---- a tile of the other CTA: bring this row's accumulator to the reference of its P' ----
            auto other_tile = [&](uint32_t t) -> bool {
                const uint32_t r = t >> 1, ps = r % NP;
                trace(tr, tc, 20 + warp, t);
                if (!mbar_wait_hot_cluster(bar(BAR_PFULL + (int)ps), (r / NP) & 1u, abort_flag, W_PFULL)) return false;
                trace(tr, tc, 100 + warp, t);
                const float m_in = reinterpret_cast<const volatile float*>(sm + PM_OFF)[ps * 128 + row];
                // m_in == -inf: the tile has no entry for this row, its P' row is zero whatever the reference.
                // A reference above this row's: the accumulator moves up to it (after the products released
                // so far).  A reference below: the accumulator stays and the row's P' is shifted down by the
                // (whole) difference in place, or zeroed when that leaves nothing representable.  References
                // therefore only ever move up and both CTAs settle on the same one.
                const bool up = (m_in != -INFINITY) && (m_run != -INFINITY) && (m_in > m_run);
                if (m_in != -INFINITY && m_run == -INFINITY) m_run = m_in;          // nothing accumulated for this row yet
                if (__any_sync(0xffffffffu, up)) {
                    if (rel_req > 0) { if (!wait_released()) return false; }
                    float alpha = 1.f;
                    if (up) { alpha = ex2(m_run - m_in); m_run = m_in; l_run *= alpha; }
                    if (rel_req > 0) scale_acc(alpha);
                }
                if (m_in != -INFINITY && m_in < m_run) {
                    const float d = m_run - m_in;
                    uint8_t* prow = sm + PS_OFF + ps * PS_BYTES + row * 64;
                    const uint32_t sw = ((uint32_t)row >> 1) & 3u;
                    uint4* c0 = reinterpret_cast<uint4*>(prow + (((2u * (uint32_t)hh) ^ sw) << 4));
                    uint4* c1 = reinterpret_cast<uint4*>(prow + (((2u * (uint32_t)hh + 1u) ^ sw) << 4));
                    if (d > 14.f) {
                        *c0 = make_uint4(0, 0, 0, 0); *c1 = make_uint4(0, 0, 0, 0);
                    } else {
                        const __half2 ratio = __float2half2_rn(ex2(-d));
                        uint4 v0 = *c0, v1 = *c1;
                        v0.x = rescale_e4m3x4(v0.x, ratio); v0.y = rescale_e4m3x4(v0.y, ratio);
                        v0.z = rescale_e4m3x4(v0.z, ratio); v0.w = rescale_e4m3x4(v0.w, ratio);
                        v1.x = rescale_e4m3x4(v1.x, ratio); v1.y = rescale_e4m3x4(v1.y, ratio);
                        v1.z = rescale_e4m3x4(v1.z, ratio); v1.w = rescale_e4m3x4(v1.w, ratio);
                        *c0 = v0; *c1 = v1;
                    }
                }
                fence_proxy_async();
                tc_fence_before();
                mbar_arrive(bar(BAR_ADOPTED + (int)ps));
                trace(tr, tc, 6, t);
                ++n_rel; ++rel_req;
                return true;
            };

            {   // the order of run_sequence, written out (head of own tiles, then rounds)
                const uint32_t t0 = it, n = (uint32_t)w.nblk;
                const uint32_t first_own = owned(t0) ? 0u : 1u, first_oth = 1u - first_own;
                const uint32_t n_own = (n > first_own) ? (n - first_own + 1) / 2 : 0, n_oth = (n > first_oth) ? (n - first_oth + 1) / 2 : 0;
                const uint32_t head = min((first_own == 0u ? 2u : 1u) + 1u, n_own);
                for (uint32_t i = 0; i < head && ok; ++i) ok = own_tile(t0 + first_own + 2 * i);
                const uint32_t rounds = max(n_own - head, n_oth);
                for (uint32_t k = 0; k < rounds && ok; ++k) {
                    if (k < n_oth) ok = other_tile(t0 + first_oth + 2 * k);
                    if (ok && head + k < n_own) ok = own_tile(t0 + first_own + 2 * (head + k));
                }
                it += n;
            }
            if (!ok) break;
            // ---- epilogue ---------------------------------------------------------------------
            {
                ok = wait_released();
                if (!ok) break;
                named_bar_sync(1 + quarter, 64);
                xch[hh * 128 + row] = l_run;
                xch[256 + hh * 128 + row] = x_max;
                named_bar_sync(1 + quarter, 64);
                const float l_own = l_run + xch[(1 - hh) * 128 + row];
                const float x_own = fmaxf(x_max, xch[256 + (1 - hh) * 128 + row]);
                // exchange (l, reference, max logit) with the other CTA: it owns the other tiles
                const uint32_t eb = n_req & 1u;
                if (hh == 0) {
                    const uint32_t e = remote(base + EPI_OFF + eb * (3 * 128 * 4) + (uint32_t)row * 4);
                    st_cluster_f32(e, l_own);
                    st_cluster_f32(e + 128 * 4, m_run);
                    st_cluster_f32(e + 2 * 128 * 4, x_own);
                    mbar_arrive_cluster(remote(bar(BAR_EPI + (int)eb)));
                }
                ok = mbar_wait_hot_cluster(bar(BAR_EPI + (int)eb), (n_req >> 1) & 1u, abort_flag, W_EPI);
                if (!ok) break;
                const volatile float* ep = reinterpret_cast<const volatile float*>(sm + EPI_OFF + eb * (3 * 128 * 4));
                const float l_p = ep[row], m_p = ep[128 + row], x_p = ep[256 + row];
                float l_all = l_own;
                float m_fin = m_run;
                if (l_p > 0.f && m_p != -INFINITY) {
                    if (m_run == -INFINITY) { l_all = l_p; m_fin = m_p; }     // (cannot happen: the other CTA's tiles were adopted)
                    else l_all = l_own + l_p * exp2f(m_p - m_run);
                }
                const float xm = fmaxf(x_own, x_p);
                float lse = (l_all > 0.f) ? (log2f(l_all) - (float)P_SHIFT + m_fin) : NEG_BIG;
                float denom = l_all;
                if (w.no_split && p.attn_sink != nullptr && live) {
                    const float sink2 = p.attn_sink[row] * LOG2E;
                    denom = l_all + ((m_fin == -INFINITY) ? INFINITY : exp2f(sink2 - m_fin + (float)P_SHIFT));
                    if (lse != NEG_BIG) lse += log2f(1.f + exp2f(sink2 - lse));
                    else lse = sink2;
                }
                const float inv = (denom > 0.f) ? 1.f / denom : 0.f;
                const int col0 = half * 256 + hh * 128;
                if (w.no_split) {
                    __nv_bfloat16* dst = p.out + ((size_t)req * p.num_heads + row) * D_V + col0;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + TM_O + 128 * hh + c, o);
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
                    if (live && half == 0 && hh == 0) {
                        p.out_lse[(size_t)req * p.num_heads + row] = lse;
                        if (p.out_max_logits) p.out_max_logits[(size_t)req * p.num_heads + row] = (xm == -INFINITY) ? NEG_BIG : xm;
                    }
                } else {
                    float* dst = p.o_accum + ((size_t)w.split_idx * p.num_heads + row) * D_V + col0;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + TM_O + 128 * hh + c, o);
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
                    if (live && half == 0 && hh == 0) p.lse_accum[(size_t)w.split_idx * p.num_heads + row] = lse;
                }
                named_bar_sync(1 + quarter, 64);
                ++n_req;
            }
        }
    } else if (warp < FX_WARP0) {
        // =================================================================== gather issuers
        // Warp pw gathers rows [16*pw, +16) of every tile.  Owned tile: the whole row (as attn_tc.cu).
        // Other CTA's tile: the 256 no-PE bytes of this CTA's output dims and the scale bytes.
        const int pw = warp - N_SM_WARPS;
        const int row0 = pw * 16;
        const int my_row = row0 + (lane & 15);
        const int pbs_shift = (p.page_block_size & (p.page_block_size - 1)) == 0 ? __ffs(p.page_block_size) - 1 : -1;
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int32_t* idx_row = p.indices + (size_t)req * p.topk;
            auto fetch_idx = [&](int j) -> int {
                const int pos = (w.blk0 + j) * BLOCK_N + my_row;
                return (j < w.nblk && pos < w.len) ? __ldg(idx_row + pos) : -1;
            };
            auto row_ptr = [&](int idx) -> const uint8_t* {
                const unsigned u = (unsigned)idx;
                return (pbs_shift >= 0)
                    ? p.kv + (int64_t)(u >> pbs_shift) * p.block_stride + (int64_t)(u & (unsigned)(p.page_block_size - 1)) * ROW_BYTES
                    : kv_row_ptr(p.kv, idx, p.page_block_size, p.block_stride);
            };
            const uint32_t t0 = it;
            const unsigned long long kv_u = reinterpret_cast<unsigned long long>(p.kv);
            // the index of this lane's row in the next tile of the order is fetched one tile ahead
            int idx_pref = fetch_idx((int)(first_in_sequence(t0, (uint32_t)w.nblk, rank) - t0));
            uint32_t t_next = 0xffffffffu;
            auto src_of = [&](uint32_t) -> unsigned long long {
                const int idx = idx_pref;
                if (t_next != 0xffffffffu) idx_pref = fetch_idx((int)(t_next - t0));
                return idx >= 0 ? reinterpret_cast<unsigned long long>(row_ptr(idx)) : 0ull;
            };
            auto gather_full = [&](uint32_t t) -> bool {
                const uint32_t r = t >> 1, st = r % NS;
                const unsigned long long my_src_u = src_of(t);      // issued before the wait for the stage
                if (r >= (uint32_t)NS) {
                    ok = mbar_wait_hot(bar(BAR_EMPTY + (int)st), ((r / NS) - 1) & 1u, abort_flag, W_EMPTY);
                    if (!ok) return false;
                }
                const uint32_t sbase = base + FS_OFF + st * ST_BYTES;
                trace(tr, tc, 60 + pw, t);
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    unsigned long long srcs[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) srcs[i] = __shfl_sync(0xffffffffu, my_src_u, hb * 8 + i);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = row0 + hb * 8 + i;
                        const uint32_t off = (lane >> 3) * KV_CHUNK + rr * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)rr & 7u)) << 4);
                        const bool v = srcs[i] != 0ull;
                        cp_async16_zfill(sbase + off, reinterpret_cast<const uint8_t*>(v ? srcs[i] + lane * 16 : kv_u), v ? 16u : 0u);
                    }
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const unsigned long long rs = __shfl_sync(0xffffffffu, my_src_u, g * 4 + (lane >> 3));
                    const int rr = row0 + g * 4 + (lane >> 3);
                    const uint32_t off = ST_ROPE + rr * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)rr & 7u)) << 4);
                    const bool v = rs != 0ull;
                    cp_async16_zfill(sbase + off, reinterpret_cast<const uint8_t*>(v ? rs + ROPE_OFF + (lane & 7) * 16 : kv_u), v ? 16u : 0u);
                }
                if (lane < 16) {
                    const bool v = my_src_u != 0ull;
                    cp_async16_zfill(sbase + ST_SCALE + my_row * 16, reinterpret_cast<const uint8_t*>(v ? my_src_u + SCALE_OFF : kv_u), v ? 16u : 0u);
                }
                cp_async_arrive_noinc(bar(BAR_LOADED + (int)st));
                trace(tr, tc, 70 + pw, t);
                return true;
            };
            auto gather_half = [&](uint32_t t) -> bool {
                const uint32_t r = t >> 1, st = r % NS;
                const unsigned long long my_src_u = src_of(t);
                if (r >= (uint32_t)NS) {
                    ok = mbar_wait_hot(bar(BAR_HEMPTY + (int)st), ((r / NS) - 1) & 1u, abort_flag, W_HEMPTY);
                    if (!ok) return false;
                }
                const uint32_t sbase = base + HS_OFF + st * HS_BYTES;
                trace(tr, tc, 64 + pw, t);
                // lanes 0-15 / 16-31: the 16 chunks (256 bytes) of two rows per pass
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rl = 2 * i + (lane >> 4);
                    const unsigned long long rs = __shfl_sync(0xffffffffu, my_src_u, rl);
                    const int rr = row0 + rl;
                    const uint32_t ch = (uint32_t)lane & 15u;      // chunk inside this CTA's 256 bytes
                    const uint32_t off = (ch >> 3) * KV_CHUNK + rr * 128 + (((ch & 7u) ^ ((uint32_t)rr & 7u)) << 4);
                    const bool v = rs != 0ull;
                    cp_async16_zfill(sbase + off, reinterpret_cast<const uint8_t*>(v ? rs + half * 256 + ch * 16 : kv_u), v ? 16u : 0u);
                }
                if (lane < 16) {
                    const bool v = my_src_u != 0ull;
                    cp_async16_zfill(sbase + HS_SCALE + my_row * 16, reinterpret_cast<const uint8_t*>(v ? my_src_u + SCALE_OFF : kv_u), v ? 16u : 0u);
                }
                cp_async_arrive_noinc(bar(BAR_HLOADED + (int)st));
                trace(tr, tc, 74 + pw, t);
                return true;
            };
            ok = run_sequence_ahead(t0, (uint32_t)w.nblk, rank, [&](uint32_t t, bool own, uint32_t tn) -> bool {
                t_next = tn;
                return own ? gather_full(t) : gather_half(t);
            });
            it += w.nblk;
        }
        cp_async_wait_all();
    } else if (warp < MMA_WARP) {
        // =================================================================== tile fix-up
        const int fw = warp - FX_WARP0;
        const int row0 = fw * FX_ROWS;
        const int my_row = row0 + (lane & 7);
        const int blk = lane >> 3;
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            auto fix_full = [&](uint32_t t) -> bool {
                const uint32_t r = t >> 1, st = r % NS;
                ok = mbar_wait_hot(bar(BAR_LOADED + (int)st), (r / NS) & 1u, abort_flag, W_LOADED);
                if (!ok) return false;
                uint8_t* sp = sm + FS_OFF + st * ST_BYTES;
                uint4 rv[2];
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int rr = row0 + g * 4 + (lane >> 3);
                    rv[g] = *reinterpret_cast<const uint4*>(sp + ST_ROPE + rr * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)rr & 7u)) << 4));
                }
                const float4 sc = *reinterpret_cast<const float4*>(sp + ST_SCALE + my_row * 16);
                const float smax = fmaxf(fmaxf(sc.x, sc.y), fmaxf(sc.z, sc.w));
                const bool uneven = (sc.x != smax) | (sc.y != smax) | (sc.z != smax) | (sc.w != smax);
                const float inv_s = (smax > 0.f) ? __uint_as_float(0x7f000000u - __float_as_uint(smax)) : 0.f;
                const float my_ratio = (blk == 0 ? sc.x : (blk == 1 ? sc.y : (blk == 2 ? sc.z : sc.w))) * inv_s;
                __syncwarp();
                if (lane < 8)
                    *reinterpret_cast<float4*>(sp + ST_SCALE + my_row * 16) =
                        make_float4(smax, (smax > 0.f) ? (float)((int)(__float_as_uint(smax) >> 23) - 127) : -INFINITY, inv_s, 0.f);
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int rl = g * 4 + (lane >> 3);
                    const int rr = row0 + rl;
                    const __nv_bfloat162 f = __float2bfloat162_rn(__shfl_sync(0xffffffffu, inv_s, rl));
                    uint4 v = rv[g];
                    v.x = mul_bf16x2(v.x, f); v.y = mul_bf16x2(v.y, f);
                    v.z = mul_bf16x2(v.z, f); v.w = mul_bf16x2(v.w, f);
                    *reinterpret_cast<uint4*>(sp + ST_ROPE + rr * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)rr & 7u)) << 4)) = v;
                }
                uint32_t fix = __ballot_sync(0xffffffffu, uneven && smax > 0.f) & 0xffu;
                while (fix) {
                    const int i = __ffs(fix) - 1;
                    fix &= fix - 1;
                    const int rr = row0 + i;
                    const float ratio_f = __shfl_sync(0xffffffffu, my_ratio, (lane & 24) + i);
                    if (ratio_f != 1.f) {
                        uint4* q4 = reinterpret_cast<uint4*>(sp + blk * KV_CHUNK + rr * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)rr & 7u)) << 4));
                        const __half2 ratio = __float2half2_rn(ratio_f);
                        uint4 v = *q4;
                        v.x = rescale_e4m3x4(v.x, ratio); v.y = rescale_e4m3x4(v.y, ratio);
                        v.z = rescale_e4m3x4(v.z, ratio); v.w = rescale_e4m3x4(v.w, ratio);
                        *q4 = v;
                    }
                }
                fence_proxy_async();
                mbar_arrive(bar(BAR_FULL + (int)st));
                trace(tr, tc, 50, t);
                return true;
            };
            auto fix_half = [&](uint32_t t) -> bool {
                const uint32_t r = t >> 1, st = r % NS;
                // the other CTA's tile: only this CTA's two no-PE chunks are here; bring them to the row scale
                ok = mbar_wait_hot(bar(BAR_HLOADED + (int)st), (r / NS) & 1u, abort_flag, W_HLOADED);
                if (!ok) return false;
                uint8_t* sp = sm + HS_OFF + st * HS_BYTES;
                const float4 sc = *reinterpret_cast<const float4*>(sp + HS_SCALE + my_row * 16);
                const float smax = fmaxf(fmaxf(sc.x, sc.y), fmaxf(sc.z, sc.w));
                const float inv_s = (smax > 0.f) ? __uint_as_float(0x7f000000u - __float_as_uint(smax)) : 0.f;
                // lane = (row lane % 8, local chunk block (lane / 8) % 2); lanes 16-31 mirror lanes 0-15
                const int lb = (lane >> 3) & 1, gb = 2 * half + lb;
                const float my_ratio = (gb == 0 ? sc.x : (gb == 1 ? sc.y : (gb == 2 ? sc.z : sc.w))) * inv_s;
                uint32_t fix = __ballot_sync(0xffffffffu, smax > 0.f && my_ratio != 1.f && lane < 16);
                fix = (fix | (fix >> 8)) & 0xffu;      // rows with at least one of the two chunks to rewrite
                while (fix) {
                    const int i = __ffs(fix) - 1;
                    fix &= fix - 1;
                    const int rr = row0 + i;
                    // 16 chunks of 16 bytes per row: lane l < 16 rewrites chunk l (block l / 8)
                    const float ratio_f = __shfl_sync(0xffffffffu, my_ratio, ((lane >> 3) & 1) * 8 + i);
                    if (lane < 16 && ratio_f != 1.f) {
                        uint4* q4 = reinterpret_cast<uint4*>(sp + (lane >> 3) * KV_CHUNK + rr * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)rr & 7u)) << 4));
                        const __half2 ratio = __float2half2_rn(ratio_f);
                        uint4 v = *q4;
                        v.x = rescale_e4m3x4(v.x, ratio); v.y = rescale_e4m3x4(v.y, ratio);
                        v.z = rescale_e4m3x4(v.z, ratio); v.w = rescale_e4m3x4(v.w, ratio);
                        *q4 = v;
                    }
                }
                fence_proxy_async();
                mbar_arrive(bar(BAR_HFULL + (int)st));
                trace(tr, tc, 54, t);
                return true;
            };
            ok = run_sequence(it, (uint32_t)w.nblk, rank, fix_full, fix_half);
            it += (uint32_t)w.nblk;
        }
    } else if (warp == MMA_WARP && lane == 0) {
        // =================================================================== score MMA issue (owned tiles)
        uint32_t it = 0, rq = 0;
        bool ok = true;
        const uint32_t qr_lo = desc_lo(base + QR_OFF, 16);
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            ok = mbar_wait_thread(bar(BAR_QREADY), rq & 1u, abort_flag, W_QREADY);
            if (!ok) break;
            ++rq;
            for (int j = 0; j < w.nblk && ok; ++j, ++it) {
                if (!owned(it)) continue;
                const uint32_t r = it >> 1, st = r % NS, b = r & 1u;
                if (r >= 2) {   // the P.V that read P' from this score buffer has completed
                    ok = mbar_wait_thread(bar(BAR_PVOWN + (int)b), ((r - 2) >> 1) & 1u, abort_flag, W_PVOWN);
                    if (!ok) break;
                }
                ok = mbar_wait_thread(bar(BAR_FULL + (int)st), (r / NS) & 1u, abort_flag, W_FULL);
                if (!ok) break;
                tc_fence_after();
                trace(tr, tc, 80, it);
                const uint32_t kb_lo = desc_lo(base + FS_OFF + st * ST_BYTES, 16);
                const uint32_t d = tmem + TM_S + 64 * b;
#pragma unroll
                for (int kc = 0; kc < 4; ++kc) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        mma_f8_ts(d, tmem + TM_Q + 32 * kc + 8 * ks,
                                  make_desc(kb_lo + ((kc * KV_CHUNK + ks * 32) >> 4), DESC_HI_SW128), IDESC_QK_F8, (kc | ks) != 0);
                    }
                }
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    mma_f16(d, make_desc(qr_lo + ((ks * 32) >> 4), DESC_HI_SW128),
                            make_desc(kb_lo + ((ST_ROPE + ks * 32) >> 4), DESC_HI_SW128), IDESC_QK_BF16, true);
                }
                tc_commit(bar(BAR_SREADY + (int)b));
                trace(tr, tc, 81, it);
            }
        }
    } else if (warp == MMA_WARP + 1 && lane == 0) {
        // =================================================================== P.V MMA issue (all tiles)
        // Follows the order in which the softmax warps release the tiles (owned tiles one ahead of
        // the other CTA's), so that every wait is a blocking one: an owned tile has P' in tensor
        // memory, a tile of the other CTA has P' in a shared-memory slot and V in the half-tile
        // ring.  After every product it commits to the next barrier of the DONE ring, which is how
        // the softmax warps learn that everything they released has completed.
        uint32_t it = 0, n_issued = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            bool first = true;        // the first product of a request overwrites the accumulator
            auto pv_own = [&](uint32_t t) -> bool {
                const uint32_t r = t >> 1, b = r & 1u, st = r % NS;
                if (!mbar_wait_thread(bar(BAR_PREADY + (int)b), (r >> 1) & 1u, abort_flag, W_PREADY)) return false;
                tc_fence_after();
                const uint32_t vb_lo = desc_lo(base + FS_OFF + st * ST_BYTES + (uint32_t)half * 2 * KV_CHUNK, KV_CHUNK);
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    mma_f8_ts(tmem + TM_O, tmem + TM_S + 64 * b + 8 * ks,
                              make_desc(vb_lo + ((ks * 4096) >> 4), DESC_HI_SW128), IDESC_PV_F8, !(first && ks == 0));
                }
                first = false;
                tc_commit(bar(BAR_EMPTY + (int)st));
                tc_commit(bar(BAR_PVOWN + (int)b));
                tc_commit(bar(BAR_DONE + (int)(n_issued % NDONE)));
                trace(tr, tc, 83, t);
                ++n_issued;
                return true;
            };
            auto pv_other = [&](uint32_t t) -> bool {
                const uint32_t r = t >> 1, ps = r % NP, st = r % NS;
                if (!mbar_wait_thread(bar(BAR_HFULL + (int)st), (r / NS) & 1u, abort_flag, W_HFULL)) return false;
                if (!mbar_wait_thread(bar(BAR_ADOPTED + (int)ps), (r / NP) & 1u, abort_flag, W_ADOPTED)) return false;
                tc_fence_after();
                // every softmax thread has seen this use of the slot: arm the next one
                mbar_arrive_expect_tx(bar(BAR_PFULL + (int)ps), PS_BYTES + 128 * 4);
                const uint32_t vb_lo = desc_lo(base + HS_OFF + st * HS_BYTES, KV_CHUNK);
                const uint32_t pa_lo = desc_lo(base + PS_OFF + ps * PS_BYTES, 16);
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    mma_f8(tmem + TM_O, make_desc(pa_lo + ((ks * 32) >> 4), DESC_HI_SW64),
                           make_desc(vb_lo + ((ks * 4096) >> 4), DESC_HI_SW128), IDESC_PV_F8, !(first && ks == 0));
                }
                first = false;
                tc_commit(bar(BAR_HEMPTY + (int)st));
                tc_commit(remote(bar(BAR_PFREE + (int)ps)));      // the owner may fill the slot again once this product has read it
                tc_commit(bar(BAR_DONE + (int)(n_issued % NDONE)));
                trace(tr, tc, 85, t);
                ++n_issued;
                return true;
            };
            ok = run_sequence(it, (uint32_t)w.nblk, rank, pv_own, pv_other);
            it += (uint32_t)w.nblk;
        }
    } else if (warp == MMA_WARP + 2 && lane == 0) {
        // =================================================================== sender
        // When the softmax warps have released an owned tile (P' staged in the tile's stage), copies
        // the P' image and the references into the other CTA's slot for that tile, once the slot is
        // free (the other CTA's P.V of the tile NP ring positions back has completed).
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            for (int j = 0; j < w.nblk && ok; ++j, ++it) {
                if (!owned(it)) continue;
                const uint32_t r = it >> 1, st = r % NS, ps = r % NP;
                ok = mbar_wait_thread(bar(BAR_STAGED + (int)st), (r / NS) & 1u, abort_flag, W_PREADY);
                if (!ok) break;
                trace(tr, tc, 90, it);
                if (r >= (uint32_t)NP) {
                    ok = mbar_wait_thread_cluster(bar(BAR_PFREE + (int)ps), ((r / NP) - 1) & 1u, abort_flag, W_PFREE);
                    if (!ok) break;
                }
                trace(tr, tc, 91, it);
                const uint32_t rbar = remote(bar(BAR_PFULL + (int)ps));
                const uint32_t stage = base + FS_OFF + st * ST_BYTES;
                bulk_copy_to_cluster(remote(base + PS_OFF + ps * PS_BYTES), stage + ST_ROPE, PS_BYTES, rbar);
                bulk_copy_to_cluster(remote(base + PM_OFF + ps * 128 * 4), stage + 2u * (1u - (uint32_t)half) * KV_CHUNK, 128 * 4, rbar);
                trace(tr, tc, 92, it);
            }
        }
    } else if (warp == MMA_WARP + 3 && lane == 0) {
        // =================================================================== receipt relay
        // The owner of a tile stages P' inside the tile's own stage; it may reuse the stage as
        // soon as the copy has landed here, long before this CTA's softmax warps get to the tile.
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            for (int j = 0; j < w.nblk && ok; ++j, ++it) {
                if (owned(it)) continue;
                const uint32_t r = it >> 1, ps = r % NP;
                ok = mbar_wait_thread_cluster(bar(BAR_PFULL + (int)ps), (r / NP) & 1u, abort_flag, W_PFULL);
                if (!ok) break;
                trace(tr, tc, 93, it);
                mbar_arrive_cluster(remote(bar(BAR_EMPTY + (int)(r % NS))));
            }
        }
    }

    // ------------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();        // the other CTA may still write to this CTA's shared memory and barriers until here
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) {
        atomicCAS(p.status, 0, *abort_flag);
        atomicAdd(p.status + 1, 1);
        p.status[2] = blockIdx.x;
    }
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace

int launch_attn_tc2(const AttnParams& p, cudaStream_t stream) {
    if (p.num_tokens == 0) return 0;
    static bool attr_set[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, attn_tc2_kernel) != cudaSuccess || fa.numRegs != REGS_LAUNCH)
            return set_error(SMLA_E_DEVICE, "attn_tc2_kernel: compiled with %d registers per thread, the warpgroup budgets assume %d",
                             fa.numRegs, REGS_LAUNCH);
        const cudaError_t e = cudaFuncSetAttribute(attn_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_ALLOC);
        if (e != cudaSuccess) return set_error((int)e, "attn_tc2_kernel: cannot reserve %u bytes of shared memory: %s",
                                               SMEM_ALLOC, cudaGetErrorString(e));
        cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        attr_set[dev] = true;
    }
    const int max_pairs = (dev < 64 && sm_count[dev] >= 2) ? sm_count[dev] / 2 : 1;
    const int parts = p.sched ? p.num_parts : (p.num_tokens < max_pairs ? p.num_tokens : max_pairs);
    Trace tr{nullptr, 0, 0};
    get_attn_trace(&tr.buf, &tr.cap);
    if (tr.buf != nullptr) {
        const char* e = getenv("SMLA_TRACE_BLOCK");      // debugging aid: which CTA records the timeline
        tr.block = e ? atoi(e) : 0;
    }
    attn_tc2_kernel<<<2 * parts, TC_THREADS, SMEM_ALLOC, stream>>>(p, tr);
    return check_launch("attn_tc2_kernel");
}

}  // namespace smla
