// Sparse-MLA attention on a pair of SMs (sm_100a): split-KV decode and prefill, tcgen05.mma.cta_group::2.
//
// Work unit.  A cluster of two CTAs owns one scheduler partition (a run of 64-token blocks of
// consecutive requests, see sched.cu; without a scheduler: a contiguous share of the requests).  Every
// MMA runs over the pair with M = 128: CTA r holds half of the (<= 128) query heads and, of every
// 128-token tile, the 64 rows it gathered itself.
//   * Q.K^T:  A = this CTA's Q rows, B = the two CTAs' own gathered rows (N = 128 tokens), so a
//     656-byte row is gathered into ONE shared memory and each CTA receives the scores of its
//     heads against all 128 tokens (lanes 0-63: tokens 0-63, lanes 64-127: tokens 64-127).
//   * P.V:    A = this CTA's P' (64 heads x 128 tokens, shared memory), B = V^T with the N = 256
//     output dims of an MMA split between the CTAs: CTA r supplies dims [256 r, 256 r + 256) of
//     all 128 tokens.  For its own tokens these are bytes it already holds (copied inside shared
//     memory into the V slots); for the partner's tokens it gathers the 256-byte half rows.
//     Each CTA accumulates O for its heads over all 512 dims (lanes 0-63: dims 0-255, lanes
//     64-127: dims 256-511; 256 columns of tensor memory).
// Per token a CTA pair takes in 656 + 2 x 256 bytes instead of 2 x 656, and no score or softmax
// work is duplicated.
//
// Numerics (the FP8 class of the reference's V32 kernels, which quantise Q and P to e4m3:
// csrc/kernel/common/fp8_quant.cuh:44-103, csrc/kernel/decode/decode_v2_kernel.cuh:414-493):
//   * Q no-PE is quantised to e4m3 with one power-of-two scale sq_h per head; Q RoPE stays bf16
//     and is pre-divided by that scale.
//   * K/V bytes are consumed as stored, re-expressed against ONE scale s per 128-token tile: the
//     largest of the 4 x 128 scales of the tile's rows.  A 128-value block with a smaller scale is
//     shifted down (a power-of-two division done on the exponent fields: exact while the shifted
//     value stays a normal e4m3 number; a value that would fall below 2^-6 is cut to the subnormal
//     grid, i.e. it is off by at most 2^-15 of the largest value the tile can hold, which is far
//     below the e4m3 rounding step of the values that dominate a dot product).  K RoPE is
//     pre-divided by s.  One accumulator then holds S = (q . k) / (sq_h * s).
//   * The tile scale of V is folded into the exponent: z = S*sq_h*s*sm_scale*log2e + log2(s),
//     P' = 2^(z - m) with m the (lazily updated) running maximum of z, so that
//     O_acc = sum_t P'_t * Vfp8_t needs no per-tile scale; the denominator is tracked apart as
//     l = sum over tiles of (sum_t P'_t) / s in fp32.  O = O_acc / l, LSE = log2(l) + m (base 2, as
//     the reference).  With one scale per tile the softmax loops read nothing per token.
//   * P' is rounded to e4m3 (times 2^P_SHIFT); the accumulator is rescaled only when a row
//     maximum grows by more than 2^RESCALE_TAU, which is exact because l and O share m.
//   * Invalid entries (index < 0, position >= topk_length) are never loaded: their shared-memory
//     rows are zero-filled and their weight is exactly 0 (NaN-safe, decode_v2_kernel.cuh:262-278).
//
// Warp roles (768 threads per CTA): warps 0-7 softmax + epilogue + Q quantisation (thread = one
// head x 32 tokens of a tile; the four warps that share 32 heads exchange row maxima through
// shared memory), warps 8-11 gather issuers (16-byte cp.async, never waiting for data), warps
// 12-19 tile fix-up (RoPE pre-division, uneven-scale rewrite, per-token scale triples, the copy
// of own V bytes), warp 20 lane 0 issues the score MMAs and warp 21 lane 0 the P.V MMAs -- in
// the even CTA only, which is also where the barriers that collect arrivals from both CTAs
// live.  Completion of MMAs reaches both CTAs through one tcgen05.commit per CTA (no multicast).
// Every wait is bounded; a wait that gives up records a code in status[] and the CTA drains and
// exits.  Warps that meet at a named barrier leave the loop together (a warp whose wait gave up
// still goes to the next named barrier, where all of them see the flag).
#include "attn_common.cuh"
#include "sm100_ptx.cuh"

namespace smla {

namespace {

using namespace ptx;
using namespace attn;

constexpr int N_SM_WARPS = 8, N_PR_WARPS = 4, N_FX_WARPS = 8;
constexpr int N_PRK_WARPS = 2;    // gather: 2 warps for the K part, 2 for the V part
constexpr int N_FXK_WARPS = 4;    // fix-up: 4 warps for own rows, 4 for the partner's
constexpr int FX_WARP0 = N_SM_WARPS + N_PR_WARPS;
constexpr int MMA_WARP = FX_WARP0 + N_FX_WARPS;
constexpr int PAIR_THREADS = (MMA_WARP + 4) * 32;
// Register budgets after the warpgroups trade registers.  setmaxnreg.inc can only draw on what the CTA
// was launched with (PAIR_THREADS x REGS_LAUNCH), so the budgets must fit it or the increase would block
// for ever; the launcher checks the compiled register count against REGS_LAUNCH before it launches.
// With 48 registers the gather and fix-up loops spilled to local memory, which made every step of
// theirs several times slower; the two MMA-issuing threads need few registers, so their warpgroup gives
// up half of its allocation too.
constexpr int REGS_LAUNCH = 80, REGS_SOFTMAX = 136, REGS_OTHER = 56, REGS_MMA = 40;
static_assert(N_SM_WARPS * 32 * REGS_SOFTMAX + (N_PR_WARPS + N_FX_WARPS) * 32 * REGS_OTHER + 128 * REGS_MMA
                  <= PAIR_THREADS * REGS_LAUNCH, "register budgets exceed what the CTA owns");
static_assert(65536 / PAIR_THREADS / 8 * 8 == REGS_LAUNCH, "launch-time registers per thread");

constexpr int TILE_N = 128;            // tokens per tile: two scheduler blocks, 64 rows gathered by each CTA
constexpr int OWN_N = 64;
constexpr int NK = 3, NV = 2;          // K stages (own rows) and V stages (V slots + scale triples)
constexpr int P_SHIFT = 5;             // P' is stored as e4m3(P' * 2^P_SHIFT)
constexpr float RESCALE_TAU = 3.0f;    // lazy-rescale threshold (log2 units); P' <= 2^TAU

// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t CHUNK = OWN_N * 128;              // one 128-dim chunk of 64 rows, K-major 128B swizzle
constexpr uint32_t QR_OFF = 0;                       // Q RoPE bf16: [64 heads x 128 B]
constexpr uint32_t PB_OFF = QR_OFF + CHUNK;          // P' e4m3: 2 buffers x [64 heads x 128 tokens]
constexpr uint32_t KS_OFF = PB_OFF + 2 * CHUNK;      // K stages
constexpr uint32_t KS_ROPE = 4 * CHUNK;              //   RoPE of the own rows
constexpr uint32_t KS_RAW = KS_ROPE + CHUNK;         //   [128 tokens x 16 B] the rows' 4 fp32 scales as gathered (own and partner rows)
constexpr uint32_t KS_BYTES = KS_RAW + TILE_N * 16;  // 43008
constexpr uint32_t VS_OFF = KS_OFF + NK * KS_BYTES;  // V stages
constexpr uint32_t VSLOT = 32 * 128;                 //   slot (kb, nb): 32 tokens x 128 dims, at (2 kb + nb) * VSLOT
constexpr uint32_t VS_RAW = 8 * VSLOT;               //   [128 tokens x 16 B] the rows' scales as gathered (all rows of the tile)
constexpr uint32_t VS_INFO = VS_RAW + TILE_N * 16;   //   tile scale (s, log2 s, 1/s, 0) and the 128 validity bits of the tile
constexpr uint32_t VS_BYTES = VS_INFO + 1024;        // 35840
constexpr uint32_t XCH_OFF = VS_OFF + NV * VS_BYTES; // row-maximum exchange [2][4][64] fp32, then Q scales [64] fp32
constexpr uint32_t XCH_BYTES = 2 * 4 * 64 * 4 + 64 * 4;
constexpr uint32_t BAR_OFF = XCH_OFF + XCH_BYTES;
// barriers (8 B each).  "P" barriers collect arrivals from both CTAs and are used in the even CTA only.
constexpr int BAR_KLOADED = 0, BAR_KFULLP = BAR_KLOADED + NK, BAR_TRIP = BAR_KFULLP + NK, BAR_KEMPTY = BAR_TRIP + NK,
              BAR_VLOADED = BAR_KEMPTY + NK, BAR_VFULLP = BAR_VLOADED + NV, BAR_VEMPTY = BAR_VFULLP + NV,
              BAR_SREADY = BAR_VEMPTY + NV, BAR_SFREEP = BAR_SREADY + 2, BAR_PREADYP = BAR_SFREEP + 2,
              BAR_PVDONE = BAR_PREADYP + 2, BAR_QREADYP = BAR_PVDONE + 2, NBAR = BAR_QREADYP + 1;
constexpr uint32_t MISC_OFF = BAR_OFF + NBAR * 8;    // tmem base (4 B), abort flag (4 B)
constexpr uint32_t SMEM_BYTES = MISC_OFF + 16;
constexpr uint32_t SMEM_ALLOC = SMEM_BYTES + 1024;   // slack for the 1024-byte alignment
static_assert(SMEM_ALLOC <= 227 * 1024, "shared memory budget");
static_assert(KS_BYTES % 1024 == 0 && VS_BYTES % 1024 == 0 && KS_OFF % 1024 == 0, "swizzled tiles need 1024-byte alignment");

constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_O = 0, TM_S = 256, TM_Q = 384;   // O 256 columns; score buffer b at 256 + 64 b; Q no-PE 128 columns

constexpr uint32_t IDESC_QK_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, false, 128, TILE_N);
constexpr uint32_t IDESC_QK_BF16 = instr_desc(FMT_BF16, FMT_BF16, false, false, 128, TILE_N);
constexpr uint32_t IDESC_PV_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, true, 128, 256);
constexpr uint32_t DESC_HI_SW128 = desc_hi(1024, (uint32_t)SWIZZLE_128B);

// give-up codes reported through status[0]
enum { W_KEMPTY = 21, W_KLOADED = 22, W_KFULL = 23, W_TRIP = 24, W_VEMPTY = 25, W_VLOADED = 26, W_VFULL = 27,
       W_SREADY = 28, W_SFREE = 29, W_PREADY = 30, W_PVDONE = 31, W_QREADY = 32 };

#ifdef SMLA_TRACE
// Timeline of one CTA (instrumented builds only): lane 0 of every warp appends (tag, tile, clock) records.
__device__ long long* g_trace_buf = nullptr;   // [warps][cap][2]
__device__ int g_trace_cap = 0;
struct TraceCursor { int n = 0; };
__device__ int g_trace_block = 0;
__device__ __forceinline__ void trace(TraceCursor& c, int tag, int tile) {
    if (g_trace_buf != nullptr && (int)blockIdx.x == g_trace_block && (threadIdx.x & 31) == 0 && c.n < g_trace_cap) {
        long long* slot = g_trace_buf + ((size_t)(threadIdx.x >> 5) * g_trace_cap + c.n) * 2;
        slot[0] = ((long long)tag << 32) | (unsigned)tile;
        slot[1] = clock64();
        ++c.n;
    }
}
#define TRACE(tag, tile) trace(tcur, tag, (int)(tile))
#else
#define TRACE(tag, tile)
#endif
#ifdef SMLA_PROF
// Cycle sum of one phase (bin SMLA_PROF, chosen at compile time) per warp of one CTA, written once at the end:
// PROF(i) adds the time since the last PROF point to the sum when i is the chosen bin.
__device__ long long* g_prof_buf = nullptr;     // [warps][2]: the sum and the kernel's length
__device__ int g_prof_block = 0;
#define PROF(i) { const unsigned now_ = (unsigned)clock(); if ((i) == SMLA_PROF) prof_acc += now_ - prof_last; prof_last = now_; }
#else
#define PROF(i)
#endif

// Scale of a tile and the validity bits of its 128 tokens from their gathered scale words ([128] float4 in
// shared memory; a row that was not loaded has all-zero scales).  Every lane returns the same values.
__device__ __forceinline__ float tile_scale(const uint8_t* raw, int lane, uint32_t (&valid)[4]) {
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 s4 = *reinterpret_cast<const float4*>(raw + (32 * j + lane) * 16);
        const float r = fmaxf(fmaxf(s4.x, s4.y), fmaxf(s4.z, s4.w));
        valid[j] = __ballot_sync(0xffffffffu, r > 0.f);
        m = fmaxf(m, r);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    return m;
}

__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk16) { return row * 128u + ((chunk16 ^ (row & 7u)) << 4); }

// ---------------------------------------------------------------------------------------------
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1) attn_pair_kernel(const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + MISC_OFF + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + MISC_OFF);
    auto bar = [&](int i) -> uint32_t { return base + BAR_OFF + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef SMLA_TRACE
    TraceCursor tcur;
#endif
#ifdef SMLA_PROF
    unsigned prof_acc = 0;
    unsigned prof_last = (unsigned)clock();
    const unsigned prof_start = prof_last;
#endif
    TRACE(1, 0);
    const uint32_t rank = cluster_ctarank();          // 0: the CTA that issues the MMAs
    const int part = blockIdx.x >> 1;
    const SchedMeta meta = load_meta(p, part);
    const int heads_cta = (p.num_heads + 1) >> 1;     // heads per CTA
    const int head0 = (int)rank * heads_cta;

    if (tid == 0) {
        for (int s = 0; s < NK; ++s) {
            mbar_init(bar(BAR_KLOADED + s), N_PRK_WARPS * 32);   // one arrive per issuer thread, when its copies have landed
            mbar_init(bar(BAR_KFULLP + s), 2 * N_FXK_WARPS);
            mbar_init(bar(BAR_TRIP + s), N_FXK_WARPS);
            mbar_init(bar(BAR_KEMPTY + s), 1 + N_FXK_WARPS);     // the score MMAs have read the stage and the own V bytes are copied
        }
        for (int s = 0; s < NV; ++s) {
            mbar_init(bar(BAR_VLOADED + s), (N_PR_WARPS - N_PRK_WARPS) * 32);
            mbar_init(bar(BAR_VFULLP + s), 2 * N_FX_WARPS);
            mbar_init(bar(BAR_VEMPTY + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(BAR_SREADY + b), 1);
            mbar_init(bar(BAR_SFREEP + b), 2 * N_SM_WARPS);
            mbar_init(bar(BAR_PREADYP + b), 2 * N_SM_WARPS);
            mbar_init(bar(BAR_PVDONE + b), 1);
        }
        mbar_init(bar(BAR_QREADYP), 2 * N_SM_WARPS);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc_pair(base + MISC_OFF, TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the partner's barriers exist before anything arrives on them
    tc_fence_after();
    TRACE(6, 0);
    const uint32_t tmem = *tmem_slot;
    auto barp = [&](int i) -> uint32_t { return mapa_shared(bar(i), 0); };   // the even CTA's copy of barrier i

    const int last_req = min(meta.end_req, p.num_tokens - 1);
    // The softmax warps read Q before anything else can start: the other warps, idle until then, ask L2 for this
    // CTA's half of the first request's Q rows (128-byte lines).
    if (warp >= N_SM_WARPS && warp < MMA_WARP && meta.begin_req <= last_req) {
        const uint8_t* q0 = reinterpret_cast<const uint8_t*>(p.q + ((size_t)meta.begin_req * p.num_heads + head0) * D_QK);
        const int lines = (min(heads_cta, max(p.num_heads - head0, 0)) * D_QK * 2 + 127) >> 7;
        for (int i = tid - N_SM_WARPS * 32; i < lines; i += (MMA_WARP - N_SM_WARPS) * 32)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(q0 + (size_t)i * 128));
    }

    if (warp < N_SM_WARPS) setmaxnreg_inc<REGS_SOFTMAX>();
    else if (warp < MMA_WARP) setmaxnreg_dec<REGS_OTHER>();
    else setmaxnreg_dec<REGS_MMA>();
    TRACE(7, 0);

    if (warp < N_SM_WARPS) {
        // =================================================================== softmax + epilogue
        const int quarter = warp & 3, ch = warp >> 2;     // TMEM lane quarter, column half of a score buffer
        const int grp = quarter & 1;                      // warps with equal grp share 32 heads
        const int thalf = quarter >> 1;                   // scores: token half; accumulator: half of the output dims
        const int hrow = grp * 32 + lane;                 // head row inside this CTA
        const int head = head0 + hrow;
        const bool live = hrow < heads_cta && head < p.num_heads;
        const int xpart = thalf * 2 + ch;                 // which of the four partial rows this thread holds
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        float* xch = reinterpret_cast<float*>(sm + XCH_OFF);   // [2][4][64]
        float* sqv = xch + 2 * 4 * 64;                         // [64]
        const bool wide_out = (reinterpret_cast<size_t>(p.out) & 31) == 0;        // rows are 1024 bytes apart
        const bool wide_acc = (reinterpret_cast<size_t>(p.o_accum) & 31) == 0;
        uint32_t it = 0;                                  // running tile counter of this CTA
        bool dead = false;                                // a wait of this warp gave up: no more work, only barriers
        bool stop = false;
        for (int req = meta.begin_req; req <= last_req && !stop; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int nst = (w.nblk + 1) >> 1;
            // ---- Q: warp (quarter, ch) quantises no-PE dims [256*ch, +256) of the 32 heads of its lane quarter into
            // tensor memory (the A operand of a pair MMA wants the CTA's 64 rows twice: quarters 2 and 3 repeat the
            // work of quarters 0 and 1).  The 16x256b store shape takes a row from four lanes: lane (g = lane/4,
            // c = lane%4) holds, for every block i of 32 dims, dims [32i + 8c, +8) of rows g and g + 8 of a 16-row
            // group, which is also how it loads them (16 bytes of bf16 per row and block).
            {
                const int g = lane >> 2, c4 = lane & 3;
#pragma unroll 1
                for (int hf = 0; hf < 2; ++hf) {
                    const int r_a = grp * 32 + 16 * hf + g, r_b = r_a + 8;      // head rows inside the CTA
                    const bool v_a = !dead && r_a < heads_cta && head0 + r_a < p.num_heads;
                    const bool v_b = !dead && r_b < heads_cta && head0 + r_b < p.num_heads;
                    const __nv_bfloat16* src_a = p.q + ((size_t)req * p.num_heads + (v_a ? head0 + r_a : 0)) * D_QK + ch * 256 + c4 * 8;
                    const __nv_bfloat16* src_b = p.q + ((size_t)req * p.num_heads + (v_b ? head0 + r_b : 0)) * D_QK + ch * 256 + c4 * 8;
                    // two passes over the rows' bytes (the second is served by L1/L2): keeping a 16-row group in
                    // registers between the maxima and the quantisation spilled
                    auto absmax8 = [](const uint4& a) {
                        return fmaxf(fmaxf(fmaxf(fabsf(bf16lo(a.x)), fabsf(bf16hi(a.x))), fmaxf(fabsf(bf16lo(a.y)), fabsf(bf16hi(a.y)))),
                                     fmaxf(fmaxf(fabsf(bf16lo(a.z)), fabsf(bf16hi(a.z))), fmaxf(fabsf(bf16lo(a.w)), fabsf(bf16hi(a.w)))));
                    };
                    float am_a = 0.f, am_b = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint4 xa = v_a ? __ldg(reinterpret_cast<const uint4*>(src_a + 32 * i)) : make_uint4(0, 0, 0, 0);
                        const uint4 xb = v_b ? __ldg(reinterpret_cast<const uint4*>(src_b + 32 * i)) : make_uint4(0, 0, 0, 0);
                        am_a = fmaxf(am_a, absmax8(xa)); am_b = fmaxf(am_b, absmax8(xb));
                    }
                    am_a = fmaxf(am_a, __shfl_xor_sync(0xffffffffu, am_a, 1)); am_b = fmaxf(am_b, __shfl_xor_sync(0xffffffffu, am_b, 1));
                    am_a = fmaxf(am_a, __shfl_xor_sync(0xffffffffu, am_a, 2)); am_b = fmaxf(am_b, __shfl_xor_sync(0xffffffffu, am_b, 2));
                    // both column halves of a row agree on one scale (the repeating quarter writes the same values)
                    if (c4 == 0) { xch[ch * 64 + r_a] = am_a; xch[ch * 64 + r_b] = am_b; }
                    named_bar_sync(1 + grp, 128);
                    am_a = fmaxf(am_a, xch[(1 - ch) * 64 + r_a]);
                    am_b = fmaxf(am_b, xch[(1 - ch) * 64 + r_b]);
                    const float sq_a = pow2_ceil(fmaxf(am_a, 1e-4f) * (1.f / 448.f)), sq_b = pow2_ceil(fmaxf(am_b, 1e-4f) * (1.f / 448.f));
                    const float ia = __uint_as_float(0x7f000000u - __float_as_uint(sq_a));   // 1/sq, sq a power of two
                    const float ib = __uint_as_float(0x7f000000u - __float_as_uint(sq_b));
                    if (c4 == 0) { sqv[r_a] = sq_a; sqv[r_b] = sq_b; }
                    if (!dead) {
#pragma unroll 1
                        for (int h4 = 0; h4 < 2; ++h4) {
                            uint32_t wq[16];
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk) {
                                const uint4 a = v_a ? __ldg(reinterpret_cast<const uint4*>(src_a + 32 * (4 * h4 + kk))) : make_uint4(0, 0, 0, 0);
                                const uint4 b4 = v_b ? __ldg(reinterpret_cast<const uint4*>(src_b + 32 * (4 * h4 + kk))) : make_uint4(0, 0, 0, 0);
                                wq[4 * kk + 0] = pack_e4m3x4(bf16lo(a.x) * ia, bf16hi(a.x) * ia, bf16lo(a.y) * ia, bf16hi(a.y) * ia);
                                wq[4 * kk + 1] = pack_e4m3x4(bf16lo(a.z) * ia, bf16hi(a.z) * ia, bf16lo(a.w) * ia, bf16hi(a.w) * ia);
                                wq[4 * kk + 2] = pack_e4m3x4(bf16lo(b4.x) * ib, bf16hi(b4.x) * ib, bf16lo(b4.y) * ib, bf16hi(b4.y) * ib);
                                wq[4 * kk + 3] = pack_e4m3x4(bf16lo(b4.z) * ib, bf16hi(b4.z) * ib, bf16lo(b4.w) * ib, bf16hi(b4.w) * ib);
                            }
                            tmem_st_16x256b_x4(tmem + ((uint32_t)(quarter * 32 + 16 * hf) << 16) + TM_Q + ch * 64 + h4 * 32, wq);
                        }
                    }
                }
                __syncwarp();
                named_bar_sync(1 + grp, 128);   // the scales of the group's 32 rows are in sqv
                // Q RoPE (shared memory, bf16, pre-divided by sq): the two warps of quarter grp store 16 rows each
                if (thalf == 0 && !dead) {
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg) {
                        const int rl = ch * 16 + gg * 4 + (lane >> 3);          // row inside the group's 32
                        const int hr = grp * 32 + rl;
                        uint4 c = make_uint4(0, 0, 0, 0);
                        if (hr < heads_cta && head0 + hr < p.num_heads)
                            c = __ldg(reinterpret_cast<const uint4*>(p.q + ((size_t)req * p.num_heads + head0 + hr) * D_QK + D_NOPE + (lane & 7) * 8));
                        const __nv_bfloat162 f = __float2bfloat162_rn(__uint_as_float(0x7f000000u - __float_as_uint(sqv[hr])));   // 1/sq
                        c.x = mul_bf16x2(c.x, f); c.y = mul_bf16x2(c.y, f); c.z = mul_bf16x2(c.z, f); c.w = mul_bf16x2(c.w, f);
                        *reinterpret_cast<uint4*>(sm + QR_OFF + swz((uint32_t)hr, (uint32_t)lane & 7u)) = c;
                    }
                    fence_proxy_async();
                }
                if (!dead) {
                    tmem_wait_st();
                    tc_fence_before();     // also orders the previous epilogue's TMEM reads before the next MMAs
                }
            }
            if (named_bar_or(1 + grp, 128, dead || *abort_flag != 0)) { stop = true; break; }
            TRACE(2, it);
            PROF(11);
            const float my_sqc = live ? sqv[hrow] * p.sm_scale * LOG2E : 0.f;
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(barp(BAR_QREADYP));

            float m_run = -INFINITY;   // running maximum of z (lags by at most RESCALE_TAU)
            float l_run = 0.f;         // this thread's share of the sum of P'/s (scaled by 2^P_SHIFT)
            float x_max = -INFINITY;   // this thread's share of the maximum of the scaled logits (max_logits output)
            for (int j = 0; j < nst; ++j, ++it) {
                const uint32_t b = it & 1u, vs = it % NV;
                float z[32];
                float mx_loc = -INFINITY, inv_tile = 0.f;
                const uint8_t* info = sm + VS_OFF + vs * VS_BYTES + VS_INFO;
                PROF(0);
                if (!dead) dead = !mbar_wait_hot(bar(BAR_SREADY + b), (it >> 1) & 1u, abort_flag, W_SREADY);
                PROF(1);
                TRACE(10, it);
                if (!dead) dead = !mbar_wait_hot(bar(BAR_TRIP + (it % NK)), (it / NK) & 1u, abort_flag, W_TRIP);
                PROF(2);
                if (!dead) {
                    tc_fence_after();
                    uint32_t sv[32];
                    tmem_ld32(lane_addr + TM_S + 64 * b + 32 * ch, sv);
                    tmem_wait_ld();
                    PROF(3);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(barp(BAR_SFREEP + b));   // the score buffer may be overwritten
                    const float4 ti = *reinterpret_cast<const float4*>(info);                 // (s, log2 s, 1/s, 0) of the tile
                    const uint32_t valid = reinterpret_cast<const uint32_t*>(info + 16)[2 * thalf + ch];   // this thread's 32 tokens
                    const float c_tile = ti.x * my_sqc, off = ti.y;
                    inv_tile = ti.z;
                    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                    for (int t = 0; t < 32; t += 4) {
                        z[t + 0] = fmaf(__uint_as_float(sv[t + 0]), c_tile, off);
                        z[t + 1] = fmaf(__uint_as_float(sv[t + 1]), c_tile, off);
                        z[t + 2] = fmaf(__uint_as_float(sv[t + 2]), c_tile, off);
                        z[t + 3] = fmaf(__uint_as_float(sv[t + 3]), c_tile, off);
                    }
                    if (valid != 0xffffffffu) {     // tokens without an entry: weight exactly 0
#pragma unroll
                        for (int t = 0; t < 32; ++t) z[t] = ((valid >> t) & 1u) ? z[t] : -INFINITY;
                    }
#pragma unroll
                    for (int t = 0; t < 32; t += 4) {
                        mx0 = fmaxf(mx0, fmaxf(z[t], z[t + 1]));
                        mx1 = fmaxf(mx1, fmaxf(z[t + 2], z[t + 3]));
                    }
                    // z - log2(s) is the scaled logit itself
                    if (p.out_max_logits != nullptr && fmaxf(mx0, mx1) > -INFINITY) x_max = fmaxf(x_max, fmaxf(mx0, mx1) - off);
                    mx_loc = fmaxf(mx0, mx1);
                    xch[(b * 4 + xpart) * 64 + hrow] = mx_loc;
                    PROF(4);
                }
                if (named_bar_or(1 + grp, 128, dead || *abort_flag != 0)) { stop = true; break; }   // the four partial row maxima are in place
                const float* xr = xch + b * 256 + hrow;
                const float mx = fmaxf(fmaxf(xr[0], xr[64]), fmaxf(xr[128], xr[192]));
                PROF(5);
                const bool grow = mx > m_run + RESCALE_TAU;   // false while the row has seen no valid entry
                if (__any_sync(0xffffffffu, grow)) {
                    if (j > 0) {   // the accumulator holds earlier tiles: wait for the last P.V, then scale it
                        dead = !mbar_wait_hot(bar(BAR_PVDONE + ((it - 1) & 1u)), ((it - 1) >> 1) & 1u, abort_flag, W_PVDONE);
                        if (dead) continue;
                        tc_fence_after();
                    }
                    const float alpha = grow ? ex2(m_run - mx) : 1.f;   // 2^-inf = 0 for the first tile
                    if (grow) { m_run = mx; l_run *= alpha; }
                    if (j > 0) {
#pragma unroll 1
                        for (int c = 0; c < 128; c += 32) {
                            uint32_t o[32];
                            tmem_ld32(lane_addr + TM_O + 128 * ch + c, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(lane_addr + TM_O + 128 * ch + c, o);
                        }
                        tmem_wait_st();
                    }
                }
                PROF(6);
                if (it >= 2) {   // the P.V that read this P' buffer two tiles ago has completed
                    dead = !mbar_wait_hot(bar(BAR_PVDONE + b), ((it - 2) >> 1) & 1u, abort_flag, W_PVDONE);
                    if (dead) continue;
                }
                PROF(7);
                const float m_off = ((m_run == -INFINITY) ? 0.f : m_run) - (float)P_SHIFT;
                uint32_t pw[8];
                float l0 = 0.f, l1 = 0.f;
#pragma unroll
                for (int t = 0; t < 32; t += 4) {
                    const float p0 = ex2(z[t + 0] - m_off), p1 = ex2(z[t + 1] - m_off);
                    const float p2 = ex2(z[t + 2] - m_off), p3 = ex2(z[t + 3] - m_off);
                    l0 += p0 + p2; l1 += p1 + p3;
                    pw[t >> 2] = pack_e4m3x4(p0, p1, p2, p3);
                }
                l_run = fmaf(l0 + l1, inv_tile, l_run);
                PROF(8);
                // P' of tokens [64*thalf + 32*ch, +32) of head hrow: two 16-byte pieces of the row
                uint8_t* pb = sm + PB_OFF + b * CHUNK;
                *reinterpret_cast<uint4*>(pb + swz(hrow, 4 * thalf + 2 * ch)) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
                *reinterpret_cast<uint4*>(pb + swz(hrow, 4 * thalf + 2 * ch + 1)) = make_uint4(pw[4], pw[5], pw[6], pw[7]);
                fence_proxy_async();
                PROF(9);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(barp(BAR_PREADYP + b));
                PROF(10);
                TRACE(14, it);
            }
            if (stop) break;
            TRACE(3, it);
            // ---- epilogue ---------------------------------------------------------------------
            {
                const uint32_t last = it - 1;
                if (!dead) dead = !mbar_wait_hot(bar(BAR_PVDONE + (last & 1u)), (last >> 1) & 1u, abort_flag, W_PVDONE);
                tc_fence_after();
                if (named_bar_or(1 + grp, 128, dead || *abort_flag != 0)) { stop = true; break; }   // the partners have read the last tile's row maxima
                xch[xpart * 64 + hrow] = l_run;
                xch[256 + xpart * 64 + hrow] = x_max;
                named_bar_sync(1 + grp, 128);
                const float l_all = (xch[hrow] + xch[64 + hrow]) + (xch[128 + hrow] + xch[192 + hrow]);
                const float xm = fmaxf(fmaxf(xch[256 + hrow], xch[320 + hrow]), fmaxf(xch[384 + hrow], xch[448 + hrow]));
                float lse = (l_all > 0.f) ? (log2f(l_all) - (float)P_SHIFT + m_run) : NEG_BIG;
                float denom = l_all;
                if (w.no_split && p.attn_sink != nullptr && live) {
                    const float sink2 = p.attn_sink[head] * LOG2E;
                    denom = l_all + ((m_run == -INFINITY) ? INFINITY : exp2f(sink2 - m_run + (float)P_SHIFT));
                    if (lse != NEG_BIG) lse += log2f(1.f + exp2f(sink2 - lse));
                    else lse = sink2;
                }
                const float inv = (denom > 0.f) ? 1.f / denom : 0.f;
                const int col0 = thalf * 256 + ch * 128;      // first output dim of this thread
                if (w.no_split) {
                    __nv_bfloat16* dst = p.out + ((size_t)req * p.num_heads + (live ? head : 0)) * D_V + col0;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + TM_O + 128 * ch + c, o);
                        tmem_wait_ld();
                        if (live) {
                            uint32_t pk[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
                                pk[i] = *reinterpret_cast<uint32_t*>(&t);
                            }
                            if (wide_out) {
                                const uint32_t lo8[8] = {pk[0], pk[1], pk[2], pk[3], pk[4], pk[5], pk[6], pk[7]};
                                const uint32_t hi8[8] = {pk[8], pk[9], pk[10], pk[11], pk[12], pk[13], pk[14], pk[15]};
                                st_global_v8(dst + c, lo8);
                                st_global_v8(dst + c + 16, hi8);
                            } else {
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    *reinterpret_cast<uint4*>(dst + c + 8 * i) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                            }
                        }
                    }
                    if (live && xpart == 0) {
                        p.out_lse[(size_t)req * p.num_heads + head] = lse;
                        if (p.out_max_logits) p.out_max_logits[(size_t)req * p.num_heads + head] = (xm == -INFINITY) ? NEG_BIG : xm;
                    }
                } else {
                    float* dst = p.o_accum + ((size_t)w.split_idx * p.num_heads + (live ? head : 0)) * D_V + col0;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + TM_O + 128 * ch + c, o);
                        tmem_wait_ld();
                        if (live) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * inv);
                            if (wide_acc) {
#pragma unroll
                                for (int i = 0; i < 32; i += 8) {
                                    const uint32_t v8[8] = {o[i], o[i + 1], o[i + 2], o[i + 3], o[i + 4], o[i + 5], o[i + 6], o[i + 7]};
                                    st_global_v8(dst + c + i, v8);
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; i += 4)
                                    *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                            }
                        }
                    }
                    if (live && xpart == 0) p.lse_accum[(size_t)w.split_idx * p.num_heads + head] = lse;
                }
                tc_fence_before();                  // the accumulator reads precede the next request's first P.V
                named_bar_sync(1 + grp, 128);       // xch is free again
                PROF(12);
                TRACE(4, it);
            }
        }
    } else if (warp < FX_WARP0) {
        // =================================================================== gather issuers
        // Warps 8-9 gather the K part of every tile (this CTA's 64 rows: the 512 no-PE bytes as one coalesced
        // 512-byte request per row, the RoPE bytes, and the scale words of these rows and of the partner's),
        // warps 10-11 the V part (bytes [256 r, +256) of the partner's rows into the V slots, and their scale
        // words).  Each of the two kinds waits only for its own stage to be free, so the V part of a tile
        // starts as soon as the P.V two tiles back has completed.  Nothing here waits for data; rows without
        // an entry are zero-filled.  A warp covers 32 rows in two passes of 16: lanes 0-15 hold the row
        // pointers of this CTA's rows, lanes 16-31 those of the partner's.
        const int pw = warp - N_SM_WARPS;
        const bool k_role = pw < N_PRK_WARPS;
        const int rows0 = (k_role ? pw : pw - N_PRK_WARPS) * 32;     // first of this warp's 32 rows
        const int peer = lane >> 4;                                  // lanes 16-31 look after the partner's rows
        const int pbs_shift = (p.page_block_size & (p.page_block_size - 1)) == 0 ? __ffs(p.page_block_size) - 1 : -1;
        const unsigned long long kv_u = reinterpret_cast<unsigned long long>(p.kv);
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int nst = (w.nblk + 1) >> 1;
            const int32_t* idx_row = p.indices + (size_t)req * p.topk;
            const int lim = min(w.len, (w.blk0 + w.nblk) * BLOCK_N);
            // index of (tile j, pass ps) for this lane: row rows0 + 16 ps + lane % 16 of this CTA or of the partner
            auto fetch_idx = [&](int j, int ps) -> int {
                const int n = (peer ? (1 - (int)rank) : (int)rank) * OWN_N + rows0 + 16 * ps + (lane & 15);
                const int pos = w.blk0 * BLOCK_N + j * TILE_N + n;
                return (j < nst && pos < lim) ? __ldg(idx_row + pos) : -1;
            };
            auto row_ptr = [&](int idx) -> unsigned long long {
                if (idx < 0) return 0ull;      // rows without an entry travel as a null source: their copies zero-fill
                const unsigned u = (unsigned)idx;
                return reinterpret_cast<unsigned long long>(
                    (pbs_shift >= 0)
                        ? p.kv + (int64_t)(u >> pbs_shift) * p.block_stride + (int64_t)(u & (unsigned)(p.page_block_size - 1)) * ROW_BYTES
                        : kv_row_ptr(p.kv, idx, p.page_block_size, p.block_stride));
            };
            int idx_a = fetch_idx(0, 0), idx_b = fetch_idx(0, 1);           // this tile, passes 0 and 1
            int nxt_a = fetch_idx(1, 0), nxt_b = fetch_idx(1, 1);           // next tile
#pragma unroll 1
            for (int k = 0; k < nst && ok; ++k) {
                const uint32_t t_it = it + k;
                const unsigned long long src_a = row_ptr(idx_a), src_b = row_ptr(idx_b);
                idx_a = nxt_a; idx_b = nxt_b;
                nxt_a = fetch_idx(k + 2, 0); nxt_b = fetch_idx(k + 2, 1);
                if (k_role) {
                    const uint32_t ks = t_it % NK;
                    if (t_it >= NK) {
                        ok = mbar_wait_hot(bar(BAR_KEMPTY + ks), ((t_it / NK) - 1) & 1u, abort_flag, W_KEMPTY);
                        if (!ok) break;
                    }
                    const uint32_t kbase = base + KS_OFF + ks * KS_BYTES;
#pragma unroll
                    for (int ps = 0; ps < 2; ++ps) {
                        const unsigned long long my_src_u = ps ? src_b : src_a;
                        const int row0 = rows0 + 16 * ps;
#pragma unroll
                        for (int hb = 0; hb < 2; ++hb) {       // two batches of 8 rows keep the register count low
                            unsigned long long srcs[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) srcs[i] = __shfl_sync(0xffffffffu, my_src_u, hb * 8 + i);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int r = row0 + hb * 8 + i;
                                const bool v = srcs[i] != 0ull;
                                cp_async16_zfill(kbase + (lane >> 3) * CHUNK + swz((uint32_t)r, (uint32_t)lane & 7u),
                                                 reinterpret_cast<const uint8_t*>(v ? srcs[i] + lane * 16 : kv_u), v ? 16u : 0u);
                            }
                        }
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const unsigned long long rs = __shfl_sync(0xffffffffu, my_src_u, g * 4 + (lane >> 3));
                            const int r = row0 + g * 4 + (lane >> 3);
                            const bool v = rs != 0ull;
                            cp_async16_zfill(kbase + KS_ROPE + swz((uint32_t)r, (uint32_t)lane & 7u),
                                             reinterpret_cast<const uint8_t*>(v ? rs + ROPE_OFF + (lane & 7) * 16 : kv_u), v ? 16u : 0u);
                        }
                        {
                            const int n = (peer ? (1 - (int)rank) : (int)rank) * OWN_N + row0 + (lane & 15);   // token index inside the tile
                            const bool v = my_src_u != 0ull;
                            cp_async16_zfill(kbase + KS_RAW + n * 16, reinterpret_cast<const uint8_t*>(v ? my_src_u + SCALE_OFF : kv_u), v ? 16u : 0u);
                        }
                    }
                    cp_async_arrive_noinc(bar(BAR_KLOADED + ks));
                } else {
                    const uint32_t vs = t_it % NV;
                    if (t_it >= NV) {
                        ok = mbar_wait_hot(bar(BAR_VEMPTY + vs), ((t_it / NV) - 1) & 1u, abort_flag, W_VEMPTY);
                        if (!ok) break;
                    }
                    const uint32_t vbase = base + VS_OFF + vs * VS_BYTES;
                    const uint32_t piece = lane & 15;                       // 16-byte piece of the 256-byte half row
#pragma unroll
                    for (int ps = 0; ps < 2; ++ps) {
                        const unsigned long long src_u = ps ? src_b : src_a;
                        const int row0 = rows0 + 16 * ps;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = row0 + 2 * i + peer;                  // partner's row (two rows per instruction)
                            const unsigned long long s = __shfl_sync(0xffffffffu, src_u, 16 + 2 * i + peer);
                            const uint32_t slot = ((2u * (1u - rank) + (uint32_t)(r >> 5)) * 2u + (piece >> 3)) * VSLOT;
                            const bool v = s != 0ull;
                            cp_async16_zfill(vbase + slot + swz((uint32_t)r & 31u, piece & 7u),
                                             reinterpret_cast<const uint8_t*>(v ? s + 256u * rank + piece * 16u : kv_u), v ? 16u : 0u);
                        }
                        {   // scale words of the tile's rows: this CTA's (lanes 0-15) and the partner's (lanes 16-31)
                            const int n = (peer ? (1 - (int)rank) : (int)rank) * OWN_N + row0 + (lane & 15);
                            const bool v = src_u != 0ull;
                            cp_async16_zfill(vbase + VS_RAW + n * 16, reinterpret_cast<const uint8_t*>(v ? src_u + SCALE_OFF : kv_u), v ? 16u : 0u);
                        }
                    }
                    cp_async_arrive_noinc(bar(BAR_VLOADED + vs));
                }
            }
            it += nst;
        }
        cp_async_wait_all();
    } else if (warp < FX_WARP0 + N_FXK_WARPS) {
        // =================================================================== tile fix-up, own rows
        // Warp kf owns rows [16*kf, +16) of this CTA's rows (two groups of 8).  First: RoPE pre-division and
        // uneven-scale rewrite (-> the score MMAs may start).  Then, once the V stage of the tile is free,
        // the scale triples of its 32 tokens (its own rows and the same rows of the partner) and the copy of
        // its rows' V bytes into the V slots (-> the K stage may be refilled).
        const int kf = warp - FX_WARP0;
        const int blk = lane >> 3;
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int nst = (w.nblk + 1) >> 1;
#pragma unroll 1
            for (int k = 0; k < nst && ok; ++k) {
                const uint32_t t_it = it + k, ks = t_it % NK, vs = t_it % NV;
                PROF(0);
                ok = mbar_wait_hot(bar(BAR_KLOADED + ks), (t_it / NK) & 1u, abort_flag, W_KLOADED);
                if (!ok) break;
                PROF(1);
                TRACE(30, t_it);
                uint8_t* kp = sm + KS_OFF + ks * KS_BYTES;
                uint8_t* vp = sm + VS_OFF + vs * VS_BYTES;
                uint32_t valid[4];
                const float s_tile = tile_scale(kp + KS_RAW, lane, valid);
                const float inv_tile = (s_tile > 0.f) ? __uint_as_float(0x7f000000u - __float_as_uint(s_tile)) : 0.f;
                const __nv_bfloat162 rope_f = __float2bfloat162_rn(inv_tile);
                // RoPE of rows [16 kf, +16), pre-divided by the tile scale: 4 passes of 4 rows x 8 chunks
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4* r4 = reinterpret_cast<uint4*>(kp + KS_ROPE + swz((uint32_t)(kf * 16 + g * 4 + (lane >> 3)), (uint32_t)lane & 7u));
                    uint4 v = *r4;
                    v.x = mul_bf16x2(v.x, rope_f); v.y = mul_bf16x2(v.y, rope_f);
                    v.z = mul_bf16x2(v.z, rope_f); v.w = mul_bf16x2(v.w, rope_f);
                    *r4 = v;
                }
                // 128-value blocks whose scale is below the tile scale are shifted onto the tile scale.  Row by row,
                // lane l looks after 16-byte chunk l of the row's 512 bytes (block l / 8); no branches between rows,
                // so that the loads of several rows are in flight together.
#pragma unroll 1
                for (int i0 = 0; i0 < 16; i0 += 4) {      // four rows at a time: their loads are issued before any store
                    uint32_t sub[4];
                    uint4 v[4];
                    uint4* q4[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int row = kf * 16 + i0 + u;
                        const float sc = *reinterpret_cast<const float*>(kp + KS_RAW + (rank * OWN_N + row) * 16 + blk * 4);
                        sub[u] = (sc > 0.f) ? shift_bytes_of_ratio(sc * inv_tile) : 0u;      // 0 for a block that is at the tile scale
                        q4[u] = reinterpret_cast<uint4*>(kp + blk * CHUNK + swz((uint32_t)row, (uint32_t)lane & 7u));
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) if (sub[u] != 0u) v[u] = *q4[u];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (sub[u] != 0u) {
                            v[u].x = shift_down_e4m3x4(v[u].x, sub[u]); v[u].y = shift_down_e4m3x4(v[u].y, sub[u]);
                            v[u].z = shift_down_e4m3x4(v[u].z, sub[u]); v[u].w = shift_down_e4m3x4(v[u].w, sub[u]);
                            *q4[u] = v[u];
                        }
                    }
                }
                PROF(2);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(barp(BAR_KFULLP + ks));
                PROF(3);
                TRACE(31, t_it);
                // the V stage of this tile is free once the P.V NV tiles back has completed
                if (t_it >= NV) {
                    ok = mbar_wait_hot(bar(BAR_VEMPTY + vs), ((t_it / NV) - 1) & 1u, abort_flag, W_VEMPTY);
                    if (!ok) break;
                }
                PROF(4);
                TRACE(32, t_it);
                // the tile's scale and validity bits for the softmax warps
                if (kf == 0 && lane == 0) {
                    *reinterpret_cast<float4*>(vp + VS_INFO) =
                        make_float4(s_tile, (s_tile > 0.f) ? (float)((int)(__float_as_uint(s_tile) >> 23) - 127) : -INFINITY, inv_tile, 0.f);
                    *reinterpret_cast<uint4*>(vp + VS_INFO + 16) = make_uint4(valid[0], valid[1], valid[2], valid[3]);
                }
                // own V bytes: rows [16 kf, +16), this CTA's two chunks -> V slots (same swizzle)
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int pidx = lane + 32 * u;                    // 16 rows x 2 chunks x 8 pieces
                    const uint32_t r = (uint32_t)(kf * 16 + (pidx >> 4)), nb = (uint32_t)(pidx >> 3) & 1u, c = (uint32_t)pidx & 7u;
                    const uint4 v = *reinterpret_cast<const uint4*>(kp + (2u * rank + nb) * CHUNK + swz(r, c));
                    *reinterpret_cast<uint4*>(vp + ((2u * rank + (r >> 5)) * 2u + nb) * VSLOT + swz(r & 31u, c)) = v;
                }
                PROF(5);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar(BAR_TRIP + ks));
                    mbar_arrive(bar(BAR_KEMPTY + ks));
                    mbar_arrive_remote(barp(BAR_VFULLP + vs));
                }
                PROF(6);
                TRACE(33, t_it);
            }
            it += nst;
        }
    } else if (warp < MMA_WARP) {
        // =================================================================== tile fix-up, partner's half rows
        // Warp vf owns rows [16*vf, +16) of the partner's rows in the V slots: uneven-scale rewrite.
        const int vf = warp - FX_WARP0 - N_FXK_WARPS;
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int nst = (w.nblk + 1) >> 1;
#pragma unroll 1
            for (int k = 0; k < nst && ok; ++k) {
                const uint32_t t_it = it + k, vs = t_it % NV;
                PROF(0);
                ok = mbar_wait_hot(bar(BAR_VLOADED + vs), (t_it / NV) & 1u, abort_flag, W_VLOADED);
                if (!ok) break;
                PROF(1);
                TRACE(34, t_it);
                uint8_t* vp = sm + VS_OFF + vs * VS_BYTES;
                uint32_t valid[4];
                const float s_tile = tile_scale(vp + VS_RAW, lane, valid);
                const float inv_tile = (s_tile > 0.f) ? __uint_as_float(0x7f000000u - __float_as_uint(s_tile)) : 0.f;
                // The partner's half rows [16 vf, +16): two rows per pass; lane l looks after row l / 16 of the pair,
                // block (l / 8) % 2 of this CTA's two, 16-byte chunk l % 8.
#pragma unroll 1
                for (int i0 = 0; i0 < 8; i0 += 4) {
                    uint32_t sub[4];
                    uint4 v[4];
                    uint4* q4[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int r = vf * 16 + 2 * (i0 + u) + (lane >> 4);
                        const uint32_t nb = (uint32_t)(lane >> 3) & 1u;
                        const float sc = *reinterpret_cast<const float*>(vp + VS_RAW + ((1 - (int)rank) * OWN_N + r) * 16 + (2 * rank + nb) * 4);
                        sub[u] = (sc > 0.f) ? shift_bytes_of_ratio(sc * inv_tile) : 0u;
                        q4[u] = reinterpret_cast<uint4*>(vp + ((2u * (1u - rank) + (uint32_t)(r >> 5)) * 2u + nb) * VSLOT + swz((uint32_t)r & 31u, (uint32_t)lane & 7u));
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) if (sub[u] != 0u) v[u] = *q4[u];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (sub[u] != 0u) {
                            v[u].x = shift_down_e4m3x4(v[u].x, sub[u]); v[u].y = shift_down_e4m3x4(v[u].y, sub[u]);
                            v[u].z = shift_down_e4m3x4(v[u].z, sub[u]); v[u].w = shift_down_e4m3x4(v[u].w, sub[u]);
                            *q4[u] = v[u];
                        }
                    }
                }
                PROF(2);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(barp(BAR_VFULLP + vs));
                PROF(3);
                TRACE(35, t_it);
            }
            it += nst;
        }
    } else if (warp == MMA_WARP && lane == 0 && rank == 0) {
        // =================================================================== score MMA issue (even CTA)
        uint32_t it = 0, rq = 0;
        bool ok = true;
        const uint32_t qr_lo = desc_lo(base + QR_OFF, 16);
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int nst = (w.nblk + 1) >> 1;
            ok = mbar_wait_thread(bar(BAR_QREADYP), rq & 1u, abort_flag, W_QREADY);
            if (!ok) break;
            ++rq;
            for (int j = 0; j < nst && ok; ++j, ++it) {
                const uint32_t ks = it % NK, b = it & 1u;
                PROF(0);
                if (it >= 2) {
                    ok = mbar_wait_thread(bar(BAR_SFREEP + b), ((it - 2) >> 1) & 1u, abort_flag, W_SFREE);
                    if (!ok) break;
                }
                PROF(1);
                ok = mbar_wait_thread(bar(BAR_KFULLP + ks), (it / NK) & 1u, abort_flag, W_KFULL);
                if (!ok) break;
                PROF(2);
                tc_fence_after();
                TRACE(40, it);
                const uint32_t kb_lo = desc_lo(base + KS_OFF + ks * KS_BYTES, 16);
                const uint32_t d = tmem + TM_S + 64 * b;
#pragma unroll
                for (int kc = 0; kc < 4; ++kc) {
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        mma_pair_f8_ts(d, tmem + TM_Q + 32 * kc + 8 * s,
                                       make_desc(kb_lo + ((kc * CHUNK + s * 32) >> 4), DESC_HI_SW128), IDESC_QK_F8, (kc | s) != 0);
                    }
                }
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    mma_pair_f16(d, make_desc(qr_lo + ((s * 32) >> 4), DESC_HI_SW128),
                                 make_desc(kb_lo + ((KS_ROPE + s * 32) >> 4), DESC_HI_SW128), IDESC_QK_BF16, true);
                }
                tc_commit_pair(bar(BAR_SREADY + b));
                tc_commit_pair(mapa_shared(bar(BAR_SREADY + b), 1));
                tc_commit_pair(bar(BAR_KEMPTY + ks));
                tc_commit_pair(mapa_shared(bar(BAR_KEMPTY + ks), 1));
                PROF(3);
                TRACE(41, it);
            }
        }
    } else if (warp == MMA_WARP + 1 && lane == 0 && rank == 0) {
        // =================================================================== P.V MMA issue (even CTA)
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int nst = (w.nblk + 1) >> 1;
            for (int j = 0; j < nst && ok; ++j, ++it) {
                const uint32_t vs = it % NV, b = it & 1u;
                PROF(0);
                ok = mbar_wait_thread(bar(BAR_PREADYP + b), (it >> 1) & 1u, abort_flag, W_PREADY);
                if (!ok) break;
                PROF(1);
                TRACE(50, it);
                ok = mbar_wait_thread(bar(BAR_VFULLP + vs), (it / NV) & 1u, abort_flag, W_VFULL);
                if (!ok) break;
                PROF(2);
                tc_fence_after();
                TRACE(51, it);
                const uint32_t pa_lo = desc_lo(base + PB_OFF + b * CHUNK, 16);
                const uint32_t vb_lo = desc_lo(base + VS_OFF + vs * VS_BYTES, VSLOT);
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
                    for (int nb = 0; nb < 2; ++nb) {
                        mma_pair_f8(tmem + TM_O + 128 * nb, make_desc(pa_lo + ((kb * 32) >> 4), DESC_HI_SW128),
                                    make_desc(vb_lo + (((2 * kb + nb) * VSLOT) >> 4), DESC_HI_SW128), IDESC_PV_F8, (j | kb) != 0);
                    }
                }
                tc_commit_pair(bar(BAR_VEMPTY + vs));
                tc_commit_pair(mapa_shared(bar(BAR_VEMPTY + vs), 1));
                tc_commit_pair(bar(BAR_PVDONE + b));
                tc_commit_pair(mapa_shared(bar(BAR_PVDONE + b), 1));
                PROF(3);
                TRACE(52, it);
            }
        }
    }

    // ------------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();        // the partner may still arrive on this CTA's barriers until here
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) {
        atomicCAS(p.status, 0, *abort_flag);
        atomicAdd(p.status + 1, 1);
        p.status[2] = blockIdx.x;
    }
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, TMEM_COLS);
    }
    TRACE(5, 0);
#ifdef SMLA_PROF
    if (g_prof_buf != nullptr && (int)blockIdx.x == g_prof_block && lane == 0) {
        g_prof_buf[warp * 2] = prof_acc;
        g_prof_buf[warp * 2 + 1] = (unsigned)clock() - prof_start;
    }
#endif
}

}  // namespace

#ifdef SMLA_TRACE
extern "C" int smla_trace_set(long long* buf, int cap, int block) {
    cudaMemcpyToSymbol(g_trace_buf, &buf, sizeof(buf));
    cudaMemcpyToSymbol(g_trace_cap, &cap, sizeof(cap));
    cudaMemcpyToSymbol(g_trace_block, &block, sizeof(block));
    return (int)cudaGetLastError();
}
#endif
#ifdef SMLA_PROF
extern "C" int smla_prof_set(long long* buf, int block) {
    cudaMemcpyToSymbol(g_prof_buf, &buf, sizeof(buf));
    cudaMemcpyToSymbol(g_prof_block, &block, sizeof(block));
    return (int)cudaGetLastError();
}
#endif

int launch_attn_pair(const AttnParams& p, cudaStream_t stream) {
    if (p.num_tokens == 0) return 0;
    static bool attr_set[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return set_error(SMLA_E_SHAPE, "attn_pair_kernel: device ordinal %d not supported", dev);
    if (!attr_set[dev]) {
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, attn_pair_kernel) != cudaSuccess || fa.numRegs != REGS_LAUNCH)
            return set_error(SMLA_E_DEVICE, "attn_pair_kernel: compiled with %d registers per thread, the warpgroup budgets assume %d",
                             fa.numRegs, REGS_LAUNCH);
        const cudaError_t e = cudaFuncSetAttribute(attn_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_ALLOC);
        if (e != cudaSuccess) return set_error((int)e, "attn_pair_kernel: cannot reserve %u bytes of shared memory: %s",
                                               SMEM_ALLOC, cudaGetErrorString(e));
        cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        attr_set[dev] = true;
    }
    // Without a scheduler the grid is persistent: at most one CTA per SM, each pair walks its share of the requests.
    const int max_pairs = sm_count[dev] >= 2 ? sm_count[dev] / 2 : 1;
    const int parts = p.sched ? p.num_parts : (p.num_tokens < max_pairs ? p.num_tokens : max_pairs);
    attn_pair_kernel<<<2 * parts, PAIR_THREADS, SMEM_ALLOC, stream>>>(p);
    return check_launch("attn_pair_kernel");
}

}  // namespace smla
