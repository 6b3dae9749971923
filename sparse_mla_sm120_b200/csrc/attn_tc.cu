// Sparse-MLA attention on tcgen05 tensor cores (sm_100a): split-KV decode and prefill.
//
// Work unit.  One CTA owns one scheduler partition (a run of 64-token blocks of consecutive
// requests, see sched.cu; without a scheduler: a contiguous share of the requests) and ONE HALF of the 512 output
// dimensions, for all (<= 128) query heads at once: heads are the M = 128 rows of every MMA.
// Tensor memory (512 columns) holds everything that is reused: the fp32 output accumulator
// (128 heads x 256 dims, 256 columns), two 64-column score buffers, and the quantised Q no-PE
// operand (128 rows x 512 e4m3 = 128 columns).  The softmax weights P' are written back over the
// score buffer they came from, so both Q and P' reach the tensor core as TMEM A operands and
// shared memory only carries the gathered KV tiles (five 64-token stages) and Q RoPE.
// The two CTAs of a partition both compute the scores and are launched next to each other so
// that the second gather of a row is served by L2.
//
// Numerics (the FP8 class of the reference's V32 kernels, which quantise Q and P to e4m3:
// csrc/kernel/common/fp8_quant.cuh:44-103, csrc/kernel/decode/decode_v2_kernel.cuh:414-493):
//   * Q no-PE is quantised to e4m3 with one power-of-two scale sq_h per head; Q RoPE stays bf16
//     and is pre-divided by that scale.
//   * K/V bytes are consumed as stored.  A row whose four 128-value tiles carry different
//     scales is re-expressed against its largest scale s_t (a power-of-two shift, exact until the
//     e4m3 subnormal range); K RoPE is pre-divided by s_t.  One accumulator then holds
//     S = (q . k) / (sq_h * s_t) for no-PE (FP8 MMA) and RoPE (BF16 MMA) together.
//     The row scales must be powers of two, as the cache format defines them.
//   * The row scale of V is folded into the exponent: z = S*sq_h*s_t*sm_scale*log2e + log2(s_t),
//     P' = 2^(z - m) with m the (lazily updated) running maximum of z, so that
//     O_acc = sum_t P'_t * Vfp8_t needs no per-tile scale; the denominator is tracked apart as
//     l = sum_t P'_t / s_t in fp32.  O = O_acc / l, LSE = log2(l) + m (base 2, as the reference).
//   * P' is rounded to e4m3 (times 2^P_SHIFT); the accumulator is rescaled only when a row
//     maximum grows by more than 2^RESCALE_TAU, which is exact because l and O share m.
//   * Invalid entries (index < 0, position >= topk_length) are never loaded: their shared-memory
//     rows are zero-filled and their weight is exactly 0 (NaN-safe, decode_v2_kernel.cuh:262-278).
//
// Warp roles (768 threads; the first five warpgroups trade registers with setmaxnreg): warps 0-7
// softmax + epilogue (thread = head row = TMEM lane; warps w and w+4 share a lane quarter and
// split the 64 score columns / the output columns; they also quantise Q, read once, into tensor
// memory at the start of a request), warps 8-11 gather issuers (coalesced 16-byte cp.async into
// 128B-swizzled tiles, never waiting for data), warps 12-19 tile fix-up (per-token scale triples,
// RoPE pre-division, uneven-scale rewrite), warp 20 issues the score MMAs and owns the TMEM
// allocation, warp 21 issues the P.V MMAs (one lane each), warps 22-23 idle.  Waits on the
// per-tile critical path block inside mbarrier.try_wait instead of sleeping between polls.
// Every wait is bounded; a wait that gives up records a code in status[] and the CTA drains and
// exits.
#include "common.cuh"
#include "attn_common.cuh"
#include "sm100_ptx.cuh"

namespace smla {

namespace {

using namespace ptx;
using namespace attn;

constexpr int N_SM_WARPS = 8, N_PR_WARPS = 4, N_FX_WARPS = 8;
constexpr int FX_ROWS = 8;    // rows of a tile per fix-up warp
constexpr int FX_WARP0 = N_SM_WARPS + N_PR_WARPS;
constexpr int MMA_WARP = FX_WARP0 + N_FX_WARPS;
constexpr int TC_THREADS = (MMA_WARP + 4) * 32;   // the two MMA-issuing warps share a warpgroup with two idle warps
// Per-thread register budgets after the warpgroups trade registers.  The MMA warps' warpgroup
// keeps its launch-time allocation (the issuing threads must not spill).  setmaxnreg.inc
// can only draw on what the CTA was launched with (TC_THREADS x REGS_LAUNCH), so the budgets
// must fit it or the increase would block for ever; the launcher checks the compiled register
// count against REGS_LAUNCH before it launches.
constexpr int REGS_LAUNCH = 80, REGS_SOFTMAX = 128, REGS_OTHER = 48;
static_assert(N_SM_WARPS * 32 * REGS_SOFTMAX + (N_PR_WARPS + N_FX_WARPS) * 32 * REGS_OTHER + 128 * REGS_LAUNCH
                  <= TC_THREADS * REGS_LAUNCH, "register budgets exceed what the CTA owns");
static_assert((N_SM_WARPS % 4) == 0 && (N_PR_WARPS % 4) == 0 && (N_FX_WARPS % 4) == 0, "setmaxnreg acts on whole warpgroups");
static_assert(65536 / TC_THREADS / 8 * 8 == REGS_LAUNCH, "launch-time registers per thread");
constexpr int NSTAGE = 5;
constexpr int P_SHIFT = 5;             // P' is stored as e4m3(P' * 2^P_SHIFT)
constexpr float RESCALE_TAU = 3.0f;    // lazy-rescale threshold (log2 units); P' <= 2^TAU

// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t QR_OFF = 0;                       // Q RoPE bf16, K-major 128B swizzle: [128 rows x 128 B]
constexpr uint32_t ST_OFF = QR_OFF + 128 * 128;      // KV stages
constexpr uint32_t KV_CHUNK = 64 * 128;              // one 128-dim chunk of a 64-token tile
constexpr uint32_t ST_ROPE = 4 * KV_CHUNK;           // RoPE tile inside a stage
constexpr uint32_t ST_SCALE = ST_ROPE + 64 * 128;    // [64 x 16 B]: the rows' 4 fp32 scales as gathered; the fix-up replaces
                                                     // them in place by (s_t, log2 s_t, 1/s_t, 0)
constexpr uint32_t ST_BYTES = ST_SCALE + 64 * 16;    // 41984 = 41 * 1024
// Pair exchange [2 buffers][2 halves][128 rows] fp32
constexpr uint32_t XCH_OFF = ST_OFF + NSTAGE * ST_BYTES;
constexpr uint32_t XCH_BYTES = 2 * 2 * 128 * 4;
constexpr uint32_t BAR_OFF = XCH_OFF + XCH_BYTES;
// barriers (8 B each): full[NSTAGE] empty[NSTAGE] loaded[NSTAGE] s_ready[2] p_ready[2] pv_done[2] q_ready
constexpr int BAR_FULL = 0, BAR_EMPTY = NSTAGE, BAR_LOADED = 2 * NSTAGE, BAR_SREADY = 3 * NSTAGE,
              BAR_PREADY = BAR_SREADY + 2, BAR_PVDONE = BAR_PREADY + 2, BAR_QREADY = BAR_PVDONE + 2, NBAR = BAR_QREADY + 1;
constexpr uint32_t MISC_OFF = BAR_OFF + NBAR * 8;    // tmem base (4 B), abort flag (4 B)
constexpr uint32_t SMEM_BYTES = MISC_OFF + 16;
constexpr uint32_t SMEM_ALLOC = SMEM_BYTES + 1024;   // slack for the 1024-byte alignment
static_assert(SMEM_ALLOC <= 227 * 1024, "shared memory budget");
static_assert(ST_BYTES % 1024 == 0 && ST_OFF % 1024 == 0, "swizzled tiles need 1024-byte alignment");

constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_O = 0, TM_S = 256, TM_Q = 384;   // O 256 cols; S buffer b at 256 + 64 b; Q 128 cols

constexpr uint32_t IDESC_QK_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, false, 128, 64);
constexpr uint32_t IDESC_QK_BF16 = instr_desc(FMT_BF16, FMT_BF16, false, false, 128, 64);
constexpr uint32_t IDESC_PV_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, true, 128, 256);
constexpr uint32_t DESC_HI_SW128 = desc_hi(1024, (uint32_t)SWIZZLE_128B);

// give-up codes reported through status[0]
enum { W_EMPTY = 1, W_FULL = 2, W_SREADY = 3, W_PREADY = 4, W_PVDONE = 5, W_QREADY = 6, W_LOADED = 7 };

// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(TC_THREADS, 1) attn_tc_kernel(const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + MISC_OFF + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + MISC_OFF);
    auto bar = [&](int i) -> uint32_t { return base + BAR_OFF + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int part = blockIdx.x >> 1, half = blockIdx.x & 1;
    const SchedMeta meta = load_meta(p, part);

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(bar(BAR_FULL + s), N_FX_WARPS * 32);
            mbar_init(bar(BAR_EMPTY + s), 1);
            mbar_init(bar(BAR_LOADED + s), N_PR_WARPS * 32);       // one arrive per issuer thread, when its copies have landed
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(BAR_SREADY + b), 1); mbar_init(bar(BAR_PREADY + b), N_SM_WARPS * 32);
            mbar_init(bar(BAR_PVDONE + b), 1);
        }
        mbar_init(bar(BAR_QREADY), N_SM_WARPS * 32);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(base + MISC_OFF, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int last_req = min(meta.end_req, p.num_tokens - 1);

    if (warp < N_SM_WARPS) setmaxnreg_inc<REGS_SOFTMAX>();
    else if (warp < MMA_WARP) setmaxnreg_dec<REGS_OTHER>();

    if (warp < N_SM_WARPS) {
        // =================================================================== softmax + epilogue
        const int quarter = warp & 3, hh = warp >> 2;     // TMEM lane quarter, column half
        const int row = quarter * 32 + lane;              // head index == TMEM lane
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        float* xch = reinterpret_cast<float*>(sm + XCH_OFF);   // [2][2][128]
        const bool live = row < p.num_heads;
        const bool wide_out = (reinterpret_cast<size_t>(p.out) & 31) == 0;        // rows are 1024 bytes apart
        const bool wide_acc = (reinterpret_cast<size_t>(p.o_accum) & 31) == 0;
        uint32_t it = 0;                          // running tile counter of this CTA
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            // ---- Q: this warp owns rows [32*quarter, +32) x no-PE dims [256*hh, +256), read once ----
            // The 16x256b store shape takes a row from four lanes: lane (g = lane/4, c = lane%4) holds,
            // for every block i of 32 dims, dims [32i + 8c, +8) of rows g and g + 8 of a 16-row group,
            // which is also how it loads them (16 bytes of bf16 per row and block).  A group is kept
            // in registers between finding its rows' maxima and quantising them.
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
                    // both halves of a row agree on one scale
                    if (c4 == 0) { xch[hh * 128 + r_a] = am_a; xch[hh * 128 + r_b] = am_b; }
                    named_bar_sync(1 + quarter, 64);
                    am_a = fmaxf(am_a, xch[(1 - hh) * 128 + r_a]);
                    am_b = fmaxf(am_b, xch[(1 - hh) * 128 + r_b]);
                    const float sq_a = pow2_ceil(fmaxf(am_a, 1e-4f) * (1.f / 448.f)), sq_b = pow2_ceil(fmaxf(am_b, 1e-4f) * (1.f / 448.f));
                    const float ia = __uint_as_float(0x7f000000u - __float_as_uint(sq_a));   // 1/sq, sq a power of two
                    const float ib = __uint_as_float(0x7f000000u - __float_as_uint(sq_b));
                    if (c4 == 0) { xch[256 + r_a] = sq_a; xch[256 + r_b] = sq_b; }   // the partner warp writes the same values
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
                __syncwarp();   // this warp has written the scales of all 32 rows of its quarter
            }
            const float sq = xch[256 + row];
            const float my_sqc = live ? sq * p.sm_scale * LOG2E : 0.f;
            // Q RoPE: warp (quarter, hh) stores rows [16*hh, +16) of its quarter, pre-divided by sq
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int rl = hh * 16 + g * 4 + (lane >> 3);          // row inside the quarter
                const int h = quarter * 32 + rl;
                uint4 c = make_uint4(0, 0, 0, 0);
                if (h < p.num_heads)
                    c = __ldg(reinterpret_cast<const uint4*>(p.q + ((size_t)req * p.num_heads + h) * D_QK + D_NOPE + (lane & 7) * 8));
                const __nv_bfloat162 f = __float2bfloat162_rn(__uint_as_float(0x7f000000u - __float_as_uint(xch[256 + h])));   // 1/sq
                c.x = mul_bf16x2(c.x, f); c.y = mul_bf16x2(c.y, f); c.z = mul_bf16x2(c.z, f); c.w = mul_bf16x2(c.w, f);
                *reinterpret_cast<uint4*>(sm + QR_OFF + h * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)h & 7u)) << 4)) = c;
            }
            tmem_wait_st();
            fence_proxy_async();
            tc_fence_before();     // also orders the previous epilogue's TMEM reads before the next MMAs
            mbar_arrive(bar(BAR_QREADY));

            float m_run = -INFINITY;   // running maximum of z (lags by at most RESCALE_TAU)
            float l_run = 0.f;         // this half's sum of P'/s_t (scaled by 2^P_SHIFT)
            float x_max = -INFINITY;   // this half's maximum of the scaled logits (max_logits output)
            for (int j = 0; j < w.nblk && ok; ++j, ++it) {
                const uint32_t b = it & 1u, st = it % NSTAGE;
                ok = mbar_wait_hot(bar(BAR_SREADY + b), (it >> 1) & 1u, abort_flag, W_SREADY);
                if (!ok) break;
                // the per-token scale arrays of this stage were published with the tile itself
                ok = (mbar_wait(bar(BAR_FULL + st), (it / NSTAGE) & 1u, abort_flag, W_FULL));
                if (!ok) break;
                tc_fence_after();
                uint32_t sv[32];
                tmem_ld32(lane_addr + TM_S + 64 * b + 32 * hh, sv);
                // per token (s_t, log2 s_t, 1/s_t, 0), published with the tile by the fix-up warps
                const float4* tok = reinterpret_cast<const float4*>(sm + ST_OFF + st * ST_BYTES + ST_SCALE) + 32 * hh;
                tmem_wait_ld();
                float z[32];
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int t = 0; t < 32; t += 4) {
                    const float2 a0 = *reinterpret_cast<const float2*>(tok + t), a1 = *reinterpret_cast<const float2*>(tok + t + 1);
                    const float2 a2 = *reinterpret_cast<const float2*>(tok + t + 2), a3 = *reinterpret_cast<const float2*>(tok + t + 3);
                    z[t + 0] = fmaf(__uint_as_float(sv[t + 0]) * a0.x, my_sqc, a0.y);
                    z[t + 1] = fmaf(__uint_as_float(sv[t + 1]) * a1.x, my_sqc, a1.y);
                    z[t + 2] = fmaf(__uint_as_float(sv[t + 2]) * a2.x, my_sqc, a2.y);
                    z[t + 3] = fmaf(__uint_as_float(sv[t + 3]) * a3.x, my_sqc, a3.y);
                    mx0 = fmaxf(mx0, fmaxf(z[t], z[t + 1]));
                    mx1 = fmaxf(mx1, fmaxf(z[t + 2], z[t + 3]));
                    if (p.out_max_logits != nullptr)   // z - log2(s_t) is the scaled logit itself (NaN for masked entries is ignored by fmaxf)
                        x_max = fmaxf(x_max, fmaxf(fmaxf(z[t] - a0.y, z[t + 1] - a1.y), fmaxf(z[t + 2] - a2.y, z[t + 3] - a3.y)));
                }
                // row maximum over both column halves
                xch[b * 256 + hh * 128 + row] = fmaxf(mx0, mx1);
                named_bar_sync(1 + quarter, 64);   // also: both warps have finished reading S[b]
                const float mx = fmaxf(fmaxf(mx0, mx1), xch[b * 256 + (1 - hh) * 128 + row]);
                const bool grow = mx > m_run + RESCALE_TAU;   // false while the row has seen no valid entry
                if (__any_sync(0xffffffffu, grow)) {
                    if (j > 0) {   // the accumulator holds earlier tiles: wait for the last P.V, then scale it
                        ok = mbar_wait_hot(bar(BAR_PVDONE + ((it - 1) & 1u)), ((it - 1) >> 1) & 1u, abort_flag, W_PVDONE);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    const float alpha = grow ? ex2(m_run - mx) : 1.f;   // 2^-inf = 0 for the first tile
                    if (grow) { m_run = mx; l_run *= alpha; }
                    if (j > 0) {
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
                    }
                }
                const float m_off = ((m_run == -INFINITY) ? 0.f : m_run) - (float)P_SHIFT;
                uint32_t pw[8];
                float l0 = 0.f, l1 = 0.f;
#pragma unroll
                for (int t = 0; t < 32; t += 4) {
                    const float p0 = ex2(z[t + 0] - m_off), p1 = ex2(z[t + 1] - m_off);
                    const float p2 = ex2(z[t + 2] - m_off), p3 = ex2(z[t + 3] - m_off);
                    l0 = fmaf(p0, tok[t].z, l0); l1 = fmaf(p1, tok[t + 1].z, l1);
                    l0 = fmaf(p2, tok[t + 2].z, l0); l1 = fmaf(p3, tok[t + 3].z, l1);
                    pw[t >> 2] = pack_e4m3x4(p0, p1, p2, p3);
                }
                l_run += l0 + l1;
                // P' of tokens [32*hh, +32) goes over the first 16 columns of the score buffer
                tmem_st8(lane_addr + TM_S + 64 * b + 8 * hh, pw);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar(BAR_PREADY + b));
            }
            if (!ok) break;
            // ---- epilogue ---------------------------------------------------------------------
            {
                const uint32_t last = it - 1;
                ok = mbar_wait_hot(bar(BAR_PVDONE + (last & 1u)), (last >> 1) & 1u, abort_flag, W_PVDONE);
                if (!ok) break;
                tc_fence_after();
                named_bar_sync(1 + quarter, 64);   // the partner has read the last tile's row maximum
                xch[hh * 128 + row] = l_run;
                xch[256 + hh * 128 + row] = x_max;
                named_bar_sync(1 + quarter, 64);
                const float l_all = l_run + xch[(1 - hh) * 128 + row];
                const float xm = fmaxf(x_max, xch[256 + (1 - hh) * 128 + row]);
                float lse = (l_all > 0.f) ? (log2f(l_all) - (float)P_SHIFT + m_run) : NEG_BIG;
                float denom = l_all;
                if (w.no_split && p.attn_sink != nullptr && live) {
                    const float sink2 = p.attn_sink[row] * LOG2E;
                    denom = l_all + ((m_run == -INFINITY) ? INFINITY : exp2f(sink2 - m_run + (float)P_SHIFT));
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
                            // a row's 64 bytes of this chunk: two full 32-byte sectors per lane (16-byte
                            // stores, half a sector each, when the output is not 32-byte aligned)
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
                    if (live && half == 0 && hh == 0) p.lse_accum[(size_t)w.split_idx * p.num_heads + row] = lse;
                }
                named_bar_sync(1 + quarter, 64);   // xch is free again
            }
        }
    } else if (warp < FX_WARP0) {
        // =================================================================== gather issuers
        // Warp pw gathers rows [16*pw, +16) of every tile and never waits for data.  Lane l copies
        // 16-byte chunk l of the 512 no-PE bytes of each of those rows (one 512-byte coalesced
        // request per row), chunk l%8 of the RoPE bytes of rows 4g + l/8, and lanes 0-15 the rows'
        // scale words.  Rows without an entry are zero-filled here.  Completion reaches the fix-up
        // warps through the LOADED barrier: one plain arrive per thread (releases the zero fills)
        // plus one arrive that fires when the thread's copies have landed.
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
            int idx_next = fetch_idx(0), idx_next2 = fetch_idx(1);
#pragma unroll 1
            for (int k = 0; k < w.nblk && ok; ++k) {
                const uint32_t t_it = it + k, st = t_it % NSTAGE;
                const int idx = idx_next;
                idx_next = idx_next2;
                idx_next2 = fetch_idx(k + 2);
                // rows without an entry travel as a null source: their copies zero-fill (size 0, nothing is read)
                unsigned long long my_src_u = 0ull;
                if (idx >= 0) my_src_u = reinterpret_cast<unsigned long long>(row_ptr(idx));
                if (t_it >= NSTAGE) {
                    ok = mbar_wait_hot(bar(BAR_EMPTY + st), ((t_it / NSTAGE) - 1) & 1u, abort_flag, W_EMPTY);
                    if (!ok) break;
                }
                const uint32_t sbase = base + ST_OFF + st * ST_BYTES;
                const unsigned long long kv_u = reinterpret_cast<unsigned long long>(p.kv);
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {       // two batches of 8 rows keep the register count low
                    unsigned long long srcs[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) srcs[i] = __shfl_sync(0xffffffffu, my_src_u, hb * 8 + i);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r = row0 + hb * 8 + i;
                        const uint32_t off = (lane >> 3) * KV_CHUNK + r * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)r & 7u)) << 4);
                        const bool v = srcs[i] != 0ull;
                        cp_async16_zfill(sbase + off, reinterpret_cast<const uint8_t*>(v ? srcs[i] + lane * 16 : kv_u), v ? 16u : 0u);
                    }
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const unsigned long long rs = __shfl_sync(0xffffffffu, my_src_u, g * 4 + (lane >> 3));
                    const int r = row0 + g * 4 + (lane >> 3);
                    const uint32_t off = ST_ROPE + r * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)r & 7u)) << 4);
                    const bool v = rs != 0ull;
                    cp_async16_zfill(sbase + off, reinterpret_cast<const uint8_t*>(v ? rs + ROPE_OFF + (lane & 7) * 16 : kv_u), v ? 16u : 0u);
                }
                if (lane < 16) {
                    const bool v = my_src_u != 0ull;
                    cp_async16_zfill(sbase + ST_SCALE + my_row * 16, reinterpret_cast<const uint8_t*>(v ? my_src_u + SCALE_OFF : kv_u), v ? 16u : 0u);
                }
                cp_async_arrive_noinc(bar(BAR_LOADED + st));
            }
            it += w.nblk;
        }
        cp_async_wait_all();
    } else if (warp < MMA_WARP) {
        // =================================================================== tile fix-up
        // Warp fw owns rows [8*fw, +8) of every tile: publishes the per-token scale arrays,
        // re-expresses no-PE tiles that carry a smaller scale than their row, and pre-divides the
        // RoPE part of K by the row scale.  Lane l holds the scales of row l % 8.
        const int fw = warp - FX_WARP0;
        const int row0 = fw * FX_ROWS;
        const int my_row = row0 + (lane & 7);
        const int blk = lane >> 3;
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
#pragma unroll 1
            for (int k = 0; k < w.nblk && ok; ++k, ++it) {
                const uint32_t st = it % NSTAGE;
                ok = mbar_wait_hot(bar(BAR_LOADED + st), (it / NSTAGE) & 1u, abort_flag, W_LOADED);
                if (!ok) break;
                uint8_t* sp = sm + ST_OFF + st * ST_BYTES;
                // RoPE chunks of this lane: 2 passes of 4 rows x 8 chunks
                uint4 rv[2];
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int r = row0 + g * 4 + (lane >> 3);
                    rv[g] = *reinterpret_cast<const uint4*>(sp + ST_ROPE + r * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)r & 7u)) << 4));
                }
                // row scale, validity (a zero-filled scale word marks a row that was not loaded)
                const float4 sc = *reinterpret_cast<const float4*>(sp + ST_SCALE + my_row * 16);
                const float smax = fmaxf(fmaxf(sc.x, sc.y), fmaxf(sc.z, sc.w));
                const bool uneven = (sc.x != smax) | (sc.y != smax) | (sc.z != smax) | (sc.w != smax);
                const float inv_s = (smax > 0.f) ? __uint_as_float(0x7f000000u - __float_as_uint(smax)) : 0.f;
                // ratio of (row lane % 8, block lane / 8) to its row scale: a power of two <= 1
                const float my_ratio = (blk == 0 ? sc.x : (blk == 1 ? sc.y : (blk == 2 ? sc.z : sc.w))) * inv_s;
                __syncwarp();   // every lane has read its row's scales before they are replaced
                if (lane < 8)
                    *reinterpret_cast<float4*>(sp + ST_SCALE + my_row * 16) =
                        make_float4(smax, (smax > 0.f) ? (float)((int)(__float_as_uint(smax) >> 23) - 127) : -INFINITY, inv_s, 0.f);
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int rl = g * 4 + (lane >> 3);
                    const int r = row0 + rl;
                    const __nv_bfloat162 f = __float2bfloat162_rn(__shfl_sync(0xffffffffu, inv_s, rl));
                    uint4 v = rv[g];
                    v.x = mul_bf16x2(v.x, f); v.y = mul_bf16x2(v.y, f);
                    v.z = mul_bf16x2(v.z, f); v.w = mul_bf16x2(v.w, f);
                    *reinterpret_cast<uint4*>(sp + ST_ROPE + r * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)r & 7u)) << 4)) = v;
                }
                // no-PE tiles whose scale is below the row scale: shift them onto the row scale.
                // Lane l rewrites 16-byte chunk l of a flagged row (block l / 8).
                uint32_t fix = __ballot_sync(0xffffffffu, uneven && smax > 0.f) & 0xffu;
                while (fix) {
                    const int i = __ffs(fix) - 1;
                    fix &= fix - 1;
                    const int r = row0 + i;
                    const float ratio_f = __shfl_sync(0xffffffffu, my_ratio, (lane & 24) + i);   // (row i, my block)
                    if (ratio_f != 1.f) {
                        uint4* q4 = reinterpret_cast<uint4*>(sp + blk * KV_CHUNK + r * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)r & 7u)) << 4));
                        const __half2 ratio = __float2half2_rn(ratio_f);
                        uint4 v = *q4;
                        v.x = rescale_e4m3x4(v.x, ratio); v.y = rescale_e4m3x4(v.y, ratio);
                        v.z = rescale_e4m3x4(v.z, ratio); v.w = rescale_e4m3x4(v.w, ratio);
                        *q4 = v;
                    }
                }
                fence_proxy_async();
                mbar_arrive(bar(BAR_FULL + st));
            }
        }
    } else if (warp == MMA_WARP && lane == 0) {
        // =================================================================== score MMA issue
        // One thread runs this role from start to end: the tensor pipe only stays busy while its
        // issuing thread keeps feeding it, so nothing warp-wide sits between two MMAs.  The P.V
        // products are issued by a second thread (below), so that a P' that becomes ready while
        // this thread is blocked on the pipe's queue does not wait for it.  MMAs of different
        // threads are not ordered against each other: score buffer b is rewritten only after the
        // P.V that read P' from it has completed (PVDONE), not merely been issued.
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
                const uint32_t st = it % NSTAGE, b = it & 1u;
                if (it >= 2) {
                    ok = mbar_wait_thread(bar(BAR_PVDONE + b), ((it - 2) >> 1) & 1u, abort_flag, W_PVDONE);
                    if (!ok) break;
                }
                ok = mbar_wait_thread(bar(BAR_FULL + st), (it / NSTAGE) & 1u, abort_flag, W_FULL);
                if (!ok) break;
                tc_fence_after();
                const uint32_t kb_lo = desc_lo(base + ST_OFF + st * ST_BYTES, 16);
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
                tc_commit(bar(BAR_SREADY + b));
            }
        }
    } else if (warp == MMA_WARP + 1 && lane == 0) {
        // =================================================================== P.V MMA issue
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            for (int j = 0; j < w.nblk && ok; ++j, ++it) {
                const uint32_t st = it % NSTAGE, b = it & 1u;
                ok = mbar_wait_thread(bar(BAR_PREADY + b), (it >> 1) & 1u, abort_flag, W_PREADY);
                if (!ok) break;
                tc_fence_after();
                // V = the no-PE bytes of the same stage, read MN-major: 128-dim chunks 8192 B apart,
                // 8-token groups 1024 B apart; this CTA's half of the output dims is two chunks.
                const uint32_t vb_lo = desc_lo(base + ST_OFF + st * ST_BYTES + (uint32_t)half * 2 * KV_CHUNK, KV_CHUNK);
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    mma_f8_ts(tmem + TM_O, tmem + TM_S + 64 * b + 8 * ks,
                              make_desc(vb_lo + ((ks * 4096) >> 4), DESC_HI_SW128), IDESC_PV_F8, (j | ks) != 0);
                }
                tc_commit(bar(BAR_EMPTY + st));
                tc_commit(bar(BAR_PVDONE + b));
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
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace

int launch_attn_tc(const AttnParams& p, cudaStream_t stream) {
    if (p.num_tokens == 0) return 0;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, attn_tc_kernel) != cudaSuccess || fa.numRegs != REGS_LAUNCH)
            return set_error(SMLA_E_DEVICE, "attn_tc_kernel: compiled with %d registers per thread, the warpgroup budgets assume %d",
                             fa.numRegs, REGS_LAUNCH);
        const cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_ALLOC);
        if (e != cudaSuccess) return set_error((int)e, "attn_tc_kernel: cannot reserve %u bytes of shared memory: %s",
                                               SMEM_ALLOC, cudaGetErrorString(e));
        attr_set[dev] = true;
    }
    static int sm_count[64] = {};
    if (dev < 64 && sm_count[dev] == 0) cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    // Without a scheduler the grid is persistent: at most one CTA per SM, each pair walks its share of the requests.
    const int max_pairs = (dev < 64 && sm_count[dev] >= 2) ? sm_count[dev] / 2 : 1;
    const int parts = p.sched ? p.num_parts : (p.num_tokens < max_pairs ? p.num_tokens : max_pairs);
    attn_tc_kernel<<<2 * parts, TC_THREADS, SMEM_ALLOC, stream>>>(p);
    return check_launch("attn_tc_kernel");
}

}  // namespace smla
