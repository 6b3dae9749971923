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
//     all 128 tokens.  These bytes are copied out of the K stages, where the rows already lie in
//     the layout the MMA wants: each CTA sends, with bulk shared-memory copies, the quarter tiles
//     of its own 64 rows to its own V slots and to its partner's (the destination CTA's barrier
//     counts the bytes as they land).  Each CTA accumulates O for its heads over all 512 dims
//     (lanes 0-63: dims 0-255, lanes 64-127: dims 256-511; 256 columns of tensor memory).
// A gathered row enters ONE SM from L2 (656 bytes per token per pair instead of 2 x 656), and no
// score or softmax work is duplicated.
//
// The kernel is a template over the cache layout (656-byte V32 rows, or MODEL1 pages with a scale footer, see Lay<>
// below) and over whether a request also walks a second cache (its blocks follow those of the main cache).
//
// Numerics (the FP8 class of the reference's V32 kernels, which quantise Q and P to e4m3:
// csrc/kernel/common/fp8_quant.cuh:44-103, csrc/kernel/decode/decode_v2_kernel.cuh:414-493):
//   * Q no-PE is quantised to e4m3 with one power-of-two scale sq_h per head; Q RoPE stays bf16
//     and is pre-divided by that scale.
//   * K/V bytes are consumed as stored, re-expressed against ONE scale s per group of eight rows (the
//     rows one gather warp handles): the largest of the 4 x 8 scales of these rows.  A 128-value
//     block with a smaller scale is shifted down (a power-of-two division done on the exponent
//     fields: exact while the shifted value stays a normal e4m3 number; a value that would fall below
//     2^-6 is cut to the subnormal grid, i.e. it is off by at most 2^-15 of the largest value the
//     group can hold, which is far below the e4m3 rounding step of the values that dominate a dot
//     product).  The shift happens in registers on the way from the raw stage to the MMA layout.
//     K RoPE is pre-divided by s.  One accumulator then holds S = (q . k) / (sq_h * s).
//   * The scale of V is folded into the exponent: z = S*sq_h*s*sm_scale*log2e + log2(s),
//     P' = 2^(z - m) with m the (lazily updated) running maximum of z, so that
//     O_acc = sum_t P'_t * Vfp8_t needs no scale; the denominator is tracked apart as
//     l = sum over groups of (sum_t P'_t) / s in fp32.  O = O_acc / l, LSE = log2(l) + m (base 2,
//     as the reference).  A softmax thread's 32 tokens are four such groups, so its loops read four
//     records per tile and nothing per token.
//   * P' is rounded to e4m3 (times 2^P_SHIFT); the accumulator is rescaled only when a row
//     maximum grows by more than 2^RESCALE_TAU, which is exact because l and O share m.
//   * Invalid entries (index < 0, position >= topk_length) are never loaded: their shared-memory
//     rows are zero-filled and their weight is exactly 0 (NaN-safe, decode_v2_kernel.cuh:262-278).
//
// Warp roles (768 threads per CTA):
//   warps 0-7    softmax + epilogue + Q quantisation (thread = one head x 32 tokens of a tile; the four
//                warps that share 32 heads exchange row maxima through shared memory).
//   warps 8-15   gather: warp g reads rows [8 g, +8) of the CTA's 64 from a raw stage (the rows as they
//                lie in the cache) into registers, takes the largest of their scales as the scale of its
//                group, every lane shifts its pieces and stores them in the layout the MMAs read.  The
//                gather warps never wait for each other.
//   warp 16      lane 0 issues the score MMAs, warp 17 lane 0 the P.V MMAs -- in the even CTA only, which
//                is also where the barriers that collect arrivals from both CTAs live.  Completion of
//                MMAs reaches both CTAs through one tcgen05.commit per CTA.
//   warp 19      lane 0 issues the bulk copies K stage -> V slots (own and partner's), sends the half
//                tile's scale records to the partner, waits for the V slots of its CTA to fill and passes
//                that on (V full to the even CTA, K stage free to both).
//   warps 20-23  copy issuers: one bulk copy global -> raw stage per row, two tiles ahead.
// Every wait is bounded; a wait that gives up records a code in status[] and the CTA drains and
// exits.  Warps that meet at a named barrier leave the loop together (a warp whose wait gave up
// still goes to the next named barrier, where all of them see the flag).
#include "attn_common.cuh"
#include "sm100_ptx.cuh"

namespace smla {

namespace {

using namespace ptx;
using namespace attn;

constexpr int N_SM_WARPS = 8, N_G_WARPS = 8;
constexpr int RPW = 64 / N_G_WARPS;     // rows of a tile per gather warp
constexpr int MMA_WARP = N_SM_WARPS + N_G_WARPS;
constexpr int FWD_WARP = MMA_WARP + 3;
constexpr int PROD_WARP0 = MMA_WARP + 4, N_P_WARPS = 4;      // copy issuers: warp p looks after the rows of gather warps 2 p and 2 p + 1
constexpr int PAIR_THREADS = (PROD_WARP0 + N_P_WARPS) * 32;
// Register budgets after the warpgroups trade registers.  setmaxnreg.inc can only draw on what the CTA
// was launched with (PAIR_THREADS x REGS_LAUNCH), so the budgets must fit it or the increase would block
// for ever; the launcher checks the compiled register count against REGS_LAUNCH before it launches.
// A gather thread keeps 8 + 2 sixteen-byte pieces in flight; the MMA-issuing and copy threads need few
// registers, so their warpgroup gives up more than half of its allocation.
constexpr int REGS_LAUNCH = 80, REGS_SOFTMAX = 120, REGS_GATHER = 80, REGS_MMA = 40, REGS_PROD = 40;
static_assert(N_SM_WARPS * 32 * REGS_SOFTMAX + N_G_WARPS * 32 * REGS_GATHER + 128 * REGS_MMA + N_P_WARPS * 32 * REGS_PROD
                  <= PAIR_THREADS * REGS_LAUNCH, "register budgets exceed what the CTA owns");
static_assert(65536 / PAIR_THREADS / 8 * 8 == REGS_LAUNCH, "launch-time registers per thread");

constexpr int TILE_N = 128;            // tokens per tile: two scheduler blocks, 64 rows gathered by each CTA
constexpr int OWN_N = 64;
constexpr int NK = 2, NV = 1, NR = 2;  // K stages (own rows, MMA layout), V stages (V slots), raw stages (own rows as they lie in the cache)
constexpr int P_SHIFT = 5;             // P' is stored as e4m3(P' * 2^P_SHIFT)
constexpr float RESCALE_TAU = 3.0f;    // lazy-rescale threshold (log2 units); P' <= 2^TAU

// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t CHUNK = OWN_N * 128;              // one 128-dim chunk of 64 rows, K-major 128B swizzle
constexpr uint32_t QR_OFF = 0;                       // Q RoPE bf16: [64 heads x 128 B]
constexpr uint32_t PB_OFF = QR_OFF + CHUNK;          // P' e4m3: 2 buffers x [64 heads x 128 tokens]
constexpr uint32_t KS_OFF = PB_OFF + 2 * CHUNK;      // K stages
constexpr uint32_t KS_ROPE = 4 * CHUNK;              //   RoPE of the own rows
constexpr uint32_t KS_BYTES = KS_ROPE + CHUNK;       // 40960
constexpr uint32_t VS_OFF = KS_OFF + NK * KS_BYTES;  // V stages
constexpr uint32_t VSLOT = 32 * 128;                 //   slot (kb, nb): 32 tokens x 128 dims, at (4 nb + kb) * VSLOT
constexpr uint32_t VS_BYTES = 8 * VSLOT;             // 32768
constexpr uint32_t RAW_OFF = VS_OFF + NV * VS_BYTES; // raw stages: [64 rows x 656 B] as they lie in the cache
constexpr uint32_t RAW_BYTES = OWN_N * ROW_BYTES;    // 41984
constexpr int INFO_RING = 8;                         // half-tile records outlive their K stage: the softmax reads them after the scores
constexpr uint32_t INFO_HALF = N_G_WARPS * 16;       // a half tile's record: per gather warp (s, log2 s, 1/s, validity bits) of its RPW rows
constexpr uint32_t INFO_OFF = RAW_OFF + NR * RAW_BYTES;  // [INFO_RING][2 halves] x INFO_HALF
constexpr uint32_t XCH_OFF = INFO_OFF + INFO_RING * 2 * INFO_HALF; // row-maximum exchange [2][4][64] fp32, then Q scales [64] fp32
constexpr uint32_t XCH_BYTES = 2 * 4 * 64 * 4 + 64 * 4;
constexpr uint32_t BAR_OFF = XCH_OFF + XCH_BYTES;
// barriers (8 B each).  "P" barriers collect arrivals from both CTAs and are used in the even CTA only.
constexpr int BAR_KSTORED = 0, BAR_KFULLP = BAR_KSTORED + NK, BAR_KEMPTY = BAR_KFULLP + NK,
              BAR_VFULL = BAR_KEMPTY + NK, BAR_VFULLP = BAR_VFULL + NV, BAR_VEMPTY = BAR_VFULLP + NV,
              BAR_INFO = BAR_VEMPTY + NV, BAR_SREADY = BAR_INFO + INFO_RING, BAR_SFREEP = BAR_SREADY + 2,
              BAR_PREADYP = BAR_SFREEP + 2, BAR_PVDONE = BAR_PREADYP + 2, BAR_QREADYP = BAR_PVDONE + 2,
              BAR_RAWFULL = BAR_QREADYP + 1, BAR_RAWEMPTY = BAR_RAWFULL + NR * N_P_WARPS, BAR_QSTAGE = BAR_RAWEMPTY + NR * N_P_WARPS,
              BAR_QFREE = BAR_QSTAGE + 1, NBAR = BAR_QFREE + 1;
constexpr uint32_t MISC_OFF = BAR_OFF + NBAR * 8;    // tmem base (4 B), abort flag (4 B)
constexpr uint32_t SMEM_BYTES = MISC_OFF + 16;
constexpr uint32_t SMEM_ALLOC = SMEM_BYTES + 1024;   // slack for the 1024-byte alignment
static_assert(SMEM_ALLOC <= 227 * 1024, "shared memory budget");
static_assert(KS_BYTES % 1024 == 0 && VS_BYTES % 1024 == 0 && KS_OFF % 1024 == 0, "swizzled tiles need 1024-byte alignment");
constexpr uint32_t QSTAGE_OFF = KS_OFF + KS_BYTES;   // the staged Q rows of the first request: K stage 1 and the V stage behind it
static_assert(NK == 2 && (NK - 1) * KS_BYTES + NV * VS_BYTES >= OWN_N * D_QK * 2, "K stage 1 + V stage hold the staged Q rows of a CTA");
static_assert(RPW == 8, "a softmax thread reads the records of four groups of eight tokens");
static_assert(BAR_OFF % 8 == 0 && INFO_OFF % 16 == 0 && RAW_OFF % 16 == 0 && RAW_BYTES % 16 == 0, "alignment of barriers and bulk-copied records");

constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_O = 0, TM_S = 256, TM_Q = 384;   // O 256 columns; score buffer b at 256 + 64 b; Q no-PE 128 columns

constexpr uint32_t IDESC_QK_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, false, 128, TILE_N);
constexpr uint32_t IDESC_QK_BF16 = instr_desc(FMT_BF16, FMT_BF16, false, false, 128, TILE_N);
constexpr uint32_t IDESC_PV_F8 = instr_desc(FMT_E4M3, FMT_E4M3, false, true, 128, 256);
constexpr uint32_t DESC_HI_SW128 = desc_hi(1024, (uint32_t)SWIZZLE_128B);

// give-up codes reported through status[0]
enum { W_QSTAGE = 33, W_QFREE = 34, W_RAWEMPTY = 35, W_RAWFULL = 36, W_KEMPTY = 21, W_KSTORED = 22, W_KFULL = 23, W_INFO = 24, W_VEMPTY = 25, W_VFULL_CTA = 26, W_VFULL = 27,
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
#ifdef SMLA_TRACE_FROM             // only the trace points with tags in [SMLA_TRACE_FROM, SMLA_TRACE_TO): the other roles keep their registers
#define TRACE(tag, tile) { if ((tag) >= SMLA_TRACE_FROM && (tag) < SMLA_TRACE_TO) trace(tcur, tag, (int)(tile)); }
#else
#define TRACE(tag, tile) trace(tcur, tag, (int)(tile))
#endif
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

__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk16) { return row * 128u + ((chunk16 ^ (row & 7u)) << 4); }

// What differs between the two cache layouts (csrc/model/kv_cache_traits.cuh:20-111).
//   V32:    a row is 512 e4m3 | 4 fp32 scales (one per 128 values) | 64 bf16 RoPE = 656 bytes; q has 576 dims, V is the
//           512 no-PE values.
//   MODEL1: a row is 448 e4m3 | 64 bf16 RoPE = 576 bytes, its 7 UE8M0 scales (one per 64 values, + 1 pad byte) lie
//           in the page's footer; q has 512 dims and V is the whole row, RoPE included.  The kernel keeps the layout
//           of the stages: the no-PE bytes fill chunks 0-2 and the lower half of chunk 3, and the row's RoPE,
//           quantised to e4m3 against the group's scale, fills the upper half of chunk 3, so that the V copies and
//           the P.V MMAs are the same; the score MMAs skip the upper half of chunk 3 and use the bf16 RoPE.
template <int LAYOUT> struct Lay;
template <> struct Lay<SMLA_LAYOUT_V32> {
    static constexpr bool M1 = false;
    static constexpr int QD = D_QK, NOPE = D_NOPE, DATA = ROW_BYTES, ROPE_AT = ROPE_OFF;
};
template <> struct Lay<SMLA_LAYOUT_MODEL1> {
    static constexpr bool M1 = true;
    static constexpr int QD = SMLA_M1_D_QK, NOPE = 448, DATA = SMLA_M1_DATA_BYTES, ROPE_AT = 448;
};

// Where row idx of a cache lies: the page's first byte (by reference) and the row's number inside the page.
struct CacheGeom {
    const uint8_t* base;
    int64_t stride;
    int pbs, shift;    // rows per page; log2 of it, or -1 when it is not a power of two
};
__device__ __forceinline__ CacheGeom cache_geom(const uint8_t* base, int64_t stride, int pbs) {
    CacheGeom c;
    c.base = base; c.stride = stride; c.pbs = pbs;
    c.shift = (pbs & (pbs - 1)) == 0 ? __ffs(pbs) - 1 : -1;
    return c;
}
__device__ __forceinline__ const uint8_t* cache_page(const CacheGeom& c, int idx, unsigned& in) {
    const unsigned u = (unsigned)idx;
    const unsigned blk = c.shift >= 0 ? (u >> c.shift) : u / (unsigned)c.pbs;
    in = u - blk * (unsigned)c.pbs;
    return c.base + (int64_t)blk * c.stride;
}

// Entry r of this CTA's rows of tile j of a request (block blk0 + 2 j + rank of the request).  EXTRA = false: the
// request walks the main cache only, `lim` is the end of its share of the index row.
template <bool EXTRA>
__device__ __forceinline__ int tile_entry(const AttnParams& p, const Work& w, int j, int rank, int r, int nst, int lim) {
    if (EXTRA) return fetch_entry(p, w, w.blk0 + 2 * j + rank, r);
    const int pos = w.blk0 * BLOCK_N + j * TILE_N + rank * OWN_N + r;
    return (j < nst && pos < lim) ? __ldg(p.indices + (size_t)w.req * p.topk + pos) : -1;
}

// STAGE_Q: the Q rows of a partition's first request come in by one bulk copy into shared memory (see below) instead
// of being read from global memory by the softmax warps (after an L2 prefetch that the copy warps issue as soon as the
// partition is known).  The copy wins where the kernel follows the scheduler and partitions are short (one request
// cut into eight partitions: 28.7 against 30.7 us); without a scheduler (whole requests per partition) reading wins or
// draws: the copy occupies K stage 1 and the V stage until Q is quantised, and the waits it adds to the loops of the
// gather warps and of the copy thread, never taken after the first tiles, cost prefill 6 % (64 requests 53.7 = 53.9 us,
// two query tokens per request 98.5 against 102.4, 4096 query tokens 2.24 against 2.37 ms).
template <int LAYOUT, bool EXTRA, bool STAGE_Q>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1) attn_pair_kernel(const AttnParams p) {
    using L = Lay<LAYOUT>;
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
    const int heads_cta = (p.num_heads + 1) >> 1;     // heads per CTA
    const int head0 = (int)rank * heads_cta;

    if (tid == 0) {
        mbar_init(bar(BAR_QSTAGE), 1);
        mbar_init(bar(BAR_QFREE), 2 * N_SM_WARPS);   // both CTAs' softmax warps: the partner's copies land in this CTA's V stage too
        for (int s = 0; s < NK; ++s) {
            mbar_init(bar(BAR_KSTORED + s), N_G_WARPS);          // this CTA's rows of the stage are in shared memory
            mbar_init(bar(BAR_KFULLP + s), 2 * N_G_WARPS);       // both CTAs' rows are
            mbar_init(bar(BAR_KEMPTY + s), 3);                   // the score MMAs have read the stage; both CTAs' V slots hold its copies
        }
        for (int s = 0; s < NV; ++s) {
            mbar_init(bar(BAR_VFULL + s), 1);                    // + the bytes of the four quarter tiles copied into this CTA's slots
            mbar_init(bar(BAR_VFULLP + s), 2);
            mbar_init(bar(BAR_VEMPTY + s), 1);
        }
        for (int s = 0; s < INFO_RING; ++s) mbar_init(bar(BAR_INFO + s), 1);   // + the bytes of the partner's record
        for (int s = 0; s < NR * N_P_WARPS; ++s) {
            mbar_init(bar(BAR_RAWFULL + s), 1);        // + the bytes of a copy warp's 16 rows of a raw stage
            mbar_init(bar(BAR_RAWEMPTY + s), 16 / RPW); // the gather warps that read these 16 rows have them in registers
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

    // Everything above needs nothing from the kernels before this one.  From here on the scheduler's records are
    // read (when this kernel was launched as a dependent of the scheduler kernel it may have started before that
    // one finished), and the kernel after this one may start its own prologue.
    grid_dep_wait();
    grid_dep_launch();
    const SchedMeta meta = load_meta(p, part);
    // The Q rows of the first request (this CTA's heads: one contiguous piece of global memory) come in by one bulk
    // copy into K stage 1 and the V stage behind it, which nothing needs before the second tile is stored and the
    // first tile's V copies are issued; the softmax warps then quantise Q out of shared memory instead of waiting
    // for global memory several times in a row.  K stage 0 takes the first tile meanwhile.
    const int last_req = min(meta.end_req, p.num_tokens - 1);
    const int live_heads = min(heads_cta, max(p.num_heads - head0, 0));
    Work w_first;
    const bool first_work = STAGE_Q && meta.begin_req <= last_req && get_work(p, meta, meta.begin_req, w_first);   // the same in both CTAs
    const bool q_staged = first_work && live_heads > 0;
    if (tid == 0 && q_staged) {
        const uint32_t bytes = (uint32_t)live_heads * L::QD * 2;
        mbar_arrive_expect_tx(bar(BAR_QSTAGE), bytes);
        bulk_copy_g2s(base + QSTAGE_OFF, reinterpret_cast<unsigned long long>(p.q + ((size_t)meta.begin_req * p.num_heads + head0) * L::QD),
                      bytes, bar(BAR_QSTAGE));
    }

    if (!STAGE_Q && warp >= PROD_WARP0 && meta.begin_req <= last_req) {
        // no staging: ask L2 for the first request's Q rows now (the copy warps have nothing to do yet); the softmax
        // warps read them a few thousand cycles from here
        const uint8_t* q0 = reinterpret_cast<const uint8_t*>(p.q + ((size_t)meta.begin_req * p.num_heads + head0) * L::QD);
        const int lines = (live_heads * L::QD * 2 + 127) >> 7;
        for (int i = tid - PROD_WARP0 * 32; i < lines; i += N_P_WARPS * 32)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(q0 + (size_t)i * 128));
    }
    if (warp < N_SM_WARPS) setmaxnreg_inc<REGS_SOFTMAX>();
    else if (warp < MMA_WARP) setmaxnreg_dec<REGS_GATHER>();
    else if (warp < PROD_WARP0) setmaxnreg_dec<REGS_MMA>();
    else setmaxnreg_dec<REGS_PROD>();
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
        // A request's epilogue runs after the NEXT request's Q phase: Q and its scales are free as soon as the last
        // scores of a request have been read, the accumulator only when its last P.V has completed, so the next
        // request's Q is quantised while that P.V runs and its first score MMAs run while the output is written.
        bool prev_valid = false, prev_no_split = false;
        int prev_req = 0, prev_split = 0;
        uint32_t prev_last = 0;
        float prev_m = 0.f, prev_l = 0.f, prev_x = 0.f;
        for (int req = meta.begin_req; req <= last_req + 1 && !stop; ++req) {
            Work w;
            const bool have = req <= last_req && get_work(p, meta, req, w);
            if (req <= last_req && !have) continue;
            const int nst = have ? (w.nblk + 1) >> 1 : 0;
            float my_sqc = 0.f;
            if (have) {
            if (prev_valid) named_bar_sync(1 + grp, 128);      // the group has read the last tile's row maxima: xch may be reused
            // ---- Q: warp (quarter, ch) quantises no-PE dims [256*ch, +256) of the 32 heads of its lane quarter into
            // tensor memory (the A operand of a pair MMA wants the CTA's 64 rows twice: quarters 2 and 3 repeat the
            // work of quarters 0 and 1).  The 16x256b store shape takes a row from four lanes: lane (g = lane/4,
            // c = lane%4) holds, for every block i of 32 dims, dims [32i + 8c, +8) of rows g and g + 8 of a 16-row
            // group, which is also how it loads them (16 bytes of bf16 per row and block).
            {
                const int g = lane >> 2, c4 = lane & 3;
                const bool from_smem = STAGE_Q && q_staged && req == meta.begin_req;
                if (from_smem && !dead) dead = !mbar_wait_hot(bar(BAR_QSTAGE), 0u, abort_flag, W_QSTAGE);
                // row (head0 + r) of the request's Q, wherever it lies
                const __nv_bfloat16* qrows = from_smem ? reinterpret_cast<const __nv_bfloat16*>(sm + QSTAGE_OFF) - (size_t)head0 * L::QD
                                                       : p.q + (size_t)req * p.num_heads * L::QD;
                // blocks of 32 dims of this warp's 256 that are no-PE dims (MODEL1: 448 = 256 + 6 x 32; the rest stays zero and no MMA reads it)
                const int nblk32 = !L::M1 ? 8 : ((L::NOPE - ch * 256 >= 256) ? 8 : (L::NOPE - ch * 256) / 32);
#pragma unroll 1
                for (int hf = 0; hf < 2; ++hf) {
                    const int r_a = grp * 32 + 16 * hf + g, r_b = r_a + 8;      // head rows inside the CTA
                    const bool v_a = !dead && r_a < heads_cta && head0 + r_a < p.num_heads;
                    const bool v_b = !dead && r_b < heads_cta && head0 + r_b < p.num_heads;
                    const __nv_bfloat16* src_a = qrows + (size_t)(head0 + (v_a ? r_a : 0)) * L::QD + ch * 256 + c4 * 8;
                    const __nv_bfloat16* src_b = qrows + (size_t)(head0 + (v_b ? r_b : 0)) * L::QD + ch * 256 + c4 * 8;
                    // One pass: all 16 loads of the lane are issued before the first is used (one round of latency) and the
                    // pieces stay in registers between the maxima (packed bf16 arithmetic, exact) and the quantisation.
                    // Two copies of the loads, so that each is a plain shared-memory or global-memory load.
                    uint4 xa[8], xb[8];
                    const __nv_bfloat16* gsrc_a = p.q + ((size_t)req * p.num_heads + head0 + (v_a ? r_a : 0)) * L::QD + ch * 256 + c4 * 8;
                    const __nv_bfloat16* gsrc_b = p.q + ((size_t)req * p.num_heads + head0 + (v_b ? r_b : 0)) * L::QD + ch * 256 + c4 * 8;
                    if (from_smem) {
                        const uint32_t sa = smem_u32(src_a), sb = smem_u32(src_b);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            xa[i] = xb[i] = make_uint4(0, 0, 0, 0);
                            if (v_a && i < nblk32)
                                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(xa[i].x), "=r"(xa[i].y), "=r"(xa[i].z), "=r"(xa[i].w) : "r"(sa + 64 * i));
                            if (v_b && i < nblk32)
                                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(xb[i].x), "=r"(xb[i].y), "=r"(xb[i].z), "=r"(xb[i].w) : "r"(sb + 64 * i));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            xa[i] = xb[i] = make_uint4(0, 0, 0, 0);
                            if (v_a && i < nblk32) xa[i] = __ldg(reinterpret_cast<const uint4*>(gsrc_a + 32 * i));
                            if (v_b && i < nblk32) xb[i] = __ldg(reinterpret_cast<const uint4*>(gsrc_b + 32 * i));
                        }
                    }
                    auto amax2 = [](uint32_t m, const uint4& a) {      // running |.| maximum of bf16 pairs
                        auto mx = [](uint32_t u, uint32_t v) {
                            const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&u),
                                                             __habs2(*reinterpret_cast<const __nv_bfloat162*>(&v)));
                            return *reinterpret_cast<const uint32_t*>(&r);
                        };
                        return mx(mx(mx(mx(m, a.x), a.y), a.z), a.w);
                    };
                    uint32_t ma = 0u, mb = 0u;
#pragma unroll
                    for (int i = 0; i < 8; ++i) { ma = amax2(ma, xa[i]); mb = amax2(mb, xb[i]); }
                    float am_a = fmaxf(bf16lo(ma), bf16hi(ma)), am_b = fmaxf(bf16lo(mb), bf16hi(mb));
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
#pragma unroll
                        for (int h4 = 0; h4 < 2; ++h4) {
                            uint32_t wq[16];
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk) {
                                const uint4 a = xa[4 * h4 + kk], b4 = xb[4 * h4 + kk];
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
                            c = *reinterpret_cast<const uint4*>(qrows + (size_t)(head0 + hr) * L::QD + L::NOPE + (lane & 7) * 8);
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
                __syncwarp();
                if (STAGE_Q && first_work && req == meta.begin_req && lane == 0) {   // this warp has read the staged rows for the last time (if any): tell both CTAs
                    mbar_arrive(bar(BAR_QFREE));
                    mbar_arrive_remote(mapa_shared(bar(BAR_QFREE), 1u - rank));
                }
            }
            if (named_bar_or(1 + grp, 128, dead || *abort_flag != 0)) { stop = true; break; }
            TRACE(2, it);
            PROF(11);
            // The next request's Q rows are read from global memory by the next Q phase, several dependent rounds of
            // loads with nothing else to do: ask L2 for them now (this CTA's heads, 128-byte lines), a whole request
            // of tiles ahead.
            if (req + 1 <= last_req) {
                const uint8_t* qn = reinterpret_cast<const uint8_t*>(p.q + ((size_t)(req + 1) * p.num_heads + head0) * L::QD);
                const int lines = (live_heads * L::QD * 2 + 127) >> 7;
                for (int i = tid; i < lines; i += N_SM_WARPS * 32)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(qn + (size_t)i * 128));
            }
            my_sqc = live ? sqv[hrow] * p.sm_scale * LOG2E : 0.f;
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(barp(BAR_QREADYP));

            }
            // ---- epilogue of the request before ------------------------------------------------
            if (prev_valid) {
                const uint32_t last = prev_last;
                if (!dead) dead = !mbar_wait_hot(bar(BAR_PVDONE + (last & 1u)), (last >> 1) & 1u, abort_flag, W_PVDONE);
                tc_fence_after();
                if (named_bar_or(1 + grp, 128, dead || *abort_flag != 0)) { stop = true; break; }   // the partners have read the last tile's row maxima
                xch[xpart * 64 + hrow] = prev_l;
                xch[256 + xpart * 64 + hrow] = prev_x;
                named_bar_sync(1 + grp, 128);
                const float l_all = (xch[hrow] + xch[64 + hrow]) + (xch[128 + hrow] + xch[192 + hrow]);
                const float xm = fmaxf(fmaxf(xch[256 + hrow], xch[320 + hrow]), fmaxf(xch[384 + hrow], xch[448 + hrow]));
                float lse = (l_all > 0.f) ? (log2f(l_all) - (float)P_SHIFT + prev_m) : NEG_BIG;
                float denom = l_all;
                if (prev_no_split && p.attn_sink != nullptr && live) {
                    const float sink2 = p.attn_sink[head] * LOG2E;
                    denom = l_all + ((prev_m == -INFINITY) ? INFINITY : exp2f(sink2 - prev_m + (float)P_SHIFT));
                    if (lse != NEG_BIG) lse += log2f(1.f + exp2f(sink2 - lse));
                    else lse = sink2;
                }
                const float inv = (denom > 0.f) ? 1.f / denom : 0.f;
                const int col0 = thalf * 256 + ch * 128;      // first output dim of this thread
                if (prev_no_split) {
                    __nv_bfloat16* dst = p.out + ((size_t)prev_req * p.num_heads + (live ? head : 0)) * D_V + col0;
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
                        p.out_lse[(size_t)prev_req * p.num_heads + head] = lse;
                        if (p.out_max_logits) p.out_max_logits[(size_t)prev_req * p.num_heads + head] = (xm == -INFINITY) ? NEG_BIG : xm;
                    }
                } else if (p.uniform_k > 1) {
                    // partial records in fp16 (the scratch is this library's own in this mode): half the bytes to write
                    // here and to read in the combine; a normalised partial is bounded by the largest |V|, and its
                    // fp16 rounding (2^-11) is an eighth of the bf16 rounding of the final output
                    __half* dst = reinterpret_cast<__half*>(p.o_accum) + ((size_t)prev_split * p.num_heads + (live ? head : 0)) * D_V + col0;
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + TM_O + 128 * ch + c, o);
                        tmem_wait_ld();
                        if (live) {
                            uint32_t pk[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const __half2 t = __floats2half2_rn(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
                                pk[i] = *reinterpret_cast<const uint32_t*>(&t);
                            }
                            if (wide_acc) {
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
                    if (live && xpart == 0) p.lse_accum[(size_t)prev_split * p.num_heads + head] = lse;
                } else {
                    float* dst = p.o_accum + ((size_t)prev_split * p.num_heads + (live ? head : 0)) * D_V + col0;
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
                    if (live && xpart == 0) p.lse_accum[(size_t)prev_split * p.num_heads + head] = lse;
                }
                tc_fence_before();                  // the accumulator reads precede the next request's first P.V
                named_bar_sync(1 + grp, 128);       // xch is free again
                PROF(12);
                TRACE(4, it);
            }
            prev_valid = false;
            if (!have) break;
            float m_run = -INFINITY;   // running maximum of z (lags by at most RESCALE_TAU)
            float l_run = 0.f;         // this thread's share of the sum of P'/s (scaled by 2^P_SHIFT)
            float x_max = -INFINITY;   // this thread's share of the maximum of the scaled logits (max_logits output)
            for (int j = 0; j < nst; ++j, ++it) {
                const uint32_t b = it & 1u;
                float z[32];
                float mx_loc = -INFINITY;
                float inv_g[4] = {0.f, 0.f, 0.f, 0.f};     // 1/s of the four groups of eight tokens that this thread holds
                // the records of this thread's 32 tokens: half tile thalf, gather warps [4 ch, 4 ch + 4)
                const uint8_t* info = sm + INFO_OFF + (it & (INFO_RING - 1)) * (2 * INFO_HALF) + thalf * INFO_HALF + ch * 64;
                PROF(0);
                if (!dead) dead = !mbar_wait_hot(bar(BAR_SREADY + b), (it >> 1) & 1u, abort_flag, W_SREADY);
                PROF(1);
                TRACE(10, it);
                if (!dead) dead = !mbar_wait_hot(bar(BAR_INFO + (it & (INFO_RING - 1))), (it / INFO_RING) & 1u, abort_flag, W_INFO);
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
                    uint32_t valid = 0u;
                    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float4 ti = *reinterpret_cast<const float4*>(info + 16 * g);    // (s, log2 s, 1/s, validity bits) of the group
                        const float c_g = ti.x * my_sqc, off = ti.y;
                        inv_g[g] = ti.z;
                        valid |= (__float_as_uint(ti.w) & 0xffu) << (8 * g);
                        float gm = -INFINITY;
#pragma unroll
                        for (int t = 8 * g; t < 8 * g + 8; ++t) {
                            z[t] = fmaf(__uint_as_float(sv[t]), c_g, off);
                            if (!((__float_as_uint(ti.w) >> (t - 8 * g)) & 1u)) z[t] = -INFINITY;   // no entry: weight exactly 0
                            gm = fmaxf(gm, z[t]);
                        }
                        // z - log2(s) is the scaled logit itself
                        if (p.out_max_logits != nullptr && gm > -INFINITY) x_max = fmaxf(x_max, gm - off);
                        if (g & 1) mx1 = fmaxf(mx1, gm); else mx0 = fmaxf(mx0, gm);
                    }
                    (void)valid;
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
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float l0 = 0.f, l1 = 0.f;
#pragma unroll
                    for (int t = 8 * g; t < 8 * g + 8; t += 4) {
                        const float p0 = ex2(z[t + 0] - m_off), p1 = ex2(z[t + 1] - m_off);
                        const float p2 = ex2(z[t + 2] - m_off), p3 = ex2(z[t + 3] - m_off);
                        l0 += p0 + p2; l1 += p1 + p3;
                        pw[t >> 2] = pack_e4m3x4(p0, p1, p2, p3);
                    }
                    l_run = fmaf(l0 + l1, inv_g[g], l_run);
                }
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
            prev_valid = true; prev_no_split = w.no_split; prev_req = req; prev_split = w.split_idx;
            prev_last = it - 1; prev_m = m_run; prev_l = l_run; prev_x = x_max;
        }
    } else if (warp < MMA_WARP) {
        // =================================================================== gather
        // Warp gw reads rows [8 gw, +8) of this CTA's 64 rows of every tile from the raw stage into registers: per
        // row one 16-byte piece of the 512 no-PE bytes per lane, plus (spread over the lanes) the rows' RoPE bytes
        // and scale words.  The largest of the rows' scales is the scale of the warp's group; every lane shifts its
        // pieces onto it and stores them in the layout the MMAs read.
        // MODEL1: 28 lanes hold the 448 no-PE bytes of a row; the rows' scale bytes do not travel with the rows (they
        // lie in the page footer), so the warp reads them from global memory itself, a tile ahead of their use.
        const int gw = warp - N_SM_WARPS;
        const int blk = lane >> 3;                                   // 128-value chunk of this lane's piece
        const CacheGeom main_c = cache_geom(p.kv, p.block_stride, p.page_block_size);
        const CacheGeom extra_c = cache_geom(p.extra_kv, p.extra_block_stride, p.extra_topk > 0 ? p.extra_page_block_size : 1);
        uint32_t it = 0;
        bool ok = true, stop = false;
        for (int req = meta.begin_req; req <= last_req && !stop; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int nst = (w.nblk + 1) >> 1;
            // tile j of this CTA is block blk0 + 2 j + rank of the request; this lane looks after row RPW gw + lane % RPW
            const int lim = min(w.len, (w.blk0 + w.nblk) * BLOCK_N);
            auto fetch_idx = [&](int j) -> int { return tile_entry<EXTRA>(p, w, j, (int)rank, gw * RPW + (lane & (RPW - 1)), nst, lim); };
            auto fetch_scales = [&](int j, int idx) -> uint2 {       // MODEL1: the row's 7 UE8M0 bytes (+ 1 pad)
                if (!L::M1 || idx < 0) return make_uint2(0u, 0u);
                const CacheGeom& c = (!EXTRA || w.blk0 + 2 * j + (int)rank < w.main_blocks) ? main_c : extra_c;
                unsigned in;
                const uint8_t* pg = cache_page(c, idx, in);
                return __ldg(reinterpret_cast<const uint2*>(pg + (int64_t)c.pbs * L::DATA + (int64_t)in * 8));
            };
            // Which of the warp's rows have an entry (the rows themselves are brought in by the copy warps).
            int idx_cur = fetch_idx(0), idx_nxt = fetch_idx(1);
            uint2 sc8_nxt = fetch_scales(0, idx_cur);
#pragma unroll 1
            for (int k = 0; k < nst; ++k) {
                const uint32_t t_it = it + k, ks = t_it % NK, rs = t_it % NR;
                PROF(0);
                TRACE(60, t_it);
                if (ok) ok = mbar_wait_hot(bar(BAR_RAWFULL + rs * N_P_WARPS + gw * RPW / 16), (t_it / NR) & 1u, abort_flag, W_RAWFULL);
                PROF(1);
                TRACE(61, t_it);
                const uint32_t vbits = __ballot_sync(0xffffffffu, idx_cur >= 0) & ((1u << RPW) - 1u);
                const uint2 sc8 = sc8_nxt;
                sc8_nxt = fetch_scales(k + 1, idx_nxt);
                idx_cur = idx_nxt;
                idx_nxt = fetch_idx(k + 2);
                const uint8_t* raw_rows = sm + RAW_OFF + rs * RAW_BYTES + (gw * RPW) * ROW_BYTES;
                uint4 nope[RPW], rp[RPW / 4];
                float sc = 0.f;
                if (ok) {
#pragma unroll
                    for (int i = 0; i < RPW; ++i)
                        nope[i] = ((vbits >> i) & 1u) ? *reinterpret_cast<const uint4*>(raw_rows + i * ROW_BYTES + lane * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int u = 0; u < RPW / 4; ++u) {                      // RoPE piece lane % 8 of row lane / 8 (+ 4 u)
                        const int r = (lane >> 3) + 4 * u;
                        rp[u] = ((vbits >> r) & 1u) ? *reinterpret_cast<const uint4*>(raw_rows + r * ROW_BYTES + L::ROPE_AT + (lane & 7) * 16)
                                                    : make_uint4(0, 0, 0, 0);
                    }
                    if (!L::M1 && lane < 4 * RPW && ((vbits >> (lane >> 2)) & 1u))     // scale lane % 4 of row lane / 4
                        sc = *reinterpret_cast<const float*>(raw_rows + (lane >> 2) * ROW_BYTES + SCALE_OFF + (lane & 3) * 4);
                } else {
#pragma unroll
                    for (int i = 0; i < RPW; ++i) nope[i] = make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int u = 0; u < RPW / 4; ++u) rp[u] = make_uint4(0, 0, 0, 0);
                }
                float wm = sc;
                if (L::M1) {
                    // The group's scale as a biased exponent: the largest of the rows' 7 scale bytes (0 for a row without
                    // an entry) and of what the rows' RoPE needs to fit e4m3 (2^ceil(log2(amax / 448))).
                    uint32_t e = __vmaxu4(sc8.x, sc8.y & 0x00ffffffu);
                    e = max(max(e & 0xffu, (e >> 8) & 0xffu), max((e >> 16) & 0xffu, e >> 24));
                    auto absmax8 = [](const uint4& a) {
                        return fmaxf(fmaxf(fmaxf(fabsf(bf16lo(a.x)), fabsf(bf16hi(a.x))), fmaxf(fabsf(bf16lo(a.y)), fabsf(bf16hi(a.y)))),
                                     fmaxf(fmaxf(fabsf(bf16lo(a.z)), fabsf(bf16hi(a.z))), fmaxf(fabsf(bf16lo(a.w)), fabsf(bf16hi(a.w)))));
                    };
                    float am = 0.f;
#pragma unroll
                    for (int u = 0; u < RPW / 4; ++u) am = fmaxf(am, absmax8(rp[u]));
                    const uint32_t ab = __float_as_uint(am * (1.f / 448.f));
                    e = max(e, (ab >> 23) + ((ab & 0x007fffffu) ? 1u : 0u));
                    if (vbits != 0u) e = max(e, 1u);
                    wm = __uint_as_float(min(e, 254u) << 23);
                }
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
                // the maximum needed the last shared-memory load of every lane (they return in order): the warp's rows
                // have left the raw stage
                if (lane == 0) mbar_arrive(bar(BAR_RAWEMPTY + rs * N_P_WARPS + gw * RPW / 16));
                PROF(2);
                TRACE(62, t_it);
                if (ok && t_it >= NK) ok = mbar_wait_hot(bar(BAR_KEMPTY + ks), ((t_it / NK) - 1) & 1u, abort_flag, W_KEMPTY);
                if (STAGE_Q && ok && t_it < NK && ks != 0 && first_work) ok = mbar_wait_hot(bar(BAR_QFREE), 0u, abort_flag, W_QFREE);   // K stage 1 held Q until now
                PROF(3);
                TRACE(63, t_it);
                if (!ok) { stop = true; break; }
                PROF(4);
                TRACE(64, t_it);
                // one scale for the warp's RPW rows: the largest of their 4 x RPW scales
                const float s_half = wm;
                const float inv_half = (s_half > 0.f) ? __uint_as_float(0x7f000000u - __float_as_uint(s_half)) : 0.f;
                const __nv_bfloat162 rope_f = __float2bfloat162_rn(inv_half);
                uint8_t* kp = sm + KS_OFF + ks * KS_BYTES;
                // V32: exponent shift of the block whose scale this lane loaded (row lane / 4, block lane % 4): 0 for a block at the scale.
                // MODEL1: lanes 0-7 pass on exponents 0-3 of row lane, lanes 8-15 exponents 4-6 of row lane - 8.
                const uint32_t my_sub = L::M1 ? ((lane & 8) ? sc8.y : sc8.x) : ((sc > 0.f) ? shift_bytes_of_ratio(sc * inv_half) : 0u);
                const uint32_t e_grp = __float_as_uint(s_half) >> 23;
                const int bk = lane >> 2;                            // MODEL1: 64-value block of this lane's piece (0-6 in the lanes that store)
#pragma unroll
                for (int i = 0; i < RPW; ++i) {
                    uint32_t sub;
                    if (L::M1) {
                        const uint32_t ew = __shfl_sync(0xffffffffu, my_sub, i + ((bk & 4) ? 8 : 0));
                        sub = min(e_grp - ((ew >> (8 * (bk & 3))) & 0xffu), 15u) * 0x08080808u;
                    } else {
                        sub = __shfl_sync(0xffffffffu, my_sub, 4 * i + blk);
                    }
                    uint4 v = nope[i];      // no branch on sub: a shift by 0 is the identity, and a branch would keep the rows' chains apart
                    v.x = shift_down_e4m3x4(v.x, sub); v.y = shift_down_e4m3x4(v.y, sub);
                    v.z = shift_down_e4m3x4(v.z, sub); v.w = shift_down_e4m3x4(v.w, sub);
                    if (!L::M1 || lane < L::NOPE / 16)
                        *reinterpret_cast<uint4*>(kp + blk * CHUNK + swz((uint32_t)(gw * RPW + i), (uint32_t)lane & 7u)) = v;
                }
                if (L::M1) {      // V's RoPE columns: e4m3(rope / s) into dims [448, 512) of the rows, the upper half of chunk 3
#pragma unroll
                    for (int u = 0; u < RPW / 4; ++u) {
                        const uint4 v = rp[u];
                        const uint32_t lo = pack_e4m3x4(bf16lo(v.x) * inv_half, bf16hi(v.x) * inv_half, bf16lo(v.y) * inv_half, bf16hi(v.y) * inv_half);
                        const uint32_t hi = pack_e4m3x4(bf16lo(v.z) * inv_half, bf16hi(v.z) * inv_half, bf16lo(v.w) * inv_half, bf16hi(v.w) * inv_half);
                        const uint32_t pc = (uint32_t)lane & 7u;      // piece of 8 values
                        *reinterpret_cast<uint2*>(kp + 3 * CHUNK + swz((uint32_t)(gw * RPW + (lane >> 3) + 4 * u), 4u + (pc >> 1)) + (pc & 1u) * 8u) =
                            make_uint2(lo, hi);
                    }
                }
#pragma unroll
                for (int u = 0; u < RPW / 4; ++u) {
                    uint4 v = rp[u];
                    v.x = mul_bf16x2(v.x, rope_f); v.y = mul_bf16x2(v.y, rope_f);
                    v.z = mul_bf16x2(v.z, rope_f); v.w = mul_bf16x2(v.w, rope_f);
                    *reinterpret_cast<uint4*>(kp + KS_ROPE + swz((uint32_t)(gw * RPW + (lane >> 3) + 4 * u), (uint32_t)lane & 7u)) = v;
                }
                if (lane == 0) {      // the record of the warp's rows: read by this CTA's softmax warps and sent to the partner's
                    uint8_t* rec = sm + INFO_OFF + (t_it & (INFO_RING - 1)) * (2 * INFO_HALF) + rank * INFO_HALF + gw * 16;
                    *reinterpret_cast<float4*>(rec) =
                        make_float4(s_half, (s_half > 0.f) ? (float)((int)(__float_as_uint(s_half) >> 23) - 127) : -INFINITY, inv_half,
                                    __uint_as_float(vbits));
                }
                PROF(5);
                TRACE(65, t_it);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar(BAR_KSTORED + ks));
                    mbar_arrive_remote(barp(BAR_KFULLP + ks));
                }
                PROF(6);
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
                        if (32 * (4 * kc + s) < L::NOPE)      // MODEL1: the last 64 bytes of chunk 3 are V's RoPE columns
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
                                    make_desc(vb_lo + (((4 * nb + kb) * VSLOT) >> 4), DESC_HI_SW128), IDESC_PV_F8, (j | kb) != 0);
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
    } else if (warp == FWD_WARP && lane == 0) {
        // =================================================================== K stage -> V slots (both CTAs)
        // The no-PE bytes of this CTA's 64 rows lie in the K stage as four chunks of [64 rows x 128 dims], which is
        // two V slots each (rows 0-31 and 32-63) in the slots' own layout.  Chunks 2 r and 2 r + 1 go to CTA r: the
        // chunks of the own dims stay in this CTA, the others cross to the partner.  The destination's barrier
        // counts the bytes.  The half tile's scale records travel the same way.  When this CTA's slots are full
        // (its own copies and the partner's have landed) the thread passes that on: V full to the even CTA,
        // K stage free to both.
        const uint32_t peer = 1u - rank;
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int nst = (w.nblk + 1) >> 1;
            for (int j = 0; j < nst && ok; ++j, ++it) {
                const uint32_t ks = it % NK, vs = it % NV, ir = it & (INFO_RING - 1);
                TRACE(70, it);
                ok = mbar_wait_thread(bar(BAR_KSTORED + ks), (it / NK) & 1u, abort_flag, W_KSTORED);
                if (!ok) break;
                TRACE(71, it);
                mbar_arrive_expect_tx(bar(BAR_INFO + ir), INFO_HALF);
                bulk_copy_to_cluster(mapa_shared(base + INFO_OFF + ir * (2 * INFO_HALF) + rank * INFO_HALF, peer),
                                     base + INFO_OFF + ir * (2 * INFO_HALF) + rank * INFO_HALF, INFO_HALF, mapa_shared(bar(BAR_INFO + ir), peer));
                if (it >= NV) {
                    ok = mbar_wait_thread(bar(BAR_VEMPTY + vs), ((it / NV) - 1) & 1u, abort_flag, W_VEMPTY);
                    if (!ok) break;
                } else if (STAGE_Q && first_work) {    // the V stages of both CTAs held Q until the softmax warps had read it
                    ok = mbar_wait_thread(bar(BAR_QFREE), 0u, abort_flag, W_QFREE);
                    if (!ok) break;
                }
                TRACE(72, it);
                mbar_arrive_expect_tx(bar(BAR_VFULL + vs), 4 * CHUNK);
#pragma unroll
                for (uint32_t r = 0; r < 2; ++r) {
#pragma unroll
                    for (uint32_t nb = 0; nb < 2; ++nb) {
                        bulk_copy_to_cluster(mapa_shared(base + VS_OFF + vs * VS_BYTES + (4 * nb + 2 * rank) * VSLOT, r),
                                             base + KS_OFF + ks * KS_BYTES + (2 * r + nb) * CHUNK, CHUNK,
                                             mapa_shared(bar(BAR_VFULL + vs), r));
                    }
                }
                TRACE(73, it);
                ok = mbar_wait_thread(bar(BAR_VFULL + vs), (it / NV) & 1u, abort_flag, W_VFULL_CTA);
                if (!ok) break;
                TRACE(74, it);
                mbar_arrive_remote(barp(BAR_VFULLP + vs));
                // the copies out of this CTA's K stage into its own slots and the partner's copies into them are done
                mbar_arrive(bar(BAR_KEMPTY + ks));
                mbar_arrive_remote(mapa_shared(bar(BAR_KEMPTY + ks), peer));
            }
        }
    }
    else if (warp >= PROD_WARP0) {
        // =================================================================== global -> raw stage (both CTAs)
        // Copy warp pw brings rows [16 pw, +16) of every tile of this CTA into the raw stage, one bulk copy per row
        // (lanes 0-15; no load/store unit and no registers involved, two tiles of the CTA are in flight).  Nothing
        // is copied for a row without an entry.  The tile NR ahead is issued as soon as the gather warps that read
        // these rows have taken the tile out of the stage; the warp's barrier of the stage counts the bytes.
        // Issuing a copy blocks while the copy unit is busy, which is why no working warp does it.
        const int pw = warp - PROD_WARP0;
        const CacheGeom main_c = cache_geom(p.kv, p.block_stride, p.page_block_size);
        const CacheGeom extra_c = cache_geom(p.extra_kv, p.extra_block_stride, p.extra_topk > 0 ? p.extra_page_block_size : 1);
        uint32_t it = 0;
        bool ok = true;
        for (int req = meta.begin_req; req <= last_req && ok; ++req) {
            Work w;
            if (!get_work(p, meta, req, w)) continue;
            const int nst = (w.nblk + 1) >> 1;
            // tile j of this CTA is block blk0 + 2 j + rank of the request; row 16 pw + lane % 16
            const int lim = min(w.len, (w.blk0 + w.nblk) * BLOCK_N);
            auto fetch_idx = [&](int j) -> int { return tile_entry<EXTRA>(p, w, j, (int)rank, pw * 16 + (lane & 15), nst, lim); };
            auto issue_rows = [&](int idx, int j, uint32_t t_it) {   // idx: lanes 0-15 hold the indices of the rows of tile j
                const uint32_t stage = t_it % NR;
                unsigned long long src = 0ull;
                if (idx >= 0) {
                    const CacheGeom& c = (!EXTRA || w.blk0 + 2 * j + (int)rank < w.main_blocks) ? main_c : extra_c;
                    unsigned in;
                    const uint8_t* pg = cache_page(c, idx, in);
                    src = reinterpret_cast<unsigned long long>(pg + (int64_t)in * L::DATA);
                }
                const uint32_t dst0 = base + RAW_OFF + stage * RAW_BYTES + (pw * 16) * ROW_BYTES;
                const uint32_t fb = bar(BAR_RAWFULL + stage * N_P_WARPS + pw);
                const uint32_t nvalid = __popc(__ballot_sync(0xffffffffu, src != 0ull) & 0xffffu);
                if (lane == 0) mbar_arrive_expect_tx(fb, nvalid * L::DATA);
                __syncwarp();
                if (lane < 16 && src != 0ull) bulk_copy_g2s(dst0 + lane * ROW_BYTES, src, L::DATA, fb);
            };
            // The raw stages that the first NR tiles of a request go to are free once the gather warps have taken the
            // last NR tiles before them out (for the very first tiles of the CTA there is nothing to wait for).
#pragma unroll 1
            for (int j = 0; j < NR && j < nst && ok; ++j) {
                const uint32_t t_it = it + j;
                const int idx = fetch_idx(j);
                if (t_it >= NR) ok = mbar_wait_hot(bar(BAR_RAWEMPTY + (t_it % NR) * N_P_WARPS + pw), ((t_it / NR) - 1) & 1u, abort_flag, W_RAWEMPTY);
                if (ok) issue_rows(idx, j, t_it);
            }
            int idx_ahead = fetch_idx(NR);               // read one tile before it is turned into addresses
#pragma unroll 1
            for (int j = 0; j + NR < nst && ok; ++j) {   // the tile NR ahead goes into the raw stage that has just been emptied
                const uint32_t t_it = it + j;
                ok = mbar_wait_hot(bar(BAR_RAWEMPTY + (t_it % NR) * N_P_WARPS + pw), (t_it / NR) & 1u, abort_flag, W_RAWEMPTY);
                if (!ok) break;
                issue_rows(idx_ahead, j + NR, t_it + NR);
                idx_ahead = fetch_idx(j + NR + 1);
            }
            it += nst;
        }
    }

    // ------------------------------------------------------------------------ teardown
    if (*abort_flag != 0) {        // a wait gave up: bulk copies into or out of this CTA may still be in flight; give them time to land
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) { }
    }
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

namespace {

template <int LAYOUT, bool EXTRA, bool STAGE_Q>
int launch_pair_instance(const AttnParams& p, cudaStream_t stream) {
    static bool attr_set[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return set_error(SMLA_E_SHAPE, "attn_pair_kernel: device ordinal %d not supported", dev);
    if (!attr_set[dev]) {
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, attn_pair_kernel<LAYOUT, EXTRA, STAGE_Q>) != cudaSuccess || fa.numRegs != REGS_LAUNCH)
            return set_error(SMLA_E_DEVICE, "attn_pair_kernel: compiled with %d registers per thread, the warpgroup budgets assume %d",
                             fa.numRegs, REGS_LAUNCH);
        const cudaError_t e = cudaFuncSetAttribute(attn_pair_kernel<LAYOUT, EXTRA, STAGE_Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_ALLOC);
        if (e != cudaSuccess) return set_error((int)e, "attn_pair_kernel: cannot reserve %u bytes of shared memory: %s",
                                               SMEM_ALLOC, cudaGetErrorString(e));
        cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        attr_set[dev] = true;
    }
    // Without a scheduler the grid is persistent: at most one CTA per SM, each pair walks its share of the requests.
    const int max_pairs = sm_count[dev] >= 2 ? sm_count[dev] / 2 : 1;
    const int parts = p.sched ? p.num_parts : p.uniform_k > 1 ? p.uniform_k * p.num_tokens
                                                              : (p.num_tokens < max_pairs ? p.num_tokens : max_pairs);
    if (p.sched != nullptr)      // the scheduler kernel runs just before: start while it finishes
        launch_dependent(attn_pair_kernel<LAYOUT, EXTRA, STAGE_Q>, dim3(2 * parts), dim3(PAIR_THREADS), SMEM_ALLOC, stream, p);
    else
        attn_pair_kernel<LAYOUT, EXTRA, STAGE_Q><<<2 * parts, PAIR_THREADS, SMEM_ALLOC, stream>>>(p);
    return check_launch("attn_pair_kernel");
}

}  // namespace

// The bulk copies that bring rows in want 16-byte aligned sources: both caches' base addresses and page strides
// (a row's offset inside its page is a multiple of 16 in both layouts).
bool attn_pair_takes(const AttnParams& p) {
    auto al = [](const void* q, int64_t stride) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0 && (stride & 15) == 0; };
    return p.num_heads >= 1 && p.num_heads <= 128 && al(p.kv, p.block_stride) &&
           (p.extra_topk == 0 || al(p.extra_kv, p.extra_block_stride));
}

int launch_attn_pair(const AttnParams& p, cudaStream_t stream) {
    if (p.num_tokens == 0) return 0;
    // Staging of the first request's Q only where the kernel follows the scheduler (see STAGE_Q).
    const bool stage = p.sched != nullptr || p.uniform_k > 1;      // short partitions
    if (p.layout == SMLA_LAYOUT_MODEL1) {
        if (p.extra_topk > 0) return stage ? launch_pair_instance<SMLA_LAYOUT_MODEL1, true, true>(p, stream)
                                           : launch_pair_instance<SMLA_LAYOUT_MODEL1, true, false>(p, stream);
        return stage ? launch_pair_instance<SMLA_LAYOUT_MODEL1, false, true>(p, stream)
                     : launch_pair_instance<SMLA_LAYOUT_MODEL1, false, false>(p, stream);
    }
    if (p.extra_topk > 0) return stage ? launch_pair_instance<SMLA_LAYOUT_V32, true, true>(p, stream)
                                       : launch_pair_instance<SMLA_LAYOUT_V32, true, false>(p, stream);
    return stage ? launch_pair_instance<SMLA_LAYOUT_V32, false, true>(p, stream)
                 : launch_pair_instance<SMLA_LAYOUT_V32, false, false>(p, stream);
}

}  // namespace smla
