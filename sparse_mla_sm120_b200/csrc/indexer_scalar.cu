// MQA-logits indexer, CUDA-core version, top-k selection and context-parallel index partition.
//
// None of the three has a counterpart in the reference project (its indices come from an
// external indexer and it has no multi-GPU path); they implement
//   logits[i, j] = k_scale[j] * sum_h w[i, h] * relu(q[i, h, :] . k[j, :]),  -inf outside [ks_i, ke_i)
// followed by a per-row top-k, and the split of a global index list into one GPU's shard.
#include <cstdint>

#include "common.cuh"

namespace smla {

namespace {

// ---------------------------------------------------------------- logits, fp32 CUDA cores
// One CTA = (128 keys, one query).  Two threads per key, each holding half of the key's 128
// values in registers; q of the query sits in shared memory as fp32.
constexpr int LK = 128;   // keys per CTA
constexpr int LD = 128;   // head dim of the indexer

__global__ void __launch_bounds__(256)
mqa_logits_scalar_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ k,
                         const float* __restrict__ k_scale, const float* __restrict__ weights,
                         const int32_t* __restrict__ ks, const int32_t* __restrict__ ke,
                         float* __restrict__ logits, int num_heads, int s_k, int64_t logits_stride) {
    extern __shared__ float qs[];  // [num_heads][LD]
    const int i = blockIdx.y;
    const int j = blockIdx.x * LK + (threadIdx.x >> 1);
    const int half = threadIdx.x & 1;
    for (int e = threadIdx.x; e < num_heads * LD; e += blockDim.x)
        qs[e] = e4m3_to_float(q[(size_t)i * num_heads * LD + e]);
    float kr[LD / 2];
    if (j < s_k) {
#pragma unroll
        for (int d = 0; d < LD / 2; ++d) kr[d] = e4m3_to_float(k[(size_t)j * LD + half * (LD / 2) + d]);
    } else {
#pragma unroll
        for (int d = 0; d < LD / 2; ++d) kr[d] = 0.f;
    }
    __syncthreads();
    float acc = 0.f;
    for (int h = 0; h < num_heads; ++h) {
        const float* qh = qs + h * LD + half * (LD / 2);
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < LD / 2; ++d) s += qh[d] * kr[d];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        acc += weights[(size_t)i * num_heads + h] * fmaxf(s, 0.f);
    }
    if (half == 0 && j < s_k) {
        const bool in = (j >= ks[i]) && (j < ke[i]);
        logits[(size_t)i * logits_stride + j] = in ? acc * k_scale[j] : -INFINITY;
    }
}

// ---------------------------------------------------------------- top-k: radix select per row
constexpr int TK_THREADS = 1024;
constexpr int TK_WARPS = TK_THREADS / 32;
constexpr int32_t TK_REDO = INT32_MIN;     // first output of a row that has more: the multi-pass kernel redoes the row

__device__ __forceinline__ uint32_t order_key(float f) {   // larger float <=> larger key
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Applies fn(column, key) to every column of [lo, hi): 16-byte loads over the aligned middle part,
// four of them in flight per thread, scalar loads at the ragged ends.
template <typename F>
__device__ __forceinline__ void for_each_key(const float* __restrict__ x, int lo, int hi, int tid, int nthreads, F fn) {
    const int a0 = min(hi, (int)(((size_t)lo + 3) & ~(size_t)3));                 // first multiple of 4 >= lo (x is 16-byte aligned)
    const int a1 = max(a0, hi & ~3);
    for (int j = lo + tid; j < a0; j += nthreads) fn(j, order_key(x[j]));
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int v0 = a0 >> 2, v1 = a1 >> 2;
    int v = v0 + tid;
    for (; v + 3 * nthreads < v1; v += 4 * nthreads) {
        const float4 f0 = x4[v], f1 = x4[v + nthreads], f2 = x4[v + 2 * nthreads], f3 = x4[v + 3 * nthreads];
        const float4 ff[4] = {f0, f1, f2, f3};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = (v + u * nthreads) << 2;
            fn(j, order_key(ff[u].x)); fn(j + 1, order_key(ff[u].y)); fn(j + 2, order_key(ff[u].z)); fn(j + 3, order_key(ff[u].w));
        }
    }
    for (; v < v1; v += nthreads) {
        const float4 f = x4[v];
        const int j = v << 2;
        fn(j, order_key(f.x)); fn(j + 1, order_key(f.y)); fn(j + 2, order_key(f.z)); fn(j + 3, order_key(f.w));
    }
    for (int j = a1 + tid; j < hi; j += nthreads) fn(j, order_key(x[j]));
}

// One CTA of 1024 threads per row, so at most two rows per SM are in flight: a row of 65536
// logits is 256 KB, the rows in flight (76 MB on 148 SMs) fit the L2 and only the first of the
// passes over a row reaches DRAM.
__global__ void __launch_bounds__(TK_THREADS, 1)
topk_kernel(const float* __restrict__ logits, const int32_t* __restrict__ ks,
            const int32_t* __restrict__ ke, int32_t* __restrict__ out, int num_cols,
            int64_t logits_stride, int k, int only_flagged) {
    // only_flagged: redo the rows that topk_select_kernel gave up on
    if (only_flagged && out[(size_t)blockIdx.x * k] != TK_REDO) return;
    __shared__ int hist[256];
    __shared__ int sel_bin, sel_need;
    __shared__ int seg_gt[TK_WARPS], seg_eq[TK_WARPS];

    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * logits_stride;
    int lo = ks ? max(ks[row], 0) : 0;
    int hi = ke ? min(ke[row], num_cols) : num_cols;
    if (hi < lo) hi = lo;
    int32_t* o = out + (size_t)row * k;
    const uint32_t NEG_INF_KEY = order_key(-INFINITY);
    const bool vec_ok = ((reinterpret_cast<size_t>(x) & 15) == 0);
    // (rows that are not 16-byte aligned are read with scalar loads only)

    // Pass 0..3: find the key of the k-th largest candidate (candidates: keys above -inf).
    uint32_t prefix = 0, prefix_mask = 0;
    int need = k;           // how many still to take among keys matching the prefix
    bool take_all = false;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int b = tid; b < 256; b += TK_THREADS) hist[b] = 0;
        __syncthreads();
        auto count = [&](int, uint32_t key) {
            if (key > NEG_INF_KEY && (key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
        };
        if (vec_ok) for_each_key(x, lo, hi, tid, TK_THREADS, count);
        else for (int j = lo + tid; j < hi; j += TK_THREADS) count(j, order_key(x[j]));
        __syncthreads();
        if (tid == 0) {
            int cum = 0, b = 255;
            for (; b >= 0; --b) {
                if (cum + hist[b] >= need) break;
                cum += hist[b];
            }
            sel_bin = b;            // -1: fewer candidates than needed
            sel_need = need - cum;
        }
        __syncthreads();
        if (sel_bin < 0) { take_all = true; break; }
        prefix |= (uint32_t)sel_bin << shift;
        prefix_mask |= 255u << shift;
        need = sel_need;
        __syncthreads();
    }
    const uint32_t thr = take_all ? NEG_INF_KEY : prefix;   // take keys > thr, plus `need` keys == thr
    const int need_eq = take_all ? 0 : need;

    // Ordered compaction: every warp owns a contiguous run of columns, counts its keys above and
    // at the threshold, and after a scan over the warps writes them in column order: positions
    // [0, n_gt) hold the greater ones, [n_gt, n_gt + need_eq) the first need_eq ties.
    const int span = hi - lo;
    const int seg = ((span + TK_WARPS - 1) / TK_WARPS + 31) & ~31;
    const int s0 = min(lo + warp * seg, hi), s1 = min(s0 + seg, hi);
    int c_gt = 0, c_eq = 0;
    for (int j = s0 + lane; j < s1; j += 32) {
        const uint32_t key = order_key(x[j]);
        c_gt += (key > thr);
        c_eq += (!take_all && key == thr);
    }
    c_gt = __reduce_add_sync(0xffffffffu, c_gt);
    c_eq = __reduce_add_sync(0xffffffffu, c_eq);
    if (lane == 0) { seg_gt[warp] = c_gt; seg_eq[warp] = c_eq; }
    __syncthreads();
    int off_gt = 0, off_eq = 0, n_gt = 0, n_eq = 0;
    for (int w = 0; w < TK_WARPS; ++w) {
        if (w < warp) { off_gt += seg_gt[w]; off_eq += seg_eq[w]; }
        n_gt += seg_gt[w]; n_eq += seg_eq[w];
    }
    const uint32_t below = (1u << lane) - 1u;
    for (int j0 = s0; j0 < s1; j0 += 32) {
        const int j = j0 + lane;
        uint32_t key = NEG_INF_KEY;
        if (j < s1) key = order_key(x[j]);
        const bool gt = key > thr;
        const bool eq = (!take_all) && key == thr && j < s1;
        const uint32_t mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
        if (gt) o[off_gt + __popc(mg & below)] = j;
        if (eq) {
            const int r = off_eq + __popc(me & below);
            if (r < need_eq) o[n_gt + r] = j;
        }
        off_gt += __popc(mg); off_eq += __popc(me);
    }
    const int filled = n_gt + (take_all ? 0 : min(need_eq, n_eq));
    for (int r = filled + tid; r < k; r += TK_THREADS) o[r] = -1;
}

// Warp 0: the highest of 256 bins at which the count cumulated from the top reaches `need`
// (bin -1 when the whole histogram holds less), and how many entries of that bin are needed.
__device__ __forceinline__ void pick_bin(const int* hist, int need, int lane, int* sel_bin, int* sel_need) {
    int h[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { h[i] = hist[8 * lane + i]; s += h[i]; }
    int suf = s;                                   // sum over lanes >= this one
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_down_sync(0xffffffffu, suf, o);
        if (lane + o < 32) suf += t;
    }
    const int above = suf - s;
    const bool here = (above < need) && (suf >= need);
    const uint32_t m = __ballot_sync(0xffffffffu, here);
    if (here) {
        int cum = above, b = 7;
        for (; b > 0; --b) {
            if (cum + h[b] >= need) break;
            cum += h[b];
        }
        *sel_bin = 8 * lane + b; *sel_need = need - cum;
    }
    if (m == 0 && lane == 0) { *sel_bin = -1; *sel_need = need - suf; }
}

// One-read selection.  A sample of the row (512 runs of 8 neighbouring logits, one 32-byte sector
// each, evenly spread) gives a threshold that, with a margin of four standard deviations of the
// estimate, lets through somewhat more than k entries (about 1.4 k for k = 2048 out of 65536).
// The single pass over the row then lists the column of every entry at or above the threshold
// in shared memory, and the exact k best are chosen among the few thousand candidates: their
// keys (read again, the row is still in the L2) go into one histogram of 4096 bins laid over the
// range the candidates span, a parallel suffix sum finds the bin of the k-th, and the handful of
// entries in that bin are ranked by (key, lower column first).  Rows whose window has at most
// TS_DIRECT columns skip the sample and list every column.  Any width of row is served (nothing
// but the candidates is kept on chip), and two CTAs fit an SM, so the read of one row overlaps
// the selection of another.  When the guess fails -- fewer than k candidates, a list overflows
// (heavy ties, logits that cluster far more than the sample saw), too many entries in the bin of
// the k-th -- the row is marked for the multi-pass kernel.
//
// The pass over the row is kept free of warp-wide votes: a lane compares its logits as floats
// (NaNs never become candidates) and only notes a bit per entry; after a stretch of eight rounds
// (65536 columns with 16 warps) the lanes of a warp exchange their counts once and every lane
// appends its own columns.
//
// Order of the output: warp w owns the 128-column blocks w, w + warps, ... of the row; its list
// holds, per stretch, the candidates of lane 0, then of lane 1, ... each in column order; the
// lists are written out one after the other.  The order is a fixed function of the
// input (no atomics decide it), though not ascending.
constexpr int TS_CAND = 8192;              // candidates a row may have in all (per warp: TS_CAND / warps)
constexpr int TS_SAMPLE = 4096;            // sampled logits: 512 runs of 8
constexpr int TS_EQ = 1024;                // entries in the bin of the k-th key, ranked one against the other
constexpr int TS_BINS = 4096;
constexpr int TS_DIRECT = TS_CAND - 128;   // windows up to this size need no threshold
constexpr int TS_KMAX = 4096;              // largest k (the lists hold 8192)
constexpr int TS_ROUNDS = 8;               // rounds of four blocks per warp between two appends
constexpr int TS_SMEM = TS_CAND * 8 + TS_BINS * 4 + TS_EQ * 8;

__device__ __forceinline__ float4 load_row4(const float* __restrict__ x, int j, int num_cols, bool vec_ok) {
    if (vec_ok && j + 3 < num_cols) return *reinterpret_cast<const float4*>(x + j);
    float4 f;
    f.x = (j + 0 < num_cols) ? x[j + 0] : -INFINITY;
    f.y = (j + 1 < num_cols) ? x[j + 1] : -INFINITY;
    f.z = (j + 2 < num_cols) ? x[j + 2] : -INFINITY;
    f.w = (j + 3 < num_cols) ? x[j + 3] : -INFINITY;
    return f;
}

__device__ __forceinline__ float key_to_float(uint32_t key) {      // inverse of order_key
    return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

// TS_THREADS = 512: two CTAs per SM, for many rows; 1024: one CTA with twice the loads in flight,
// for the few rows of a decode step (every row then has an SM to itself).
template <int TS_THREADS>
__global__ void __launch_bounds__(TS_THREADS, 1024 / TS_THREADS)
topk_select_kernel(const float* __restrict__ logits, const int32_t* __restrict__ ks,
                   const int32_t* __restrict__ ke, int32_t* __restrict__ out, int num_cols,
                   int64_t logits_stride, int k) {
    constexpr int TS_WARPS = TS_THREADS / 32;
    constexpr int TS_LIST = TS_CAND / TS_WARPS;        // candidates per warp
    constexpr int TS_BPT = TS_BINS / TS_THREADS;       // histogram bins per thread in the suffix sums
    extern __shared__ __align__(16) uint8_t ts_smem[];
    int* lists = reinterpret_cast<int*>(ts_smem);                               // [TS_WARPS][TS_LIST] candidate columns
    uint32_t* keys = reinterpret_cast<uint32_t*>(ts_smem) + TS_WARPS * TS_LIST; // their keys
    int* hist = reinterpret_cast<int*>(keys + TS_WARPS * TS_LIST);              // [TS_BINS]
    uint32_t* eq_key = reinterpret_cast<uint32_t*>(hist + TS_BINS);             // [TS_EQ]
    int* eq_col = reinterpret_cast<int*>(eq_key + TS_EQ);                       // [TS_EQ]
    __shared__ int sel_bin, sel_need, n_eq_s;
    __shared__ uint32_t kmin_s, kmax_s, last_key_s;
    __shared__ int last_col_s;
    __shared__ int cw[TS_WARPS], cc[TS_WARPS], wsum[TS_WARPS];

    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * logits_stride;
    int lo = ks ? max(ks[row], 0) : 0;
    int hi = ke ? min(ke[row], num_cols) : num_cols;
    if (hi < lo) hi = lo;
    int32_t* o = out + (size_t)row * k;
    const uint32_t NEG_INF_KEY = order_key(-INFINITY);
    constexpr uint32_t VALID16 = 0x007fu;      // key >> 16 of -inf: candidates lie strictly above
    const bool vec_ok = ((reinterpret_cast<size_t>(x) & 15) == 0);
    const int base = lo & ~3;
    const int span = hi - lo;
    const uint32_t below = (1u << lane) - 1u;

    // ---- threshold from a sample (two 256-bin histograms at the start of hist[])
    uint32_t t_lo = NEG_INF_KEY + 1u;          // entries with key >= t_lo become candidates
    const bool sampled = (hi - base) > TS_DIRECT;
    if (tid == 0) { n_eq_s = 0; kmin_s = 0xffffffffu; kmax_s = 0u; }
    if (sampled) {
        if (tid < 512) hist[tid] = 0;
        __syncthreads();
        const int run_stride = span / (TS_SAMPLE / 8);   // >= 15: the runs of 8 do not overlap
        uint32_t h[TS_SAMPLE / TS_THREADS];
#pragma unroll
        for (int r = 0; r < TS_SAMPLE / TS_THREADS; ++r) {
            const int i = tid + TS_THREADS * r;
            h[r] = order_key(x[lo + (i >> 3) * run_stride + (i & 7)]) >> 16;
        }
#pragma unroll
        for (int r = 0; r < TS_SAMPLE / TS_THREADS; ++r)
            if (h[r] > VALID16) atomicAdd(&hist[h[r] >> 8], 1);
        __syncthreads();
        // expected rank of the row's k-th entry inside the sample, plus four standard deviations
        const float m = (float)k * (float)TS_SAMPLE / (float)span;
        const int need_s = (int)(m + 4.f * sqrtf(m)) + 4;
        if (warp == 0) pick_bin(hist, need_s, lane, &sel_bin, &sel_need);
        __syncthreads();
        if (sel_bin >= 0) {
            const uint32_t b1 = (uint32_t)sel_bin;
            const int need1 = sel_need;
#pragma unroll
            for (int r = 0; r < TS_SAMPLE / TS_THREADS; ++r)
                if (h[r] > VALID16 && (h[r] >> 8) == b1) atomicAdd(&hist[256 + (h[r] & 255u)], 1);
            __syncthreads();
            if (warp == 0) pick_bin(hist + 256, need1, lane, &sel_bin, &sel_need);
            __syncthreads();
            t_lo = max(((b1 << 8) | (uint32_t)sel_bin) << 16, NEG_INF_KEY + 1u);
        }
    }
    const float t_f = key_to_float(t_lo);

    // ---- the one pass over the row
    const int nblk = (hi - base + 127) >> 7;
    int* mine = lists + warp * TS_LIST;
    uint32_t* mykeys = keys + warp * TS_LIST;
    int cnt = 0;                               // entries this warp has met (beyond TS_LIST they are only counted)
    const float4 none = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    auto load_blk = [&](int blk) -> float4 {   // blocks past the end read as -inf
        return (blk < nblk) ? load_row4(x, base + blk * 128 + 4 * lane, num_cols, vec_ok) : none;
    };
    for (int stretch = 0; stretch < nblk; stretch += TS_ROUNDS * 4 * TS_WARPS) {
        uint32_t marks[TS_ROUNDS];             // bit 4u + e: entry e of the lane's float4 in block u of the round
        float4 f[4], g[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) f[u] = load_blk(stretch + warp + u * TS_WARPS);
#pragma unroll
        for (int r = 0; r < TS_ROUNDS; ++r) {
            const int blk0 = stretch + r * 4 * TS_WARPS + warp;
            if (r + 1 < TS_ROUNDS) {           // the next round's loads go out before this round is looked at
#pragma unroll
                for (int u = 0; u < 4; ++u) g[u] = load_blk(blk0 + (4 + u) * TS_WARPS);
            }
            uint32_t m = 0;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                m |= (uint32_t)(f[u].x >= t_f) << (4 * u) | (uint32_t)(f[u].y >= t_f) << (4 * u + 1) |
                     (uint32_t)(f[u].z >= t_f) << (4 * u + 2) | (uint32_t)(f[u].w >= t_f) << (4 * u + 3);
            }
            if (m != 0 && (blk0 == 0 || blk0 + 3 * TS_WARPS >= nblk - 1)) {       // the window's edges
#pragma unroll
                for (int b = 0; b < 16; ++b) {
                    const int j = base + (blk0 + (b >> 2) * TS_WARPS) * 128 + 4 * lane + (b & 3);
                    if (j < lo || j >= hi) m &= ~(1u << b);
                }
            }
            marks[r] = m;
#pragma unroll
            for (int u = 0; u < 4; ++u) f[u] = g[u];
        }
        int c = 0;
#pragma unroll
        for (int r = 0; r < TS_ROUNDS; ++r) c += __popc(marks[r]);
        int incl = c;                          // inclusive prefix over the lanes
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        int at = cnt + incl - c;
#pragma unroll
        for (int r = 0; r < TS_ROUNDS; ++r) {
            uint32_t m = marks[r];
            const int j0 = base + (stretch + r * 4 * TS_WARPS + warp) * 128 + 4 * lane;
            while (m) {
                const int b = __ffs(m) - 1;
                m &= m - 1;
                if (at < TS_LIST) mine[at] = j0 + (b >> 2) * (TS_WARPS * 128) + (b & 3);
                ++at;
            }
        }
        cnt += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) cw[warp] = cnt;
    for (int b = tid; b < TS_BINS; b += TS_THREADS) hist[b] = 0;
    __syncthreads();
    int total = 0;
    bool overflow = false;
#pragma unroll
    for (int w = 0; w < TS_WARPS; ++w) { total += cw[w]; overflow |= cw[w] > TS_LIST; }
    if (overflow || (sampled && total < k)) {  // (uniform) the guess failed: the multi-pass kernel redoes the row
        if (tid == 0) o[0] = TK_REDO;
        return;
    }
    const int mycount = cnt;
    const bool take_all = total <= k;
    int thr_bin = -1, need_eq = 0, shift = 0;  // chosen: bin > thr_bin, and need_eq of the entries of bin thr_bin
    uint32_t kmin = 0;
    // Bins are linear in key space (robust against outliers: a key step is a relative step of the
    // value) unless the candidates lie on both sides of zero: most of the key range between a
    // small negative and a small positive value belongs to magnitudes no logit has, so the bins
    // are then linear in the value itself.
    bool by_value = false;
    float vmin_f = 0.f, vscale = 0.f;
    auto bin_of = [&](uint32_t key) -> int {
        if (!by_value) return (int)((key - kmin) >> shift);
        return min((int)((key_to_float(key) - vmin_f) * vscale), TS_BINS - 1);
    };
    if (!take_all) {
        // ---- keys of the candidates, and the range they span
        uint32_t vmin = 0xffffffffu, vmax = 0u;
#pragma unroll 4
        for (int i = lane; i < mycount; i += 32) {
            const uint32_t key = order_key(x[mine[i]]);
            mykeys[i] = key;
            vmin = min(vmin, key); vmax = max(vmax, key);
        }
        vmin = __reduce_min_sync(0xffffffffu, vmin);
        vmax = __reduce_max_sync(0xffffffffu, vmax);
        if (lane == 0 && mycount > 0) { atomicMin(&kmin_s, vmin); atomicMax(&kmax_s, vmax); }
        __syncthreads();
        kmin = kmin_s;
        const uint32_t range = kmax_s - kmin;
        shift = max(0, 20 - (int)__clz(range | 1u));          // (range >> shift) < TS_BINS
        vmin_f = key_to_float(kmin);
        const float vmax_f = key_to_float(kmax_s);
        by_value = vmin_f < 0.f && vmax_f > 0.f && (vmax_f - vmin_f) < INFINITY;
        vscale = by_value ? (float)TS_BINS / (vmax_f - vmin_f) : 0.f;
        for (int i = lane; i < mycount; i += 32) atomicAdd(&hist[bin_of(mykeys[i])], 1);
        __syncthreads();
        // ---- the bin of the k-th: suffix sums over the bins, TS_BPT bins per thread
        {
            int hb[TS_BPT], s = 0;
#pragma unroll
            for (int i = 0; i < TS_BPT; ++i) { hb[i] = hist[TS_BPT * tid + i]; s += hb[i]; }
            int suf = s;                       // sum over the lanes >= this one
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_down_sync(0xffffffffu, suf, d);
                if (lane + d < 32) suf += t;
            }
            if (lane == 0) wsum[warp] = suf;
            __syncthreads();
            int above = suf - s;
#pragma unroll
            for (int w = 0; w < TS_WARPS; ++w) above += (w > warp) ? wsum[w] : 0;
            if (above < k && above + s >= k) {  // exactly one thread: total > k
                int cum = above, b = TS_BPT - 1;
#pragma unroll
                for (int i = TS_BPT - 1; i > 0; --i) {
                    if (b == i && cum + hb[i] < k) { cum += hb[i]; b = i - 1; }
                }
                sel_bin = TS_BPT * tid + b; sel_need = k - cum;
            }
            __syncthreads();
        }
        thr_bin = sel_bin;
        need_eq = sel_need;
        // ---- the entries of that bin, to be ranked one against the other
        for (int i = lane; i < mycount; i += 32) {
            const uint32_t key = mykeys[i];
            if (bin_of(key) == thr_bin) {
                const int at = atomicAdd(&n_eq_s, 1);
                if (at < TS_EQ) { eq_key[at] = key; eq_col[at] = mine[i]; }
            }
        }
        __syncthreads();
        if (n_eq_s > TS_EQ) {                  // (uniform)
            if (tid == 0) o[0] = TK_REDO;
            return;
        }
    }
    const int n_eq = take_all ? 0 : n_eq_s;
    // The last of the bin's entries to be taken, in the order (key descending, column ascending):
    // every entry of the bin finds its own rank once (n_eq^2 comparisons spread over the CTA), the
    // one of rank need_eq - 1 publishes itself, and membership is then a comparison with it.
    if (!take_all && need_eq < n_eq) {
        for (int i = tid; i < n_eq; i += TS_THREADS) {
            const uint32_t key = eq_key[i];
            const int c = eq_col[i];
            int rank = 0;
            for (int j = 0; j < n_eq; ++j) rank += (eq_key[j] > key) || (eq_key[j] == key && eq_col[j] < c);
            if (rank == need_eq - 1) { last_key_s = key; last_col_s = c; }
        }
        __syncthreads();
    }
    const bool all_eq = need_eq >= n_eq;
    const uint32_t last_key = all_eq ? 0u : last_key_s;
    const int last_col = all_eq ? 0x7fffffff : last_col_s;
    auto chosen = [&](int i) -> bool {
        if (take_all) return true;
        const uint32_t key = mykeys[i];
        const int bin = bin_of(key);
        if (bin != thr_bin) return bin > thr_bin;
        return key > last_key || (key == last_key && mine[i] <= last_col);
    };
    // ---- write: every warp its own list, in list order
    int nsel = 0;
    for (int i0 = 0; i0 < mycount; i0 += 32) {
        const bool ch = (i0 + lane < mycount) && chosen(i0 + lane);
        nsel += __popc(__ballot_sync(0xffffffffu, ch));
    }
    if (lane == 0) cc[warp] = nsel;
    __syncthreads();
    int off = 0, filled = 0;
#pragma unroll
    for (int w = 0; w < TS_WARPS; ++w) { if (w < warp) off += cc[w]; filled += cc[w]; }
    for (int i0 = 0; i0 < mycount; i0 += 32) {
        const bool ch = (i0 + lane < mycount) && chosen(i0 + lane);
        const uint32_t mc = __ballot_sync(0xffffffffu, ch);
        if (ch) o[off + __popc(mc & below)] = mine[i0 + lane];
        off += __popc(mc);
    }
    for (int r = filled + tid; r < k; r += TS_THREADS) o[r] = -1;
}

// ---------------------------------------------------------------- context-parallel partition
// One warp per row: stable compaction of the entries inside [lo, hi), rebased to lo.
__global__ void __launch_bounds__(256)
cp_partition_kernel(const int32_t* __restrict__ indices, int32_t* __restrict__ local_indices,
                    int32_t* __restrict__ local_length, int num_tokens, int topk, int lo, int hi) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= num_tokens) return;
    const int32_t* in = indices + (size_t)row * topk;
    int32_t* o = local_indices + (size_t)row * topk;
    int n = 0;
    for (int j0 = 0; j0 < topk; j0 += 32) {
        const int j = j0 + lane;
        const int v = (j < topk) ? in[j] : -1;
        const bool keep = (v >= lo) && (v < hi);
        const uint32_t m = __ballot_sync(0xffffffffu, keep);
        if (keep) o[n + __popc(m & ((1u << lane) - 1u))] = v - lo;
        n += __popc(m);
    }
    for (int j = n + lane; j < topk; j += 32) o[j] = -1;
    if (lane == 0) local_length[row] = n;
}


// ---------------------------------------------------------------- distributed top-k: the glue
// Window of every token clipped to the shard [lo, hi), in shard-local positions.
__global__ void cp_window_kernel(const int32_t* __restrict__ ks, const int32_t* __restrict__ ke,
                                 int32_t* __restrict__ ks_local, int32_t* __restrict__ ke_local,
                                 int num_tokens, int lo, int hi) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_tokens) return;
    const int n = hi - lo;
    ks_local[i] = min(max(ks[i] - lo, 0), n);
    ke_local[i] = min(max(ke[i] - lo, 0), n);
}

// The shard's candidates of a token: logit and global position of every picked column
// (-inf / -1 where the shard had fewer than k).
__global__ void cp_candidates_kernel(const float* __restrict__ logits, int64_t logits_stride,
                                     const int32_t* __restrict__ picked, float* __restrict__ values,
                                     int32_t* __restrict__ positions, int num_tokens, int k, int lo) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)num_tokens * k) return;
    const int c = picked[i];
    values[i] = (c >= 0) ? logits[(i / k) * logits_stride + c] : -INFINITY;
    positions[i] = (c >= 0) ? c + lo : -1;
}

// gathered [world][2][num_tokens][k] (values, then positions, of every rank) -> the candidates of
// a token side by side: values / positions [num_tokens][world * k].
__global__ void cp_interleave_kernel(const int32_t* __restrict__ gathered, int32_t* __restrict__ values,
                                     int32_t* __restrict__ positions, int world, int num_tokens, int k) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // index into [num_tokens][world][k]
    const int64_t per = (int64_t)num_tokens * k;
    if (i >= per * world) return;
    const int j = (int)(i % k), g = (int)((i / k) % world);
    const int64_t t = i / ((int64_t)k * world);
    const int32_t* src = gathered + (int64_t)g * 2 * per + t * k + j;
    values[i] = src[0];
    positions[i] = src[per];
}

// out[t][i] = positions[t][pick[t][i]] (-1 where pick is -1).
__global__ void cp_pick_kernel(const int32_t* __restrict__ positions, const int32_t* __restrict__ pick,
                               int32_t* __restrict__ out, int num_tokens, int k, int num_candidates) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)num_tokens * k) return;
    const int c = pick[i];
    out[i] = (c >= 0) ? positions[(i / k) * num_candidates + c] : -1;
}

}  // namespace

int launch_mqa_logits_scalar(const uint8_t* q, const uint8_t* k, const float* k_scale, const float* weights,
                             const int32_t* ks, const int32_t* ke, float* logits, int s_q, int num_heads,
                             int s_k, int64_t logits_stride, cudaStream_t stream) {
    if (s_q == 0 || s_k == 0) return 0;
    const size_t smem = (size_t)num_heads * LD * sizeof(float);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev < 64 && !attr_set[dev]) {
        cudaFuncSetAttribute(mqa_logits_scalar_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
        attr_set[dev] = true;
    }
    dim3 grid((s_k + LK - 1) / LK, s_q);
    mqa_logits_scalar_kernel<<<grid, 256, smem, stream>>>(q, k, k_scale, weights, ks, ke, logits, num_heads,
                                                        s_k, logits_stride);
    return check_launch("mqa_logits_scalar_kernel");
}

int launch_topk(const float* logits, const int32_t* ks, const int32_t* ke, int32_t* out, int num_rows,
                int num_cols, int64_t logits_stride, int k, cudaStream_t stream) {
    if (num_rows == 0 || k == 0) return 0;
    if (k > TS_KMAX) {
        topk_kernel<<<num_rows, TK_THREADS, 0, stream>>>(logits, ks, ke, out, num_cols, logits_stride, k, 0);
        return check_launch("topk_kernel");
    }
    static bool attr_set[64] = {};
    static int sms[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(topk_select_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, TS_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(topk_select_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, TS_SMEM);
        if (e != cudaSuccess) return set_error((int)e, "topk_select_kernel: shared memory: %s", cudaGetErrorString(e));
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        attr_set[dev] = true;
    }
    if (num_rows <= sms[dev < 64 ? dev : 0])       // every row has an SM to itself
        topk_select_kernel<1024><<<num_rows, 1024, TS_SMEM, stream>>>(logits, ks, ke, out, num_cols, logits_stride, k);
    else
        topk_select_kernel<512><<<num_rows, 512, TS_SMEM, stream>>>(logits, ks, ke, out, num_cols, logits_stride, k);
    if (const int rc = check_launch("topk_select_kernel")) return rc;
    // rows the one-read kernel gave up on (it marks them) are redone by the multi-pass kernel
    topk_kernel<<<num_rows, TK_THREADS, 0, stream>>>(logits, ks, ke, out, num_cols, logits_stride, k, 1);
    return check_launch("topk_kernel");
}

int launch_cp_partition(const int32_t* indices, int32_t* local_indices, int32_t* local_length,
                        int num_tokens, int topk, int lo, int hi, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    cp_partition_kernel<<<(num_tokens + 7) / 8, 256, 0, stream>>>(indices, local_indices, local_length,
                                                                  num_tokens, topk, lo, hi);
    return check_launch("cp_partition_kernel");
}

int launch_cp_window(const int32_t* ks, const int32_t* ke, int32_t* ks_local, int32_t* ke_local, int num_tokens,
                     int lo, int hi, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    cp_window_kernel<<<(num_tokens + 255) / 256, 256, 0, stream>>>(ks, ke, ks_local, ke_local, num_tokens, lo, hi);
    return check_launch("cp_window_kernel");
}

int launch_cp_candidates(const float* logits, int64_t logits_stride, const int32_t* picked, float* values,
                         int32_t* positions, int num_tokens, int k, int lo, cudaStream_t stream) {
    const int64_t n = (int64_t)num_tokens * k;
    if (n == 0) return 0;
    cp_candidates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(logits, logits_stride, picked, values, positions,
                                                                           num_tokens, k, lo);
    return check_launch("cp_candidates_kernel");
}

int launch_cp_interleave(const int32_t* gathered, int32_t* values, int32_t* positions, int world, int num_tokens, int k,
                         cudaStream_t stream) {
    const int64_t n = (int64_t)num_tokens * k * world;
    if (n == 0) return 0;
    cp_interleave_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(gathered, values, positions, world, num_tokens, k);
    return check_launch("cp_interleave_kernel");
}

int launch_cp_pick(const int32_t* positions, const int32_t* pick, int32_t* out, int num_tokens, int k, int num_candidates,
                   cudaStream_t stream) {
    const int64_t n = (int64_t)num_tokens * k;
    if (n == 0) return 0;
    cp_pick_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(positions, pick, out, num_tokens, k, num_candidates);
    return check_launch("cp_pick_kernel");
}

}  // namespace smla
