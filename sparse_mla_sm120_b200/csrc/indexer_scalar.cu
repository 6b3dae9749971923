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
constexpr int TK_CAND = 1024;              // candidates (entries of the threshold's 16-bit bin) topk16_kernel resolves itself
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
    // only_flagged: redo the rows that topk16_kernel marked as beyond its candidate list
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

// Two-read variant for rows of at most 65536 columns.  The first read of the row leaves the top
// 16 bits of every key in shared memory (128 KB) and a histogram of the top 8; the second 8 bits
// are resolved from shared memory, which fixes the threshold's 16-bit bin.  Entries above the bin
// are written in column order; the entries inside it (a few dozen for real logits) are the only
// ones whose full keys are read again, and the needed number of them is chosen by rank (key
// descending, lower column first) and written after the others, again in column order.  A row
// with more than TK_CAND entries in its bin is marked for the multi-pass kernel.
__global__ void __launch_bounds__(TK_THREADS, 1)
topk16_kernel(const float* __restrict__ logits, const int32_t* __restrict__ ks,
              const int32_t* __restrict__ ke, int32_t* __restrict__ out, int num_cols,
              int64_t logits_stride, int k) {
    extern __shared__ uint16_t k16[];          // top 16 key bits of columns [lo, hi)
    __shared__ int hist[256];
    __shared__ int sel_bin, sel_need;
    __shared__ int seg_gt[TK_WARPS], seg_eq[TK_WARPS];
    __shared__ uint32_t cand_key[TK_CAND];
    __shared__ int cand_col[TK_CAND];

    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * logits_stride;
    int lo = ks ? max(ks[row], 0) : 0;
    int hi = ke ? min(ke[row], num_cols) : num_cols;
    if (hi < lo) hi = lo;
    int32_t* o = out + (size_t)row * k;
    constexpr uint32_t VALID16 = 0x007fu;      // key16 of -inf (and of negative NaNs): candidates lie strictly above
    const bool vec_ok = ((reinterpret_cast<size_t>(x) & 15) == 0);

    // ---- read 1: 16-bit keys to shared memory, histogram of the top 8 bits
    for (int b = tid; b < 256; b += TK_THREADS) hist[b] = 0;
    __syncthreads();
    auto first = [&](int j, uint32_t key) {
        const uint32_t h = key >> 16;
        k16[j - lo] = (uint16_t)h;
        if (h > VALID16) atomicAdd(&hist[h >> 8], 1);
    };
    if (vec_ok) for_each_key(x, lo, hi, tid, TK_THREADS, first);
    else for (int j = lo + tid; j < hi; j += TK_THREADS) first(j, order_key(x[j]));
    __syncthreads();
    auto pick = [&](int need) {        // thread 0: highest bin at which the cumulated count reaches `need`
        int cum = 0, b = 255;
        for (; b >= 0; --b) {
            if (cum + hist[b] >= need) break;
            cum += hist[b];
        }
        sel_bin = b; sel_need = need - cum;
    };
    if (tid == 0) pick(k);
    __syncthreads();
    bool take_all = sel_bin < 0;               // fewer candidates than k: every one is taken
    uint32_t t16 = VALID16;                    // entries with key16 > t16 are taken outright
    int need = 0;                              // and `need` of those with key16 == t16
    if (!take_all) {
        const uint32_t b1 = (uint32_t)sel_bin;
        const int need1 = sel_need;
        __syncthreads();
        // ---- second 8 bits, from shared memory
        for (int b = tid; b < 256; b += TK_THREADS) hist[b] = 0;
        __syncthreads();
        for (int i = tid; i < hi - lo; i += TK_THREADS) {
            const uint32_t h = k16[i];
            if (h > VALID16 && (h >> 8) == b1) atomicAdd(&hist[h & 255u], 1);
        }
        __syncthreads();
        if (tid == 0) pick(need1);
        __syncthreads();
        t16 = (b1 << 8) | (uint32_t)sel_bin;   // sel_bin >= 0: the bin b1 holds at least need1 entries
        need = sel_need;
    }

    // ---- ordered write of the entries above the bin; the bin's entries go to the candidate list
    const int span = hi - lo;
    const int seg = ((span + TK_WARPS - 1) / TK_WARPS + 31) & ~31;
    const int s0 = min(warp * seg, span), s1 = min(s0 + seg, span);
    int c_gt = 0, c_eq = 0;
    for (int i = s0 + lane; i < s1; i += 32) {
        const uint32_t h = k16[i];
        c_gt += (h > t16);
        c_eq += (!take_all && h == t16);
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
    if (n_eq > TK_CAND) {                       // (uniform) too many for the list: leave the row to the multi-pass kernel
        if (tid == 0) o[0] = TK_REDO;
        return;
    }
    const uint32_t below = (1u << lane) - 1u;
    for (int i0 = s0; i0 < s1; i0 += 32) {
        const int i = i0 + lane;
        const uint32_t h = (i < s1) ? k16[i] : 0u;
        const bool gt = (i < s1) && h > t16;
        const bool eq = (i < s1) && !take_all && h == t16;
        const uint32_t mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
        if (gt) o[off_gt + __popc(mg & below)] = lo + i;
        if (eq) cand_col[off_eq + __popc(me & below)] = lo + i;
        off_gt += __popc(mg); off_eq += __popc(me);
    }
    __syncthreads();
    // ---- the bin's entries: full keys (second read, these few only), rank, ordered write of the chosen ones
    int taken = 0;
    if (n_eq > 0) {
        if (tid < n_eq) cand_key[tid] = order_key(x[cand_col[tid]]);
        __syncthreads();
        bool chosen = false;
        if (tid < n_eq) {
            if (need >= n_eq) chosen = true;
            else {
                const uint32_t mine = cand_key[tid];
                int rank = 0;                   // entries that go before this one: larger key, or equal key and lower column
                for (int j = 0; j < n_eq; ++j) {
                    const uint32_t kj = cand_key[j];
                    rank += (kj > mine) || (kj == mine && j < tid);
                }
                chosen = rank < need;
            }
        }
        const uint32_t mc = __ballot_sync(0xffffffffu, chosen);
        if (lane == 0) seg_eq[warp] = __popc(mc);
        __syncthreads();
        int off = 0;
        for (int w = 0; w < warp; ++w) off += seg_eq[w];
        if (chosen) o[n_gt + off + __popc(mc & below)] = cand_col[tid];
        taken = min(need, n_eq);
    }
    for (int r = n_gt + taken + tid; r < k; r += TK_THREADS) o[r] = -1;
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
    if (num_cols > 65536) {
        topk_kernel<<<num_rows, TK_THREADS, 0, stream>>>(logits, ks, ke, out, num_cols, logits_stride, k, 0);
        return check_launch("topk_kernel");
    }
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int smem = 65536 * (int)sizeof(uint16_t);
    if (dev < 64 && !attr_set[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(topk16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return set_error((int)e, "topk16_kernel: shared memory: %s", cudaGetErrorString(e));
        attr_set[dev] = true;
    }
    topk16_kernel<<<num_rows, TK_THREADS, smem, stream>>>(logits, ks, ke, out, num_cols, logits_stride, k);
    if (int e = check_launch("topk16_kernel")) return e;
    // rows whose threshold bin was larger than the candidate list (marked in their first output) are redone
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

}  // namespace smla
