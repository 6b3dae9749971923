// Split-KV tile scheduler: assigns contiguous runs of 64-token blocks to partitions.
//
// Behaviour matches the reference scheduler (csrc/kernel/sched/get_sched_meta.cu:25-125):
// every request costs its block count plus a fixed overhead, each partition receives
// ceil(total / parts) + overhead units, and a request that straddles a partition boundary
// becomes one more split.  One warp: lanes count blocks in parallel, lane 0 walks the
// partitions (the walk is inherently sequential and a few hundred steps long) recording only
// the state at which each partition starts; all lanes then assemble the records and the prefix
// sum of the split counts.
#include "common.cuh"

namespace smla {

namespace {

struct SchedArgs {
    int b, topk, extra_topk, parts, overhead;
    const int32_t* topk_length;
    const int32_t* extra_topk_length;
    SchedMeta* meta;
    int32_t* num_splits;
};

__global__ void __launch_bounds__(32) sched_meta_kernel(const SchedArgs a) {
    grid_dep_launch();   // the attention kernel may start its prologue; it waits for this kernel before it reads the records
    extern __shared__ int sh[];
    int* nblk = sh;                    // [b]   blocks of request i
    int* nsp = sh + a.b;               // [b+1] nsp[i+1] = splits of request i, then their prefix sum
    int* state = sh + ((2 * a.b + 1 + 3) & ~3);   // [parts+1][4] (request, block, split) at which a partition starts, 16-byte aligned
    const int lane = threadIdx.x;

    int cost = 0;
    for (int i = lane; i < a.b; i += 32) {
        int len = a.topk_length ? a.topk_length[i] : a.topk;
        if (len == 0) len = 1;
        if (a.extra_topk > 0) {
            len = (len + BLOCK_N - 1) / BLOCK_N * BLOCK_N;
            len += a.extra_topk_length ? a.extra_topk_length[i] : a.extra_topk;
        }
        const int n = (len > 0 ? (len - 1) / BLOCK_N : 0) + 1;
        nblk[i] = n;
        nsp[i + 1] = 0;
        cost += n + a.overhead;
    }
    if (lane == 0) nsp[0] = 0;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) cost += __shfl_xor_sync(0xffffffffu, cost, o);
    __syncwarp();

    // The walk over the partitions is sequential; lane 0 keeps it to the bare state transitions
    // (the records are assembled from the recorded states by all lanes afterwards).
    if (lane == 0) {
        const int budget = (cost + a.parts - 1) / a.parts + a.overhead;
        int req = 0, blk = 0, nsplit = 0;
        int cur = (a.b > 0) ? nblk[0] : 0;   // nblk[req]
        for (int p = 0; p < a.parts; ++p) {
            *reinterpret_cast<int4*>(state + 4 * p) = make_int4(req, blk, nsplit, 0);
            int left = budget;
            while (req < a.b) {
                const int rest = cur - blk;
                if (left >= rest + a.overhead) {      // the rest of this request fits
                    nsp[req + 1] = nsplit + 1;
                    left -= rest + a.overhead;
                    ++req; blk = 0; nsplit = 0;
                    cur = (req < a.b) ? nblk[req] : 0;
                } else {                              // take what fits, leave the request split
                    if (left > a.overhead) { blk += left - a.overhead; ++nsplit; }
                    break;
                }
            }
        }
        *reinterpret_cast<int4*>(state + 4 * a.parts) = make_int4(req, blk, nsplit, 0);
    }
    __syncwarp();

    static_assert(sizeof(SchedMeta) == 32, "scheduler records are eight 32-bit words");
    for (int p = lane; p < a.parts; p += 32) {
        const int4 s0 = *reinterpret_cast<const int4*>(state + 4 * p);
        const int4 s1 = *reinterpret_cast<const int4*>(state + 4 * (p + 1));
        SchedMeta m;
        m.begin_req = s0.x;
        m.begin_block = (s0.x < a.b) ? s0.y : 0;
        m.begin_split = s0.z;
        m.first_split = (s0.y != 0);
        m.end_req = (s1.y > 0) ? s1.x : s1.x - 1;
        m.end_block = (s1.y > 0) ? s1.y : (s1.x > 0 ? nblk[s1.x - 1] : 0);
        m.last_split = (m.end_req >= 0 && m.end_req < a.b && m.end_block != nblk[m.end_req]);
        if (m.begin_req == m.end_req) m.first_split = m.last_split = (m.first_split | m.last_split);
        m.pad = 0;
        a.meta[p] = m;
    }
    // prefix sum of the per-request split counts
    int carry = 0;
    for (int i0 = 0; i0 <= a.b; i0 += 32) {
        const int i = i0 + lane;
        int v = (i <= a.b) ? nsp[i] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += t;
        }
        if (i <= a.b) a.num_splits[i] = v + carry;
        carry += __shfl_sync(0xffffffffu, v, 31);
    }
}

}  // namespace

int launch_sched_meta(int b, int topk, int extra_topk, int num_sm_parts, int fixed_overhead,
                      const int32_t* topk_length, const int32_t* extra_topk_length,
                      int32_t* sched_meta, int32_t* num_splits, cudaStream_t stream) {
    SchedArgs a{b, topk, extra_topk, num_sm_parts, fixed_overhead, topk_length, extra_topk_length,
                reinterpret_cast<SchedMeta*>(sched_meta), num_splits};
    const size_t smem = sizeof(int) * (2 * (size_t)b + 4 + 4 * ((size_t)num_sm_parts + 1));
    static bool big_smem[64] = {};
    if (smem > 48 * 1024) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 64 && !big_smem[dev]) {
            cudaFuncSetAttribute(sched_meta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            big_smem[dev] = true;
        }
    }
    sched_meta_kernel<<<1, 32, smem, stream>>>(a);
    return check_launch("sched_meta_kernel");
}

}  // namespace smla
