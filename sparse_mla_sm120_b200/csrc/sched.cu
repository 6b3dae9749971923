// Split-KV tile scheduler: assigns contiguous runs of 64-token blocks to partitions.
//
// Behaviour matches the reference scheduler (csrc/kernel/sched/get_sched_meta.cu:25-125):
// every request costs its block count plus a fixed overhead, each partition receives
// ceil(total / parts) + overhead units, and a request that straddles a partition boundary
// becomes one more split.  One warp: lanes count blocks in parallel, lane 0 walks the
// partitions (the walk is inherently sequential and a few hundred steps long) entirely in
// shared memory, then all lanes copy the records out.
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
    extern __shared__ int sh[];
    int* nblk = sh;               // [b]   blocks of request i
    int* splits = sh + a.b;       // [b+1] prefix sum of splits
    int* meta_sh = sh + 2 * a.b + 1;   // [parts][8] records, copied out at the end
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
        cost += n + a.overhead;
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) cost += __shfl_xor_sync(0xffffffffu, cost, o);
    __syncwarp();

    if (lane == 0) {
        const int budget = (cost + a.parts - 1) / a.parts + a.overhead;
        int req = 0, blk = 0, nsplit = 0, cum = 0;
        splits[0] = 0;
        for (int p = 0; p < a.parts; ++p) {
            SchedMeta m;
            m.begin_req = req;
            m.begin_block = (req < a.b) ? blk : 0;
            m.begin_split = nsplit;
            m.first_split = (blk != 0);
            int left = budget;
            while (req < a.b) {
                const int rest = nblk[req] - blk;
                if (left >= rest + a.overhead) {      // the rest of this request fits
                    cum += nsplit + 1;
                    splits[req + 1] = cum;
                    left -= rest + a.overhead;
                    ++req; blk = 0; nsplit = 0;
                } else {                              // take what fits, leave the request split
                    if (left > a.overhead) { blk += left - a.overhead; ++nsplit; }
                    break;
                }
            }
            m.end_req = (blk > 0) ? req : req - 1;
            m.end_block = (blk > 0) ? blk : (req > 0 ? nblk[req - 1] : 0);
            m.last_split = (m.end_req >= 0 && m.end_req < a.b && m.end_block != nblk[m.end_req]);
            if (m.begin_req == m.end_req) m.first_split = m.last_split = (m.first_split | m.last_split);
            m.pad = 0;
            *reinterpret_cast<SchedMeta*>(meta_sh + 8 * p) = m;
        }
    }
    __syncwarp();
    static_assert(sizeof(SchedMeta) == 32, "scheduler records are eight 32-bit words");
    int* meta_out = reinterpret_cast<int*>(a.meta);
    for (int i = lane; i < 8 * a.parts; i += 32) meta_out[i] = meta_sh[i];
    for (int i = lane; i <= a.b; i += 32) a.num_splits[i] = splits[i];
}

}  // namespace

int launch_sched_meta(int b, int topk, int extra_topk, int num_sm_parts, int fixed_overhead,
                      const int32_t* topk_length, const int32_t* extra_topk_length,
                      int32_t* sched_meta, int32_t* num_splits, cudaStream_t stream) {
    SchedArgs a{b, topk, extra_topk, num_sm_parts, fixed_overhead, topk_length, extra_topk_length,
                reinterpret_cast<SchedMeta*>(sched_meta), num_splits};
    const size_t smem = sizeof(int) * (2 * (size_t)b + 1 + 8 * (size_t)num_sm_parts + 8);
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
