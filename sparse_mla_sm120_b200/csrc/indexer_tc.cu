// FP8 MQA-logits indexer on tcgen05 tensor cores (sm_100a).
//
//   logits[i, j] = k_scale[j] * sum_h w[i, h] * relu(q[i, h, :] . k[j, :]),   -inf outside [ks_i, ke_i)
//
// No counterpart in the reference project (its indices come from an external indexer).  The
// contraction is run transposed: a tile of 128 keys is the M side, the (query, head) pairs of
// four queries are the N side (N = 4 * heads <= 256), K = 128 e4m3 values, so that one thread of
// the epilogue owns one key (one TMEM lane) and the ReLU / head-weighted sum runs along the
// columns it holds, with no cross-thread reduction.  Two accumulators (2 x 256 TMEM columns) let
// the MMAs of the next key tile run under the epilogue of the current one.
//
// One CTA walks query groups (4 queries) round-robin and, per group, the key tiles up to the
// largest ke of the group.  Warps: 0-15 epilogue (warp w: TMEM lane quarter w % 4, query w / 4
// of the group; the epilogue is bound by instruction issue, so it gets four warps per scheduler),
// 16 loader (one TMA tile load per key tile and per q group: both are contiguous rows of 128
// bytes in global memory and land 128B-swizzled, K-major; rows past the end arrive as zeros),
// 17 MMA issue (one thread).
// The kernel is tensor-bound at the benchmark shape (4.26 TFLOP) with the logits write
// (1.07 GB) as the second term.  Every wait is bounded.
#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace smla {

namespace {

using namespace ptx;

constexpr int LX_D = 128;            // head dim of the indexer (bytes per row)
constexpr int LX_KT = 128;           // keys per tile
constexpr int LX_QG = 4;             // queries per group
constexpr int LX_EPI_WARPS = 16;
constexpr int LX_LOAD_WARP = 16, LX_MMA_WARP = 17;
constexpr int LX_THREADS = 18 * 32;
constexpr int LX_KSTAGE = 4;

constexpr uint32_t LX_Q_OFF = 0;                              // q group: [<=256 rows x 128 B] K-major 128B swizzle
constexpr uint32_t LX_K_OFF = 256 * 128;                      // key tiles: LX_KSTAGE x [128 rows x 128 B]
constexpr uint32_t LX_W_OFF = LX_K_OFF + LX_KSTAGE * LX_KT * 128;   // weights: 4 rotating buffers of [4 queries][64] fp32
constexpr uint32_t LX_W_BYTES = LX_QG * 64 * 4;
constexpr uint32_t LX_BAR_OFF = LX_W_OFF + 4 * LX_W_BYTES;
// barriers: kfull[4] kempty[4] dfull[2] dempty[2] qfull qempty
constexpr int LXB_KFULL = 0, LXB_KEMPTY = LX_KSTAGE, LXB_DFULL = 2 * LX_KSTAGE, LXB_DEMPTY = LXB_DFULL + 2,
              LXB_QFULL = LXB_DEMPTY + 2, LXB_QEMPTY = LXB_QFULL + 1, LXB_N = LXB_QEMPTY + 1;
constexpr uint32_t LX_MISC_OFF = LX_BAR_OFF + LXB_N * 8;
constexpr uint32_t LX_SMEM_NEED = LX_MISC_OFF + 16 + 1024;
// one CTA per SM (each allocates all 512 TMEM columns): ask for more than half of the SM's shared memory
constexpr uint32_t LX_SMEM = LX_SMEM_NEED > 118 * 1024 ? LX_SMEM_NEED : 118 * 1024;

struct LogitsParams {
    const uint8_t* q; const uint8_t* k; const float* k_scale; const float* w;
    const int32_t* ks; const int32_t* ke; float* logits; int32_t* status;
    int s_q, heads, s_k; int64_t stride;
    int chunk_tiles;   // key tiles per work item (a work item: one query group x one run of key tiles)
};

__global__ void __launch_bounds__(LX_THREADS, 1) mqa_logits_tc_kernel(const LogitsParams p, const __grid_constant__ CUtensorMap qmap,
                                                                      const __grid_constant__ CUtensorMap kmap) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + LX_MISC_OFF + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + LX_MISC_OFF);
    auto bar = [&](int i) -> uint32_t { return base + LX_BAR_OFF + 8u * i; };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int H = p.heads, N = LX_QG * H;

    if (tid == 0) {
        for (int s = 0; s < LX_KSTAGE; ++s) { mbar_init(bar(LXB_KFULL + s), 1); mbar_init(bar(LXB_KEMPTY + s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar(LXB_DFULL + b), 1); mbar_init(bar(LXB_DEMPTY + b), LX_EPI_WARPS * 32); }
        mbar_init(bar(LXB_QFULL), 32);
        mbar_init(bar(LXB_QEMPTY), 1 + LX_EPI_WARPS);   // the MMAs have read q and every epilogue warp has seen the group's phase
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == LX_MMA_WARP) { tmem_alloc(base + LX_MISC_OFF, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int num_groups = (p.s_q + LX_QG - 1) / LX_QG;
    // key tiles a group needs: up to the largest ke of its queries (and from the smallest ks)
    auto group_range = [&](int g, int& t0, int& t1) {
        int lo = p.s_k, hi = 0;
        for (int i = 0; i < LX_QG; ++i) {
            const int qi = g * LX_QG + i;
            if (qi < p.s_q) { lo = min(lo, max(p.ks[qi], 0)); hi = max(hi, min(p.ke[qi], p.s_k)); }
        }
        t0 = (hi > lo) ? lo / LX_KT : 0;
        t1 = (hi > lo) ? (hi + LX_KT - 1) / LX_KT : 0;
    };
    // Work items: item w is query group w % num_groups over the key tiles [c * chunk_tiles, (c + 1) *
    // chunk_tiles) with c = w / num_groups, so that a few decode tokens over a long context still
    // fill the machine and neighbouring CTAs read the same keys.  [t0, t1) are the tiles of the item
    // that the group needs, [j0, j1) the logits columns the item is responsible for.
    const int num_chunks = ((p.s_k + LX_KT - 1) / LX_KT + p.chunk_tiles - 1) / p.chunk_tiles;
    const int num_items = num_groups * num_chunks;
    auto item_range = [&](int w, int& g, int& t0, int& t1, int& j0, int& j1) {
        g = w % num_groups;
        const int c = w / num_groups;
        group_range(g, t0, t1);
        t0 = max(t0, c * p.chunk_tiles);
        t1 = min(t1, (c + 1) * p.chunk_tiles);
        if (t1 < t0) t1 = t0;
        j0 = c * p.chunk_tiles * LX_KT;
        j1 = min(p.s_k, (c + 1) * p.chunk_tiles * LX_KT);
    };

    if (warp < LX_EPI_WARPS) {
        // =================================================================== epilogue
        const int quarter = warp & 3, qp = warp >> 2;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        uint32_t it = 0, qn = 0;   // tiles and non-empty groups seen by this CTA
        bool ok = true;
        for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
            int g, t0, t1, j0, j1;
            item_range(w, g, t0, t1, j0, j1);
            const float* wsm = reinterpret_cast<const float*>(sm + LX_W_OFF + (qn & 3u) * LX_W_BYTES);
            const int q0 = g * LX_QG + qp;
            const int ks0 = q0 < p.s_q ? p.ks[q0] : 0, ke0 = q0 < p.s_q ? p.ke[q0] : 0;
            // columns of the item outside every tile the group needs are -inf: written here, 128 keys per pass
            if (q0 < p.s_q) {
                float* row = p.logits + (size_t)q0 * p.stride;
                for (int j = j0 + quarter * 32 + lane; j < j1; j += 128)
                    if (j < t0 * LX_KT || j >= t1 * LX_KT) row[j] = -INFINITY;
            }
            if (t1 > t0) {
                ok = mbar_wait(bar(LXB_QFULL), qn & 1u, abort_flag, 11);   // weights of the group are in shared memory
                if (!ok) break;
                // The loader may arm the next group only after this warp has seen this one: otherwise two phases
                // of QFULL could complete before a slow epilogue warp waits for the first (a group of one or two
                // tiles needs nothing from the epilogue), and its parity wait would then refer to a later phase.
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(LXB_QEMPTY));
                ++qn;
            }
            for (int t = t0; t < t1 && ok; ++t, ++it) {
                const uint32_t b = it & 1u;
                ok = mbar_wait_hot(bar(LXB_DFULL + b), (it >> 1) & 1u, abort_flag, 12);
                if (!ok) break;
                tc_fence_after();
                const int key = t * LX_KT + quarter * 32 + lane;
                const float sc = key < p.s_k ? __ldg(p.k_scale + key) : 0.f;
                // Chunks of 32 score columns of this warp's query (heads [0,32), [32,64)); the
                // tensor-memory load of the next chunk is in flight while the current one is reduced,
                // and four partial sums per chunk keep the FMA chains short.
                float acc = 0.f;
                const int nch = H >> 5;                          // 1 or 2 chunks
                const uint32_t col0 = lane_addr + 256 * b + qp * H;
                const float* wq = wsm + qp * 64;
                uint32_t d0[32], d1[32];
                tmem_ld32(col0, d0);
                // two scores per instruction: packed fp32 FMAs (same products, same four partial sums
                // as four scalar FMA chains)
                auto reduce = [&](const uint32_t (&d)[32], int c) {
                    uint64_t a01 = 0ull, a23 = 0ull;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const ulonglong2 w4 = *reinterpret_cast<const ulonglong2*>(wq + c + i);      // (w0, w1), (w2, w3)
                        fma_f32x2(a01, pack_f32x2(fmaxf(__uint_as_float(d[i + 0]), 0.f), fmaxf(__uint_as_float(d[i + 1]), 0.f)), w4.x);
                        fma_f32x2(a23, pack_f32x2(fmaxf(__uint_as_float(d[i + 2]), 0.f), fmaxf(__uint_as_float(d[i + 3]), 0.f)), w4.y);
                    }
                    float a0, a1, a2, a3;
                    unpack_f32x2(a01, a0, a1);
                    unpack_f32x2(a23, a2, a3);
                    acc += (a0 + a1) + (a2 + a3);
                };
                tmem_wait_ld();
                if (nch > 1) tmem_ld32(col0 + 32, d1);
                reduce(d0, 0);
                if (nch > 1) { tmem_wait_ld(); reduce(d1, 32); }
                tc_fence_before();
                mbar_arrive(bar(LXB_DEMPTY + b));
                if (key < p.s_k && q0 < p.s_q)
                    p.logits[(size_t)q0 * p.stride + key] = (key >= ks0 && key < ke0) ? acc * sc : -INFINITY;
            }
        }
    } else if (warp == LX_LOAD_WARP) {
        // =================================================================== loader
        uint32_t it = 0, qn = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
            int g, t0, t1, j0, j1;
            item_range(w, g, t0, t1, j0, j1);
            if (t1 <= t0) continue;
            if (qn > 0) {   // the MMAs of the previous group have finished reading q
                ok = mbar_wait(bar(LXB_QEMPTY), (qn - 1) & 1u, abort_flag, 13);
                if (!ok) break;
            }
            // q group: N rows of 128 B, one tile load (rows past s_q * H arrive as zeros); the head
            // weights go to shared memory with plain stores, every lane arrives once
            for (int c = lane; c < LX_QG * 64; c += 32) {
                const int qi = g * LX_QG + (c >> 6), h = c & 63;
                reinterpret_cast<float*>(sm + LX_W_OFF + (qn & 3u) * LX_W_BYTES)[c] = (qi < p.s_q && h < H) ? p.w[(size_t)qi * H + h] : 0.f;
            }
            if (lane == 0) {
                mbar_arrive_expect_tx(bar(LXB_QFULL), (uint32_t)N * LX_D);
                tma_load_2d(base + LX_Q_OFF, &qmap, 0, g * LX_QG * H, bar(LXB_QFULL));
            } else {
                mbar_arrive(bar(LXB_QFULL));
            }
            ++qn;
            for (int t = t0; t < t1 && ok; ++t, ++it) {
                const uint32_t st = it % LX_KSTAGE;
                if (it >= LX_KSTAGE) {
                    ok = mbar_wait_hot(bar(LXB_KEMPTY + st), ((it / LX_KSTAGE) - 1) & 1u, abort_flag, 14);
                    if (!ok) break;
                }
                if (lane == 0) {
                    mbar_arrive_expect_tx(bar(LXB_KFULL + st), LX_KT * LX_D);
                    tma_load_2d(base + LX_K_OFF + st * (LX_KT * 128), &kmap, 0, t * LX_KT, bar(LXB_KFULL + st));
                }
            }
        }
    } else if (warp == LX_MMA_WARP && lane == 0) {
        // =================================================================== MMA issue (one thread)
        constexpr uint32_t HI = desc_hi(1024, (uint32_t)SWIZZLE_128B);
        const uint32_t idesc = instr_desc(FMT_E4M3, FMT_E4M3, false, false, 128, (uint32_t)N);
        const uint32_t q_lo = desc_lo(base + LX_Q_OFF, 16);
        uint32_t it = 0, qn = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
            int g, t0, t1, j0, j1;
            item_range(w, g, t0, t1, j0, j1);
            if (t1 <= t0) continue;
            ok = mbar_wait_thread(bar(LXB_QFULL), qn & 1u, abort_flag, 15);
            if (!ok) break;
            ++qn;
            for (int t = t0; t < t1; ++t, ++it) {
                const uint32_t st = it % LX_KSTAGE, b = it & 1u;
                ok = mbar_wait_thread(bar(LXB_KFULL + st), (it / LX_KSTAGE) & 1u, abort_flag, 16);
                if (!ok) break;
                if (it >= 2) {
                    ok = mbar_wait_thread(bar(LXB_DEMPTY + b), ((it >> 1) - 1) & 1u, abort_flag, 17);
                    if (!ok) break;
                }
                tc_fence_after();
                const uint32_t k_lo = desc_lo(base + LX_K_OFF + st * (LX_KT * 128), 16);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_f8(tmem + 256 * b, make_desc(k_lo + ks * 2, HI), make_desc(q_lo + ks * 2, HI), idesc, ks != 0);
                tc_commit(bar(LXB_KEMPTY + st));
                tc_commit(bar(LXB_DFULL + b));
            }
            if (ok) tc_commit(bar(LXB_QEMPTY));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) {
        atomicCAS(p.status, 0, *abort_flag);
        atomicAdd(p.status + 1, 1);
        p.status[2] = blockIdx.x;
    }
    if (warp == LX_MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

}  // namespace

int launch_mqa_logits_tc(const uint8_t* q, const uint8_t* k, const float* k_scale, const float* weights,
                         const int32_t* ks, const int32_t* ke, float* logits, int s_q, int num_heads,
                         int s_k, int64_t logits_stride, int32_t* status, cudaStream_t stream) {
    if (s_q == 0 || s_k == 0) return 0;
    // the tensor-core kernel reads its accumulator 32 columns at a time: 32 or 64 heads
    if (num_heads % 32 != 0 || num_heads > 64)
        return launch_mqa_logits_scalar(q, k, k_scale, weights, ks, ke, logits, s_q, num_heads, s_k, logits_stride, stream);
    static bool attr_set[64] = {};
    static int sms[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(mqa_logits_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LX_SMEM);
        if (e != cudaSuccess) return set_error((int)e, "mqa_logits_tc_kernel: shared memory: %s", cudaGetErrorString(e));
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        attr_set[dev] = true;
    }
    // tensor maps of q ([s_q * heads rows] x 128 B, box of one query group) and k ([s_k rows] x 128 B, box of one key tile)
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (encode == nullptr) {
        cudaDriverEntryPointQueryResult qres;
        void* fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || fn == nullptr)
            return set_error(SMLA_E_DEVICE, "mqa_logits_tc_kernel: the driver has no cuTensorMapEncodeTiled");
        encode = (EncodeFn)fn;
    }
    CUtensorMap qmap, kmap;
    {
        const cuuint64_t qdims[2] = {(cuuint64_t)LX_D, (cuuint64_t)s_q * num_heads}, kdims[2] = {(cuuint64_t)LX_D, (cuuint64_t)s_k};
        const cuuint64_t strides[1] = {(cuuint64_t)LX_D};
        const cuuint32_t qbox[2] = {(cuuint32_t)LX_D, (cuuint32_t)(LX_QG * num_heads)}, kbox[2] = {(cuuint32_t)LX_D, (cuuint32_t)LX_KT};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r1 = encode(&qmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(q), qdims, strides, qbox, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        const CUresult r2 = encode(&kmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(k), kdims, strides, kbox, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r1 != CUDA_SUCCESS || r2 != CUDA_SUCCESS)
            return set_error(SMLA_E_DEVICE, "mqa_logits_tc_kernel: cuTensorMapEncodeTiled failed (%d, %d)", (int)r1, (int)r2);
    }
    const int groups = (s_q + LX_QG - 1) / LX_QG;
    const int nsm = sms[dev < 64 ? dev : 0];
    const int tiles = (s_k + LX_KT - 1) / LX_KT;
    // About eight work items per SM, so that the CTAs finish together: with few query groups the
    // key tiles are cut into runs (at least 8 tiles long, so that the q load and the pipeline fill
    // stay a small share).
    int chunks = groups >= 8 * nsm ? 1 : (8 * nsm + groups - 1) / groups;
    if (chunks > (tiles + 7) / 8) chunks = (tiles + 7) / 8;
    if (chunks < 1) chunks = 1;
    const int chunk_tiles = (tiles + chunks - 1) / chunks;
    const int items = groups * ((tiles + chunk_tiles - 1) / chunk_tiles);
    LogitsParams p{q, k, k_scale, weights, ks, ke, logits, status, s_q, num_heads, s_k, logits_stride, chunk_tiles};
    const int grid = items < nsm ? items : nsm;
    mqa_logits_tc_kernel<<<grid, LX_THREADS, LX_SMEM, stream>>>(p, qmap, kmap);
    return check_launch("mqa_logits_tc_kernel");
}

}  // namespace smla
