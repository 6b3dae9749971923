// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier with bounded
// waits, cp.async, tcgen05 (TMEM allocation, MMA, commit, ld/st, fences) and the shared-memory
// matrix / instruction descriptors of tcgen05.mma.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace smla {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One poll; the hardware may suspend the thread for up to `hint_ns` while the phase is incomplete.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    (void)hint_ns;     // passing the hint as the instruction's time limit made waits on the critical path wake later
    return ok != 0;
}
// One non-blocking poll.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Warp-wide wait for the phase with the given parity.  Lane 0 polls (32 lanes polling one
// mbarrier only add shared-memory traffic), the warp reconverges on the result.  The wait gives
// up after a bounded number of polls (about half a second) or as soon as another thread of the
// CTA has given up (*abort != 0); it then returns false and records `code` in *abort so that the
// kernel can report where it stopped.  Must be called by all 32 lanes.
constexpr uint32_t WAIT_POLLS = 1u << 22;
constexpr uint32_t WAIT_HINT_NS = 2000;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort, int code) {
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) {
        ok = 0;
        for (uint32_t i = 0; i < WAIT_POLLS; ++i) {
            if (mbar_try_wait(bar, parity, WAIT_HINT_NS)) { ok = 1; break; }
            __nanosleep(32);   // a spinning poller would take issue slots from the working warps of its scheduler
            if ((i & 255u) == 255u && *abort != 0) break;
        }
        if (!ok) atomicCAS(const_cast<int*>(abort), 0, code);
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
}

// Variant for waits on the critical path: every lane blocks in mbarrier.try_wait itself (the
// hardware parks the thread until the phase completes or its own time limit passes), so the warp
// resumes as soon as the barrier flips instead of after a sleep interval.  Same bounds and
// give-up protocol as mbar_wait.
__device__ __forceinline__ bool mbar_wait_hot(uint32_t bar, uint32_t parity, volatile int* abort, int code) {
    uint32_t ok = 0;
    for (uint32_t i = 0; i < WAIT_POLLS; ++i) {
        if (mbar_try_wait(bar, parity, WAIT_HINT_NS)) { ok = 1; break; }
        if ((i & 255u) == 255u && *abort != 0) break;
    }
    if (!ok) atomicCAS(const_cast<int*>(abort), 0, code);
    return __all_sync(0xffffffffu, ok != 0);
}

// ------------------------------------------------------------------ thread-block cluster
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// Cluster-wide barrier; executed by every thread of every CTA of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Packed fp32 pairs (sm_100): one FMA instruction for two independent fp32 lanes, each rounded as fmaf does.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void fma_f32x2(uint64_t& acc, uint64_t a, uint64_t b) {   // acc += a * b, per lane
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

// 256-bit global store (sm_100): one full 32-byte sector per lane; p must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&v)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
                 "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}

__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Arrive on a barrier of another CTA of the cluster; releases this thread's earlier writes to it.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// Arrive on a barrier given by its shared::cluster address (this CTA's or, through mapa_shared, another
// CTA's) with the default CTA-scope release.  For signals that only say "my part is ready" about data
// that stays inside this SM (shared-memory operands of a pair MMA, tensor memory): a cluster-scope
// release makes every such arrive wait for a memory barrier (about a thousand cycles under load).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// Arrive on a barrier of another CTA and add `bytes` to its pending transaction count.
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t remote_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(remote_bar), "r"(bytes) : "memory");
}
// Bulk copy from this CTA's shared memory into another CTA's (both 16-byte aligned, size a
// multiple of 16); the destination CTA's barrier receives the byte count when the data has landed.
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t remote_dst, uint32_t local_src, uint32_t bytes, uint32_t remote_bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(remote_dst), "r"(local_src), "r"(bytes), "r"(remote_bar) : "memory");
}
// Untiled bulk copy global -> this CTA's shared memory (both 16-byte aligned, size a multiple of 16);
// the barrier receives the byte count when the data has landed.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, unsigned long long src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// One poll with cluster-scope acquire: for barriers that another CTA arrives on after writing here.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// mbar_wait_hot with cluster-scope acquire.
__device__ __forceinline__ bool mbar_wait_hot_cluster(uint32_t bar, uint32_t parity, volatile int* abort, int code) {
    uint32_t ok = 0;
    for (uint32_t i = 0; i < WAIT_POLLS; ++i) {
        if (mbar_try_wait_cluster(bar, parity)) { ok = 1; break; }
        if ((i & 255u) == 255u && *abort != 0) break;
    }
    if (!ok) atomicCAS(const_cast<int*>(abort), 0, code);
    return __all_sync(0xffffffffu, ok != 0);
}
__device__ __forceinline__ bool mbar_wait_thread_cluster(uint32_t bar, uint32_t parity, volatile int* abort, int code) {
    for (uint32_t i = 0; i < WAIT_POLLS; ++i) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort != 0) return false;
    }
    atomicCAS(const_cast<int*>(abort), 0, code);
    return false;
}

// Single-thread variant of mbar_wait (same bounds and give-up protocol), for a role that is run
// by one lane only.
__device__ __forceinline__ bool mbar_wait_thread(uint32_t bar, uint32_t parity, volatile int* abort, int code) {
    for (uint32_t i = 0; i < WAIT_POLLS; ++i) {
        if (mbar_try_wait(bar, parity, WAIT_HINT_NS)) return true;
        if ((i & 255u) == 255u && *abort != 0) return false;
    }
    atomicCAS(const_cast<int*>(abort), 0, code);
    return false;
}

// ------------------------------------------------------------------ cp.async (16-byte, L2 only)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Copies src_bytes (0 or 16) bytes and zero-fills the rest of the 16-byte destination.
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// ------------------------------------------------------------------ TMA (tiled bulk tensor copy)
// Adds `bytes` to the barrier's pending transaction count and arrives once.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Loads the box of the 2-D tensor map at element coordinates (x, y) into shared memory; the
// barrier receives the byte count when the data has landed.  x * element size must be a
// multiple of 16 bytes; rows outside the tensor arrive as zeros.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tensor_map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tensor_map), "r"(x), "r"(y), "r"(bar) : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Arrives on the mbarrier (without adding to its pending count) once every cp.async issued so
// far by this thread has landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// Makes generic-proxy writes to shared memory visible to the async proxy (tcgen05.mma operands).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------ tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Arrives once on the mbarrier when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp receives columns [c, c+32) of lane
// (32 * (warp % 4) + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// 16 lanes x 32 columns in the 16x256b fragment shape: for every block i of 8 columns, thread t
// supplies columns 2*(t%4), 2*(t%4)+1 of lane t/4 (registers 4i, 4i+1) and of lane t/4 + 8
// (registers 4i+2, 4i+3).  The lane field of taddr selects the first of the 16 lanes.
__device__ __forceinline__ void tmem_st_16x256b_x4(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// 32 lanes x 8 columns: thread i of the warp writes 8 consecutive columns of its lane.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

// Register reallocation between warpgroups (all four warps of a warpgroup execute it together).
template <int N> __device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// Named barrier among `threads` threads (ids 1..15; id 0 is __syncthreads).
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Named barrier that also ORs a predicate over its participants: every thread receives the same
// answer, so warps that must leave a loop together can decide on it.
__device__ __forceinline__ bool named_bar_or(uint32_t id, uint32_t threads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"(id), "r"(threads), "r"((uint32_t)pred) : "memory");
    return r != 0;
}

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor of tcgen05.mma: start address, leading / stride byte offsets
// (all in 16-byte units), descriptor version 1 (bits 46-47) and the swizzle mode (bits 61-63).
enum : uint64_t { SWIZZLE_NONE = 0, SWIZZLE_128B = 2, SWIZZLE_64B = 4, SWIZZLE_32B = 6 };
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t swizzle) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (swizzle << 61);
}

// Instruction descriptor: fp32 accumulator, operand formats, majorness, N >> 3, M >> 4.
constexpr uint32_t FMT_F16 = 0, FMT_BF16 = 1, FMT_E4M3 = 0, FMT_E5M2 = 1;
__host__ __device__ constexpr uint32_t instr_desc(uint32_t a_fmt, uint32_t b_fmt, bool a_mn_major, bool b_mn_major,
                                                   uint32_t m, uint32_t n) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) |
           ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}

// Same with the A operand read from tensor memory (lane = row, K packed along the columns).
__device__ __forceinline__ void mma_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}

// ------------------------------------------------------------------ CTA-pair forms (cta_group::2)
// Tensor-memory allocation for a pair of CTAs (ranks 2k, 2k+1 of a cluster): executed by one warp
// with the same index in both CTAs, each passing the same shared-memory offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// Arrives once on the barrier (a shared::cluster address: this CTA's or, through mapa_shared, the
// partner's) when every pair MMA issued so far by this thread has completed in both CTAs.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D (+)= A * B over the pair, M = 128: each CTA supplies 64 rows of A and N/2 rows of B at the same
// shared-memory offsets and receives its 64 rows of D as 128 lanes x N/2 columns (lanes 0-63 hold
// columns [0, N/2) of the rows, lanes 64-127 columns [N/2, N)).  Issued by one thread of the even CTA.
__device__ __forceinline__ void mma_pair_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
// The same with A read from tensor memory: lane = row, K packed along the columns; the 64 rows of a
// CTA must be present twice, in lanes 0-63 and again in lanes 64-127.
__device__ __forceinline__ void mma_pair_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
__device__ __forceinline__ void mma_pair_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}

// Descriptor halves for operands whose address changes while everything else stays fixed:
// desc = (hi << 32) | (lo(addr) ), lo(addr + off) = lo(addr) + (off >> 4).
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
    return ((addr >> 4) & 0x3fffu) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
__host__ __device__ constexpr uint32_t desc_hi(uint32_t sbo_bytes, uint32_t swizzle) {
    return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (swizzle << 29);
}
__device__ __forceinline__ uint64_t make_desc(uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; }

}  // namespace ptx
}  // namespace smla
