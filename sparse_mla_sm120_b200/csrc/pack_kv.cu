// KV-cache writer: bf16 [rows, 576] -> packed 656-byte rows.
//
// Row format (specified by the reference's tests/test_decode.py:33-57): 512 e4m3 values in four
// tiles of 128, each tile with one fp32 scale 2^ceil(log2(max(amax,1e-4)/448)) (floored at
// 2^ceil(log2(1e-4))), then the 64 RoPE values verbatim as bf16.  HBM-bound streaming kernel:
// one warp per row, 16 values per lane, 32-byte loads and 16-byte stores.
#include "common.cuh"

namespace smla {

namespace {

__device__ __forceinline__ float pow2_ceil(float x) {   // smallest power of two >= x (x > 0, normal)
    uint32_t b = __float_as_uint(x);
    if (b & 0x007fffffu) b = (b + 0x00800000u) & 0x7f800000u;
    return __uint_as_float(b);
}

__global__ void __launch_bounds__(256) pack_kv_kernel(const __nv_bfloat16* __restrict__ kv,
                                                      uint8_t* __restrict__ packed, int64_t rows) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const __nv_bfloat16* src = kv + row * D_QK;
    uint8_t* dst = packed + row * ROW_BYTES;

    const uint4 a = __ldcs(reinterpret_cast<const uint4*>(src + lane * 16));
    const uint4 b = __ldcs(reinterpret_cast<const uint4*>(src + lane * 16 + 8));
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float v[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float scale = pow2_ceil(fmaxf(fmaxf(amax, 1e-4f) / 448.f, 1e-4f));
    const float inv = 1.f / scale;  // exact: power of two
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float x = fminf(fmaxf(v[4 * i + j] * inv, -448.f), 448.f);
            word |= (uint32_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3) << (8 * j);
        }
        o[i] = word;
    }
    *reinterpret_cast<uint4*>(dst + lane * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    if ((lane & 7) == 0) *reinterpret_cast<float*>(dst + SCALE_OFF + (lane >> 3) * 4) = scale;
    if (lane < 8) {
        const uint4 r = __ldcs(reinterpret_cast<const uint4*>(src + D_NOPE + lane * 8));
        *reinterpret_cast<uint4*>(dst + ROPE_OFF + lane * 16) = r;
    }
}

}  // namespace

int launch_pack_kv(const __nv_bfloat16* kv, uint8_t* packed, int64_t num_rows, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    const unsigned grid = (unsigned)((num_rows + 7) / 8);
    pack_kv_kernel<<<grid, 256, 0, stream>>>(kv, packed, num_rows);
    return check_launch("pack_kv_kernel");
}

}  // namespace smla
