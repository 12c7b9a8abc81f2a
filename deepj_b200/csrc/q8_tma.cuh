// Device helpers of the Q8 kernels that stream weights through the tensor-memory accelerator (q8_gemv_tma.cu,
// q8_batch_tma.cu): mbarriers, tiled bulk copies, ldmatrix, and the host-side tensor maps over a Q8 weight.
#pragma once
#include <cuda.h>

#include "kernels.h"
#include "q8_common.cuh"

namespace dj {

constexpr int kTmaItemK = 128;              // reduction length of one ring item: 16 rows × 128 code bytes + 16 × 4 scales

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// one box of a two-dimensional tensor map → shared memory; x counts elements of the inner dimension, y rows
__device__ __forceinline__ void tma_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
// exact for |v| < 2^22: the integer lands in the mantissa of 1.5 · 2^23
__device__ __forceinline__ float int_to_float_exact(int v) { return __int_as_float(v + 0x4B400000) - 12582912.0f; }

// Tensor maps over one Q8 weight: codes [N][Kp] bytes in boxes of 8 rows × 128 bytes (128-byte swizzle) and scales
// [N][nb] floats in boxes of 8 rows × 4.  False when the driver's encoder is missing or the layout does not qualify
// (16-byte aligned bases and row pitches).
bool q8_encode_weight_maps(const Q8View& w, CUtensorMap* codes, CUtensorMap* scales);

}  // namespace dj
