// Device helpers shared by the Q8 integer-tensor-pipe kernels: asynchronous copies, the
// programmatic-dependent-launch fences, the int8 MMA, and the conversion of fp32 activations
// into three signed base-256 digit columns with a power-of-two scale per 32-k block.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace dj {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void mma_s8_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// GELU as the reference's CPU backend computes it (tensor/cpu/CpuBackend.java:338-343): the tanh
// form in fp32 with the square root and tanh evaluated in double and rounded.
__device__ __forceinline__ float gelu_ref(float x) {
    const float c = (float)sqrt((double)(2.0f / 3.14159274101257324f));
    const float x3 = x * x * x;
    const float t = c * (x + 0.044715f * x3);
    return 0.5f * x * (1.0f + (float)tanh((double)t));
}

__device__ __forceinline__ void load16(const float* src, bool vec, float (&v)[16]) {
    if (vec) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float4 v4 = reinterpret_cast<const float4*>(src)[j];
            v[4 * j] = v4.x; v[4 * j + 1] = v4.y; v[4 * j + 2] = v4.z; v[4 * j + 3] = v4.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] = src[j];
    }
}

// Half a 32-k block (16 values, the lane pair shares the block) → three int8 digit columns and the
// block's power-of-two scale.  q = rne(v·2^23/s) with |q| ≤ 2^22; adding 128 at every digit turns
// the balanced digits e2,e1,e0 ∈ [−128,127] into the plain bytes of q + 0x808080, and flipping each
// top bit turns them back: one add per value, a 4×4 byte transpose per four values.
__device__ __forceinline__ void digits16(const float (&v)[16], bool on, int8_t* dcol, int ldxs, int hb, float* xscRow) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));      // the other half of the 32-k block
    // s = 2^(exponent(amax)+2): |v|/s < 1/2, so the 23-bit fixed-point value fits three signed digits
    int sbits = 0x3f800000;
    if (amax > 0.0f && amax < 1e36f) sbits = (__float_as_int(amax) & 0x7f800000) + 0x01000000;
    const float mul = __int_as_float(0x7f000000 - sbits) * 8388608.0f;     // 2^23 / s, exact
    uint32_t w2[4], w1[4], w0[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t u[4];
#pragma unroll
        for (int i = 0; i < 4; i++) u[i] = (uint32_t)(__float2int_rn(v[4 * j + i] * mul) + 0x808080);
        const uint32_t t0 = __byte_perm(u[0], u[1], 0x5140), t1 = __byte_perm(u[2], u[3], 0x5140);
        const uint32_t t2 = __byte_perm(u[0], u[1], 0x7362), t3 = __byte_perm(u[2], u[3], 0x7362);
        w0[j] = __byte_perm(t0, t1, 0x5410) ^ 0x80808080u;
        w1[j] = __byte_perm(t0, t1, 0x7632) ^ 0x80808080u;
        w2[j] = __byte_perm(t2, t3, 0x5410) ^ 0x80808080u;
    }
    if (on) {
        *reinterpret_cast<uint4*>(dcol + hb * 16) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
        *reinterpret_cast<uint4*>(dcol + ldxs + hb * 16) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
        *reinterpret_cast<uint4*>(dcol + 2 * ldxs + hb * 16) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
        if ((hb & 1) == 0) xscRow[hb >> 1] = __int_as_float(sbits) * (1.0f / 8388608.0f);
    }
}

}  // namespace dj
