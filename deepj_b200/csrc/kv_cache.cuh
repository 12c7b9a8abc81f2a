// Element access of the K/V cache for the attention kernels.  The cache holds fp32 (the reference's precision) or,
// as an option, fp16: keys are rotated in fp32 and rounded to nearest-even when they are appended, values are rounded
// when they are appended, and every kernel widens what it reads back to fp32 — scores, softmax and the weighted
// sum are accumulated in fp32 either way.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace dj {

template <typename T> struct KvIo;

template <> struct KvIo<float> {
    // the value a later step will read back for x (fp32 cache: x itself)
    static __device__ __forceinline__ float stored(float x) { return x; }
    static __device__ __forceinline__ float4 ld4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
    static __device__ __forceinline__ void ld16_stream(const float* p, float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float4 a = __ldcs(reinterpret_cast<const float4*>(p) + j);
            v[4 * j] = a.x; v[4 * j + 1] = a.y; v[4 * j + 2] = a.z; v[4 * j + 3] = a.w;
        }
    }
    static __device__ __forceinline__ void ld16_shared(const float* p, float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float4 a = reinterpret_cast<const float4*>(p)[j];
            v[4 * j] = a.x; v[4 * j + 1] = a.y; v[4 * j + 2] = a.z; v[4 * j + 3] = a.w;
        }
    }
    static __device__ __forceinline__ void st16(float* p, const float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 4; j++) reinterpret_cast<float4*>(p)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    static __device__ __forceinline__ void st2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};

template <> struct KvIo<__half> {
    static __device__ __forceinline__ float stored(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ float4 ld4(const __half* p) {
        const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void ld16_stream(const __half* p, float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p) + j);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
                v[8 * j + 2 * q] = f.x; v[8 * j + 2 * q + 1] = f.y;
            }
        }
    }
    static __device__ __forceinline__ void ld16_shared(const __half* p, float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint4 u = reinterpret_cast<const uint4*>(p)[j];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
                v[8 * j + 2 * q] = f.x; v[8 * j + 2 * q + 1] = f.y;
            }
        }
    }
    static __device__ __forceinline__ void st16(__half* p, const float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const __half2 h = __floats2half2_rn(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
                w[q] = *reinterpret_cast<const uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(p)[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    static __device__ __forceinline__ void st2(__half* p, float a, float b) { *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b); }
};

}  // namespace dj
