// Single-token causal attention over a K/V cache resident in HBM.
//
// Replaces, for one new token per sequence, the reference's split-heads / RoPE /
// per-head QKᵀ / mask / softmax / PV / merge chain (HeadOps.java:33-140,
// RotaryEmbedding.java:81-122).  Masked positions contribute exactly +0 to the
// reference's softmax, so attending over 0..pos only is the same function.
//
//  k_rope_append : rotate q and k at the sequence's position (interleaved pairs,
//                  x0·c − x1·s, x0·s + x1·c), write k and v into the cache.
//  k_attn_split  : flash-decoding.  grid (splits, heads, batch); a CTA streams its
//                  slice of the cache once, hd/16 lanes per position with 128-bit
//                  loads, online softmax in fp32, and leaves (acc[hd], m, l).
//  k_attn_combine: merges the split partials into the merged-heads row.
// HBM-bound: the algorithmic traffic is the K and V rows of 0..pos, read once.
#include "kernels.h"

namespace dj {

namespace {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__global__ void k_rope_append(float* __restrict__ qkv, int q_off, int k_off, int v_off, int ld,
                              float* __restrict__ kcache, float* __restrict__ vcache, int maxSeq,
                              const float* __restrict__ posbuf, const float* __restrict__ cosT, const float* __restrict__ sinT,
                              int H, int hd) {
    pdl_wait();
    pdl_launch_dependents();
    int h = blockIdx.x, b = blockIdx.y, i = threadIdx.x, half = hd >> 1;
    int pos = (int)posbuf[b];
    if (pos < 0 || pos >= maxSeq || i >= half) return;
    float c = cosT[(size_t)pos * half + i], s = sinT[(size_t)pos * half + i];
    float* row = qkv + (size_t)b * ld;
    float* q = row + q_off + h * hd;
    float q0 = q[2 * i], q1 = q[2 * i + 1];
    q[2 * i] = q0 * c - q1 * s;
    q[2 * i + 1] = q0 * s + q1 * c;
    const float* k = row + k_off + h * hd;
    float k0 = k[2 * i], k1 = k[2 * i + 1];
    size_t dst = (((size_t)b * H + h) * maxSeq + pos) * hd;
    kcache[dst + 2 * i] = k0 * c - k1 * s;
    kcache[dst + 2 * i + 1] = k0 * s + k1 * c;
    const float* v = row + v_off + h * hd;
    vcache[dst + 2 * i] = v[2 * i];
    vcache[dst + 2 * i + 1] = v[2 * i + 1];
}

constexpr int kAttnWarps = 4;

template <int LPP>   // lanes per position = hd / 16
__global__ void __launch_bounds__(kAttnWarps * 32) k_attn_split(
        const float* __restrict__ qkv, int q_off, int ld,
        const float* __restrict__ kcache, const float* __restrict__ vcache, int maxSeq,
        const float* __restrict__ posbuf, float* __restrict__ ws, int H, float scale) {
    constexpr int HD = LPP * 16;
    constexpr int PPW = 32 / LPP;                 // positions per warp iteration
    constexpr int G = kAttnWarps * PPW;           // position groups per CTA
    __shared__ float s_acc[G][HD];
    __shared__ float s_m[G], s_l[G];

    pdl_wait();
    pdl_launch_dependents();
    const int split = blockIdx.x, splits = gridDim.x, h = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = lane / LPP, gl = lane % LPP;
    int pos = (int)posbuf[b];
    if (pos >= maxSeq) pos = maxSeq - 1;
    const int seq = pos + 1;
    const int chunk = (seq + splits - 1) / splits;
    const int start = split * chunk;
    const int end = min(seq, start + chunk);

    float q[16];
    {
        const float4* qp = reinterpret_cast<const float4*>(qkv + (size_t)b * ld + q_off + h * HD + gl * 16);
#pragma unroll
        for (int j = 0; j < 4; j++) { float4 v = qp[j]; q[4 * j] = v.x; q[4 * j + 1] = v.y; q[4 * j + 2] = v.z; q[4 * j + 3] = v.w; }
    }
    const float* kbase = kcache + ((size_t)b * H + h) * maxSeq * HD + gl * 16;
    const float* vbase = vcache + ((size_t)b * H + h) * maxSeq * HD + gl * 16;

    float m = -INFINITY, l = 0.0f, acc[16];
#pragma unroll
    for (int j = 0; j < 16; j++) acc[j] = 0.0f;

    for (int base = start + warp * PPW; base < end; base += G) {
        int p = base + group;
        bool valid = p < end;
        float4 kf[4], vf[4];
        if (valid) {
            const float4* kp = reinterpret_cast<const float4*>(kbase + (size_t)p * HD);
            const float4* vp = reinterpret_cast<const float4*>(vbase + (size_t)p * HD);
#pragma unroll
            for (int j = 0; j < 4; j++) { kf[j] = __ldcs(kp + j); vf[j] = __ldcs(vp + j); }
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) { kf[j] = make_float4(0.f, 0.f, 0.f, 0.f); vf[j] = kf[j]; }
        }
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            dot = fmaf(q[4 * j], kf[j].x, dot); dot = fmaf(q[4 * j + 1], kf[j].y, dot);
            dot = fmaf(q[4 * j + 2], kf[j].z, dot); dot = fmaf(q[4 * j + 3], kf[j].w, dot);
        }
#pragma unroll
        for (int o = LPP / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (valid) {
            float s = dot * scale;
            float mn = fmaxf(m, s);
            float corr = expf(m - mn);
            float pe = expf(s - mn);
            l = l * corr + pe;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                acc[4 * j] = fmaf(pe, vf[j].x, acc[4 * j] * corr);
                acc[4 * j + 1] = fmaf(pe, vf[j].y, acc[4 * j + 1] * corr);
                acc[4 * j + 2] = fmaf(pe, vf[j].z, acc[4 * j + 2] * corr);
                acc[4 * j + 3] = fmaf(pe, vf[j].w, acc[4 * j + 3] * corr);
            }
            m = mn;
        }
    }
    const int g = warp * PPW + group;
#pragma unroll
    for (int j = 0; j < 16; j++) s_acc[g][gl * 16 + j] = acc[j];
    if (gl == 0) { s_m[g] = m; s_l[g] = l; }
    __syncthreads();
    float* out = ws + (((size_t)b * H + h) * splits + split) * (HD + 2);
    for (int j = threadIdx.x; j < HD; j += blockDim.x) {
        float M = -INFINITY;
#pragma unroll 4
        for (int gg = 0; gg < G; gg++) M = fmaxf(M, s_m[gg]);
        float a = 0.0f, L = 0.0f;
        if (M > -INFINITY) {
            for (int gg = 0; gg < G; gg++) {
                float e = expf(s_m[gg] - M);
                a = fmaf(s_acc[gg][j], e, a);
                L = fmaf(s_l[gg], e, L);
            }
        }
        out[j] = a;
        if (j == 0) { out[HD] = M; out[HD + 1] = L; }
    }
}

__global__ void k_attn_combine(const float* __restrict__ ws, float* __restrict__ out, int ldo, int H, int hd, int splits) {
    pdl_wait();
    pdl_launch_dependents();
    int h = blockIdx.x, b = blockIdx.y;
    const float* base = ws + ((size_t)b * H + h) * splits * (hd + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; s++) M = fmaxf(M, base[(size_t)s * (hd + 2) + hd]);
    for (int j = threadIdx.x; j < hd; j += blockDim.x) {
        float a = 0.0f, L = 0.0f;
        for (int s = 0; s < splits; s++) {
            const float* p = base + (size_t)s * (hd + 2);
            float e = expf(p[hd] - M);
            a = fmaf(p[j], e, a);
            L = fmaf(p[hd + 1], e, L);
        }
        out[(size_t)b * ldo + h * hd + j] = a / L;
    }
}

}  // namespace

int attn_decode_splits(int B, int H, int maxSeq) {
    int want = (4 * g_num_sms + B * H - 1) / (B * H);
    int cap = (maxSeq + 63) / 64;
    int s = want < cap ? want : cap;
    return s < 1 ? 1 : s;
}
size_t attn_decode_ws_floats(int B, int H, int hd, int splits) {
    return (size_t)B * H * splits * (hd + 2);
}

void launch_attn_decode(const AttnDecodeArgs& a, cudaStream_t s) {
    int lpp = a.hd / 16;
    if (a.hd % 16 != 0 || (lpp != 1 && lpp != 2 && lpp != 4 && lpp != 8 && lpp != 16 && lpp != 32))
        throw std::runtime_error("attention: head dim " + std::to_string(a.hd) + " is not one of 16,32,64,128,256,512");
    launch_k(k_rope_append, dim3(a.H, a.B), dim3(a.hd / 2 < 32 ? 32 : a.hd / 2), 0, s, true,
             a.qkv, a.q_off, a.k_off, a.v_off, a.ld, a.kcache, a.vcache, a.maxSeq, a.pos, a.cosT, a.sinT, a.H, a.hd);
    dim3 grid(a.splits, a.H, a.B), block(kAttnWarps * 32);
#define DJ_ATTN_CASE(L)                                                                                   \
    case L: launch_k(k_attn_split<L>, grid, block, 0, s, true, (const float*)a.qkv, a.q_off, a.ld,      \
                     (const float*)a.kcache, (const float*)a.vcache, a.maxSeq, a.pos, a.ws, a.H, a.scale); break;
    switch (lpp) {
        DJ_ATTN_CASE(1) DJ_ATTN_CASE(2) DJ_ATTN_CASE(4) DJ_ATTN_CASE(8) DJ_ATTN_CASE(16) DJ_ATTN_CASE(32)
    }
#undef DJ_ATTN_CASE
    launch_k(k_attn_combine, dim3(a.H, a.B), dim3(a.hd < 32 ? 32 : (a.hd > 256 ? 256 : a.hd)), 0, s, true,
             (const float*)a.ws, a.out, a.ldo, a.H, a.hd, a.splits);
}

}  // namespace dj
