// Shared helpers for the fairchem_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fairchem_b200.h"

namespace fcb200 {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

// ---- lmax = mmax = 2 coefficient bookkeeping -------------------------------------------------
// M-major row -> L-major index: m=0:(l0,l1,l2) | m=+1:(l1,l2) | m=-1:(l1,l2) | m=+2:(l2) | m=-2:(l2)
__host__ __device__ constexpr int m2l(int m) {
    constexpr int t[9] = {0, 2, 6, 3, 7, 1, 5, 8, 4};
    return t[m];
}
__host__ __device__ constexpr int l2m(int L) {
    constexpr int t[9] = {0, 5, 1, 3, 8, 6, 2, 4, 7};
    return t[L];
}
__host__ __device__ constexpr int deg_of(int L) { return L == 0 ? 0 : (L < 4 ? 1 : 2); }
// offset of block l inside the compact 35-entry Wigner
__host__ __device__ constexpr int woff(int l) { return l == 0 ? 0 : (l == 1 ? 1 : 10); }
// compact index of entry (row L, col K) of the block-diagonal matrix; both in the same l block
__host__ __device__ constexpr int wix(int L, int K) {
    return woff(deg_of(L)) + (L - deg_of(L) * deg_of(L)) * (2 * deg_of(L) + 1) + (K - deg_of(L) * deg_of(L));
}
// radial slot (in units of 2C) that multiplies M-major row m: [m0: 0,1,2 | m1: 3,4 (shared by +-1) | m2: 5]
__host__ __device__ constexpr int radslot(int m) {
    constexpr int t[9] = {0, 1, 2, 3, 4, 3, 4, 5, 5};
    return t[m];
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 f4zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ float4 fma4(float a, float4 x, float4 acc) {
    acc.x = fmaf(a, x.x, acc.x);
    acc.y = fmaf(a, x.y, acc.y);
    acc.z = fmaf(a, x.z, acc.z);
    acc.w = fmaf(a, x.w, acc.w);
    return acc;
}
__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 sub4(float4 a, float4 b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }
__device__ __forceinline__ float4 scale4(float a, float4 b) { return make_float4(a * b.x, a * b.y, a * b.z, a * b.w); }
__device__ __forceinline__ float dot4(float4 a, float4 b) { return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w))); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

// Sum each of 35 per-lane partial values over the warp.  The first 32 go through a transposed butterfly
// (at offset h every lane hands over the half it will not own: 16+8+4+2+1 = 31 shuffles, after which
// lane l holds the total of value l); the last 3 use plain warp sums.  46 shuffles instead of 175.
__device__ __forceinline__ void warp_reduce_wig(float (&v)[FCB200_WIG], int lane, float& first32, float& last3) {
#pragma unroll
    for (int h = 16; h >= 1; h >>= 1) {
        const bool upper = (lane & h) != 0;
#pragma unroll
        for (int i = 0; i < h; ++i) {
            const float a = v[i], b = v[i + h];
            const float send = upper ? a : b;
            const float keep = upper ? b : a;
            v[i] = keep + __shfl_xor_sync(kFull, send, h);
        }
    }
    first32 = v[0];
    last3 = 0.f;
#pragma unroll
    for (int j = 0; j < FCB200_WIG - 32; ++j) {
        const float t = warp_sum(v[32 + j]);
        if (lane == j) last3 = t;
    }
}

// Sum each of N per-lane partial values over the warp and store total i at out[i].  Values are taken in groups
// of 32 through the transposed butterfly of warp_reduce_wig (31 shuffles per group, a short group is padded with
// zeros), after which lane l holds the total of value 32 g + l and stores it.
template <int N>
__device__ __forceinline__ void warp_reduce_store(const float (&v)[N], int lane, float* __restrict__ out, float scale = 1.0f) {
#pragma unroll
    for (int g = 0; g < (N + 31) / 32; ++g) {
        float t[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) t[i] = (g * 32 + i < N) ? v[g * 32 + i] : 0.f;
#pragma unroll
        for (int h = 16; h >= 1; h >>= 1) {
            const bool upper = (lane & h) != 0;
#pragma unroll
            for (int i = 0; i < h; ++i) {
                const float a = t[i], b = t[i + h];
                const float send = upper ? a : b;
                const float keep = upper ? b : a;
                t[i] = keep + __shfl_xor_sync(kFull, send, h);
            }
        }
        if (g * 32 + lane < N) out[g * 32 + lane] = t[0] * scale;
    }
}

// Load the 35 compact Wigner entries of one edge into registers, identical in every lane.
__device__ __forceinline__ void load_wig(const float* __restrict__ wig, int64_t e, int lane, float (&w)[FCB200_WIG]) {
    const float* p = wig + e * FCB200_WIG;
    float a = p[lane];
    float b = lane < FCB200_WIG - 32 ? p[32 + lane] : 0.f;
#pragma unroll
    for (int i = 0; i < FCB200_WIG; ++i) w[i] = i < 32 ? __shfl_sync(kFull, a, i) : __shfl_sync(kFull, b, i - 32);
}

// ---- output policies of the kernels that feed the dense contractions ---------------------------
// OutF32 stores float32.  OutSplit stores the half-precision split the tensor cores consume directly:
// hi = half(v * s), lo = half((v * s - hi) * 2^11), in two planes of the same shape (same bytes as float32).
struct OutF32 {
    float* p;
    __device__ __forceinline__ void load_scale(const float*) {}
    __device__ __forceinline__ void st(int64_t off, float4 v) const { st4(p + off, v); }
};
struct OutSplit {
    __half* hi;
    __half* lo;
    float s;
    __device__ __forceinline__ void load_scale(const float* sp) { s = sp ? *sp : 1.0f; }
    __device__ __forceinline__ void st(int64_t off, float4 v) const {
        v = scale4(s, v);
        const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
        const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
        const __half2 l0 = __floats2half2_rn((v.x - f0.x) * 2048.0f, (v.y - f0.y) * 2048.0f);
        const __half2 l1 = __floats2half2_rn((v.z - f1.x) * 2048.0f, (v.w - f1.y) * 2048.0f);
        uint2 ph, pl;
        ph.x = *reinterpret_cast<const uint32_t*>(&h0);
        ph.y = *reinterpret_cast<const uint32_t*>(&h1);
        pl.x = *reinterpret_cast<const uint32_t*>(&l0);
        pl.y = *reinterpret_cast<const uint32_t*>(&l1);
        *reinterpret_cast<uint2*>(hi + off) = ph;
        *reinterpret_cast<uint2*>(lo + off) = pl;
    }
};
inline bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int launch_status() {
    cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? FCB200_OK : static_cast<int>(err);
}

// number of blocks for a warp-per-item kernel with `warps_per_block`, capped to a few waves of 148 SMs
inline int warp_grid(int64_t items, int warps_per_block, int max_blocks = 148 * 16) {
    int64_t b = (items + warps_per_block - 1) / warps_per_block;
    if (b < 1) b = 1;
    if (b > max_blocks) b = max_blocks;
    return static_cast<int>(b);
}

}  // namespace fcb200
