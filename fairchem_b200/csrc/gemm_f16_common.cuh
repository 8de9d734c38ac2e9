// Pieces shared by the half-precision split tensor-core kernels (kind::f16 tcgen05 MMAs on 64-byte-swizzled
// K-major half tiles): tile shape, shared-memory and instruction descriptors, the MMA issue wrapper.
#pragma once

#include <cuda_fp16.h>

#include "gemm_common.cuh"

namespace fcb200 {
namespace f16 {

constexpr int BM = 128, BN = 128, BK = 32;
constexpr float kLoScale = 2048.0f;      // 2^11
constexpr float kHalfMax = 65504.0f;

// K-major, 64-byte swizzle: rows at a 64 B pitch, 8-row groups 512 B apart, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t smem_desc64(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;           // leading byte offset (unused for swizzled K-major), encoded 1
    d |= (uint64_t)(512 >> 4) << 32;  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;           // version
    d |= (uint64_t)4 << 61;           // SWIZZLE_64B
    return d;
}

// tcgen05 instruction descriptor: D=f32, A=B=f16 (format 0), both K-major, M=BM, N = BN or 2*BN
constexpr uint32_t instr_desc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24); }

template <int N>
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(instr_desc(N)), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}


}  // namespace f16
}  // namespace fcb200
