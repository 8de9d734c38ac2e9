// C[M,N] = A[M,K] * W[N,K]^T (+ bias) in float32 on the sm_100a tensor cores (tcgen05, TF32 inputs,
// float32 accumulation in tensor memory).
//
// One CTA computes one 128 x 128 output tile.  Warp roles (192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor (no multicast) of a 128x32 A tile and a 128x32 W
//               tile per k-block into a 128-byte-swizzled shared-memory ring; also owns the TMEM allocation
//   warp 1      one elected thread issues tcgen05.mma (M=128, N=128, K=8) and commits to mbarriers
//   warps 2..5  PRECISION 3: split each landed tile into TF32 high and low parts in shared memory
//               (hi = rna(a), lo = rna(a - hi); same swizzled offsets, so the layout is untouched);
//               afterwards the epilogue: tcgen05.ld of the accumulator, + bias, float4 stores
// PRECISION 3 issues lo*hi + hi*lo + hi*hi per k-step, which restores float32-level accuracy; PRECISION 1
// feeds the float32 bits directly (the tensor core reads them as TF32).  The tensor core truncates
// (rounds toward zero) each time it adds into the float32 accumulator, a bias that grows with the
// number of MMAs into one accumulator; the two small correction products therefore go to a second
// TMEM accumulator (columns 128..255) and the epilogue adds the two, which cuts the truncating adds
// into the large accumulator by 3x.
//
// Every mbarrier wait is bounded (about one second of SM clock); on expiry the kernel raises a
// flag in shared memory, all roles leave their loops, TMEM is released and *status is set.
#include <cuda.h>

#include "common.cuh"

namespace fcb200 {

constexpr int BM = 128, BN = 128, BK = 32;
constexpr int kTileBytes = BM * BK * 4;  // 16 KiB, A and W tiles alike
constexpr int kGemmThreads = 192;
constexpr long long kWaitCycles = 1LL << 31;  // ~1.1 s at 1.9 GHz

template <int P> struct GemmCfg {
    static constexpr int kStages = P == 3 ? 3 : 6;
    static constexpr int kTilesPerStage = P == 3 ? 4 : 2;  // A, W (, A_lo, W_lo)
    static constexpr int kStageBytes = kTilesPerStage * kTileBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises *abort_flag) when the limit expires or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    const long long t0 = clock64();
    int polls = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++polls & 255) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitCycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// K-major, 128-byte swizzle: rows at a 128 B pitch, 8-row groups 1024 B apart, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;            // leading byte offset (unused for swizzled K-major), encoded 1
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;            // version
    d |= (uint64_t)2 << 61;            // SWIZZLE_128B
    return d;
}

// tcgen05 instruction descriptor: D=f32, A=B=tf32, both K-major, N=BN, M=BM
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(kInstrDesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ float to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}
__device__ __forceinline__ void split_tile(uint32_t hi_addr, uint32_t lo_addr, int tid, int nthreads) {
    for (int i = tid; i < kTileBytes / 16; i += nthreads) {
        float4 v;
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(hi_addr + i * 16));
        float4 h = make_float4(to_tf32(v.x), to_tf32(v.y), to_tf32(v.z), to_tf32(v.w));
        float4 l = make_float4(to_tf32(v.x - h.x), to_tf32(v.y - h.y), to_tf32(v.z - h.z), to_tf32(v.w - h.w));
        asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(hi_addr + i * 16), "f"(h.x), "f"(h.y), "f"(h.z), "f"(h.w) : "memory");
        asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(lo_addr + i * 16), "f"(l.x), "f"(l.y), "f"(l.z), "f"(l.w) : "memory");
    }
}

template <int P>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                     const float* __restrict__ bias, float* __restrict__ c, int64_t ldc, int64_t m_total, int n_total,
                     int k_total, int tiles_n, int32_t* __restrict__ status) {
    using Cfg = GemmCfg<P>;
    constexpr int S = Cfg::kStages;
    constexpr int kTmemCols = P == 3 ? 2 * BN : BN;  // main accumulator (+ correction accumulator)
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = base + S * Cfg::kStageBytes;
    // barrier block: full[S] | conv[S] | empty[S] | accum | tmem slot | abort flag
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto conv_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * S + s); };
    const uint32_t accum_bar = bar_base + 8u * (3 * S);
    uint8_t* const bar_generic = smem_raw + (bar_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_generic + 8 * (3 * S + 1));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (3 * S + 1) + 4);
    auto tile_addr = [&](int s, int which) { return base + s * Cfg::kStageBytes + which * kTileBytes; };  // 0 A, 1 W, 2 A_lo, 3 W_lo

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x % tiles_n;
    const int64_t tile_m = blockIdx.x / tiles_n;
    const int num_kb = (k_total + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(conv_bar(s), 128);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % S, it = kb / S;
                if (!mbar_wait(empty_bar(s), (it & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(full_bar(s), 2 * kTileBytes);
                tma_load_2d(tile_addr(s, 0), &map_a, kb * BK, (int)(tile_m * BM), full_bar(s));
                tma_load_2d(tile_addr(s, 1), &map_w, kb * BK, tile_n * BN, full_bar(s));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % S, it = kb / S;
                ok = mbar_wait(P == 3 ? conv_bar(s) : full_bar(s), it & 1, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = smem_desc(tile_addr(s, 0)), dw = smem_desc(tile_addr(s, 1));
                const uint64_t da_lo = P == 3 ? smem_desc(tile_addr(s, 2)) : 0, dw_lo = P == 3 ? smem_desc(tile_addr(s, 3)) : 0;
#pragma unroll
                for (int j = 0; j < BK / 8; ++j) {
                    const uint64_t adv = (uint64_t)(j * 2);  // 32 bytes per k-step, in 16-byte units
                    const uint32_t first = (kb > 0 || j > 0) ? 1u : 0u;
                    if (P == 3) {
                        umma_tf32(tmem_acc + BN, da_lo + adv, dw + adv, first);
                        umma_tf32(tmem_acc + BN, da + adv, dw_lo + adv, 1u);
                        umma_tf32(tmem_acc, da + adv, dw + adv, first);
                    } else {
                        umma_tf32(tmem_acc, da + adv, dw + adv, first);
                    }
                }
                umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
            }
            if (ok) umma_commit(accum_bar);
        }
    } else {
        const int tid = threadIdx.x - 64;  // 0..127
        bool ok = true;
        if (P == 3) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % S, it = kb / S;
                ok = mbar_wait(full_bar(s), it & 1, abort_flag);
                if (!ok) break;
                split_tile(tile_addr(s, 0), tile_addr(s, 2), tid, 128);
                split_tile(tile_addr(s, 1), tile_addr(s, 3), tid, 128);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(conv_bar(s));
            }
        }
        // epilogue: warp q = warp % 4 owns TMEM lanes [32q, 32q+32)
        if (ok) ok = mbar_wait(accum_bar, 0, abort_flag);
        ok = __all_sync(kFull, ok);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int q = warp & 3;
            const int64_t row = tile_m * BM + q * 32 + lane;
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc) {
                uint32_t r[32];
                const uint32_t taddr = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(cc * 32);
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
                if (P == 3) {
                    uint32_t t[32];
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(t[0]), "=r"(t[1]), "=r"(t[2]), "=r"(t[3]), "=r"(t[4]), "=r"(t[5]), "=r"(t[6]), "=r"(t[7]),
                          "=r"(t[8]), "=r"(t[9]), "=r"(t[10]), "=r"(t[11]), "=r"(t[12]), "=r"(t[13]), "=r"(t[14]), "=r"(t[15]),
                          "=r"(t[16]), "=r"(t[17]), "=r"(t[18]), "=r"(t[19]), "=r"(t[20]), "=r"(t[21]), "=r"(t[22]), "=r"(t[23]),
                          "=r"(t[24]), "=r"(t[25]), "=r"(t[26]), "=r"(t[27]), "=r"(t[28]), "=r"(t[29]), "=r"(t[30]), "=r"(t[31])
                        : "r"(taddr + (uint32_t)BN)
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(t[i]));
                } else {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                }
                if (row < m_total) {
                    float* crow = c + row * ldc;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const int col = tile_n * BN + cc * 32 + v * 4;
                        if (col < n_total) {
                            float4 o = make_float4(__uint_as_float(r[v * 4 + 0]), __uint_as_float(r[v * 4 + 1]),
                                                   __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
                            if (bias) o = add4(o, ld4(bias + col));
                            st4(crow + col, o);
                        }
                    }
                }
            }
        }
    }

    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, 1);
}

// ---- host side ------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

// 2-D float32 row-major [rows, cols] with row stride ld (floats); box = 32 columns x 128 rows, 128-byte swizzle
static int make_map(CUtensorMap* map, const float* ptr, int64_t rows, int64_t cols, int64_t ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return FCB200_EINVAL;
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FCB200_OK : FCB200_EINVAL;
}

template <int P>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw, const float* bias, float* c, int64_t ldc, int64_t m, int n,
                       int k, int32_t* status, cudaStream_t s) {
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_tf32_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<P>::kSmemBytes) != cudaSuccess)
            return static_cast<int>(cudaGetLastError());
        attr_set = true;
    }
    const int tiles_n = (n + BN - 1) / BN;
    const int64_t tiles_m = (m + BM - 1) / BM;
    if (tiles_m * tiles_n >= (1LL << 31)) return FCB200_ERANGE;
    gemm_tf32_kernel<P><<<(unsigned)(tiles_m * tiles_n), kGemmThreads, GemmCfg<P>::kSmemBytes, s>>>(ma, mw, bias, c, ldc, m, n, k,
                                                                                                 tiles_n, status);
    return launch_status();
}

}  // namespace fcb200

using namespace fcb200;

extern "C" int fcb200_gemm_tf32(const float* a, int64_t lda, const float* w, int64_t ldw, const float* bias, float* c, int64_t ldc,
                                int64_t m, int32_t n, int32_t k, int32_t precision, int32_t* status, void* stream) {
    if (!a || !w || !c || m < 0 || n <= 0 || k <= 0) return FCB200_EINVAL;
    if (precision != 1 && precision != 3) return FCB200_EINVAL;
    if (n % 4 || k % 4 || lda % 4 || ldw % 4 || ldc % 4 || lda < k || ldw < k || ldc < n) return FCB200_EINVAL;
    if (!aligned16(a) || !aligned16(w) || !aligned16(c) || (bias && !aligned16(bias))) return FCB200_EALIGN;
    if (m == 0) return FCB200_OK;
    CUtensorMap ma, mw;
    int rc = make_map(&ma, a, m, k, lda);
    if (rc) return rc;
    rc = make_map(&mw, w, n, k, ldw);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return precision == 3 ? launch_gemm<3>(ma, mw, bias, c, ldc, m, n, k, status, s)
                          : launch_gemm<1>(ma, mw, bias, c, ldc, m, n, k, status, s);
}
