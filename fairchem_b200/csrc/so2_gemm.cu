// C[M,N] = A[M,K] * W[N,K]^T (+ bias) in float32 on the sm_100a tensor cores (tcgen05, TF32 inputs,
// float32 accumulation in tensor memory).
//
// Persistent kernel: one CTA per SM walks over 128 x 128 output tiles (N fastest, so CTAs that run
// together share A tiles through L2).  Warp roles (320 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor (no multicast) of 128x32 tiles of A and of the
//               weights into a 128-byte-swizzled shared-memory ring; owns the TMEM allocation
//   warp 1      one elected thread issues tcgen05.mma (M=128, N=128, K=8) and commits to mbarriers
//   warps 2..5  PRECISION 3 only: write the TF32 low part of each landed A tile next to it
//   warps 6..9  epilogue: tcgen05.ld of a finished accumulator, + bias, then each warp stages its 32x32
//               sub-tiles in 128-byte-swizzled shared memory and writes them with TMA stores (coalesced,
//               clipped at the matrix edge); runs while the next tile's main loop fills the other
//               accumulator (TMEM is double buffered)
//
// PRECISION 1 feeds float32 bits to the tensor core, which reads them as TF32 (low 13 mantissa bits
// ignored).  PRECISION 3 restores float32-level accuracy with three products per k-step,
//     a_lo*w_hi + a_hi*w_lo + a_hi*w_hi,
// where w_hi/w_lo are the weights split once on the device (fcb200_split_tf32: round-to-nearest hi,
// remainder lo) and A is split on the fly: the tensor core's own view of the float32 word is a_hi, and
// a_lo = tf32(a - a_hi) is written to a second tile at the same swizzled offsets, so the UMMA layout
// is untouched and only the low part costs shared-memory writes.
// The tensor core truncates (rounds toward zero) every time it adds into the float32 accumulator, a
// bias that grows with the number of MMAs into one accumulator; the two small correction products
// therefore go to a second accumulator and the epilogue adds the two.
//
// Every mbarrier wait is bounded (about one second of SM clock); on expiry the kernel raises a flag in
// shared memory, all roles leave their loops, TMEM is released and *status is set.
#include "gemm_common.cuh"

namespace fcb200 {

constexpr int BM = 128, BN = 128, BK = 32;
constexpr int kTileBytes = BM * BK * 4;  // 16 KiB: A, A_lo, W_hi and W_lo tiles alike
constexpr int kGemmThreads = 320;

template <int P> struct GemmCfg {
    static constexpr int kStages = P == 3 ? 3 : 6;
    static constexpr int kTilesPerStage = P == 3 ? 4 : 2;  // A, W_hi (, A_lo, W_lo)
    static constexpr int kStageBytes = kTilesPerStage * kTileBytes;
    static constexpr int kAccCols = P == 3 ? 2 * BN : BN;  // main (+ correction) accumulator
    static constexpr int kTmemCols = 2 * kAccCols;         // double buffered
    static constexpr int kEpiBytes = 4 * 2 * 4096;         // 4 warps x 2 buffers x (32 rows x 128 B)
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*align*/ + 256 /*barriers*/;
};

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
__device__ __forceinline__ float to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}
// the value the tensor core sees when handed a float32 word as TF32: low 13 mantissa bits dropped
__device__ __forceinline__ float tf32_view(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }
__device__ __forceinline__ float lo_part(float v) { return to_tf32(v - tf32_view(v)); }

// a_lo tile from the landed A tile; 128 threads, 8 float4 each, all loads issued before the stores
__device__ __forceinline__ void write_low_tile(uint32_t a_addr, uint32_t lo_addr, int tid) {
    float4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t off = (uint32_t)(tid + i * 128) * 16u;
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v[i].x), "=f"(v[i].y), "=f"(v[i].z), "=f"(v[i].w) : "r"(a_addr + off));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t off = (uint32_t)(tid + i * 128) * 16u;
        asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(lo_addr + off), "f"(lo_part(v[i].x)), "f"(lo_part(v[i].y)),
                     "f"(lo_part(v[i].z)), "f"(lo_part(v[i].w))
                     : "memory");
    }
}

template <int P>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                     const __grid_constant__ CUtensorMap map_wlo, const __grid_constant__ CUtensorMap map_c,
                     const float* __restrict__ bias, int64_t m_total, int n_total, int k_total, int tiles_n, int64_t num_tiles,
                     int32_t* __restrict__ status) {
    using Cfg = GemmCfg<P>;
    constexpr int S = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi_base = base + S * Cfg::kStageBytes;  // 1024-byte aligned staging buffers of the epilogue warps
    const uint32_t bar_base = epi_base + Cfg::kEpiBytes;
    // barrier block: full[S] | conv[S] | empty[S] | tmem_full[2] | tmem_empty[2] | tmem slot | abort flag
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto conv_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * S + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (3 * S + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (3 * S + 2 + b); };
    uint8_t* const bar_generic = smem_raw + (bar_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_generic + 8 * (3 * S + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (3 * S + 4) + 4);
    // tile slots of a stage: 0 A, 1 W_hi, 2 A_lo, 3 W_lo
    auto tile_addr = [&](int s, int which) { return base + s * Cfg::kStageBytes + which * kTileBytes; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (k_total + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(conv_bar(s), 128);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), 128);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                     "r"((uint32_t)Cfg::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int64_t it = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int tile_n = (int)(tile % tiles_n);
                const int64_t tile_m = tile / tiles_n;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = (int)(it % S);
                    const uint32_t ph = (uint32_t)((it / S) & 1);
                    ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(full_bar(s), (P == 3 ? 3 : 2) * kTileBytes);
                    tma_load_2d(tile_addr(s, 0), &map_a, kb * BK, (int)(tile_m * BM), full_bar(s));
                    tma_load_2d(tile_addr(s, 1), &map_w, kb * BK, tile_n * BN, full_bar(s));
                    if (P == 3) tma_load_2d(tile_addr(s, 3), &map_wlo, kb * BK, tile_n * BN, full_bar(s));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int64_t it = 0, tcount = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
                const int buf = (int)(tcount & 1);
                const uint32_t use = (uint32_t)((tcount >> 1) & 1);
                ok = mbar_wait(tempty_bar(buf), use ^ 1u, abort_flag);  // epilogue has drained this accumulator
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + (uint32_t)(buf * Cfg::kAccCols);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = (int)(it % S);
                    const uint32_t ph = (uint32_t)((it / S) & 1);
                    ok = mbar_wait(P == 3 ? conv_bar(s) : full_bar(s), ph, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = smem_desc(tile_addr(s, 0)), dw = smem_desc(tile_addr(s, 1));
                    const uint64_t da_lo = P == 3 ? smem_desc(tile_addr(s, 2)) : 0, dw_lo = P == 3 ? smem_desc(tile_addr(s, 3)) : 0;
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        const uint64_t adv = (uint64_t)(j * 2);  // 32 bytes per k-step, in 16-byte units
                        const uint32_t first = (kb > 0 || j > 0) ? 1u : 0u;
                        if (P == 3) {
                            umma_tf32(acc + BN, da_lo + adv, dw + adv, first);
                            umma_tf32(acc + BN, da + adv, dw_lo + adv, 1u);
                        }
                        umma_tf32(acc, da + adv, dw + adv, first);
                    }
                    umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(tfull_bar(buf));
            }
        }
    } else if (warp < 6) {
        if (P == 3) {
            const int tid = threadIdx.x - 64;  // 0..127
            int64_t it = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = (int)(it % S);
                    const uint32_t ph = (uint32_t)((it / S) & 1);
                    ok = mbar_wait(full_bar(s), ph, abort_flag);
                    if (!ok) break;
                    write_low_tile(tile_addr(s, 0), tile_addr(s, 2), tid);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_arrive(conv_bar(s));
                }
            }
        }
    } else {
        // epilogue: warp q = warp % 4 owns TMEM lanes [32q, 32q+32)
        const int q = warp & 3;
        int64_t tcount = 0;
        int chunk = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
            const int tile_n = (int)(tile % tiles_n);
            const int64_t tile_m = tile / tiles_n;
            const int buf = (int)(tcount & 1);
            const uint32_t use = (uint32_t)((tcount >> 1) & 1);
            ok = mbar_wait(tfull_bar(buf), use, abort_flag);
            ok = __all_sync(kFull, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t row0 = tile_m * BM + q * 32;
            const uint32_t acc = tmem_base + (uint32_t)(buf * Cfg::kAccCols) + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc, ++chunk) {
                const int col0 = tile_n * BN + cc * 32;
                uint32_t r[32];
                FCB_TMEM_LD32(r, acc + (uint32_t)(cc * 32));
                if (P == 3) {
                    uint32_t t[32];
                    FCB_TMEM_LD32(t, acc + (uint32_t)(BN + cc * 32));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(t[i]));
                } else {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                }
                if (row0 >= m_total || col0 >= n_total) continue;  // sub-tile entirely outside the matrix
                // the store issued two chunks ago read this staging buffer; let it finish before overwriting
                const uint32_t stage = epi_base + (uint32_t)((q * 2 + (chunk & 1)) * 4096);
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                __syncwarp();
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    float4 o = make_float4(__uint_as_float(r[v * 4 + 0]), __uint_as_float(r[v * 4 + 1]), __uint_as_float(r[v * 4 + 2]),
                                           __uint_as_float(r[v * 4 + 3]));
                    if (bias && col0 + v * 4 < n_total) o = add4(o, ld4(bias + col0 + v * 4));
                    // row `lane` of the 32x32 sub-tile, 16-byte chunk v, 128-byte swizzle: chunk index XOR (row % 8)
                    const uint32_t dst = stage + (uint32_t)(lane * 128 + ((v ^ (lane & 7)) * 16));
                    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&map_c, stage, col0, (int)row0);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(tempty_bar(buf));  // 128 arrivals hand the accumulator back to the MMA thread
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all stores of this warp have landed
    }

    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, 1);
}

__global__ void split_tf32_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = w[i];
    const float h = to_tf32(v);
    hi[i] = h;
    lo[i] = to_tf32(v - h);
}

// ---- host side ------------------------------------------------------------------------------

// 2-D float32 row-major [rows, cols] with row stride ld (floats); box = 32 columns x box_rows rows, 128-byte swizzle
static int make_map(CUtensorMap* map, const float* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows = BM) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return FCB200_EINVAL;
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FCB200_OK : FCB200_EINVAL;
}

template <int P>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mwlo, const CUtensorMap& mc,
                       const float* bias, int64_t m, int n, int k, int32_t* status, cudaStream_t s) {
    static bool attr_done[64] = {};
    if (const int rc = ensure_dynamic_smem(gemm_tf32_kernel<P>, GemmCfg<P>::kSmemBytes, attr_done)) return rc;
    const int tiles_n = (n + BN - 1) / BN;
    const int64_t tiles_m = (m + BM - 1) / BM;
    const int64_t num_tiles = tiles_m * tiles_n;
    const int grid = (int)(num_tiles < sm_count() ? num_tiles : sm_count());
    gemm_tf32_kernel<P><<<grid, kGemmThreads, GemmCfg<P>::kSmemBytes, s>>>(ma, mw, mwlo, mc, bias, m, n, k, tiles_n, num_tiles, status);
    return launch_status();
}

}  // namespace fcb200

using namespace fcb200;

extern "C" int fcb200_split_tf32(const float* w, float* w_hi, float* w_lo, int64_t count, void* stream) {
    if (!w || !w_hi || !w_lo || count < 0) return FCB200_EINVAL;
    if (count == 0) return FCB200_OK;
    split_tf32_kernel<<<(unsigned)((count + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(w, w_hi, w_lo, count);
    return launch_status();
}

extern "C" int fcb200_gemm_tf32(const float* a, int64_t lda, const float* w, const float* w_lo, int64_t ldw, const float* bias,
                                float* c, int64_t ldc, int64_t m, int32_t n, int32_t k, int32_t precision, int32_t* status,
                                void* stream) {
    if (!a || !w || !c || m < 0 || n <= 0 || k <= 0) return FCB200_EINVAL;
    if (precision != 1 && precision != 3) return FCB200_EINVAL;
    if (precision == 3 && !w_lo) return FCB200_EINVAL;
    if (n % 4 || k % 4 || lda % 4 || ldw % 4 || ldc % 4 || lda < k || ldw < k || ldc < n) return FCB200_EINVAL;
    if (!aligned16(a) || !aligned16(w) || !aligned16(c) || (bias && !aligned16(bias)) || (w_lo && !aligned16(w_lo)))
        return FCB200_EALIGN;
    if (m == 0) return FCB200_OK;
    CUtensorMap ma, mw, mwlo, mc;
    int rc = make_map(&ma, a, m, k, lda);
    if (rc) return rc;
    rc = make_map(&mw, w, n, k, ldw);
    if (rc) return rc;
    rc = make_map(&mwlo, precision == 3 ? w_lo : w, n, k, ldw);
    if (rc) return rc;
    rc = make_map(&mc, c, m, n, ldc, 32);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return precision == 3 ? launch_gemm<3>(ma, mw, mwlo, mc, bias, m, n, k, status, s)
                          : launch_gemm<1>(ma, mw, mwlo, mc, bias, m, n, k, status, s);
}
