// C[M,N] = A[M,K] * W[N,K]^T (+ bias) in float32 on the sm_100a tensor cores with half-precision split
// operands: float32-level accuracy from three kind::f16 MMAs per product, which issue at twice the TF32
// rate and read half the shared-memory bytes per operand.
//
// Every float32 value v (times a power-of-two scale s that centres the tensor in the half range) is
// represented as hi + lo * 2^-11 with hi = half(v s) and lo = half((v s - hi) * 2^11): 22 significant bits.
//     C = [ sum hi_a hi_w  +  2^-11 * sum (lo_a hi_w + hi_a lo_w) ] / (s_a s_w)
// The weights are split once on the device (fcb200_split_f16).  A arrives as float32 through TMA and is
// split by four warps into two half tiles; because a 128-byte-swizzled float32 row of 32 values and a
// 64-byte-swizzled half row of 32 values permute their 32-byte / 16-byte units by the same XOR of the row
// index, a thread converts one 32-byte unit in place: same unit index, half the pitch.
//
// Structure is that of the TF32 kernel (persistent CTAs, 128 x 128 tiles, N fastest; warp 0 TMA producer
// and TMEM owner, warp 1 MMA issue, two groups of four warps split A tiles in turn, four epilogue warps with TMA stores; main and
// correction accumulators, both double buffered = 512 TMEM columns).  Every mbarrier wait is bounded; on
// expiry the roles leave their loops, TMEM is released and *status is set to 1.  *status is set to 2 when
// a scaled A value leaves the finite half range (the result is then invalid).
#include <cuda_fp16.h>

#include "gemm_f16_common.cuh"

namespace fcb200 {

namespace f16 {

constexpr int kA32Bytes = BM * BK * 4;   // 16 KiB float32 A tile as landed by TMA
constexpr int kHalfBytes = BM * BK * 2;  // 8 KiB: A_hi, A_lo, W_hi, W_lo tiles
constexpr int kSplitGroups = 2;  // groups of four warps that split A tiles, taking k-steps in turn
constexpr int kAccCols = 2 * BN;         // main + correction
constexpr int kTmemCols = 2 * kAccCols;  // double buffered
constexpr int kEpiBytes = 4 * 2 * 4096;  // 4 warps x 2 buffers x (32 rows x 128 B)

// PRESPLIT: A arrives already split (two half planes written by the producing kernel); no float32 staging
// tile and no split warps, so a stage is 32 KiB and the ring is deeper.
template <bool PRESPLIT> struct Cfg {
    static constexpr int kA32 = PRESPLIT ? 0 : kA32Bytes;
    static constexpr int kStageBytes = kA32 + 4 * kHalfBytes;  // 32 or 48 KiB
    static constexpr int kStages = PRESPLIT ? 6 : 4;
    static constexpr int kSplitWarps = PRESPLIT ? 0 : 4 * kSplitGroups;
    static constexpr int kThreads = 64 + 32 * kSplitWarps + 128;
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*align*/ + 256 /*barriers*/;
};
__device__ __forceinline__ void split2(float a, float b, float s, uint32_t& hi, uint32_t& lo, float& amax) {
    a *= s;
    b *= s;
    amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
    const __half2 h = __floats2half2_rn(a, b);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn((a - hf.x) * kLoScale, (b - hf.y) * kLoScale);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// Split the landed float32 A tile into half hi / lo tiles.  128 threads; a thread owns four 32-byte units
// (8 floats -> 8 + 8 halves).  Unit p of row r sits at r*128 + p*32 in the float32 tile and its halves go to
// r*64 + p*16 in each half tile (both swizzles XOR the unit index with (r >> 1) & 3); for odd r the
// float32 swizzle also swaps the two 16-byte halves of the unit.
__device__ __forceinline__ float split_tile(uint32_t a32, uint32_t a_hi, uint32_t a_lo, int tid, float s) {
    float4 v[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t src = a32 + (uint32_t)(tid + i * 128) * 32u;
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v[2 * i].x), "=f"(v[2 * i].y), "=f"(v[2 * i].z), "=f"(v[2 * i].w) : "r"(src));
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(v[2 * i + 1].x), "=f"(v[2 * i + 1].y), "=f"(v[2 * i + 1].z), "=f"(v[2 * i + 1].w)
                     : "r"(src + 16u));
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int unit = tid + i * 128;
        const int r = unit >> 2;
        const bool odd = (r & 1) != 0;
        const float4 x0 = odd ? v[2 * i + 1] : v[2 * i];
        const float4 x1 = odd ? v[2 * i] : v[2 * i + 1];
        uint32_t h[4], l[4];
        split2(x0.x, x0.y, s, h[0], l[0], amax);
        split2(x0.z, x0.w, s, h[1], l[1], amax);
        split2(x1.x, x1.y, s, h[2], l[2], amax);
        split2(x1.z, x1.w, s, h[3], l[3], amax);
        const uint32_t off = (uint32_t)unit * 16u;
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a_hi + off), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a_lo + off), "r"(l[0]), "r"(l[1]), "r"(l[2]), "r"(l[3]) : "memory");
    }
    return amax;
}


template <bool PRESPLIT>
__device__ __forceinline__ void gemm_f16x2_body(const CUtensorMap& map_a, const CUtensorMap& map_alo, const CUtensorMap& map_whi,
                                                const CUtensorMap& map_wlo, const CUtensorMap& map_c,
                                                const float* __restrict__ bias, const float* __restrict__ a_scale_ptr,
                                                float w_scale, int64_t m_total, int n_total, int k_total, int tiles_n,
                                                int64_t num_tiles, int32_t* __restrict__ status) {
    using C = Cfg<PRESPLIT>;
    constexpr int S = C::kStages;
    constexpr int kStageBytes = C::kStageBytes;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi_base = base + S * kStageBytes;
    const uint32_t bar_base = epi_base + kEpiBytes;
    // barrier block: full[S] | conv[S] | empty[S] | tmem_full[2] | tmem_empty[2] | tmem slot | abort flag | range flag
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto conv_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * S + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (3 * S + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (3 * S + 2 + b); };
    uint8_t* const bar_generic = smem_raw + (bar_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_generic + 8 * (3 * S + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (3 * S + 4) + 4);
    volatile int* range_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (3 * S + 4) + 8);
    // a stage: float32 A tile | A_hi | A_lo | W_hi | W_lo
    auto a32_addr = [&](int s) { return base + s * kStageBytes; };
    auto half_addr = [&](int s, int which) { return base + s * kStageBytes + C::kA32 + which * kHalfBytes; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (k_total + BK - 1) / BK;
    const float a_scale = a_scale_ptr ? *a_scale_ptr : 1.0f;

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
        *range_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                     "r"((uint32_t)kTmemCols)
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
                    if (PRESPLIT) {
                        mbar_expect_tx(full_bar(s), 4 * kHalfBytes);
                        tma_load_2d(half_addr(s, 0), &map_a, kb * BK, (int)(tile_m * BM), full_bar(s));
                        tma_load_2d(half_addr(s, 1), &map_alo, kb * BK, (int)(tile_m * BM), full_bar(s));
                    } else {
                        mbar_expect_tx(full_bar(s), kA32Bytes + 2 * kHalfBytes);
                        tma_load_2d(a32_addr(s), &map_a, kb * BK, (int)(tile_m * BM), full_bar(s));
                    }
                    tma_load_2d(half_addr(s, 2), &map_whi, kb * BK, tile_n * BN, full_bar(s));
                    tma_load_2d(half_addr(s, 3), &map_wlo, kb * BK, tile_n * BN, full_bar(s));
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
                const uint32_t acc = tmem_base + (uint32_t)(buf * kAccCols);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = (int)(it % S);
                    const uint32_t ph = (uint32_t)((it / S) & 1);
                    // A split done (which implies the TMA data landed), or just the TMA data when A came split
                    ok = mbar_wait(PRESPLIT ? full_bar(s) : conv_bar(s), ph, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // The W_hi and W_lo tiles are adjacent in shared memory, so one 256-wide MMA on a_hi yields
                    // a_hi*w_hi in the main accumulator and a_hi*w_lo in the correction accumulator beside it (a_hi is
                    // read once for both); a 128-wide MMA then adds a_lo*w_hi to the correction accumulator.
                    const uint64_t da_hi = smem_desc64(half_addr(s, 0)), da_lo = smem_desc64(half_addr(s, 1));
                    const uint64_t dw = smem_desc64(half_addr(s, 2));
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j) {
                        const uint64_t adv = (uint64_t)(j * 2);  // 16 halves = 32 bytes per MMA, in 16-byte units
                        const uint32_t first = (kb > 0 || j > 0) ? 1u : 0u;
                        umma_f16<2 * BN>(acc, da_hi + adv, dw + adv, first);
                        umma_f16<BN>(acc + BN, da_lo + adv, dw + adv, 1u);
                    }
                    umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(tfull_bar(buf));
            }
        }
    } else if (warp < 2 + C::kSplitWarps) {
        const int group = (warp - 2) >> 2;
        const int tid = (threadIdx.x - 64) & 127;  // 0..127 within the group
        int64_t it = 0;
        bool ok = true;
        float amax = 0.f;
        for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                if ((int)(it % kSplitGroups) != group) continue;
                const int s = (int)(it % S);
                const uint32_t ph = (uint32_t)((it / S) & 1);
                ok = mbar_wait(full_bar(s), ph, abort_flag);
                if (!ok) break;
                amax = fmaxf(amax, split_tile(a32_addr(s), half_addr(s, 0), half_addr(s, 1), tid, a_scale));
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(conv_bar(s));
            }
        }
        if (!(amax <= kHalfMax)) *range_flag = 1;  // also catches NaN
    } else {
        // epilogue: warp q = warp % 4 owns TMEM lanes [32q, 32q+32)
        const int q = warp & 3;
        const float out_scale = 1.0f / (a_scale * w_scale);
        const float corr_scale = out_scale / kLoScale;
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
            const uint32_t acc = tmem_base + (uint32_t)(buf * kAccCols) + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc, ++chunk) {
                const int col0 = tile_n * BN + cc * 32;
                uint32_t r[32], t[32];
                FCB_TMEM_LD32(r, acc + (uint32_t)(cc * 32));
                FCB_TMEM_LD32(t, acc + (uint32_t)(BN + cc * 32));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    r[i] = __float_as_uint(fmaf(__uint_as_float(t[i]), corr_scale, __uint_as_float(r[i]) * out_scale));
                if (row0 >= m_total || col0 >= n_total) continue;  // sub-tile entirely outside the matrix
                {  // a half that overflowed upstream shows up here as inf or NaN (exponent bits all set)
                    uint32_t bad = 0;
#pragma unroll
                    for (int i = 0; i < 32; ++i) bad |= (uint32_t)((r[i] & 0x7f800000u) == 0x7f800000u);
                    if (bad) *range_flag = 1;
                }
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && status) {
        if (*abort_flag) atomicExch(status, 1);
        else if (*range_flag) atomicCAS(status, 0, 2);
    }
}

// A as float32, split by the kernel
__global__ void __launch_bounds__(Cfg<false>::kThreads, 1)
    gemm_f16x2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_whi,
                      const __grid_constant__ CUtensorMap map_wlo, const __grid_constant__ CUtensorMap map_c,
                      const float* __restrict__ bias, const float* __restrict__ a_scale_ptr, float w_scale, int64_t m_total,
                      int n_total, int k_total, int tiles_n, int64_t num_tiles, int32_t* __restrict__ status) {
    gemm_f16x2_body<false>(map_a, map_a, map_whi, map_wlo, map_c, bias, a_scale_ptr, w_scale, m_total, n_total, k_total, tiles_n,
                           num_tiles, status);
}

// A as the two half planes its producer wrote
__global__ void __launch_bounds__(Cfg<true>::kThreads, 1)
    gemm_f16x2_presplit_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
                               const __grid_constant__ CUtensorMap map_whi, const __grid_constant__ CUtensorMap map_wlo,
                               const __grid_constant__ CUtensorMap map_c, const float* __restrict__ bias,
                               const float* __restrict__ a_scale_ptr, float w_scale, int64_t m_total, int n_total, int k_total,
                               int tiles_n, int64_t num_tiles, int32_t* __restrict__ status) {
    gemm_f16x2_body<true>(map_ahi, map_alo, map_whi, map_wlo, map_c, bias, a_scale_ptr, w_scale, m_total, n_total, k_total, tiles_n,
                          num_tiles, status);
}

// w [rows, cols] float32 with row stride ldw -> contiguous half hi / lo [rows, cols], both of (w * scale)
__global__ void split_f16_kernel(const float* __restrict__ w, int64_t ldw, __half* __restrict__ hi, __half* __restrict__ lo,
                                 float scale, int64_t rows, int64_t cols) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * cols) return;
    const float v = w[(i / cols) * ldw + (i % cols)] * scale;
    const __half h = __float2half_rn(v);
    hi[i] = h;
    lo[i] = __float2half_rn((v - __half2float(h)) * kLoScale);
}

// 2-D row-major [rows, cols] with row stride ld (elements); box = 32 columns x box_rows rows
static int make_map_f32(CUtensorMap* map, const float* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return FCB200_EINVAL;
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {32u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FCB200_OK : FCB200_EINVAL;
}

static int make_map_f16(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return FCB200_EINVAL;
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BN};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FCB200_OK : FCB200_EINVAL;
}

}  // namespace f16

}  // namespace fcb200

using namespace fcb200;

extern "C" int fcb200_split_f16(const float* w, int64_t ldw, void* w_hi, void* w_lo, float scale, int64_t rows, int64_t cols,
                                void* stream) {
    if (!w || !w_hi || !w_lo || rows < 0 || cols < 0 || ldw < cols || !(scale > 0.f)) return FCB200_EINVAL;
    if (rows * cols == 0) return FCB200_OK;
    f16::split_f16_kernel<<<(unsigned)((rows * cols + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        w, ldw, static_cast<__half*>(w_hi), static_cast<__half*>(w_lo), scale, rows, cols);
    return launch_status();
}

namespace {

template <bool PRESPLIT>
int launch_f16(const CUtensorMap& ma, const CUtensorMap& malo, const CUtensorMap& mh, const CUtensorMap& ml, const CUtensorMap& mc,
               const float* bias, const float* a_scale, float w_scale, int64_t m, int n, int k, int32_t* status, cudaStream_t s) {
    using C = f16::Cfg<PRESPLIT>;
    static bool attr_done[64] = {};
    const int arc = PRESPLIT ? ensure_dynamic_smem(f16::gemm_f16x2_presplit_kernel, C::kSmemBytes, attr_done)
                             : ensure_dynamic_smem(f16::gemm_f16x2_kernel, C::kSmemBytes, attr_done);
    if (arc) return arc;
    const int tiles_n = (n + f16::BN - 1) / f16::BN;
    const int64_t tiles_m = (m + f16::BM - 1) / f16::BM;
    const int64_t num_tiles = tiles_m * tiles_n;
    const int grid = (int)(num_tiles < sm_count() ? num_tiles : sm_count());
    if (PRESPLIT)
        f16::gemm_f16x2_presplit_kernel<<<grid, C::kThreads, C::kSmemBytes, s>>>(ma, malo, mh, ml, mc, bias, a_scale, w_scale, m, n, k,
                                                                                tiles_n, num_tiles, status);
    else
        f16::gemm_f16x2_kernel<<<grid, C::kThreads, C::kSmemBytes, s>>>(ma, mh, ml, mc, bias, a_scale, w_scale, m, n, k, tiles_n,
                                                                       num_tiles, status);
    return launch_status();
}

}  // namespace

extern "C" int fcb200_gemm_f16x2(const float* a, int64_t lda, const void* w_hi, const void* w_lo, int64_t ldw, float w_scale,
                                 const float* a_scale, const float* bias, float* c, int64_t ldc, int64_t m, int32_t n, int32_t k,
                                 int32_t* status, void* stream) {
    if (!a || !w_hi || !w_lo || !c || m < 0 || n <= 0 || k <= 0 || !(w_scale > 0.f)) return FCB200_EINVAL;
    if (n % 4 || k % 8 || lda % 4 || ldw % 8 || ldc % 4 || lda < k || ldw < k || ldc < n) return FCB200_EINVAL;
    if (!aligned16(a) || !aligned16(w_hi) || !aligned16(w_lo) || !aligned16(c) || (bias && !aligned16(bias))) return FCB200_EALIGN;
    if (m == 0) return FCB200_OK;
    CUtensorMap ma, mh, ml, mc;
    int rc = f16::make_map_f32(&ma, a, m, k, lda, f16::BM);
    if (rc) return rc;
    rc = f16::make_map_f16(&mh, w_hi, n, k, ldw);
    if (rc) return rc;
    rc = f16::make_map_f16(&ml, w_lo, n, k, ldw);
    if (rc) return rc;
    rc = f16::make_map_f32(&mc, c, m, n, ldc, 32);
    if (rc) return rc;
    return launch_f16<false>(ma, ma, mh, ml, mc, bias, a_scale, w_scale, m, n, k, status, static_cast<cudaStream_t>(stream));
}

extern "C" int fcb200_gemm_f16x2_presplit(const void* a_hi, const void* a_lo, int64_t lda, const void* w_hi, const void* w_lo,
                                          int64_t ldw, float w_scale, const float* a_scale, const float* bias, float* c,
                                          int64_t ldc, int64_t m, int32_t n, int32_t k, int32_t* status, void* stream) {
    if (!a_hi || !a_lo || !w_hi || !w_lo || !c || m < 0 || n <= 0 || k <= 0 || !(w_scale > 0.f)) return FCB200_EINVAL;
    if (n % 4 || k % 8 || lda % 8 || ldw % 8 || ldc % 4 || lda < k || ldw < k || ldc < n) return FCB200_EINVAL;
    if (!aligned16(a_hi) || !aligned16(a_lo) || !aligned16(w_hi) || !aligned16(w_lo) || !aligned16(c) || (bias && !aligned16(bias)))
        return FCB200_EALIGN;
    if (m == 0) return FCB200_OK;
    CUtensorMap mah, mal, mh, ml, mc;
    int rc = f16::make_map_f16(&mah, a_hi, m, k, lda);
    if (rc) return rc;
    rc = f16::make_map_f16(&mal, a_lo, m, k, lda);
    if (rc) return rc;
    rc = f16::make_map_f16(&mh, w_hi, n, k, ldw);
    if (rc) return rc;
    rc = f16::make_map_f16(&ml, w_lo, n, k, ldw);
    if (rc) return rc;
    rc = f16::make_map_f32(&mc, c, m, n, ldc, 32);
    if (rc) return rc;
    return launch_f16<true>(mah, mal, mh, ml, mc, bias, a_scale, w_scale, m, n, k, status, static_cast<cudaStream_t>(stream));
}
