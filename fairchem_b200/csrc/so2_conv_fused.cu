// One launch per SO(2) convolution: a persistent CTA owns a 128-edge row tile and walks the output column
// tiles of all m-blocks of the convolution in turn (each with its own slice of the input columns, weight
// matrix and K extent), with the gate activation -- or its derivative -- applied in the epilogue, so that
// the convolution output never makes a round trip through memory as float32 just to be gated:
//
//   conv 1 forward : A = rotated+radial-scaled rows (hi, lo planes)  ->  tiles [gate scalars | rows]
//                    gate tiles  : raw float32 into y (later tiles of the same warp read them back through TMA)
//                    row tiles   : row 0 -> v * sigmoid(v); row (l, m) -> v * sigmoid(gate[l-1]); written as the
//                                  (hi, lo) half planes conv 2 reads; raw y rows are stored only when the backward
//                                  pass will want them
//   conv 2 forward : plain float32 output (messages)
//   conv 2 backward: A = message gradient planes -> tiles = rows of the gate output's gradient; the epilogue
//                    reads the kept y, writes the gradient of the conv-1 output as (hi, lo) planes and sums the
//                    gate-scalar gradients over the rows of a degree in registers (the tiles of a degree are
//                    consecutive: the first resets the sums, the last writes them into the planes)
//   conv 1 backward: plain float32 output (gradient of the rotated rows)
//
// Replaces SO2_Convolution.forward + GateActivation.forward of the reference
// (src/fairchem/core/models/uma/nn/so2_layers.py:600-647, src/fairchem/core/models/uma/nn/activation.py:146-165)
// and their autograd twins.  Arithmetic, tile shape, operand format, accumulators and the bounded waits are those
// of gemm_f16x2_presplit_kernel; what differs is the tile schedule (row tile outermost, so the gate scalars and
// all rows of an edge pass through one thread), eight epilogue warps (two per TMEM lane quarter, each taking
// half of the tile's columns) and the epilogue modes.
#include "gemm_f16_common.cuh"

namespace fcb200 {
namespace fused {

using namespace f16;

enum Mode : int32_t {
    kPlain = 0,     // float32 tile -> y[:, out_col ...] through TMA
    kGateRaw = 1,   // (unused: gate scalars are kPlain tiles listed before Plan::rot_begin)
    kSilu = 2,      // planes[:, out_col ...] = split(v * sigmoid(v));                       keep: y[:, y_col ...] = v
    kGated = 3,     // planes[:, out_col ...] = split(v * sigmoid(y[:, gate_col ...]));      keep: y[:, y_col ...] = v
    kSiluBwd = 4,   // planes[:, out_col ...] = split(v * d/dy silu(y[:, y_col ...]))
    kGatedBwd = 5,  // planes[:, out_col ...] = split(v * sigmoid(gate)); gate gradient summed over consecutive tiles
};
enum Flags : int32_t { kFirst = 1, kLast = 2, kKeep = 4 };

struct Tile {
    int32_t a_col;     // first input column of this tile's K range
    int32_t k;         // K extent (multiple of 32)
    int32_t w;         // weight matrix 0..2
    int32_t w_row;     // first output row of the weight matrix (multiple of 128)
    int32_t out_col;   // where the result goes (column of y for float32 modes, of the planes for split modes)
    int32_t mode;
    int32_t y_col;     // column of y holding this row's raw value (kSilu/kGated keep, kSiluBwd/kGatedBwd read)
    int32_t gate_col;  // column of y (and of the gradient planes / scratch) of the gate scalars of this row's degree
    int32_t flags;
    int32_t pad;
};
constexpr int kMaxTiles = 40;  // lmax 4: 19 rows x 2C = 38 column tiles in the conv-1 backward
struct Plan {
    int32_t ntiles;
    int32_t rot_begin;  // tiles [rot_begin, ntiles) may run in any order: every CTA starts at a different one of them
    int32_t pad[2];
    Tile t[kMaxTiles];
};

// Loop position -> tile.  All CTAs walk the same weight tiles; started together they would ask L2 for the same lines
// at the same moment, so each CTA (or pair) begins the freely ordered part of the list at its own offset.
__device__ __forceinline__ int tile_at(const Plan& plan, int pos, int rot) {
    const int free = plan.ntiles - plan.rot_begin;
    return (pos < plan.rot_begin || free <= 1) ? pos : plan.rot_begin + (pos - plan.rot_begin + rot) % free;
}

// NBUF staging tiles per epilogue warp: 3 for plans with gated modes, 2 for plans of plain tiles only, which leaves
// room for one more stage of the operand ring (the ring's depth is what covers the latency of the operand loads)
template <int NBUF> struct Cfg {
    static constexpr int kStages = NBUF == 3 ? 4 : 5;
    static constexpr int kPairStages = NBUF == 3 ? 5 : 6;
    static constexpr int kEpiWarpBytes = NBUF * 4096;
};
constexpr int kStageBytes = 4 * BM * BK * 2;           // A_hi | A_lo | W_hi | W_lo, 8 KiB each
constexpr int kHalfTile = BM * BK * 2;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;          // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int kAccCols = 2 * BN, kTmemCols = 2 * kAccCols;
// KB = k extent of one ring stage: 32 (64-byte rows, 64-byte swizzle) or 64 (128-byte rows, 128-byte swizzle, two
// stages of 64 KiB)
template <int NBUF, int KB> constexpr int ring_stages() { return KB == 64 ? 2 : Cfg<NBUF>::kStages; }
template <int NBUF, int KB = BK> constexpr int smem_bytes() {
    return ring_stages<NBUF, KB>() * 4 * BM * KB * 2 + kEpiWarps * Cfg<NBUF>::kEpiWarpBytes + 1024 + 256;
}
// K-major, 128-byte swizzle: rows at a 128 B pitch, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t smem_desc128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}

struct Params {
    const float* bias[3];
    float w_scale[3];
    float* y;          // raw conv-1 output / float32 output
    int64_t ldy;
    const float* a_scale;  // power of two the A planes were written with (null = 1)
    const float* o_scale;  // power of two the output planes are written with (null = 1)
    int64_t m_total;
    int32_t* status;
};

// 1 / (1 + e^-v) on the special-function unit (ex2.approx, rcp.approx): relative error ~2^-22, a few instructions
// instead of the ~20 of expf and an IEEE division -- the epilogue evaluates it for every output element
__device__ __forceinline__ float sigmoid_f(float v) { return __fdividef(1.0f, 1.0f + __expf(-v)); }

// pack (a, b) * already-applied scale into hi and lo half pairs; track the largest magnitude
__device__ __forceinline__ void pack2(float a, float b, uint32_t& hi, uint32_t& lo, float& amax) {
    amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
    const __half2 h = __floats2half2_rn(a, b);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn((a - hf.x) * kLoScale, (b - hf.y) * kLoScale);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// 8 consecutive values -> one 16-byte unit of the hi staging tile and one of the lo staging tile.
// Row `lane` of a 32-row x 64-byte tile with the 64-byte swizzle: unit index XOR ((row >> 1) & 3).
__device__ __forceinline__ void stage_split8(uint32_t hi_base, uint32_t lo_base, int lane, int unit, const float (&v)[8], float& amax) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pack2(v[2 * i], v[2 * i + 1], h[i], l[i], amax);
    const uint32_t off = (uint32_t)(lane * 64 + ((unit ^ ((lane >> 1) & 3)) * 16));
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(hi_base + off), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(lo_base + off), "r"(l[0]), "r"(l[1]), "r"(l[2]), "r"(l[3]) : "memory");
}

// 4 consecutive float32 -> 16-byte chunk `v4` of row `lane` of a 32-row x 128-byte tile with the 128-byte swizzle
__device__ __forceinline__ void stage_f32x4(uint32_t base, int lane, int v4, float a, float b, float c, float d) {
    const uint32_t dst = base + (uint32_t)(lane * 128 + ((v4 ^ (lane & 7)) * 16));
    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}



// ---- CTA pairs (cta_group::2): two CTAs of a cluster share a 256-row tile and each holds half of the B operand ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// TMA load whose completion is signalled on a barrier that may live in the peer CTA (no multicast: the data lands in
// this CTA's own shared memory only)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// arrive on the barrier at this offset in both CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}
// instruction descriptor of the pair MMA: M = 256 (128 rows in each CTA), N columns
constexpr uint32_t instr_desc_pair(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24); }
template <int N>
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(instr_desc_pair(N)), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u),
          "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

// own row (`lane`) of a 32 x 32 float32 tile that TMA landed with the 128-byte swizzle: values [8u, 8u + 8)
__device__ __forceinline__ void ld_row8(uint32_t base, int lane, int u, float (&o)[8]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t src = base + (uint32_t)(lane * 128 + (((2 * u + h) ^ (lane & 7)) * 16));
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(o[4 * h]), "=f"(o[4 * h + 1]), "=f"(o[4 * h + 2]), "=f"(o[4 * h + 3]) : "r"(src));
    }
}

// Epilogue warps 2..9: warp w reads TMEM lanes [32 (w % 4), +32) -- one accumulator row per thread -- and takes the
// 64 columns [64 h, 64 h + 64) of every tile, h = (w - 2) / 4, in two chunks of 32.  Per warp three 4 KiB
// shared-memory tiles: B0 and B1 receive the 32 x 32 float32 tiles of y a gated mode reads (TMA loads, so the
// global reads are whole lines and each thread then takes its own row from shared memory), B2 stages the output;
// B1 doubles as the staging tile of a kept y row or of a finished gate gradient.  Launches of plain tiles rotate
// the output over all three.
// PAIR: the CTA is one of a pair that shares 256-row tiles; `unit` is the tile stride owner (CTA or pair index),
// `units` their number, `row_off` this CTA's first row inside a tile, and `tempty0` a shared::cluster address of the
// leader's accumulator-free barriers.
template <bool PAIR, int NBUF>
__device__ __forceinline__ void epilogue(const CUtensorMap& map_y, const CUtensorMap& map_ohi, const CUtensorMap& map_olo,
                                         const Plan& plan, const Params& prm, int64_t tiles_m, uint32_t tmem_base,
                                         uint32_t epi_base, uint32_t tfull0, uint32_t tempty0, uint32_t ld_bar0,
                                         volatile int* abort_flag, volatile int* range_flag, int64_t unit, int64_t units,
                                         int row_off) {
    constexpr int kTileRows = PAIR ? 2 * BM : BM;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q = warp & 3;
    const int ew = warp - 2;
    const int half = ew >> 2;
    const uint32_t b0 = epi_base + (uint32_t)(ew * Cfg<NBUF>::kEpiWarpBytes), b1 = b0 + 4096u, b2 = b0 + 8192u;  // b2 only if NBUF == 3
    const uint32_t ld_bar = ld_bar0 + 8u * ew;
    uint32_t ld_phase = 0;
    int rot = 0;             // plain chunks staged so far (output buffer = rot % 3)
    int last_kind = -1;      // 0 plain, 1 anything else
    bool b1_stored = false;  // the previous chunk issued a store that reads B1
    const float a_scale = prm.a_scale ? *prm.a_scale : 1.0f;
    const float o_scale = prm.o_scale ? *prm.o_scale : 1.0f;
    const int ntiles = plan.ntiles;
    const uint64_t stream_out = l2_policy_evict_first();  // outputs are not read again by this kernel (the gate scalars are: default policy)
    float amax = 0.f;
    float acc[2][32];  // gate-gradient sums over the rows of a degree (kGatedBwd), per chunk
    int64_t tcount = 0;
    bool ok = true;
    for (int64_t mt = unit; mt < tiles_m && ok; mt += units) {
        const int64_t row0 = mt * kTileRows + row_off + q * 32;
        const bool live = row0 < prm.m_total;  // else this warp's 32 rows lie entirely below the matrix
        for (int ti = 0; ti < ntiles; ++ti, ++tcount) {
            const Tile& t = plan.t[tile_at(plan, ti, (int)(unit % 64))];
            const int buf = (int)(tcount & 1);
            const uint32_t use = (uint32_t)((tcount >> 1) & 1);
            ok = mbar_wait(tfull0 + 8u * buf, use, abort_flag);
            ok = __all_sync(kFull, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float out_scale = 1.0f / (a_scale * prm.w_scale[t.w]);
            const float corr_scale = out_scale / kLoScale;
            const float* bias = prm.bias[t.w];
            const uint32_t acc_t = tmem_base + (uint32_t)(buf * kAccCols) + ((uint32_t)(q * 32) << 16);
            const int mode = t.mode;
            const bool keep = (t.flags & kKeep) != 0 && (mode == kSilu || mode == kGated);
            const bool fin = mode == kGatedBwd && (t.flags & kLast) != 0;
            const int n_in = mode == kGatedBwd ? 2 : ((mode == kGated || mode == kSiluBwd) ? 1 : 0);
#pragma unroll
            for (int c2 = 0; c2 < 2; ++c2) {
                const int col = (half * 2 + c2) * 32;  // within the tile
                // 1. inputs of the gated modes, fetched while the accumulator is read
                if (live && n_in > 0) {
                    if (lane == 0) {
                        if (last_kind == 0 || (n_in == 2 && b1_stored)) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        // first tile after the gate scalars: this thread's stores of them have landed before they are read back
                        if (ti == plan.rot_begin && plan.rot_begin > 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                        mbar_expect_tx(ld_bar, (uint32_t)(n_in * 4096));
                        tma_load_2d(b0, &map_y, (mode == kSiluBwd ? t.y_col : t.gate_col) + col, (int)row0, ld_bar);
                        if (n_in == 2) tma_load_2d(b1, &map_y, t.y_col + col, (int)row0, ld_bar);
                    }
                }
                // 2. accumulator -> registers
                float v[32];
                {
                    uint32_t r[32], c[32];
                    // single CTA: main sums in columns [0, 128), corrections in [128, 256).  Pair: 64-column blocks
                    // hh(0:32, 64:96) | corr(0:64) | hh(32:64, 96:128) | corr(64:128)
                    const int chunk = half * 2 + c2;
                    const uint32_t main_col = PAIR ? (uint32_t)((chunk & 1) * 128 + (chunk >> 1) * 32) : (uint32_t)col;
                    const uint32_t corr_col = PAIR ? (uint32_t)(64 + (chunk >> 1) * 128 + (chunk & 1) * 32) : (uint32_t)(BN + col);
                    FCB_TMEM_LD32(r, acc_t + main_col);
                    FCB_TMEM_LD32(c, acc_t + corr_col);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    float poison = 0.f;  // becomes NaN if any value is inf or NaN (an overflowed half upstream)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        v[i] = fmaf(__uint_as_float(c[i]), corr_scale, __uint_as_float(r[i]) * out_scale);
                        poison = fmaf(v[i], 0.f, poison);
                    }
                    if (poison != poison && row0 + lane < prm.m_total) *range_flag = 1;
                }
                if (!live) continue;
                if (bias) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 b = ld4(bias + t.w_row + col + 4 * i);
                        v[4 * i] += b.x, v[4 * i + 1] += b.y, v[4 * i + 2] += b.z, v[4 * i + 3] += b.w;
                    }
                }
                // 3. staging tiles free, inputs landed
                uint32_t st_out;
                if (mode == kPlain) {
                    if (lane == 0) {
                        if (last_kind != 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        else if (NBUF == 3) asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory");
                        else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    }
                    st_out = b0 + (uint32_t)((rot % NBUF) * 4096);
                    ++rot;
                    last_kind = 0;
                } else {
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    st_out = b2;
                    last_kind = 1;
                }
                if (n_in > 0) {
                    ok = mbar_wait(ld_bar, ld_phase, abort_flag);
                    ld_phase ^= 1u;
                }
                ok = __all_sync(kFull, ok);  // also orders lane 0's wait before everybody's staging writes
                if (!ok) break;
                // 4. the mode's arithmetic, staged for the stores
                if (mode == kPlain || keep) {
                    const uint32_t st_f32 = mode == kPlain ? st_out : b1;
#pragma unroll
                    for (int i = 0; i < 8; ++i) stage_f32x4(st_f32, lane, i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                }
                if (mode != kPlain) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float o[8];
                        if (mode == kSilu) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) o[i] = v[8 * u + i] * sigmoid_f(v[8 * u + i]) * o_scale;
                        } else if (mode == kGated) {
                            float g[8];
                            ld_row8(b0, lane, u, g);
#pragma unroll
                            for (int i = 0; i < 8; ++i) o[i] = v[8 * u + i] * sigmoid_f(g[i]) * o_scale;
                        } else if (mode == kSiluBwd) {
                            float y0[8];
                            ld_row8(b0, lane, u, y0);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float sg = sigmoid_f(y0[i]);
                                o[i] = v[8 * u + i] * sg * (1.f + y0[i] * (1.f - sg)) * o_scale;
                            }
                        } else {  // kGatedBwd
                            float g[8], yr[8];
                            ld_row8(b0, lane, u, g);
                            ld_row8(b1, lane, u, yr);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                g[i] = sigmoid_f(g[i]);
                                o[i] = v[8 * u + i] * g[i] * o_scale;
                                const float prev = (t.flags & kFirst) ? 0.f : acc[c2][8 * u + i];
                                acc[c2][8 * u + i] = fmaf(v[8 * u + i], yr[i], prev);
                                if (fin) acc[c2][8 * u + i] *= g[i] * (1.f - g[i]) * o_scale;
                            }
                        }
                        stage_split8(st_out, st_out + 2048u, lane, u, o, amax);
                    }
                    if (fin) {  // every thread has read its y row out of B1: stage the finished gate gradient there
                        __syncwarp();
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            float a[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) a[i] = acc[c2][8 * u + i];
                            stage_split8(b1, b1 + 2048u, lane, u, a, amax);
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    if (mode == kPlain) {
                        if (ti < plan.rot_begin) tma_store_2d(&map_y, st_out, t.out_col + col, (int)row0);  // gate scalars: read back
                        else tma_store_2d_hint(&map_y, st_out, t.out_col + col, (int)row0, stream_out);
                    } else {
                        if (keep) tma_store_2d_hint(&map_y, b1, t.y_col + col, (int)row0, stream_out);
                        tma_store_2d_hint(&map_ohi, st_out, t.out_col + col, (int)row0, stream_out);
                        tma_store_2d_hint(&map_olo, st_out + 2048u, t.out_col + col, (int)row0, stream_out);
                        if (fin) {
                            tma_store_2d_hint(&map_ohi, b1, t.gate_col + col, (int)row0, stream_out);
                            tma_store_2d_hint(&map_olo, b1 + 2048u, t.gate_col + col, (int)row0, stream_out);
                        }
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                b1_stored = keep || fin;
            }
            if (!ok) break;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            // hand the accumulator back to the MMA thread: every thread in the single-CTA kernel, one lane per warp in
            // the pair kernel (there the barrier may sit in the other SM and an arrive is a round trip)
            if (PAIR) {
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * buf);
            } else {
                mbar_arrive(tempty0 + 8u * buf);
            }
        }
    }
    if (!(amax <= kHalfMax)) *range_flag = 1;  // also catches NaN
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all stores of this warp have landed
}

template <int NBUF, int KB = BK>
__global__ void __launch_bounds__(kThreads, 1)
    so2_conv_fused_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
                          const __grid_constant__ CUtensorMap map_whi0, const __grid_constant__ CUtensorMap map_wlo0,
                          const __grid_constant__ CUtensorMap map_whi1, const __grid_constant__ CUtensorMap map_wlo1,
                          const __grid_constant__ CUtensorMap map_whi2, const __grid_constant__ CUtensorMap map_wlo2,
                          const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_ohi,
                          const __grid_constant__ CUtensorMap map_olo, const __grid_constant__ Plan plan,
                          const __grid_constant__ Params prm, int64_t tiles_m) {
    constexpr int S = ring_stages<NBUF, KB>();
    constexpr int kStage = 4 * BM * KB * 2, kPart = BM * KB * 2;  // A_hi | A_lo | W_hi | W_lo
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi_base = base + S * kStage;
    const uint32_t bar_base = epi_base + kEpiWarps * Cfg<NBUF>::kEpiWarpBytes;
    // barrier block: full[S] | empty[S] | tmem_full[2] | tmem_empty[2] | tmem slot, abort flag, range flag, pad | ld[8]
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * S + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * S + 2 + b); };
    auto ld_bar = [&](int w) { return bar_base + 8u * (2 * S + 6 + w); };  // one per epilogue warp, after the flag words
    uint8_t* const bar_generic = smem_raw + (bar_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_generic + 8 * (2 * S + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (2 * S + 4) + 4);
    volatile int* range_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (2 * S + 4) + 8);
    auto half_addr = [&](int s, int which) { return base + s * kStage + which * kPart; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntiles = plan.ntiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), 32 * kEpiWarps);
        }
        for (int w = 0; w < kEpiWarps; ++w) mbar_init(ld_bar(w), 1);
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
            // an A tile is fetched again for each of the output tiles of its m-block, the weights by every CTA: keep
            // both in L2 ahead of the streamed outputs
            const uint64_t keep = l2_policy_evict_last();
            for (int64_t mt = blockIdx.x; mt < tiles_m && ok; mt += gridDim.x) {
                for (int ti = 0; ti < ntiles && ok; ++ti) {
                    const Tile& t = plan.t[tile_at(plan, ti, (int)(blockIdx.x % 64))];
                    const CUtensorMap* whi = t.w == 0 ? &map_whi0 : (t.w == 1 ? &map_whi1 : &map_whi2);
                    const CUtensorMap* wlo = t.w == 0 ? &map_wlo0 : (t.w == 1 ? &map_wlo1 : &map_wlo2);
                    const int num_kb = t.k / KB;
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const int s = (int)(it % S);
                        const uint32_t ph = (uint32_t)((it / S) & 1);
                        ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag);
                        if (!ok) break;
                        mbar_expect_tx(full_bar(s), kStage);
                        tma_load_2d_hint(half_addr(s, 0), &map_ahi, t.a_col + kb * KB, (int)(mt * BM), full_bar(s), keep);
                        tma_load_2d_hint(half_addr(s, 1), &map_alo, t.a_col + kb * KB, (int)(mt * BM), full_bar(s), keep);
                        tma_load_2d_hint(half_addr(s, 2), whi, kb * KB, t.w_row, full_bar(s), keep);
                        tma_load_2d_hint(half_addr(s, 3), wlo, kb * KB, t.w_row, full_bar(s), keep);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int64_t it = 0, tcount = 0;
            bool ok = true;
            for (int64_t mt = blockIdx.x; mt < tiles_m && ok; mt += gridDim.x) {
                for (int ti = 0; ti < ntiles && ok; ++ti, ++tcount) {
                    const int num_kb = plan.t[tile_at(plan, ti, (int)(blockIdx.x % 64))].k / KB;
                    const int buf = (int)(tcount & 1);
                    const uint32_t use = (uint32_t)((tcount >> 1) & 1);
                    ok = mbar_wait(tempty_bar(buf), use ^ 1u, abort_flag);  // epilogue has drained this accumulator
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t acc = tmem_base + (uint32_t)(buf * kAccCols);
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const int s = (int)(it % S);
                        const uint32_t ph = (uint32_t)((it / S) & 1);
                        ok = mbar_wait(full_bar(s), ph, abort_flag);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        // W_hi | W_lo are adjacent: one 256-wide MMA on a_hi gives a_hi*w_hi (main accumulator) and
                        // a_hi*w_lo (correction accumulator); a 128-wide MMA adds a_lo*w_hi to the correction
                        auto desc = [](uint32_t addr) { return KB == 64 ? smem_desc128(addr) : smem_desc64(addr); };
                        const uint64_t da_hi = desc(half_addr(s, 0)), da_lo = desc(half_addr(s, 1));
                        const uint64_t dw = desc(half_addr(s, 2));
#pragma unroll
                        for (int j = 0; j < KB / 16; ++j) {
                            const uint64_t adv = (uint64_t)(j * 2);
                            const uint32_t first = (kb > 0 || j > 0) ? 1u : 0u;
                            umma_f16<2 * BN>(acc, da_hi + adv, dw + adv, first);
                            umma_f16<BN>(acc + BN, da_lo + adv, dw + adv, 1u);
                        }
                        umma_commit(empty_bar(s));
                    }
                    if (ok) umma_commit(tfull_bar(buf));
                }
            }
        }
    } else {
        epilogue<false, NBUF>(map_y, map_ohi, map_olo, plan, prm, tiles_m, tmem_base, epi_base, tfull_bar(0), tempty_bar(0), ld_bar(0),
                        abort_flag, range_flag, blockIdx.x, gridDim.x, 0);
    }

    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && prm.status) {
        if (*abort_flag) atomicExch(prm.status, 1);
        else if (*range_flag) atomicCAS(prm.status, 0, 2);
    }
}


// ---------------------------------------------------------------------------------------------------------------
// The same schedule on CTA pairs.  Two CTAs of a cluster own a 256-edge row tile (128 rows each); one thread of
// the leader CTA issues tcgen05.mma.cta_group::2 (M = 256), which reads each CTA's A rows from that CTA's shared
// memory and half of the B rows from each.  What bounds these contractions is the stream of operand bytes from L2
// into shared memory (a 128 x 128 tile re-reads 32 KiB per 32-deep k-step); in a pair each CTA fetches only half of
// the weight tile, 24 KiB per k-step, and the ring is one stage deeper.  Per stage a CTA holds
//     A_hi | A_lo (its 128 rows) | X (128 weight rows, see below)
//     X leader: W_hi[0:32) ; W_hi[64:96) ; W_lo[0:64)        X peer: W_hi[32:64) ; W_hi[96:128) ; W_lo[64:128)
// (row ranges relative to the tile's first output column).  Then
//     a_hi x [X_leader ; X_peer]                 (N = 256)  fills 64-column blocks  hh(0:32,64:96) | hl(0:64) | hh(32:64,96:128) | hl(64:128)
//     a_lo x [X_leader[0:32)  ; X_peer[0:32)]    (N = 64)   adds  lh(0:64)   to the second block
//     a_lo x [X_leader[32:64) ; X_peer[32:64)]   (N = 64)   adds  lh(64:128) to the fourth block
// so every weight row is fetched once per pair and the main and correction sums of a 32-column chunk are still two
// contiguous TMEM ranges.  TMA loads carry no multicast: every CTA fetches what lands in its own shared memory;
// their completion is counted on the leader's barrier.  tcgen05.commit with the pair mask frees a stage / publishes
// an accumulator in both CTAs.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kPairStageBytes = 3 * kHalfTile;  // 24 KiB
template <int NBUF> constexpr int pair_smem_bytes() {
    return Cfg<NBUF>::kPairStages * kPairStageBytes + kEpiWarps * Cfg<NBUF>::kEpiWarpBytes + 1024 + 256;
}

template <int NBUF>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    so2_conv_pair_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
                         const __grid_constant__ CUtensorMap map_whi0, const __grid_constant__ CUtensorMap map_wlo0,
                         const __grid_constant__ CUtensorMap map_whi1, const __grid_constant__ CUtensorMap map_wlo1,
                         const __grid_constant__ CUtensorMap map_whi2, const __grid_constant__ CUtensorMap map_wlo2,
                         const __grid_constant__ CUtensorMap map_y,
                         const __grid_constant__ CUtensorMap map_ohi, const __grid_constant__ CUtensorMap map_olo,
                         const __grid_constant__ Plan plan, const __grid_constant__ Params prm, int64_t tiles_m) {
    constexpr int S = Cfg<NBUF>::kPairStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi_base = base + S * kPairStageBytes;
    const uint32_t bar_base = epi_base + kEpiWarps * Cfg<NBUF>::kEpiWarpBytes;
    // barrier block as in the single-CTA kernel; full[] and tmem_empty[] are used in the leader only
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * S + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * S + 2 + b); };
    auto ld_bar = [&](int w) { return bar_base + 8u * (2 * S + 6 + w); };
    uint8_t* const bar_generic = smem_raw + (bar_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_generic + 8 * (2 * S + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (2 * S + 4) + 4);
    volatile int* range_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (2 * S + 4) + 8);
    // a stage: A_hi | A_lo | X   (the weight maps here have 32-row (W_hi) and 64-row (W_lo) boxes)
    auto part_addr = [&](int s, int which) { return base + s * kPairStageBytes + which * kHalfTile; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntiles = plan.ntiles;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int64_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);   // the leader's producer expects both CTAs' bytes; the peer only issues its loads
            mbar_init(empty_bar(s), 1);  // the leader's commit, delivered to both CTAs
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), 2 * kEpiWarps);  // one lane of every epilogue warp of both CTAs
        }
        for (int w = 0; w < kEpiWarps; ++w) mbar_init(ld_bar(w), 1);
        *abort_flag = 0;
        *range_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                     "r"((uint32_t)kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // both CTAs' barriers are initialised before either signals the other
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int64_t it = 0;
            bool ok = true;
            for (int64_t mt = pair; mt < tiles_m && ok; mt += pairs) {
                const int row = (int)(mt * 2 * BM + rank * BM);
                for (int ti = 0; ti < ntiles && ok; ++ti) {
                    const Tile& t = plan.t[tile_at(plan, ti, (int)(pair % 64))];
                    const CUtensorMap* whi = t.w == 0 ? &map_whi0 : (t.w == 1 ? &map_whi1 : &map_whi2);
                    const CUtensorMap* wlo = t.w == 0 ? &map_wlo0 : (t.w == 1 ? &map_wlo1 : &map_wlo2);
                    const int r_hi = t.w_row + (int)rank * 32, r_lo = t.w_row + (int)rank * 64;
                    const int num_kb = t.k / BK;
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const int s = (int)(it % S);
                        const uint32_t ph = (uint32_t)((it / S) & 1);
                        ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag);
                        if (!ok) break;
                        const uint32_t lead_full = map_to_cta(full_bar(s), 0);
                        // a remote arrive costs the issuing thread a round trip to the other SM: the leader alone announces
                        // the bytes of both CTAs, the peer's loads just complete on the leader's barrier
                        if (leader) mbar_expect_tx(full_bar(s), 2 * kPairStageBytes);
                        tma_load_2d_pair(part_addr(s, 0), &map_ahi, t.a_col + kb * BK, row, lead_full);
                        tma_load_2d_pair(part_addr(s, 1), &map_alo, t.a_col + kb * BK, row, lead_full);
                        tma_load_2d_pair(part_addr(s, 2), whi, kb * BK, r_hi, lead_full);
                        tma_load_2d_pair(part_addr(s, 2) + 2048u, whi, kb * BK, r_hi + 64, lead_full);
                        tma_load_2d_pair(part_addr(s, 2) + 4096u, wlo, kb * BK, r_lo, lead_full);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            int64_t it = 0, tcount = 0;
            bool ok = true;
            for (int64_t mt = pair; mt < tiles_m && ok; mt += pairs) {
                for (int ti = 0; ti < ntiles && ok; ++ti, ++tcount) {
                    const int num_kb = plan.t[tile_at(plan, ti, (int)(pair % 64))].k / BK;
                    const int buf = (int)(tcount & 1);
                    const uint32_t use = (uint32_t)((tcount >> 1) & 1);
                    ok = mbar_wait(tempty_bar(buf), use ^ 1u, abort_flag);  // both epilogues have drained this accumulator
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t acc = tmem_base + (uint32_t)(buf * kAccCols);
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const int s = (int)(it % S);
                        const uint32_t ph = (uint32_t)((it / S) & 1);
                        ok = mbar_wait(full_bar(s), ph, abort_flag);  // both CTAs' tiles have landed
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t da_hi = smem_desc64(part_addr(s, 0)), da_lo = smem_desc64(part_addr(s, 1));
                        const uint64_t dx = smem_desc64(part_addr(s, 2)), dx32 = smem_desc64(part_addr(s, 2) + 2048u);
#pragma unroll
                        for (int j = 0; j < BK / 16; ++j) {
                            const uint64_t adv = (uint64_t)(j * 2);
                            const uint32_t first = (kb > 0 || j > 0) ? 1u : 0u;
                            umma_f16_pair<2 * BN>(acc, da_hi + adv, dx + adv, first);
                            umma_f16_pair<BN / 2>(acc + 64, da_lo + adv, dx + adv, 1u);
                            umma_f16_pair<BN / 2>(acc + 192, da_lo + adv, dx32 + adv, 1u);
                        }
                        umma_commit_pair(empty_bar(s));
                    }
                    if (ok) umma_commit_pair(tfull_bar(buf));
                }
            }
        }
    } else {
        epilogue<true, NBUF>(map_y, map_ohi, map_olo, plan, prm, tiles_m, tmem_base, epi_base, tfull_bar(0), map_to_cta(tempty_bar(0), 0),
                       ld_bar(0), abort_flag, range_flag, pair, pairs, (int)rank * BM);
    }

    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // neither CTA leaves, nor frees tensor memory, while its peer can still reach it
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && prm.status) {
        if (*abort_flag) atomicExch(prm.status, 1);
        else if (*range_flag) atomicCAS(prm.status, 0, 2);
    }
}

// 2-D row-major half matrix [rows, cols], row stride ld elements; box = 32 columns x box_rows rows, 64-byte swizzle
static int map_half(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows, int box_cols = 32) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return FCB200_EINVAL;
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FCB200_OK : FCB200_EINVAL;
}

// float32 [rows, cols] with row stride ld; box = 32 x 32, 128-byte swizzle
static int map_f32(CUtensorMap* map, const float* ptr, int64_t rows, int64_t cols, int64_t ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return FCB200_EINVAL;
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {32u, 32u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FCB200_OK : FCB200_EINVAL;
}

// How many CTA pairs the device runs at once with this kernel's resources (cached per device); 0 on failure.
static int pair_capacity() {
    static int cap[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    const bool cached = dev >= 0 && dev < 64;
    if (cached && cap[dev] > 0) return cap[dev];
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = pair_smem_bytes<3>();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, so2_conv_pair_kernel<3>, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = sm_count() / 2;
    }
    if (cached) cap[dev] = n;
    return n;
}

}  // namespace fused
}  // namespace fcb200

using namespace fcb200;

extern "C" int fcb200_conv_pair_capacity(void) { return fused::pair_capacity(); }

extern "C" int fcb200_so2_conv_fused(const void* a_hi, const void* a_lo, int64_t lda, int64_t a_cols, const void* const* w_hi,
                                     const void* const* w_lo, const int64_t* w_rows, const int64_t* w_cols,
                                     const float* w_scale, const float* const* bias, const int32_t* tiles, int32_t num_tiles,
                                     int32_t rot_begin, float* y, int64_t ldy, int64_t y_cols, void* o_hi, void* o_lo, int64_t ldo, int64_t o_cols,
                                     const float* a_scale, const float* o_scale, int64_t m, int32_t variant, int32_t* status,
                                     void* stream) {
    using namespace fused;
    if (!a_hi || !a_lo || !w_hi || !w_lo || !w_rows || !w_cols || !w_scale || !tiles || !y || m < 0) return FCB200_EINVAL;
    Plan plan{};
    Params prm{};
    if (num_tiles <= 0 || num_tiles > kMaxTiles) return FCB200_ERANGE;
    if (variant < 0 || variant > 2) return FCB200_EINVAL;
    if (variant == 2)  // 64-deep stages need every K extent to be a multiple of 64; otherwise the 32-deep form runs
        for (int i = 0; i < num_tiles; ++i)
            if (tiles[9 * i + 1] % 64) variant = 0;
    const int kb_cols = variant == 2 ? 64 : 32;  // k extent of a ring stage
    if (lda % 8 || lda < a_cols || ldy % 4 || ldy < y_cols) return FCB200_EINVAL;
    if (!aligned16(a_hi) || !aligned16(a_lo) || !aligned16(y)) return FCB200_EALIGN;
    if (o_hi || o_lo) {
        if (!o_hi || !o_lo || ldo % 8 || ldo < o_cols) return FCB200_EINVAL;
        if (!aligned16(o_hi) || !aligned16(o_lo)) return FCB200_EALIGN;
    }
    if (rot_begin < 0 || rot_begin > num_tiles) return FCB200_EINVAL;
    plan.ntiles = num_tiles;
    plan.rot_begin = rot_begin;
    bool used[3] = {false, false, false};
    bool plain_only = true;
    for (int i = 0; i < num_tiles; ++i) {
        Tile& t = plan.t[i];
        const int32_t* d = tiles + 9 * i;
        t.a_col = d[0], t.k = d[1], t.w = d[2], t.w_row = d[3], t.out_col = d[4], t.mode = d[5], t.y_col = d[6], t.gate_col = d[7];
        t.flags = d[8];
        if (t.w < 0 || t.w > 2 || !w_hi[t.w] || !w_lo[t.w]) return FCB200_EINVAL;
        if (t.k <= 0 || t.k % kb_cols || t.k > w_cols[t.w] || t.a_col < 0 || t.a_col % 8 || t.a_col + t.k > a_cols) return FCB200_EINVAL;
        if (t.w_row < 0 || t.w_row % BN || t.w_row + BN > w_rows[t.w]) return FCB200_EINVAL;
        if (t.mode < kPlain || t.mode > kGatedBwd || t.mode == kGateRaw || t.out_col < 0 || t.out_col % 8) return FCB200_EINVAL;
        const bool split = t.mode >= kSilu;
        if (split && (!o_hi || t.out_col + BN > o_cols)) return FCB200_EINVAL;
        if (!split && t.out_col + BN > y_cols) return FCB200_EINVAL;
        const bool reads_gate = t.mode == kGated || t.mode == kGatedBwd;
        if (reads_gate && (t.gate_col < 0 || t.gate_col % 4 || t.gate_col + BN > y_cols)) return FCB200_EINVAL;
        const bool uses_y = t.mode == kSiluBwd || t.mode == kGatedBwd || ((t.mode == kSilu || t.mode == kGated) && (t.flags & kKeep));
        if (uses_y && (t.y_col < 0 || t.y_col % 4 || t.y_col + BN > y_cols)) return FCB200_EINVAL;
        if (t.mode == kGatedBwd && t.gate_col + BN > o_cols) return FCB200_EINVAL;
        used[t.w] = true;
        plain_only = plain_only && t.mode == kPlain;
    }
    if (m == 0) return FCB200_OK;
    CUtensorMap mah, mal, mw[6], my, moh, mol;
    int rc = map_half(&mah, a_hi, m, a_cols, lda, BM, kb_cols);
    if (!rc) rc = map_half(&mal, a_lo, m, a_cols, lda, BM, kb_cols);
    int first = -1;
    for (int i = 0; i < 3 && !rc; ++i) {
        if (!used[i]) continue;
        if (first < 0) first = i;
        if (w_cols[i] % 8 || !aligned16(w_hi[i]) || !aligned16(w_lo[i]) || !(w_scale[i] > 0.f)) return FCB200_EINVAL;
        rc = map_half(&mw[2 * i], w_hi[i], w_rows[i], w_cols[i], w_cols[i], BN, kb_cols);
        if (!rc) rc = map_half(&mw[2 * i + 1], w_lo[i], w_rows[i], w_cols[i], w_cols[i], BN, kb_cols);
        prm.w_scale[i] = w_scale[i];
        prm.bias[i] = bias ? bias[i] : nullptr;
        if (prm.bias[i] && !aligned16(prm.bias[i])) return FCB200_EALIGN;
    }
    if (rc) return rc;
    for (int i = 0; i < 3; ++i)
        if (!used[i]) {  // never dereferenced; keep the parameter block initialised
            mw[2 * i] = mw[2 * first], mw[2 * i + 1] = mw[2 * first + 1];
            prm.w_scale[i] = 1.f;
        }
    rc = map_f32(&my, y, m, y_cols, ldy);
    if (rc) return rc;
    if (o_hi) {
        rc = map_half(&moh, o_hi, m, o_cols, ldo, 32);
        if (!rc) rc = map_half(&mol, o_lo, m, o_cols, ldo, 32);
        if (rc) return rc;
    } else {
        moh = mah, mol = mal;  // no split-output tile exists (checked above)
    }
    prm.y = y, prm.ldy = ldy, prm.a_scale = a_scale, prm.o_scale = o_scale;
    prm.m_total = m, prm.status = status;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (variant == 1) {
        CUtensorMap mp[6];  // W_hi with 32-row boxes, W_lo with 64-row boxes
        for (int i = 0; i < 3; ++i) {
            const int j = used[i] ? i : first;
            rc = map_half(&mp[2 * i], w_hi[j], w_rows[j], w_cols[j], w_cols[j], 32);
            if (!rc) rc = map_half(&mp[2 * i + 1], w_lo[j], w_rows[j], w_cols[j], w_cols[j], 64);
            if (rc) return rc;
        }
        const int64_t tiles_m = (m + 2 * BM - 1) / (2 * BM);
        const int max_pairs = pair_capacity();
        if (max_pairs <= 0) return FCB200_EINVAL;
        const int pairs = (int)(tiles_m < max_pairs ? tiles_m : max_pairs);
        if (plain_only) {
            static bool attr_done[64] = {};
            if (const int arc = ensure_dynamic_smem(so2_conv_pair_kernel<2>, pair_smem_bytes<2>(), attr_done)) return arc;
            so2_conv_pair_kernel<2><<<2 * pairs, kThreads, pair_smem_bytes<2>(), st>>>(mah, mal, mp[0], mp[1], mp[2], mp[3], mp[4],
                                                                                      mp[5], my, moh, mol, plan, prm, tiles_m);
        } else {
            static bool attr_done[64] = {};
            if (const int arc = ensure_dynamic_smem(so2_conv_pair_kernel<3>, pair_smem_bytes<3>(), attr_done)) return arc;
            so2_conv_pair_kernel<3><<<2 * pairs, kThreads, pair_smem_bytes<3>(), st>>>(mah, mal, mp[0], mp[1], mp[2], mp[3], mp[4],
                                                                                      mp[5], my, moh, mol, plan, prm, tiles_m);
        }
        return launch_status();
    }
    const int64_t tiles_m = (m + BM - 1) / BM;
    const int grid = (int)(tiles_m < sm_count() ? tiles_m : sm_count());
    if (variant == 2) {
        if (plain_only) {
            static bool attr_done[64] = {};
            if (const int arc = ensure_dynamic_smem(so2_conv_fused_kernel<2, 64>, smem_bytes<2, 64>(), attr_done)) return arc;
            so2_conv_fused_kernel<2, 64><<<grid, kThreads, smem_bytes<2, 64>(), st>>>(mah, mal, mw[0], mw[1], mw[2], mw[3], mw[4],
                                                                                     mw[5], my, moh, mol, plan, prm, tiles_m);
        } else {
            static bool attr_done[64] = {};
            if (const int arc = ensure_dynamic_smem(so2_conv_fused_kernel<3, 64>, smem_bytes<3, 64>(), attr_done)) return arc;
            so2_conv_fused_kernel<3, 64><<<grid, kThreads, smem_bytes<3, 64>(), st>>>(mah, mal, mw[0], mw[1], mw[2], mw[3], mw[4],
                                                                                     mw[5], my, moh, mol, plan, prm, tiles_m);
        }
        return launch_status();
    }
    if (plain_only) {
        static bool attr_done[64] = {};
        if (const int arc = ensure_dynamic_smem(so2_conv_fused_kernel<2>, smem_bytes<2>(), attr_done)) return arc;
        so2_conv_fused_kernel<2><<<grid, kThreads, smem_bytes<2>(), st>>>(mah, mal, mw[0], mw[1], mw[2], mw[3], mw[4], mw[5], my, moh,
                                                                         mol, plan, prm, tiles_m);
    } else {
        static bool attr_done[64] = {};
        if (const int arc = ensure_dynamic_smem(so2_conv_fused_kernel<3>, smem_bytes<3>(), attr_done)) return arc;
        so2_conv_fused_kernel<3><<<grid, kThreads, smem_bytes<3>(), st>>>(mah, mal, mw[0], mw[1], mw[2], mw[3], mw[4], mw[5], my, moh,
                                                                         mol, plan, prm, tiles_m);
    }
    return launch_status();
}
