// Edge-block kernels of the eSCN-MD message-passing layer for lmax = mmax = 2 (sm_100a).
//
// All kernels are HBM-bound streaming kernels: one warp owns one edge (or one node segment),
// a lane owns 4 consecutive channels (one float4) of a 128-channel tile, node/edge rows move as
// 512-byte coalesced warp transactions, and the 35 Wigner entries of the edge live in registers
// (broadcast once per edge by shuffles).  Reductions over edges are segmented (CSR) sums with a
// fixed order: no atomics anywhere.
#include "common.cuh"

namespace fcb200 {

constexpr int kWarpsPerBlock = 8;

// Row m (M-major) of edge e inside an [E, 9, w] buffer.  The SO(2) GEMMs read their operands as column
// ranges of the flattened [E, 9*w] matrix: rows 0-2 (m = 0), rows 3-6 (m = 1: real pair | imaginary
// pair) and rows 7-8 (m = 2), so nothing is repacked between the rotation kernels and the GEMMs.
template <class P>
__device__ __forceinline__ P* edge_row(P* buf, int64_t e, int m, int w) {
    return buf + (e * 9 + m) * (int64_t)w;
}

// ---------------------------------------------------------------------------------------------
// gather + rotate (+ radial scale) forward
// ---------------------------------------------------------------------------------------------
template <bool HAS_RAD, class Out>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, 2)
    gather_rotate_fwd_kernel(const float* __restrict__ x, const int32_t* __restrict__ src, const int32_t* __restrict__ tgt,
                             const float* __restrict__ wig, const float* __restrict__ radial, Out out,
                             const float* __restrict__ scale_ptr, int64_t num_edges, int channels) {
    out.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    const int64_t node_stride = 9LL * channels;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        float w[FCB200_WIG];
        load_wig(wig, e, lane, w);
        const float* r_base = HAS_RAD ? radial + e * 12LL * channels : nullptr;
        // source half, then target half: nine node rows live at a time instead of eighteen, which lets two blocks share an
        // SM and doubles the loads in flight
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const float* x_base = x + (int64_t)(half == 0 ? src[e] : tgt[e]) * node_stride;
            for (int c0 = lane * 4; c0 < channels; c0 += 128) {
                float4 xv[9];
#pragma unroll
                for (int L = 0; L < 9; ++L) xv[L] = ld4(x_base + L * channels + c0);
#pragma unroll
                for (int m = 0; m < 9; ++m) {
                    const int L = m2l(m);
                    const int l = deg_of(L);
                    float4 a = f4zero();
#pragma unroll
                    for (int b = 0; b < 5; ++b)
                        if (b < 2 * l + 1) a = fma4(w[wix(L, l * l + b)], xv[l * l + b], a);
                    if (HAS_RAD) a = mul4(a, ld4(r_base + radslot(m) * 2 * channels + half * channels + c0));
                    out.st((e * 9 + m) * 2LL * channels + half * channels + c0, a);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// rotate back + segmented reduce by target (forward), optional residual input and scale
// ---------------------------------------------------------------------------------------------
// MODE 0: full 9-row messages.  MODE 1: edge-degree embedding (3 m=0 rows), out = x_in + sum / rescale.
template <int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp)
    rotate_back_reduce_kernel(const float* __restrict__ msg, const float* __restrict__ winv, const int32_t* __restrict__ row_ptr,
                              const float* __restrict__ x_in, float* __restrict__ out, float rescale, int64_t num_nodes,
                              int channels) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    const int rows_in = MODE == 0 ? 9 : 3;
    for (int64_t n = warp0; n < num_nodes; n += nwarps) {
        const int e0 = row_ptr[n], e1 = row_ptr[n + 1];
        for (int c0 = lane * 4; c0 < channels; c0 += 128) {
            float4 acc[9];
#pragma unroll
            for (int L = 0; L < 9; ++L) acc[L] = f4zero();
            for (int e = e0; e < e1; ++e) {
                float w[FCB200_WIG];
                load_wig(winv, e, lane, w);
                const float* y_base = msg + (int64_t)e * rows_in * channels + c0;
                if (MODE == 0) {
                    float4 y[9];
#pragma unroll
                    for (int m = 0; m < 9; ++m) y[m] = ld4(y_base + m * channels);
#pragma unroll
                    for (int L = 0; L < 9; ++L) {
                        const int l = deg_of(L);
#pragma unroll
                        for (int b = 0; b < 5; ++b)
                            if (b < 2 * l + 1) acc[L] = fma4(w[wix(L, l * l + b)], y[l2m(l * l + b)], acc[L]);
                    }
                } else {
                    float4 y[3];
#pragma unroll
                    for (int j = 0; j < 3; ++j) y[j] = ld4(y_base + j * channels);
#pragma unroll
                    for (int L = 0; L < 9; ++L) {
                        const int l = deg_of(L);
                        acc[L] = fma4(w[wix(L, l * l + l)], y[l], acc[L]);  // only the m=0 column of each block
                    }
                }
            }
            float* o = out + n * 9LL * channels + c0;
#pragma unroll
            for (int L = 0; L < 9; ++L) {
                float4 v = acc[L];
                if (MODE == 1) {
                    v = make_float4(v.x / rescale, v.y / rescale, v.z / rescale, v.w / rescale);
                    if (x_in != nullptr) v = add4(v, ld4(x_in + n * 9LL * channels + L * channels + c0));
                }
                st4(o + L * channels, v);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// gather + rotate backward (per edge): g_src, g_tgt, grad_wig, grad_radial
// ---------------------------------------------------------------------------------------------
template <bool HAS_RAD, int HALVES = 2>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp)
    gather_rotate_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ x, const int32_t* __restrict__ src,
                             const int32_t* __restrict__ tgt, const float* __restrict__ wig, const float* __restrict__ radial,
                             float* __restrict__ g_src, float* __restrict__ g_tgt, float* __restrict__ grad_wig,
                             float* __restrict__ grad_radial, int64_t num_edges, int channels) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    const int64_t node_stride = 9LL * channels;
    // row order that finishes each shared radial slot right after its second row
    constexpr int order[9] = {0, 1, 2, 3, 5, 4, 6, 7, 8};
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        float w[FCB200_WIG], dw[FCB200_WIG];
        load_wig(wig, e, lane, w);
#pragma unroll
        for (int i = 0; i < FCB200_WIG; ++i) dw[i] = 0.f;
#pragma unroll
        for (int half = 0; half < HALVES; ++half) {
            const int64_t node = half == 0 ? src[e] : tgt[e];
            const float* x_base = x + node * node_stride;
            float* g_base = (half == 0 ? g_src : g_tgt) + e * node_stride;
            for (int c0 = lane * 4; c0 < channels; c0 += 128) {
                float4 xv[9], g[9];
#pragma unroll
                for (int L = 0; L < 9; ++L) {
                    xv[L] = ld4(x_base + L * channels + c0);
                    g[L] = f4zero();
                }
                float4 pend = f4zero();
#pragma unroll
                for (int k = 0; k < 9; ++k) {
                    const int m = order[k];
                    const int L = m2l(m);
                    const int l = deg_of(L);
                    float4 go = ld4(edge_row(grad_out, e, m, 2 * channels) + half * channels + c0);
                    if (HAS_RAD) {
                        float4 rot = f4zero();
#pragma unroll
                        for (int b = 0; b < 5; ++b)
                            if (b < 2 * l + 1) rot = fma4(w[wix(L, l * l + b)], xv[l * l + b], rot);
                        const int64_t roff = e * 12LL * channels + radslot(m) * 2 * channels + half * channels + c0;
                        float4 contrib = mul4(go, rot);
                        if (m < 3) {
                            st4(grad_radial + roff, contrib);
                        } else if (m == 3 || m == 4 || m == 7) {
                            pend = contrib;
                        } else {
                            st4(grad_radial + roff, add4(pend, contrib));
                        }
                        go = mul4(go, ld4(radial + roff));
                    }
#pragma unroll
                    for (int b = 0; b < 5; ++b) {
                        if (b < 2 * l + 1) {
                            const int idx = wix(L, l * l + b);
                            g[l * l + b] = fma4(w[idx], go, g[l * l + b]);
                            dw[idx] += dot4(go, xv[l * l + b]);
                        }
                    }
                }
#pragma unroll
                for (int L = 0; L < 9; ++L) st4(g_base + L * channels + c0, g[L]);
            }
        }
        float mine, mine2;
        warp_reduce_wig(dw, lane, mine, mine2);
        grad_wig[e * FCB200_WIG + lane] = mine;
        if (lane < FCB200_WIG - 32) grad_wig[e * FCB200_WIG + 32 + lane] = mine2;
    }
}

// ---- gather + rotate backward, one degree at a time ------------------------------------------------------------
// Working through the block-diagonal rotation degree by degree keeps at most the l = 2 block alive (25 Wigner entries,
// 25 gradient sums, 5 node rows, 5 gradient rows: ~90 registers instead of ~180), so two blocks share an SM.
template <int N, bool ACC>
__device__ __forceinline__ void reduce_block(const float (&v)[N], int lane, float* __restrict__ out) {
    if (N == 1) {
        const float t = warp_sum(v[0]);
        if (lane == 0) out[0] = ACC ? out[0] + t : t;
        return;
    }
    float t[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) t[i] = i < N ? v[i] : 0.f;
#pragma unroll
    for (int h = 16; h >= 1; h >>= 1) {
        const bool upper = (lane & h) != 0;
#pragma unroll
        for (int i = 0; i < h; ++i) {
            const float a = t[i], b = t[i + h];
            t[i] = (upper ? b : a) + __shfl_xor_sync(kFull, upper ? a : b, h);
        }
    }
    if (lane < N) out[lane] = ACC ? out[lane] + t[0] : t[0];
}

// M-major rows of degree l in the order that finishes a shared radial slot right after its second row
template <int l> struct DegRows;
template <> struct DegRows<0> { static constexpr int n = 1; __device__ static constexpr int row(int i) { return 0; } };
template <> struct DegRows<1> { static constexpr int n = 3; __device__ static constexpr int row(int i) { constexpr int t[3] = {1, 3, 5}; return t[i]; } };
template <> struct DegRows<2> { static constexpr int n = 5; __device__ static constexpr int row(int i) { constexpr int t[5] = {2, 4, 6, 7, 8}; return t[i]; } };

// One edge, one half (source or target columns), one degree: g[b] += W^T grad rows, dw += grad (x) x, radial gradient.
// RadOut: OutF32 or OutSplit for the radial gradient (it only feeds the radial MLP's backward contraction)
template <int l, bool HAS_RAD, class RadOut>
__device__ __forceinline__ void bwd_degree_rows(const float* __restrict__ grad_out, const float* __restrict__ radial,
                                                const RadOut& grad_radial, int64_t e, int half, int channels, int c0,
                                                const float (&w)[(2 * l + 1) * (2 * l + 1)], const float4 (&xv)[2 * l + 1],
                                                float4 (&g)[2 * l + 1], float (&dw)[(2 * l + 1) * (2 * l + 1)]) {
    constexpr int n = 2 * l + 1;
    float4 pend = f4zero();
#pragma unroll
    for (int i = 0; i < DegRows<l>::n; ++i) {
        const int m = DegRows<l>::row(i);
        const int r = m2l(m) - l * l;  // row of the block
        float4 go = ld4(edge_row(grad_out, e, m, 2 * channels) + half * channels + c0);
        if (HAS_RAD) {
            float4 rot = f4zero();
#pragma unroll
            for (int b = 0; b < n; ++b) rot = fma4(w[r * n + b], xv[b], rot);
            const int64_t roff = e * 12LL * channels + radslot(m) * 2 * channels + half * channels + c0;
            const float4 contrib = mul4(go, rot);
            if (m < 3) {
                grad_radial.st(roff, contrib);
            } else if (m == 3 || m == 4 || m == 7) {
                pend = contrib;
            } else {
                grad_radial.st(roff, add4(pend, contrib));
            }
            go = mul4(go, ld4(radial + roff));
        }
#pragma unroll
        for (int b = 0; b < n; ++b) {
            g[b] = fma4(w[r * n + b], go, g[b]);
            dw[r * n + b] += dot4(go, xv[b]);
        }
    }
}

// source half, one warp per edge
template <int l, bool HAS_RAD, class RadOut>
__device__ __forceinline__ void bwd_src_degree(const float* __restrict__ grad_out, const float* __restrict__ x_base,
                                               const float* __restrict__ wig_e, const float* __restrict__ radial,
                                               float* __restrict__ g_base, float* __restrict__ grad_wig_e,
                                               const RadOut& grad_radial, int64_t e, int lane, int channels) {
    constexpr int n = 2 * l + 1, L0 = l * l;
    float w[n * n], dw[n * n];
#pragma unroll
    for (int i = 0; i < n * n; ++i) {
        w[i] = __ldg(wig_e + woff(l) + i);
        dw[i] = 0.f;
    }
    for (int c0 = lane * 4; c0 < channels; c0 += 128) {
        float4 xv[n], g[n];
#pragma unroll
        for (int b = 0; b < n; ++b) {
            xv[b] = ld4(x_base + (L0 + b) * channels + c0);
            g[b] = f4zero();
        }
        bwd_degree_rows<l, HAS_RAD, RadOut>(grad_out, radial, grad_radial, e, 0, channels, c0, w, xv, g, dw);
#pragma unroll
        for (int b = 0; b < n; ++b) st4(g_base + (L0 + b) * channels + c0, g[b]);
    }
    reduce_block<n * n, false>(dw, lane, grad_wig_e + woff(l));
}

template <bool HAS_RAD, class RadOut>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, 2)
    gather_rotate_bwd_src_kernel(const float* __restrict__ grad_out, const float* __restrict__ x, const int32_t* __restrict__ src,
                                 const float* __restrict__ wig, const float* __restrict__ radial, float* __restrict__ g_src,
                                 float* __restrict__ grad_wig, RadOut grad_radial, const float* __restrict__ scale_ptr,
                                 int64_t num_edges, int channels) {
    grad_radial.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    const int64_t node_stride = 9LL * channels;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        const float* x_base = x + (int64_t)src[e] * node_stride;
        float* g_base = g_src + e * node_stride;
        const float* wig_e = wig + e * FCB200_WIG;
        float* gw = grad_wig + e * FCB200_WIG;
        bwd_src_degree<0, HAS_RAD, RadOut>(grad_out, x_base, wig_e, radial, g_base, gw, grad_radial, e, lane, channels);
        bwd_src_degree<1, HAS_RAD, RadOut>(grad_out, x_base, wig_e, radial, g_base, gw, grad_radial, e, lane, channels);
        bwd_src_degree<2, HAS_RAD, RadOut>(grad_out, x_base, wig_e, radial, g_base, gw, grad_radial, e, lane, channels);
    }
}

// One half (HALF 0 = source columns, 1 = target columns), one warp per node and degree (128 channels): the node
// gradient of the degree's rows is summed over the node's edges in registers and added to the node rows once.  The
// edges of a target are consecutive (PERM = false, edges [eb, ee)); the edges of a source come through the by-source
// permutation of the chunk's edges (PERM = true, edges perm[eb .. ee)).  ACC_W: add the Wigner gradient to what the
// other half stored, else store it.
template <int l, bool HAS_RAD, class RadOut, int HALF, bool ACC_W, bool PERM>
__device__ __forceinline__ void bwd_node_degree(const float* __restrict__ grad_out, const float* __restrict__ x_base,
                                                const float* __restrict__ wig, const float* __restrict__ radial,
                                                float* __restrict__ g_base, float* __restrict__ grad_wig,
                                                const RadOut& grad_radial, const int32_t* __restrict__ perm, int eb, int ee,
                                                int lane) {
    constexpr int n = 2 * l + 1, L0 = l * l, channels = 128;
    const int c0 = lane * 4;
    float4 xv[n], gt[n];
#pragma unroll
    for (int b = 0; b < n; ++b) {
        xv[b] = ld4(x_base + (L0 + b) * channels + c0);
        gt[b] = f4zero();
    }
    for (int k = eb; k < ee; ++k) {
        const int64_t e = PERM ? (int64_t)__ldg(perm + k) : (int64_t)k;
        float w[n * n], dw[n * n];
#pragma unroll
        for (int i = 0; i < n * n; ++i) {
            w[i] = __ldg(wig + e * FCB200_WIG + woff(l) + i);
            dw[i] = 0.f;
        }
        bwd_degree_rows<l, HAS_RAD, RadOut>(grad_out, radial, grad_radial, e, HALF, channels, c0, w, xv, gt, dw);
        reduce_block<n * n, ACC_W>(dw, lane, grad_wig + e * FCB200_WIG + woff(l));
    }
#pragma unroll
    for (int b = 0; b < n; ++b) st4(g_base + (L0 + b) * channels + c0, add4(ld4(g_base + (L0 + b) * channels + c0), gt[b]));
}

// Degrees 0 and 1 of one node in a single pass over its edges: together they hold fewer registers than the l = 2 block
// alone, and one pass with four rows in flight per edge hides the latency of the per-edge loads better than two passes
// with one and three.
template <bool HAS_RAD, class RadOut, int HALF, bool ACC_W, bool PERM>
__device__ __forceinline__ void bwd_node_degrees01(const float* __restrict__ grad_out, const float* __restrict__ x_base,
                                                   const float* __restrict__ wig, const float* __restrict__ radial,
                                                   float* __restrict__ g_base, float* __restrict__ grad_wig,
                                                   const RadOut& grad_radial, const int32_t* __restrict__ perm, int eb, int ee,
                                                   int lane) {
    constexpr int channels = 128;
    const int c0 = lane * 4;
    float4 xv0[1], gt0[1], xv1[3], gt1[3];
    xv0[0] = ld4(x_base + c0);
    gt0[0] = f4zero();
#pragma unroll
    for (int b = 0; b < 3; ++b) {
        xv1[b] = ld4(x_base + (1 + b) * channels + c0);
        gt1[b] = f4zero();
    }
    for (int k = eb; k < ee; ++k) {
        const int64_t e = PERM ? (int64_t)__ldg(perm + k) : (int64_t)k;
        float w0[1], dw0[1], w1[9], dw1[9];
        w0[0] = __ldg(wig + e * FCB200_WIG + woff(0));
        dw0[0] = 0.f;
#pragma unroll
        for (int i = 0; i < 9; ++i) {
            w1[i] = __ldg(wig + e * FCB200_WIG + woff(1) + i);
            dw1[i] = 0.f;
        }
        bwd_degree_rows<0, HAS_RAD, RadOut>(grad_out, radial, grad_radial, e, HALF, channels, c0, w0, xv0, gt0, dw0);
        bwd_degree_rows<1, HAS_RAD, RadOut>(grad_out, radial, grad_radial, e, HALF, channels, c0, w1, xv1, gt1, dw1);
        reduce_block<1, ACC_W>(dw0, lane, grad_wig + e * FCB200_WIG + woff(0));
        reduce_block<9, ACC_W>(dw1, lane, grad_wig + e * FCB200_WIG + woff(1));
    }
    st4(g_base + c0, add4(ld4(g_base + c0), gt0[0]));
#pragma unroll
    for (int b = 0; b < 3; ++b) st4(g_base + (1 + b) * channels + c0, add4(ld4(g_base + (1 + b) * channels + c0), gt1[b]));
}

template <bool HAS_RAD, class RadOut>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, 2)
    gather_rotate_bwd_tgt_kernel(const float* __restrict__ grad_out, const float* __restrict__ x, const int32_t* __restrict__ row_ptr,
                                  int64_t tgt_base, const float* __restrict__ wig, const float* __restrict__ radial,
                                  float* __restrict__ gx_tgt, float* __restrict__ grad_wig, RadOut grad_radial,
                                  const float* __restrict__ scale_ptr, int64_t num_targets) {
    grad_radial.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t n = warp0; n < num_targets; n += nwarps) {
        const int eb = row_ptr[n], ee = row_ptr[n + 1];
        if (eb == ee) continue;
        const float* x_base = x + (tgt_base + n) * 9LL * 128;
        float* g_base = gx_tgt + n * 9LL * 128;
        bwd_node_degrees01<HAS_RAD, RadOut, 1, true, false>(grad_out, x_base, wig, radial, g_base, grad_wig, grad_radial, nullptr, eb, ee, lane);
        bwd_node_degree<2, HAS_RAD, RadOut, 1, true, false>(grad_out, x_base, wig, radial, g_base, grad_wig, grad_radial, nullptr, eb, ee, lane);
    }
}

// source half summed per source node: one warp per distinct source of the chunk, its edges through the by-source
// permutation.  Stores the Wigner gradient (runs before the target kernel, which adds to it) and adds the node
// gradient to gx[src_nodes[u]]; distinct sources are distinct rows, so no two warps touch the same row.
template <bool HAS_RAD, class RadOut>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, 2)
    gather_rotate_bwd_srcnode_kernel(const float* __restrict__ grad_out, const float* __restrict__ x,
                                     const int32_t* __restrict__ src_nodes, const int32_t* __restrict__ src_ptr,
                                     const int32_t* __restrict__ src_perm, const float* __restrict__ wig,
                                     const float* __restrict__ radial, float* __restrict__ gx, float* __restrict__ grad_wig,
                                     RadOut grad_radial, const float* __restrict__ scale_ptr, int64_t num_sources) {
    grad_radial.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t u = warp0; u < num_sources; u += nwarps) {
        const int eb = src_ptr[u], ee = src_ptr[u + 1];
        if (eb == ee) continue;
        const int64_t node = src_nodes[u];
        const float* x_base = x + node * 9LL * 128;
        float* g_base = gx + node * 9LL * 128;
        bwd_node_degrees01<HAS_RAD, RadOut, 0, false, true>(grad_out, x_base, wig, radial, g_base, grad_wig, grad_radial, src_perm, eb, ee, lane);
        bwd_node_degree<2, HAS_RAD, RadOut, 0, false, true>(grad_out, x_base, wig, radial, g_base, grad_wig, grad_radial, src_perm, eb, ee, lane);
    }
}

// rotate-back backward with the Wigner gradient, one degree at a time (see the gather backward above): the l = 2 block
// needs 25 + 25 entries, 5 gradient rows and 5 message rows, so two blocks share an SM
template <int l, class Out>
__device__ __forceinline__ void rotate_back_bwd_degree(const float* __restrict__ go_base, const float* __restrict__ msg_e,
                                                       const float* __restrict__ winv_e, Out& grad_msg, int64_t out_base,
                                                       float* __restrict__ grad_winv_e, int lane, int channels) {
    constexpr int n = 2 * l + 1, L0 = l * l;
    float w[n * n], dw[n * n];
#pragma unroll
    for (int i = 0; i < n * n; ++i) {
        w[i] = __ldg(winv_e + woff(l) + i);
        dw[i] = 0.f;
    }
    for (int c0 = lane * 4; c0 < channels; c0 += 128) {
        float4 go[n];
#pragma unroll
        for (int a = 0; a < n; ++a) go[a] = ld4(go_base + (L0 + a) * channels + c0);
#pragma unroll
        for (int i = 0; i < DegRows<l>::n; ++i) {
            const int m = DegRows<l>::row(i);
            const int col = m2l(m) - L0;  // column of the block
            const float4 y = ld4(msg_e + m * channels + c0);
            float4 acc = f4zero();
#pragma unroll
            for (int a = 0; a < n; ++a) {
                acc = fma4(w[a * n + col], go[a], acc);
                dw[a * n + col] += dot4(go[a], y);
            }
            grad_msg.st(out_base + m * channels + c0, acc);
        }
    }
    reduce_block<n * n, false>(dw, lane, grad_winv_e + woff(l));
}

template <class Out>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, 2)
    rotate_back_bwd_deg_kernel(const float* __restrict__ grad_out, const float* __restrict__ msg, const float* __restrict__ winv,
                               const int32_t* __restrict__ tgt, Out grad_msg, const float* __restrict__ scale_ptr,
                               float* __restrict__ grad_winv, int64_t num_edges, int channels) {
    grad_msg.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        const float* go_base = grad_out + (int64_t)tgt[e] * 9LL * channels;
        const float* msg_e = msg + e * 9LL * channels;
        const float* winv_e = winv + e * FCB200_WIG;
        float* gw = grad_winv + e * FCB200_WIG;
        rotate_back_bwd_degree<0>(go_base, msg_e, winv_e, grad_msg, e * 9LL * channels, gw, lane, channels);
        rotate_back_bwd_degree<1>(go_base, msg_e, winv_e, grad_msg, e * 9LL * channels, gw, lane, channels);
        rotate_back_bwd_degree<2>(go_base, msg_e, winv_e, grad_msg, e * 9LL * channels, gw, lane, channels);
    }
}

// ---------------------------------------------------------------------------------------------
// rotate back backward (per edge): grad_msg (M-major) and grad_winv
// ---------------------------------------------------------------------------------------------
// MODE 0: full messages.  MODE 1: edge-degree (3 rows), with 1/rescale.
template <int MODE, bool WANT_DW, class Out>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp)
    rotate_back_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ msg, const float* __restrict__ winv,
                           const int32_t* __restrict__ tgt, Out grad_msg, const float* __restrict__ scale_ptr,
                           float* __restrict__ grad_winv, float rescale, int64_t num_edges, int channels) {
    grad_msg.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    const int rows_in = MODE == 0 ? 9 : 3;
    const float inv = MODE == 1 ? 1.0f / rescale : 1.0f;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        float w[FCB200_WIG], dw[FCB200_WIG];
        load_wig(winv, e, lane, w);
#pragma unroll
        for (int i = 0; i < FCB200_WIG; ++i) dw[i] = 0.f;
        const float* go_base = grad_out + (int64_t)tgt[e] * 9LL * channels;
        for (int c0 = lane * 4; c0 < channels; c0 += 128) {
            float4 go[9];
#pragma unroll
            for (int L = 0; L < 9; ++L) go[L] = ld4(go_base + L * channels + c0);
            if (MODE == 0) {
                float4 y[9];
                if (WANT_DW) {
#pragma unroll
                    for (int m = 0; m < 9; ++m) y[m] = ld4(msg + e * 9LL * channels + m * channels + c0);
                }
#pragma unroll
                for (int m = 0; m < 9; ++m) {
                    const int K = m2l(m);  // column of Winv
                    const int l = deg_of(K);
                    float4 acc = f4zero();
#pragma unroll
                    for (int a = 0; a < 5; ++a) {
                        if (a < 2 * l + 1) {
                            const int idx = wix(l * l + a, K);
                            acc = fma4(w[idx], go[l * l + a], acc);
                            if (WANT_DW) dw[idx] += dot4(go[l * l + a], y[m]);
                        }
                    }
                    grad_msg.st(e * 9LL * channels + m * channels + c0, acc);
                }
            } else {
#pragma unroll
                for (int l = 0; l < 3; ++l) {
                    const int K = l * l + l;
                    float4 y = f4zero();
                    if (WANT_DW) y = ld4(msg + e * 3LL * channels + l * channels + c0);
                    float4 acc = f4zero();
#pragma unroll
                    for (int a = 0; a < 5; ++a) {
                        if (a < 2 * l + 1) {
                            const int idx = wix(l * l + a, K);
                            acc = fma4(w[idx], go[l * l + a], acc);
                            if (WANT_DW) dw[idx] += dot4(go[l * l + a], y);
                        }
                    }
                    grad_msg.st(e * 3LL * channels + l * channels + c0, scale4(inv, acc));
                }
            }
        }
        (void)rows_in;
        if (WANT_DW) {
            float mine, mine2;
            warp_reduce_wig(dw, lane, mine, mine2);
            mine *= inv;
            mine2 *= inv;
            grad_winv[e * FCB200_WIG + lane] = mine;
            if (lane < FCB200_WIG - 32) grad_winv[e * FCB200_WIG + 32 + lane] = mine2;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// segmented sum of rows
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp)
    segment_sum_vec_kernel(const float* __restrict__ rows, const int32_t* __restrict__ ptr, const int32_t* __restrict__ perm,
                           const int32_t* __restrict__ out_index, float* __restrict__ out, int accumulate, float scale,
                           int64_t num_segments, int64_t width) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t n = warp0; n < num_segments; n += nwarps) {
        const int k0 = ptr[n], k1 = ptr[n + 1];
        for (int64_t c0 = lane * 4; c0 < width; c0 += 128 * 3) {
            // three float4 per lane per pass (width 1152 = 9*128 is covered in exactly three passes)
            float4 a0 = f4zero(), a1 = f4zero(), a2 = f4zero();
            const bool h1 = c0 + 128 < width, h2 = c0 + 256 < width;
            for (int k = k0; k < k1; ++k) {
                const int64_t r = perm ? perm[k] : k;
                const float* p = rows + r * width + c0;
                a0 = add4(a0, ld4(p));
                if (h1) a1 = add4(a1, ld4(p + 128));
                if (h2) a2 = add4(a2, ld4(p + 256));
            }
            float* o = out + (out_index ? (int64_t)out_index[n] : n) * width + c0;
            a0 = scale4(scale, a0); a1 = scale4(scale, a1); a2 = scale4(scale, a2);
            if (accumulate) {
                a0 = add4(a0, ld4(o));
                if (h1) a1 = add4(a1, ld4(o + 128));
                if (h2) a2 = add4(a2, ld4(o + 256));
            }
            st4(o, a0);
            if (h1) st4(o + 128, a1);
            if (h2) st4(o + 256, a2);
        }
    }
}

__global__ void segment_sum_scalar_kernel(const float* __restrict__ rows, const int32_t* __restrict__ ptr,
                                          const int32_t* __restrict__ perm, const int32_t* __restrict__ out_index,
                                          float* __restrict__ out, int accumulate, float scale, int64_t num_segments,
                                          int64_t width) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_segments * width) return;
    const int64_t n = i / width, c = i % width;
    float acc = 0.f;
    for (int k = ptr[n]; k < ptr[n + 1]; ++k) acc += rows[(int64_t)(perm ? perm[k] : k) * width + c];
    const int64_t o = (out_index ? (int64_t)out_index[n] : n) * width + c;
    out[o] = accumulate ? out[o] + scale * acc : scale * acc;
}

// ---------------------------------------------------------------------------------------------
// gate activation between the two SO(2) convolutions
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoid_acc(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float4 sig4(float4 v) {
    return make_float4(sigmoid_acc(v.x), sigmoid_acc(v.y), sigmoid_acc(v.z), sigmoid_acc(v.w));
}
// gate index (0: l=1 gate, 1: l=2 gate) of M-major rows 1..8: [l1,l2 | l1,l2 | l1,l2 | l2 | l2]
__host__ __device__ constexpr int gate_of(int m) {
    constexpr int t[9] = {0, 0, 1, 0, 1, 0, 1, 1, 1};
    return t[m];
}

// y [E, 11H] = [gate scalars 2H | rows 0..8 (9H)] (the three conv-1 GEMMs write it side by side);
// out [E, 9, H]: row 0 -> SiLU, rows 1..8 -> value * sigmoid(gate of the row's degree).
template <class Out>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, 3)
    so2_gate_fwd_kernel(const float* __restrict__ y, Out out, const float* __restrict__ scale_ptr, int64_t num_edges, int ch) {
    out.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        const float* p = y + e * 11LL * ch;
        const int64_t o = e * 9LL * ch;
        for (int c = lane * 4; c < ch; c += 128) {
            float4 gate[2] = {sig4(ld4(p + c)), sig4(ld4(p + ch + c))};
            const float4 v0 = ld4(p + 2 * ch + c);
            out.st(o + c, mul4(v0, sig4(v0)));
#pragma unroll
            for (int m = 1; m < 9; ++m) out.st(o + m * ch + c, mul4(ld4(p + (2 + m) * ch + c), gate[gate_of(m)]));
        }
    }
}

template <class Out>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, 3)
    so2_gate_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ y, Out grad_y,
                        const float* __restrict__ scale_ptr, int64_t num_edges, int ch) {
    grad_y.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        const float* p = y + e * 11LL * ch;
        const float* go = grad_out + e * 9LL * ch;
        const int64_t q = e * 11LL * ch;
        for (int c = lane * 4; c < ch; c += 128) {
            const float4 gate[2] = {sig4(ld4(p + c)), sig4(ld4(p + ch + c))};
            float4 dgate[2] = {f4zero(), f4zero()};
            {
                const float4 v = ld4(p + 2 * ch + c), s = sig4(v), d = ld4(go + c);
                grad_y.st(q + 2 * ch + c, make_float4(d.x * s.x * (1.f + v.x * (1.f - s.x)), d.y * s.y * (1.f + v.y * (1.f - s.y)),
                                                      d.z * s.z * (1.f + v.z * (1.f - s.z)), d.w * s.w * (1.f + v.w * (1.f - s.w))));
            }
#pragma unroll
            for (int m = 1; m < 9; ++m) {
                const float4 d = ld4(go + m * ch + c);
                grad_y.st(q + (2 + m) * ch + c, mul4(d, gate[gate_of(m)]));
                dgate[gate_of(m)] = add4(dgate[gate_of(m)], mul4(d, ld4(p + (2 + m) * ch + c)));
            }
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const float4 s = gate[g], d = dgate[g];
                grad_y.st(q + g * ch + c, make_float4(d.x * s.x * (1.f - s.x), d.y * s.y * (1.f - s.y), d.z * s.z * (1.f - s.z), d.w * s.w * (1.f - s.w)));
            }
        }
    }
}

static int check_common(const void* a, const void* b, int64_t n, int32_t channels) {
    if (a == nullptr || b == nullptr || n < 0) return FCB200_EINVAL;
    if (channels <= 0 || channels % 128 != 0) return FCB200_EINVAL;
    if (!aligned16(a) || !aligned16(b)) return FCB200_EALIGN;
    return FCB200_OK;
}

}  // namespace fcb200

using namespace fcb200;

extern "C" {

int fcb200_version(void) { return 1000; }

#define FCB_STREAM static_cast<cudaStream_t>(stream)
#define FCB_LAUNCH(items) warp_grid(items, kWarpsPerBlock), kWarpsPerBlock * kWarp, 0, FCB_STREAM

int fcb200_gather_rotate_fwd(const float* x, const int32_t* src, const int32_t* tgt, const float* wig, const float* radial,
                             float* out, int64_t num_edges, int64_t num_nodes, int32_t channels, void* stream) {
    int rc = check_common(x, out, num_edges, channels);
    if (rc) return rc;
    if (!src || !tgt || !wig || num_nodes < 0) return FCB200_EINVAL;
    if (radial && !aligned16(radial)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    if (radial)
        gather_rotate_fwd_kernel<true, OutF32><<<FCB_LAUNCH(num_edges)>>>(x, src, tgt, wig, radial, OutF32{out}, nullptr, num_edges, channels);
    else
        gather_rotate_fwd_kernel<false, OutF32><<<FCB_LAUNCH(num_edges)>>>(x, src, tgt, wig, nullptr, OutF32{out}, nullptr, num_edges, channels);
    return launch_status();
}

int fcb200_rotate_back_reduce_fwd(const float* msg, const float* winv, const int32_t* row_ptr, float* out, int64_t num_edges,
                                  int64_t num_nodes, int32_t channels, void* stream) {
    if (num_nodes == 0) return FCB200_OK;
    if (!out || !row_ptr || num_edges < 0 || num_nodes < 0 || channels <= 0 || channels % 128) return FCB200_EINVAL;
    if (num_edges > 0 && (!msg || !winv)) return FCB200_EINVAL;
    if (!aligned16(out) || (msg && !aligned16(msg))) return FCB200_EALIGN;
    rotate_back_reduce_kernel<0><<<FCB_LAUNCH(num_nodes)>>>(msg, winv, row_ptr, nullptr, out, 1.0f, num_nodes, channels);
    return launch_status();
}

int fcb200_edge_degree_fwd(const float* radial3, const float* winv, const int32_t* row_ptr, const float* x_in, float* out,
                           float rescale, int64_t num_edges, int64_t num_nodes, int32_t channels, void* stream) {
    if (num_nodes == 0) return FCB200_OK;
    if (!out || !row_ptr || num_edges < 0 || num_nodes < 0 || channels <= 0 || channels % 128 || rescale == 0.f)
        return FCB200_EINVAL;
    if (num_edges > 0 && (!radial3 || !winv)) return FCB200_EINVAL;
    if (!aligned16(out) || (radial3 && !aligned16(radial3)) || (x_in && !aligned16(x_in))) return FCB200_EALIGN;
    rotate_back_reduce_kernel<1><<<FCB_LAUNCH(num_nodes)>>>(radial3, winv, row_ptr, x_in, out, rescale, num_nodes, channels);
    return launch_status();
}

int fcb200_gather_rotate_bwd(const float* grad_out, const float* x, const int32_t* src, const int32_t* tgt, const float* wig,
                             const float* radial, float* g_src, float* g_tgt, float* grad_wig, float* grad_radial,
                             int64_t num_edges, int64_t num_nodes, int32_t channels, void* stream) {
    int rc = check_common(grad_out, x, num_edges, channels);
    if (rc) return rc;
    if (!src || !tgt || !wig || !g_src || !g_tgt || !grad_wig || num_nodes < 0) return FCB200_EINVAL;
    if ((radial == nullptr) != (grad_radial == nullptr)) return FCB200_EINVAL;
    if (!aligned16(g_src) || !aligned16(g_tgt) || (radial && (!aligned16(radial) || !aligned16(grad_radial)))) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    if (radial)
        gather_rotate_bwd_kernel<true><<<FCB_LAUNCH(num_edges)>>>(grad_out, x, src, tgt, wig, radial, g_src, g_tgt, grad_wig,
                                                                  grad_radial, num_edges, channels);
    else
        gather_rotate_bwd_kernel<false><<<FCB_LAUNCH(num_edges)>>>(grad_out, x, src, tgt, wig, nullptr, g_src, g_tgt, grad_wig,
                                                                   nullptr, num_edges, channels);
    return launch_status();
}

int fcb200_gather_rotate_bwd_csr(const float* grad_out, const float* x, const int32_t* src, const int32_t* tgt,
                                 const int32_t* row_ptr, int64_t tgt_base, int64_t num_targets, const float* wig,
                                 const float* radial, float* g_src, float* gx_tgt, float* grad_wig, float* grad_radial,
                                 int64_t num_edges, int64_t num_nodes, int32_t channels, void* stream) {
    int rc = check_common(grad_out, x, num_edges, channels);
    if (rc) return rc;
    if (channels != 128) return FCB200_EINVAL;
    if (!src || !tgt || !row_ptr || !wig || !g_src || !gx_tgt || !grad_wig || num_nodes < 0 || num_targets < 0 || tgt_base < 0 ||
        tgt_base + num_targets > num_nodes)
        return FCB200_EINVAL;
    if ((radial == nullptr) != (grad_radial == nullptr)) return FCB200_EINVAL;
    if (!aligned16(g_src) || !aligned16(gx_tgt) || (radial && (!aligned16(radial) || !aligned16(grad_radial)))) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    cudaStream_t st = FCB_STREAM;
    const int tgrid = warp_grid(num_targets, kWarpsPerBlock);
    if (radial) {
        gather_rotate_bwd_src_kernel<true, OutF32><<<FCB_LAUNCH(num_edges)>>>(grad_out, x, src, wig, radial, g_src, grad_wig,
                                                                              OutF32{grad_radial}, nullptr, num_edges, channels);
        gather_rotate_bwd_tgt_kernel<true, OutF32><<<tgrid, kWarpsPerBlock * kWarp, 0, st>>>(
            grad_out, x, row_ptr, tgt_base, wig, radial, gx_tgt, grad_wig, OutF32{grad_radial}, nullptr, num_targets);
    } else {
        gather_rotate_bwd_src_kernel<false, OutF32><<<FCB_LAUNCH(num_edges)>>>(grad_out, x, src, wig, nullptr, g_src, grad_wig,
                                                                               OutF32{nullptr}, nullptr, num_edges, channels);
        gather_rotate_bwd_tgt_kernel<false, OutF32><<<tgrid, kWarpsPerBlock * kWarp, 0, st>>>(
            grad_out, x, row_ptr, tgt_base, wig, nullptr, gx_tgt, grad_wig, OutF32{nullptr}, nullptr, num_targets);
    }
    return launch_status();
}

int fcb200_gather_rotate_bwd_csr_h(const float* grad_out, const float* x, const int32_t* src, const int32_t* tgt,
                                   const int32_t* row_ptr, int64_t tgt_base, int64_t num_targets, const float* wig,
                                   const float* radial, float* g_src, float* gx_tgt, float* grad_wig, void* grad_radial_hi,
                                   void* grad_radial_lo, const float* scale, int64_t num_edges, int64_t num_nodes,
                                   int32_t channels, void* stream) {
    int rc = check_common(grad_out, x, num_edges, channels);
    if (rc) return rc;
    if (channels != 128) return FCB200_EINVAL;
    if (!src || !tgt || !row_ptr || !wig || !radial || !g_src || !gx_tgt || !grad_wig || !grad_radial_hi || !grad_radial_lo ||
        num_nodes < 0 || num_targets < 0 || tgt_base < 0 || tgt_base + num_targets > num_nodes)
        return FCB200_EINVAL;
    if (!aligned16(g_src) || !aligned16(gx_tgt) || !aligned16(radial) || !aligned8(grad_radial_hi) || !aligned8(grad_radial_lo))
        return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    cudaStream_t st = FCB_STREAM;
    const int tgrid = warp_grid(num_targets, kWarpsPerBlock);
    const OutSplit out{static_cast<__half*>(grad_radial_hi), static_cast<__half*>(grad_radial_lo), 1.0f};
    gather_rotate_bwd_src_kernel<true, OutSplit><<<FCB_LAUNCH(num_edges)>>>(grad_out, x, src, wig, radial, g_src, grad_wig, out, scale,
                                                                            num_edges, channels);
    gather_rotate_bwd_tgt_kernel<true, OutSplit><<<tgrid, kWarpsPerBlock * kWarp, 0, st>>>(grad_out, x, row_ptr, tgt_base, wig, radial,
                                                                                         gx_tgt, grad_wig, out, scale, num_targets);
    return launch_status();
}

int fcb200_gather_rotate_bwd_nodes(const float* grad_out, const float* x, const int32_t* src_nodes, const int32_t* src_ptr,
                                   const int32_t* src_perm, int64_t num_sources, const int32_t* row_ptr, int64_t tgt_base,
                                   int64_t num_targets, const float* wig, const float* radial, float* gx, float* grad_wig,
                                   float* grad_radial, int64_t num_edges, int64_t num_nodes, int32_t channels, void* stream) {
    int rc = check_common(grad_out, x, num_edges, channels);
    if (rc) return rc;
    if (channels != 128) return FCB200_EINVAL;
    if (!src_nodes || !src_ptr || !src_perm || !row_ptr || !wig || !gx || !grad_wig || num_nodes < 0 || num_targets < 0 ||
        num_sources < 0 || tgt_base < 0 || tgt_base + num_targets > num_nodes)
        return FCB200_EINVAL;
    if ((radial == nullptr) != (grad_radial == nullptr)) return FCB200_EINVAL;
    if (!aligned16(gx) || (radial && (!aligned16(radial) || !aligned16(grad_radial)))) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    cudaStream_t st = FCB_STREAM;
    const int sgrid = warp_grid(num_sources, kWarpsPerBlock), tgrid = warp_grid(num_targets, kWarpsPerBlock);
    float* gx_tgt = gx + tgt_base * 9LL * 128;
    if (radial) {
        gather_rotate_bwd_srcnode_kernel<true, OutF32><<<sgrid, kWarpsPerBlock * kWarp, 0, st>>>(
            grad_out, x, src_nodes, src_ptr, src_perm, wig, radial, gx, grad_wig, OutF32{grad_radial}, nullptr, num_sources);
        gather_rotate_bwd_tgt_kernel<true, OutF32><<<tgrid, kWarpsPerBlock * kWarp, 0, st>>>(
            grad_out, x, row_ptr, tgt_base, wig, radial, gx_tgt, grad_wig, OutF32{grad_radial}, nullptr, num_targets);
    } else {
        gather_rotate_bwd_srcnode_kernel<false, OutF32><<<sgrid, kWarpsPerBlock * kWarp, 0, st>>>(
            grad_out, x, src_nodes, src_ptr, src_perm, wig, nullptr, gx, grad_wig, OutF32{nullptr}, nullptr, num_sources);
        gather_rotate_bwd_tgt_kernel<false, OutF32><<<tgrid, kWarpsPerBlock * kWarp, 0, st>>>(
            grad_out, x, row_ptr, tgt_base, wig, nullptr, gx_tgt, grad_wig, OutF32{nullptr}, nullptr, num_targets);
    }
    return launch_status();
}

int fcb200_gather_rotate_bwd_nodes_h(const float* grad_out, const float* x, const int32_t* src_nodes, const int32_t* src_ptr,
                                     const int32_t* src_perm, int64_t num_sources, const int32_t* row_ptr, int64_t tgt_base,
                                     int64_t num_targets, const float* wig, const float* radial, float* gx, float* grad_wig,
                                     void* grad_radial_hi, void* grad_radial_lo, const float* scale, int64_t num_edges,
                                     int64_t num_nodes, int32_t channels, void* stream) {
    int rc = check_common(grad_out, x, num_edges, channels);
    if (rc) return rc;
    if (channels != 128) return FCB200_EINVAL;
    if (!src_nodes || !src_ptr || !src_perm || !row_ptr || !wig || !radial || !gx || !grad_wig || !grad_radial_hi ||
        !grad_radial_lo || num_nodes < 0 || num_targets < 0 || num_sources < 0 || tgt_base < 0 || tgt_base + num_targets > num_nodes)
        return FCB200_EINVAL;
    if (!aligned16(gx) || !aligned16(radial) || !aligned8(grad_radial_hi) || !aligned8(grad_radial_lo)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    cudaStream_t st = FCB_STREAM;
    const int sgrid = warp_grid(num_sources, kWarpsPerBlock), tgrid = warp_grid(num_targets, kWarpsPerBlock);
    const OutSplit out{static_cast<__half*>(grad_radial_hi), static_cast<__half*>(grad_radial_lo), 1.0f};
    gather_rotate_bwd_srcnode_kernel<true, OutSplit><<<sgrid, kWarpsPerBlock * kWarp, 0, st>>>(
        grad_out, x, src_nodes, src_ptr, src_perm, wig, radial, gx, grad_wig, out, scale, num_sources);
    gather_rotate_bwd_tgt_kernel<true, OutSplit><<<tgrid, kWarpsPerBlock * kWarp, 0, st>>>(
        grad_out, x, row_ptr, tgt_base, wig, radial, gx + tgt_base * 9LL * 128, grad_wig, out, scale, num_targets);
    return launch_status();
}

int fcb200_rotate_back_bwd(const float* grad_out, const float* msg, const float* winv, const int32_t* tgt, float* grad_msg,
                           float* grad_winv, int64_t num_edges, int64_t num_nodes, int32_t channels, void* stream) {
    int rc = check_common(grad_out, grad_msg, num_edges, channels);
    if (rc) return rc;
    if (!winv || !tgt || num_nodes < 0) return FCB200_EINVAL;
    if ((msg == nullptr) != (grad_winv == nullptr)) return FCB200_EINVAL;
    if (msg && !aligned16(msg)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    if (msg)
        rotate_back_bwd_deg_kernel<OutF32><<<FCB_LAUNCH(num_edges)>>>(grad_out, msg, winv, tgt, OutF32{grad_msg}, nullptr, grad_winv, num_edges, channels);
    else
        rotate_back_bwd_kernel<0, false, OutF32><<<FCB_LAUNCH(num_edges)>>>(grad_out, nullptr, winv, tgt, OutF32{grad_msg}, nullptr, nullptr, 1.f, num_edges,
                                                                    channels);
    return launch_status();
}

int fcb200_edge_degree_bwd(const float* grad_out, const float* radial3, const float* winv, const int32_t* tgt,
                           float* grad_radial3, float* grad_winv, float rescale, int64_t num_edges, int64_t num_nodes,
                           int32_t channels, void* stream) {
    int rc = check_common(grad_out, grad_radial3, num_edges, channels);
    if (rc) return rc;
    if (!radial3 || !winv || !tgt || !grad_winv || num_nodes < 0 || rescale == 0.f) return FCB200_EINVAL;
    if (!aligned16(radial3)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    rotate_back_bwd_kernel<1, true, OutF32><<<FCB_LAUNCH(num_edges)>>>(grad_out, radial3, winv, tgt, OutF32{grad_radial3}, nullptr, grad_winv, rescale,
                                                               num_edges, channels);
    return launch_status();
}

int fcb200_segment_sum(const float* rows, const int32_t* ptr, const int32_t* perm, const int32_t* out_index, float* out,
                       int32_t accumulate, float scale, int64_t num_segments, int64_t width, void* stream) {
    if (num_segments == 0) return FCB200_OK;
    if (!ptr || !out || num_segments < 0 || width <= 0) return FCB200_EINVAL;
    if (width % 4 == 0 && aligned16(rows) && aligned16(out)) {
        segment_sum_vec_kernel<<<FCB_LAUNCH(num_segments)>>>(rows, ptr, perm, out_index, out, accumulate, scale, num_segments, width);
    } else {
        const int64_t total = num_segments * width;
        segment_sum_scalar_kernel<<<(unsigned)((total + 255) / 256), 256, 0, FCB_STREAM>>>(rows, ptr, perm, out_index, out, accumulate,
                                                                                        scale, num_segments, width);
    }
    return launch_status();
}

int fcb200_so2_gate_fwd(const float* y, float* out, int64_t num_edges, int32_t hidden, void* stream) {
    int rc = check_common(y, out, num_edges, hidden);
    if (rc) return rc;
    if (num_edges == 0) return FCB200_OK;
    so2_gate_fwd_kernel<OutF32><<<FCB_LAUNCH(num_edges)>>>(y, OutF32{out}, nullptr, num_edges, hidden);
    return launch_status();
}

int fcb200_so2_gate_bwd(const float* grad_out, const float* y, float* grad_y, int64_t num_edges, int32_t hidden, void* stream) {
    int rc = check_common(grad_out, y, num_edges, hidden);
    if (rc) return rc;
    if (!grad_y) return FCB200_EINVAL;
    if (!aligned16(grad_y)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    so2_gate_bwd_kernel<OutF32><<<FCB_LAUNCH(num_edges)>>>(grad_out, y, OutF32{grad_y}, nullptr, num_edges, hidden);
    return launch_status();
}

// ---- the same four producers writing the half-precision split the tensor-core contraction reads directly ----

int fcb200_gather_rotate_fwd_h(const float* x, const int32_t* src, const int32_t* tgt, const float* wig, const float* radial,
                               void* out_hi, void* out_lo, const float* scale, int64_t num_edges, int64_t num_nodes,
                               int32_t channels, void* stream) {
    if (!x || !out_hi || !out_lo || !src || !tgt || !wig || num_edges < 0 || num_nodes < 0) return FCB200_EINVAL;
    if (channels <= 0 || channels % 128 != 0) return FCB200_EINVAL;
    if (!aligned16(x) || !aligned8(out_hi) || !aligned8(out_lo) || (radial && !aligned16(radial))) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    const OutSplit out{static_cast<__half*>(out_hi), static_cast<__half*>(out_lo), 1.0f};
    if (radial)
        gather_rotate_fwd_kernel<true, OutSplit><<<FCB_LAUNCH(num_edges)>>>(x, src, tgt, wig, radial, out, scale, num_edges, channels);
    else
        gather_rotate_fwd_kernel<false, OutSplit><<<FCB_LAUNCH(num_edges)>>>(x, src, tgt, wig, nullptr, out, scale, num_edges, channels);
    return launch_status();
}

int fcb200_rotate_back_bwd_h(const float* grad_out, const float* msg, const float* winv, const int32_t* tgt, void* grad_msg_hi,
                             void* grad_msg_lo, const float* scale, float* grad_winv, int64_t num_edges, int64_t num_nodes,
                             int32_t channels, void* stream) {
    if (!grad_out || !winv || !tgt || !grad_msg_hi || !grad_msg_lo || num_edges < 0 || num_nodes < 0) return FCB200_EINVAL;
    if (channels <= 0 || channels % 128 != 0) return FCB200_EINVAL;
    if ((grad_winv != nullptr) && (msg == nullptr)) return FCB200_EINVAL;
    if (!aligned16(grad_out) || !aligned8(grad_msg_hi) || !aligned8(grad_msg_lo) || (msg && !aligned16(msg))) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    const OutSplit out{static_cast<__half*>(grad_msg_hi), static_cast<__half*>(grad_msg_lo), 1.0f};
    if (grad_winv)
        rotate_back_bwd_deg_kernel<OutSplit><<<FCB_LAUNCH(num_edges)>>>(grad_out, msg, winv, tgt, out, scale, grad_winv, num_edges, channels);
    else
        rotate_back_bwd_kernel<0, false, OutSplit><<<FCB_LAUNCH(num_edges)>>>(grad_out, nullptr, winv, tgt, out, scale, nullptr, 1.f,
                                                                              num_edges, channels);
    return launch_status();
}

int fcb200_so2_gate_fwd_h(const float* y, void* out_hi, void* out_lo, const float* scale, int64_t num_edges, int32_t hidden,
                          void* stream) {
    if (!y || !out_hi || !out_lo || num_edges < 0 || hidden <= 0 || hidden % 128) return FCB200_EINVAL;
    if (!aligned16(y) || !aligned8(out_hi) || !aligned8(out_lo)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    so2_gate_fwd_kernel<OutSplit><<<FCB_LAUNCH(num_edges)>>>(
        y, OutSplit{static_cast<__half*>(out_hi), static_cast<__half*>(out_lo), 1.0f}, scale, num_edges, hidden);
    return launch_status();
}

int fcb200_so2_gate_bwd_h(const float* grad_out, const float* y, void* grad_y_hi, void* grad_y_lo, const float* scale,
                          int64_t num_edges, int32_t hidden, void* stream) {
    if (!grad_out || !y || !grad_y_hi || !grad_y_lo || num_edges < 0 || hidden <= 0 || hidden % 128) return FCB200_EINVAL;
    if (!aligned16(grad_out) || !aligned16(y) || !aligned8(grad_y_hi) || !aligned8(grad_y_lo)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    so2_gate_bwd_kernel<OutSplit><<<FCB_LAUNCH(num_edges)>>>(
        grad_out, y, OutSplit{static_cast<__half*>(grad_y_hi), static_cast<__half*>(grad_y_lo), 1.0f}, scale, num_edges, hidden);
    return launch_status();
}

}  // extern "C"
