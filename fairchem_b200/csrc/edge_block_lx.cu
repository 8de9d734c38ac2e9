// Edge-block kernels for any lmax with mmax = 2 (instantiated for lmax = 2 and 4), sm_100a.
//
// Same data flow as edge_block.cu (one warp per edge or per node, a lane owns a float4 of a
// 128-channel tile, segmented CSR reductions, no atomics) but written over compile-time shape tables
// and processed one degree l at a time, so the live register state stays bounded when a node has 25
// coefficient rows.  The Wigner entries of an edge (only the rows |m| <= 2 of every block are ever
// needed, 115 floats for lmax = 4) are staged in shared memory per warp and read as broadcasts.
//
// Layouts
//   node features   [N, (lmax+1)^2, C]  L-major
//   edge features   [E, NM, w]          M-major rows: m=0 (l=0..lmax) | m=+1 (l=1..) | m=-1 | m=+2 (l=2..) | m=-2
//   compact Wigner  [E, NW]             block l holds rows m = -mm..mm (mm = min(l,2)) x columns m' = -l..l of D^l
//   inverse         same layout as the compact Wigner, times the envelope (D is orthogonal: D^-1 = D^T)
#include <type_traits>

#include "common.cuh"
#include "shape_lx.cuh"

namespace fcb200 {

constexpr int kLxWarps = 4;
constexpr int kWigSlot = 128;  // floats of shared memory per warp for the staged Wigner entries

// copy the kW compact entries of edge e into this warp's shared-memory slot
template <int KW>
__device__ __forceinline__ void stage_wig(const float* __restrict__ wig, int64_t e, int lane, float* slot) {
    __syncwarp();
#pragma unroll
    for (int i = lane; i < KW; i += 32) slot[i] = wig[e * KW + i];
    __syncwarp();
}

// Warp-reduce the first rows(l) * (2l+1) entries of a per-lane block gradient and store them.  `l` is a compile-time
// constant at every call site (the degree loops are fully unrolled), so the switch folds away.
template <int LMAX, int KMAX>
__device__ __forceinline__ void reduce_block(const float (&dw)[KMAX], int l, int lane, float* __restrict__ out, float scale) {
    using S = Shape<LMAX>;
    auto run = [&](auto tag) {
        constexpr int n = decltype(tag)::value;
        float v[n];
#pragma unroll
        for (int i = 0; i < n; ++i) v[i] = dw[i];
        warp_reduce_store<n>(v, lane, out, scale);
    };
    switch (l) {
        case 0: run(std::integral_constant<int, S::rows(0) * 1>{}); break;
        case 1: run(std::integral_constant<int, S::rows(1) * 3>{}); break;
        case 2: run(std::integral_constant<int, S::rows(2) * 5>{}); break;
        case 3: if constexpr (LMAX >= 3) run(std::integral_constant<int, S::rows(3) * 7>{}); break;
        default: if constexpr (LMAX >= 4) run(std::integral_constant<int, S::rows(4) * 9>{}); break;
    }
}

// ---------------------------------------------------------------------------------------------
// gather + rotate (+ radial) forward: out[e, mrow(l,m), :] = rad * sum_j D[(l,m), j] * cat(x[src], x[tgt])[l^2 + j]
// ---------------------------------------------------------------------------------------------
template <int LMAX, bool HAS_RAD, class Out>
__global__ void __launch_bounds__(kLxWarps* kWarp)
    lx_gather_rotate_fwd_kernel(const float* __restrict__ x, const int32_t* __restrict__ src, const int32_t* __restrict__ tgt,
                                const float* __restrict__ wig, const float* __restrict__ radial, Out out,
                                const float* __restrict__ scale_ptr, int64_t num_edges, int channels) {
    using S = Shape<LMAX>;
    out.load_scale(scale_ptr);
    __shared__ float sw[kLxWarps][kWigSlot];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * kLxWarps + wid;
    const int64_t nwarps = (int64_t)gridDim.x * kLxWarps;
    float* w = sw[wid];
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        stage_wig<S::kW>(wig, e, lane, w);
        const float* xs_base = x + (int64_t)src[e] * S::kL * channels;
        const float* xt_base = x + (int64_t)tgt[e] * S::kL * channels;
        const int64_t o_base = e * (int64_t)S::kM * 2 * channels;
        const float* r_base = HAS_RAD ? radial + e * (int64_t)S::kRad * 2 * channels : nullptr;
        for (int c0 = lane * 4; c0 < channels; c0 += 128) {
#pragma unroll
            for (int l = 0; l <= LMAX; ++l) {
                float4 xs[2 * LMAX + 1], xt[2 * LMAX + 1];
#pragma unroll
                for (int j = 0; j < 2 * l + 1; ++j) {
                    xs[j] = ld4(xs_base + (l * l + j) * channels + c0);
                    xt[j] = ld4(xt_base + (l * l + j) * channels + c0);
                }
#pragma unroll
                for (int k = 0; k < S::rows(l); ++k) {
                    const int m = k - S::mm(l);
                    float4 as = f4zero(), at = f4zero();
#pragma unroll
                    for (int j = 0; j < 2 * l + 1; ++j) {
                        const float wv = w[S::woff(l) + k * (2 * l + 1) + j];
                        as = fma4(wv, xs[j], as);
                        at = fma4(wv, xt[j], at);
                    }
                    if (HAS_RAD) {
                        const float* r = r_base + S::radslot(l, m) * 2 * channels + c0;
                        as = mul4(as, ld4(r));
                        at = mul4(at, ld4(r + channels));
                    }
                    const int64_t o = o_base + S::mrow(l, m) * 2 * channels + c0;
                    out.st(o, as);
                    out.st(o + channels, at);
                }
            }
        }
    }
}

// backward per edge: g_src / g_tgt (L-major, before the node reduction), grad_wig, grad_radial
template <int LMAX, bool HAS_RAD>
__global__ void __launch_bounds__(kLxWarps* kWarp)
    lx_gather_rotate_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ x, const int32_t* __restrict__ src,
                                const int32_t* __restrict__ tgt, const float* __restrict__ wig, const float* __restrict__ radial,
                                float* __restrict__ g_src, float* __restrict__ g_tgt, float* __restrict__ grad_wig,
                                float* __restrict__ grad_radial, int64_t num_edges, int channels) {
    using S = Shape<LMAX>;
    __shared__ float sw[kLxWarps][kWigSlot];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * kLxWarps + wid;
    const int64_t nwarps = (int64_t)gridDim.x * kLxWarps;
    float* w = sw[wid];
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        stage_wig<S::kW>(wig, e, lane, w);
        const float* go_base = grad_out + e * (int64_t)S::kM * 2 * channels;
        const int64_t rad_base = e * (int64_t)S::kRad * 2 * channels;
#pragma unroll
        for (int l = 0; l <= LMAX; ++l) {
            float dw[5 * (2 * LMAX + 1)];
#pragma unroll
            for (int i = 0; i < S::rows(l) * (2 * l + 1); ++i) dw[i] = 0.f;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int64_t node = half == 0 ? src[e] : tgt[e];
                const float* x_base = x + node * S::kL * channels;
                float* g_base = (half == 0 ? g_src : g_tgt) + e * (int64_t)S::kL * channels;
                for (int c0 = lane * 4; c0 < channels; c0 += 128) {
                    float4 xv[2 * LMAX + 1], g[2 * LMAX + 1];
#pragma unroll
                    for (int j = 0; j < 2 * l + 1; ++j) {
                        xv[j] = ld4(x_base + (l * l + j) * channels + c0);
                        g[j] = f4zero();
                    }
                    float4 drad[3] = {f4zero(), f4zero(), f4zero()};  // per |m|
#pragma unroll
                    for (int k = 0; k < S::rows(l); ++k) {
                        const int m = k - S::mm(l);
                        const int am = m < 0 ? -m : m;
                        float4 go = ld4(go_base + S::mrow(l, m) * 2 * channels + half * channels + c0);
                        if (HAS_RAD) {
                            float4 rot = f4zero();
#pragma unroll
                            for (int j = 0; j < 2 * l + 1; ++j) rot = fma4(w[S::woff(l) + k * (2 * l + 1) + j], xv[j], rot);
                            drad[am] = add4(drad[am], mul4(go, rot));
                            go = mul4(go, ld4(radial + rad_base + S::radslot(l, m) * 2 * channels + half * channels + c0));
                        }
#pragma unroll
                        for (int j = 0; j < 2 * l + 1; ++j) {
                            g[j] = fma4(w[S::woff(l) + k * (2 * l + 1) + j], go, g[j]);
                            dw[k * (2 * l + 1) + j] += dot4(go, xv[j]);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 2 * l + 1; ++j) st4(g_base + (l * l + j) * channels + c0, g[j]);
                    if (HAS_RAD) {
#pragma unroll
                        for (int am = 0; am <= S::mm(l); ++am)
                            st4(grad_radial + rad_base + S::radslot(l, am) * 2 * channels + half * channels + c0, drad[am]);
                    }
                }
            }
            // entries past rows(l) * (2l+1) are zero and not stored
            reduce_block<LMAX>(dw, l, lane, grad_wig + e * S::kW + S::woff(l), 1.0f);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// rotate back + segmented reduce by target.  MODE 0: NM-row messages.  MODE 1: edge-degree embedding
// (lmax+1 rows, m = 0 only), out = x_in + sum / rescale.
// out[n, l^2 + j] = sum_e sum_k winv[e, (l,k,j)] * y[e, mrow(l, k - mm)]
// ---------------------------------------------------------------------------------------------
template <int LMAX, int MODE>
__global__ void __launch_bounds__(kLxWarps* kWarp)
    lx_rotate_back_reduce_kernel(const float* __restrict__ msg, const float* __restrict__ winv, const int32_t* __restrict__ row_ptr,
                                 const float* __restrict__ x_in, float* __restrict__ out, float rescale, int64_t num_nodes,
                                 int channels) {
    using S = Shape<LMAX>;
    __shared__ float sw[kLxWarps][kWigSlot];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * kLxWarps + wid;
    const int64_t nwarps = (int64_t)gridDim.x * kLxWarps;
    constexpr int rows_in = MODE == 0 ? S::kM : LMAX + 1;
    float* w = sw[wid];
    for (int64_t n = warp0; n < num_nodes; n += nwarps) {
        const int e0 = row_ptr[n], e1 = row_ptr[n + 1];
        for (int c0 = lane * 4; c0 < channels; c0 += 128) {
            float4 acc[S::kL];
#pragma unroll
            for (int L = 0; L < S::kL; ++L) acc[L] = f4zero();
            for (int e = e0; e < e1; ++e) {
                stage_wig<S::kW>(winv, e, lane, w);
                const float* y_base = msg + (int64_t)e * rows_in * channels + c0;
#pragma unroll
                for (int l = 0; l <= LMAX; ++l) {
                    if (MODE == 0) {
#pragma unroll
                        for (int k = 0; k < S::rows(l); ++k) {
                            const float4 y = ld4(y_base + S::mrow(l, k - S::mm(l)) * channels);
#pragma unroll
                            for (int j = 0; j < 2 * l + 1; ++j)
                                acc[l * l + j] = fma4(w[S::woff(l) + k * (2 * l + 1) + j], y, acc[l * l + j]);
                        }
                    } else {
                        const float4 y = ld4(y_base + l * channels);
#pragma unroll
                        for (int j = 0; j < 2 * l + 1; ++j)
                            acc[l * l + j] = fma4(w[S::woff(l) + S::mm(l) * (2 * l + 1) + j], y, acc[l * l + j]);
                    }
                }
            }
            float* o = out + n * (int64_t)S::kL * channels + c0;
#pragma unroll
            for (int L = 0; L < S::kL; ++L) {
                float4 v = acc[L];
                if (MODE == 1) {
                    v = make_float4(v.x / rescale, v.y / rescale, v.z / rescale, v.w / rescale);
                    if (x_in != nullptr) v = add4(v, ld4(x_in + n * (int64_t)S::kL * channels + L * channels + c0));
                }
                st4(o + L * channels, v);
            }
        }
    }
}

// backward per edge: grad_msg[e, mrow(l,m)] = sum_j winv[(l,k,j)] * go[tgt, l^2+j];  grad_winv[(l,k,j)] = <go[l^2+j], y[mrow]>
template <int LMAX, int MODE, bool WANT_DW, class Out>
__global__ void __launch_bounds__(kLxWarps* kWarp)
    lx_rotate_back_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ msg, const float* __restrict__ winv,
                              const int32_t* __restrict__ tgt, Out grad_msg, const float* __restrict__ scale_ptr,
                              float* __restrict__ grad_winv, float rescale, int64_t num_edges, int channels) {
    using S = Shape<LMAX>;
    grad_msg.load_scale(scale_ptr);
    __shared__ float sw[kLxWarps][kWigSlot];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * kLxWarps + wid;
    const int64_t nwarps = (int64_t)gridDim.x * kLxWarps;
    constexpr int rows_in = MODE == 0 ? S::kM : LMAX + 1;
    const float inv = MODE == 1 ? 1.0f / rescale : 1.0f;
    float* w = sw[wid];
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        stage_wig<S::kW>(winv, e, lane, w);
        const float* go_base = grad_out + (int64_t)tgt[e] * S::kL * channels;
        const float* y_base = msg + e * (int64_t)rows_in * channels;
        const int64_t gm_base = e * (int64_t)rows_in * channels;
#pragma unroll
        for (int l = 0; l <= LMAX; ++l) {
            constexpr int kmax = 5 * (2 * LMAX + 1);
            float dw[kmax];
#pragma unroll
            for (int i = 0; i < kmax; ++i) dw[i] = 0.f;
            for (int c0 = lane * 4; c0 < channels; c0 += 128) {
                float4 go[2 * LMAX + 1];
#pragma unroll
                for (int j = 0; j < 2 * l + 1; ++j) go[j] = ld4(go_base + (l * l + j) * channels + c0);
#pragma unroll
                for (int k = 0; k < S::rows(l); ++k) {
                    if (MODE == 1 && k != S::mm(l)) continue;
                    const int row = MODE == 0 ? S::mrow(l, k - S::mm(l)) : l;
                    float4 y = f4zero();
                    if (WANT_DW) y = ld4(y_base + row * channels + c0);
                    float4 acc = f4zero();
#pragma unroll
                    for (int j = 0; j < 2 * l + 1; ++j) {
                        acc = fma4(w[S::woff(l) + k * (2 * l + 1) + j], go[j], acc);
                        if (WANT_DW) dw[k * (2 * l + 1) + j] += dot4(go[j], y);
                    }
                    grad_msg.st(gm_base + row * channels + c0, scale4(inv, acc));
                }
            }
            if (WANT_DW) reduce_block<LMAX>(dw, l, lane, grad_winv + e * S::kW + S::woff(l), inv);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// gate activation between the two SO(2) convolutions
// y [E, (LMAX + NM) H] = [gate scalars LMAX*H | rows 0..NM-1]; out [E, NM, H]:
// row 0 -> SiLU, any other row (l, m) -> value * sigmoid(gate l-1)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float lx_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float4 lx_sig4(float4 v) {
    return make_float4(lx_sigmoid(v.x), lx_sigmoid(v.y), lx_sigmoid(v.z), lx_sigmoid(v.w));
}

template <int LMAX, class Out>
__global__ void __launch_bounds__(kLxWarps* kWarp, 6)
    lx_so2_gate_fwd_kernel(const float* __restrict__ y, Out out, const float* __restrict__ scale_ptr, int64_t num_edges, int ch) {
    using S = Shape<LMAX>;
    out.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kLxWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kLxWarps;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        const float* p = y + e * (int64_t)(LMAX + S::kM) * ch;
        const int64_t o = e * (int64_t)S::kM * ch;
        for (int c = lane * 4; c < ch; c += 128) {
            const float4 v0 = ld4(p + LMAX * ch + c);
            out.st(o + c, mul4(v0, lx_sig4(v0)));
#pragma unroll
            for (int l = 1; l <= LMAX; ++l) {
                const float4 gate = lx_sig4(ld4(p + (l - 1) * ch + c));
#pragma unroll
                for (int k = 0; k < S::rows(l); ++k) {
                    const int row = S::mrow(l, k - S::mm(l));
                    out.st(o + row * ch + c, mul4(ld4(p + (LMAX + row) * ch + c), gate));
                }
            }
        }
    }
}

template <int LMAX, class Out>
__global__ void __launch_bounds__(kLxWarps* kWarp, 6)
    lx_so2_gate_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ y, Out grad_y,
                           const float* __restrict__ scale_ptr, int64_t num_edges, int ch) {
    using S = Shape<LMAX>;
    grad_y.load_scale(scale_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kLxWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kLxWarps;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        const float* p = y + e * (int64_t)(LMAX + S::kM) * ch;
        const float* go = grad_out + e * (int64_t)S::kM * ch;
        const int64_t q = e * (int64_t)(LMAX + S::kM) * ch;
        for (int c = lane * 4; c < ch; c += 128) {
            {
                const float4 v = ld4(p + LMAX * ch + c), s = lx_sig4(v), d = ld4(go + c);
                grad_y.st(q + LMAX * ch + c, make_float4(d.x * s.x * (1.f + v.x * (1.f - s.x)), d.y * s.y * (1.f + v.y * (1.f - s.y)),
                                                   d.z * s.z * (1.f + v.z * (1.f - s.z)), d.w * s.w * (1.f + v.w * (1.f - s.w))));
            }
#pragma unroll
            for (int l = 1; l <= LMAX; ++l) {
                const float4 s = lx_sig4(ld4(p + (l - 1) * ch + c));
                float4 dg = f4zero();
#pragma unroll
                for (int k = 0; k < S::rows(l); ++k) {
                    const int row = S::mrow(l, k - S::mm(l));
                    const float4 d = ld4(go + row * ch + c);
                    grad_y.st(q + (LMAX + row) * ch + c, mul4(d, s));
                    dg = add4(dg, mul4(d, ld4(p + (LMAX + row) * ch + c)));
                }
                grad_y.st(q + (l - 1) * ch + c,
                    make_float4(dg.x * s.x * (1.f - s.x), dg.y * s.y * (1.f - s.y), dg.z * s.z * (1.f - s.z), dg.w * s.w * (1.f - s.w)));
            }
        }
    }
}

}  // namespace fcb200

using namespace fcb200;

namespace {

int lx_check(const void* a, const void* b, int64_t n, int32_t channels, int32_t lmax) {
    if (a == nullptr || b == nullptr || n < 0) return FCB200_EINVAL;
    if (channels <= 0 || channels % 128 != 0) return FCB200_EINVAL;
    if (lmax != 2 && lmax != 4) return FCB200_EINVAL;
    if (!aligned16(a) || !aligned16(b)) return FCB200_EALIGN;
    return FCB200_OK;
}

}  // namespace

// launch `kernel<LMAX, extra template arguments...>` for the runtime lmax (2 or 4; checked by lx_check)
#define LX_GRID(items) warp_grid(items, kLxWarps), kLxWarps * kWarp, 0, static_cast<cudaStream_t>(stream)
#define LX_DISPATCH(items, kernel, targs, ...)                                   \
    do {                                                                         \
        if (lmax == 2)                                                           \
            kernel<2 targs><<<LX_GRID(items)>>>(__VA_ARGS__);                    \
        else                                                                     \
            kernel<4 targs><<<LX_GRID(items)>>>(__VA_ARGS__);                    \
    } while (0)
#define LX_COMMA ,

extern "C" {

int fcb200_lx_gather_rotate_fwd(const float* x, const int32_t* src, const int32_t* tgt, const float* wig, const float* radial,
                                float* out, int64_t num_edges, int64_t num_nodes, int32_t channels, int32_t lmax, void* stream) {
    int rc = lx_check(x, out, num_edges, channels, lmax);
    if (rc != FCB200_OK) return rc;
    if (!src || !tgt || !wig || num_nodes < 0) return FCB200_EINVAL;
    if (radial && !aligned16(radial)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    if (radial)
        LX_DISPATCH(num_edges, lx_gather_rotate_fwd_kernel, LX_COMMA true LX_COMMA OutF32, x, src, tgt, wig, radial, OutF32{out},
                    nullptr, num_edges, channels);
    else
        LX_DISPATCH(num_edges, lx_gather_rotate_fwd_kernel, LX_COMMA false LX_COMMA OutF32, x, src, tgt, wig, nullptr, OutF32{out},
                    nullptr, num_edges, channels);
    return launch_status();
}

int fcb200_lx_gather_rotate_bwd(const float* grad_out, const float* x, const int32_t* src, const int32_t* tgt, const float* wig,
                                const float* radial, float* g_src, float* g_tgt, float* grad_wig, float* grad_radial,
                                int64_t num_edges, int64_t num_nodes, int32_t channels, int32_t lmax, void* stream) {
    int rc = lx_check(grad_out, x, num_edges, channels, lmax);
    if (rc != FCB200_OK) return rc;
    if (!src || !tgt || !wig || !g_src || !g_tgt || !grad_wig || num_nodes < 0) return FCB200_EINVAL;
    if ((radial == nullptr) != (grad_radial == nullptr)) return FCB200_EINVAL;
    if (!aligned16(g_src) || !aligned16(g_tgt) || (radial && (!aligned16(radial) || !aligned16(grad_radial)))) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    if (radial)
        LX_DISPATCH(num_edges, lx_gather_rotate_bwd_kernel, LX_COMMA true, grad_out, x, src, tgt, wig, radial, g_src, g_tgt,
                    grad_wig, grad_radial, num_edges, channels);
    else
        LX_DISPATCH(num_edges, lx_gather_rotate_bwd_kernel, LX_COMMA false, grad_out, x, src, tgt, wig, nullptr, g_src, g_tgt,
                    grad_wig, nullptr, num_edges, channels);
    return launch_status();
}

int fcb200_lx_rotate_back_reduce_fwd(const float* msg, const float* winv, const int32_t* row_ptr, float* out, int64_t num_edges,
                                     int64_t num_nodes, int32_t channels, int32_t lmax, void* stream) {
    int rc = lx_check(msg, out, num_nodes, channels, lmax);
    if (rc != FCB200_OK) return rc;
    if (!winv || !row_ptr || num_edges < 0) return FCB200_EINVAL;
    if (num_nodes == 0) return FCB200_OK;
    LX_DISPATCH(num_nodes, lx_rotate_back_reduce_kernel, LX_COMMA 0, msg, winv, row_ptr, nullptr, out, 1.0f, num_nodes, channels);
    return launch_status();
}

int fcb200_lx_edge_degree_fwd(const float* radial0, const float* winv, const int32_t* row_ptr, const float* x_in, float* out,
                              float rescale, int64_t num_edges, int64_t num_nodes, int32_t channels, int32_t lmax, void* stream) {
    int rc = lx_check(radial0, out, num_nodes, channels, lmax);
    if (rc != FCB200_OK) return rc;
    if (!winv || !row_ptr || num_edges < 0 || rescale == 0.f) return FCB200_EINVAL;
    if (x_in && !aligned16(x_in)) return FCB200_EALIGN;
    if (num_nodes == 0) return FCB200_OK;
    LX_DISPATCH(num_nodes, lx_rotate_back_reduce_kernel, LX_COMMA 1, radial0, winv, row_ptr, x_in, out, rescale, num_nodes, channels);
    return launch_status();
}

int fcb200_lx_rotate_back_bwd(const float* grad_out, const float* msg, const float* winv, const int32_t* tgt, float* grad_msg,
                              float* grad_winv, int64_t num_edges, int64_t num_nodes, int32_t channels, int32_t lmax,
                              void* stream) {
    int rc = lx_check(grad_out, grad_msg, num_edges, channels, lmax);
    if (rc != FCB200_OK) return rc;
    if (!winv || !tgt || num_nodes < 0) return FCB200_EINVAL;
    if ((grad_winv != nullptr) && (msg == nullptr)) return FCB200_EINVAL;
    if (msg && !aligned16(msg)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    if (grad_winv)
        LX_DISPATCH(num_edges, lx_rotate_back_bwd_kernel, LX_COMMA 0 LX_COMMA true LX_COMMA OutF32, grad_out, msg, winv, tgt,
                    OutF32{grad_msg}, nullptr, grad_winv, 1.f, num_edges, channels);
    else
        LX_DISPATCH(num_edges, lx_rotate_back_bwd_kernel, LX_COMMA 0 LX_COMMA false LX_COMMA OutF32, grad_out, nullptr, winv, tgt,
                    OutF32{grad_msg}, nullptr, nullptr, 1.f, num_edges, channels);
    return launch_status();
}

int fcb200_lx_edge_degree_bwd(const float* grad_out, const float* radial0, const float* winv, const int32_t* tgt,
                              float* grad_radial0, float* grad_winv, float rescale, int64_t num_edges, int64_t num_nodes,
                              int32_t channels, int32_t lmax, void* stream) {
    int rc = lx_check(grad_out, grad_radial0, num_edges, channels, lmax);
    if (rc != FCB200_OK) return rc;
    if (!radial0 || !winv || !tgt || !grad_winv || num_nodes < 0 || rescale == 0.f) return FCB200_EINVAL;
    if (!aligned16(radial0)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    // every entry of grad_winv is written (zeros in the rows m != 0, which this op does not read)
    LX_DISPATCH(num_edges, lx_rotate_back_bwd_kernel, LX_COMMA 1 LX_COMMA true LX_COMMA OutF32, grad_out, radial0, winv, tgt,
                OutF32{grad_radial0}, nullptr, grad_winv, rescale, num_edges, channels);
    return launch_status();
}

int fcb200_lx_so2_gate_fwd(const float* y, float* out, int64_t num_edges, int32_t hidden, int32_t lmax, void* stream) {
    int rc = lx_check(y, out, num_edges, hidden, lmax);
    if (rc != FCB200_OK) return rc;
    if (num_edges == 0) return FCB200_OK;
    LX_DISPATCH(num_edges, lx_so2_gate_fwd_kernel, LX_COMMA OutF32, y, OutF32{out}, nullptr, num_edges, hidden);
    return launch_status();
}

int fcb200_lx_so2_gate_bwd(const float* grad_out, const float* y, float* grad_y, int64_t num_edges, int32_t hidden, int32_t lmax,
                           void* stream) {
    int rc = lx_check(grad_out, y, num_edges, hidden, lmax);
    if (rc != FCB200_OK) return rc;
    if (!grad_y) return FCB200_EINVAL;
    if (!aligned16(grad_y)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    LX_DISPATCH(num_edges, lx_so2_gate_bwd_kernel, LX_COMMA OutF32, grad_out, y, OutF32{grad_y}, nullptr, num_edges, hidden);
    return launch_status();
}

// ---- the same four producers writing the half-precision split the tensor-core contraction reads directly ----

int fcb200_lx_gather_rotate_fwd_h(const float* x, const int32_t* src, const int32_t* tgt, const float* wig, const float* radial,
                                  void* out_hi, void* out_lo, const float* scale, int64_t num_edges, int64_t num_nodes,
                                  int32_t channels, int32_t lmax, void* stream) {
    int rc = lx_check(x, x, num_edges, channels, lmax);
    if (rc != FCB200_OK) return rc;
    if (!out_hi || !out_lo || !src || !tgt || !wig || num_nodes < 0) return FCB200_EINVAL;
    if (!aligned8(out_hi) || !aligned8(out_lo) || (radial && !aligned16(radial))) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    const OutSplit out{static_cast<__half*>(out_hi), static_cast<__half*>(out_lo), 1.0f};
    if (radial)
        LX_DISPATCH(num_edges, lx_gather_rotate_fwd_kernel, LX_COMMA true LX_COMMA OutSplit, x, src, tgt, wig, radial, out, scale,
                    num_edges, channels);
    else
        LX_DISPATCH(num_edges, lx_gather_rotate_fwd_kernel, LX_COMMA false LX_COMMA OutSplit, x, src, tgt, wig, nullptr, out, scale,
                    num_edges, channels);
    return launch_status();
}

int fcb200_lx_rotate_back_bwd_h(const float* grad_out, const float* msg, const float* winv, const int32_t* tgt, void* grad_msg_hi,
                                void* grad_msg_lo, const float* scale, float* grad_winv, int64_t num_edges, int64_t num_nodes,
                                int32_t channels, int32_t lmax, void* stream) {
    int rc = lx_check(grad_out, grad_out, num_edges, channels, lmax);
    if (rc != FCB200_OK) return rc;
    if (!winv || !tgt || !grad_msg_hi || !grad_msg_lo || num_nodes < 0) return FCB200_EINVAL;
    if ((grad_winv != nullptr) && (msg == nullptr)) return FCB200_EINVAL;
    if (!aligned8(grad_msg_hi) || !aligned8(grad_msg_lo) || (msg && !aligned16(msg))) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    const OutSplit out{static_cast<__half*>(grad_msg_hi), static_cast<__half*>(grad_msg_lo), 1.0f};
    if (grad_winv)
        LX_DISPATCH(num_edges, lx_rotate_back_bwd_kernel, LX_COMMA 0 LX_COMMA true LX_COMMA OutSplit, grad_out, msg, winv, tgt, out,
                    scale, grad_winv, 1.f, num_edges, channels);
    else
        LX_DISPATCH(num_edges, lx_rotate_back_bwd_kernel, LX_COMMA 0 LX_COMMA false LX_COMMA OutSplit, grad_out, nullptr, winv, tgt,
                    out, scale, nullptr, 1.f, num_edges, channels);
    return launch_status();
}

int fcb200_lx_so2_gate_fwd_h(const float* y, void* out_hi, void* out_lo, const float* scale, int64_t num_edges, int32_t hidden,
                             int32_t lmax, void* stream) {
    int rc = lx_check(y, y, num_edges, hidden, lmax);
    if (rc != FCB200_OK) return rc;
    if (!out_hi || !out_lo) return FCB200_EINVAL;
    if (!aligned8(out_hi) || !aligned8(out_lo)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    const OutSplit out{static_cast<__half*>(out_hi), static_cast<__half*>(out_lo), 1.0f};
    LX_DISPATCH(num_edges, lx_so2_gate_fwd_kernel, LX_COMMA OutSplit, y, out, scale, num_edges, hidden);
    return launch_status();
}

int fcb200_lx_so2_gate_bwd_h(const float* grad_out, const float* y, void* grad_y_hi, void* grad_y_lo, const float* scale,
                             int64_t num_edges, int32_t hidden, int32_t lmax, void* stream) {
    int rc = lx_check(grad_out, y, num_edges, hidden, lmax);
    if (rc != FCB200_OK) return rc;
    if (!grad_y_hi || !grad_y_lo) return FCB200_EINVAL;
    if (!aligned8(grad_y_hi) || !aligned8(grad_y_lo)) return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    const OutSplit out{static_cast<__half*>(grad_y_hi), static_cast<__half*>(grad_y_lo), 1.0f};
    LX_DISPATCH(num_edges, lx_so2_gate_bwd_kernel, LX_COMMA OutSplit, grad_out, y, out, scale, num_edges, hidden);
    return launch_status();
}

}  // extern "C"
