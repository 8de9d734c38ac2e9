// Node-wise kernels that bracket the edge block: the degree-balanced RMS norm over a node's (lmax+1)^2 x C
// spherical-harmonic coefficients (forward and backward), one warp per node, a lane owns one float4 of
// each of the rows.  HBM-bound: one read and one write of the node tensor per pass.
#include "common.cuh"

namespace fcb200 {

constexpr int kNodeWarps = 8;

// degree of L-major row L
__host__ __device__ constexpr int degree_of(int L) {
    int l = 0;
    while ((l + 1) * (l + 1) <= L) ++l;
    return l;
}
// weight of row L in the norm: 1 / ((2l+1) * (lmax+1))
template <int LMAX> __host__ __device__ constexpr float balance_of(int L) {
    return 1.0f / (float)((2 * degree_of(L) + 1) * (LMAX + 1));
}

__device__ __forceinline__ float hsum4(float4 v) { return v.x + v.y + v.z + v.w; }

// out_i = y_i * rsqrt(mean_c sum_i bal_i y_i^2 + eps) * w[l_i] (+ bias, + extra on row 0), y_0 = x_0 - mean_c x_0
template <int LMAX>
__global__ void __launch_bounds__(kNodeWarps* kWarp)
    rms_norm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ weight, const float* __restrict__ bias,
                        const float* __restrict__ extra, float* __restrict__ out, float* __restrict__ stats, float eps,
                        int64_t num_nodes, int channels) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kNodeWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kNodeWarps;
    const float inv_c = 1.0f / (float)channels;
    constexpr int kL = (LMAX + 1) * (LMAX + 1);
    for (int64_t n = warp0; n < num_nodes; n += nwarps) {
        const float* xb = x + n * (int64_t)kL * channels;
        float* ob = out + n * (int64_t)kL * channels;
        // pass 1: mean of row 0 and the balanced sum of squares (channels > 128 loop over tiles)
        float s0 = 0.f;
        for (int c = lane * 4; c < channels; c += 128) s0 += hsum4(ld4(xb + c));
        const float mean0 = warp_sum(s0) * inv_c;
        float acc = 0.f;
        for (int c = lane * 4; c < channels; c += 128) {
#pragma unroll
            for (int L = 0; L < kL; ++L) {
                float4 v = ld4(xb + L * channels + c);
                if (L == 0) v = make_float4(v.x - mean0, v.y - mean0, v.z - mean0, v.w - mean0);
                acc = fmaf(balance_of<LMAX>(L), dot4(v, v), acc);
            }
        }
        const float scale = rsqrtf(warp_sum(acc) * inv_c + eps);
        for (int c = lane * 4; c < channels; c += 128) {
#pragma unroll
            for (int L = 0; L < kL; ++L) {
                float4 v = ld4(xb + L * channels + c);
                if (L == 0) v = make_float4(v.x - mean0, v.y - mean0, v.z - mean0, v.w - mean0);
                float4 o = mul4(scale4(scale, v), ld4(weight + degree_of(L) * channels + c));
                if (L == 0) {
                    o = add4(o, ld4(bias + c));
                    if (extra) o = add4(o, ld4(extra + n * channels + c));
                }
                st4(ob + L * channels + c, o);
            }
        }
        if (lane == 0) {
            stats[n * 2 + 0] = mean0;
            stats[n * 2 + 1] = scale;
        }
    }
}

template <int LMAX>
__global__ void __launch_bounds__(kNodeWarps* kWarp)
    rms_norm_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ x, const float* __restrict__ weight,
                        const float* __restrict__ stats, float* __restrict__ grad_x, int64_t num_nodes, int channels) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kNodeWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kNodeWarps;
    const float inv_c = 1.0f / (float)channels;
    constexpr int kL = (LMAX + 1) * (LMAX + 1);
    for (int64_t n = warp0; n < num_nodes; n += nwarps) {
        const float* xb = x + n * (int64_t)kL * channels;
        const float* gb = grad_out + n * (int64_t)kL * channels;
        float* qb = grad_x + n * (int64_t)kL * channels;
        const float mean0 = stats[n * 2 + 0], scale = stats[n * 2 + 1];
        // dL/dscale = sum_{i,c} g_i w_i y_i ; also sum_c g_0 w_0 for the centering term
        float ds = 0.f, g0w = 0.f, y0b = 0.f;
        for (int c = lane * 4; c < channels; c += 128) {
#pragma unroll
            for (int L = 0; L < kL; ++L) {
                float4 v = ld4(xb + L * channels + c);
                if (L == 0) v = make_float4(v.x - mean0, v.y - mean0, v.z - mean0, v.w - mean0);
                const float4 gw = mul4(ld4(gb + L * channels + c), ld4(weight + degree_of(L) * channels + c));
                ds += dot4(gw, v);
                if (L == 0) {
                    g0w += hsum4(gw);
                    y0b += hsum4(v);
                }
            }
        }
        ds = warp_sum(ds);
        g0w = warp_sum(g0w);
        y0b = warp_sum(y0b);
        // dL/dy_i = g_i w_i scale - scale^3 * ds * bal_i * y_i / C ; dL/dx_0 = dL/dy_0 - mean_c dL/dy_0
        const float k = scale * scale * scale * ds * inv_c;
        const float mean_dy0 = (g0w * scale - k * balance_of<LMAX>(0) * y0b) * inv_c;
        for (int c = lane * 4; c < channels; c += 128) {
#pragma unroll
            for (int L = 0; L < kL; ++L) {
                float4 v = ld4(xb + L * channels + c);
                if (L == 0) v = make_float4(v.x - mean0, v.y - mean0, v.z - mean0, v.w - mean0);
                const float4 gw = mul4(ld4(gb + L * channels + c), ld4(weight + degree_of(L) * channels + c));
                const float kb = k * balance_of<LMAX>(L);
                float4 d = make_float4(fmaf(gw.x, scale, -kb * v.x), fmaf(gw.y, scale, -kb * v.y), fmaf(gw.z, scale, -kb * v.z),
                                       fmaf(gw.w, scale, -kb * v.w));
                if (L == 0) d = make_float4(d.x - mean_dy0, d.y - mean_dy0, d.z - mean_dy0, d.w - mean_dy0);
                st4(qb + L * channels + c, d);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// gate of the node-wise feed-forward (SpectralAtomwise): y [N, NL, H] L-major, gate_pre [N, LMAX*H] (the
// scalar Linear's output); out row 0 = SiLU(y_0), rows of degree l >= 1 = y * sigmoid(SiLU(gate_pre[l-1]))
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigm(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu_f(float v) { return v * sigm(v); }
__device__ __forceinline__ float dsilu_f(float v) {
    const float s = sigm(v);
    return s * (1.0f + v * (1.0f - s));
}
template <class F> __device__ __forceinline__ float4 map4(float4 v, F f) { return make_float4(f(v.x), f(v.y), f(v.z), f(v.w)); }

template <int LMAX>
__global__ void __launch_bounds__(kNodeWarps* kWarp)
    node_gate_fwd_kernel(const float* __restrict__ y, const float* __restrict__ gate_pre, float* __restrict__ out,
                         int64_t num_nodes, int ch) {
    constexpr int kL = (LMAX + 1) * (LMAX + 1);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kNodeWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kNodeWarps;
    for (int64_t n = warp0; n < num_nodes; n += nwarps) {
        const float* yb = y + n * (int64_t)kL * ch;
        float* ob = out + n * (int64_t)kL * ch;
        for (int c = lane * 4; c < ch; c += 128) {
            st4(ob + c, map4(ld4(yb + c), silu_f));
#pragma unroll
            for (int l = 1; l <= LMAX; ++l) {
                const float4 g = map4(ld4(gate_pre + n * (int64_t)LMAX * ch + (l - 1) * ch + c), [](float v) { return sigm(silu_f(v)); });
#pragma unroll
                for (int j = 0; j < 2 * l + 1; ++j) st4(ob + (l * l + j) * ch + c, mul4(ld4(yb + (l * l + j) * ch + c), g));
            }
        }
    }
}

template <int LMAX>
__global__ void __launch_bounds__(kNodeWarps* kWarp)
    node_gate_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ y, const float* __restrict__ gate_pre,
                         float* __restrict__ grad_y, float* __restrict__ grad_gate_pre, int64_t num_nodes, int ch) {
    constexpr int kL = (LMAX + 1) * (LMAX + 1);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kNodeWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kNodeWarps;
    for (int64_t n = warp0; n < num_nodes; n += nwarps) {
        const float* yb = y + n * (int64_t)kL * ch;
        const float* gb = grad_out + n * (int64_t)kL * ch;
        float* qb = grad_y + n * (int64_t)kL * ch;
        for (int c = lane * 4; c < ch; c += 128) {
            st4(qb + c, mul4(ld4(gb + c), map4(ld4(yb + c), dsilu_f)));
#pragma unroll
            for (int l = 1; l <= LMAX; ++l) {
                const float4 pre = ld4(gate_pre + n * (int64_t)LMAX * ch + (l - 1) * ch + c);
                const float4 g = map4(pre, [](float v) { return sigm(silu_f(v)); });
                float4 dg = f4zero();
#pragma unroll
                for (int j = 0; j < 2 * l + 1; ++j) {
                    const float4 d = ld4(gb + (l * l + j) * ch + c);
                    st4(qb + (l * l + j) * ch + c, mul4(d, g));
                    dg = add4(dg, mul4(d, ld4(yb + (l * l + j) * ch + c)));
                }
                // d/dpre sigmoid(SiLU(pre)) = g (1 - g) SiLU'(pre)
                const float4 chain = mul4(mul4(g, make_float4(1.f - g.x, 1.f - g.y, 1.f - g.z, 1.f - g.w)), map4(pre, dsilu_f));
                st4(grad_gate_pre + n * (int64_t)LMAX * ch + (l - 1) * ch + c, mul4(dg, chain));
            }
        }
    }
}

}  // namespace fcb200

using namespace fcb200;

extern "C" {

#define FCB_NODE_LAUNCH(kernel, ...)                                                                                          \
    do {                                                                                                                      \
        const int grid = warp_grid(num_nodes, kNodeWarps);                                                                    \
        if (lmax == 2)                                                                                                        \
            kernel<2><<<grid, kNodeWarps * kWarp, 0, static_cast<cudaStream_t>(stream)>>>(__VA_ARGS__);                       \
        else if (lmax == 4)                                                                                                   \
            kernel<4><<<grid, kNodeWarps * kWarp, 0, static_cast<cudaStream_t>(stream)>>>(__VA_ARGS__);                       \
        else                                                                                                                  \
            return FCB200_EINVAL;                                                                                             \
    } while (0)

int fcb200_lx_rms_norm_sh_fwd(const float* x, const float* weight, const float* bias, const float* extra, float* out, float* stats,
                              float eps, int64_t num_nodes, int32_t channels, int32_t lmax, void* stream) {
    if (!x || !weight || !bias || !out || !stats || num_nodes < 0 || channels <= 0 || channels % 128) return FCB200_EINVAL;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(bias) || !aligned16(out) || (extra && !aligned16(extra))) return FCB200_EALIGN;
    if (lmax != 2 && lmax != 4) return FCB200_EINVAL;
    if (num_nodes == 0) return FCB200_OK;
    FCB_NODE_LAUNCH(rms_norm_fwd_kernel, x, weight, bias, extra, out, stats, eps, num_nodes, channels);
    return launch_status();
}

int fcb200_lx_rms_norm_sh_bwd(const float* grad_out, const float* x, const float* weight, const float* stats, float* grad_x,
                              int64_t num_nodes, int32_t channels, int32_t lmax, void* stream) {
    if (!grad_out || !x || !weight || !stats || !grad_x || num_nodes < 0 || channels <= 0 || channels % 128) return FCB200_EINVAL;
    if (!aligned16(grad_out) || !aligned16(x) || !aligned16(weight) || !aligned16(grad_x)) return FCB200_EALIGN;
    if (lmax != 2 && lmax != 4) return FCB200_EINVAL;
    if (num_nodes == 0) return FCB200_OK;
    FCB_NODE_LAUNCH(rms_norm_bwd_kernel, grad_out, x, weight, stats, grad_x, num_nodes, channels);
    return launch_status();
}

int fcb200_node_gate_fwd(const float* y, const float* gate_pre, float* out, int64_t num_nodes, int32_t hidden, int32_t lmax,
                         void* stream) {
    if (!y || !gate_pre || !out || num_nodes < 0 || hidden <= 0 || hidden % 128) return FCB200_EINVAL;
    if (!aligned16(y) || !aligned16(gate_pre) || !aligned16(out)) return FCB200_EALIGN;
    if (lmax != 2 && lmax != 4) return FCB200_EINVAL;
    if (num_nodes == 0) return FCB200_OK;
    FCB_NODE_LAUNCH(node_gate_fwd_kernel, y, gate_pre, out, num_nodes, hidden);
    return launch_status();
}

int fcb200_node_gate_bwd(const float* grad_out, const float* y, const float* gate_pre, float* grad_y, float* grad_gate_pre,
                         int64_t num_nodes, int32_t hidden, int32_t lmax, void* stream) {
    if (!grad_out || !y || !gate_pre || !grad_y || !grad_gate_pre || num_nodes < 0 || hidden <= 0 || hidden % 128) return FCB200_EINVAL;
    if (!aligned16(grad_out) || !aligned16(y) || !aligned16(gate_pre) || !aligned16(grad_y) || !aligned16(grad_gate_pre))
        return FCB200_EALIGN;
    if (lmax != 2 && lmax != 4) return FCB200_EINVAL;
    if (num_nodes == 0) return FCB200_OK;
    FCB_NODE_LAUNCH(node_gate_bwd_kernel, grad_out, y, gate_pre, grad_y, grad_gate_pre, num_nodes, hidden);
    return launch_status();
}

int fcb200_rms_norm_sh_fwd(const float* x, const float* weight, const float* bias, const float* extra, float* out, float* stats,
                           float eps, int64_t num_nodes, int32_t channels, void* stream) {
    return fcb200_lx_rms_norm_sh_fwd(x, weight, bias, extra, out, stats, eps, num_nodes, channels, 2, stream);
}

int fcb200_rms_norm_sh_bwd(const float* grad_out, const float* x, const float* weight, const float* stats, float* grad_x,
                           int64_t num_nodes, int32_t channels, void* stream) {
    return fcb200_lx_rms_norm_sh_bwd(grad_out, x, weight, stats, grad_x, num_nodes, channels, 2, stream);
}

}  // extern "C"
