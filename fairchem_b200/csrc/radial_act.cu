// Hidden-layer activation of the radial MLP, fused: add the two per-element embedding tables, LayerNorm
// over the row, SiLU -- one pass over a [E, W] tensor (W = 128), one warp per row, a lane owns a float4.
// HBM-bound: reads 4W (+ two L2-resident table rows), writes 4W + 8 bytes per edge.
#include <cuda_fp16.h>

#include "common.cuh"

namespace fcb200 {

constexpr int kActWarps = 8;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

__device__ __forceinline__ float4 load_row(const float* __restrict__ pre, const float* __restrict__ ts, const float* __restrict__ tt,
                                           const int32_t* __restrict__ zs, const int32_t* __restrict__ zt, int64_t e, int w, int c) {
    float4 y = ld4(pre + e * w + c);
    if (ts) y = add4(y, ld4(ts + (int64_t)zs[e] * w + c));
    if (tt) y = add4(y, ld4(tt + (int64_t)zt[e] * w + c));
    return y;
}

// Out = OutF32 (float32 rows) or OutSplit (the half-precision hi / lo planes the next contraction reads directly)
template <class Out>
__global__ void __launch_bounds__(kActWarps* kWarp)
    radial_act_fwd_kernel(const float* __restrict__ pre, const float* __restrict__ ts, const float* __restrict__ tt,
                          const int32_t* __restrict__ zs, const int32_t* __restrict__ zt, const float* __restrict__ gamma,
                          const float* __restrict__ beta, float eps, Out out, float* __restrict__ stats,
                          int64_t num_edges, int w) {
    out.load_scale(nullptr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kActWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kActWarps;
    const int c = lane * 4;  // W == 128
    const float4 g = ld4(gamma + c), b = ld4(beta + c);
    const float inv_w = 1.0f / (float)w;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        const float4 y = load_row(pre, ts, tt, zs, zt, e, w, c);
        const float mean = warp_sum(y.x + y.y + y.z + y.w) * inv_w;
        const float4 d = make_float4(y.x - mean, y.y - mean, y.z - mean, y.w - mean);
        const float var = warp_sum(d.x * d.x + d.y * d.y + d.z * d.z + d.w * d.w) * inv_w;
        const float rstd = rsqrtf(var + eps);
        float4 v = make_float4(fmaf(d.x * rstd, g.x, b.x), fmaf(d.y * rstd, g.y, b.y), fmaf(d.z * rstd, g.z, b.z),
                               fmaf(d.w * rstd, g.w, b.w));
        out.st(e * w + c, make_float4(v.x * sigmoid_f(v.x), v.y * sigmoid_f(v.y), v.z * sigmoid_f(v.z), v.w * sigmoid_f(v.w)));
        if (lane == 0) {
            stats[e * 2 + 0] = mean;
            stats[e * 2 + 1] = rstd;
        }
    }
}

__global__ void __launch_bounds__(kActWarps* kWarp)
    radial_act_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ pre, const float* __restrict__ ts,
                          const float* __restrict__ tt, const int32_t* __restrict__ zs, const int32_t* __restrict__ zt,
                          const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ stats,
                          float* __restrict__ grad_pre, int64_t num_edges, int w) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kActWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kActWarps;
    const int c = lane * 4;
    const float4 g = ld4(gamma + c), b = ld4(beta + c);
    const float inv_w = 1.0f / (float)w;
    for (int64_t e = warp0; e < num_edges; e += nwarps) {
        const float4 y = load_row(pre, ts, tt, zs, zt, e, w, c);
        const float mean = stats[e * 2 + 0], rstd = stats[e * 2 + 1];
        const float4 xh = make_float4((y.x - mean) * rstd, (y.y - mean) * rstd, (y.z - mean) * rstd, (y.w - mean) * rstd);
        const float4 go = ld4(grad_out + e * w + c);
        float dx[4];
        const float xhv[4] = {xh.x, xh.y, xh.z, xh.w}, gv[4] = {g.x, g.y, g.z, g.w}, bv[4] = {b.x, b.y, b.z, b.w},
                    gov[4] = {go.x, go.y, go.z, go.w};
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float v = fmaf(xhv[i], gv[i], bv[i]);
            const float s = sigmoid_f(v);
            const float dv = gov[i] * s * (1.0f + v * (1.0f - s));  // d silu
            dx[i] = dv * gv[i];                                     // d/d xhat
            s1 += dx[i];
            s2 += dx[i] * xhv[i];
        }
        s1 = warp_sum(s1) * inv_w;
        s2 = warp_sum(s2) * inv_w;
        st4(grad_pre + e * w + c, make_float4(rstd * (dx[0] - s1 - xhv[0] * s2), rstd * (dx[1] - s1 - xhv[1] * s2),
                                              rstd * (dx[2] - s1 - xhv[2] * s2), rstd * (dx[3] - s1 - xhv[3] * s2)));
    }
}

}  // namespace fcb200

using namespace fcb200;

extern "C" {

int fcb200_radial_act_fwd(const float* pre, const float* table_src, const float* table_tgt, const int32_t* z_src,
                          const int32_t* z_tgt, const float* ln_weight, const float* ln_bias, float eps, float* out, float* stats,
                          int64_t num_edges, int32_t width, void* stream) {
    if (!pre || !ln_weight || !ln_bias || !out || !stats || num_edges < 0 || width != 128) return FCB200_EINVAL;
    if ((table_src && !z_src) || (table_tgt && !z_tgt)) return FCB200_EINVAL;
    if (!aligned16(pre) || !aligned16(out) || !aligned16(ln_weight) || !aligned16(ln_bias) || (table_src && !aligned16(table_src)) ||
        (table_tgt && !aligned16(table_tgt)))
        return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    radial_act_fwd_kernel<OutF32><<<warp_grid(num_edges, kActWarps), kActWarps * kWarp, 0, static_cast<cudaStream_t>(stream)>>>(
        pre, table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias, eps, OutF32{out}, stats, num_edges, width);
    return launch_status();
}

int fcb200_radial_act_fwd_h(const float* pre, const float* table_src, const float* table_tgt, const int32_t* z_src,
                            const int32_t* z_tgt, const float* ln_weight, const float* ln_bias, float eps, void* out_hi,
                            void* out_lo, float* stats, int64_t num_edges, int32_t width, void* stream) {
    if (!pre || !ln_weight || !ln_bias || !out_hi || !out_lo || !stats || num_edges < 0 || width != 128) return FCB200_EINVAL;
    if ((table_src && !z_src) || (table_tgt && !z_tgt)) return FCB200_EINVAL;
    if (!aligned16(pre) || !aligned16(out_hi) || !aligned16(out_lo) || !aligned16(ln_weight) || !aligned16(ln_bias) ||
        (table_src && !aligned16(table_src)) || (table_tgt && !aligned16(table_tgt)))
        return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    radial_act_fwd_kernel<OutSplit><<<warp_grid(num_edges, kActWarps), kActWarps * kWarp, 0, static_cast<cudaStream_t>(stream)>>>(
        pre, table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias, eps,
        OutSplit{static_cast<__half*>(out_hi), static_cast<__half*>(out_lo), 1.0f}, stats, num_edges, width);
    return launch_status();
}

int fcb200_radial_act_bwd(const float* grad_out, const float* pre, const float* table_src, const float* table_tgt,
                          const int32_t* z_src, const int32_t* z_tgt, const float* ln_weight, const float* ln_bias,
                          const float* stats, float* grad_pre, int64_t num_edges, int32_t width, void* stream) {
    if (!grad_out || !pre || !ln_weight || !ln_bias || !stats || !grad_pre || num_edges < 0 || width != 128) return FCB200_EINVAL;
    if ((table_src && !z_src) || (table_tgt && !z_tgt)) return FCB200_EINVAL;
    if (!aligned16(grad_out) || !aligned16(pre) || !aligned16(grad_pre) || !aligned16(ln_weight) || !aligned16(ln_bias) ||
        (table_src && !aligned16(table_src)) || (table_tgt && !aligned16(table_tgt)))
        return FCB200_EALIGN;
    if (num_edges == 0) return FCB200_OK;
    radial_act_bwd_kernel<<<warp_grid(num_edges, kActWarps), kActWarps * kWarp, 0, static_cast<cudaStream_t>(stream)>>>(
        grad_out, pre, table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias, stats, grad_pre, num_edges, width);
    return launch_status();
}

}  // extern "C"
