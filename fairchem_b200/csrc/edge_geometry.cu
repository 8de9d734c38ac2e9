// Per-edge geometry: edge vector, length, envelope, Gaussian basis and the compact Wigner-D of the
// rotation that takes the edge direction to +Y (l <= 2, or l <= 4 with rows |m| <= 2), forward and backward.
//
// The rotation code is written once as a template over the scalar type.  Instantiated with
// float it is the forward pass; instantiated with Dual3 (value + three tangents, one per component
// of the edge vector) it yields d(wigner)/d(vec) exactly, which the backward kernel contracts with
// the incoming gradient.  35 outputs against 3 inputs makes forward mode the cheap direction.
#include "common.cuh"
#include "shape_lx.cuh"

namespace fcb200 {

struct Dual3 {
    float v, a, b, c;
};

__device__ __forceinline__ Dual3 mk(float v) { return {v, 0.f, 0.f, 0.f}; }
__device__ __forceinline__ Dual3 operator+(Dual3 x, Dual3 y) { return {x.v + y.v, x.a + y.a, x.b + y.b, x.c + y.c}; }
__device__ __forceinline__ Dual3 operator-(Dual3 x, Dual3 y) { return {x.v - y.v, x.a - y.a, x.b - y.b, x.c - y.c}; }
__device__ __forceinline__ Dual3 operator-(Dual3 x) { return {-x.v, -x.a, -x.b, -x.c}; }
__device__ __forceinline__ Dual3 operator*(Dual3 x, Dual3 y) {
    return {x.v * y.v, x.a * y.v + x.v * y.a, x.b * y.v + x.v * y.b, x.c * y.v + x.v * y.c};
}
__device__ __forceinline__ Dual3 operator*(float s, Dual3 x) { return {s * x.v, s * x.a, s * x.b, s * x.c}; }
__device__ __forceinline__ Dual3 operator+(float s, Dual3 x) { return {s + x.v, x.a, x.b, x.c}; }
__device__ __forceinline__ Dual3 operator-(float s, Dual3 x) { return {s - x.v, -x.a, -x.b, -x.c}; }
__device__ __forceinline__ Dual3 operator/(Dual3 x, Dual3 y) {
    const float inv = 1.0f / y.v;
    const float q = x.v * inv;
    return {q, (x.a - q * y.a) * inv, (x.b - q * y.b) * inv, (x.c - q * y.c) * inv};
}
template <class T> struct Ops;
template <> struct Ops<float> {
    static __device__ __forceinline__ float val(float x) { return x; }
    static __device__ __forceinline__ float lit(float x) { return x; }
    static __device__ __forceinline__ float sqrt_(float x) { return sqrtf(x); }
    static __device__ __forceinline__ float sigmoid_(float x) { return 1.0f / (1.0f + expf(-x)); }
    // max(x, lo) with zero derivative on the clamped side
    static __device__ __forceinline__ float clamp_min(float x, float lo) { return x < lo ? lo : x; }
    static __device__ __forceinline__ float clamp01(float x) { return x < 0.f ? 0.f : (x > 1.f ? 1.f : x); }
};
template <> struct Ops<Dual3> {
    static __device__ __forceinline__ float val(Dual3 x) { return x.v; }
    static __device__ __forceinline__ Dual3 lit(float x) { return mk(x); }
    static __device__ __forceinline__ Dual3 sqrt_(Dual3 x) {
        const float s = sqrtf(x.v);
        const float h = 0.5f / s;
        return {s, x.a * h, x.b * h, x.c * h};
    }
    static __device__ __forceinline__ Dual3 sigmoid_(Dual3 x) {
        const float s = 1.0f / (1.0f + expf(-x.v));
        const float d = s * (1.0f - s);
        // d == 0 when the sigmoid saturates; the tangent may be huge there, keep the product at 0
        return {s, d == 0.f ? 0.f : d * x.a, d == 0.f ? 0.f : d * x.b, d == 0.f ? 0.f : d * x.c};
    }
    static __device__ __forceinline__ Dual3 clamp_min(Dual3 x, float lo) { return x.v < lo ? mk(lo) : x; }
    static __device__ __forceinline__ Dual3 clamp01(Dual3 x) { return x.v < 0.f ? mk(0.f) : (x.v > 1.f ? mk(1.f) : x); }
};

constexpr float kEps = 1.1920928955078125e-07f;  // float32 machine epsilon

// Unit quaternion (w,x,y,z): edge direction -> +Y through two charts blended by a C-infinity step
// in e_y, then a roll by gamma about Y.
template <class T>
__device__ __forceinline__ void edge_quaternion(T vx, T vy, T vz, float gamma, T (&q)[4]) {
    using O = Ops<T>;
    const T n2 = vx * vx + vy * vy + vz * vz;
    const T n = O::clamp_min(O::sqrt_(n2), 1e-12f);
    const T ex = vx / n, ey = vy / n, ez = vz / n;
    // chart 1: (1+ey, -ez, 0, ex), singular at -Y; chart 2: (-ez, 1-ey, ex, 0), singular at +Y
    T a0 = 1.0f + ey, a1 = -ez, a3 = ex;
    const T an = O::sqrt_(O::clamp_min(a0 * a0 + a1 * a1 + a3 * a3, kEps));
    a0 = a0 / an; a1 = a1 / an; a3 = a3 / an;
    T b0 = -ez, b1 = 1.0f - ey, b2 = ex;
    const T bn = O::sqrt_(O::clamp_min(b0 * b0 + b1 * b1 + b2 * b2, kEps));
    b0 = b0 / bn; b1 = b1 / bn; b2 = b2 / bn;
    // smooth step of t = (ey + 0.9) / 1.8
    const T t = O::clamp01((1.0f / 1.8f) * (0.9f + ey));
    T s;
    if (O::val(t) < kEps) {
        s = O::lit(0.f);
    } else if (O::val(t) > 1.0f - kEps) {
        s = O::lit(1.f);
    } else {
        const T den = O::clamp_min(t * (1.0f - t), kEps);
        s = O::sigmoid_((2.0f * t - O::lit(1.0f)) / den);
    }
    // nlerp(chart2 -> chart1, s) with sign alignment of chart 2
    const float dot = O::val(b0) * O::val(a0) + O::val(b1) * O::val(a1) + 0.f + 0.f;
    if (dot < 0.f) { b0 = -b0; b1 = -b1; b2 = -b2; }
    const T u = 1.0f - s;
    T q0 = u * b0 + s * a0, q1 = u * b1 + s * a1, q2 = u * b2, q3 = s * a3;
    const T qn = O::clamp_min(O::sqrt_(q0 * q0 + q1 * q1 + q2 * q2 + q3 * q3), 1e-12f);
    q0 = q0 / qn; q1 = q1 / qn; q2 = q2 / qn; q3 = q3 / qn;
    if (gamma != 0.f) {
        const float gw = cosf(0.5f * gamma), gy = sinf(0.5f * gamma);
        // Hamilton product (gw, 0, gy, 0) * q
        q[0] = gw * q0 - gy * q2;
        q[1] = gw * q1 + gy * q3;
        q[2] = gw * q2 + gy * q0;
        q[3] = gw * q3 - gy * q1;
    } else {
        q[0] = q0; q[1] = q1; q[2] = q2; q[3] = q3;
    }
}

// Compact block-diagonal Wigner-D (35 entries) of quaternion q.  l=1 is the Cartesian rotation
// matrix R; l=2 follows from R through the quadratic forms A_i of the real l=2 harmonics
// (y polar axis, m = -2..2: sqrt3 xz, sqrt3 xy, y^2-(x^2+z^2)/2, sqrt3 yz, sqrt3/2 (z^2-x^2)):
// D2[i][j] = (2/3) tr(A_i R A_j R^T).  `emit(index, value)` receives each entry.
template <class T, class F>
__device__ __forceinline__ void wigner_from_quaternion(const T (&q)[4], F&& emit) {
    using O = Ops<T>;
    const T w = q[0], x = q[1], y = q[2], z = q[3];
    const T x2 = x * x, y2 = y * y, z2 = z * z, xy = x * y, xz = x * z, yz = y * z, wx = w * x, wy = w * y, wz = w * z;
    T r[3][3];
    r[0][0] = 1.0f - 2.0f * (y2 + z2); r[0][1] = 2.0f * (xy - wz);        r[0][2] = 2.0f * (xz + wy);
    r[1][0] = 2.0f * (xy + wz);        r[1][1] = 1.0f - 2.0f * (x2 + z2); r[1][2] = 2.0f * (yz - wx);
    r[2][0] = 2.0f * (xz - wy);        r[2][1] = 2.0f * (yz + wx);        r[2][2] = 1.0f - 2.0f * (x2 + y2);
    emit(0, O::lit(1.0f));
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
        for (int j = 0; j < 3; ++j) emit(1 + i * 3 + j, r[i][j]);
    // G_j = R A_j R^T as a symmetric 3x3 (6 entries); D2[i][j] = (2/3) <A_i, G_j>
    const float s3 = 1.7320508075688772f;
#pragma unroll
    for (int j = 0; j < 5; ++j) {
        T g[3][3];
#pragma unroll
        for (int a = 0; a < 3; ++a)
#pragma unroll
            for (int d = a; d < 3; ++d) {
                T v;
                // (R A_j R^T)[a][d] = sum_{b,c} R[a][b] A_j[b][c] R[d][c]
                if (j == 0) v = (0.5f * s3) * (r[a][0] * r[d][2] + r[a][2] * r[d][0]);
                else if (j == 1) v = (0.5f * s3) * (r[a][0] * r[d][1] + r[a][1] * r[d][0]);
                else if (j == 2) v = r[a][1] * r[d][1] - 0.5f * (r[a][0] * r[d][0] + r[a][2] * r[d][2]);
                else if (j == 3) v = (0.5f * s3) * (r[a][1] * r[d][2] + r[a][2] * r[d][1]);
                else v = (0.5f * s3) * (r[a][2] * r[d][2] - r[a][0] * r[d][0]);
                g[a][d] = v;
            }
        const float k = 2.0f / 3.0f;
        emit(10 + 0 * 5 + j, (k * s3) * g[0][2]);
        emit(10 + 1 * 5 + j, (k * s3) * g[0][1]);
        emit(10 + 2 * 5 + j, k * (g[1][1] - 0.5f * (g[0][0] + g[2][2])));
        emit(10 + 3 * 5 + j, (k * s3) * g[1][2]);
        emit(10 + 4 * 5 + j, (k * 0.5f * s3) * (g[2][2] - g[0][0]));
    }
}

// ---- degrees l >= 3: the recursion of Ivanic and Ruedenberg (J. Phys. Chem. 100 (1996) 6342, erratum 1998) ----
// R^l[m][m'] = u P(0,m,m') + v V(m,m') + w W(m,m'), built from R^(l-1) and the l = 1 block; rows and
// columns run m = -l..l.  All coefficients are compile-time constants.
constexpr double csqrt(double x) {
    if (x <= 0.0) return 0.0;
    double g = x > 1.0 ? x : 1.0;
    for (int i = 0; i < 64; ++i) g = 0.5 * (g + x / g);
    return g;
}

template <int L> struct IR {
    static constexpr int P = 2 * L - 1;  // side of the degree l-1 block
    // P(i, a, b) of the paper: i indexes the l = 1 row (-1, 0, 1), a the row of R^(l-1), b the target column
    template <class T, int I, int A, int B>
    static __device__ __forceinline__ T p(const T (&r)[3][3], const T (&prev)[P][P]) {
        if constexpr (B < L && B > -L) {
            return r[I + 1][1] * prev[A + L - 1][B + L - 1];
        } else if constexpr (B == L) {
            return r[I + 1][2] * prev[A + L - 1][2 * L - 2] - r[I + 1][0] * prev[A + L - 1][0];
        } else {
            return r[I + 1][2] * prev[A + L - 1][0] + r[I + 1][0] * prev[A + L - 1][2 * L - 2];
        }
    }
    template <class T, int M, int MP>
    static __device__ __forceinline__ T entry(const T (&r)[3][3], const T (&prev)[P][P]) {
        constexpr int am = M < 0 ? -M : M;
        constexpr double den = (MP < L && MP > -L) ? (double)((L + MP) * (L - MP)) : (double)((2 * L) * (2 * L - 1));
        constexpr double d0 = M == 0 ? 1.0 : 0.0;
        constexpr float u = (float)csqrt((double)((L + M) * (L - M)) / den);
        constexpr float v = (float)(0.5 * csqrt((1.0 + d0) * (double)((L + am - 1) * (L + am)) / den) * (1.0 - 2.0 * d0));
        constexpr float w = (float)(-0.5 * csqrt((double)((L - am - 1) * (L - am)) / den) * (1.0 - d0));
        constexpr float s2 = 1.41421356237309504880f;
        T val = Ops<T>::lit(0.f);
        if constexpr (u != 0.f) val = u * p<T, 0, M, MP>(r, prev);
        if constexpr (v != 0.f) {
            if constexpr (M == 0) {
                val = val + v * (p<T, 1, 1, MP>(r, prev) + p<T, -1, -1, MP>(r, prev));
            } else if constexpr (M == 1) {
                val = val + (v * s2) * p<T, 1, 0, MP>(r, prev);
            } else if constexpr (M > 1) {
                val = val + v * (p<T, 1, M - 1, MP>(r, prev) - p<T, -1, -M + 1, MP>(r, prev));
            } else if constexpr (M == -1) {
                val = val + (v * s2) * p<T, -1, 0, MP>(r, prev);
            } else {
                val = val + v * (p<T, 1, M + 1, MP>(r, prev) + p<T, -1, -M - 1, MP>(r, prev));
            }
        }
        if constexpr (w != 0.f) {
            if constexpr (M > 0) {
                val = val + w * (p<T, 1, M + 1, MP>(r, prev) + p<T, -1, -M - 1, MP>(r, prev));
            } else {
                val = val + w * (p<T, 1, M - 1, MP>(r, prev) - p<T, -1, -M + 1, MP>(r, prev));
            }
        }
        return val;
    }
    template <class T, int M, int MP, class F>
    static __device__ __forceinline__ void cols(const T (&r)[3][3], const T (&prev)[P][P], F&& f) {
        f(M, MP, entry<T, M, MP>(r, prev));
        if constexpr (MP < L) cols<T, M, MP + 1>(r, prev, f);
    }
    // f(m, m', value) for rows m = MLO..MHI, all columns
    template <class T, int MLO, int MHI, class F>
    static __device__ __forceinline__ void rows(const T (&r)[3][3], const T (&prev)[P][P], F&& f) {
        cols<T, MLO, -L>(r, prev, f);
        if constexpr (MLO < MHI) rows<T, MLO + 1, MHI>(r, prev, f);
    }
};

// Compact Wigner entries for lmax = 4 (rows |m| <= 2 of every block): degrees 0..2 as above, then
// the full degree-3 block and rows -2..2 of degree 4 by the recursion.
template <class T, class F>
__device__ __forceinline__ void wigner_from_quaternion_l4(const T (&q)[4], F&& emit) {
    using S = Shape<4>;
    T r[3][3], d2[5][5];
    wigner_from_quaternion<T>(q, [&](int i, T v) {
        if (i >= 1 && i < 10) r[(i - 1) / 3][(i - 1) % 3] = v;
        if (i >= 10) d2[(i - 10) / 5][(i - 10) % 5] = v;
        emit(i, v);
    });
    T d3[7][7];
    IR<3>::template rows<T, -3, 3>(r, d2, [&](int m, int mp, T v) {
        d3[m + 3][mp + 3] = v;
        if (m >= -2 && m <= 2) emit(S::woff(3) + (m + 2) * 7 + (mp + 3), v);
    });
    IR<4>::template rows<T, -2, 2>(r, d3, [&](int m, int mp, T v) { emit(S::woff(4) + (m + 2) * 9 + (mp + 4), v); });
}

template <int LMAX, class T, class F>
__device__ __forceinline__ void wigner_compact(const T (&q)[4], F&& emit) {
    if constexpr (LMAX == 2) wigner_from_quaternion<T>(q, emit);
    else wigner_from_quaternion_l4<T>(q, emit);
}

__device__ __forceinline__ void edge_vector(const float* __restrict__ pos, const int32_t* __restrict__ src,
                                            const int32_t* __restrict__ tgt, const float* __restrict__ shift, int64_t e,
                                            float& vx, float& vy, float& vz) {
    const int64_t s = src[e], t = tgt[e];
    vx = pos[s * 3 + 0] - pos[t * 3 + 0];
    vy = pos[s * 3 + 1] - pos[t * 3 + 1];
    vz = pos[s * 3 + 2] - pos[t * 3 + 2];
    if (shift) {
        vx += shift[e * 3 + 0];
        vy += shift[e * 3 + 1];
        vz += shift[e * 3 + 2];
    }
}

struct BasisParams {
    float cutoff, start, step, coeff;
    int num;
};

template <int LMAX>
__global__ void __launch_bounds__(128)
    edge_geometry_fwd_kernel(const float* __restrict__ pos, const int32_t* __restrict__ src, const int32_t* __restrict__ tgt,
                             const float* __restrict__ shift, const float* __restrict__ gamma, float* __restrict__ vec,
                             float* __restrict__ dist, float* __restrict__ env, float* __restrict__ wig,
                             float* __restrict__ gauss, BasisParams bp, int64_t num_edges) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= num_edges) return;
    float vx, vy, vz;
    edge_vector(pos, src, tgt, shift, e, vx, vy, vz);
    const float d = sqrtf(vx * vx + vy * vy + vz * vz);
    if (vec) { vec[e * 3 + 0] = vx; vec[e * 3 + 1] = vy; vec[e * 3 + 2] = vz; }
    if (dist) dist[e] = d;
    if (env) {
        const float u = d / bp.cutoff;
        const float u2 = u * u;
        const float u5 = u2 * u2 * u;
        env[e] = u < 1.0f ? 1.0f + u5 * (-21.0f + u * (35.0f - 15.0f * u)) : 0.0f;
    }
    if (gauss) {
        for (int k = 0; k < bp.num; ++k) {
            const float t = d - (bp.start + bp.step * k);
            gauss[e * bp.num + k] = expf(bp.coeff * t * t);
        }
    }
    if (wig) {
        float q[4];
        edge_quaternion<float>(vx, vy, vz, gamma ? gamma[e] : 0.f, q);
        float* w = wig + e * Shape<LMAX>::kW;
        wigner_compact<LMAX, float>(q, [&](int i, float v) { w[i] = v; });
    }
}

template <int LMAX>
__global__ void __launch_bounds__(128)
    edge_geometry_bwd_kernel(const float* __restrict__ pos, const int32_t* __restrict__ src, const int32_t* __restrict__ tgt,
                             const float* __restrict__ shift, const float* __restrict__ gamma,
                             const float* __restrict__ grad_wig, const float* __restrict__ grad_env,
                             const float* __restrict__ grad_gauss, const float* __restrict__ grad_dist,
                             float* __restrict__ grad_vec, BasisParams bp, int64_t num_edges) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= num_edges) return;
    float vx, vy, vz;
    edge_vector(pos, src, tgt, shift, e, vx, vy, vz);
    const float d = sqrtf(vx * vx + vy * vy + vz * vz);
    float gx = 0.f, gy = 0.f, gz = 0.f;
    // scalar chain through the length
    float gd = grad_dist ? grad_dist[e] : 0.f;
    if (grad_env) {
        const float u = d / bp.cutoff;
        if (u < 1.0f) {
            const float u2 = u * u, u4 = u2 * u2;
            // d/du [u^5 (a + b u + c u^2)] = u^4 (5a + 6b u + 7c u^2), a=-21 b=35 c=-15
            gd += grad_env[e] * (u4 * (-105.0f + u * (210.0f - 105.0f * u))) / bp.cutoff;
        }
    }
    if (grad_gauss) {
        for (int k = 0; k < bp.num; ++k) {
            const float t = d - (bp.start + bp.step * k);
            gd += grad_gauss[e * bp.num + k] * expf(bp.coeff * t * t) * (2.0f * bp.coeff * t);
        }
    }
    if (d > 0.f) {
        const float s = gd / d;
        gx = s * vx; gy = s * vy; gz = s * vz;
    }
    if (grad_wig) {
        Dual3 q[4];
        const Dual3 dx{vx, 1.f, 0.f, 0.f}, dy{vy, 0.f, 1.f, 0.f}, dz{vz, 0.f, 0.f, 1.f};
        edge_quaternion<Dual3>(dx, dy, dz, gamma ? gamma[e] : 0.f, q);
        const float* gw = grad_wig + e * Shape<LMAX>::kW;
        wigner_compact<LMAX, Dual3>(q, [&](int i, Dual3 v) {
            const float g = gw[i];
            gx = fmaf(g, v.a, gx);
            gy = fmaf(g, v.b, gy);
            gz = fmaf(g, v.c, gz);
        });
    }
    grad_vec[e * 3 + 0] = gx;
    grad_vec[e * 3 + 1] = gy;
    grad_vec[e * 3 + 2] = gz;
}

static BasisParams make_basis(float cutoff, int32_t num_basis, float start, float stop, float width) {
    BasisParams bp;
    bp.cutoff = cutoff;
    bp.num = num_basis;
    bp.start = start;
    bp.step = num_basis > 1 ? (stop - start) / (float)(num_basis - 1) : 0.f;
    const float w = width * bp.step;
    bp.coeff = w != 0.f ? -0.5f / (w * w) : 0.f;
    return bp;
}

}  // namespace fcb200

using namespace fcb200;

extern "C" {

int fcb200_lx_edge_geometry_fwd(const float* pos, const int32_t* src, const int32_t* tgt, const float* shift, const float* gamma,
                                float* vec, float* dist, float* env, float* wig, float* gauss, float cutoff, int32_t num_basis,
                                float basis_start, float basis_stop, float basis_width, int64_t num_edges, int64_t num_nodes,
                                int32_t lmax, void* stream) {
    if (!pos || !src || !tgt || num_edges < 0 || num_nodes < 0 || cutoff <= 0.f) return FCB200_EINVAL;
    if (gauss && num_basis < 2) return FCB200_EINVAL;
    if (lmax != 2 && lmax != 4) return FCB200_EINVAL;
    if (num_edges == 0) return FCB200_OK;
    const BasisParams bp = make_basis(cutoff, num_basis, basis_start, basis_stop, basis_width);
    const unsigned grid = (unsigned)((num_edges + 127) / 128);
    if (lmax == 2)
        edge_geometry_fwd_kernel<2><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(pos, src, tgt, shift, gamma, vec, dist, env,
                                                                                         wig, gauss, bp, num_edges);
    else
        edge_geometry_fwd_kernel<4><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(pos, src, tgt, shift, gamma, vec, dist, env,
                                                                                         wig, gauss, bp, num_edges);
    return launch_status();
}

int fcb200_lx_edge_geometry_bwd(const float* pos, const int32_t* src, const int32_t* tgt, const float* shift, const float* gamma,
                                const float* grad_wig, const float* grad_env, const float* grad_gauss, const float* grad_dist,
                                float* grad_vec, float cutoff, int32_t num_basis, float basis_start, float basis_stop,
                                float basis_width, int64_t num_edges, int64_t num_nodes, int32_t lmax, void* stream) {
    if (!pos || !src || !tgt || !grad_vec || num_edges < 0 || num_nodes < 0 || cutoff <= 0.f) return FCB200_EINVAL;
    if (grad_gauss && num_basis < 2) return FCB200_EINVAL;
    if (lmax != 2 && lmax != 4) return FCB200_EINVAL;
    if (num_edges == 0) return FCB200_OK;
    const BasisParams bp = make_basis(cutoff, num_basis, basis_start, basis_stop, basis_width);
    const unsigned grid = (unsigned)((num_edges + 127) / 128);
    if (lmax == 2)
        edge_geometry_bwd_kernel<2><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
            pos, src, tgt, shift, gamma, grad_wig, grad_env, grad_gauss, grad_dist, grad_vec, bp, num_edges);
    else
        edge_geometry_bwd_kernel<4><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
            pos, src, tgt, shift, gamma, grad_wig, grad_env, grad_gauss, grad_dist, grad_vec, bp, num_edges);
    return launch_status();
}

int fcb200_edge_geometry_fwd(const float* pos, const int32_t* src, const int32_t* tgt, const float* shift, const float* gamma,
                             float* vec, float* dist, float* env, float* wig, float* gauss, float cutoff, int32_t num_basis,
                             float basis_start, float basis_stop, float basis_width, int64_t num_edges, int64_t num_nodes,
                             void* stream) {
    return fcb200_lx_edge_geometry_fwd(pos, src, tgt, shift, gamma, vec, dist, env, wig, gauss, cutoff, num_basis, basis_start,
                                       basis_stop, basis_width, num_edges, num_nodes, 2, stream);
}

int fcb200_edge_geometry_bwd(const float* pos, const int32_t* src, const int32_t* tgt, const float* shift, const float* gamma,
                             const float* grad_wig, const float* grad_env, const float* grad_gauss, const float* grad_dist,
                             float* grad_vec, float cutoff, int32_t num_basis, float basis_start, float basis_stop,
                             float basis_width, int64_t num_edges, int64_t num_nodes, void* stream) {
    return fcb200_lx_edge_geometry_bwd(pos, src, tgt, shift, gamma, grad_wig, grad_env, grad_gauss, grad_dist, grad_vec, cutoff,
                                       num_basis, basis_start, basis_stop, basis_width, num_edges, num_nodes, 2, stream);
}

}  // extern "C"
