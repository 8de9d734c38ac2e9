// Compile-time shape tables of the coefficient layouts for any lmax with mmax = 2.
//   node features   [N, (lmax+1)^2, C]  L-major
//   edge features   [E, kM, w]          M-major rows: m=0 (l=0..lmax) | m=+1 (l=1..) | m=-1 | m=+2 (l=2..) | m=-2
//   compact Wigner  [E, kW]             block l holds rows m = -mm..mm (mm = min(l,2)) x columns m' = -l..l of D^l
#pragma once

namespace fcb200 {

template <int LMAX> struct Shape {
    static constexpr int kL = (LMAX + 1) * (LMAX + 1);
    __host__ __device__ static constexpr int mm(int l) { return l < 2 ? l : 2; }
    __host__ __device__ static constexpr int rows(int l) { return 2 * mm(l) + 1; }
    __host__ __device__ static constexpr int woff(int l) {
        int s = 0;
        for (int i = 0; i < l; ++i) s += rows(i) * (2 * i + 1);
        return s;
    }
    static constexpr int kW = woff(LMAX + 1);
    __host__ __device__ static constexpr int nm() {
        int s = 0;
        for (int i = 0; i <= LMAX; ++i) s += rows(i);
        return s;
    }
    static constexpr int kM = nm();
    static constexpr int kRad = 3 * LMAX;  // radial slots: (lmax+1) + lmax + (lmax-1)
    // M-major position of coefficient (l, m), |m| <= 2
    __host__ __device__ static constexpr int mrow(int l, int m) {
        if (m == 0) return l;
        if (m == 1) return (LMAX + 1) + (l - 1);
        if (m == -1) return (LMAX + 1) + LMAX + (l - 1);
        if (m == 2) return (LMAX + 1) + 2 * LMAX + (l - 2);
        return (LMAX + 1) + 2 * LMAX + (LMAX - 1) + (l - 2);
    }
    __host__ __device__ static constexpr int radslot(int l, int m) {
        const int a = m < 0 ? -m : m;
        return a == 0 ? l : (a == 1 ? (LMAX + 1) + (l - 1) : (LMAX + 1) + LMAX + (l - 2));
    }
};

static_assert(Shape<2>::kW == 35 && Shape<2>::kM == 9 && Shape<2>::kRad == 6, "lmax = 2 tables");
static_assert(Shape<4>::kW == 115 && Shape<4>::kM == 19 && Shape<4>::kRad == 12, "lmax = 4 tables");
static_assert(Shape<2>::mrow(2, -2) == 8 && Shape<2>::mrow(1, -1) == 5 && Shape<4>::mrow(4, -2) == 18, "M-major order");

}  // namespace fcb200
