// Periodic radius graph as integer cell-list kernels (sm_100a).
//
// Candidate pairs come from a uniform grid (cell size >= radius/2, +-2 cell stencil); which pairs
// are kept is decided by float32 arithmetic carried out in a fixed order with explicit
// round-to-nearest multiplies and adds, never contracted into FMAs:
//     source = pos[src] + ((n0*c0 + n1*c1) + n2*c2)          (periodic image n of the source atom)
//     d      = target - source,   d2 = (dx*dx + dy*dy) + dz*dz
//     keep candidates with d2 <= r*r and d2 != 0
//     a target with more than k candidates keeps d2 <= d2_sorted[k] + 0.01f
// Bucket contents are sorted by source id and candidates are enumerated stencil-row by
// stencil-row, so the output order is fixed from run to run.
#include "common.cuh"

namespace fcb200 {

struct Sys {
    int atom_begin, atom_end, r0, r1, r2, nimg, source_begin, grid_begin, d0, d1, d2;
    float ox, oy, oz, inv_h;
    float c[9];
};

__device__ __forceinline__ Sys load_sys(const int32_t* __restrict__ sys, int s) {
    const int32_t* w = sys + (int64_t)s * FCB200_SYS_WORDS;
    Sys v;
    v.atom_begin = w[0]; v.atom_end = w[1]; v.r0 = w[2]; v.r1 = w[3]; v.r2 = w[4]; v.nimg = w[5];
    v.source_begin = w[6]; v.grid_begin = w[7]; v.d0 = w[8]; v.d1 = w[9]; v.d2 = w[10];
    v.ox = __int_as_float(w[11]); v.oy = __int_as_float(w[12]); v.oz = __int_as_float(w[13]);
    v.inv_h = __int_as_float(w[14]);
#pragma unroll
    for (int i = 0; i < 9; ++i) v.c[i] = __int_as_float(w[15 + i]);
    return v;
}

__device__ __forceinline__ int find_system(const int32_t* __restrict__ sys, int nsys, int64_t sid) {
    int lo = 0, hi = nsys - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((int64_t)sys[(int64_t)mid * FCB200_SYS_WORDS + 6] <= sid) lo = mid; else hi = mid - 1;
    }
    return lo;
}

__device__ __forceinline__ void decode_image(const Sys& s, int img, int& n0, int& n1, int& n2) {
    const int w2 = 2 * s.r2 + 1, w1 = 2 * s.r1 + 1;
    n2 = img % w2 - s.r2;
    img /= w2;
    n1 = img % w1 - s.r1;
    n0 = img / w1 - s.r0;
}

// position of periodic image (n0,n1,n2) of an atom; each product and sum rounded separately
__device__ __forceinline__ void image_position(const Sys& s, const float* __restrict__ pos, int atom, int n0, int n1, int n2,
                                               float& px, float& py, float& pz) {
    const float f0 = (float)n0, f1 = (float)n1, f2 = (float)n2;
    const float ox = __fadd_rn(__fadd_rn(__fmul_rn(f0, s.c[0]), __fmul_rn(f1, s.c[3])), __fmul_rn(f2, s.c[6]));
    const float oy = __fadd_rn(__fadd_rn(__fmul_rn(f0, s.c[1]), __fmul_rn(f1, s.c[4])), __fmul_rn(f2, s.c[7]));
    const float oz = __fadd_rn(__fadd_rn(__fmul_rn(f0, s.c[2]), __fmul_rn(f1, s.c[5])), __fmul_rn(f2, s.c[8]));
    px = __fadd_rn(pos[(int64_t)atom * 3 + 0], ox);
    py = __fadd_rn(pos[(int64_t)atom * 3 + 1], oy);
    pz = __fadd_rn(pos[(int64_t)atom * 3 + 2], oz);
}

__device__ __forceinline__ void grid_coords(const Sys& s, float px, float py, float pz, int& gx, int& gy, int& gz) {
    gx = (int)floorf((px - s.ox) * s.inv_h);
    gy = (int)floorf((py - s.oy) * s.inv_h);
    gz = (int)floorf((pz - s.oz) * s.inv_h);
}

__device__ __forceinline__ bool source_of(const int32_t* __restrict__ sys, int nsys, const float* __restrict__ pos, int64_t sid,
                                          Sys& s, float& px, float& py, float& pz, int& cell) {
    s = load_sys(sys, find_system(sys, nsys, sid));
    const int local = (int)(sid - s.source_begin);
    const int atom = s.atom_begin + local / s.nimg;
    int n0, n1, n2;
    decode_image(s, local % s.nimg, n0, n1, n2);
    image_position(s, pos, atom, n0, n1, n2, px, py, pz);
    int gx, gy, gz;
    grid_coords(s, px, py, pz, gx, gy, gz);
    if (gx < 0 || gy < 0 || gz < 0 || gx >= s.d0 || gy >= s.d1 || gz >= s.d2) {
        cell = -1;
        return false;
    }
    cell = s.grid_begin + gx + s.d0 * (gy + s.d1 * gz);
    return true;
}

// max_cells bounds the cell index against the caller's arrays: a system table that describes more cells than the
// caller sized its counters for must not write past them (such sources are dropped like sources outside the grid)
__global__ void rg_count_sources_kernel(const float* __restrict__ pos, const int32_t* __restrict__ sys, int nsys,
                                        int64_t num_sources, int32_t* __restrict__ cell_count, int32_t* __restrict__ source_cell,
                                        int64_t max_cells) {
    const int64_t sid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (sid >= num_sources) return;
    Sys s;
    float px, py, pz;
    int cell;
    if (source_of(sys, nsys, pos, sid, s, px, py, pz, cell) && cell < max_cells) atomicAdd(cell_count + cell, 1);
    else cell = -1;
    source_cell[sid] = cell;
}

__global__ void rg_fill_kernel(const float* __restrict__ pos, const int32_t* __restrict__ sys, int nsys, int64_t num_sources,
                               const int32_t* __restrict__ source_cell, const int32_t* __restrict__ cell_ptr,
                               int32_t* __restrict__ cell_fill, float4* __restrict__ bucket) {
    const int64_t sid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (sid >= num_sources) return;
    const int cell = source_cell[sid];
    if (cell < 0) return;
    Sys s;
    float px, py, pz;
    int c2;
    source_of(sys, nsys, pos, sid, s, px, py, pz, c2);
    const int slot = atomicAdd(cell_fill + cell, 1);
    bucket[cell_ptr[cell] + slot] = make_float4(px, py, pz, __int_as_float((int)sid));
}

// order each bucket by source id (buckets hold a handful of entries)
__global__ void rg_sort_buckets_kernel(const int32_t* __restrict__ cell_ptr, float4* __restrict__ bucket, int64_t num_cells) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= num_cells) return;
    const int b = cell_ptr[c], e = cell_ptr[c + 1];
    for (int i = b + 1; i < e; ++i) {
        const float4 v = bucket[i];
        const int key = __float_as_int(v.w);
        int j = i - 1;
        while (j >= b && __float_as_int(bucket[j].w) > key) {
            bucket[j + 1] = bucket[j];
            --j;
        }
        bucket[j + 1] = v;
    }
}

__global__ void __launch_bounds__(1024) exclusive_scan_kernel(const int32_t* __restrict__ counts, int32_t* __restrict__ ptr, int64_t n) {
    __shared__ int warp_tot[32];
    __shared__ int carry;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (tid == 0) carry = 0;
    __syncthreads();
    for (int64_t base = 0; base < n; base += 4096) {
        const int64_t i0 = base + (int64_t)tid * 4;
        int v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = i0 + j < n ? counts[i0 + j] : 0;
        const int tsum = v[0] + v[1] + v[2] + v[3];
        int incl = tsum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        if (wid == 0) {
            const int t0 = warp_tot[lane];
            int wi = t0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(kFull, wi, o);
                if (lane >= o) wi += t;
            }
            warp_tot[lane] = wi - t0;  // exclusive over warps
        }
        __syncthreads();
        int run = carry + warp_tot[wid] + incl - tsum;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (i0 + j < n) ptr[i0 + j] = run;
            run += v[j];
        }
        __syncthreads();
        if (tid == 1023) carry = run;
        __syncthreads();
    }
    if (tid == 0) ptr[n] = carry;
}

__device__ __forceinline__ float dist_sq(float tx, float ty, float tz, float4 sp) {
    const float dx = __fsub_rn(tx, sp.x), dy = __fsub_rn(ty, sp.y), dz = __fsub_rn(tz, sp.z);
    return __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz));
}

// one warp per target; lanes 0..24 each own one (dy,dz) stencil row of 5 x-contiguous cells
__global__ void __launch_bounds__(256)
    rg_search_kernel(const float* __restrict__ pos, const int32_t* __restrict__ sys, const int32_t* __restrict__ targets,
                     const int32_t* __restrict__ target_sys, int64_t num_targets, const int32_t* __restrict__ cell_ptr,
                     const float4* __restrict__ bucket, float radius_sq, int32_t* __restrict__ cand_count,
                     const int32_t* __restrict__ cand_ptr, int32_t* __restrict__ cand_id, float* __restrict__ cand_d2) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= num_targets) return;
    const int atom = targets ? targets[t] : (int)t;
    const Sys s = load_sys(sys, target_sys[t]);
    const float tx = pos[(int64_t)atom * 3 + 0], ty = pos[(int64_t)atom * 3 + 1], tz = pos[(int64_t)atom * 3 + 2];
    int gx, gy, gz;
    grid_coords(s, tx, ty, tz, gx, gy, gz);
    gx = min(max(gx, 0), s.d0 - 1);
    gy = min(max(gy, 0), s.d1 - 1);
    gz = min(max(gz, 0), s.d2 - 1);
    int b = 0, e = 0;
    if (lane < 25) {
        const int yy = gy + lane / 5 - 2, zz = gz + lane % 5 - 2;
        if (yy >= 0 && yy < s.d1 && zz >= 0 && zz < s.d2) {
            const int x0 = max(gx - 2, 0), x1 = min(gx + 2, s.d0 - 1);
            const int c0 = s.grid_begin + x0 + s.d0 * (yy + s.d1 * zz);
            b = cell_ptr[c0];
            e = cell_ptr[c0 + (x1 - x0) + 1];
        }
    }
    int cnt = 0;
    for (int i = b; i < e; ++i) {
        const float d2 = dist_sq(tx, ty, tz, bucket[i]);
        cnt += (d2 <= radius_sq && d2 != 0.0f) ? 1 : 0;
    }
    if (cand_ptr == nullptr) {
        const int tot = warp_sum_i(cnt);
        if (lane == 0) cand_count[t] = tot;
        return;
    }
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(kFull, incl, o);
        if (lane >= o) incl += v;
    }
    int w = cand_ptr[t] + incl - cnt;
    for (int i = b; i < e; ++i) {
        const float4 sp = bucket[i];
        const float d2 = dist_sq(tx, ty, tz, sp);
        if (d2 <= radius_sq && d2 != 0.0f) {
            cand_id[w] = __float_as_int(sp.w);
            cand_d2[w] = d2;
            ++w;
        }
    }
}

// Distances of a kept candidate list at new positions: same arithmetic as the search (image position as the binning
// computes it, unfused squared distance), +inf for a pair that is out of range now.  One warp per target.
__global__ void __launch_bounds__(256)
    rg_refresh_kernel(const float* __restrict__ pos, const int32_t* __restrict__ sys, int nsys, const int32_t* __restrict__ targets,
                      int64_t num_targets, const int32_t* __restrict__ cand_ptr, const int32_t* __restrict__ cand_id,
                      float radius_sq, float* __restrict__ cand_d2) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= num_targets) return;
    const int atom = targets ? targets[t] : (int)t;
    const float tx = pos[(int64_t)atom * 3 + 0], ty = pos[(int64_t)atom * 3 + 1], tz = pos[(int64_t)atom * 3 + 2];
    const int b = cand_ptr[t], e = cand_ptr[t + 1];
    for (int i = b + lane; i < e; i += 32) {
        Sys s;
        float px, py, pz;
        int cell;
        source_of(sys, nsys, pos, cand_id[i], s, px, py, pz, cell);
        const float d2 = dist_sq(tx, ty, tz, make_float4(px, py, pz, 0.f));
        cand_d2[i] = (d2 <= radius_sq && d2 != 0.0f) ? d2 : __int_as_float(0x7f800000);
    }
}

// one warp per target: max-neighbour threshold by bisection on the float bit patterns, then ordered compaction
__global__ void __launch_bounds__(256)
    rg_select_kernel(const int32_t* __restrict__ sys, const int32_t* __restrict__ targets, const int32_t* __restrict__ target_sys,
                     int64_t num_targets, const int32_t* __restrict__ cand_ptr, const int32_t* __restrict__ cand_id,
                     const float* __restrict__ cand_d2, int max_neighbors, int strict, int32_t* __restrict__ keep_count,
                     const int32_t* __restrict__ edge_ptr, int64_t* __restrict__ edge_src, int64_t* __restrict__ edge_tgt,
                     int32_t* __restrict__ edge_offsets) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= num_targets) return;
    const int b = cand_ptr[t], m = cand_ptr[t + 1] - b;
    // entries marked +inf are candidates of a wider list that are out of range now (fcb200_rg_refresh): never kept
    constexpr unsigned kInf = 0x7f800000u;
    float thr = __uint_as_float(kInf - 1u);  // largest finite value: keep every live candidate
    int live = m;
    if (max_neighbors > 0 && m > max_neighbors) {
        int c = 0;
        for (int i = lane; i < m; i += 32) c += (__float_as_uint(cand_d2[b + i]) < kInf) ? 1 : 0;
        live = warp_sum_i(c);
    }
    if (max_neighbors > 0 && live > max_neighbors) {
        unsigned lo = 0u, hi = kInf;
        while (lo < hi) {  // at most 31 rounds
            const unsigned mid = lo + ((hi - lo) >> 1);
            int c = 0;
            for (int i = lane; i < m; i += 32) c += (__float_as_uint(cand_d2[b + i]) <= mid) ? 1 : 0;
            c = warp_sum_i(c);
            if (c >= max_neighbors + (strict ? 0 : 1)) hi = mid; else lo = mid + 1;
        }
        thr = fminf(__fadd_rn(__uint_as_float(lo), 0.01f), __uint_as_float(kInf - 1u));
        if (strict) thr = __uint_as_float(lo);  // exactly the k nearest: see below
    }
    // strict rule (enforce_max_neighbors_strictly, radius_graph_pbc.py:151-154): the k nearest and nothing else.  The
    // bisection above found the k-th smallest value; everything below it is kept and the first of the candidates
    // equal to it, in list order, fill what is left of the k places.
    int quota = 0;
    const bool strict_cut = strict && max_neighbors > 0 && live > max_neighbors;
    if (strict_cut) {
        int c = 0;
        for (int i = lane; i < m; i += 32) c += (cand_d2[b + i] < thr) ? 1 : 0;
        quota = max_neighbors - warp_sum_i(c);
    }
    if (edge_ptr == nullptr) {
        int c = 0;
        for (int i = lane; i < m; i += 32) c += (strict_cut ? cand_d2[b + i] < thr : cand_d2[b + i] <= thr) ? 1 : 0;
        c = warp_sum_i(c);
        if (lane == 0) keep_count[t] = c + (strict_cut ? quota : 0);
        return;
    }
    const Sys s = load_sys(sys, target_sys[t]);
    const int atom = targets ? targets[t] : (int)t;
    int w = edge_ptr[t];
    int ties_taken = 0;
    for (int i0 = 0; i0 < m; i0 += 32) {
        const int i = i0 + lane;
        const float d2 = i < m ? cand_d2[b + i] : __uint_as_float(kInf);
        bool keep = i < m && (strict_cut ? d2 < thr : d2 <= thr);
        if (strict_cut) {
            const unsigned tied = __ballot_sync(kFull, i < m && d2 == thr);
            keep = keep || (i < m && d2 == thr && ties_taken + __popc(tied & ((1u << lane) - 1u)) < quota);
            ties_taken += __popc(tied);
        }
        const unsigned mask = __ballot_sync(kFull, keep);
        if (keep) {
            const int64_t o = w + __popc(mask & ((1u << lane) - 1u));
            const int local = cand_id[b + i] - s.source_begin;
            int n0, n1, n2;
            decode_image(s, local % s.nimg, n0, n1, n2);
            edge_src[o] = s.atom_begin + local / s.nimg;
            edge_tgt[o] = atom;
            edge_offsets[o * 3 + 0] = n0;
            edge_offsets[o * 3 + 1] = n1;
            edge_offsets[o * 3 + 2] = n2;
        }
        w += __popc(mask);
    }
}

// ---------------------------------------------------------------------------------------------
// allocation-free variant of the candidate search
// ---------------------------------------------------------------------------------------------
// Scratch of the cell list for fcb200_rg_neighbor_counts_static: counters, offsets and fill cursors
// for up to kStaticMaxCells grid cells, the cell of each source and the bucket array for up to
// kStaticMaxSources image-replicated source atoms (about 6 MiB).  Every GPU that loads the library
// holds this array until the process exits.
constexpr int64_t kStaticMaxCells = FCB200_STATIC_MAX_CELLS;
constexpr int64_t kStaticMaxSources = FCB200_STATIC_MAX_SOURCES;
constexpr int64_t kOffCount = 0;
constexpr int64_t kOffPtr = kOffCount + (kStaticMaxCells + 64) * 4;
constexpr int64_t kOffFill = kOffPtr + (kStaticMaxCells + 64) * 4;
constexpr int64_t kOffSourceCell = kOffFill + (kStaticMaxCells + 64) * 4;
constexpr int64_t kOffBucket = kOffSourceCell + kStaticMaxSources * 4;
constexpr int64_t kStaticBytes = kOffBucket + kStaticMaxSources * 16;
static_assert(kOffBucket % 256 == 0 && kOffPtr % 256 == 0 && kOffFill % 256 == 0 && kOffSourceCell % 256 == 0, "sub-arrays stay aligned");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

// In host code the name above is only a handle of the symbol, not an address the GPU can use: the
// device address has to be asked for, once per device, with that device current.
constexpr int kMaxDevices = 64;
static unsigned char* g_static_scratch_addr[kMaxDevices] = {};

static int static_scratch_address(unsigned char** out) {
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (dev < 0 || dev >= kMaxDevices) return FCB200_ERANGE;
    if (g_static_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_static_scratch);
        if (err != cudaSuccess) return static_cast<int>(err);
        g_static_scratch_addr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_static_scratch_addr[dev];
    return FCB200_OK;
}

}  // namespace fcb200

using namespace fcb200;

extern "C" {

int fcb200_rg_count_sources(const float* pos, const int32_t* sys, int32_t num_systems, int64_t num_sources, int32_t* cell_count,
                            int32_t* source_cell, void* stream) {
    if (!pos || !sys || !cell_count || !source_cell || num_systems <= 0 || num_sources < 0) return FCB200_EINVAL;
    if (num_sources >= (1LL << 31)) return FCB200_ERANGE;
    if (num_sources == 0) return FCB200_OK;
    rg_count_sources_kernel<<<(unsigned)((num_sources + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        pos, sys, num_systems, num_sources, cell_count, source_cell, (int64_t)1 << 40);  // the caller sized cell_count from the same table
    return launch_status();
}

int fcb200_exclusive_scan_i32(const int32_t* counts, int32_t* ptr, int64_t n, void* stream) {
    if (!ptr || n < 0 || (n > 0 && !counts)) return FCB200_EINVAL;
    if (n >= (1LL << 31)) return FCB200_ERANGE;
    exclusive_scan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(counts, ptr, n);
    return launch_status();
}

int fcb200_rg_fill_buckets(const float* pos, const int32_t* sys, int32_t num_systems, int64_t num_sources,
                           const int32_t* source_cell, const int32_t* cell_ptr, int32_t* cell_fill, float* bucket,
                           int64_t num_cells, void* stream) {
    if (!pos || !sys || !source_cell || !cell_ptr || !cell_fill || num_systems <= 0 || num_sources < 0 || num_cells < 0)
        return FCB200_EINVAL;
    if (num_sources == 0 || num_cells == 0) return FCB200_OK;
    if (!bucket) return FCB200_EINVAL;
    if (!aligned16(bucket)) return FCB200_EALIGN;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rg_fill_kernel<<<(unsigned)((num_sources + 255) / 256), 256, 0, s>>>(pos, sys, num_systems, num_sources, source_cell, cell_ptr,
                                                                         cell_fill, reinterpret_cast<float4*>(bucket));
    int rc = launch_status();
    if (rc) return rc;
    rg_sort_buckets_kernel<<<(unsigned)((num_cells + 255) / 256), 256, 0, s>>>(cell_ptr, reinterpret_cast<float4*>(bucket), num_cells);
    return launch_status();
}

int fcb200_rg_search(const float* pos, const int32_t* sys, const int32_t* targets, const int32_t* target_sys, int64_t num_targets,
                     const int32_t* cell_ptr, const float* bucket, float radius_sq, int32_t* cand_count, const int32_t* cand_ptr,
                     int32_t* cand_id, float* cand_d2, void* stream) {
    if (!pos || !sys || !target_sys || !cell_ptr || num_targets < 0) return FCB200_EINVAL;
    if (cand_ptr == nullptr ? !cand_count : (!cand_id || !cand_d2)) return FCB200_EINVAL;
    if (bucket && !aligned16(bucket)) return FCB200_EALIGN;
    if (num_targets == 0) return FCB200_OK;
    rg_search_kernel<<<(unsigned)((num_targets + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        pos, sys, targets, target_sys, num_targets, cell_ptr, reinterpret_cast<const float4*>(bucket), radius_sq, cand_count,
        cand_ptr, cand_id, cand_d2);
    return launch_status();
}

int fcb200_rg_select(const int32_t* sys, const int32_t* targets, const int32_t* target_sys, int64_t num_targets,
                     const int32_t* cand_ptr, const int32_t* cand_id, const float* cand_d2, int32_t max_neighbors, int32_t strict,
                     int32_t* keep_count, const int32_t* edge_ptr, int64_t* edge_src, int64_t* edge_tgt, int32_t* edge_offsets,
                     void* stream) {
    if (!sys || !target_sys || !cand_ptr || num_targets < 0) return FCB200_EINVAL;
    if (edge_ptr == nullptr ? !keep_count : (!edge_src || !edge_tgt || !edge_offsets)) return FCB200_EINVAL;
    if (num_targets == 0) return FCB200_OK;
    rg_select_kernel<<<(unsigned)((num_targets + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sys, targets, target_sys, num_targets, cand_ptr, cand_id, cand_d2, max_neighbors, strict != 0, keep_count, edge_ptr, edge_src,
        edge_tgt, edge_offsets);
    return launch_status();
}

int fcb200_rg_refresh(const float* pos, const int32_t* sys, int32_t num_systems, const int32_t* targets, int64_t num_targets,
                      const int32_t* cand_ptr, const int32_t* cand_id, float radius_sq, float* cand_d2, void* stream) {
    if (!pos || !sys || !cand_ptr || !cand_id || !cand_d2 || num_systems <= 0 || num_targets < 0) return FCB200_EINVAL;
    if (num_targets == 0) return FCB200_OK;
    rg_refresh_kernel<<<(unsigned)((num_targets + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        pos, sys, num_systems, targets, num_targets, cand_ptr, cand_id, radius_sq, cand_d2);
    return launch_status();
}

int fcb200_rg_neighbor_counts_static(const float* pos, const int32_t* sys, int32_t num_systems, int64_t num_sources,
                                     int64_t num_cells, const int32_t* targets, const int32_t* target_sys, int64_t num_targets,
                                     float radius_sq, int32_t* cand_count, void* stream) {
    if (!pos || !sys || !target_sys || !cand_count || num_systems <= 0 || num_sources < 0 || num_cells < 0 || num_targets < 0)
        return FCB200_EINVAL;
    // sizes beyond the built-in scratch are refused, never truncated
    if (num_sources > kStaticMaxSources || num_cells > kStaticMaxCells) return FCB200_ERANGE;
    if (num_targets == 0) return FCB200_OK;
    unsigned char* base = nullptr;
    int rc = static_scratch_address(&base);  // first call on a device resolves the symbol address
    if (rc) return rc;
    int32_t* cell_count = reinterpret_cast<int32_t*>(base + kOffCount);
    int32_t* cell_ptr = reinterpret_cast<int32_t*>(base + kOffPtr);
    int32_t* cell_fill = reinterpret_cast<int32_t*>(base + kOffFill);
    int32_t* source_cell = reinterpret_cast<int32_t*>(base + kOffSourceCell);
    float4* bucket = reinterpret_cast<float4*>(base + kOffBucket);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array still holds the previous call's counters: the two that are accumulated into start at zero
    cudaError_t err = cudaMemsetAsync(cell_count, 0, (size_t)(num_cells + 1) * 4, s);
    if (err != cudaSuccess) return static_cast<int>(err);
    err = cudaMemsetAsync(cell_fill, 0, (size_t)(num_cells + 1) * 4, s);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (num_sources > 0) {
        // num_cells (checked against the fixed scratch above) bounds every cell index the kernels derive from the table
        rg_count_sources_kernel<<<(unsigned)((num_sources + 255) / 256), 256, 0, s>>>(pos, sys, num_systems, num_sources, cell_count,
                                                                                    source_cell, num_cells);
        rc = launch_status();
        if (rc) return rc;
    }
    exclusive_scan_kernel<<<1, 1024, 0, s>>>(cell_count, cell_ptr, num_cells);
    rc = launch_status();
    if (rc) return rc;
    if (num_sources > 0 && num_cells > 0) {
        rg_fill_kernel<<<(unsigned)((num_sources + 255) / 256), 256, 0, s>>>(pos, sys, num_systems, num_sources, source_cell, cell_ptr,
                                                                           cell_fill, bucket);
        rc = launch_status();
        if (rc) return rc;
        rg_sort_buckets_kernel<<<(unsigned)((num_cells + 255) / 256), 256, 0, s>>>(cell_ptr, bucket, num_cells);
        rc = launch_status();
        if (rc) return rc;
    }
    rg_search_kernel<<<(unsigned)((num_targets + 7) / 8), 256, 0, s>>>(pos, sys, targets, target_sys, num_targets, cell_ptr, bucket,
                                                                     radius_sq, cand_count, nullptr, nullptr, nullptr);
    return launch_status();
}

}  // extern "C"
