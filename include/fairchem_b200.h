/*
 * fairchem_b200 -- C ABI of the B200 (sm_100a) edge message-passing path of eSCN-MD / UMA.
 *
 * Every entry point is what a binding of fairchem's per-layer edge block would call in place
 * of the reference's Triton ops / ATen calls.  Citations are paths inside
 * facebookresearch/fairchem (file:line).
 *
 * Conventions
 *   - all pointers are DEVICE pointers of the current CUDA device unless a name ends in _host;
 *   - the caller owns every buffer (inputs, outputs and scratch) and the stream; entry points
 *     neither allocate, free nor synchronise;
 *   - float tensors are contiguous float32; rows that are read as float4 must be 16-byte aligned;
 *   - edges are CSR-sorted by target node: row_ptr[n]..row_ptr[n+1] are the edges whose target is n;
 *   - node features are L-major [N, (lmax+1)^2, C]; edge features are M-major
 *     (m=0:(l=0..lmax) | m=+1:(l=1..) | m=-1 | m=+2 | m=-2), lmax = mmax = 2, C a multiple of 128;
 *   - `wig` is the block-diagonal Wigner-D of an edge in compact form [E, 35]:
 *     entry 0 = l0 block, entries 1..9 = l1 block (3x3 row-major), 10..34 = l2 block (5x5 row-major);
 *   - return value: 0 on success, a negative FCB200_E* code otherwise (nothing was launched),
 *     or a positive cudaError_t from the launch.
 */
#ifndef FAIRCHEM_B200_H
#define FAIRCHEM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FCB200_OK 0
#define FCB200_EINVAL (-1)   /* null pointer, negative size or unsupported shape */
#define FCB200_EALIGN (-2)   /* pointer not 16-byte aligned */
#define FCB200_ERANGE (-3)   /* size exceeds a documented limit */

#define FCB200_WIG 35        /* compact Wigner entries per edge for lmax = 2 */

/* Library/ABI version (major*1000 + minor). */
int fcb200_version(void);

/* ---------------------------------------------------------------- edge block, forward */

/*
 * Gather source and target node rows of every edge, rotate them into the edge frame and emit
 * the M-major, GEMM-ready operands of the first SO(2) convolution.
 * Replaces ExecutionBackend.node_to_edge_wigner_permute
 * (src/fairchem/core/models/uma/nn/execution_backends.py:160-182) and, with `radial` != NULL,
 * UMASFastGPUBackend.fused_node_to_edge_conv1_pack (execution_backends.py:432-461; Triton kernel
 * wigner_conv1_fused_fwd_kernel, src/fairchem/core/models/uma/triton/kernels.py:1589).
 *   x        [N, 9, C]         node features
 *   src,tgt  [E] int32         node index of the edge's source / target
 *   wig      [E, 35]           compact Wigner-D (edge frame <- global frame)
 *   radial   [E, 6*2C] or NULL per-edge radial weights: [3*2C | 2*2C | 2C] for m = 0,1,2
 *   out      [E, 9, 2C]        M-major rows; the SO(2) GEMMs read their operands as column ranges of the
 *                              flattened [E, 9*2C] matrix: rows 0-2 (m=0), rows 3-6 (m=1: real pair |
 *                              imaginary pair, the operand of the block-form GEMM), rows 7-8 (m=2)
 */
int fcb200_gather_rotate_fwd(const float* x, const int32_t* src, const int32_t* tgt, const float* wig,
                             const float* radial, float* out, int64_t num_edges, int64_t num_nodes, int32_t channels,
                             void* stream);

/*
 * Rotate edge messages back to the global frame and sum them into their target nodes with a
 * segmented (CSR) reduction: one warp owns one target node, no atomics, fixed summation order.
 * Replaces ExecutionBackend.permute_wigner_inv_edge_to_node (execution_backends.py:184-215) and
 * UMASFastGPUBackend.fused_conv2_inv_edge_to_node (execution_backends.py:463-507; Triton kernel
 * wigner_inv_conv2_fused_fwd_kernel, triton/kernels.py:1964, followed by ATen index_add_).
 *   msg      [E, 9, C]   M-major edge messages
 *   winv     [E, 35]     compact inverse rotation with the envelope folded in
 *   row_ptr  [N+1] int32 CSR offsets by target
 *   out      [N, 9, C]   L-major node rows (every row is written; empty segments give zeros)
 */
int fcb200_rotate_back_reduce_fwd(const float* msg, const float* winv, const int32_t* row_ptr, float* out,
                                  int64_t num_edges, int64_t num_nodes, int32_t channels, void* stream);

/*
 * Edge-degree embedding: rotate the m=0 radial coefficients of every edge to the global frame,
 * segment-sum by target, scale by 1/rescale and add to x_in.
 * Replaces ExecutionBackend.edge_degree_scatter (execution_backends.py:217-263).
 *   radial3  [E, 3, C]   m=0 coefficients (l = 0,1,2)
 *   x_in     [N, 9, C] or NULL
 *   out      [N, 9, C]   x_in + sum/rescale
 */
int fcb200_edge_degree_fwd(const float* radial3, const float* winv, const int32_t* row_ptr, const float* x_in,
                           float* out, float rescale, int64_t num_edges, int64_t num_nodes, int32_t channels,
                           void* stream);

/* ---------------------------------------------------------------- edge block, backward */

/*
 * Backward of fcb200_gather_rotate_fwd w.r.t. x (per edge, before the node reduction), wig and
 * radial.  Replaces wigner_conv1_fused_bwd_kernel (triton/kernels.py:1697) /
 * node_to_edge_wigner_permute_bwd_dx_kernel (triton/kernels.py:573) plus the torch.bmm for dW
 * (src/fairchem/core/models/uma/triton/node_to_edge_wigner_permute.py:148-167).
 *   grad_out   [E, 9, 2C]
 *   g_src      [E, 9, C]   out: W^T grad (source half), L-major, to be summed by source node
 *   g_tgt      [E, 9, C]   out: W^T grad (target half), L-major, to be summed by target node
 *   grad_wig   [E, 35]     out
 *   grad_radial[E, 6*2C]   out, or NULL when radial == NULL
 */
int fcb200_gather_rotate_bwd(const float* grad_out, const float* x, const int32_t* src, const int32_t* tgt,
                             const float* wig, const float* radial, float* g_src, float* g_tgt, float* grad_wig,
                             float* grad_radial, int64_t num_edges, int64_t num_nodes, int32_t channels,
                             void* stream);

/*
 * fcb200_gather_rotate_bwd for a run of edges that is CSR-sorted by target (the chunks of the edge block are): the
 * source half is done per edge as above, the target half by one warp per target node, which sums the node gradient
 * over the target's edges in registers and ADDS it to the node's row once -- the reference scatters both halves with
 * index_add_ atomics (src/fairchem/core/models/uma/triton/fused_wigner.py:228-236).  No per-edge target gradient is
 * written and none has to be reduced afterwards.  lmax = 2, channels = 128.
 *   row_ptr  [num_targets + 1] int32, relative to the first edge of the run; target t is node tgt_base + t
 *   g_src    [E, 9, C]  out, to be summed by source node (fcb200_segment_sum)
 *   gx_tgt   [num_targets, 9, C]  in/out: rows of the node-gradient array starting at node tgt_base
 */
int fcb200_gather_rotate_bwd_csr(const float* grad_out, const float* x, const int32_t* src, const int32_t* tgt,
                                 const int32_t* row_ptr, int64_t tgt_base, int64_t num_targets, const float* wig,
                                 const float* radial, float* g_src, float* gx_tgt, float* grad_wig, float* grad_radial,
                                 int64_t num_edges, int64_t num_nodes, int32_t channels, void* stream);
/* fcb200_gather_rotate_bwd_csr with the radial gradient written as half planes (values times *scale, a device pointer to
 * a power of two or NULL): it only feeds the backward contraction of the radial MLP's output layer. */
int fcb200_gather_rotate_bwd_csr_h(const float* grad_out, const float* x, const int32_t* src, const int32_t* tgt,
                                   const int32_t* row_ptr, int64_t tgt_base, int64_t num_targets, const float* wig,
                                   const float* radial, float* g_src, float* gx_tgt, float* grad_wig, void* grad_radial_hi,
                                   void* grad_radial_lo, const float* scale, int64_t num_edges, int64_t num_nodes,
                                   int32_t channels, void* stream);

/*
 * fcb200_gather_rotate_bwd_csr with the source half summed per node as well: one warp per distinct source of the run
 * walks that source's edges through a by-source permutation of the run's edges, sums the node gradient in registers and
 * ADDS it to gx[src_nodes[u]] once, so no per-edge node gradient is written at all (the reference's two index_add_
 * scatters, src/fairchem/core/models/uma/triton/fused_wigner.py:228-236).  lmax = 2, channels = 128.
 *   src_nodes [num_sources] int32   distinct source nodes of the run
 *   src_ptr   [num_sources + 1] int32, src_perm [E] int32: edges of source u are src_perm[src_ptr[u] .. src_ptr[u+1]),
 *             relative to the first edge of the run; every edge of the run appears exactly once
 *   gx        [num_nodes, 9, C]  in/out node-gradient array; targets are the rows from tgt_base on
 */
int fcb200_gather_rotate_bwd_nodes(const float* grad_out, const float* x, const int32_t* src_nodes, const int32_t* src_ptr,
                                   const int32_t* src_perm, int64_t num_sources, const int32_t* row_ptr, int64_t tgt_base,
                                   int64_t num_targets, const float* wig, const float* radial, float* gx, float* grad_wig,
                                   float* grad_radial, int64_t num_edges, int64_t num_nodes, int32_t channels, void* stream);
/* fcb200_gather_rotate_bwd_nodes with the radial gradient as half planes (see fcb200_gather_rotate_bwd_csr_h). */
int fcb200_gather_rotate_bwd_nodes_h(const float* grad_out, const float* x, const int32_t* src_nodes, const int32_t* src_ptr,
                                     const int32_t* src_perm, int64_t num_sources, const int32_t* row_ptr, int64_t tgt_base,
                                     int64_t num_targets, const float* wig, const float* radial, float* gx, float* grad_wig,
                                     void* grad_radial_hi, void* grad_radial_lo, const float* scale, int64_t num_edges,
                                     int64_t num_nodes, int32_t channels, void* stream);

/*
 * Backward of fcb200_rotate_back_reduce_fwd: grad_msg = Winv^T grad_out[tgt] (M-major) and
 * grad_winv = sum_c grad_out[tgt] (x) msg on the block entries.  Replaces
 * permute_wigner_inv_edge_to_node_bwd_dx/_bwd_dw kernels (triton/kernels.py:1181, 1334) and
 * wigner_inv_conv2_fused_bwd_kernel (triton/kernels.py:2015).
 *   msg may be NULL together with grad_winv when only grad_msg is wanted.
 */
int fcb200_rotate_back_bwd(const float* grad_out, const float* msg, const float* winv, const int32_t* tgt,
                           float* grad_msg, float* grad_winv, int64_t num_edges, int64_t num_nodes,
                           int32_t channels, void* stream);

/* Backward of fcb200_edge_degree_fwd w.r.t. radial3 and winv (grad w.r.t. x_in is grad_out). */
int fcb200_edge_degree_bwd(const float* grad_out, const float* radial3, const float* winv, const int32_t* tgt,
                           float* grad_radial3, float* grad_winv, float rescale, int64_t num_edges,
                           int64_t num_nodes, int32_t channels, void* stream);

/*
 * Segmented sum of per-edge rows into node rows:
 *   out[oi(n)] (+)= scale * sum_{k in [ptr[n], ptr[n+1])} rows[perm ? perm[k] : k],  oi(n) = out_index ? out_index[n] : n.
 * The atomic-free replacement of the index_add_ calls in the reference's backward
 * (src/fairchem/core/models/uma/triton/fused_wigner.py:228-236).  out_index entries must be distinct;
 * accumulate != 0 adds to the existing row.  `width` floats per row.
 */
int fcb200_segment_sum(const float* rows, const int32_t* ptr, const int32_t* perm, const int32_t* out_index, float* out,
                       int32_t accumulate, float scale, int64_t num_segments, int64_t width, void* stream);

/* ---------------------------------------------------------------- SO(2) activation glue */

/*
 * Gate activation between the two SO(2) convolutions, one pass.
 * The m>0 convolutions run in block form ([x_re | x_im] @ [[Wa, -Wb], [Wb, Wa]]^T, the reference's
 * SO2_m_Conv_Block, src/fairchem/core/models/uma/nn/so2_layers.py:83-169), so the three conv-1 GEMMs
 * write one matrix y [E, 11H] = [gate scalars 2H | m=0 rows 3H | m=1 rows 4H | m=2 rows 2H] side by side
 * and no separate complex-combine or concatenation pass exists (so2_layers.py:72-80, 642).
 * Replaces GateActivation.forward (src/fairchem/core/models/uma/nn/activation.py:146-165):
 *   out [E, 9, H]: row 0 = SiLU(row 0), rows 1..8 = row * sigmoid(gate of the row's degree).
 */
int fcb200_so2_gate_fwd(const float* y, float* out, int64_t num_edges, int32_t hidden, void* stream);
/* Backward of fcb200_so2_gate_fwd: grad_y [E, 11H] from grad_out [E, 9, H] (y is re-read). */
int fcb200_so2_gate_bwd(const float* grad_out, const float* y, float* grad_y, int64_t num_edges, int32_t hidden,
                        void* stream);

/* ---------------------------------------------------------------- radial MLP hidden activation */

/*
 * out = SiLU(LayerNorm(pre + table_src[z_src] + table_tgt[z_tgt])) over rows of width 128, with the
 * row statistics (mean, 1/std) saved for the backward pass.  One pass, one warp per row.
 * Replaces the LayerNorm + SiLU pairs of RadialMLP (src/fairchem/core/models/uma/nn/radial.py:61-86)
 * and, through the two tables (embedding @ W^T of the first Linear), the source/target embedding
 * columns of x_edge (src/fairchem/core/models/uma/escn_md.py:844-853).  Tables may be NULL.
 *   pre [E,128]; table_* [num_elements,128]; z_* [E] int32; ln_weight, ln_bias [128]; stats [E,2] out
 */
int fcb200_radial_act_fwd(const float* pre, const float* table_src, const float* table_tgt, const int32_t* z_src,
                          const int32_t* z_tgt, const float* ln_weight, const float* ln_bias, float eps, float* out,
                          float* stats, int64_t num_edges, int32_t width, void* stream);
/*
 * fcb200_radial_act_fwd with the activation written as the half-precision split (planes out_hi / out_lo of shape
 * [E,128], scale 1) that the next Linear of the radial MLP reads with fcb200_gemm_f16x2_presplit /
 * fcb200_so2_conv_fused: the hidden activations of RadialMLP (uma/nn/radial.py:61-86) only ever feed a contraction.
 */
int fcb200_radial_act_fwd_h(const float* pre, const float* table_src, const float* table_tgt, const int32_t* z_src,
                            const int32_t* z_tgt, const float* ln_weight, const float* ln_bias, float eps, void* out_hi,
                            void* out_lo, float* stats, int64_t num_edges, int32_t width, void* stream);
/* Backward of fcb200_radial_act_fwd w.r.t. pre (the tables and LayerNorm parameters are frozen). */
int fcb200_radial_act_bwd(const float* grad_out, const float* pre, const float* table_src, const float* table_tgt,
                          const int32_t* z_src, const int32_t* z_tgt, const float* ln_weight, const float* ln_bias,
                          const float* stats, float* grad_pre, int64_t num_edges, int32_t width, void* stream);

/* ---------------------------------------------------------------- node-wise norm */

/*
 * Degree-balanced RMS norm of node features x [N, 9, C] (lmax = 2), one pass:
 *   y_0 = x_0 - mean_c(x_0), y_i = x_i (i > 0);  s = rsqrt(mean_c sum_i y_i^2 / ((2 l_i + 1) * 3) + eps);
 *   out_i = y_i * s * weight[l_i] ; out_0 += bias (+ extra[n], the per-system embedding added after the
 *   first norm of a layer, src/fairchem/core/models/uma/escn_md_block.py:440-443).
 * Replaces EquivariantRMSNormArraySphericalHarmonicsV2.forward
 * (src/fairchem/core/models/uma/nn/layer_norm.py:372-419).  stats [N,2] = (mean_c x_0, s) for the backward.
 */
int fcb200_rms_norm_sh_fwd(const float* x, const float* weight, const float* bias, const float* extra, float* out,
                           float* stats, float eps, int64_t num_nodes, int32_t channels, void* stream);
/* Backward of fcb200_rms_norm_sh_fwd w.r.t. x (affine parameters are frozen; grad of extra is grad_out row 0). */
int fcb200_rms_norm_sh_bwd(const float* grad_out, const float* x, const float* weight, const float* stats,
                           float* grad_x, int64_t num_nodes, int32_t channels, void* stream);

/* ---------------------------------------------------------------- edge geometry */

/*
 * Per-edge geometry from positions: edge vector, length, polynomial envelope (p = 5), Gaussian
 * distance basis and the compact Wigner-D of the rotation edge -> +Y (roll angle gamma).
 * Replaces get_pbc_distances (src/fairchem/core/graph/compute.py:75-113), axis_angle_wigner_hybrid
 * for l <= 2 (src/fairchem/core/models/uma/common/quaternion/wigner_d_hybrid.py:134-205),
 * PolynomialEnvelope and GaussianSmearing (src/fairchem/core/models/uma/nn/radial.py:22-58).
 *   pos [N,3]; src,tgt [E] int32; shift [E,3] = cell_offsets @ cell (or NULL); gamma [E] or NULL (= 0)
 *   vec [E,3], dist [E], env [E], wig [E,35], gauss [E, num_basis] (any of the outputs may be NULL)
 */
int fcb200_edge_geometry_fwd(const float* pos, const int32_t* src, const int32_t* tgt, const float* shift,
                             const float* gamma, float* vec, float* dist, float* env, float* wig, float* gauss,
                             float cutoff, int32_t num_basis, float basis_start, float basis_stop,
                             float basis_width, int64_t num_edges, int64_t num_nodes, void* stream);
/*
 * Backward: d(vec)[E,3] = J^T (grad_wig, grad_env, grad_gauss, grad_dist), by forward-mode
 * differentiation of the same code in the three components of the edge vector.  The caller
 * turns grad_vec into forces with two segmented sums (+ by source, - by target).
 * Replaces the autograd replay of the modules cited above (src/fairchem/core/models/uma/outputs.py:137-162).
 */
int fcb200_edge_geometry_bwd(const float* pos, const int32_t* src, const int32_t* tgt, const float* shift,
                             const float* gamma, const float* grad_wig, const float* grad_env,
                             const float* grad_gauss, const float* grad_dist, float* grad_vec, float cutoff,
                             int32_t num_basis, float basis_start, float basis_stop, float basis_width,
                             int64_t num_edges, int64_t num_nodes, void* stream);

/* ---------------------------------------------------------------- radius graph (cell list) */

/*
 * Periodic radius graph with the reference's float32 membership rule, as integer cell-list
 * kernels.  Replaces radius_graph_pbc_v2 and get_max_neighbors_mask
 * (src/fairchem/core/graph/radius_graph_pbc.py:412-813, 74-189).  The host side
 * (fairchem_b200/graph.py) sizes the buffers between phases.
 *
 * System table `sys` [B, FCB200_SYS_WORDS] int32/float32 words per system:
 *   0 atom_begin  1 atom_end  2..4 reps (images -rep..rep per lattice vector)  5 num_images
 *   6 source_begin (exclusive prefix of natoms*num_images)  7 grid_begin (first cell of its grid)
 *   8..10 grid dims  11..13 grid origin (float bits)  14 inv_cell_size (float bits)
 *   15..23 cell matrix row-major (float bits)
 */
#define FCB200_SYS_WORDS 24

/* Phase 1: count image-replicated source atoms per grid cell (cell_count must be zeroed). */
int fcb200_rg_count_sources(const float* pos, const int32_t* sys, int32_t num_systems, int64_t num_sources,
                            int32_t* cell_count, int32_t* source_cell, void* stream);
/* Exclusive scan of int32 counts into ptr[n+1] (single launch; n <= 2^31-1).  Also usable for CSR offsets. */
int fcb200_exclusive_scan_i32(const int32_t* counts, int32_t* ptr, int64_t n, void* stream);
/* Phase 2: place sources in their cell bucket, bucket entries sorted by source id.
 * bucket [num_kept_sources] float4 = (x, y, z, source id bits); cell_fill must be zeroed. */
int fcb200_rg_fill_buckets(const float* pos, const int32_t* sys, int32_t num_systems, int64_t num_sources,
                           const int32_t* source_cell, const int32_t* cell_ptr, int32_t* cell_fill, float* bucket,
                           int64_t num_cells, void* stream);
/*
 * Phase 3 (two passes): candidates of every target within the radius.  Pass A: cand_ptr == NULL,
 * writes cand_count[t].  Pass B: cand_ptr given, writes cand_id / cand_d2 in a fixed order.
 *   targets [T] int32 atom ids (or NULL = all atoms), target_sys [T] int32 system of each target
 */
int fcb200_rg_search(const float* pos, const int32_t* sys, const int32_t* targets, const int32_t* target_sys,
                     int64_t num_targets, const int32_t* cell_ptr, const float* bucket, float radius_sq,
                     int32_t* cand_count, const int32_t* cand_ptr, int32_t* cand_id, float* cand_d2, void* stream);
/*
 * Phase 4: max-neighbour rule per target (get_max_neighbors_mask, graph/radius_graph_pbc.py:74-189).  strict == 0:
 * keep d2 <= d2_sorted[k] + 0.01f when a target has more than k candidates; strict != 0: exactly the k nearest
 * (candidates tied with the k-th keep their list order).  Candidates marked +inf (fcb200_rg_refresh) are skipped.
 * Pass A: edge_ptr == NULL, writes keep_count[t].  Pass B: writes the kept edges: src/tgt atom ids (int64, the
 * reference's edge_index rows), cell offsets [E,3] int32.
 */
int fcb200_rg_select(const int32_t* sys, const int32_t* targets, const int32_t* target_sys, int64_t num_targets,
                     const int32_t* cand_ptr, const int32_t* cand_id, const float* cand_d2, int32_t max_neighbors, int32_t strict,
                     int32_t* keep_count, const int32_t* edge_ptr, int64_t* edge_src, int64_t* edge_tgt,
                     int32_t* edge_offsets, void* stream);

/*
 * Skin-distance reuse of a candidate list (the Verlet-list practice of MD drivers; the reference rebuilds its graph
 * on every call, src/fairchem/core/calculate/ase_calculator.py:237-240): a list searched once with radius
 * cutoff + skin (fcb200_rg_search) stays a superset of every later neighbourhood while no atom has moved by more
 * than skin / 2.  This entry recomputes the squared distances of the kept candidates at the current positions with
 * the search's own arithmetic and marks pairs beyond radius_sq (or coincident) with +inf; fcb200_rg_select skips
 * such entries, so the selected edge set equals that of a fresh search at the current positions.
 *   cand_ptr [T+1], cand_id [cand_ptr[T]] as written by fcb200_rg_search; cand_d2 [cand_ptr[T]] out
 */
int fcb200_rg_refresh(const float* pos, const int32_t* sys, int32_t num_systems, const int32_t* targets, int64_t num_targets,
                      const int32_t* cand_ptr, const int32_t* cand_id, float radius_sq, float* cand_d2, void* stream);

/*
 * Allocation-free neighbour counting (no counterpart in the reference; added for embedders).
 *
 * Some hosts of this library cannot let it, or themselves, call cudaMalloc inside a time step: an MD
 * engine that reserved the device memory for its own pools at start-up, or a driver loop that must
 * not take the device-wide synchronisation an allocation or a free implies.  For them this entry
 * point runs phases 1-3A above (bin the periodic source images, scan, fill the buckets, count the
 * candidates of every target within the radius) with the cell-list scratch held in a fixed array
 * inside the library instead of caller buffers.  It calls no cudaMalloc/cudaFree and no allocating
 * library routine; the caller still passes inputs and the output.
 *
 *   limits      num_sources <= FCB200_STATIC_MAX_SOURCES and num_cells <= FCB200_STATIC_MAX_CELLS
 *               (about 6 MiB of device memory per GPU that loads the library, held until exit);
 *               larger sizes return FCB200_ERANGE and launch nothing
 *   sys         must describe exactly num_cells grid cells; a source whose cell index falls beyond num_cells is
 *               dropped, never written
 *   first call  on each device looks up the array's device address (cudaGetSymbolAddress); make that
 *               call during set-up, before any stream capture
 *   sharing     all calls on a device use the same array, which keeps the previous call's contents
 *               (the counters that must start at zero are cleared on the stream first); two calls
 *               whose work overlaps on the GPU race on it - serialise them on one stream
 *   cand_count  [num_targets] out: candidates per target, identical to fcb200_rg_search pass A
 */
#define FCB200_STATIC_MAX_SOURCES 262144
#define FCB200_STATIC_MAX_CELLS 65536
int fcb200_rg_neighbor_counts_static(const float* pos, const int32_t* sys, int32_t num_systems, int64_t num_sources,
                                     int64_t num_cells, const int32_t* targets, const int32_t* target_sys,
                                     int64_t num_targets, float radius_sq, int32_t* cand_count, void* stream);

/* ---------------------------------------------------------------- dense contraction */

/*
 * C[M,N] = A[M,K] * W[N,K]^T (+ bias) in float32 through tcgen05 TF32 tensor-core MMAs with float32
 * accumulation in tensor memory (persistent kernel, TMA loads, double-buffered accumulators).
 * precision = 1: single TF32 pass, `w` is the float32 weight, `w_lo` is ignored (may be NULL).
 * precision = 3: `w` = high parts and `w_lo` = low parts produced by fcb200_split_tf32 (same shape and
 * row stride); A is split on the fly and three MMAs per k-step (lo*hi + hi*lo + hi*hi) restore
 * float32-level accuracy.
 * Replaces the cuBLAS calls under SO2_Convolution / SO2_m_Conv
 * (src/fairchem/core/models/uma/nn/so2_layers.py:67-80, 600-647) and RadialMLP
 * (src/fairchem/core/models/uma/nn/radial.py:61-86).  lda/ldw/ldc are row strides in floats (multiples
 * of 4); K and N multiples of 4.  `status` is a device int32 the kernel sets non-zero if one of its
 * bounded waits expired (the result is then invalid).
 */
int fcb200_gemm_tf32(const float* a, int64_t lda, const float* w, const float* w_lo, int64_t ldw, const float* bias,
                     float* c, int64_t ldc, int64_t m, int32_t n, int32_t k, int32_t precision, int32_t* status,
                     void* stream);

/*
 * Split float32 values into TF32 high and low parts: hi = tf32_round(w), lo = tf32_round(w - hi).
 * Done once per weight matrix; there is no counterpart in the reference (its float32 GEMMs run on
 * CUDA cores through cuBLAS).
 */
int fcb200_split_tf32(const float* w, float* w_hi, float* w_lo, int64_t count, void* stream);

/*
 * The same contraction with half-precision split operands (three kind::f16 tcgen05 MMAs per product,
 * twice the TF32 issue rate, float32 accumulation): every value v is carried as hi + lo * 2^-11 with
 * hi = half(v * scale), lo = half((v * scale - hi) * 2^11), 22 significant bits as long as v * scale lies in
 * the normal half range (6.1e-5 .. 65504); smaller values keep an absolute accuracy of 3e-11 / scale.
 *   w_hi, w_lo  [N, K] half, row stride ldw (halves, multiple of 8): fcb200_split_f16 of the float32 weight
 *   w_scale     the power of two the weight was multiplied by before the split
 *   a_scale     DEVICE pointer to the power of two A is multiplied by before its split, or NULL for 1;
 *               choose it so that max|A| * a_scale stays well below 65504
 *   status      set to 1 if a bounded wait expired, to 2 if a scaled A value left the half range
 * K a multiple of 8, N a multiple of 4.  Same role in the reference as fcb200_gemm_tf32.
 */
int fcb200_gemm_f16x2(const float* a, int64_t lda, const void* w_hi, const void* w_lo, int64_t ldw, float w_scale,
                      const float* a_scale, const float* bias, float* c, int64_t ldc, int64_t m, int32_t n, int32_t k,
                      int32_t* status, void* stream);

/*
 * fcb200_gemm_f16x2 with A already split by the kernel that produced it: a_hi / a_lo [M, K] half, row stride
 * lda (halves, multiple of 8), both of (A * *a_scale).  The contraction then needs no conversion pass over A
 * in shared memory; `a_scale` is only used to undo the scale in the epilogue.  *status = 2 also when an
 * output is not finite (a producer's half overflowed).
 */
int fcb200_gemm_f16x2_presplit(const void* a_hi, const void* a_lo, int64_t lda, const void* w_hi, const void* w_lo,
                               int64_t ldw, float w_scale, const float* a_scale, const float* bias, float* c, int64_t ldc,
                               int64_t m, int32_t n, int32_t k, int32_t* status, void* stream);

/*
 * One launch for a whole SO(2) convolution (all m-blocks) with the gate activation, or its derivative, applied
 * in the epilogue: replaces SO2_Convolution.forward (uma/nn/so2_layers.py:600-647; block form :83-169) followed by
 * GateActivation.forward (uma/nn/activation.py:146-165), and their autograd twins, which the reference runs as
 * separate cuBLAS GEMMs, elementwise kernels and concatenations.  A CTA owns 128 edges and walks the listed
 * 128-column output tiles in order; the float32 convolution output between GEMM and gate never exists in memory
 * unless the caller asks to keep it for the backward pass.
 *   a_hi, a_lo   [M, a_cols] half planes (row stride lda halves), both of (A * *a_scale)
 *   w_hi, w_lo   HOST arrays of 3 device pointers: half-split weights [w_rows[i], w_cols[i]] contiguous (unused: NULL)
 *   w_scale      HOST array of 3 floats; bias: HOST array of 3 device pointers (or NULL entries / NULL array)
 *   tiles        HOST array, 9 int32 per tile: a_col, k, w, w_row, out_col, mode, y_col, gate_col, flags
 *                mode 0  float32 tile -> y[:, out_col..]
 *                mode 2  planes[:, out_col..] = split(v * sigmoid(v));                    flag 4: also y[:, y_col..] = v
 *                mode 3  planes[:, out_col..] = split(v * sigmoid(y[:, gate_col..]));     flag 4: also y[:, y_col..] = v
 *                mode 4  planes[:, out_col..] = split(v * silu'(y[:, y_col..]))
 *                mode 5  planes[:, out_col..] = split(v * sigmoid(y[:, gate_col..])) and the gate gradient
 *                        sum_rows v * y[:, y_col..] summed over CONSECUTIVE tiles (flag 1: first row of the
 *                        degree, flag 2: last row -> planes[:, gate_col..] = split(sum * s * (1 - s)))
 *   rot_begin    tiles [rot_begin, num_tiles) may run in any order (each CTA starts at a different one, so that the
 *                CTAs do not all ask L2 for the same weight lines at once); mode-0 tiles that write gate scalars
 *                read by mode-3 tiles come before rot_begin; num_tiles for a mode-5 plan (its order matters)
 *   y            [M, y_cols] float32, row stride ldy; o_hi/o_lo [M, o_cols] half planes, row stride ldo, written
 *                times *o_scale (device pointers to powers of two, NULL = 1)
 *   status       as in fcb200_gemm_f16x2_presplit
 *   variant      0: one CTA per 128-edge tile, operand ring of 32-deep k stages; 1: CTA pairs (tcgen05
 *                cta_group::2) on 256-edge tiles, each CTA streaming half of the weight operand; 2: as 0 with
 *                64-deep k stages (128-byte swizzle; runs as 0 when some k is not a multiple of 64).  Same results.
 * At most 40 tiles; every k a multiple of 32, w_row a multiple of 128.
 */
/* Number of CTA pairs variant 1 of fcb200_so2_conv_fused runs at once on the current device (0 if it cannot be told). */
int fcb200_conv_pair_capacity(void);

int fcb200_so2_conv_fused(const void* a_hi, const void* a_lo, int64_t lda, int64_t a_cols, const void* const* w_hi,
                          const void* const* w_lo, const int64_t* w_rows, const int64_t* w_cols, const float* w_scale,
                          const float* const* bias, const int32_t* tiles, int32_t num_tiles, int32_t rot_begin, float* y,
                          int64_t ldy,
                          int64_t y_cols, void* o_hi, void* o_lo, int64_t ldo, int64_t o_cols, const float* a_scale,
                          const float* o_scale, int64_t m, int32_t variant, int32_t* status, void* stream);

/*
 * The four kernels whose output is consumed only by an SO(2) contraction, writing that output as the
 * half-precision split (two planes `*_hi`, `*_lo` of the float32 tensor's shape, values times *scale; scale
 * is a DEVICE pointer to a power of two, or NULL for 1) instead of float32: same bytes written, and the
 * contraction reads them with fcb200_gemm_f16x2_presplit.  Arguments otherwise as in the float32 versions
 * (fcb200_gather_rotate_fwd, fcb200_rotate_back_bwd, fcb200_so2_gate_fwd, fcb200_so2_gate_bwd and their
 * fcb200_lx_* counterparts).
 */
int fcb200_gather_rotate_fwd_h(const float* x, const int32_t* src, const int32_t* tgt, const float* wig, const float* radial,
                               void* out_hi, void* out_lo, const float* scale, int64_t num_edges, int64_t num_nodes,
                               int32_t channels, void* stream);
int fcb200_rotate_back_bwd_h(const float* grad_out, const float* msg, const float* winv, const int32_t* tgt, void* grad_msg_hi,
                             void* grad_msg_lo, const float* scale, float* grad_winv, int64_t num_edges, int64_t num_nodes,
                             int32_t channels, void* stream);
int fcb200_so2_gate_fwd_h(const float* y, void* out_hi, void* out_lo, const float* scale, int64_t num_edges, int32_t hidden,
                          void* stream);
int fcb200_so2_gate_bwd_h(const float* grad_out, const float* y, void* grad_y_hi, void* grad_y_lo, const float* scale,
                          int64_t num_edges, int32_t hidden, void* stream);
int fcb200_lx_gather_rotate_fwd_h(const float* x, const int32_t* src, const int32_t* tgt, const float* wig,
                                  const float* radial, void* out_hi, void* out_lo, const float* scale, int64_t num_edges,
                                  int64_t num_nodes, int32_t channels, int32_t lmax, void* stream);
int fcb200_lx_rotate_back_bwd_h(const float* grad_out, const float* msg, const float* winv, const int32_t* tgt,
                                void* grad_msg_hi, void* grad_msg_lo, const float* scale, float* grad_winv, int64_t num_edges,
                                int64_t num_nodes, int32_t channels, int32_t lmax, void* stream);
int fcb200_lx_so2_gate_fwd_h(const float* y, void* out_hi, void* out_lo, const float* scale, int64_t num_edges, int32_t hidden,
                             int32_t lmax, void* stream);
int fcb200_lx_so2_gate_bwd_h(const float* grad_out, const float* y, void* grad_y_hi, void* grad_y_lo, const float* scale,
                             int64_t num_edges, int32_t hidden, int32_t lmax, void* stream);

/* w [rows, cols] float32 (row stride ldw) -> contiguous half hi / lo parts of w * scale (see fcb200_gemm_f16x2). */
int fcb200_split_f16(const float* w, int64_t ldw, void* w_hi, void* w_lo, float scale, int64_t rows, int64_t cols,
                     void* stream);

/* ---------------------------------------------------------------- any lmax with mmax = 2 (lmax = 2 or 4) */

/*
 * The `fcb200_lx_*` family is the same set of operations for the 10-layer lmax = 4, mmax = 2
 * configuration of the backbone (src/fairchem/core/models/uma/escn_md.py:76-160 with lmax=4, mmax=2;
 * coefficient selection as CoefficientMapping, src/fairchem/core/models/uma/common/so3.py:19-160); `lmax` is
 * 2 or 4 (FCB200_EINVAL otherwise).  With NL = (lmax+1)^2, NM = sum_l min(2l+1, 5) (9 / 19):
 *   - node features [N, NL, C] L-major; edge features [E, NM, w] M-major
 *     (m=0: l=0..lmax | m=+1: l=1.. | m=-1 | m=+2: l=2.. | m=-2);
 *   - compact Wigner [E, NW], NW = FCB200_WIG (35) / FCB200_WIG_L4 (115): block l stores the rows
 *     m = -min(l,2)..min(l,2) of D^l, each with its 2l+1 columns, row-major, blocks in order of l
 *     (for lmax = 2 this is the layout described at the top of this file);
 *   - the inverse rotation is passed in the SAME layout (entry (l,m,m') of D times the envelope), not
 *     transposed: D is orthogonal, so the kernels read D^-1[m',m] = D[m,m'];
 *   - radial weights [E, 3*lmax * 2C]: slots of width 2C, (lmax+1) for m=0 (l=0..), lmax for |m|=1
 *     (l=1.., shared by +1 and -1), lmax-1 for |m|=2;
 *   - gate input y [E, (lmax + NM) H] = [lmax gate scalars (degree 1..lmax) | NM rows].
 * Argument meaning otherwise follows the entry point of the same name without `lx_`.
 */
#define FCB200_WIG_L4 115

int fcb200_lx_gather_rotate_fwd(const float* x, const int32_t* src, const int32_t* tgt, const float* wig,
                                const float* radial, float* out, int64_t num_edges, int64_t num_nodes,
                                int32_t channels, int32_t lmax, void* stream);

int fcb200_lx_gather_rotate_bwd(const float* grad_out, const float* x, const int32_t* src, const int32_t* tgt,
                                const float* wig, const float* radial, float* g_src, float* g_tgt, float* grad_wig,
                                float* grad_radial, int64_t num_edges, int64_t num_nodes, int32_t channels,
                                int32_t lmax, void* stream);

int fcb200_lx_rotate_back_reduce_fwd(const float* msg, const float* winv, const int32_t* row_ptr, float* out,
                                     int64_t num_edges, int64_t num_nodes, int32_t channels, int32_t lmax,
                                     void* stream);

/* radial0 [E, lmax+1, C]: the m = 0 rows of the edge-degree embedding (nn/embedding.py:77-94) */
int fcb200_lx_edge_degree_fwd(const float* radial0, const float* winv, const int32_t* row_ptr, const float* x_in,
                              float* out, float rescale, int64_t num_edges, int64_t num_nodes, int32_t channels,
                              int32_t lmax, void* stream);

int fcb200_lx_rotate_back_bwd(const float* grad_out, const float* msg, const float* winv, const int32_t* tgt,
                              float* grad_msg, float* grad_winv, int64_t num_edges, int64_t num_nodes,
                              int32_t channels, int32_t lmax, void* stream);

int fcb200_lx_edge_degree_bwd(const float* grad_out, const float* radial0, const float* winv, const int32_t* tgt,
                              float* grad_radial0, float* grad_winv, float rescale, int64_t num_edges,
                              int64_t num_nodes, int32_t channels, int32_t lmax, void* stream);

int fcb200_lx_so2_gate_fwd(const float* y, float* out, int64_t num_edges, int32_t hidden, int32_t lmax, void* stream);

int fcb200_lx_so2_gate_bwd(const float* grad_out, const float* y, float* grad_y, int64_t num_edges, int32_t hidden,
                           int32_t lmax, void* stream);

int fcb200_lx_rms_norm_sh_fwd(const float* x, const float* weight, const float* bias, const float* extra, float* out,
                              float* stats, float eps, int64_t num_nodes, int32_t channels, int32_t lmax, void* stream);

int fcb200_lx_rms_norm_sh_bwd(const float* grad_out, const float* x, const float* weight, const float* stats,
                              float* grad_x, int64_t num_nodes, int32_t channels, int32_t lmax, void* stream);

/*
 * Gate of the node-wise feed-forward (SpectralAtomwise, src/fairchem/core/models/uma/escn_md_block.py:288-328 with
 * GateActivation, src/fairchem/core/models/uma/nn/activation.py:146-165), fused: y [N, NL, H] L-major, gate_pre
 * [N, lmax*H] the scalar Linear's output; out row 0 = SiLU(y_0), rows of degree l = y * sigmoid(SiLU(gate_pre[l-1])).
 * The backward writes grad_y [N, NL, H] and grad_gate_pre [N, lmax*H].
 */
int fcb200_node_gate_fwd(const float* y, const float* gate_pre, float* out, int64_t num_nodes, int32_t hidden, int32_t lmax,
                         void* stream);
int fcb200_node_gate_bwd(const float* grad_out, const float* y, const float* gate_pre, float* grad_y, float* grad_gate_pre,
                         int64_t num_nodes, int32_t hidden, int32_t lmax, void* stream);

/*
 * Edge geometry with the compact Wigner-D of the given lmax [E, NW].  Degrees 3 and 4 follow from the
 * degree-1 and degree-(l-1) blocks by the recursion of Ivanic and Ruedenberg; the reference evaluates the
 * same matrices as polynomials of the quaternion (src/fairchem/core/models/uma/common/wigner_d_custom_kernels.py:196-356).
 */
int fcb200_lx_edge_geometry_fwd(const float* pos, const int32_t* src, const int32_t* tgt, const float* shift,
                                const float* gamma, float* vec, float* dist, float* env, float* wig, float* gauss,
                                float cutoff, int32_t num_basis, float basis_start, float basis_stop,
                                float basis_width, int64_t num_edges, int64_t num_nodes, int32_t lmax, void* stream);

int fcb200_lx_edge_geometry_bwd(const float* pos, const int32_t* src, const int32_t* tgt, const float* shift,
                                const float* gamma, const float* grad_wig, const float* grad_env,
                                const float* grad_gauss, const float* grad_dist, float* grad_vec, float cutoff,
                                int32_t num_basis, float basis_start, float basis_stop, float basis_width,
                                int64_t num_edges, int64_t num_nodes, int32_t lmax, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FAIRCHEM_B200_H */
