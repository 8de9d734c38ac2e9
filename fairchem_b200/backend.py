"""``B200Backend``: the reference's execution-backend op table on the sm_100a kernels.

Same static-method names, argument meaning and return shapes as fairchem's ``ExecutionBackend``
(src/fairchem/core/models/uma/nn/execution_backends.py:46-263) and the fused pair of
``UMASFastGPUBackend`` (:432-507), so ``Edgewise.forward_chunk`` / ``EdgeDegreeEmbedding.forward_chunk``
(src/fairchem/core/models/uma/escn_md_block.py:204-285, nn/embedding.py:77-94) can call it unchanged.
Like ``UMASFastGPUBackend`` it takes the raw block-diagonal Wigner matrices ``[E,9,9]`` (L-major) and does
the L<->M permutation inside the kernels; ``prepare_wigner`` is therefore a pass-through.

The kernels want edges grouped by target node.  ``generate_graph`` already returns them so; any other
order is handled by sorting once per edge list (cached) and un-permuting per-edge results.
"""

from __future__ import annotations

import torch

from . import ops
from .backbone import dense_to_compact_index
from .ops import EdgeGraph

_FLAT: dict = {}
_GRAPH_CACHE: dict = {}
_LMAX_OF_NL = {s.nl: l for l, s in ops.SHAPES.items()}


def _compact(wigner: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Dense [E,NL,NL] block-diagonal matrix -> compact [E,NW] (differentiable gather).  An inverse
    rotation goes to the layout the rotate-back kernels of its lmax expect."""
    nl = wigner.shape[1]
    lmax = _LMAX_OF_NL.get(nl)
    if lmax is None or wigner.shape[2] != nl:
        raise ValueError("B200Backend takes square block-diagonal Wigner matrices of lmax = 2 or 4")
    transposed = inverse and not ops.uses_transposed_inverse(lmax)
    key = (lmax, transposed, wigner.device)
    if key not in _FLAT:
        _FLAT[key] = torch.tensor(dense_to_compact_index(lmax, transposed), device=wigner.device)
    return wigner.reshape(wigner.shape[0], nl * nl).index_select(1, _FLAT[key])


def _graph_for(src: torch.Tensor, tgt: torch.Tensor, num_nodes: int, num_targets: int):
    """(EdgeGraph over target-sorted edges, permutation or None, inverse permutation or None), cached per edge list."""
    key = (src.data_ptr(), tgt.data_ptr(), int(src.shape[0]), num_nodes, num_targets, src._version, tgt._version)
    key_tensors = (src, tgt)
    hit = _GRAPH_CACHE.get(key)
    if hit is not None:
        return hit[:3]
    if len(_GRAPH_CACHE) > 8:
        _GRAPH_CACHE.clear()
    perm = inv = None
    if src.shape[0] > 1 and bool((tgt[1:] < tgt[:-1]).any()):
        perm = torch.sort(tgt, stable=True).indices
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.shape[0], device=perm.device)
        src, tgt = src[perm], tgt[perm]
    hit = (EdgeGraph(src, tgt, num_nodes, num_targets), perm, inv)
    # the entry keeps the caller's tensors alive: their addresses (the key) cannot be reused by other edge lists
    _GRAPH_CACHE[key] = hit + (key_tensors,)
    return hit


class B200Backend:
    """Parameterless op table; every method is static (the reference's backends carry no state)."""

    supports_fused_edgewise = True

    @staticmethod
    def validate(lmax: int, mmax: int, settings=None) -> None:
        if mmax != 2 or lmax not in ops.SHAPES:
            raise ValueError("B200Backend kernels are built for mmax = 2 with lmax = 2 or 4")
        if settings is not None and getattr(settings, "activation_checkpointing", False):
            raise ValueError("B200Backend chunks and recomputes inside its own edge block; "
                             "turn activation_checkpointing off")

    @staticmethod
    def prepare_model_for_inference(model: torch.nn.Module) -> None:
        for p in model.parameters():
            p.requires_grad_(False)

    @staticmethod
    def get_layer_radial_emb(x_edge: torch.Tensor, model: torch.nn.Module) -> list:
        # fused path: conv 1 consumes the radial weights, so they are computed per layer up front
        return [blk.edge_wise.so2_conv_1.rad_func(x_edge) for blk in model.blocks]

    @staticmethod
    def prepare_wigner(wigner, wigner_inv, mappingReduced=None, coefficient_index=None):
        # the kernels select the |m| <= 2 coefficients themselves: they take the square block-diagonal matrices
        return wigner, wigner_inv

    @staticmethod
    def node_to_edge_wigner_permute(x_full, edge_index, wigner):
        """[N,9,C], [2,E], [E,9,9] -> M-major edge messages [E,9,2C]."""
        graph, perm, inv = _graph_for(edge_index[0], edge_index[1], x_full.shape[0], x_full.shape[0])
        w = _compact(wigner)
        out = ops.GatherRotate.apply(x_full, w if perm is None else w[perm], None, graph)
        return out if inv is None else out[inv]

    @staticmethod
    def permute_wigner_inv_edge_to_node(x_message, wigner_inv, scatter_target, num_nodes):
        """[E,9,C] (M-major), [E,9,9], [E] -> [num_nodes,9,C]."""
        graph, perm, _ = _graph_for(scatter_target, scatter_target, num_nodes, num_nodes)
        w = _compact(wigner_inv, inverse=True)
        if perm is not None:
            x_message, w = x_message[perm], w[perm]
        return ops.RotateBackReduce.apply(x_message, w, graph)

    @staticmethod
    def edge_degree_scatter(x, radial_output, wigner_inv, scatter_target, m_0_num_coefficients, sphere_channels,
                            rescale_factor):
        graph, perm, _ = _graph_for(scatter_target, scatter_target, x.shape[0], x.shape[0])
        radial = radial_output.reshape(-1, m_0_num_coefficients, sphere_channels)
        w = _compact(wigner_inv, inverse=True)
        if perm is not None:
            radial, w = radial[perm], w[perm]
        return ops.EdgeDegree.apply(x, radial, w, graph, float(rescale_factor))

    @staticmethod
    def fused_node_to_edge_conv1_pack(x_full, edge_index, wigner, radial, sphere_channels):
        """Gather + rotate + radial scale; returns the three GEMM operands m0 [E,(lmax+1)*2C], m1 [E,2*lmax*2C],
        m2 [E,2*(lmax-1)*2C] as column ranges of one [E, NM*2C] buffer."""
        graph, perm, inv = _graph_for(edge_index[0], edge_index[1], x_full.shape[0], x_full.shape[0])
        w = _compact(wigner)
        if perm is not None:
            w, radial = w[perm], radial[perm]
        out = ops.GatherRotate.apply(x_full, w, radial, graph)
        if inv is not None:
            out = out[inv]
        flat = out.reshape(out.shape[0], -1)
        c2 = 2 * sphere_channels
        ms = ops.SHAPES[_LMAX_OF_NL[x_full.shape[1]]].m_size
        a, b = ms[0] * c2, (ms[0] + 2 * ms[1]) * c2
        return flat[:, :a], flat[:, a:b], flat[:, b:]

    @staticmethod
    def fused_conv2_inv_edge_to_node(g0, g1, g2, wigner_inv_envelope, scatter_target, num_nodes, sphere_channels):
        """Block-GEMM outputs g0 [E,(lmax+1)C], g1 [E,2*lmax*C], g2 [E,2*(lmax-1)C] -> rotate back and sum into
        [num_nodes,NL,C]."""
        msg = torch.cat([g0, g1, g2], dim=1).view(g0.shape[0], -1, sphere_channels)
        return B200Backend.permute_wigner_inv_edge_to_node(msg, wigner_inv_envelope, scatter_target, num_nodes)
