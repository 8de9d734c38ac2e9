"""Host-side tables and policies that need no GPU: coefficient layouts against the oracle's tables, the compact
Wigner index maps, the keep-level policy, the power-of-two gradient scale, batching of inputs."""

import math

import numpy as np
import pytest
import torch

from fairchem_b200 import ops, synthetic, weights
from fairchem_b200 import backbone as B
from oracle import escn_md_oracle as O


@pytest.mark.parametrize("lmax", [2, 4])
def test_shape_tables_match_the_reference_coefficient_mapping(lmax):
    """SHShape restates CoefficientMapping (common/so3.py:19-160) for mmax = 2; the oracle's tables come from it."""
    sh = ops.SHAPES[lmax]
    l_of, m_of, m_order, m_size = O.lm_tables(lmax, 2)
    kept = O.kept_full_indices(lmax, 2)
    assert sh.m_size == list(m_size) and sh.nm == len(m_order) and sh.nl == (lmax + 1) ** 2
    assert sh.m2l == [kept[i] for i in m_order]
    assert sh.l_of == [l for l in range(lmax + 1) for _ in range(2 * l + 1)]
    assert sh.nw == {2: 35, 4: 115}[lmax] and sh.nrad == sum(sh.m_size)
    # every M-major row is a coefficient (l, m) with |m| <= 2, each exactly once
    assert sorted(sh.m2l) == sorted(l * l + l + m for l in range(lmax + 1) for m in range(-min(l, 2), min(l, 2) + 1))


@pytest.mark.parametrize("lmax", [2, 4])
def test_compact_wigner_index_maps(lmax):
    sh = ops.SHAPES[lmax]
    g = torch.Generator().manual_seed(lmax)
    d = O.wigner_blocks(O.edge_quaternion(torch.randn(6, 3, generator=g, dtype=torch.float64)), lmax)
    flat = d.reshape(6, -1)
    direct = flat[:, torch.tensor(B.dense_to_compact_index(lmax))]
    from_inverse = d.transpose(1, 2).reshape(6, -1)[:, torch.tensor(B.dense_to_compact_index(lmax, transposed=True))]
    assert torch.equal(direct, from_inverse)                     # compact(D) read out of the dense inverse D^T
    # block l holds rows m = -min(l,2)..min(l,2) with all 2l+1 columns, row-major
    for l in range(lmax + 1):
        mm = min(l, 2)
        blk = direct[:, sh.woff[l]:sh.woff[l + 1]].view(6, 2 * mm + 1, 2 * l + 1)
        assert torch.equal(blk, d[:, l * l + l - mm:l * l + l + mm + 1, l * l:(l + 1) ** 2])
    if lmax == 2:  # the tuned kernels read the inverse as the compact form of D^T
        t = torch.tensor(B._transpose_index())
        assert torch.equal(direct[:, t], d.transpose(1, 2).reshape(6, -1)[:, torch.tensor(B.dense_to_compact_index(2))])
        assert ops.uses_transposed_inverse(2) and not ops.uses_transposed_inverse(4)


def test_keep_level_policy(monkeypatch):
    bb = B.eSCNMDBackboneB200(**weights.UMA_S)
    dev = torch.device("cuda", 0)
    total = 183 * 2 ** 30
    edges = 3_100_000
    rows = -(-edges // 65536) * 65536
    need_1 = rows * (11 * 128 + 2 * 128 + 4) * 4        # conv-1 output + radial pre-activations and statistics
    need_2 = need_1 + rows * 9 * 128 * 4                # + messages
    need_3 = need_2 + rows * 6 * 256 * 4                # + radial weights

    def with_free(free, num_edges=edges):
        monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (free, total))
        monkeypatch.setattr(torch.cuda, "memory_reserved", lambda device=None: 0)
        monkeypatch.setattr(torch.cuda, "memory_allocated", lambda device=None: 0)
        return bb._keep_level_for_next_layer(num_edges, dev)

    # reserve for the per-chunk temporaries of both passes: 6 % of the device + 6 operand buffers of one chunk
    reserve = 0.06 * total + 6 * int(1.25 * bb.edge_chunk_size) * 9 * 2 * 128 * 4
    assert with_free(175 * 2 ** 30) == 2                     # the 100k-atom box: level 3 would not fit in all four layers
    assert with_free(int(4 * need_3 + 1.5 * reserve) + 2 ** 20) == 3
    assert with_free(175 * 2 ** 30, num_edges=edges // 4) == 3   # a quarter of the edges (4 ranks): everything is kept
    assert with_free(int(need_2 + reserve) + 2 ** 20) == 2
    assert with_free(int(need_2 + reserve) - 2 ** 20) == 1   # the reserve no longer fits beside level 2
    assert with_free(int(need_1 + reserve) - 2 ** 20) == 0
    assert with_free(0) == 0
    # memory the caching allocator holds but does not use counts as free
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (0, total))
    monkeypatch.setattr(torch.cuda, "memory_reserved", lambda device=None: 175 * 2 ** 30)
    monkeypatch.setattr(torch.cuda, "memory_allocated", lambda device=None: 2 ** 30)
    assert bb._keep_level_for_next_layer(edges, dev) == 2
    assert bb._keep_level_for_next_layer(edges, torch.device("cpu")) == 0
    bb.keep_level = 1
    assert bb._keep_level_for_next_layer(edges, dev) == 1  # an explicit level wins


def test_gradient_scale_is_a_power_of_two_that_centres_the_half_range():
    for mag in (3e-9, 1e-4, 0.7, 1.0, 5.0, 3e4, 0.0):
        s = float(B._pow2_scale(torch.tensor(mag)))
        assert math.log2(s) == round(math.log2(s))
        if mag > 0:
            assert 32.0 < mag * s <= 64.0
    t = torch.tensor([[0.5, -3.0], [2.0, 1.0]])
    assert float(B._absmax(t)) == 3.0 and float(B._absmax(-t)) == 3.0


def test_merge_builds_a_batch():
    a, b = synthetic.fcc_cu((2, 2, 2), seed=0), synthetic.molecule_batch(3, seed=1)
    m = synthetic.merge([a, b])
    assert m.pos.shape[0] == a.pos.shape[0] + b.pos.shape[0] and len(m.natoms) == 4 and len(m.dataset) == 4
    assert torch.equal(m.batch[: a.pos.shape[0]], a.batch) and int(m.batch.max()) == 3
    assert torch.equal(torch.bincount(m.batch), m.natoms)
    assert np.array_equal(m.cell[0].numpy(), a.cell[0].numpy()) and m.dataset[0] == "omat" and m.dataset[-1] == "omol"
