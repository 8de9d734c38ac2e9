"""Deterministic random-init weights with the eSCN-MD backbone's ``state_dict`` contract.

Keys and shapes follow fairchem's ``eSCNMDBackbone.state_dict()`` plus the energy head
(``src/fairchem/core/models/uma/escn_md.py:417-525, 1085-1091``) so the same dict loads into
the reference module (``strict=False``: the reference also carries ``Jd_*`` buffers), into the
CPU oracle and into :class:`fairchem_b200.backbone.eSCNMDBackboneB200`.  Values are drawn
from ``numpy.random.default_rng(seed)`` (platform-stable) with the distributions the
reference's constructors use: Linear weight/bias U(+-1/sqrt(fan_in)), embeddings N(0,1),
source/target embeddings U(+-1e-3) (``escn_md.py:468-469``), SO(2) m>0 weights scaled by
1/sqrt(2) (``so2_layers.py:65``), SO3 linear weights U(+-1/sqrt(fan_in)) with zero bias
(``so3_layers.py:29-32``), norm and LayerNorm affine = identity.
"""

from __future__ import annotations

import math

import numpy as np
import torch

UMA_S = dict(sphere_channels=128, lmax=2, mmax=2, num_layers=4, hidden_channels=128, edge_channels=128,
             num_distance_basis=64, cutoff=6.0, max_neighbors=30, max_num_elements=100,
             dataset_mapping={"omat": "omat", "omol": "omol"})

ESCN_MD_L4 = dict(UMA_S, lmax=4, mmax=2, num_layers=10)


def random_init_state_dict(cfg: dict | None = None, seed: int = 0, dtype=torch.float32) -> dict:
    cfg = dict(UMA_S if cfg is None else cfg)
    rng = np.random.default_rng(seed)
    c, h, ec = cfg["sphere_channels"], cfg["hidden_channels"], cfg["edge_channels"]
    lmax, mmax, nl = cfg["lmax"], cfg["mmax"], cfg["num_layers"]
    nel = cfg.get("max_num_elements", 100)
    sd: dict[str, torch.Tensor] = {}

    def put(name, arr):
        sd[name] = torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float64)).to(dtype)

    def uniform(shape, bound):
        return rng.uniform(-bound, bound, shape)

    def linear(prefix, fan_in, fan_out, bias=True, scale=1.0):
        b = 1.0 / math.sqrt(fan_in)
        put(prefix + "weight", uniform((fan_out, fan_in), b) * scale)
        if bias:
            put(prefix + "bias", uniform((fan_out,), b))

    def layer_norm(prefix, width):
        put(prefix + "weight", np.ones(width))
        put(prefix + "bias", np.zeros(width))

    def radial(prefix, widths):
        idx = 0
        for i in range(1, len(widths)):
            linear(f"{prefix}net.{idx}.", widths[i - 1], widths[i])
            idx += 1
            if i != len(widths) - 1:
                layer_norm(f"{prefix}net.{idx}.", widths[i])
                idx += 2

    def sh_norm(prefix):
        put(prefix + "affine_weight", np.ones((lmax + 1, c)))
        put(prefix + "affine_bias", np.zeros(c))

    put("sphere_embedding.weight", rng.normal(size=(nel, c)))
    put("charge_embedding.rand_emb.weight", rng.normal(size=(201, c)))
    put("spin_embedding.rand_emb.weight", rng.normal(size=(101, c)))
    for name in sorted(set(cfg["dataset_mapping"].values())):
        put(f"dataset_embedding.dataset_emb_dict.{name}.weight", rng.normal(size=(1, c)))
    linear("mix_csd.", 3 * c, c)
    put("source_embedding.weight", uniform((nel, ec), 1e-3))
    put("target_embedding.weight", uniform((nel, ec), 1e-3))
    edge_in = cfg["num_distance_basis"] + 2 * ec
    radial("edge_degree_embedding.rad_func.", [edge_in, ec, ec, (lmax + 1) * c])

    def m_count(m):
        return lmax - m + 1

    for i in range(nl):
        p = f"blocks.{i}."
        sh_norm(p + "norm_1.")
        sh_norm(p + "norm_2.")
        # conv1: 2C -> H with lmax*H extra gate scalars, radial-modulated (escn_md_block.py:96-105)
        cin, cout = 2 * c, h
        k0 = (lmax + 1) * cin
        linear(p + "edge_wise.so2_conv_1.fc_m0.", k0, (lmax + 1) * cout + lmax * h)
        n_rad = k0
        for m in range(1, mmax + 1):
            km = m_count(m) * cin
            linear(p + f"edge_wise.so2_conv_1.so2_m_conv.{m - 1}.fc.", km, 2 * m_count(m) * cout, bias=False,
                   scale=1.0 / math.sqrt(2.0))
            n_rad += km
        radial(p + "edge_wise.so2_conv_1.rad_func.", [edge_in, ec, ec, n_rad])
        # conv2: H -> C, internal weights
        cin, cout = h, c
        linear(p + "edge_wise.so2_conv_2.fc_m0.", (lmax + 1) * cin, (lmax + 1) * cout)
        for m in range(1, mmax + 1):
            linear(p + f"edge_wise.so2_conv_2.so2_m_conv.{m - 1}.fc.", m_count(m) * cin, 2 * m_count(m) * cout,
                   bias=False, scale=1.0 / math.sqrt(2.0))
        linear(p + "atom_wise.scalar_mlp.0.", c, lmax * h)
        put(p + "atom_wise.so3_linear_1.weight", uniform((lmax + 1, h, c), 1.0 / math.sqrt(c)))
        put(p + "atom_wise.so3_linear_1.bias", np.zeros(h))
        put(p + "atom_wise.so3_linear_2.weight", uniform((lmax + 1, c, h), 1.0 / math.sqrt(h)))
        put(p + "atom_wise.so3_linear_2.bias", np.zeros(c))
    sh_norm("norm.")
    linear("energy_block.0.", c, h)
    linear("energy_block.2.", h, h)
    linear("energy_block.4.", h, 1)
    return sd


def split_head(sd: dict) -> tuple[dict, dict]:
    """Split a combined dict into (backbone entries, head ``energy_block`` entries without prefix)."""
    bb = {k: v for k, v in sd.items() if not k.startswith("energy_block.")}
    head = {k[len("energy_block."):]: v for k, v in sd.items() if k.startswith("energy_block.")}
    return bb, head
