"""Mixture-of-linear-experts (MOLE) checkpoints -> the single-expert weights the B200 kernels take.

Released UMA checkpoints store every SO(2) linear layer of the edge block as ``num_experts`` weight matrices
(``...fc_m0.weights``, ``...so2_m_conv.j.fc.weights`` of shape [experts, out, in]) together with a routing MLP that
turns the system's charge/spin/dataset embedding -- and optionally its mean composition embedding -- into mixing
coefficients.  For inference on one system the reference contracts the experts with those coefficients once and
continues with an ordinary backbone (``eSCNMDMoeBackbone.merge_MOLE_model``,
src/fairchem/core/models/uma/escn_moe.py:92-123; coefficients ``set_MOLE_coefficients`` :125-168; the contraction is
``MOLE.merged_linear_layer``, src/fairchem/core/models/uma/nn/mole.py:150-168).  This module does the same on a
``state_dict``: it is weight preparation, done once per system composition on whatever device the tensors live on,
not part of the per-step path.
"""

from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch
import torch.nn.functional as F

ROUTING_PREFIX = "routing_mlp."
COMPOSITION_KEY = "composition_embedding.weight"


def is_mole_state_dict(state_dict: Mapping[str, torch.Tensor]) -> bool:
    return any(k.startswith(ROUTING_PREFIX) for k in state_dict)


def _normalise(x: torch.Tensor, kind: str) -> torch.Tensor:
    """Expert-coefficient normalisations of the reference (nn/mole.py:43-58)."""
    if kind == "softmax":
        return torch.softmax(x, dim=1) + 0.005
    if kind == "pnorm":
        return F.normalize(x.abs() + 2 / x.shape[0], p=1.0, dim=1)
    raise ValueError(f"unknown expert coefficient norm {kind!r}")


def csd_embedding(sd: Mapping[str, torch.Tensor], charge: torch.Tensor, spin: torch.Tensor, dataset: Sequence[str],
                  dataset_mapping: Optional[Mapping[str, str]] = None) -> torch.Tensor:
    """SiLU(mix_csd([charge_emb | spin_emb | dataset_emb])) per system (escn_md.py:590-601, rand_emb tables)."""
    chg = sd["charge_embedding.rand_emb.weight"][charge.long() + 100]
    spn = sd["spin_embedding.rand_emb.weight"][spin.long()]
    parts = [chg, spn]
    if any(k.startswith("dataset_embedding.") for k in sd):
        names = [dataset_mapping[d] if dataset_mapping else d for d in dataset]
        parts.append(torch.stack([sd[f"dataset_embedding.dataset_emb_dict.{n}.weight"][0] for n in names], dim=0))
    return F.silu(F.linear(torch.cat(parts, dim=1), sd["mix_csd.weight"], sd["mix_csd.bias"]))


def expert_coefficients(sd: Mapping[str, torch.Tensor], atomic_numbers: torch.Tensor, batch: torch.Tensor,
                        charge: torch.Tensor, spin: torch.Tensor, dataset: Sequence[str],
                        dataset_mapping: Optional[Mapping[str, str]] = None, norm: str = "softmax",
                        include_self_in_mean: bool = False) -> torch.Tensor:
    """[systems, experts] mixing coefficients: routing MLP (three Linear+SiLU) on [mean composition embedding | csd
    embedding] (escn_moe.py:125-168).  ``include_self_in_mean`` reproduces the one released generation whose mean
    over atoms also counts the zero the accumulator starts from."""
    csd = csd_embedding(sd, charge, spin, dataset, dataset_mapping)
    feats = []
    if COMPOSITION_KEY in sd:
        by_atom = sd[COMPOSITION_KEY][atomic_numbers.long()]
        comp = torch.zeros(csd.shape[0], by_atom.shape[1], dtype=by_atom.dtype, device=by_atom.device)
        comp.index_add_(0, batch.long(), by_atom)
        count = torch.bincount(batch.long(), minlength=csd.shape[0]).to(by_atom.dtype)
        comp = comp / (count + (1.0 if include_self_in_mean else 0.0)).clamp_min(1.0).unsqueeze(1)
        feats.append(comp)
    feats.append(csd)
    h = torch.cat(feats, dim=1)
    for i in (0, 2, 4):
        h = F.silu(F.linear(h, sd[f"{ROUTING_PREFIX}{i}.weight"], sd[f"{ROUTING_PREFIX}{i}.bias"]))
    return _normalise(h, norm)


def merge_mole_state_dict(sd: Mapping[str, torch.Tensor], data, dataset_mapping: Optional[Mapping[str, str]] = None,
                          norm: str = "softmax", include_self_in_mean: bool = False) -> dict:
    """Single-expert ``state_dict`` for the system in ``data`` (fields atomic_numbers, batch, charge, spin, dataset):
    every ``*.weights`` [experts, out, in] becomes ``*.weight`` = sum_e c_e W_e, routing and composition tables are
    dropped, everything else passes through.  Like the reference's merge this is valid for one system (one set of
    coefficients); a batch of several systems is rejected."""
    if not is_mole_state_dict(sd):
        return dict(sd)
    charge, spin = data["charge"], data["spin"]
    if int(charge.shape[0]) != 1:
        raise ValueError("MOLE weights can be merged for one system at a time (the coefficients are per system)")
    coeff = expert_coefficients(sd, data["atomic_numbers"], data["batch"], charge, spin, data["dataset"], dataset_mapping,
                                norm, include_self_in_mean)[0]
    out = {}
    for k, v in sd.items():
        if k.startswith(ROUTING_PREFIX) or k == COMPOSITION_KEY:
            continue
        if k.endswith(".weights") and v.dim() == 3:
            if v.shape[0] != coeff.shape[0]:
                raise ValueError(f"{k}: {v.shape[0]} experts, routing MLP yields {coeff.shape[0]} coefficients")
            out[k[:-1]] = torch.einsum("eoi,e->oi", v.float(), coeff.float().to(v.device)).to(v.dtype)
        else:
            out[k] = v
    return out
