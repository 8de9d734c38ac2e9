"""Routed-expert (MOLE) checkpoints merged into single-expert weights, against the reference's own merge
(src/fairchem/core/models/uma/escn_moe.py:92-168) on a small seeded model; fixture made by tests/golden/make_golden.py."""

import pytest
import torch

from fairchem_b200 import mole


def _case(golden, tag):
    g = golden("mole_merge.npz")
    sd_in = {k.split("/", 2)[2]: torch.from_numpy(g[k]) for k in g.files if k.startswith(f"{tag}/in/")}
    sd_out = {k.split("/", 2)[2]: torch.from_numpy(g[k]) for k in g.files if k.startswith(f"{tag}/out/")}
    data = {"atomic_numbers": torch.from_numpy(g["atomic_numbers"]), "batch": torch.from_numpy(g["batch"]),
            "charge": torch.from_numpy(g["charge"]), "spin": torch.from_numpy(g["spin"]), "dataset": [str(d) for d in g["dataset"]]}
    return sd_in, sd_out, data, torch.from_numpy(g[f"{tag}/coeff"])


@pytest.mark.parametrize("tag", ["comp", "nocomp"])
def test_merge_matches_the_reference(golden, tag):
    sd_in, sd_out, data, coeff = _case(golden, tag)
    assert mole.is_mole_state_dict(sd_in) and not mole.is_mole_state_dict(sd_out)
    got_c = mole.expert_coefficients(sd_in, data["atomic_numbers"], data["batch"], data["charge"], data["spin"], data["dataset"])
    torch.testing.assert_close(got_c, coeff, rtol=1e-6, atol=1e-7)
    assert float(coeff.max() - coeff.min()) > 0.05  # the experts really are mixed unevenly in this fixture
    merged = mole.merge_mole_state_dict(sd_in, data)
    assert set(merged) == set(sd_out)
    for k, want in sd_out.items():
        torch.testing.assert_close(merged[k], want, rtol=1e-6, atol=1e-7, msg=k)
    # a merged state_dict passes through untouched
    again = mole.merge_mole_state_dict(merged, data)
    assert all(again[k] is merged[k] for k in merged)


def test_merge_rejects_batches_and_expert_mismatch(golden):
    sd_in, _, data, _ = _case(golden, "comp")
    two = dict(data, charge=torch.tensor([0, 0]), spin=torch.tensor([1, 1]), dataset=["omol", "omol"])
    with pytest.raises(ValueError):
        mole.merge_mole_state_dict(sd_in, two)
    bad = dict(sd_in)
    k = next(k for k in bad if k.endswith("fc_m0.weights"))
    bad[k] = bad[k][:2]
    with pytest.raises(ValueError):
        mole.merge_mole_state_dict(bad, data)
