"""TEST INFRASTRUCTURE ONLY -- CPU restatement of fairchem's eSCN-MD (UMA) energy+force path.

A functional, dense-matrix restatement (torch on CPU, autograd for the forces) of what the
reference computes with ``execution_mode="general"``.  It takes the reference's own
``state_dict`` (same keys), so identical random-init weights can be fed to the reference,
to this oracle and to the CUDA path.  It is the checker for the GPU parity tests and the
timed CPU baseline of ``bench.py``; the product package never imports it.

Parity pin: ``tests/test_oracle_vs_golden.py`` checks this file against vectors generated
by running the unmodified reference (``tests/golden/make_golden.py``).

Reference files restated here (paths inside facebookresearch/fairchem):
  backbone forward ........ src/fairchem/core/models/uma/escn_md.py:761-905
  layer / edge block ...... src/fairchem/core/models/uma/escn_md_block.py:204-250, 427-465
  general rotate/scatter .. src/fairchem/core/models/uma/nn/execution_backends.py:121-263
  SO(2) convolution ....... src/fairchem/core/models/uma/nn/so2_layers.py:67-80, 600-647
  gate activation ......... src/fairchem/core/models/uma/nn/activation.py:146-165
  radial MLP / envelope ... src/fairchem/core/models/uma/nn/radial.py:22-86
  edge-degree embedding ... src/fairchem/core/models/uma/nn/embedding.py:77-94
  RMS norm (SH) ........... src/fairchem/core/models/uma/nn/layer_norm.py:372-419
  SO3 linear .............. src/fairchem/core/models/uma/nn/so3_layers.py:40-52
  edge -> quaternion ...... src/fairchem/core/models/uma/common/quaternion/quaternion_utils.py:28-239
  Wigner-D blocks ......... src/fairchem/core/models/uma/common/quaternion/wigner_d_hybrid.py:55-205
  energy / forces ......... src/fairchem/core/models/uma/outputs.py:41-162
  PBC edge vectors ........ src/fairchem/core/graph/compute.py:75-113
"""

from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

# ----------------------------------------------------------------------------------------
# coefficient bookkeeping (so3.py:16-118)
# ----------------------------------------------------------------------------------------


def lm_tables(lmax: int, mmax: int):
    """(l, m) of each kept coefficient in L-major order, and the M-major permutation.

    Returns ``l_of, m_of`` (lists over the kept coefficients, L-major: l ascending, m from
    -min(l,mmax)..+min(l,mmax)), ``m_order`` (for each M-major position the index into the
    kept L-major list) and ``m_size`` (count of l's per |m|).
    """
    l_of, m_of = [], []
    for l in range(lmax + 1):
        mm = min(mmax, l)
        for m in range(-mm, mm + 1):
            l_of.append(l)
            m_of.append(m)
    m_order, m_size = [], []
    for m in range(mmax + 1):
        plus = [i for i in range(len(l_of)) if m_of[i] == m]
        m_order += plus
        m_size.append(len(plus))
        if m != 0:
            m_order += [i for i in range(len(l_of)) if m_of[i] == -m]
    return l_of, m_of, m_order, m_size


def kept_full_indices(lmax: int, mmax: int):
    """Index of each kept coefficient inside the full (lmax+1)^2 L-major list."""
    out = []
    for l in range(lmax + 1):
        mm = min(mmax, l)
        for m in range(-mm, mm + 1):
            out.append(l * l + l + m)
    return out


# ----------------------------------------------------------------------------------------
# edge vector -> quaternion -> Wigner-D
# ----------------------------------------------------------------------------------------

_BLEND_START, _BLEND_WIDTH = -0.9, 1.8


def _smooth_step(t):
    tc = t.clamp(0, 1)
    eps = torch.finfo(t.dtype).eps
    arg = (2.0 * tc - 1.0) / (tc * (1.0 - tc)).clamp(min=eps)
    s = torch.sigmoid(arg)
    s = torch.where(tc < eps, torch.zeros_like(s), s)
    return torch.where(tc > 1 - eps, torch.ones_like(s), s)


def edge_quaternion(edge_vec: torch.Tensor, gamma: torch.Tensor | None = None) -> torch.Tensor:
    """Unit quaternion (w,x,y,z) rotating the edge direction onto +Y, then rolled by gamma about Y."""
    e = F.normalize(edge_vec, dim=-1)
    ex, ey, ez = e[:, 0], e[:, 1], e[:, 2]
    zero = torch.zeros_like(ex)
    eps = torch.finfo(e.dtype).eps
    q1 = torch.stack([1.0 + ey, -ez, zero, ex], dim=-1)
    q1 = q1 / torch.sqrt(torch.clamp((q1 * q1).sum(-1, keepdim=True), min=eps))
    q2 = torch.stack([-ez, 1.0 - ey, ex, zero], dim=-1)
    q2 = q2 / torch.sqrt(torch.clamp((q2 * q2).sum(-1, keepdim=True), min=eps))
    s = _smooth_step((ey - _BLEND_START) / _BLEND_WIDTH).unsqueeze(-1)
    dot = (q2 * q1).sum(-1, keepdim=True)
    q2a = torch.where(dot < 0, -q2, q2)
    q = F.normalize((1.0 - s) * q2a + s * q1, dim=-1)
    if gamma is not None:
        h = gamma / 2
        gw, gy = torch.cos(h), torch.sin(h)
        w2, x2, y2, z2 = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
        # Hamilton product (gw, 0, gy, 0) * q
        q = torch.stack([gw * w2 - gy * y2, gw * x2 + gy * z2, gw * y2 + gy * w2, gw * z2 - gy * x2], dim=-1)
    return q


def rotation_from_quaternion(q: torch.Tensor) -> torch.Tensor:
    w, x, y, z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    return torch.stack([
        torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)], dim=-1),
        torch.stack([2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)], dim=-1),
        torch.stack([2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], dim=-1),
    ], dim=-2)


def _l2_quadratic_forms() -> np.ndarray:
    """Symmetric 3x3 matrices A_i with Y_i(r) = r^T A_i r for the real l=2 harmonics in the
    (x,y,z) frame with y as polar axis, ordered m=-2..2:
    sqrt3*x*z, sqrt3*x*y, y^2-(x^2+z^2)/2, sqrt3*y*z, sqrt3/2*(z^2-x^2).  tr(A_i A_j) = 1.5*delta_ij."""
    s3 = math.sqrt(3.0)
    a = np.zeros((5, 3, 3))
    a[0, 0, 2] = a[0, 2, 0] = s3 / 2
    a[1, 0, 1] = a[1, 1, 0] = s3 / 2
    a[2] = np.diag([-0.5, 1.0, -0.5])
    a[3, 1, 2] = a[3, 2, 1] = s3 / 2
    a[4] = np.diag([-s3 / 2, 0.0, s3 / 2])
    return a


_A2 = _l2_quadratic_forms()


def _next_degree(r1: torch.Tensor, prev: torch.Tensor, l: int) -> torch.Tensor:
    """Real rotation matrix of degree l from degree l-1 and degree 1 (rows/columns m = -l..l): the
    recursion of Ivanic and Ruedenberg, J. Phys. Chem. 100 (1996) 6342 (with the 1998 erratum)."""
    n = r1.shape[0]
    out = torch.zeros(n, 2 * l + 1, 2 * l + 1, dtype=r1.dtype)

    def one(i, j):
        return r1[:, i + 1, j + 1]

    def low(a, b):
        return prev[:, a + l - 1, b + l - 1]

    def p(i, a, b):
        if abs(b) < l:
            return one(i, 0) * low(a, b)
        if b == l:
            return one(i, 1) * low(a, l - 1) - one(i, -1) * low(a, -l + 1)
        return one(i, 1) * low(a, -l + 1) + one(i, -1) * low(a, l - 1)

    for m in range(-l, l + 1):
        for mp in range(-l, l + 1):
            den = (l + mp) * (l - mp) if abs(mp) < l else (2 * l) * (2 * l - 1)
            d0 = 1.0 if m == 0 else 0.0
            u = math.sqrt((l + m) * (l - m) / den)
            v = 0.5 * math.sqrt((1 + d0) * (l + abs(m) - 1) * (l + abs(m)) / den) * (1 - 2 * d0)
            w = -0.5 * math.sqrt((l - abs(m) - 1) * (l - abs(m)) / den) * (1 - d0)
            val = 0
            if u != 0:
                val = val + u * p(0, m, mp)
            if v != 0:
                if m == 0:
                    vv = p(1, 1, mp) + p(-1, -1, mp)
                elif m > 0:
                    d1 = 1.0 if m == 1 else 0.0
                    vv = p(1, m - 1, mp) * math.sqrt(1 + d1) - p(-1, -m + 1, mp) * (1 - d1)
                else:
                    d1 = 1.0 if m == -1 else 0.0
                    vv = p(1, m + 1, mp) * (1 - d1) + p(-1, -m - 1, mp) * math.sqrt(1 + d1)
                val = val + v * vv
            if w != 0:
                ww = p(1, m + 1, mp) + p(-1, -m - 1, mp) if m > 0 else p(1, m - 1, mp) - p(-1, -m + 1, mp)
                val = val + w * ww
            out[:, m + l, mp + l] = val
    return out


def wigner_blocks(q: torch.Tensor, lmax: int) -> torch.Tensor:
    """Block-diagonal real Wigner-D [E,(lmax+1)^2,(lmax+1)^2] of the rotation q.

    l=1 is the Cartesian rotation matrix R (x,y,z order = m -1,0,1 in the y-polar convention); l=2
    follows from it through the quadratic forms of the l=2 harmonics, D2[i,j] = (2/3) tr(A_i R A_j R^T);
    l>=3 by the Ivanic-Ruedenberg recursion from the l-1 and l=1 blocks.  The reference evaluates the
    same matrices as polynomials in q from coefficient tables (wigner_d_custom_kernels.py:196-356);
    the two routes agree to rounding (checked on l = 2, 3, 4 against the reference's output).
    """
    n = q.shape[0]
    size = (lmax + 1) ** 2
    blocks = [torch.ones(n, 1, 1, dtype=q.dtype)]
    if lmax >= 1:
        r = rotation_from_quaternion(q)
        blocks.append(r)
    if lmax >= 2:
        a = torch.tensor(_A2, dtype=q.dtype)
        blocks.append((2.0 / 3.0) * torch.einsum("iab,nbc,jcd,nad->nij", a, r, a, r))
    for l in range(3, lmax + 1):
        blocks.append(_next_degree(r, blocks[-1], l))
    d = torch.zeros(n, size, size, dtype=q.dtype)
    for l, b in enumerate(blocks):
        d[:, l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] = b
    return d


# ----------------------------------------------------------------------------------------
# small layers
# ----------------------------------------------------------------------------------------


def radial_mlp(sd, prefix: str, x: torch.Tensor) -> torch.Tensor:
    """Linear-LayerNorm-SiLU-Linear-LayerNorm-SiLU-Linear (radial.py:61-86)."""
    h = F.linear(x, sd[prefix + "net.0.weight"], sd[prefix + "net.0.bias"])
    h = F.silu(F.layer_norm(h, h.shape[-1:], sd[prefix + "net.1.weight"], sd[prefix + "net.1.bias"], 1e-5))
    h = F.linear(h, sd[prefix + "net.3.weight"], sd[prefix + "net.3.bias"])
    h = F.silu(F.layer_norm(h, h.shape[-1:], sd[prefix + "net.4.weight"], sd[prefix + "net.4.bias"], 1e-5))
    return F.linear(h, sd[prefix + "net.6.weight"], sd[prefix + "net.6.bias"])


def envelope(d_scaled: torch.Tensor, p: float = 5.0) -> torch.Tensor:
    a, b, c = -(p + 1) * (p + 2) / 2, p * (p + 2), -p * (p + 1) / 2
    val = 1 + (d_scaled ** p) * (a + d_scaled * (b + c * d_scaled))
    return torch.where(d_scaled < 1, val, torch.zeros_like(val))


def gaussian_smearing(dist: torch.Tensor, start: float, stop: float, num: int, width: float) -> torch.Tensor:
    offset = torch.linspace(start, stop, num, dtype=torch.float32)
    coeff = -0.5 / (width * (offset[1] - offset[0])).item() ** 2
    diff = dist.view(-1, 1) - offset.to(dist.dtype).view(1, -1)
    return torch.exp(coeff * diff * diff)


def rms_norm_sh(x, weight, bias, lmax: int, eps: float = 1e-5):
    l_of = [l for l in range(lmax + 1) for _ in range(2 * l + 1)]
    x0 = x[:, :1] - x[:, :1].mean(dim=2, keepdim=True)
    feat = torch.cat([x0, x[:, 1:]], dim=1)
    bal = torch.tensor([1.0 / ((2 * l + 1) * (lmax + 1)) for l in l_of], dtype=x.dtype).view(1, -1, 1)
    nrm = (feat * feat * bal).sum(dim=1, keepdim=True).mean(dim=2, keepdim=True)
    scale = (nrm + eps).pow(-0.5) * weight[l_of].unsqueeze(0)
    out = feat * scale
    return torch.cat([out[:, :1] + bias.view(1, 1, -1), out[:, 1:]], dim=1)


def so3_linear(x, weight, bias, lmax: int):
    l_of = [l for l in range(lmax + 1) for _ in range(2 * l + 1)]
    out = torch.einsum("bmi,moi->bmo", x, weight[l_of])
    return torch.cat([out[:, :1] + bias.view(1, 1, -1), out[:, 1:]], dim=1)


def gate_activation(gating, x, expand_index, lmax: int):
    g = torch.sigmoid(gating).view(gating.shape[0], lmax, -1)[:, expand_index]
    return torch.cat([F.silu(x[:, :1]), x[:, 1:] * g], dim=1)


def so2_convolution(sd, prefix: str, x, rad, m_size, m_out: int, extra_m0: int):
    """SO(2) convolution on M-major input x [E,M,Cin] (so2_layers.py:600-647)."""
    e = x.shape[0]
    c_in = x.shape[2]
    mmax = len(m_size) - 1
    rad_off = 0
    x0 = x[:, : m_size[0]].reshape(e, -1)
    if rad is not None:
        x0 = x0 * rad[:, : x0.shape[1]]
        rad_off = x0.shape[1]
    y0 = F.linear(x0, sd[prefix + "fc_m0.weight"], sd[prefix + "fc_m0.bias"])
    extra = None
    if extra_m0:
        extra, y0 = y0[:, :extra_m0], y0[:, extra_m0:]
    out = [y0.reshape(e, -1, m_out)]
    off = m_size[0]
    for m in range(1, mmax + 1):
        k = m_size[m] * c_in
        xm = x[:, off: off + 2 * m_size[m]].reshape(e, 2, k)
        if rad is not None:
            xm = xm * rad[:, rad_off: rad_off + k].unsqueeze(1)
            rad_off += k
        w = sd[prefix + f"so2_m_conv.{m - 1}.fc.weight"]
        half = w.shape[0] // 2
        y = torch.matmul(xm, w.t())  # [E,2,2*half]
        real = y[:, 0, :half] - y[:, 1, half:]
        imag = y[:, 1, :half] + y[:, 0, half:]
        out += [real.reshape(e, -1, m_out), imag.reshape(e, -1, m_out)]
        off += 2 * m_size[m]
    return torch.cat(out, dim=1), extra


# ----------------------------------------------------------------------------------------
# full forward
# ----------------------------------------------------------------------------------------


def edge_vectors(pos, cell, edge_index, cell_offsets, edge_system):
    """vec = pos[src] - pos[tgt] + offsets @ cell (graph/compute.py:75-113)."""
    shift = torch.einsum("ej,ejk->ek", cell_offsets.to(pos.dtype), cell[edge_system])
    return pos[edge_index[0]] - pos[edge_index[1]] + shift


def energy_and_forces(sd, cfg: dict, data, edge_index, cell_offsets, gamma=None, want_forces=True,
                      return_intermediates=False, want_stress=False):
    """Energy [B] (float64) and forces [N,3] for one batch, given the edge list.

    ``sd``: backbone state_dict plus head entries under ``energy_block.*``; ``cfg``: dict with
    lmax, mmax, sphere_channels, hidden_channels, num_layers, cutoff, num_distance_basis.
    ``edge_index`` [2,E] (src;tgt), ``cell_offsets`` [E,3] integers.
    """
    lmax, mmax = cfg["lmax"], cfg["mmax"]
    c, h, nl = cfg["sphere_channels"], cfg["hidden_channels"], cfg["num_layers"]
    cutoff = float(cfg["cutoff"])
    dtype = sd["sphere_embedding.weight"].dtype
    l_of, m_of, m_order, m_size = lm_tables(lmax, mmax)
    kept = kept_full_indices(lmax, mmax)
    rows = [kept[i] for i in m_order]  # full L index of each M-major row
    n_full = (lmax + 1) ** 2

    pos = data["pos"].detach().to(dtype).clone().requires_grad_(want_forces)
    cell = data["cell"].detach().to(dtype).clone().requires_grad_(want_stress)
    z = data["atomic_numbers"].long()
    batch = data["batch"].long()
    n = pos.shape[0]
    nsys = len(data["natoms"])
    src, tgt = edge_index[0].long(), edge_index[1].long()
    inter = {}

    # system embedding (escn_md.py:590-601, 820-821)
    chg = sd["charge_embedding.rand_emb.weight"][data["charge"].long() + 100]
    spn = sd["spin_embedding.rand_emb.weight"][data["spin"].long()]
    dse = torch.stack([sd[f"dataset_embedding.dataset_emb_dict.{cfg['dataset_mapping'][t]}.weight"][0]
                       for t in data["dataset"]])
    csd = F.silu(F.linear(torch.cat([chg, spn, dse], dim=1), sd["mix_csd.weight"], sd["mix_csd.bias"]))
    sys_node = csd[batch]

    # geometry
    vec = edge_vectors(pos, cell, edge_index, cell_offsets, batch[tgt])
    dist = vec.norm(dim=-1)
    q = edge_quaternion(vec, gamma)
    d_full = wigner_blocks(q, lmax)  # [E,L2,L2]
    wigner = d_full[:, rows, :]  # M-major rows
    env = envelope(dist / cutoff).view(-1, 1, 1)
    wigner_inv_env = d_full.transpose(1, 2)[:, :, rows] * env  # [E,L2,M]
    inter.update(vec=vec, dist=dist, wigner=d_full, env=env.view(-1))

    # edge scalar features (escn_md.py:838-853)
    x_edge = torch.cat([
        gaussian_smearing(dist, 0.0, cutoff, cfg["num_distance_basis"], 2.0),
        sd["source_embedding.weight"][z[src]], sd["target_embedding.weight"][z[tgt]]], dim=1)

    # node init + edge-degree embedding (escn_md.py:811-863, embedding.py:77-94)
    x = torch.zeros(n, n_full, c, dtype=dtype)
    x = torch.cat([(sd["sphere_embedding.weight"][z] + sys_node).unsqueeze(1), x[:, 1:]], dim=1)
    rad0 = radial_mlp(sd, "edge_degree_embedding.rad_func.", x_edge).reshape(-1, m_size[0], c)
    x = x.index_add(0, tgt, torch.bmm(wigner_inv_env[:, :, : m_size[0]], rad0) / 5.0)
    inter["x_after_edge_degree"] = x

    # gate expand index in m-prime order (activation.py:122-137)
    expand = list(range(lmax))
    for m in range(1, mmax + 1):
        expand += list(range(m - 1, lmax)) * 2
    expand_l = [l - 1 for l in range(1, lmax + 1) for _ in range(2 * l + 1)]

    for i in range(nl):
        p = f"blocks.{i}."
        x_res = x
        xn = rms_norm_sh(x, sd[p + "norm_1.affine_weight"], sd[p + "norm_1.affine_bias"], lmax)
        xn = torch.cat([xn[:, :1] + sys_node.unsqueeze(1), xn[:, 1:]], dim=1)
        # edge block (escn_md_block.py:235-246)
        msg = torch.bmm(wigner, torch.cat([xn[src], xn[tgt]], dim=2))
        rad = radial_mlp(sd, p + "edge_wise.so2_conv_1.rad_func.", x_edge)
        msg, gating = so2_convolution(sd, p + "edge_wise.so2_conv_1.", msg, rad, m_size, h, lmax * h)
        msg = gate_activation(gating, msg, expand, lmax)
        msg, _ = so2_convolution(sd, p + "edge_wise.so2_conv_2.", msg, None, m_size, c, 0)
        agg = torch.zeros(n, n_full, c, dtype=dtype).index_add(0, tgt, torch.bmm(wigner_inv_env, msg))
        x = agg + x_res
        if return_intermediates:
            inter[f"edgewise_out_{i}"] = agg
        # node-wise feed-forward (escn_md_block.py:323-328)
        x_res = x
        xn = rms_norm_sh(x, sd[p + "norm_2.affine_weight"], sd[p + "norm_2.affine_bias"], lmax)
        gates = F.silu(F.linear(xn[:, 0], sd[p + "atom_wise.scalar_mlp.0.weight"], sd[p + "atom_wise.scalar_mlp.0.bias"]))
        y = so3_linear(xn, sd[p + "atom_wise.so3_linear_1.weight"], sd[p + "atom_wise.so3_linear_1.bias"], lmax)
        y = gate_activation(gates, y, expand_l, lmax)
        y = so3_linear(y, sd[p + "atom_wise.so3_linear_2.weight"], sd[p + "atom_wise.so3_linear_2.bias"], lmax)
        x = y + x_res

    x = rms_norm_sh(x, sd["norm.affine_weight"], sd["norm.affine_bias"], lmax)
    inter["node_embedding"] = x
    e_node = F.linear(F.silu(F.linear(F.silu(F.linear(
        x[:, 0], sd["energy_block.0.weight"], sd["energy_block.0.bias"])),
        sd["energy_block.2.weight"], sd["energy_block.2.bias"])),
        sd["energy_block.4.weight"], sd["energy_block.4.bias"]).view(-1)
    energy = torch.zeros(nsys, dtype=torch.float64).index_add(0, batch, e_node.double())
    forces = None
    if want_stress:
        # virial from the position and cell gradients, stress = virial / volume, flattened [B,9] (outputs.py:165-226)
        g_r, g_h = torch.autograd.grad(energy.sum(), [pos, cell])
        forces = -g_r
        pos_virial = torch.zeros(nsys, 3, 3, dtype=dtype).index_add(0, batch, g_r.unsqueeze(2) * pos.detach().unsqueeze(1))
        cell_virial = cell.detach().transpose(1, 2) @ g_h
        virial = (pos_virial + pos_virial.transpose(1, 2) + cell_virial + cell_virial.transpose(1, 2)) / 2
        stress = (virial / torch.det(cell.detach()).abs().view(-1, 1, 1)).reshape(-1, 9)
        return energy.detach(), forces, stress
    if want_forces:
        (grad,) = torch.autograd.grad(energy.sum(), pos)
        forces = -grad
    if return_intermediates:
        return energy.detach(), forces, {k: v.detach() for k, v in inter.items()}
    return energy.detach(), forces
