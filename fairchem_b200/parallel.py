"""Spatial domain decomposition of one large system over the GPUs of a box, one process per GPU.

Mirrors fairchem's graph-parallel all-to-all mode (src/fairchem/core/common/parallelism/
graph_parallel_a2a.py:63-595, graph_partition.py:38-97, and the call sites in
src/fairchem/core/models/uma/escn_md.py:603-759 and escn_md_block.py:141-146):

* positions are replicated; atoms are assigned to ranks along a 30-bit Morton curve
  (``morton_partition``), so every rank owns a compact region of equal atom count;
* a rank builds the radius graph for its own target atoms only, renumbers nodes as
  ``[own atoms | halo atoms grouped by owner rank]`` and tells every owner which rows it needs
  (two small all-to-alls, once per step: ``build_plan``);
* every layer fetches the halo rows with one all-to-all into a local buffer
  (``HaloExchange.collect``; its backward sends the halo gradients home and adds them to the owners'
  rows); remote rows are always copied into this GPU's memory before any kernel reads them;
* energies are summed and per-rank force contributions (gradients w.r.t. the replicated positions)
  are all-reduced.

The collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs, Gloo in the CPU tests).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


def _expand_bits_10(v: torch.Tensor) -> torch.Tensor:
    v = (v | (v << 16)) & 0x030000FF
    v = (v | (v << 8)) & 0x0300F00F
    v = (v | (v << 4)) & 0x030C30C3
    v = (v | (v << 2)) & 0x09249249
    return v


def morton_partition(pos: torch.Tensor, num_ranks: int) -> torch.Tensor:
    """Rank of every atom: positions scaled by the largest box extent to 10 bits per axis, bits
    interleaved (x lowest), atoms sorted by code and cut into ``num_ranks`` runs of equal length
    (``i * P // N``), as ``partition_atoms_spatial`` does (graph_partition.py:38-97).  The sort is
    stable, so replicated positions give the same answer on every rank."""
    n = pos.shape[0]
    if num_ranks == 1:
        return torch.zeros(n, dtype=torch.long, device=pos.device)
    if num_ranks >= n:
        return torch.arange(n, dtype=torch.long, device=pos.device)
    lo = pos.min(0)[0]
    extent = (pos.max(0)[0] - lo).max().clamp(min=1e-8)
    q = ((pos - lo) / extent * 1023).long().clamp(0, 1023)
    code = _expand_bits_10(q[:, 0]) | (_expand_bits_10(q[:, 1]) << 1) | (_expand_bits_10(q[:, 2]) << 2)
    order = torch.sort(code, stable=True).indices
    out = torch.empty(n, dtype=torch.long, device=pos.device)
    out[order] = torch.arange(n, device=pos.device) * num_ranks // n
    return out


def _all_to_all(out: torch.Tensor, inp: torch.Tensor, out_splits: list[int], in_splits: list[int], group) -> None:
    """all_to_all_single with variable splits along dim 0; point-to-point fallback where the backend
    lacks the collective (Gloo), as the reference does (graph_parallel_a2a.py:24-60)."""
    world = dist.get_world_size(group)
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)
        return
    rank = dist.get_rank(group)
    ins = list(inp.split(in_splits, dim=0))
    outs = list(out.split(out_splits, dim=0))
    outs[rank].copy_(ins[rank])
    reqs = []
    for peer in range(world):
        if peer == rank:
            continue
        if out_splits[peer]:
            reqs.append(dist.irecv(outs[peer], src=dist.get_global_rank(group, peer) if group is not None else peer, group=group))
        if in_splits[peer]:
            reqs.append(dist.isend(ins[peer].contiguous(), dst=dist.get_global_rank(group, peer) if group is not None else peer, group=group))
    for r in reqs:
        r.wait()


@dataclass
class GPPlan:
    """Everything one rank needs for a step: its atoms, its halo and the exchange pattern."""

    rank: int
    world: int
    group: object
    node_partition: torch.Tensor    # [n_local] global ids of the atoms this rank owns (ascending)
    halo_ids: torch.Tensor          # [n_halo] global ids of remote source atoms, grouped by owner rank
    full_ids: torch.Tensor          # [n_local + n_halo] = cat(node_partition, halo_ids)
    edge_index_local: torch.Tensor  # [2,E]: source in [0, n_local+n_halo), target in [0, n_local), grouped by target
    cell_offsets: torch.Tensor      # [E,3]
    send_idx: torch.Tensor          # [n_send] local rows other ranks asked for, grouped by destination rank
    send_splits: list               # rows sent to each rank per exchange
    recv_splits: list               # rows received from each rank per exchange (sums to n_halo)

    @property
    def n_local(self) -> int:
        return int(self.node_partition.shape[0])

    @property
    def n_halo(self) -> int:
        return int(self.halo_ids.shape[0])


def build_plan(edge_index: torch.Tensor, cell_offsets: torch.Tensor, assignments: torch.Tensor, rank: int, world: int,
               group=None) -> GPPlan:
    """Local numbering and exchange pattern from this rank's edges (global ids, targets owned by
    ``rank`` and grouped by target); counterpart of ``build_gp_context`` (graph_parallel_a2a.py:234-357)."""
    dev = edge_index.device
    n = assignments.shape[0]
    node_partition = (assignments == rank).nonzero(as_tuple=True)[0]
    n_local = int(node_partition.shape[0])
    src_g, tgt_g = edge_index[0], edge_index[1]
    remote = assignments[src_g] != rank
    needed = torch.unique(src_g[remote])
    owner = assignments[needed]
    order = torch.sort(owner, stable=True).indices
    halo_ids = needed[order]
    recv_splits = torch.bincount(owner, minlength=world)
    g2l = torch.full((n,), -1, dtype=torch.long, device=dev)
    g2l[node_partition] = torch.arange(n_local, device=dev)
    g2l[halo_ids] = n_local + torch.arange(halo_ids.shape[0], device=dev)
    edge_local = torch.stack([g2l[src_g], g2l[tgt_g]])
    # tell every owner which of its atoms this rank needs
    send_splits = torch.empty_like(recv_splits)
    ones = [1] * world
    _all_to_all(send_splits, recv_splits, ones, ones, group)
    recv_l, send_l = recv_splits.tolist(), send_splits.tolist()
    wanted = torch.empty(sum(send_l), dtype=torch.long, device=dev)
    _all_to_all(wanted, halo_ids, send_l, recv_l, group)
    send_idx = g2l[wanted]
    if wanted.numel() and bool(((send_idx < 0) | (send_idx >= n_local)).any()):
        raise RuntimeError("graph-parallel plan: a rank was asked for an atom it does not own")
    return GPPlan(rank, world, group, node_partition, halo_ids, torch.cat([node_partition, halo_ids]), edge_local,
                  cell_offsets, send_idx, send_l, recv_l)


class _HaloCollect(torch.autograd.Function):
    """x_local [n_local, ...] -> x_full [n_local + n_halo, ...]: own rows followed by the rows fetched
    from their owners (AllToAllCollect, graph_parallel_a2a.py:360-562)."""

    @staticmethod
    def forward(ctx, x_local, plan: GPPlan):
        send = x_local.index_select(0, plan.send_idx).contiguous()
        out = torch.empty((plan.n_local + plan.n_halo,) + tuple(x_local.shape[1:]), dtype=x_local.dtype, device=x_local.device)
        out[: plan.n_local].copy_(x_local)
        _all_to_all(out[plan.n_local:], send, plan.recv_splits, plan.send_splits, plan.group)
        ctx.plan = plan
        return out

    @staticmethod
    def backward(ctx, grad_full):
        plan = ctx.plan
        grad_full = grad_full.contiguous()
        back = torch.empty((len(plan.send_idx),) + tuple(grad_full.shape[1:]), dtype=grad_full.dtype, device=grad_full.device)
        _all_to_all(back, grad_full[plan.n_local:].contiguous(), plan.send_splits, plan.recv_splits, plan.group)
        grad_local = grad_full[: plan.n_local].clone()
        grad_local.index_add_(0, plan.send_idx, back)
        return grad_local, None


def halo_collect(x_local: torch.Tensor, plan: Optional[GPPlan]) -> torch.Tensor:
    return x_local if plan is None else _HaloCollect.apply(x_local, plan)


class PartitionedStepper:
    """Energy+forces of one replicated system, computed by ``world`` ranks that each own a Morton region."""

    def __init__(self, backbone, head, host_data, device, rank: int, world: int, group=None):
        self.bb, self.head = backbone, head
        self.rank, self.world, self.group, self.device = rank, world, group, device
        self.last_plan: Optional[GPPlan] = None

    def step(self, data):
        """One energy+forces evaluation.  The contraction status word is agreed on by all ranks before anyone acts on
        it: either every rank repeats the step with the TF32 split (half-range overflow on any rank) or every rank
        raises (expired wait on any rank), so no rank is left waiting in a collective its peers never enter."""
        from . import backbone as B

        return run_agreed(lambda: self._step_once(data), self.group, B.read_gemm_status, B.raise_gemm_status,
                          lambda: B._GemmState.precision, B.set_gemm_precision, self.device)

    def _step_once(self, data):
        from .graph import radius_graph_pbc_b200

        if data["pos"].grad is not None:
            data["pos"].grad = None
        pos = data["pos"].detach()
        # every rank must see the same positions: rank 0's are authoritative (predict.py:828-833)
        dist.broadcast(pos, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0, group=self.group)
        with torch.no_grad():
            assign = morton_partition(pos, self.world)
            part = (assign == self.rank).nonzero(as_tuple=True)[0]
            if part.numel() == 0:
                raise RuntimeError("graph-parallel: this rank owns no atoms")
            data["node_partition"] = part
            edge_index, cell_offsets, _ = radius_graph_pbc_b200(data, self.bb.cutoff, self.bb.max_neighbors, False, data["pbc"])
            del data["node_partition"]
            plan = build_plan(edge_index, cell_offsets, assign, self.rank, self.world, self.group)
        self.last_plan = plan
        data["gp_plan"] = plan
        emb = self.bb(data)
        out = self.head(data, emb, check_status=False)
        del data["gp_plan"]
        energy, forces = out["energy"], out["forces"]
        dist.all_reduce(energy, group=self.group)
        dist.all_reduce(forces, group=self.group)
        if "stress" in out:  # every rank holds the virial of its own targets' edges
            dist.all_reduce(out["stress"], group=self.group)
            self.last_stress = out["stress"]
        return energy, forces


def agree_on_status(code: int, group, device) -> int:
    """The largest status code any rank of ``group`` holds (one small all-reduce)."""
    t = torch.tensor([int(code)], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return int(t.item())


def run_agreed(step_once, group, read_status, raise_status, get_precision, set_precision, device):
    """Run ``step_once`` on every rank, then act on the ranks' *common* status: 0 returns the result, 2 (half-range
    overflow somewhere) repeats the step on all ranks with precision 3 and restores the mode, anything else raises on
    all ranks.  The step's collectives all complete before the status is looked at."""
    result = step_once()
    code = agree_on_status(read_status(), group, device)
    if code == 0:
        return result
    if code != 2 or get_precision() != 2:
        raise_status(code)
    set_precision(3)
    try:
        result = step_once()
        raise_status(agree_on_status(read_status(), group, device))
        return result
    finally:
        set_precision(2)
