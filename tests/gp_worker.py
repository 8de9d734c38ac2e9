"""Worker for tests/test_gpu_multi.py: one rank of a graph-parallel energy+force evaluation.

Launched with ``python -m torch.distributed.run --nproc-per-node N tests/gp_worker.py OUT.pt [natoms] [uma_s|escn_md_l4]``.
"""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from fairchem_b200 import parallel, synthetic, weights  # noqa: E402
from fairchem_b200.backbone import build_model  # noqa: E402


def main():
    out_path = sys.argv[1]
    natoms = int(sys.argv[2]) if len(sys.argv) > 2 else 3000
    cfg = weights.ESCN_MD_L4 if len(sys.argv) > 3 and sys.argv[3] == "escn_md_l4" else weights.UMA_S
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    sd = weights.random_init_state_dict(cfg, 0)
    bb, head = build_model(cfg, sd, device=dev, edge_chunk_size=8192, regress_stress=True)
    host = synthetic.water_box(natoms, seed=1)
    data = host.to(dev)
    stepper = parallel.PartitionedStepper(bb, head, host, dev, rank, world)
    energy, forces = stepper.step(data)
    stress = stepper.last_stress.clone()
    energy2, forces2 = stepper.step(data)  # a second step reuses nothing stale
    plan = stepper.last_plan
    stats = torch.tensor([plan.n_local, plan.n_halo, plan.edge_index_local.shape[1]], device=dev)
    gathered = [torch.zeros_like(stats) for _ in range(world)]
    dist.all_gather(gathered, stats)
    if rank == 0:
        torch.save({"energy": energy.cpu(), "forces": forces.cpu(), "energy2": energy2.cpu(), "forces2": forces2.cpu(), "stress": stress.cpu(),
                    "stats": torch.stack(gathered).cpu()}, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
