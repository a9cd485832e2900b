"""World-size-2 checks on CPU (gloo): tensor-parallel ranks shard the KV heads, plan identically
from the same slot mapping, and agree on every tier decision after the canary mean."""

import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from echokv_b200.canary import tp_mean
    from echokv_b200.controller import ControllerParams, LayerController
    from echokv_b200.write_plan import WritePlanner

    # each rank's canary sees only its own KV heads: different local deltas
    rng = np.random.default_rng(100 + rank)
    ctl = [LayerController(ControllerParams(tau0=0.01, alpha=0.5, init_bits=8)) for _ in range(6)]
    planner = WritePlanner(16, 16, 8, 16)
    trace = []
    for step in range(12):
        local = torch.from_numpy(np.abs(rng.standard_normal((6, 3))) * np.array([0.03, 0.008, 0.0005])).float()
        mean = tp_mean(local.clone())
        gathered = [torch.zeros_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        assert torch.allclose(mean, sum(gathered) / world, atol=1e-7)
        for c, row in zip(ctl, mean.tolist()):
            c.observe(dict(zip((2, 4, 8), row)), 4096.0)
        # host planning is replicated: same slot mapping on every rank -> same plan
        slots = np.arange(step * 5, step * 5 + 5)
        plan = planner.plan(torch.from_numpy(slots))
        trace.append([c.bits for c in ctl] + plan.tok_res.tolist() + plan.tok_kref.tolist() + [plan.n_fin])
    np.save(os.path.join(out_dir, f"trace{rank}.npy"), np.array(trace))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_agree_on_tiers_and_plans(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "trace0.npy"), np.load(tmp_path / "trace1.npy")
    assert np.array_equal(a, b)
    assert len({tuple(r[:6]) for r in a}) > 1  # tiers actually moved during the run


def test_tp_mean_is_identity_without_a_group():
    from echokv_b200.canary import tp_mean

    x = torch.arange(6.0).view(2, 3)
    assert tp_mean(x) is x
