"""Multi-rank host logic on CPU (gloo, world_size 2 and 3): scene-group sharding and the
Morton-range partition with its halo plan and exchange.  Neighbour search and Morton codes
come from the oracle here; on GPUs the same code uses the native kernels."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kernel_map as km
from oracle import sparse_conv as osc
from warpconvnet_b200.datasets import synthetic
from warpconvnet_b200.dist.halo import morton_partition, plan_halo
from warpconvnet_b200.dist.sharding import split_scene_groups


def test_split_scene_groups():
    offs = [0, 100, 250, 300, 700, 720, 1000, 1100, 1200]
    for w in (1, 2, 4, 8):
        groups = split_scene_groups(offs, w)
        assert groups[0][0] == 0 and groups[-1][1] == 8
        assert all(groups[i][1] == groups[i + 1][0] for i in range(w - 1))
    assert split_scene_groups(offs, 8) == [(i, i + 1) for i in range(8)]
    g2 = split_scene_groups(offs, 2)
    assert g2 == [(0, 4), (4, 8)]  # 700 is the boundary nearest to half of 1200
    assert split_scene_groups([0, 10, 20], 4)[-1][1] == 2  # more ranks than scenes: some groups empty
    assert split_scene_groups([0], 2) == [(0, 0), (0, 0)]


def _oracle_neighbor_fn(global_coords, owned):
    return torch.from_numpy(km.kernel_map_found(global_coords.numpy(), owned.numpy(), (1, 1, 1), (3, 3, 3)))


def _oracle_morton_fn(xyz):
    return torch.from_numpy(km.morton_code(xyz.numpy()))


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        xyz = synthetic.room_scene(6000, 0.05, 77, "raster_crop")
        coords = torch.from_numpy(np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1))
        g = torch.Generator().manual_seed(0)
        feats = torch.randn(len(xyz), 8, generator=g)
        w = torch.randn(27, 8, 12, generator=g) * 0.2
        perm, bounds = morton_partition(coords, world, morton_fn=_oracle_morton_fn)
        gc, gf = coords[perm], feats[perm]
        plan = plan_halo(gc, bounds, rank, world, neighbor_fn=_oracle_neighbor_fn)
        lo, hi = bounds[rank], bounds[rank + 1]
        assert plan.num_owned == hi - lo and sum(plan.recv_counts) == plan.num_halo
        assert plan.recv_counts[rank] == 0 and plan.send_counts[rank] == 0
        # the owned rows split into those whose window needs a halo row and those that do not
        both = torch.cat([plan.interior_rows, plan.boundary_rows]).sort().values
        assert torch.equal(both, torch.arange(plan.num_owned, dtype=torch.int32))
        assert int((plan.nbr_local[:, plan.interior_rows.long()] >= plan.num_owned).sum()) == 0
        assert bool((plan.nbr_local[:, plan.boundary_rows.long()] >= plan.num_owned).any(dim=0).all())
        local = plan.exchange(gf[lo:hi])
        # received halo rows are exactly the global rows the plan names
        assert torch.equal(local[plan.num_owned:], gf[plan.halo_global])
        # owned outputs from local rows == rows of the single-process convolution
        i, o, f, iden = km.generate_kernel_map(gc.numpy(), gc.numpy(), (1, 1, 1), (3, 3, 3))
        ref = osc.explicit_gemm_forward(gf, w, i, o, f, iden, len(gc))[lo:hi]
        out = torch.zeros(hi - lo, 12)
        nl = plan.nbr_local.long()
        for k in range(27):
            hit = nl[k] >= 0
            out[hit] += local[nl[k][hit]] @ w[k]
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)
        open(os.path.join(out_dir, f"ok{rank}"), "w").write(f"{plan.num_owned} {plan.num_halo}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,port", [(2, 29541), (3, 29543)])
def test_morton_partition_and_halo_exchange_gloo(world, port, tmp_path):
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    done = sorted(os.listdir(tmp_path))
    assert done == [f"ok{r}" for r in range(world)]
    halos = [int(open(tmp_path / f).read().split()[1]) for f in done]
    assert all(h > 0 for h in halos)


def _fail_worker(rank, world, port, out_dir):
    """A rank that raises before the exchange: the others must get an error from the
    collective (short process-group timeout), not hang."""
    import datetime
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 1:
            raise RuntimeError("injected host-side failure")
        x = torch.zeros(4)
        y = torch.empty(4)
        try:
            dist.all_to_all_single(y, x, [2, 2], [2, 2])
            outcome = "completed"
        except Exception as e:  # noqa: BLE001 - any collective error is the expected outcome
            outcome = "error:" + type(e).__name__
        open(os.path.join(out_dir, f"r{rank}"), "w").write(outcome)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_peer_failure_surfaces_as_collective_error(tmp_path):
    ctx = mp.spawn(_fail_worker, args=(2, 29547, str(tmp_path)), nprocs=2, join=False)
    deadline = 60
    import time
    t0 = time.time()
    while time.time() - t0 < deadline and not os.path.exists(tmp_path / "r0"):
        time.sleep(0.2)
    for p in ctx.processes:
        p.join(timeout=10)
        if p.is_alive():
            p.terminate()
    assert os.path.exists(tmp_path / "r0"), "surviving rank hung instead of failing"
    assert open(tmp_path / "r0").read().startswith("error:")
