"""Ray sharding and the gradient all-reduce on CPU ranks (gloo, world size 2).

Each rank renders its slice with the CPU oracle (the CUDA kernels need a GPU);
what is under test is the host logic of svox_b200.distributed: slices tile the
batch, the reduced gradient equals the single-process gradient, and gathered
outputs come back in order.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from svox_b200 import distributed as D


def test_shard_bounds_tile_the_batch():
    for n in (0, 1, 7, 32, 1000, 1 << 20):
        for world in (1, 2, 3, 8):
            cuts = [D.shard_bounds(n, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from golden.cases import CASES
        from oracle import oracle as orc
        case = CASES["shell_sh9_rays"]()
        tree = case["tree"]
        if rank != 0:                      # replicas start empty and receive rank 0's tree
            with torch.no_grad():
                tree.data.zero_()
        D.broadcast_tree(tree, src=0)
        rays = D.shard_rays(case["rays"])
        gout = D.shard_rows(case["grad_out"])
        ot = orc.Tree.from_n3tree(tree)
        opt = orc.options(basis_dim=9)
        o, d, v = [t.numpy() for t in rays]
        out = torch.from_numpy(orc.volume_render(ot, o, d, v, opt))
        grad = orc.volume_render_backward(ot, o, d, v, opt, gout.numpy())
        tree.data.grad = torch.from_numpy(grad).float()
        D.allreduce_grad(tree)
        full = D.gather_rows(out, case["rays"].origins.shape[0])
        if rank == 0:
            np.savez(os.path.join(out_dir, "dist.npz"), out=full.numpy(),
                     grad=tree.data.grad.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_ranks_match_single_process(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    z = np.load(tmp_path / "dist.npz")
    import parity_util as P
    from golden.cases import CASES
    single = P.run_oracle(CASES["shell_sh9_rays"]())
    assert np.array_equal(z["out"], single["out"])          # shards are bit-equal, in order
    err = np.abs(z["grad"] - single["grad"]).max() / np.abs(single["grad"]).max()
    assert err <= 1e-6                                      # float32 sum of two double sums
