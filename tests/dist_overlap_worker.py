"""Worker of the multi-GPU tests (one process per GPU under torchrun): the gradient summed
range by range inside the backward, and the gradient summed by the switch in symmetric memory,
equal the gradient summed by one all-reduce."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import svox_b200  # noqa: E402
from golden.cases import CASES  # noqa: E402
from svox_b200 import distributed as D  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    case = CASES["shell_sh9_rays"]()
    tree = case["tree"].to(dev)
    rays = D.shard_rays(svox_b200.Rays(*[t.to(dev) for t in case["rays"]]))
    gout = D.shard_rows(case["grad_out"].to(dev))
    renderer = svox_b200.VolumeRenderer(tree)

    def step():
        tree.zero_grad(set_to_none=True)
        renderer(rays).backward(gout)
        D.allreduce_grad(tree)
        return tree.data.grad.clone()

    step()                      # lets the item-log estimate settle
    plain = step()
    D.overlap_grad_allreduce(4, reserve_sms=16)
    over = step()
    D.overlap_grad_allreduce(0)
    scale = plain.abs().max().item()
    err = (over - plain).abs().max().item() / scale
    # the gradient in symmetric memory, summed by the switch (where the GPUs offer multicast
    # memory; asked for with SVOXB_TEST_MULTICAST=1)
    err_mc = 0.0
    if os.environ.get("SVOXB_TEST_MULTICAST") == "1":
        try:
            mc = D.MulticastGradient(tree)
        except Exception as e:                      # no multicast memory here
            mc = None
            print(f"rank {dist.get_rank()}: no multicast gradient ({e!r})"[:200], flush=True)
        have = torch.tensor([int(mc is not None)], device=dev)
        dist.all_reduce(have, op=dist.ReduceOp.MIN)
        if have.item():
            mc.enable()
            summed = step()
            assert mc.owns(tree.data.grad)
            D.MulticastGradient.disable()
            err_mc = (summed - plain).abs().max().item() / scale
            if dist.get_rank() == 0:
                print(f"multicast_vs_plain max_rel_err {err_mc:.3e}", flush=True)
    svox_b200.csrc.check_device_status()
    ok = torch.tensor([1 if max(err, err_mc) < 1e-5 else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if dist.get_rank() == 0:
        print(f"overlap_vs_plain max_rel_err {err:.3e} ok {int(ok.item())}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
