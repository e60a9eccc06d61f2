"""Worker for the 2-GPU expert-parallel test: the fused peer-load dispatch/combine path and the
collective baseline against a single-rank evaluation of the same MoE layer on all tokens."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from brain_b200.ops import _cuda
    from brain_b200.ops.moe import moe_forward
    from brain_b200.parallel.ep import ExpertParallel

    torch.manual_seed(0)
    n, d, E, k, ff = 384, 256, 8, 2, 128
    x_all = torch.randn(world * n, d, device=dev).bfloat16()
    router = (0.3 * torch.randn(E, d, device=dev)).bfloat16()
    wgu = (0.05 * torch.randn(E, 2 * ff, d, device=dev)).bfloat16()
    wd = (0.05 * torch.randn(E, d, ff, device=dev)).bfloat16()
    dy_all = torch.randn(world * n, d, device=dev).bfloat16()
    El = E // world

    # single-rank oracle over all tokens with all experts (same kernels, no parallelism)
    xr = x_all.clone().requires_grad_()
    gr, dr = wgu.clone().requires_grad_(), wd.clone().requires_grad_()
    yr, _, _ = moe_forward(xr, router, gr, dr, k, True, 1.0, 0.0, 0.0)
    yr.backward(dy_all)

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()

    ok, msgs = True, []
    for impl in ("fused", "nccl"):
        ep = ExpertParallel(impl=impl, device=dev, arena_mb=256)
        for it in range(2):
            x = x_all[rank * n:(rank + 1) * n].clone().requires_grad_()
            g = wgu[rank * El:(rank + 1) * El].clone().requires_grad_()
            dn = wd[rank * El:(rank + 1) * El].clone().requires_grad_()
            y, _, _ = moe_forward(x, router, g, dn, k, True, 1.0, 0.0, 0.0, ep=ep)
            y.backward(dy_all[rank * n:(rank + 1) * n])
            torch.cuda.synchronize()
            _cuda.check_error()
            errs = (rel(y, yr[rank * n:(rank + 1) * n]), rel(x.grad, xr.grad[rank * n:(rank + 1) * n]),
                    rel(g.grad, gr.grad[rank * El:(rank + 1) * El]),
                    rel(dn.grad, dr.grad[rank * El:(rank + 1) * El]))
            msgs.append((impl, it, errs))
            ok = ok and all(e < 3e-2 for e in errs)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP_PARITY", msgs, "ok=%d" % int(flag.item()))
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
