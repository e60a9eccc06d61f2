"""Worker for the 2-GPU tensor-parallel test: fused AG->GEMM / GEMM->RS / one-shot all-reduce
kernels against the NCCL baseline and against an unsharded fp32 reference."""
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
    from brain_b200.parallel.tp import TensorParallel, column_parallel_linear, row_parallel_linear

    fused = TensorParallel(impl="fused", device=dev, arena_mb=256)
    base = TensorParallel(impl="nccl")
    torch.manual_seed(0)  # same tensors on every rank
    S, d, ff = 1024, 512, 1024
    x = (torch.randn(S, d, device=dev) * 0.5).bfloat16()
    w1 = (torch.randn(ff, d, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(d, ff, device=dev) * 0.05).bfloat16()
    rows, cols = S // world, ff // world
    ok = True
    msgs = []

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()

    for it in range(3):   # repeated calls exercise the double-buffered slots and epochs
        res = {}
        for name, tp in (("fused", fused), ("nccl", base)):
            xs = x[rank * rows:(rank + 1) * rows].clone().requires_grad_()
            w1s = w1[rank * cols:(rank + 1) * cols].clone().requires_grad_()
            w2s = w2[:, rank * cols:(rank + 1) * cols].clone().contiguous().requires_grad_()
            h = column_parallel_linear(xs, w1s, tp)
            y = row_parallel_linear(h, w2s, tp)
            dy = torch.ones_like(y) * 0.01
            y.backward(dy)
            res[name] = (y.detach(), xs.grad, w1s.grad, w2s.grad)
        torch.cuda.synchronize()
        _cuda.check_error()
        want_y = (x.float() @ w1.float().t() @ w2.float().t())[rank * rows:(rank + 1) * rows]
        e0 = rel(res["fused"][0], want_y)
        errs = [rel(a, b) for a, b in zip(res["fused"], res["nccl"])]
        msgs.append((it, e0, errs))
        ok = ok and e0 < 3e-2 and all(e < 2e-2 for e in errs)
    # one-shot all-reduce
    for it in range(4):
        t = (torch.randn(256, 1024, device=dev) * (rank + 1)).bfloat16()
        a = fused.all_reduce(t)
        b = base.all_reduce(t)
        torch.cuda.synchronize()
        e = rel(a, b)
        ok = ok and e < 1e-2
        msgs.append(("ar", it, e))
    _cuda.check_error()
    if fused.nvls:
        # BRAIN_TP_NVLS=1 and a multicast binding: the calls above went through the switch; every
        # rank must hold the SAME bits (one sum per slice, written to all ranks by the switch)
        t = (torch.randn(64, 2048, device=dev) * (rank + 1)).bfloat16()
        a = fused.all_reduce(t).clone()
        ref0 = a.clone()
        dist.broadcast(ref0, 0)
        same = bool((ref0 == a).all().item())
        ok = ok and same
        msgs.append(("nvls_bit_identical", same))
    else:
        msgs.append(("nvls", "off"))
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_PARITY", msgs, "ok=%d" % int(flag.item()))
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
