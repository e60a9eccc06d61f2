"""Worker for the multi-GPU data-parallel parity test (launched by torch.distributed.run):
trains the same tiny Qwen3 for a few steps with the NCCL baseline and with the fused NVLink
kernels and checks that both reach the same weights, and that the ranks agree with each other."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(impl, dev, rank, world, steps=3, overlap=None):
    if overlap is not None:     # read when the fused step is built: buckets under backward (1) or after it (0)
        os.environ["BRAIN_DP_OVERLAP"] = overlap
    from brain_b200.engine import Trainer
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.parallel.zero import ZeroDP

    cfg = QwenConfig(vocab=1024, block_size=256, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2,
                     head_dim=64, d_ff=512)
    model = Qwen3(cfg).init_weights(seed=0)
    tr = Trainer(model, device=dev, dp=ZeroDP(impl=impl))
    g = torch.Generator().manual_seed(100 + rank)
    losses = []
    for _ in range(steps):
        ids = torch.randint(0, cfg.vocab, (2, 257), generator=g, dtype=torch.int32)
        loss = tr.train_step(ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), 1e-3, 1,
                             global_count=2 * 256 * world)
        losses.append(float(loss.item()))
    torch.cuda.synchronize()
    return tr.store.weights[: tr.store.n_train].float().clone(), losses


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from brain_b200.ops import _cuda

    w_nccl, l_nccl = run("nccl", dev, rank, world)
    w_fused, l_fused = run("fused", dev, rank, world, overlap="0")
    # the same with every gradient bucket's reduce-scatter started under the last micro-batch's backward
    # (what large models get by default); four steps so that the learnt schedule is used at least twice
    w_over, l_over = run("fused", dev, rank, world, steps=3, overlap="1")
    _cuda.check_error()
    err = max(((w_fused - w_nccl).norm() / w_nccl.norm()).item(),
              ((w_over - w_nccl).norm() / w_nccl.norm()).item())
    assert torch.equal(w_over, w_fused), "overlapped and post-backward bucket reduce must give the same bits"
    # every rank must hold identical weights after the all-gather
    ref = w_fused.clone()
    dist.broadcast(ref, 0)
    same = bool((ref == w_fused).all().item())
    ok = torch.tensor([1 if (err < 2e-3 and same) else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"DP_PARITY world={world} rel_err={err:.3e} ranks_identical={same} "
              f"loss_nccl={l_nccl} loss_fused={l_fused} ok={int(ok.item())}")
    dist.destroy_process_group()
    sys.exit(0 if int(ok.item()) == 1 else 1)


if __name__ == "__main__":
    main()
