"""Distributed logic on CPU ranks (gloo processes and native host collectives): grid, planners,
collectives, thread data parallelism, ZeRO baseline, tensor-parallel primitives and the pipeline
schedules — N-rank result == 1-rank result."""
import threading

import pytest
import numpy as np
import torch

from brain_b200.parallel.collective import CollectiveError, HostCollective, NetworkCollective
from brain_b200.parallel.grid import Grid
from brain_b200.parallel.plan import (Hardware, ModelShape, ShardCost, plan_balanced, plan_by_capacity,
                                      plan_tp, schedule, tp_step_secs)
from tests.mp_util import run_ranks


def test_grid_rank_formula_and_groups():
    g = Grid(tp=2, pp=2, dp=2)
    assert g.world == 8
    for r in range(8):
        assert g.rank_of(*g.coord_of(r)) == r
    assert g.tp_group(5) == [4, 5] and g.pp_group(5) == [5, 7] and g.dp_group(5) == [1, 5]
    assert len(g.all_groups("dp")) == 4 and sorted(sum(g.all_groups("pp"), [])) == list(range(8))


def test_local_groups_reduce_inside_each_group():
    """Thread ranks of a 2 x 1 x 2 grid: the tensor-parallel all-reduce sums inside each TP pair, the
    data-parallel one across the pairs."""
    import threading
    from brain_b200.parallel.grid import Grid, LocalGroups
    g = Grid(tp=2, pp=1, dp=2)
    lg = LocalGroups(g, timeout_s=10.0)
    tp_out, dp_out = [None] * 4, [None] * 4

    def work(r):
        t = torch.full((3,), float(r + 1))
        lg.tp(r).all_reduce(t)
        tp_out[r] = t.clone()
        d = torch.full((3,), float(r + 1))
        lg.dp(r).all_reduce(d)
        dp_out[r] = d
    ths = [threading.Thread(target=work, args=(r,)) for r in range(4)]
    [t.start() for t in ths]
    [t.join(20) for t in ths]
    # ranks 0,1 form one TP group (dp 0), ranks 2,3 the other; DP groups are {0,2} and {1,3}
    assert [float(t[0]) for t in tp_out] == [3.0, 3.0, 7.0, 7.0]
    assert [float(t[0]) for t in dp_out] == [4.0, 6.0, 4.0, 6.0]
    assert lg.pp(2) is not None and lg.tp(0) is not lg.tp(2)


def test_planners():
    p = plan_balanced(ShardCost(12, 1.0, 0.0, 0.0), [0, 1, 2])
    assert [(s.start, s.end) for s in p] == [(0, 4), (4, 8), (8, 12)] and p[0].embed and p[-1].head
    p = plan_balanced(ShardCost(10, 1.0, 0.0, 4.0), [0, 1])       # heavy head pulls the cut right
    assert p[0].end > 5
    assert plan_by_capacity(8, 10.0, 5.0, 5.0, [30.0, 30.0]) is None
    q = plan_by_capacity(8, 10.0, 5.0, 5.0, [40.0, 40.0, 40.0])
    assert q is not None and q[-1].end == 8
    hw = Hardware(n_gpus=8, mem_bytes=100.0)
    assert plan_tp(hw, ModelShape(1024, 1024, 4096, 4, 50.0, 10.0)).degree == 1
    t = plan_tp(hw, ModelShape(1024, 1024, 4096, 4, 300.0, 10.0))
    assert t.degree == 4 and t.fits
    assert not plan_tp(hw, ModelShape(1024, 1024, 4096, 4, 1e6, 10.0)).fits
    assert tp_step_secs(Hardware(), ModelShape(4096, 4096, 16384, 32, 0, 0), 2) > 0
    # measured, uneven per-layer costs: exact min-max against brute force, slack with the early stages
    import itertools
    from brain_b200.parallel.plan import plan_stages
    rng = np.random.default_rng(0)
    for _ in range(20):
        L, k = int(rng.integers(3, 10)), int(rng.integers(2, 4))
        cost = rng.uniform(0.5, 3.0, L)
        emb, head = float(rng.uniform(0, 2)), float(rng.uniform(0, 4))
        got = plan_stages(cost, list(range(k)), emb, head)
        def worst(cuts):
            b = [0, *cuts, L]
            return max(cost[b[i]:b[i + 1]].sum() + (emb if i == 0 else 0) + (head if i == k - 1 else 0) for i in range(k))
        brute = min(worst(c_) for c_ in itertools.combinations_with_replacement(range(L + 1), k - 1))
        assert abs(worst([s.end for s in got[:-1]]) - brute) < 1e-9
    even = plan_stages([1.0] * 10, [0, 1, 2, 3])
    assert [s.end - s.start for s in even] == [1, 3, 3, 3]      # bottleneck 3; the spare room sits in stage 0
    big = ModelShape(8192, 8192, 28672, 80, 200.0, 10.0)
    hw2 = Hardware(n_gpus=8, mem_bytes=1e12)
    assert plan_tp(hw2, big).degree == 1 and plan_tp(hw2, big, fastest=True).degree == 8
    assert tp_step_secs(hw2, big, 8) < tp_step_secs(hw2, big, 1)
    assert schedule("1f1b", 0, 4, 6) == [1, 2, 3, 4, -1, 5, -2, 6, -3, -4, -5, -6]
    assert schedule("1f1b", 3, 4, 6) == [1, -1, 2, -2, 3, -3, 4, -4, 5, -5, 6, -6]
    assert schedule("gpipe", 1, 2, 3) == [1, 2, 3, -3, -2, -1]


def test_host_collective_threads_and_abort():
    g = HostCollective.group(3)
    res = [None] * 3

    def work(r):
        t = torch.full((5,), float(r + 1))
        g[r].all_reduce(t)
        rs = g[r].reduce_scatter(torch.arange(6, dtype=torch.float32) * (r + 1))
        ag = g[r].all_gather(torch.tensor([float(r)]))
        b = torch.full((2,), float(r))
        g[r].broadcast(b, root=2)
        res[r] = (t.tolist(), rs.tolist(), ag.tolist(), b.tolist())

    ths = [threading.Thread(target=work, args=(r,)) for r in range(3)]
    [t.start() for t in ths]
    [t.join() for t in ths]
    assert all(r[0] == [6.0] * 5 and r[2] == [0.0, 1.0, 2.0] and r[3] == [2.0, 2.0] for r in res)
    assert res[1][1] == [12.0, 18.0]
    # a rank that never joins: the waiting rank times out with an error instead of hanging
    g2 = HostCollective.group(2, timeout_s=0.3)
    with pytest.raises(CollectiveError):
        g2[0].all_reduce(torch.ones(3))


def test_network_collective_loopback_and_dropped_peer():
    co = NetworkCollective.coordinator(2)
    out = {}

    def w():
        n = NetworkCollective.worker(1, 2, co.port)
        t = torch.ones(4) * 2
        n.all_reduce(t)
        out["w"] = t.tolist()
        out["g"] = n.all_gather(torch.tensor([5.0])).tolist()
        n.close()   # leaves between steps

    th = threading.Thread(target=w)
    th.start()
    co.accept()
    t = torch.ones(4)
    co.all_reduce(t)
    g = co.all_gather(torch.tensor([3.0])).tolist()
    th.join()
    assert t.tolist() == [3.0] * 4 == out["w"] and g == [3.0, 5.0] == out["g"]
    with pytest.raises(CollectiveError) as e:     # the worker is gone: named, not ignored
        co.all_reduce(torch.ones(4))
    assert "rank 1" in str(e.value)


def test_thread_data_parallel_matches_single_replica():
    from brain_b200.engine import Trainer
    from brain_b200.models.config import GptConfig
    from brain_b200.models.gpt2 import Gpt2
    from brain_b200.parallel.dp import DataParallel
    cfg = GptConfig(vocab=50, block_size=16, n_layers=2, d_model=32, n_heads=2, d_ff=64)
    mk = lambda: Gpt2(cfg).init_weights(0)
    dp = DataParallel(mk, 2, betas=(0.9, 0.95))
    g = torch.Generator().manual_seed(0)
    mbs = [(torch.randint(0, 50, (4, 16), generator=g), torch.randint(0, 50, (4, 16), generator=g))
           for _ in range(2)]
    single = Trainer(mk(), device="cpu", betas=(0.9, 0.95), weight_decay=0.1, grad_clip=1.0)
    tok, tgt = torch.cat([m[0] for m in mbs]), torch.cat([m[1] for m in mbs])
    for _ in range(2):
        l = dp.train_step(mbs, 3e-3, 0.1, 1.0)
        l1 = float(single.train_step(tok, tgt, 3e-3, 4))
        assert abs(l - l1) < 1e-3 * abs(l1)
    assert torch.equal(dp.stores[0].weights, dp.stores[1].weights)


# ------------------------------------------------------------------ gloo process ranks
def _zero_rank(rank, world):
    from brain_b200.engine import Trainer
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.parallel.zero import ZeroDP
    cfg = QwenConfig.tiny()
    tr = Trainer(Qwen3(cfg).init_weights(0), device="cpu", dp=ZeroDP())
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (4, 13), generator=g)
    mine = ids[rank * 2:(rank + 1) * 2]
    losses = [float(tr.train_step(mine[:, :-1].contiguous(), mine[:, 1:].contiguous(), 1e-2, 1, 4 * 12))
              for _ in range(3)]
    return tr.store.weights.clone(), losses


def test_zero_dp_two_gloo_ranks_match_single():
    from brain_b200.engine import Trainer
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    outs = run_ranks(_zero_rank, 2)
    assert torch.equal(outs[0][0], outs[1][0])
    cfg = QwenConfig.tiny()
    tr = Trainer(Qwen3(cfg).init_weights(0), device="cpu")
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (4, 13), generator=g)
    for _ in range(3):
        tr.train_step(ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), 1e-2, 2, 4 * 12)
    n = tr.store.n_train
    rel = ((outs[0][0][:n] - tr.store.weights[:n]).norm() / tr.store.weights[:n].norm()).item()
    assert rel < 1e-3


def _tp_rank(rank, world):
    from brain_b200.parallel.tp import TensorParallel, column_parallel_linear, row_parallel_linear
    torch.manual_seed(0)
    S, d, ff = 8, 16, 32
    x = torch.randn(S, d)
    w1, w2 = torch.randn(ff, d) * 0.2, torch.randn(d, ff) * 0.2
    tp = TensorParallel()
    rows, cols = S // world, ff // world
    xs = x[rank * rows:(rank + 1) * rows].clone().requires_grad_()
    w1s = w1[rank * cols:(rank + 1) * cols].clone().requires_grad_()
    w2s = w2[:, rank * cols:(rank + 1) * cols].clone().requires_grad_()
    h = torch.relu(column_parallel_linear(xs, w1s, tp))
    y = row_parallel_linear(h, w2s, tp)
    dy = torch.arange(S * d, dtype=torch.float32).reshape(S, d) / 100
    y.backward(dy[rank * rows:(rank + 1) * rows])
    return y.detach(), xs.grad, w1s.grad, w2s.grad


def test_tensor_parallel_mlp_matches_unsharded():
    outs = run_ranks(_tp_rank, 2)
    torch.manual_seed(0)
    S, d, ff = 8, 16, 32
    x = torch.randn(S, d).requires_grad_()
    w1, w2 = (torch.randn(ff, d) * 0.2).requires_grad_(), (torch.randn(d, ff) * 0.2).requires_grad_()
    y = torch.relu(x @ w1.t()) @ w2.t()
    dy = torch.arange(S * d, dtype=torch.float32).reshape(S, d) / 100
    y.backward(dy)
    assert torch.allclose(torch.cat([o[0] for o in outs]), y.detach(), atol=1e-5)
    assert torch.allclose(torch.cat([o[1] for o in outs]), x.grad, atol=1e-5)
    assert torch.allclose(torch.cat([o[2] for o in outs]), w1.grad, atol=1e-5)
    assert torch.allclose(torch.cat([o[3] for o in outs], dim=1), w2.grad, atol=1e-5)


def _pp_rank(rank, world, sched):
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.parallel.pipeline import PipelineStage
    cfg = QwenConfig.tiny()
    cfg.n_layers = 4
    full = Qwen3(cfg).init_weights(0)
    bounds = [0, 2, 4]
    stage = Qwen3(cfg, layers=range(bounds[rank], bounds[rank + 1]), first=rank == 0, last=rank == world - 1)
    stage.load_reference_state(full.reference_state(), strict=True)
    import torch.distributed as dist
    tied = dist.new_group([0, world - 1])
    pp = PipelineStage(stage, rank, world, rank - 1 if rank > 0 else None,
                       rank + 1 if rank < world - 1 else None, tied_group=tied, schedule=sched)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab, (4, 13), generator=g)
    toks = [ids[i:i + 1, :-1].contiguous() for i in range(4)]
    tgts = [ids[i:i + 1, 1:].contiguous() for i in range(4)]
    loss = pp.forward_backward(toks, tgts, 1.0 / (4 * 12))
    pp.sync_tied_embeddings()
    grads = {n: p.grad.clone() for n, p in stage.reference_state().items() if p.grad is not None}
    return (None if loss is None else float(loss)), grads


@pytest.mark.parametrize("sched", ["1f1b", "gpipe"])
def test_pipeline_two_stages_match_single(sched):
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    outs = run_ranks(_pp_rank, 2, sched)
    cfg = QwenConfig.tiny()
    cfg.n_layers = 4
    full = Qwen3(cfg).init_weights(0)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab, (4, 13), generator=g)
    loss = full.loss(ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), 1.0 / (4 * 12))
    loss.backward()
    assert abs(outs[1][0] - float(loss)) < 1e-4
    want = {n: p.grad for n, p in full.reference_state().items()}
    for r in range(2):
        for n, gr in outs[r][1].items():
            assert torch.allclose(gr, want[n], atol=2e-5), (sched, r, n)


def _trainer3d_worker(rank, world, tp, pp, sched, dp=1, recompute=False):
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.parallel.grid import Grid
    from brain_b200.parallel.trainer3d import Trainer3D, gather_state
    cfg = QwenConfig(vocab=96, block_size=128, n_layers=4, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64,
                     tie_embeddings=True)
    full = Qwen3(cfg).init_weights(5)
    state = {k: v.detach().clone() for k, v in full.reference_state().items()}
    tr = Trainer3D(cfg, Grid(tp=tp, pp=pp, dp=dp), "cpu", schedule=sched, full_state=state, grad_clip=1.0,
                   weight_decay=0.1, recompute=recompute)
    g = torch.Generator().manual_seed(3)
    toks = [torch.randint(0, 96, (2, 128), generator=g, dtype=torch.int32) for _ in range(4)]
    tgts = [torch.randint(0, 96, (2, 128), generator=g) for _ in range(4)]
    losses = [float(tr.train_step(toks, tgts, 1e-2)) for _ in range(2)]
    out = gather_state(tr)
    return {"losses": losses, "state": out, "norm": float(tr.last_grad_norm)}


@pytest.mark.parametrize("tp,pp,sched,dp,recompute", [(2, 2, "1f1b", 1, False), (2, 1, "1f1b", 1, False),
                                                       (1, 2, "gpipe", 1, True), (1, 2, "1f1b", 2, False),
                                                       (2, 1, "1f1b", 2, True)])
def test_trainer3d_matches_single_process(tp, pp, sched, dp, recompute, monkeypatch):
    """Tensor x pipeline parallel training on gloo CPU ranks reproduces the single-process step:
    same losses, same global gradient norm, same weights after two optimiser steps.  The gpipe case
    also posts its stage-to-stage receives one op ahead (second step on), the others where needed."""
    monkeypatch.setenv("BRAIN_PP_PREFETCH", "1" if sched == "gpipe" else "0")
    from brain_b200.engine import Trainer
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    res = run_ranks(_trainer3d_worker, tp * pp * dp, tp, pp, sched, dp, recompute)
    cfg = QwenConfig(vocab=96, block_size=128, n_layers=4, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64,
                     tie_embeddings=True)
    full = Qwen3(cfg).init_weights(5)
    tr = Trainer(full, device="cpu", weight_decay=0.1, grad_clip=1.0)
    g = torch.Generator().manual_seed(3)
    toks = [torch.randint(0, 96, (2, 128), generator=g, dtype=torch.int32) for _ in range(4)]
    tgts = [torch.randint(0, 96, (2, 128), generator=g) for _ in range(4)]
    want = []
    for _ in range(2):
        want.append(float(tr.train_step(torch.cat(toks), torch.cat(tgts), 1e-2, micro_batch=2)))
    for r in res:
        assert r["losses"] == pytest.approx(want, rel=2e-4)
    assert res[0]["norm"] == pytest.approx(float(tr.opt.last_grad_norm), rel=2e-3)
    ref_state = full.reference_state()
    got = res[0]["state"]
    assert set(got) == set(ref_state)
    for k, v in ref_state.items():
        assert torch.allclose(got[k], v.detach().reshape(-1), atol=2e-4), k


def _trainer_ep_worker(rank, world, recompute="none"):
    from brain_b200.models.config import MoeConfig
    from brain_b200.models.moe import MoeModel
    from brain_b200.parallel.ep import ExpertParallel
    from brain_b200.parallel.trainer_ep import TrainerEP, is_expert_param
    cfg = MoeConfig(vocab=64, block_size=16, n_layers=2, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, n_experts=4,
                    top_k=2, d_ff=16, aux_coef=0.0, z_coef=0.0, tie_embeddings=True)
    ep = ExpertParallel(impl="nccl")
    model = MoeModel(cfg, ep=ep).init_weights(7)
    model.recompute_blocks = recompute == "blocks"
    model.recompute_experts = recompute == "experts"
    tr = TrainerEP(model, "cpu", betas=(0.9, 0.95), weight_decay=0.1, grad_clip=1.0)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 64, (4, 16), generator=g, dtype=torch.int32)
    tgts = torch.randint(0, 64, (4, 16), generator=g)
    mine = slice(2 * rank, 2 * rank + 2)
    losses = []
    for _ in range(2):
        losses.append(float(tr.train_step(toks[mine], tgts[mine], 1e-2, global_count=4 * 16)))
    state = {n: p.detach().clone() for n, p in model.named_parameters()}
    return {"losses": losses, "norm": float(tr.last_grad_norm), "state": state,
            "e_first": model.blocks[0].moe.e_first, "e_local": model.blocks[0].moe.e_local}


@pytest.mark.parametrize("recompute", ["none", "experts", "blocks"])
def test_trainer_ep_two_gloo_ranks_match_single_process(recompute):
    """Expert-parallel training (experts split over 2 CPU ranks, each rank its own sequences)
    reproduces single-process training on all sequences: summed losses, global gradient norm,
    shared weights and each rank's expert slice after two optimiser steps.  The same holds when
    backward re-runs only the expert layers, or whole blocks, instead of keeping their activations
    (the re-run repeats the dispatch and combine collectives on every rank alike)."""
    from brain_b200.engine import Trainer
    from brain_b200.models.config import MoeConfig
    from brain_b200.models.moe import MoeModel
    from brain_b200.parallel.trainer_ep import is_expert_param
    res = run_ranks(_trainer_ep_worker, 2, recompute)
    cfg = MoeConfig(vocab=64, block_size=16, n_layers=2, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, n_experts=4,
                    top_k=2, d_ff=16, aux_coef=0.0, z_coef=0.0, tie_embeddings=True)
    full = MoeModel(cfg).init_weights(7)
    tr = Trainer(full, device="cpu", betas=(0.9, 0.95), weight_decay=0.1, grad_clip=1.0)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 64, (4, 16), generator=g, dtype=torch.int32)
    tgts = torch.randint(0, 64, (4, 16), generator=g)
    want = [float(tr.train_step(toks, tgts, 1e-2, micro_batch=2)) for _ in range(2)]
    got = [res[0]["losses"][i] + res[1]["losses"][i] for i in range(2)]
    assert got == pytest.approx(want, rel=2e-4)
    assert res[0]["norm"] == pytest.approx(float(tr.opt.last_grad_norm), rel=2e-3)
    assert res[1]["norm"] == pytest.approx(res[0]["norm"], rel=1e-6)
    ref_state = dict(full.named_parameters())
    for r in res:
        lo, n = r["e_first"], r["e_local"]
        for k, v in r["state"].items():
            want_t = ref_state[k].detach()
            if is_expert_param(k):
                want_t = want_t[lo:lo + n]
            assert torch.allclose(v, want_t, atol=2e-4), (k, float((v - want_t).abs().max()))


def test_bucket_tracker_learns_counts_and_reruns_early_buckets():
    """Host logic of the overlapped data-parallel step: buckets are cut inside rank shards and listed
    back to front; a bucket is released by the last expected accumulation of its parameters; an
    accumulation that arrives after its bucket went out marks the bucket for a second run."""
    from brain_b200.parallel.fused_dp import BucketTracker, make_buckets
    buckets = make_buckets(64, 2, 16)
    assert buckets == [(1, 48, 64), (1, 32, 48), (0, 16, 32), (0, 0, 16)]
    # parameters: E (tied embedding, accumulated twice) [0,20), A [20,40), B [40,64)
    slots = [(1, 0, 20), (2, 20, 20), (3, 40, 24)]
    t = BucketTracker(buckets, slots)
    order = [1, 3, 2, 1]                        # head's dW into E, then B, A, then the embedding scatter
    t.begin()
    assert [t.notify(k) for k in order] == [[], [], [], []]      # first step: nothing is known yet
    assert t.finish() == [0, 1, 2, 3]
    t.begin()
    got = [t.notify(k) for k in order]
    assert got == [[], [0], [1], [2, 3]]        # B frees bucket 0; A frees 1 (B+A done); E's 2nd frees 2 and 3
    assert t.finish() == []
    # a step in which E is accumulated a third time: its buckets were already out -> run again
    t.begin()
    for k in order:
        t.notify(k)
    assert t.notify(1) == []
    assert t.finish() == [2, 3]
    t.begin()                                   # and the new count is the expectation from now on
    got = [t.notify(k) for k in order + [1]]
    assert got[-1] == [2, 3] and got[3] == []


def test_ep_row_transfers_go_inside_the_gemm_only_for_wide_experts(monkeypatch):
    """``auto``: the dispatch / combine ride inside the grouped GEMMs from an expert GEMM width of 4096
    columns; explicit 1 / 0 override it in both directions."""
    from brain_b200.parallel.ep import ExpertParallel
    ep = ExpertParallel.__new__(ExpertParallel)
    ep._fuse_mode = ("auto", "auto")
    assert not ep.fuse_dispatch(1536) and not ep.fuse_combine(1536)
    assert ep.fuse_dispatch(4096) and ep.fuse_combine(8192)
    ep._fuse_mode = ("1", "0")
    assert ep.fuse_dispatch(64) and not ep.fuse_combine(1 << 20)


def test_dp_buckets_cover_every_shard_once_and_in_backward_order():
    from brain_b200.parallel.fused_dp import BucketTracker, make_buckets
    n, world = 8 * 4 * 100, 4
    b = make_buckets(n, world, 8 * 30)
    covered = sorted((a, e) for _, a, e in b)
    assert covered[0][0] == 0 and covered[-1][1] == n
    assert all(covered[i][1] == covered[i + 1][0] for i in range(len(covered) - 1))
    shard = n // world
    assert all(a // shard == o and (e - 1) // shard == o for o, a, e in b), "a bucket crosses its owner's shard"
    assert [a for _, a, _ in b] == sorted((a for _, a, _ in b), reverse=True), "buckets are listed from the end"
    # a parameter spanning two buckets completes both; a second accumulation (tied weight) is awaited
    slots = [(1, 0, 300), (2, 300, n - 300)]
    t = BucketTracker(b, slots)
    t.notify(2); t.notify(1); t.notify(1)
    assert sorted(t.finish()) == list(range(len(b)))          # first step: learning, everything runs after backward
    t.begin()
    first = t.notify(2)
    assert first and all(i not in first for i in t.of_param[1]), "buckets fed by parameter 1 must wait for it"
    assert t.notify(1) == []                                   # parameter 1 accumulates twice per backward
    rest = t.notify(1)
    assert sorted(first + rest) == list(range(len(b))) and t.finish() == []


def test_experts_only_recompute_keeps_loss_and_gradients_with_router_losses():
    """Re-running only the expert layers in backward changes neither the loss nor any gradient,
    the router's auxiliary and z losses included."""
    from brain_b200.models.config import MoeConfig
    from brain_b200.models.moe import MoeModel
    cfg = MoeConfig(vocab=64, block_size=16, n_layers=2, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, n_experts=4,
                    top_k=2, d_ff=16, aux_coef=0.01, z_coef=0.001, tie_embeddings=True)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, 64, (2, 16), generator=g, dtype=torch.int32)
    tgts = torch.randint(0, 64, (2, 16), generator=g)
    out = {}
    for mode in ("none", "experts"):
        m = MoeModel(cfg).init_weights(11)
        m.recompute_experts = mode == "experts"
        loss = m.loss(toks, tgts)
        loss.backward()
        out[mode] = (float(loss), {n: p.grad.clone() for n, p in m.named_parameters()})
    assert out["none"][0] == out["experts"][0]
    for n, gref in out["none"][1].items():
        assert torch.equal(out["experts"][1][n], gref), n


def test_native_cpu_adamw_and_norm_match_the_pytorch_expression(monkeypatch):
    """The CPU backend's one-pass native AdamW (with clipping and a no-decay run) tracks the PyTorch
    fp32 expression, and its gradient norm does not depend on the thread count."""
    from brain_b200 import _host
    from brain_b200.models.config import GptConfig
    from brain_b200.models.gpt2 import Gpt2
    from brain_b200.optim.adamw import AdamW
    from brain_b200.paramstore import ParamStore
    cfg = GptConfig(vocab=64, block_size=16, n_layers=2, d_model=32, n_heads=4, d_ff=64)
    out = {}
    for mode in ("native", "torch"):
        monkeypatch.setenv("BRAIN_CPU_ADAM", mode)
        st = ParamStore(Gpt2(cfg).init_weights(3), device="cpu")
        opt = AdamW(st, betas=(0.9, 0.95))
        g = torch.Generator().manual_seed(1)
        for _ in range(3):
            st.grads.copy_(torch.randn(st.grads.shape, generator=g) * 0.3)
            opt.step(1e-2, 0.1, clip=1.0, extra_scale=0.5)
        out[mode] = (st.weights.clone(), opt.m.clone(), opt.v.clone(), float(opt.last_grad_norm))
    for a, b in zip(out["native"][:3], out["torch"][:3]):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-7)
    assert out["native"][3] == pytest.approx(out["torch"][3], rel=1e-6)
    x = torch.randn(1_000_003, generator=torch.Generator().manual_seed(2))
    ss = [_host.lib().bbh_sumsq_f32(x.data_ptr(), x.numel(), t) for t in (1, 3, 8)]
    assert ss[0] == ss[1] == ss[2] and ss[0] == pytest.approx(float((x.double() ** 2).sum()), rel=1e-12)


def test_host_all_reduce_in_place_gives_every_rank_the_same_bits():
    """Thread ranks: each rank sums its slice of every rank's buffer in rank order and writes it
    back into all of them; odd lengths and three ranks included."""
    import threading
    from brain_b200.parallel.collective import HostCollective
    for world, n in ((2, 1000), (3, 70001), (4, 17)):
        coll = HostCollective.group(world)
        g = torch.Generator().manual_seed(world)
        bufs = [torch.randn(n, generator=g) for _ in range(world)]
        want = bufs[0].clone()
        for b in bufs[1:]:
            want = want + b
        ths = [threading.Thread(target=lambda r=r: coll[r].all_reduce(bufs[r])) for r in range(world)]
        [t.start() for t in ths]
        [t.join() for t in ths]
        for b in bufs:
            assert torch.equal(b, want)
