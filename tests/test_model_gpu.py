"""Qwen3 on the native kernels vs the same model on the fp32 CPU reference path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_qwen3_loss_and_grads_match_cpu_reference():
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.ops import _cuda
    from brain_b200.paramstore import ParamStore

    cfg = QwenConfig(vocab=512, block_size=256, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2,
                     head_dim=64, d_ff=384)
    torch.manual_seed(0)
    ref_model = Qwen3(cfg).init_weights(seed=3)
    gpu_model = Qwen3(cfg)
    gpu_model.load_state_dict(ref_model.state_dict())
    # bf16-round the reference weights so both sides start from identical values
    with torch.no_grad():
        for p in ref_model.parameters():
            p.copy_(p.bfloat16().float())
    store = ParamStore(gpu_model, device="cuda:0")
    ids = torch.randint(0, cfg.vocab, (2, 257))
    tok, tgt = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    tgt[0, :5] = -1
    loss_ref = ref_model.loss(tok, tgt)
    loss_ref.backward()
    loss = gpu_model.loss(tok.cuda(), tgt.cuda())
    loss.backward()
    _cuda.check_error()
    assert abs(loss.item() - loss_ref.item()) < 2e-2 * abs(loss_ref.item())
    worst = 0.0
    for (n, p), (_, q) in zip(ref_model.named_parameters(), gpu_model.named_parameters()):
        g = q.main_grad.float().cpu()
        e = ((g - p.grad).norm() / p.grad.norm().clamp_min(1e-8)).item()
        worst = max(worst, e)
        assert e < 8e-2, (n, e)
    assert store.grads.abs().sum() > 0


def test_smoke_entry():
    import __graft_entry__ as ge
    ge.smoke()
