"""Upstream parity (the reference compares with goldens dumped from Hugging Face transformers,
crates/qwen3/tests/parity.rs): a randomly initialised tiny transformers Qwen3 / Qwen2 model is saved
as a Hugging Face directory, imported with the framework's importer, and both sides must produce
the same logits; the export writes a directory transformers loads back to the same logits."""
import json
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _hf_model(tmp, kind):
    torch.manual_seed(0)
    common = dict(vocab_size=97, hidden_size=64, intermediate_size=160, num_hidden_layers=3,
                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                  rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=(kind == "tied"),
                  attention_dropout=0.0)
    if kind == "qwen2":
        cfg = transformers.Qwen2Config(**common)
        m = transformers.Qwen2ForCausalLM(cfg)
    else:
        cfg = transformers.Qwen3Config(head_dim=32, **common)      # head_dim != hidden / heads on purpose
        m = transformers.Qwen3ForCausalLM(cfg)
    m = m.float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() == 1:                 # norm gains (and Qwen2's biases): not all ones / zeros
                p.add_(0.1 * torch.randn_like(p))
    d = os.path.join(tmp, kind)
    m.save_pretrained(d, safe_serialization=True)
    return m, d


@pytest.mark.parametrize("kind", ["qwen3", "tied", "qwen2"])
def test_imported_checkpoint_matches_transformers_logits(tmp_path, kind):
    from brain_b200.checkpoint import st
    from brain_b200.checkpoint.hf_import import export_hf, import_qwen
    hf, d = _hf_model(str(tmp_path), kind)
    out = str(tmp_path / f"{kind}.safetensors")
    import_qwen(d, out, block=64)
    model, cfg, _ = st.load_model(out)
    model = model.float().eval()
    ids = torch.randint(0, 97, (2, 37), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids).logits
        got = model(ids.to(torch.int32)).float()
    assert got.shape == want.shape
    err = (got - want).abs().max().item()
    assert err < 2e-4 * max(want.abs().max().item(), 1.0), err
    assert (got.argmax(-1) == want.argmax(-1)).all()
    # and back: the exported directory loads in transformers with the same logits
    back = str(tmp_path / f"{kind}_export")
    export_hf(out, back, dtype="F32")
    assert json.load(open(os.path.join(back, "config.json")))["num_hidden_layers"] == 3
    cls = transformers.Qwen2ForCausalLM if kind == "qwen2" else transformers.Qwen3ForCausalLM
    hf2 = cls.from_pretrained(back, torch_dtype=torch.float32).eval()
    with torch.no_grad():
        again = hf2(ids).logits
    assert (again - want).abs().max().item() < 1e-5


def test_gpt2_block_semantics_match_transformers(tmp_path):
    """The GPT-2 model computes what transformers' GPT2LMHeadModel computes (pre-LN blocks, fused
    qkv with bias, tanh GELU, learned positions, final LayerNorm) once the weights are mapped:
    transformers stores its projections transposed (Conv1D) and ties the head to the embedding."""
    from brain_b200.models.config import GptConfig
    from brain_b200.models.gpt2 import Gpt2
    torch.manual_seed(0)
    hc = transformers.GPT2Config(vocab_size=83, n_positions=48, n_embd=48, n_layer=2, n_head=4, n_inner=None,
                                 resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    hf = transformers.GPT2LMHeadModel(hc).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))      # biases and LayerNorm parameters away from 0 / 1
    m = Gpt2(GptConfig(vocab=83, block_size=48, n_layers=2, d_model=48, n_heads=4, d_ff=192)).init_weights(1)
    sd = hf.state_dict()
    with torch.no_grad():
        m.tok.copy_(sd["transformer.wte.weight"])
        m.pos.copy_(sd["transformer.wpe.weight"])
        m.lm_head.copy_(sd["transformer.wte.weight"])
        m.ln_w.copy_(sd["transformer.ln_f.weight"])
        m.ln_b.copy_(sd["transformer.ln_f.bias"])
        for i, b in enumerate(m.blocks):
            h = f"transformer.h.{i}."
            b.ln1_w.copy_(sd[h + "ln_1.weight"]); b.ln1_b.copy_(sd[h + "ln_1.bias"])
            b.ln2_w.copy_(sd[h + "ln_2.weight"]); b.ln2_b.copy_(sd[h + "ln_2.bias"])
            b.qkv_w.copy_(sd[h + "attn.c_attn.weight"].t()); b.qkv_b.copy_(sd[h + "attn.c_attn.bias"])
            b.out_w.copy_(sd[h + "attn.c_proj.weight"].t()); b.out_b.copy_(sd[h + "attn.c_proj.bias"])
            b.fc_w.copy_(sd[h + "mlp.c_fc.weight"].t()); b.fc_b.copy_(sd[h + "mlp.c_fc.bias"])
            b.proj_w.copy_(sd[h + "mlp.c_proj.weight"].t()); b.proj_b.copy_(sd[h + "mlp.c_proj.bias"])
    ids = torch.randint(0, 83, (2, 29), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = hf(ids).logits
        got = m.eval()(ids.to(torch.int32)).float()
    assert (got - want).abs().max().item() < 2e-4 * max(want.abs().max().item(), 1.0)


def _hf_bpe(kind, corpus):
    from tokenizers import Regex, Tokenizer, decoders, models, normalizers, pre_tokenizers, trainers
    from brain_b200.data.tokenizer import QWEN_SPLIT
    tok = Tokenizer(models.BPE())
    if kind == "qwen":
        tok.normalizer = normalizers.NFC()
        tok.pre_tokenizer = pre_tokenizers.Sequence([
            pre_tokenizers.Split(Regex(QWEN_SPLIT), behavior="isolated", invert=False),
            pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
        special = ["<|endoftext|>", "<|im_start|>", "<|im_end|>"]
    else:
        tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
        special = ["<|endoftext|>"]
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=600, special_tokens=[], show_progress=False,
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    tok.add_special_tokens(special)
    if kind == "qwen":
        tok.add_tokens(["<think>", "</think>"])       # added, matched whole, but not control tokens
    return tok


@pytest.mark.parametrize("kind", ["qwen", "gpt2"])
def test_bpe_tokenizer_matches_the_tokenizers_library(tmp_path, kind):
    """A byte-level BPE trained with the Hugging Face `tokenizers` library (Qwen-style: NFC + split
    regex + byte mapping; GPT-2 style: ByteLevel with its own regex) and saved as tokenizer.json
    encodes and decodes identically through the native merge loop."""
    pytest.importorskip("tokenizers")
    import random
    from brain_b200.data.tokenizer import BpeTokenizer
    corpus = ["The quick brown fox jumps over the lazy dog. " * 3,
              "Hello, world! I'm here; you're there — it's 12345 o'clock.",
              "def f(x):\n    return x**2 + 1\n\n\nprint(f(3))\r\n",
              "naïve café résumé Ångström 日本語のテキスト 한국어 \U0001f642\U0001f680",
              "  leading spaces and   multiple   spaces\t\ttabs \n trailing  ",
              "numbers 3.14159 1,000,000 0x1F 2024-01-01", "I'LL WE'VE DON'T they'D"] * 4
    hf = _hf_bpe(kind, corpus)
    path = str(tmp_path / "tokenizer.json")
    hf.save(path)
    mine = BpeTokenizer.from_file(path)
    cases = corpus[:7] + ["<|im_start|>user\nhi there<|im_end|>\n<|im_start|>assistant\n", "é vs é", "", " ",
                          "\n\n", "a" * 50, "tab\tsep", "mixed123abc456", "'s 'S 't", "x  \n  y", "end<|endoftext|>"]
    rnd = random.Random(5)
    alphabet = "abc XYZ 019 .,!?'\n\t\r-_/éü中文́\U0001f600"
    cases += ["".join(rnd.choice(alphabet) for _ in range(rnd.randint(1, 60))) for _ in range(200)]
    cases.append("<|im_start|>assistant\n<think>\nhm</think>\n\nyes<|im_end|>")
    for s in cases:
        want = hf.encode(s).ids
        got = mine.encode(s)
        assert got == want, repr(s)
        assert mine.decode(got) == hf.decode(want, skip_special_tokens=False), repr(s)
        # control tokens are dropped, added non-special tokens (the reasoning markers) stay
        assert mine.decode(got, skip_special=True) == hf.decode(want, skip_special_tokens=True), repr(s)


CHATML_TEMPLATE = """{%- if tools %}
{{- '<|im_start|>system\\n' }}
{%- if messages[0].role == 'system' %}{{- messages[0].content + '\\n\\n' }}{%- endif %}
{{- "# Tools\\n<tools>" }}
{%- for tool in tools %}
{{- "\\n" }}{{- tool | tojson }}
{%- endfor %}
{{- "\\n</tools><|im_end|>\\n" }}
{%- else %}
{%- if messages[0].role == 'system' %}{{- '<|im_start|>system\\n' + messages[0].content + '<|im_end|>\\n' }}{%- endif %}
{%- endif %}
{%- for message in messages %}
{%- if message.role == 'user' or (message.role == 'system' and not loop.first) %}
{{- '<|im_start|>' + message.role + '\\n' + message.content + '<|im_end|>' + '\\n' }}
{%- elif message.role == 'assistant' %}
{{- '<|im_start|>assistant\\n' + message.content }}
{%- if message.tool_calls %}
{%- for tc in message.tool_calls %}
{{- '\\n<tool_call>\\n{"name": "' + tc.function.name + '", "arguments": ' }}{{- tc.function.arguments | tojson }}{{- '}\\n</tool_call>' }}
{%- endfor %}
{%- endif %}
{{- '<|im_end|>\\n' }}
{%- elif message.role == 'tool' %}
{{- '<|im_start|>user\\n<tool_response>\\n' + message.content + '\\n</tool_response><|im_end|>\\n' }}
{%- elif message.role == 'system' %}
{%- else %}
{{- raise_exception('unknown role ' + message.role) }}
{%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
{{- '<|im_start|>assistant\\n' }}
{%- if enable_thinking is defined and enable_thinking is false %}{{- '<think>\\n\\n</think>\\n\\n' }}{%- endif %}
{%- endif %}"""


def test_chat_template_renders_like_transformers(tmp_path):
    """The checkpoint's own Jinja chat template renders to the same text as transformers'
    `apply_chat_template`: whitespace control, the `tojson` filter on non-ASCII text, tool lists, tool
    calls, extra template variables and `raise_exception`."""
    pytest.importorskip("tokenizers")
    from brain_b200.data.chat_template import ChatTemplate, TemplateError
    hf_tok = transformers.PreTrainedTokenizerFast(tokenizer_object=_hf_bpe("qwen", ["hello world"] * 4),
                                                  eos_token="<|im_end|>")
    hf_tok.chat_template = CHATML_TEMPLATE
    mine = ChatTemplate(CHATML_TEMPLATE, eos_token="<|im_end|>")
    tools = [{"type": "function", "function": {"name": "väder", "description": "Weather — per city",
                                               "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]
    convs = [
        ([{"role": "user", "content": "hi"}], None, {}),
        ([{"role": "system", "content": "Be brief."}, {"role": "user", "content": "hi"},
          {"role": "assistant", "content": "hello"}, {"role": "user", "content": "again\n\nplease "}], None, {}),
        ([{"role": "system", "content": "S"}, {"role": "user", "content": "weather in Malmö?"},
          {"role": "assistant", "content": "", "tool_calls": [
              {"type": "function", "function": {"name": "väder", "arguments": {"city": "Malmö", "n": 2}}}]},
          {"role": "tool", "content": "{\"temp\": 7}"}], tools, {}),
        ([{"role": "user", "content": "no thinking"}], None, {"enable_thinking": False}),
    ]
    for msgs, tl, extra in convs:
        for gen in (True, False):
            want = hf_tok.apply_chat_template(msgs, tools=tl, tokenize=False, add_generation_prompt=gen, **extra)
            got = mine.render(msgs, add_generation_prompt=gen, tools=tl, **extra)
            assert got == want
    with pytest.raises(TemplateError):
        mine.render([{"role": "narrator", "content": "x"}])


@pytest.mark.parametrize("layout", ["fused", "per_expert"])
def test_qwen3_moe_import_matches_transformers_logits(tmp_path, layout):
    """A tiny random transformers Qwen3-MoE (top-2 of 8 experts, gate weights renormalised in one case and raw in the other) imported
    from its Hugging Face directory gives the same logits; both expert layouts are read: the fused
    [E, 2*ff, d] tensors transformers 5 writes and the per-expert tensors of published checkpoints."""
    from safetensors.torch import load_file, save_file
    from brain_b200.checkpoint import st
    from brain_b200.checkpoint.hf_import import import_hf
    torch.manual_seed(0)
    hc = transformers.Qwen3MoeConfig(
        vocab_size=97, hidden_size=64, intermediate_size=160, moe_intermediate_size=48, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=8, num_experts_per_tok=2,
        norm_topk_prob=(layout == "fused"), decoder_sparse_step=1, mlp_only_layers=[], rope_theta=10000.0,
        max_position_embeddings=128, tie_word_embeddings=False)
    hf = transformers.Qwen3MoeForCausalLM(hc).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            if "experts" in n or "gate.weight" in n:
                p.normal_(0, 0.2)          # routing far from ties, experts that matter
    d = str(tmp_path / "hf")
    hf.save_pretrained(d, safe_serialization=True)
    if layout == "per_expert":
        path = os.path.join(d, "model.safetensors")
        sd = load_file(path)
        if any(k.endswith("experts.gate_up_proj") for k in sd):
            new = {}
            for k, v in sd.items():
                if k.endswith("experts.gate_up_proj"):
                    base = k[: -len("gate_up_proj")]
                    for e in range(v.shape[0]):
                        new[f"{base}{e}.gate_proj.weight"] = v[e, :48].contiguous()
                        new[f"{base}{e}.up_proj.weight"] = v[e, 48:].contiguous()
                elif k.endswith("experts.down_proj"):
                    base = k[: -len("down_proj")]
                    for e in range(v.shape[0]):
                        new[f"{base}{e}.down_proj.weight"] = v[e].contiguous()
                else:
                    new[k] = v
            save_file(new, path, metadata={"format": "pt"})
    out = str(tmp_path / "moe.safetensors")
    cfg = import_hf(d, out, block=64)
    assert cfg.n_experts == 8 and cfg.top_k == 2 and cfg.d_ff == 48 and cfg.rope_theta == 10000.0
    model, _, card = st.load_model(out)
    model = model.float().eval()
    ids = torch.randint(0, 97, (2, 23), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = hf(ids).logits
        got = model(ids.to(torch.int32)).float()
    assert (got - want).abs().max().item() < 2e-4 * max(want.abs().max().item(), 1.0)


def test_trainer_steps_match_a_plain_pytorch_loop():
    """Five optimiser steps of the framework trainer (flat parameter store, own AdamW, global-norm
    clip, micro-batched gradient accumulation) land on the same weights and losses as the textbook
    loop: F.cross_entropy mean over counted targets, clip_grad_norm_, torch.optim.AdamW with
    decoupled weight decay on every tensor."""
    import copy
    from brain_b200.engine import Trainer
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    cfg = QwenConfig(vocab=53, block_size=16, n_layers=2, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=48)
    a = Qwen3(cfg).init_weights(5)
    b = copy.deepcopy(a)
    tr = Trainer(a, device="cpu", betas=(0.9, 0.999), weight_decay=0.1, grad_clip=0.5)
    opt = torch.optim.AdamW(b.parameters(), lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    g = torch.Generator().manual_seed(3)
    for step in range(5):
        x = torch.randint(0, 53, (4, 16), generator=g)
        y = torch.randint(0, 53, (4, 16), generator=g)
        y[0, :5] = -1                                          # masked positions are not counted
        lr = 1e-2 * (step + 1) / 5
        la = float(tr.train_step(x, y, lr, micro_batch=2))      # two micro-batches, one update
        for pg in opt.param_groups:
            pg["lr"] = lr
        opt.zero_grad()
        logits = b(x.to(torch.int32)).float()
        lb = torch.nn.functional.cross_entropy(logits.reshape(-1, 53), y.reshape(-1), ignore_index=-1)
        lb.backward()
        torch.nn.utils.clip_grad_norm_(b.parameters(), 0.5)
        opt.step()
        assert la == pytest.approx(float(lb), rel=2e-5, abs=2e-5)
    for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.allclose(pa.detach().float(), pb.detach().float(), rtol=2e-4, atol=2e-5), n


def test_engine_greedy_tokens_match_transformers_generate(tmp_path):
    """End to end: transformers model -> Hugging Face directory -> importer -> paged-KV engine and
    scheduler (chunked prefill, batched decode, mixed steps) produce the greedy continuation that
    `generate(do_sample=False)` produces."""
    from brain_b200.checkpoint import st
    from brain_b200.checkpoint.hf_import import import_hf
    from brain_b200.serve.engine import QwenEngine
    from brain_b200.serve.scheduler import Scheduler
    hf, d = _hf_model(str(tmp_path), "qwen3")
    with torch.no_grad():
        for p in hf.parameters():
            p.mul_(3.0)                      # well separated logits: greedy choices survive rounding
    hf.save_pretrained(d, safe_serialization=True)
    out = str(tmp_path / "m.safetensors")
    import_hf(d, out, block=64)
    model, _, _ = st.load_model(out)
    eng = QwenEngine(model.float().eval(), block_size=4, num_blocks=64, max_seq_len=64, max_prefill=8)
    sched = Scheduler(eng, max_batch=3, window=2, mixed=True)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (5, 19, 11, 3)]
    ids = [sched.submit(p, 9) for p in prompts]
    sched.run_until_idle()
    for p, r in zip(prompts, ids):
        with torch.no_grad():
            ii = torch.tensor([p])       # explicit mask: a prompt may contain the id used for padding
            want = hf.generate(ii, attention_mask=torch.ones_like(ii), max_new_tokens=9, do_sample=False,
                               pad_token_id=0, eos_token_id=None)[0, len(p):].tolist()
        assert sched.tokens_of(r) == want


def test_rng_is_splitmix64_offset_by_one_step():
    """The dataset generator is SplitMix64 whose state starts one increment past the seed
    (crates/data/src/rng.rs:20-35): seed 0 yields the published SplitMix64 test vector from its
    second value on, and the float helpers use the top 53 bits."""
    from brain_b200.data.rng import Rng
    published = [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F, 0xF88BB8A8724C81EC]
    r = Rng(0)
    assert [r.next_u64() for _ in range(3)] == published[1:]
    r = Rng(0)
    assert r.next_f64() == (published[1] >> 11) / float(1 << 53)
    r = Rng(0)
    assert r.gen_range_inclusive(3, 12) == 3 + published[1] % 10
    assert Rng(2**64 - 1).next_u64() == Rng(-1 & (2**64 - 1)).next_u64()      # wrapping seed arithmetic


def test_sharded_bf16_directory_imports(tmp_path):
    """The layout of published checkpoints: bf16 tensors spread over several shard files behind
    model.safetensors.index.json, tied head absent from the files."""
    from brain_b200.checkpoint import st
    from brain_b200.checkpoint.hf_import import import_hf
    hf, _ = _hf_model(str(tmp_path), "tied")
    hf = hf.to(torch.bfloat16)
    d = str(tmp_path / "sharded")
    hf.save_pretrained(d, safe_serialization=True, max_shard_size="60KB")
    assert os.path.exists(os.path.join(d, "model.safetensors.index.json"))
    assert len([f for f in os.listdir(d) if f.endswith(".safetensors")]) > 2
    out = str(tmp_path / "m.safetensors")
    import_hf(d, out, block=64, dtype="BF16")
    model, cfg, _ = st.load_model(out)
    assert cfg["tie_word_embeddings"] is True
    ids = torch.randint(0, 97, (1, 17), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf.float()(ids).logits
        got = model.float()(ids.to(torch.int32)).float()
    assert (got - want).abs().max().item() < 2e-3


def test_rope_base_is_read_from_either_config_generation():
    from brain_b200.checkpoint.hf_import import config_from_hf
    base = {"hidden_size": 64, "num_attention_heads": 4, "num_hidden_layers": 1, "intermediate_size": 96,
            "vocab_size": 50, "model_type": "qwen3"}
    assert config_from_hf(dict(base, rope_theta=5e5)).rope_theta == 5e5
    assert config_from_hf(dict(base, rope_parameters={"rope_theta": 1e4, "rope_type": "default"})).rope_theta == 1e4
    assert config_from_hf(dict(base, rope_theta=1e6, rope_scaling=None)).rope_theta == 1e6
    assert config_from_hf(base).rope_theta == 1e6
    with pytest.raises(ValueError, match="yarn"):
        config_from_hf(dict(base, rope_theta=1e6, rope_scaling={"type": "yarn", "factor": 4.0}))


def test_user_journey_import_store_serve_chat_matches_transformers(tmp_path):
    """The whole path a user takes, with real processes: a Hugging Face directory (weights,
    tokenizer.json, chat template) -> `brain qwen3 import --id` into the model store -> `brain serve
    --stdio` selected by BRAIN_MODEL -> a chat turn through brain_py.  The reply equals what
    transformers produces from the same directory (template, tokenizer, greedy generate)."""
    pytest.importorskip("tokenizers")
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from brain_py import Brain
    corpus = ["hello world, how are you today? fine thanks. " * 5, "the capital of sweden is stockholm. " * 5] * 4
    tok = _hf_bpe("qwen", corpus)
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(vocab_size=tok.get_vocab_size(), hidden_size=64, intermediate_size=160,
                                   num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                   max_position_embeddings=256, rope_theta=10000.0, tie_word_embeddings=True)
    hf = transformers.Qwen3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.mul_(3.0)
    d = str(tmp_path / "hf")
    hf.save_pretrained(d, safe_serialization=True)
    tok.save(os.path.join(d, "tokenizer.json"))
    with open(os.path.join(d, "tokenizer_config.json"), "w") as f:
        json.dump({"chat_template": CHATML_TEMPLATE, "eos_token": "<|im_end|>"}, f)
    store = str(tmp_path / "store")
    env = dict(os.environ, PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    brain = os.path.join(root, "brain")
    r = subprocess.run([sys.executable, brain, "qwen3", "import", d, "--id", "Acme/Tiny-Qwen3", "--models-dir", store,
                        "--block", "128"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "hello world"}]
    hf_tok = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<|im_end|>")
    hf_tok.chat_template = CHATML_TEMPLATE
    ids = hf_tok.apply_chat_template(msgs, add_generation_prompt=True, tokenize=True, return_tensors="pt")
    ids = ids["input_ids"] if not isinstance(ids, torch.Tensor) else ids
    with torch.no_grad():
        gen = hf.generate(ids, attention_mask=torch.ones_like(ids), max_new_tokens=10, do_sample=False,
                          pad_token_id=0, eos_token_id=None)[0, ids.shape[1]:]
    env2 = dict(env, BRAIN_MODEL="Acme/Tiny-Qwen3", BRAIN_MODELS_DIR=store, BRAIN_QWEN_CTX="128")
    with Brain(transport="jsonl", brain_bin=brain, env=env2) as b:
        assert b.models() == ["Acme/Tiny-Qwen3"]
        out = b.generate(messages=msgs, model="Acme/Tiny-Qwen3", max_new=10, temp=0.0, ignore_eos=True)
    assert out.get("prompt_tokens") == ids.shape[1]
    assert out.get("completion_tokens") == 10
    assert out.text() == hf_tok.decode(gen, skip_special_tokens=True)
