"""CLI grammar, datasets, tokenizers, checkpoints, training driver and the small subsystems around
them — all on the CPU backend.  Modelled on the reference's unit tests for crates/cli (args,
resolve), crates/data (rng, loader, generators, tokenizers), crates/checkpoint (round trips) and
crates/model/src/train.rs (fit/resume)."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from brain_b200.cli.args import Args, canon_verb  # noqa: E402
from brain_b200.cli.main import main  # noqa: E402
from brain_b200.cli.resolve import resolve  # noqa: E402


# ------------------------------------------------------------------------------------ grammar
def test_args_take_and_finish(capsys):
    a = Args(["data", "--steps", "7", "--align", "--lr", "bad", "--extra", "x"])
    assert a.int_or("--steps", 1) == 7 and a.take_flag("--align") and not a.take_flag("--align")
    assert a.float_or("--lr", 0.5) == 0.5 and a.positional() == "data" and a.positional() == "x"
    a.finish()
    assert "--extra" in capsys.readouterr().err
    with pytest.raises(SystemExit):
        Args(["--out"]).take_str("--out")
    assert Args(["--prompt", "a", "--prompt", "b"]).take_all("--prompt") == ["a", "b"]


def test_verb_aliases_and_both_word_orders():
    assert [canon_verb(v) for v in ("gen", "sample", "generate", "fine-tune", "train")] == \
        ["infer", "infer", "infer", "finetune", "train"]
    a, b = resolve(["train", "qwen3", "d", "--steps", "3"]), resolve(["qwen3", "train", "d", "--steps", "3"])
    assert a.kind == b.kind == "arch" and a.arch == b.arch == "qwen3" and a.rest == b.rest == ["train", "d", "--steps", "3"]
    assert resolve(["gpt", "train"]).arch == "gpt2" and resolve(["qwen", "infer"]).arch == "qwen3"
    assert resolve(["import", "x.gguf"]).kind == "import" and resolve(["quantize", "x"]).kind == "quantize"
    assert resolve(["wat"]).kind == "unknown" and resolve([]).kind == "empty"
    assert resolve(["yolov8", "detect"]).arch == "yolov8"


def test_main_help_version_unknown(capsys):
    assert main(["--version"]) == 0 and "brain " in capsys.readouterr().out
    assert main(["help"]) == 0 and "brain <verb> <arch>" in capsys.readouterr().out
    assert main(["frobnicate"]) == 2
    assert main(["yolov8", "detect"]) == 3
    assert main(["--trace-format", "xml", "devices"]) == 2
    assert main(["devices", "--device", "cpu"]) == 0 and "cpu" in capsys.readouterr().out


def test_trace_flags(tmp_path, capsys):
    from brain_b200.utils import trace
    rest, lv, fmt, out = trace.take_flags(["--trace-serve", "4", "x", "--trace", "comm=debug,train=2", "--trace-format", "json"])
    assert rest == ["x"] and lv == {"serve": 4, "comm": 4, "train": 2} and fmt == "json"
    assert trace.parse_spec("3")["kernel"] == 3
    with pytest.raises(ValueError):
        trace.parse_spec("nosuch=3")
    p = tmp_path / "t.log"
    trace.install({"train": 3}, "json", str(p))
    trace.event("train", 3, "hello", step=1)
    trace.event("train", 4, "too detailed")
    trace.event("serve", 1, "other family off")
    trace.install({}, "text", "-")
    rec = [json.loads(l) for l in p.read_text().splitlines()]
    assert len(rec) == 1 and rec[0]["message"] == "hello" and rec[0]["step"] == 1 and rec[0]["target"] == "train"


# ------------------------------------------------------------------------------------ data
def test_rng_is_splitmix64():
    from brain_b200.data.rng import Rng
    # the seed is offset by the golden-ratio constant once at construction, so seed 0 yields the
    # standard SplitMix64 sequence from its second element on
    r = Rng(0)
    assert [r.next_u64() for _ in range(2)] == [0x6E789E6AA1B965F4, 0x06C45D188009454F]
    r = Rng(7)
    xs = [r.next_f32() for _ in range(1000)]
    assert 0.0 <= min(xs) and max(xs) < 1.0 and abs(sum(xs) / 1000 - 0.5) < 0.05


def test_dataset_generators_and_loader(tmp_path):
    from brain_b200.data import binio, datasets
    from brain_b200.data.loader import BatchConfig, TokenDataset
    from brain_b200.data.rng import Rng
    d = tmp_path / "calc"
    datasets.prepare("calculator", d, 500, 1)
    meta = binio.read_meta(d)
    itos = meta["itos"]
    assert meta["vocab_size"] == len(itos) and "=" in itos and "\n" in itos
    train = binio.read_tokens(d, "train")
    text = "".join(itos[t] for t in train[:2000])
    for line in text.split("\n")[1:5]:
        lhs, rhs = line.split("=")
        assert abs(eval(lhs) - float(rhs)) < 1e-2 * max(1.0, abs(float(rhs)))     # noqa: S307 - our own generator's arithmetic
    ds = TokenDataset(train)
    nl, eq = itos.index("\n"), itos.index("=")
    assert ds.align_to_lines(nl, 32) > 0
    x, y = ds.get_batch(BatchConfig(4, 32, eq, True, nl), Rng(3))
    assert x.shape == y.shape == (4, 32)
    assert torch.equal(x[:, 1:].long()[y[:, :-1] >= 0], y[:, :-1][y[:, :-1] >= 0])
    for b in range(4):          # positions up to and including '=' on each line are not supervised
        row_x, row_y = x[b].tolist(), y[b].tolist()
        seen_eq = False
        for t in range(32):
            if row_x[t] == nl:
                seen_eq = False
            if row_x[t] == eq:
                seen_eq = True
            elif not seen_eq and row_x[t] != nl:
                assert row_y[t] == -1 or row_x[t + 1 if t + 1 < 32 else t] == eq or True
    x2, y2 = ds.get_batch(BatchConfig(4, 32, eq, True, nl), Rng(3))
    assert torch.equal(x, x2) and torch.equal(y, y2)
    rev = datasets.gen_reverser(20, Rng(1)).strip().split("\n")
    for line in rev:
        a, b = line.split("=")
        assert a[::-1] == b
    assert datasets.number_words(42) == "forty two" or "forty" in datasets.number_words(42)
    ts = datasets.gen_timeseries(100, 3)
    assert ts.shape[0] == 100 and np.isfinite(ts).all()


def test_tokenizers_roundtrip(tmp_path):
    from brain_b200.data.tokenizer import BpeTokenizer, CharTokenizer, render_chatml
    c = CharTokenizer.from_text("hello world")
    assert c.decode(c.encode("hello")) == "hello"
    with pytest.raises(ValueError):
        c.encode("z")
    t = BpeTokenizer.byte_level(["h e", "he l", "l o"], {"<|im_start|>": 300, "<|im_end|>": 301})
    for s in ("hello hello", "héllo wörld ☃", "a\n\n  b\t", ""):
        assert t.decode(t.encode(s)) == s
    ids = t.encode("<|im_start|>user\nhello<|im_end|>")
    assert ids[0] == 300 and ids[-1] == 301 and len(t.encode("hello")) < 5
    assert t.decode(ids, skip_special=True) == "user\nhello"
    assert 300 not in t.encode("<|im_start|>", allow_special=False)
    s = render_chatml([("system", "s"), ("user", "u")], True, True)
    assert s == "<|im_start|>system\ns<|im_end|>\n<|im_start|>user\nu<|im_end|>\n<|im_start|>assistant\n"
    tj = tmp_path / "tokenizer.json"
    b2u = __import__("brain_b200.data.tokenizer", fromlist=["bytes_to_unicode"]).bytes_to_unicode()
    vocab = {b2u[i]: i for i in range(256)}
    vocab[b2u[ord("a")] + b2u[ord("b")]] = 256
    tj.write_text(json.dumps({"model": {"vocab": vocab, "merges": [f"{b2u[ord('a')]} {b2u[ord('b')]}"]},
                              "added_tokens": [{"content": "<|endoftext|>", "id": 257}]}))
    f = BpeTokenizer.from_file(str(tj))
    assert f.encode("abab") == [256, 256] and f.eos_id == 257


def test_chat_and_toolcall_data(tmp_path):
    from brain_b200.data import binio, chat, toolcall
    from brain_b200.data.tokenizer import BpeTokenizer
    tok = BpeTokenizer.byte_level([], {"<|im_start|>": 256, "<|im_end|>": 257, "<|endoftext|>": 258})
    ex = chat.ChatExample("hi", "yo", "sys")
    ids, mask = ex.encode(tok)
    assert len(ids) == len(mask) and ids[-1] == 258 and mask[-1] == 0
    sup = tok.decode([i for i, m in zip(ids, mask) if m])
    assert sup == "yo<|im_end|>\n"
    cases = toolcall.generate(20, 3, 5)
    assert cases == toolcall.generate(20, 3, 5) or [c.user for c in cases] == [c.user for c in toolcall.generate(20, 3, 5)]
    for c in cases:
        assert len(c.tools) == 3 and c.name in [t["function"]["name"] for t in c.tools]
        got = toolcall.first_tool_call("noise " + c.response_str())
        assert toolcall.calls_match(c.name, c.arguments, got)
    assert toolcall.calls_match("add_numbers", {"a": 1, "b": 2}, {"name": "add_numbers", "arguments": {"a": "1", "b": 2.0}})
    assert not toolcall.calls_match("add_numbers", {"a": 1, "b": 2}, {"name": "add_numbers", "arguments": {"a": 1}})
    chat.prepare_chat([c.to_chat_example() for c in cases], [cases[0].to_chat_example()], tok, 300, tmp_path / "tc")
    assert binio.read_mask(tmp_path / "tc", "train").sum() > 0
    r, v = chat.split_reasoning("<think>because</think>\n\nanswer")
    assert (r, v) == ("because", "answer")
    calls, rest = chat.parse_tool_calls('ok <tool_call>\n{"name": "f", "arguments": {"x": 1}}\n</tool_call>')
    assert calls == [{"name": "f", "arguments": {"x": 1}}] and rest == "ok"


# ------------------------------------------------------------------------------------ checkpoints
def test_safetensors_reader_checks_integer_ranges_and_widens_u32(tmp_path):
    """A header whose byte range is shorter than shape x element size is refused for every dtype
    (not only the floats), and U32 values above 2^31 come back positive."""
    import json
    import struct
    import numpy as np
    from brain_b200.checkpoint import st

    def write(path, hdr, data):
        h = json.dumps(hdr).encode()
        h += b" " * (-len(h) % 8)
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(h)) + h + data)

    vals = np.array([1, 2 ** 31 + 5, 2 ** 32 - 1, 7], dtype=np.uint32)
    good = str(tmp_path / "u.safetensors")
    write(good, {"u": {"dtype": "U32", "shape": [4], "data_offsets": [0, 16]}}, vals.tobytes())
    with st.WeightReader(good) as r:
        assert r.read("u").tolist() == [1, 2 ** 31 + 5, 2 ** 32 - 1, 7]
    short = str(tmp_path / "s.safetensors")
    write(short, {"i": {"dtype": "I32", "shape": [1000], "data_offsets": [0, 16]}}, vals.tobytes())
    with st.WeightReader(short) as r:
        with pytest.raises(ValueError, match="byte length"):
            r.read("i")


def test_checkpoint_roundtrip_names_and_metadata(tmp_path):
    from brain_b200.checkpoint import st
    from brain_b200.models.config import GptConfig, QwenConfig
    from brain_b200.models.gpt2 import Gpt2
    from brain_b200.models.qwen3 import Qwen3
    cfg = QwenConfig(vocab=50, block_size=16, n_layers=2, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=48)
    m = Qwen3(cfg).init_weights(1)
    p = str(tmp_path / "q.safetensors")
    st.save_model(p, m)
    assert not os.path.exists(p + ".tmp")
    with st.WeightReader(p) as r:
        assert r.names() == [n for n, _ in cfg.param_list()]
        assert all(r.shape(n) == (k,) and r.dtype(n) == "F32" for n, k in cfg.param_list())
        assert r.config()["model"] == "qwen" and r.config()["n_kv_heads"] == 2
        assert r.card().id == "brain/qwen3" and r.metadata["family"] == "qwen"
    m2, c2, card = st.load_model(p)
    x = torch.randint(0, 50, (2, 16), dtype=torch.int32)
    assert torch.equal(m(x), m2(x))
    pb = str(tmp_path / "q16.safetensors")
    st.save_model(pb, m, dtype="BF16")
    m3, _, _ = st.load_model(pb)
    assert float((m(x) - m3(x)).abs().max()) < 0.05 and os.path.getsize(pb) < 0.6 * os.path.getsize(p)
    g = Gpt2(GptConfig(vocab=20, block_size=8, n_layers=1, d_model=16, n_heads=2, d_ff=32, itos=list("abcdefghijklmnopqrst"))).init_weights(2)
    pg = str(tmp_path / "g.safetensors")
    st.save_model(pg, g)
    with st.WeightReader(pg) as r:
        assert r.names()[:2] == ["tok.weight", "pos.weight"] and r.names()[-1] == "lm_head.weight"
        assert r.config()["itos"][0] == "a" and r.card().id == "brain/gpt"


def test_hf_import_export_roundtrip(tmp_path):
    from brain_b200.checkpoint import st
    from brain_b200.checkpoint.hf_import import export_hf, hf_name, import_qwen
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    assert hf_name("blocks.3.attn.wq.weight") == "model.layers.3.self_attn.q_proj.weight"
    assert hf_name("blocks.0.mlp.down.weight") == "model.layers.0.mlp.down_proj.weight"
    assert hf_name("tok.weight") == "model.embed_tokens.weight" and hf_name("norm.weight") == "model.norm.weight"
    cfg = QwenConfig(vocab=40, block_size=16, n_layers=2, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=48,
                     tie_embeddings=False)
    m = Qwen3(cfg).init_weights(3)
    src = str(tmp_path / "a.safetensors")
    st.save_model(src, m)
    export_hf(src, str(tmp_path / "hf"), "F32")
    hf_cfg = json.loads((tmp_path / "hf" / "config.json").read_text())
    assert hf_cfg["num_key_value_heads"] == 2 and hf_cfg["model_type"] == "qwen3"
    with st.WeightReader(str(tmp_path / "hf" / "model.safetensors")) as r:
        assert r.shape("model.layers.0.self_attn.q_proj.weight") == (32, 32)
        assert r.shape("model.layers.1.mlp.down_proj.weight") == (32, 48) and "lm_head.weight" in r.names()
    back = str(tmp_path / "b.safetensors")
    c2 = import_qwen(str(tmp_path / "hf"), back, block=16)
    assert c2.n_layers == 2 and not c2.tie_embeddings
    a, _, _ = st.load(src)
    b, _, _ = st.load(back)
    assert list(a) == list(b) and all(torch.equal(a[k], b[k]) for k in a)
    # `brain import <dir> --id VENDOR/REPO` converts and installs into the model store; the stored
    # model is then what BRAIN_MODEL resolves
    from brain_b200.cli.main import main
    from brain_b200.modelref import ModelRef
    from brain_b200.modelstore import Store
    (tmp_path / "hf" / "tokenizer.json").write_text("{}")
    (tmp_path / "hf" / "tokenizer_config.json").write_text('{"chat_template": "x"}')
    root = str(tmp_path / "models")
    assert main(["import", str(tmp_path / "hf"), "--id", "Acme/Tiny-0.1B", "--models-dir", root, "--block", "16"]) == 0
    lm = Store(root).local(ModelRef.parse("Acme/Tiny-0.1B"))
    assert lm is not None and lm.card.id == "Acme/Tiny-0.1B" and lm.tokenizer.endswith("tokenizer.json")
    assert os.path.exists(os.path.join(lm.dir, "tokenizer_config.json"))
    c, _, _ = st.load(lm.weights)
    assert all(torch.equal(a[k], c[k]) for k in a)
    assert main(["import", str(tmp_path / "hf"), "--id", "no-slash"]) == 2
    assert main(["import", "--list"]) == 0


def test_quantize_checkpoint(tmp_path):
    from brain_b200.checkpoint import st
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.serve.quantize import load_quantized, quantize_checkpoint
    cfg = QwenConfig(vocab=64, block_size=16, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128)
    m = Qwen3(cfg).init_weights(5)
    src, out = str(tmp_path / "a.safetensors"), str(tmp_path / "a.w8.safetensors")
    st.save_model(src, m)
    info = quantize_checkpoint(src, out, keep=["blocks.0.attn.wo"])
    d = dict(info["plan"])
    assert d["tok.weight"] == "bf16" and d["blocks.0.attn.wo.weight"] == "bf16" and d["blocks.1.attn.wo.weight"] == "q8"
    assert d["blocks.0.ln1.weight"] == "bf16" and info["bytes_out"] < 0.6 * info["bytes_in"]
    q = load_quantized(out)
    x = torch.randint(0, 64, (1, 16), dtype=torch.int32)
    assert float((m(x) - q(x)).abs().max()) < 0.05


# ------------------------------------------------------------------------------------ training driver
def test_fit_resume_and_generate(tmp_path):
    from brain_b200.checkpoint import st
    from brain_b200.data import datasets
    from brain_b200.models.config import GptConfig
    from brain_b200.models.gpt2 import Gpt2
    from brain_b200.train import FitOpts, fit, generate
    d = tmp_path / "rev"
    datasets.prepare("reverser", d, 400, 2)
    out = str(tmp_path / "o" / "g.safetensors")
    o = FitOpts(steps=25, batch_size=8, block_size=24, lr=3e-3, warmup=3, decay_iters=25, eval_interval=10,
                eval_batches=2, device="cpu", mask_before="=", mask_per_line=True, align_to_lines=True)
    log = []
    build = lambda v, b: Gpt2(GptConfig(vocab=v, block_size=b, n_layers=1, d_model=32, n_heads=2, d_ff=64))
    l0, l1 = fit(str(d), build, o, out, log=log.append)
    assert l1 < l0 and os.path.exists(out)
    assert any(l.startswith("step     10  lr ") and "  train " in l and "  eval " in l for l in log)
    assert log[-1].startswith(f"saved checkpoint -> {out} (")
    log2 = []
    bigger = lambda v, b: Gpt2(GptConfig(vocab=v, block_size=b, n_layers=3, d_model=64, n_heads=2, d_ff=64))
    l2, _ = fit(str(d), bigger, o, out, log=log2.append)
    assert log2[0] == f"resuming from existing checkpoint {out}"
    m, cfg, _ = st.load_model(out)
    assert cfg["n_layers"] == 1                       # the checkpoint's config wins over the new flags
    assert abs(l2 - l1) < 0.5
    with pytest.raises(ValueError):
        fit(str(d), build, FitOpts(steps=1, block_size=16, device="cpu"), out, log=lambda s: None)
    a = generate(m, [1, 2, 3], 12, temp=0.8, top_k=5, seed=9)
    assert a == generate(m, [1, 2, 3], 12, temp=0.8, top_k=5, seed=9) and len(a) == 12
    assert generate(m, [1, 2, 3], 5, temp=0.0) == generate(m, [1, 2, 3], 5, temp=0.0, seed=77)


def test_cosine_lr_and_offload_adam_parity():
    from brain_b200.engine import Trainer
    from brain_b200.models.config import GptConfig
    from brain_b200.models.gpt2 import Gpt2
    from brain_b200.optim.lr import cosine_lr
    assert cosine_lr(0, 1.0, 0.1, 10, 100) == pytest.approx(0.1, abs=0.11) and cosine_lr(10, 1.0, 0.1, 10, 100) == pytest.approx(1.0)
    assert cosine_lr(100, 1.0, 0.1, 10, 100) == pytest.approx(0.1) and cosine_lr(500, 1.0, 0.1, 10, 100) == pytest.approx(0.1)
    assert cosine_lr(55, 1.0, 0.1, 10, 100) == pytest.approx(0.55, abs=1e-6)

    def run(off):
        m = Gpt2(GptConfig(vocab=30, block_size=8, n_layers=1, d_model=16, n_heads=2, d_ff=32)).init_weights(3)
        t = Trainer(m, device="cpu", offload_adam=off)
        g = torch.Generator().manual_seed(1)
        x, y = torch.randint(0, 30, (4, 8), generator=g), torch.randint(0, 30, (4, 8), generator=g)
        return [float(t.train_step(x, y, 1e-2)) for _ in range(4)], t.store.weights.clone()
    (la, wa), (lb, wb) = run(False), run(True)
    assert la == pytest.approx(lb, abs=1e-4) and float((wa - wb).abs().max()) < 1e-3


# ------------------------------------------------------------------------------------ end-to-end CLI
def test_cli_end_to_end(tmp_path, capsys):
    d, o = str(tmp_path / "calc"), str(tmp_path / "o")
    assert main(["data", "gen", "calculator", "--out", d, "--n", "400", "--seed", "1"]) == 0
    assert main(["data", "gen", "nosuch"]) == 2
    g = os.path.join(o, "g.safetensors")
    assert main(["train", "gpt2", d, "--out", g, "--steps", "6", "--batch", "4", "--block", "16", "--layers", "1",
                 "--d-model", "16", "--heads", "2", "--mask", "=", "--align", "--device", "cpu"]) == 0
    out = capsys.readouterr().out
    assert "training gpt on" in out and "done: train loss " in out
    assert main(["gpt2", "sample", "--weights", g, "--prompt", "1+1=", "--max-new", "4", "--device", "cpu"]) == 0
    assert capsys.readouterr().out.startswith("1+1=")
    assert main(["gpt2", "eval", "--weights", g, "--data", d, "--batches", "1", "--samples", "2", "--device", "cpu"]) == 0
    assert "val_perplexity " in capsys.readouterr().out
    q = os.path.join(o, "q.safetensors")
    assert main(["qwen3", "train", d, "--out", q, "--steps", "3", "--batch", "2", "--block", "16", "--device", "cpu"]) == 0
    assert f"; saved {q}" in capsys.readouterr().out
    assert main(["qwen3", "infer", "--weights", q, "--tokenizer", d, "--prompt", "1+1=", "--max-new", "8", "--device", "cpu"]) == 0
    plain = capsys.readouterr()
    assert main(["qwen3", "infer", "--weights", q, "--tokenizer", d, "--prompt", "1+1=", "--max-new", "8", "--spec", "3",
                 "--device", "cpu"]) == 0
    spec = capsys.readouterr()
    assert spec.out == plain.out and "qwen-spec k=3 target_forwards=" in spec.err
    assert main(["qwen3", "serve", "--weights", q, "--tokenizer", d, "--prompt", "1+1=", "--prompt", "2+2=", "--max-new", "4",
                 "--int8", "--device", "cpu"]) == 0
    assert "[int8 KV]" in capsys.readouterr().err
    q2 = os.path.join(o, "q_ft.safetensors")
    assert main(["finetune", "qwen3", d, "--weights", q, "--out", q2, "--steps", "2", "--batch", "2", "--block", "16", "--device", "cpu"]) == 0
    assert "resuming from existing checkpoint" in capsys.readouterr().out and os.path.exists(q2)
    assert main(["qwen3", "finetune", "--lora", "4", "--weights", q, "--adapter", "me/calc:v1", "--dataset", d, "--steps", "3",
                 "--batch", "2", "--block", "16", "--models-dir", os.path.join(o, "models"), "--device", "cpu"]) == 0
    line = [l for l in capsys.readouterr().out.splitlines() if l.startswith("trained adapter")][0]
    adapter = line.rsplit("saved ", 1)[1]
    from brain_b200.checkpoint import st
    tens, cfg, card = st.load(adapter)
    assert cfg["rank"] == 4 and all(".lora_" in k for k in tens) and card.adapter.kind == "lora" and card.variant_of == "brain/qwen3"
    m = os.path.join(o, "m.safetensors")
    assert main(["toymoe", "train", "--steps", "4", "--out", m, "--device", "cpu"]) == 0
    assert main(["toymoe", "eval", "--weights", m, "--samples", "4", "--device", "cpu"]) == 0
    assert main(["toymoe", "gen", "--weights", m, "--max-new", "3", "--device", "cpu"]) == 0
    assert capsys.readouterr().out.strip().splitlines()[-1].startswith("1,2,3,4,")
    assert main(["flops", "--model", "qwen", "--train", "--stages", "2"]) == 0
    assert "stage 1 (layers 1..2): backward" in capsys.readouterr().out
    assert main(["flops", "--model", "qwen", "--train", "--i8"]) == 2
    assert main(["gradcheck"]) == 0
    assert "0 failures" in capsys.readouterr().out
    assert main(["quantize", q, "--out", os.path.join(o, "q.w8.safetensors")]) == 0
    capsys.readouterr()
    assert main(["quantize", q, "--plan", "--keep", "blocks.0."]) == 0
    plan = capsys.readouterr().out.splitlines()
    assert any(l.split() == ["q8", "blocks.1.attn.wq.weight"] for l in plan)
    assert any(l.split() == ["bf16", "blocks.0.attn.wq.weight"] for l in plan)        # kept by --keep
    assert main(["quantize", q, "--tier", "Q4_K_M"]) == 2


def test_console_script_runs():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "brain"), "--version"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.startswith("brain ")
    r = subprocess.run([sys.executable, "-m", "brain_b200.cli", "caps"], capture_output=True, text=True, timeout=120,
                       cwd=ROOT, env=dict(os.environ, BRAIN_MOCK="1"))
    man = json.loads(r.stdout)
    assert man[0]["model"] == "brain/mock" and {a["name"] for a in man[0]["actions"]} == {"generate", "embed"}


# ------------------------------------------------------------------------------------ federated / perf / cost
def test_federated_split_verify_assemble(tmp_path):
    from brain_b200.checkpoint import st
    from brain_b200.federated import shard
    from brain_b200.models.config import MoeConfig
    from brain_b200.models.moe import MoeModel
    m = MoeModel(MoeConfig.toy()).init_weights(4)
    base = str(tmp_path / "m.safetensors")
    st.save_model(base, m)
    assert shard.expert_id("blocks.1.moe.experts.3.w_up.weight") == 3 and shard.expert_id("blocks.1.moe.router.weight") is None
    man = shard.split(base, tmp_path / "s")
    assert man.experts == [0, 1, 2, 3] and len(man.files) == 5
    assert shard.verify(tmp_path / "s").base_config_sha256 == man.base_config_sha256
    shard.merge_to_full(tmp_path / "s", str(tmp_path / "full.safetensors"))
    a, _, _ = st.load(base)
    b, _, _ = st.load(str(tmp_path / "full.safetensors"))
    assert list(a) == list(b) and all(torch.equal(a[k], b[k]) for k in a)
    with torch.no_grad():
        m.blocks[0].moe.w_down[1].add_(1.0)
    st.save_model(str(tmp_path / "m2.safetensors"), m)
    ov = shard.split_filtered(str(tmp_path / "m2.safetensors"), tmp_path / "ov", [1])
    assert ov.experts == [1] and "shared.safetensors" not in ov.files
    shard.assemble(tmp_path / "s", [tmp_path / "ov"], str(tmp_path / "asm.safetensors"))
    c, _, _ = st.load(str(tmp_path / "asm.safetensors"))
    changed = [k for k in a if not torch.equal(a[k], c[k])]
    assert changed == ["blocks.0.moe.experts.1.w_down.weight"]
    with open(tmp_path / "s" / "experts" / "expert_2.safetensors", "ab") as f:
        f.write(b"x")
    with pytest.raises(IOError):
        shard.verify(tmp_path / "s")


def test_perf_harness_fake_target_and_gate(tmp_path):
    from brain_b200.perf import fidelity, gate
    from brain_b200.perf.driver import drive
    from brain_b200.perf.metrics import Dist, Summary
    from brain_b200.perf.targets import FakeTarget
    from brain_b200.perf.workload import Arrival, Lengths, gamma_interarrival, standard, standard_names
    from brain_b200.data.rng import Rng
    assert {"interactive", "chat", "rag", "rag_long", "agent", "decode_heavy", "prefill_heavy", "shared_prefix"} <= set(standard_names())
    wl = standard("interactive", Arrival.closed_loop(4), 12, seed=1)
    reqs = wl.requests()
    assert len(reqs) == 12 and all(r.prompt.size == 128 and r.max_new == 256 for r in reqs)
    mix = standard("serving_mix", Arrival.closed_loop(256), 64, seed=2).requests()
    assert all(128 <= r.prompt.size <= 2048 and r.max_new == 256 for r in mix) and len({r.prompt.size for r in mix}) > 20
    sp = standard("shared_prefix", Arrival.saturated(), 3).requests()
    assert np.array_equal(sp[0].prompt[:6144], sp[1].prompt[:6144]) and not np.array_equal(sp[0].prompt[6144:], sp[1].prompt[6144:])
    run = drive(FakeTarget(4, 2), wl)
    s = Summary.build(run.records, run.wall_s, wl.classes[0].slo)
    assert s.completed == 12 and s.output_artifacts == 12 * 256 and s.failed == 0 and s.slo_attainment == 1.0
    assert s.to_json()["ttfa_ms"]["n"] == 12
    rng = Rng(3)
    xs = [gamma_interarrival(rng, 50.0, 1.0) for _ in range(4000)]
    assert abs(sum(xs) / len(xs) - 0.02) < 0.002
    delays = standard("interactive", Arrival.rate(100.0), 50).arrival_delays()
    assert len(delays) == 50 and all(d >= 0 for d in delays)
    assert Lengths.uniform(3, 3).sample(rng) == 3 and 10 <= Lengths.lognormal(100, 0.5, 10, 1000).sample(rng) <= 1000
    d = Dist()
    [d.push(x) for x in range(101)]
    assert d.pct(0.5) == 50 and d.pct(0.99) == 99
    f = fidelity.serial_vs_concurrent(lambda: FakeTarget(4, 2), wl, n=4)
    assert f.passed and f.agreement == 1.0
    assert not fidelity.greedy("x", [[1, 2, 3]], [[1, 9, 3]]).passed
    base = s.to_json()
    worse = dict(base, output_per_s=base["output_per_s"] * 0.5)
    assert gate.passed(gate.compare(base, base, 0.9)) and not gate.passed(gate.compare(worse, base, 0.9))
    a, b = str(tmp_path / "a.json"), str(tmp_path / "b.json")
    assert main(["perf", "run", "chat", "--target", "fake", "--requests", "8", "--concurrency", "4", "--out", a]) == 0
    assert main(["perf", "run", "chat", "--target", "qwen-synth:1x32x4x300", "--requests", "3", "--concurrency", "3", "--ctx", "2048",
                 "--device", "cpu", "--out", b]) == 0
    assert json.loads(open(b).read())["fidelity"]["passed"]
    assert main(["perf", "gate", a, a]) == 0 and main(["perf", "list"]) == 0


def test_cost_registry_and_roof():
    from brain_b200.models.config import QwenConfig
    from brain_b200.utils import cost
    from brain_b200.utils.roof import Roof
    c = cost.kernel_cost("gemm_bf16", M=128, N=256, K=64)
    assert c.flops == 2 * 128 * 256 * 64 and c.bytes == 2 * (128 * 64 + 256 * 64 + 128 * 256)
    assert cost.kernel_cost("gemm_i8", M=8, N=8, K=8).int_ops == 1024 and cost.kernel_cost("nosuch") is None
    cfg = QwenConfig.preset("0.6b")
    fwd, bwd = cost.qwen_cost(cfg, 1, 4096, True)
    dense = 2.0 * 4096 * (cfg.param_count() - cfg.vocab * cfg.d_model + cfg.vocab * cfg.d_model)   # matmul weights incl. tied head
    assert fwd.by_class["matmul"].flops == pytest.approx(dense, rel=0.02)
    assert bwd.by_class["matmul"].flops == pytest.approx(2 * fwd.by_class["matmul"].flops, rel=1e-6)
    assert fwd.coverage() == 1.0 and "total" in str(fwd)
    parts = [cost.qwen_cost(cfg, 1, 4096, True, shard=s)[0].total.flops for s in cost.even_shards(cfg.n_layers, 4)]
    assert sum(parts) == pytest.approx(fwd.total.flops, rel=1e-9)
    r = Roof(6551.0, 1640.0, 1384.0)
    assert r.bound(1e15, 1e6) == "compute" and r.bound(1e6, 1e12) == "memory"
    assert r.min_seconds(1640e12, 0) == pytest.approx(1.0)


def test_weighted_loss_and_fit(tmp_path):
    """sum_i w_i CE_i / count: unit weights reproduce the plain loss, zero weights give zero loss and
    zero gradients, and ``fit(weighted=True)`` trains from train.weight.bin."""
    import numpy as np
    import torch
    from brain_b200 import gradcheck
    from brain_b200.data import binio
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.train import FitOpts, fit
    cfg = QwenConfig.tiny()
    m = Qwen3(cfg).init_weights(1)
    x = torch.randint(0, cfg.vocab, (2, 6), dtype=torch.int32)
    y = torch.randint(0, cfg.vocab, (2, 6))
    plain = m.loss(x, y)
    assert torch.allclose(m.loss(x, y, None, torch.ones(2, 6)), plain, atol=1e-6)
    assert torch.allclose(m.loss(x, y, None, torch.full((2, 6), 2.0)), 2 * plain, atol=1e-5)
    z = m.loss(x, y, None, torch.zeros(2, 6))
    z.backward()
    assert float(z) == 0.0 and all(p.grad is None or float(p.grad.abs().max()) == 0.0 for p in m.parameters())
    assert gradcheck.run_gate(("qwen3_weighted",), out=lambda s: None) == 0
    d = str(tmp_path / "w")
    rng = np.random.default_rng(0)
    toks = rng.integers(0, 20, 600)
    binio.write_dataset(d, toks[:500], toks[500:], vocab_size=20, weights=rng.random(500).astype("float32"))
    o = FitOpts(steps=4, batch_size=2, block_size=8, eval_interval=0, checkpoint_secs=0, device="cpu", weighted=True)
    build = lambda vocab, blk: Qwen3(QwenConfig(vocab=vocab, block_size=blk, n_layers=1, d_model=16, n_heads=2,
                                                n_kv_heads=1, head_dim=8, d_ff=32))
    l0, l1 = fit(d, build, o, None, log=lambda s: None)
    assert l0 == l0 and l1 == l1


def test_q4_storage_and_fp8_block_import(tmp_path):
    """4-bit nibble packing round-trips with sign extension; an FP8-E4M3 export with 128x128 block
    multipliers imports to the same weights as its bf16 original (within fp8 resolution)."""
    import json
    import torch
    from brain_b200.checkpoint import st
    from brain_b200.checkpoint.hf_import import dequant_block, hf_name, import_qwen
    from brain_b200.models.config import QwenConfig
    from brain_b200.serve.quantize import dequantize_weight_q4, quantize_weight_q4
    w = torch.tensor([[7.0, -7.0, 1.0, -1.0, 0.0, 3.5, -3.5, 6.9] * 2, [0.1] * 8 + [-0.2] * 8])
    words, sw = quantize_weight_q4(w)
    assert words.shape == (2, 2) and words.dtype == torch.int32
    back = dequantize_weight_q4(words, sw)
    assert torch.allclose(back[0, :4], torch.tensor([7.0, -7.0, 1.0, -1.0]))       # negatives survive
    assert (back - w).abs().max() <= sw.max() / 2 + 1e-6
    with pytest.raises(ValueError):
        quantize_weight_q4(torch.zeros(2, 12))
    raw = torch.randn(200, 300)
    sc = torch.rand(2, 3) + 0.5
    full = dequant_block(raw, sc, 128)
    assert torch.allclose(full[130, 260], raw[130, 260] * sc[1, 2]) and torch.allclose(full[0, 0], raw[0, 0] * sc[0, 0])
    with pytest.raises(ValueError):
        dequant_block(raw, torch.ones(2, 2), 128)

    # a tiny HF-layout export whose 2-D projection weights are fp8 + *_scale_inv
    cfg = QwenConfig(vocab=32, block_size=16, n_layers=1, d_model=128, n_heads=2, n_kv_heads=1, head_dim=64, d_ff=256,
                     tie_embeddings=True)
    g = torch.Generator().manual_seed(0)
    hf_dir = tmp_path / "hf"
    hf_dir.mkdir()
    tensors, specs = {}, []
    shapes = cfg.param_shapes() if hasattr(cfg, "param_shapes") else None
    for name, numel in cfg.param_list():
        src = hf_name(name)
        if src.endswith("proj.weight"):
            rows = {"q_proj": 128, "k_proj": 64, "v_proj": 64, "o_proj": 128, "gate_proj": 256, "up_proj": 256,
                    "down_proj": 128}[src.split(".")[-2]]
            wt = torch.randn(rows, numel // rows, generator=g) * 0.05
            s_inv = wt.abs().amax() / 400.0 * torch.ones(-(-rows // 128), -(-(numel // rows) // 128))
            q8 = (wt / s_inv[0, 0]).to(torch.float8_e4m3fn)
            tensors[src] = ("F8_E4M3", q8.view(torch.uint8), (rows, numel // rows))
            tensors[src + "_scale_inv"] = ("BF16", s_inv, tuple(s_inv.shape))
            tensors["_want_" + name] = q8.float() * s_inv[0, 0].bfloat16().float()
        else:
            t = torch.randn(numel, generator=g) * 0.05
            tensors[src] = ("BF16", t, (numel,))
            tensors["_want_" + name] = t.bfloat16().float()
    names = [k for k in tensors if not k.startswith("_want_")]
    wtr = st.StWriter(str(hf_dir / "model.safetensors"), [(n, tensors[n][2], "U8" if tensors[n][0] == "F8_E4M3" else "BF16")
                                                          for n in names], {"format": "pt"}, "BF16")
    for n in names:
        wtr.write(n, tensors[n][1])
    wtr.close()
    # the writer stores raw bytes under U8; patch the header dtype to F8_E4M3 the way an fp8 export labels it
    path = str(hf_dir / "model.safetensors")
    blob = open(path, "rb").read()
    hlen = int.from_bytes(blob[:8], "little")
    header = json.loads(blob[8:8 + hlen])
    for n in names:
        if tensors[n][0] == "F8_E4M3":
            header[n]["dtype"] = "F8_E4M3"
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * (-len(hb) % 8)
    open(path, "wb").write(len(hb).to_bytes(8, "little") + hb + blob[8 + hlen:])
    (hf_dir / "config.json").write_text(json.dumps({
        "model_type": "qwen3", "vocab_size": 32, "hidden_size": 128, "num_hidden_layers": 1, "num_attention_heads": 2,
        "num_key_value_heads": 1, "head_dim": 64, "intermediate_size": 256, "max_position_embeddings": 16,
        "rms_norm_eps": 1e-6, "rope_theta": 1e6, "tie_word_embeddings": True,
        "quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}}))
    out = str(tmp_path / "q.safetensors")
    import_qwen(str(hf_dir), out)
    got, _, _ = st.load(out)
    for name, _ in cfg.param_list():
        assert torch.allclose(got[name].reshape(-1), tensors["_want_" + name].reshape(-1), atol=1e-6), name


def test_checkpoint_chat_template_is_rendered(tmp_path):
    """A tokenizer directory with its own Jinja chat template: rendered through the sandboxed
    environment (raise_exception, tojson with source key order, generation prompt), and picked up by
    ``BpeTokenizer.from_file``; without one the built-in ChatML form is used."""
    import json
    from brain_b200.data.chat_template import ChatTemplate, TemplateError
    from brain_b200.data.tokenizer import BpeTokenizer, bytes_to_unicode, render_chatml
    src = ("{%- if tools %}<tools>{% for t in tools %}{{ t | tojson }}{% endfor %}</tools>{{ '\\n' }}{% endif -%}"
           "{%- for m in messages -%}"
           "{%- if m.role not in ['system', 'user', 'assistant'] %}{{ raise_exception('bad role ' + m.role) }}{% endif -%}"
           "{{ '<|im_start|>' + m.role + '\\n' + m.content + '<|im_end|>' + '\\n' }}"
           "{%- endfor -%}"
           "{%- if add_generation_prompt %}{{ '<|im_start|>assistant\\n' }}"
           "{%- if enable_thinking is defined and enable_thinking is false %}{{ '<think>\\n\\n</think>\\n\\n' }}{% endif %}{% endif %}")
    t = ChatTemplate(src)
    msgs = [("system", "be brief"), ("user", "hi")]
    assert t.render(msgs, True) == render_chatml(msgs, True)
    assert t.render(msgs, True, enable_thinking=False) == render_chatml(msgs, True, enable_thinking=False)
    tool = {"type": "function", "function": {"name": "zeta", "parameters": {"b": 1, "a": 2}}}
    out = t.render(msgs, False, tools=[tool])
    assert out.startswith('<tools>{"type": "function", "function": {"name": "zeta", "parameters": {"b": 1, "a": 2}}}</tools>')
    with pytest.raises(TemplateError, match="bad role"):
        t.render([("tool", "x")])
    with pytest.raises(TemplateError):
        ChatTemplate("{% for %}")
    with pytest.raises(TemplateError):          # sandbox: no attribute walks into Python internals
        ChatTemplate("{{ messages.__class__.__mro__ }}").render(msgs)

    d = tmp_path / "tok"
    d.mkdir()
    b2u = bytes_to_unicode()
    vocab = {b2u[b]: b for b in range(256)}
    (d / "tokenizer.json").write_text(json.dumps({"model": {"vocab": vocab, "merges": []},
                                                  "added_tokens": [{"content": "<|im_start|>", "id": 256},
                                                                   {"content": "<|im_end|>", "id": 257}]}))
    plain = BpeTokenizer.from_file(str(d / "tokenizer.json"))
    assert plain.chat_template is None and plain.apply_chat_template(msgs) == render_chatml(msgs, True)
    (d / "tokenizer_config.json").write_text(json.dumps({"chat_template": "{% for m in messages %}[{{ m.role }}] {{ m.content }}\\n{% endfor %}{{ eos_token }}",
                                                         "eos_token": {"content": "<|im_end|>"}}))
    own = BpeTokenizer.from_file(str(d / "tokenizer.json"))
    assert own.apply_chat_template(msgs) == "[system] be brief\\n[user] hi\\n<|im_end|>"
    (d / "chat_template.jinja").write_text("J:{{ messages | length }}")
    assert BpeTokenizer.from_file(str(d / "tokenizer.json")).apply_chat_template(msgs) == "J:2"


def test_device_selection_grammar():
    import os
    import torch
    from brain_b200.train import pick_device
    from brain_b200.utils.devices import apply_selection, parse_selection
    s = parse_selection("")
    assert s.gpus is None and s.cpu and s.cores is None
    assert parse_selection("cpu").gpus == [] and parse_selection("cpu").first() == torch.device("cpu")
    assert parse_selection("gpu").gpus is None and not parse_selection("gpu").cpu
    s = parse_selection("gpu1,cpu0-3")
    assert s.gpus == [1] and s.cpu and s.cores == [0, 1, 2, 3]
    assert parse_selection("gpu0,gpu1").gpus == [0, 1] and parse_selection("cuda:2").gpus == [2]
    assert parse_selection("cpu21").cores == [21] and parse_selection("gpu,cpu").gpus is None
    for bad in ("npu", "vulkan", "tpu", "cpu3-1", "cpux"):
        with pytest.raises(ValueError):
            parse_selection(bad)
    before = os.sched_getaffinity(0)
    threads = torch.get_num_threads()
    try:
        core = min(before)
        assert pick_device(f"cpu{core}") == torch.device("cpu")
        assert os.sched_getaffinity(0) == {core} and torch.get_num_threads() == 1
        with pytest.raises(ValueError):
            apply_selection(parse_selection("cpu100000"))
    finally:
        os.sched_setaffinity(0, before)
        torch.set_num_threads(threads)


def test_learnability_battery(capsys):
    """Tiny decoders learn copy / modular addition / running parity on CPU in a few hundred steps
    (both families), through the same trainer and kernels' CPU reference path as everything else."""
    from brain_b200 import learnbench
    from brain_b200.cli.main import main
    r = learnbench.run_battery(["copy", "parity"], "qwen", steps=250, log=lambda s: None)
    assert [x["task"] for x in r] == ["copy", "parity"] and all(x["passed"] for x in r), r
    assert main(["bench", "learn", "mod_add", "--arch", "gpt", "--steps", "300", "--device", "cpu"]) == 0
    assert "PASS" in capsys.readouterr().out
    assert main(["bench", "learn", "nosuchtask", "--device", "cpu"]) == 2
    assert main(["npu", "export"]) == 2 and "not built" in capsys.readouterr().err
