"""Serving stack on CPU: native paged-KV bookkeeping, scheduler semantics with a deterministic
fake decoder, and the Qwen engine (paged == contiguous, batched == per-sequence, chunked prefill ==
whole, warm prefix-cache prefill == cold, cancel reclaims blocks)."""
import numpy as np
import pytest
import torch

from brain_b200.data.rng import Rng
from brain_b200.serve.paged import BlockAllocator, BlockTable, PrefixCache
from brain_b200.serve.sampling import SampleParams, sample_from_topk
from brain_b200.serve.scheduler import FINISHED, RejectReason, Scheduler


def test_allocator_and_table():
    a = BlockAllocator(4, 4)
    t = BlockTable()
    for i in range(6):
        b, o = t.append(a)
        assert o == i % 4
    assert len(t) == 6 and t.blocks() == [0, 1] and a.free_blocks() == 2
    assert t.reserve(3, a) == 6 and len(t) == 9 and len(t.blocks()) == 3
    t.truncate(5, a)
    assert len(t.blocks()) == 2 and a.free_blocks() == 2
    f = t.fork(a)
    assert a.refcount(1) == 2
    old, new = f.unshare_tail(a)
    assert old == 1 and new != 1 and a.refcount(1) == 1
    t.release(a)
    f.release(a)
    assert a.free_blocks() == 4
    with pytest.raises(RuntimeError):
        a.decref(0)
    t2 = BlockTable()
    for _ in range(16):
        t2.append(a)
    with pytest.raises(MemoryError):
        t2.append(a)


def test_prefix_cache_lru():
    a = BlockAllocator(8, 2)
    pc = PrefixCache()
    t = BlockTable()
    prompt = [1, 2, 3, 4, 5, 6, 7]
    t.reserve(len(prompt), a)
    pc.insert_chain(prompt, t.blocks(), 0, a)
    assert len(pc) == 3
    assert pc.lookup(prompt, 2, 6) == t.blocks()[:3]
    assert pc.lookup(prompt, 2, 4) == t.blocks()[:2]
    assert pc.lookup([1, 2, 9, 9], 2, 4) == t.blocks()[:1]
    assert pc.evict(2, a) == 0          # still referenced by the sequence
    blocks = t.blocks()
    t.release(a)
    assert a.free_blocks() == 8 - 3      # cache keeps the three full blocks
    pc.lookup(prompt[:2], 2, 2)          # touch the first block: most recently used
    assert pc.evict(1, a) == 1 and a.refcount(blocks[0]) == 1


def test_prefix_index_evicts_leaves_first_and_never_matches_through_a_recycled_parent():
    a = BlockAllocator(8, 2)
    pc = PrefixCache()
    t = BlockTable()
    prompt = [1, 2, 3, 4, 5, 6]
    t.reserve(len(prompt), a)
    blocks = t.blocks()
    pc.insert_chain(prompt, blocks, 0, a)
    t.release(a)                                   # three idle cached blocks, tail released first
    assert pc.evict(1, a) == 1 and a.refcount(blocks[2]) == 0      # the leaf went, not the root
    assert pc.lookup(prompt, 2, 6) == blocks[:2]
    # a sequence that adopts the chain pins it: nothing is evictable while it runs
    t2 = BlockTable()
    t2.adopt_prefix(pc.lookup(prompt, 2, 4), a)
    assert pc.evict(4, a) == 0
    t2.release(a)
    # evict the root only (touch the second block so the root is the least recently used) ...
    assert pc.evict(2, a) == 2 and len(pc) == 0
    # ... and publish other content: an old child hash can never be reached through a new parent
    t3 = BlockTable()
    other = [9, 9, 3, 4]
    t3.reserve(len(other), a)
    pc.insert_chain(other, t3.blocks(), 0, a)
    assert pc.lookup([1, 2, 3, 4], 2, 4) == []
    assert pc.lookup(other, 2, 4) == t3.blocks()
    # a duplicate of a cached prefix under another physical block keeps the canonical copy
    t4 = BlockTable()
    t4.reserve(len(other), a)
    pc.insert_chain(other, t4.blocks(), 0, a)
    assert len(pc) == 2 and pc.lookup(other, 2, 4) == t3.blocks()


def test_sample_from_topk():
    cands = [(7, 3.0), (2, 2.0), (9, 0.5)]
    assert sample_from_topk(cands, SampleParams.greedy(), Rng(0)) == 7
    seen = {sample_from_topk(cands, SampleParams(1.0, 2, 1.0), Rng(s)) for s in range(50)}
    assert seen == {7, 2}
    assert {sample_from_topk(cands, SampleParams(1.0, 0, 0.1), Rng(s)) for s in range(20)} == {7}


class FakeDecoder:
    """Deterministic token function: next = (last + position) % vocab."""
    vocab, block_size, num_blocks = 50, 4, 32
    max_prefill_tokens, max_seq_len, topk_capacity = 8, 64, 8

    def __init__(self):
        self.prefill_calls = []
        self.decode_calls = []

    def prefill_chunk(self, tokens, start, block_table, last, greedy):
        self.prefill_calls.append((len(tokens), start, last))
        if not last:
            return None, None
        t = int(tokens[-1] + start + len(tokens)) % self.vocab
        return t, [(t, 1.0), ((t + 1) % self.vocab, 0.5)]

    def decode(self, tokens, positions, block_tables, window, greedy):
        self.decode_calls.append((len(tokens), window))
        out = []
        for t, p in zip(tokens, positions):
            row, cur = [], int(t)
            for w in range(window):
                cur = (cur + int(p) + w + 1) % self.vocab
                row.append(cur)
            out.append(row)
        cand = None if greedy else [[(r[0], 1.0), ((r[0] + 1) % self.vocab, 0.1)] for r in out]
        return out, cand


def expected_stream(prompt, n):
    toks, cur, pos = [], prompt[-1], len(prompt)
    for _ in range(n):
        cur = (cur + pos) % 50
        toks.append(cur)
        pos += 1
    return toks


def test_scheduler_continuous_batching():
    dec = FakeDecoder()
    s = Scheduler(dec, max_batch=4, window=4)
    a = s.submit([1, 2, 3], 6)
    b = s.submit(list(range(20)), 5)     # needs chunked prefill (max_prefill 8)
    s.run_until_idle()
    assert s.tokens_of(a) == expected_stream([1, 2, 3], 6)
    assert s.tokens_of(b) == expected_stream(list(range(20)), 5)
    assert s.info(a).state == FINISHED and s.info(a).finish == "length"
    assert any(n == 8 and not last for n, _, last in dec.prefill_calls)   # a non-final chunk happened
    assert any(w > 1 for _, w in dec.decode_calls)                        # window decode was used
    st = s.stats()
    assert st["free_blocks"] + st["prefix_entries"] == st["num_blocks"]


def test_scheduler_rejects_and_cancel_and_eos():
    dec = FakeDecoder()
    s = Scheduler(dec, max_batch=2, eos=7, window=1)
    with pytest.raises(RejectReason) as e:
        s.submit([1] * 60, 10)
    assert e.value.kind == "exceeds_capacity" and "needs 70 tokens, engine capacity is 64" in str(e.value)
    with pytest.raises(RejectReason) as e:
        s.submit([99], 4)
    assert e.value.kind == "invalid_token"
    with pytest.raises(RejectReason):
        s.submit([], 4)
    free0 = s.stats()["free_blocks"]
    r = s.submit([3, 4], 30)
    s.step()
    s.step()
    got = s.cancel(r)
    assert len(got) >= 1 and s.stats()["free_blocks"] == free0
    # EOS stops the stream and is not appended: prompt [1, 4] -> first token (4 + 2) = 6, then 6+2=8 ...
    r2 = s.submit([2, 5], 20)            # 5+2 = 7 = EOS immediately
    s.run_until_idle()
    assert s.tokens_of(r2) == [] and s.info(r2).finish == "stop"
    q = Scheduler(FakeDecoder(), max_batch=1, policy="max_queue_depth", policy_arg=1)
    q.submit([1], 2)
    with pytest.raises(RejectReason) as e:
        q.submit([1], 2)
    assert e.value.kind == "policy_rejected"


def test_scheduler_sampling_is_seeded():
    outs = []
    for _ in range(2):
        s = Scheduler(FakeDecoder(), max_batch=2, window=1)
        r = s.submit([5, 6, 7], 8, SampleParams(1.0, 2, 1.0), seed=42)
        s.run_until_idle()
        outs.append(s.tokens_of(r))
    assert outs[0] == outs[1] and len(outs[0]) == 8


# ---------------------------------------------------------------------------------------- engine
def _tiny_engine(weights="bf16", **kw):
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.serve.engine import QwenEngine
    cfg = QwenConfig(vocab=61, block_size=64, n_layers=2, d_model=32, n_heads=4, n_kv_heads=2,
                     head_dim=8, d_ff=48)
    torch.manual_seed(0)
    m = Qwen3(cfg).init_weights(3)
    with torch.no_grad():
        for p in m.parameters():
            p.mul_(4.0)   # make logits well separated so greedy choices are stable
    return QwenEngine(m, block_size=4, num_blocks=64, max_seq_len=64, max_prefill=8, weights=weights, **kw), m


def _greedy_reference(eng, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(eng.logits_all(toks)[-1].argmax()))
    return toks[len(prompt):]


def test_engine_paged_equals_contiguous_and_batched_equals_single():
    eng, _ = _tiny_engine()
    prompts = [[3, 9, 27, 11, 5], list(range(1, 20)), [7]]
    want = [_greedy_reference(eng, p, 6) for p in prompts]
    s = Scheduler(eng, max_batch=4, window=4)
    ids = [s.submit(p, 6) for p in prompts]
    s.run_until_idle()
    assert [s.tokens_of(i) for i in ids] == want
    # one at a time gives the same streams
    eng2, _ = _tiny_engine()
    for p, w in zip(prompts, want):
        s2 = Scheduler(eng2, max_batch=1, window=1)
        r = s2.submit(p, 6)
        s2.run_until_idle()
        assert s2.tokens_of(r) == w


def test_engine_prefix_cache_warm_equals_cold():
    eng, _ = _tiny_engine()
    s = Scheduler(eng, max_batch=2, window=1)
    prompt = list(range(2, 19))
    a = s.submit(prompt, 5)
    s.run_until_idle()
    b = s.submit(prompt, 5)           # warm: adopts the cached full blocks
    s.run_until_idle()
    assert s.tokens_of(a) == s.tokens_of(b)
    assert s.info(b).prefix_hit >= 12 and s.stats()["kv_prefix_hit_tokens"] >= 12


def test_engine_int8_tracks_full_precision():
    eng, _ = _tiny_engine()
    eng8, _ = _tiny_engine("int8")
    toks = list(range(3, 23))
    a, b = eng.logits_all(toks), eng8.logits_all(toks)
    rel = ((a - b).norm() / a.norm()).item()
    assert rel < 0.08
    assert eng8.weight_bytes() < 0.6 * eng.weight_bytes()


def test_full_pool_with_prefix_cache_still_completes_every_request():
    """A pool sized for exactly `concurrency` full-length sequences fills up with cached prompt
    blocks of finished requests; admission must evict them (and keep room for what running
    sequences may still claim) so that every request runs to its full length and every finish is
    reported — a closed-loop driver would otherwise wait forever."""
    from brain_b200.perf.driver import drive
    from brain_b200.perf.metrics import Summary
    from brain_b200.perf.targets import SchedulerTarget, synth_qwen
    from brain_b200.perf.workload import Arrival, standard
    from brain_b200.serve.engine import QwenEngine
    m = synth_qwen("1x32x4x300", "cpu")
    conc, out = 6, 12
    ctx = 512 + out + 16
    per_seq = -(-ctx // 16)
    eng = QwenEngine(m, block_size=16, num_blocks=per_seq * conc + conc, max_seq_len=per_seq * 16, max_prefill=512)
    wl = standard("serving_mix", Arrival.closed_loop(conc), 30, seed=0, vocab=300)
    wl.classes[0].input.lo, wl.classes[0].input.hi = 64, 512
    wl.classes[0].output.n = out
    t = SchedulerTarget(None, max_batch=conc, ctx=per_seq * 16, engine=eng)
    run = drive(t, wl, max_seconds=120)
    s = Summary.build(run.records, run.wall_s, wl.classes[0].slo)
    assert s.completed == 30 and s.failed == 0 and s.rejected == 0
    assert all(r.output_artifacts() == out for r in run.records)
    st = t.sched.stats()
    assert st["running"] == 0 and st["waiting"] == 0 and st["finished"] == 30


def test_packed_prefill_equals_one_by_one():
    """Several prompts (and a continuation chunk) prefilled in one packed forward leave the same
    paged KV and pick the same first tokens as prefilling them one at a time."""
    import torch
    from brain_b200.perf.targets import synth_qwen
    from brain_b200.serve.engine import QwenEngine
    m = synth_qwen("2x32x4x200", "cpu")
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 200, n).astype(np.int32) for n in (37, 64, 21)]

    def tables(eng):
        out, nxt = [], 0
        for p in prompts:
            nb = -(-(len(p) + 8) // eng.block_size)
            bt = np.full(eng.max_blocks, -1, dtype=np.int32)
            bt[:nb] = np.arange(nxt, nxt + nb)
            nxt += nb
            out.append(bt)
        return out
    a = QwenEngine(m, block_size=16, num_blocks=64, max_seq_len=128, max_prefill=64)
    b = QwenEngine(m, block_size=16, num_blocks=64, max_seq_len=128, max_prefill=64)
    ta, tb = tables(a), tables(b)
    # engine a: one by one; the second prompt in two chunks (32 + 32)
    ra = [a.prefill_chunk(prompts[0], 0, ta[0], True)]
    a.prefill_chunk(prompts[1][:32], 0, ta[1], False)
    ra.append(a.prefill_chunk(prompts[1][32:], 32, ta[1], True))
    ra.append(a.prefill_chunk(prompts[2], 0, ta[2], True, greedy=False))
    # engine b: first chunk of prompt 1 alone, then everything else packed (incl. the continuation)
    b.prefill_chunk(prompts[1][:32], 0, tb[1], False)
    rb = b.prefill_batch([(prompts[0], 0, tb[0], True, True), (prompts[1][32:], 32, tb[1], True, True),
                          (prompts[2], 0, tb[2], True, False)])
    assert [r[0] for r in ra] == [r[0] for r in rb]
    assert rb[0][1] is None or len(rb[0][1]) > 0
    assert [c[0] for c in ra[2][1][:5]] == [c[0] for c in rb[2][1][:5]]
    for li in range(2):
        assert torch.allclose(a.kc[li][:12], b.kc[li][:12], atol=1e-5)
        assert torch.allclose(a.vc[li][:12], b.vc[li][:12], atol=1e-5)


def test_admission_batching_takes_requests_in_groups():
    from brain_b200.perf.driver import drive
    from brain_b200.perf.metrics import Summary
    from brain_b200.perf.targets import SchedulerTarget, synth_qwen
    from brain_b200.perf.workload import Arrival, standard
    m = synth_qwen("1x32x4x300", "cpu")

    def run(admit, wait=64):
        wl = standard("serving_mix", Arrival.closed_loop(8), 32, seed=0, vocab=300)
        wl.classes[0].input.lo, wl.classes[0].input.hi = 16, 64
        wl.classes[0].output = type(wl.classes[0].output).uniform(4, 24)
        t = SchedulerTarget(m, max_batch=8, ctx=256, admit_batch=admit, admit_max_wait=wait)
        r = drive(t, wl, max_seconds=120)
        s = Summary.build(r.records, r.wall_s, wl.classes[0].slo)
        return s, t.sched.stats(), [t.outputs(i) for i in r.ids]
    s1, st1, o1 = run(1)
    s4, st4, o4 = run(4)
    assert s1.completed == s4.completed == 32 and s4.output_artifacts == s1.output_artifacts
    assert o1 == o4                                  # batching admissions never changes greedy outputs
    # admission every few steps: held requests do not switch off the on-device decode window, so
    # there are fewer engine calls for the same tokens, and still the same outputs
    sw, stw, ow = run(8, wait=3)
    assert sw.completed == 32 and ow == o1
    assert stw["steps"] <= st1["steps"]


def test_mixed_steps_equal_separate_prefill_and_decode():
    """With ``mixed`` the steps that carry prompt chunks and a decode batch run as one forward; every
    stream (greedy and seeded sampling) is the same as with separate forwards."""
    prompts = [[3, 9, 27, 11, 5], list(range(1, 20)), [7], list(range(20, 33)), [4, 4, 8]]

    def run(mixed):
        eng, _ = _tiny_engine()
        s = Scheduler(eng, max_batch=2, window=1, mixed=mixed)
        ids = [s.submit(p, 7) for p in prompts[:4]]
        ids.append(s.submit(prompts[4], 7, SampleParams(0.8, 5, 0.9), seed=11))
        n_mixed = 0
        while not s.is_idle():
            n_mixed += int(s.step().mixed)
        return [s.tokens_of(i) for i in ids], n_mixed, eng
    sep, n0, _ = run(False)
    mix, n1, eng = run(True)
    assert n0 == 0 and n1 > 0 and eng.acct["mixed_calls"] == n1
    assert mix == sep
    assert mix[0] == _greedy_reference(eng, prompts[0], 7)


def test_first_token_budget_policy_bounds_the_queue_by_measured_prefill_rate():
    """``ttft_budget``: admission rejects a request whose first token, at the prefill rate the
    scheduler measured from its own steps, would come after the budget.  A synthetic clock makes a
    prompt token cost exactly one millisecond."""
    class Clock:
        t = 0.0

        def __call__(self):
            return self.t

    class TimedDecoder(FakeDecoder):
        def __init__(self, clock):
            super().__init__()
            self.clock = clock

        def prefill_chunk(self, tokens, start, block_table, last, greedy):
            self.clock.t += len(tokens) * 1e-3
            return super().prefill_chunk(tokens, start, block_table, last, greedy)

    clk = Clock()
    s = Scheduler(TimedDecoder(clk), max_batch=1, window=1, policy="ttft_budget", policy_arg=20.0)
    s.clock = clk
    # no measurement yet: nothing is rejected, however long the queue
    a = s.submit(list(range(16)), 2)
    b = s.submit(list(range(16)), 2)
    assert s.pending_prefill_tokens() == 32
    s.step()                                  # prefills 8 tokens of `a` in 8 ms -> 1 token / ms
    assert s.prefill_tokens_per_ms == pytest.approx(1.0)
    assert s.pending_prefill_tokens() == 24
    # 24 tokens ahead: a 4-token prompt would see its first token after 28 ms > 20 ms
    with pytest.raises(RejectReason) as e:
        s.submit([1, 2, 3, 4], 2)
    assert e.value.kind == "policy_rejected"
    s.step()                                  # rest of `a`
    assert s.pending_prefill_tokens() == 16
    c_ = s.submit([1, 2, 3, 4], 2)            # 16 + 4 = 20 ms: inside the budget
    with pytest.raises(RejectReason):
        s.submit([1], 2)                      # 21 ms
    s.run_until_idle()
    for r in (a, b, c_):
        assert s.info(r).state == FINISHED
    assert s.pending_prefill_tokens() == 0
    s.submit(list(range(20)), 2)              # an empty engine takes a prompt as long as the budget


def test_deadline_aware_policy_is_fed_by_the_measured_time_in_system():
    """``deadline_aware`` rejects while queue length x mean time in the system exceeds the budget;
    the mean comes from the scheduler's own clock (submit -> finished)."""
    class Clock:
        t = 0.0

        def __call__(self):
            return self.t

    clk = Clock()

    class TimedDecoder(FakeDecoder):
        def decode(self, tokens, positions, block_tables, window, greedy):
            clk.t += 5e-3
            return super().decode(tokens, positions, block_tables, window, greedy)

    s = Scheduler(TimedDecoder(), max_batch=1, window=1, policy="deadline_aware", policy_arg=25.0)
    s.clock = clk
    r = s.submit([1, 2], 3)                   # first token from prefill, then two decode steps of 5 ms
    s.run_until_idle()
    assert s.info(r).state == FINISHED and s.service_ms == pytest.approx(10.0)
    ids = [s.submit([1, 2], 3) for _ in range(3)]      # queue 0, 1, 2 -> 0, 10, 20 ms: admitted
    with pytest.raises(RejectReason) as e:
        s.submit([1, 2], 3)                            # queue 3 -> 30 ms > 25 ms
    assert e.value.kind == "policy_rejected"
    s.run_until_idle()
    assert all(s.info(i).state == FINISHED for i in ids)
