"""Greedy speculative decoding (reference: crates/qwen3/src/serve.rs:1892-1975 ``spec_decode``).

A draft proposes up to ``k`` tokens from the running context; the target checks them in ONE forward
over ``[pending, proposals…]``, keeps the longest prefix it agrees with plus its own next token (the
correction, or the bonus token when every proposal was accepted), and rolls the paged cache back
over the rejected rows.  The output equals plain greedy decoding of the target; the gain is fewer
target forwards when the draft guesses well."""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np

from .paged import BlockAllocator, BlockTable

Draft = Callable[[Sequence[int], int], Sequence[int]]


def spec_decode(engine, prompt: Sequence[int], max_new: int, k: int, draft: Draft,
                alloc: Optional[BlockAllocator] = None) -> Tuple[List[int], int]:
    """Returns (generated tokens, number of target forwards after the prompt prefill).
    ``alloc``: the allocator that owns the engine's block pool (a private one by default, for
    offline use of an engine no scheduler is driving)."""
    if not prompt or k < 1:
        raise ValueError("spec_decode needs a non-empty prompt and k >= 1")
    if len(prompt) + max_new > engine.max_seq_len:
        raise ValueError("prompt + max_new exceeds the engine's context")
    alloc = alloc or BlockAllocator(engine.num_blocks, engine.block_size)
    table = BlockTable()
    bt = np.zeros(engine.max_blocks, dtype=np.int32)

    def reserve(n: int):
        table.reserve(n, alloc)   # raises MemoryError when the pool is exhausted
        blocks = table.blocks()
        bt[:len(blocks)] = blocks

    try:
        head = list(prompt[:-1])
        step = engine.max_prefill_tokens
        for st in range(0, len(head), step):
            chunk = np.asarray(head[st:st + step], dtype=np.int32)
            reserve(len(chunk))
            engine.prefill_chunk(chunk, st, bt, last=False)
        pending = int(prompt[-1])
        ctx = list(prompt)
        out: List[int] = []
        forwards = 0
        while len(out) < max_new:
            want = min(max_new - len(out), k)
            props = [int(t) for t in list(draft(ctx, want))[:want]]
            base = len(table)
            rows = len(props) + 1
            reserve(rows)
            pred = engine.verify_chunk(np.asarray([pending] + props, dtype=np.int32), base, bt)
            forwards += 1
            accepted = 0
            while accepted < len(props) and int(pred[accepted]) == props[accepted]:
                accepted += 1
            correction = int(pred[accepted])
            out.extend(props[:accepted])
            out.append(correction)
            ctx.extend(props[:accepted])
            ctx.append(correction)
            # keep pending + the accepted proposals; the correction is the next pending token
            table.truncate(base + accepted + 1, alloc)
            pending = correction
        return out[:max_new], forwards
    finally:
        table.release(alloc)


def ngram_draft(n: int = 3) -> Draft:
    """Prompt-lookup drafting: propose what followed the most recent earlier occurrence of the
    context's last ``n`` tokens (no second model; effective on repetitive text)."""
    def draft(ctx: Sequence[int], want: int) -> List[int]:
        ctx = list(ctx)
        for m in range(min(n, len(ctx) - 1), 0, -1):
            tail = ctx[-m:]
            for i in range(len(ctx) - m - 1, -1, -1):
                if ctx[i:i + m] == tail:
                    nxt = ctx[i + m:i + m + want]
                    if nxt:
                        return nxt + [nxt[-1]] * (want - len(nxt))
        return [ctx[-1]] * want
    return draft
