"""Paged-KV inference engine for the dense Qwen3 family (reference: crates/qwen3/src/serve.rs:
432-530 Engine state, 1194-1304 batched decode steps, 1350-1394 greedy head, 1557-1623 chunked
prefill with prefix-cache reuse).

* KV cache: per layer K and V pools ``[num_blocks, n_kv_heads, block_size, head_dim]`` bf16, or
  with ``kv_dtype='int8'`` int8 rows plus one fp32 scale per stored row (``min(absmax, ceiling)/127``
  with the per-head ceilings of ``brain qwen3 calib``); the first chunk of a prompt attends over its
  own unquantised K/V, everything later reads the quantised pool.
* ``prefill_chunk``: one chunk of one prompt; K/V rows are appended to the sequence's pages, and
  attention runs the tcgen05 flash kernel over (pages gathered to a contiguous buffer when the chunk
  has a past, else the chunk itself).
* ``decode``: one batched step (or a window of k greedy steps fed back on the device) over all
  running sequences with the split-KV paged attention kernel; greedy head = on-device argmax.
* ``weights='int4'``: W4A8 — 4-bit per-output-channel symmetric weights (half a byte per parameter in
  device memory, crates/model/src/int4.rs:46-73) expanded into one shared int8 scratch right before
  each projection's int8 GEMM; activations as in W8A8.
* ``weights='int8'``: W8A8 — per-output-channel symmetric int8 weights, dynamic per-token int8
  activations, tcgen05 ``kind::i8`` GEMM with both scales applied in the epilogue
  (crates/model/src/int8.rs:33-59, 221-235).
* Tensor parallel serving: with a ``tp`` group every rank holds a head-/column-slice of the
  projections and the row-parallel outputs are summed by the one-shot peer all-reduce
  (``parallel.tp``).
"""
from __future__ import annotations

import math
import os
import time
from typing import List, Optional, Tuple

import numpy as np
import torch

from ..models.config import QwenConfig
from ..ops import functional as F
from ..ops import reference as ref
from ..ops import _cuda
from ..ops._cuda import L, call, stream_ptr
from ..ops.attention import flash_attention, flash_attention_into


class _Lin:
    """A projection held as bf16 weights, as W8A8 int8 weights + per-channel scales, or as W4A8:
    4-bit weights (half a byte per parameter in memory) that are expanded into a scratch int8 buffer
    shared by all projections right before the int8 GEMM that consumes them."""

    _scratch = {}       # device -> int8 scratch for the expanded 4-bit weights (grows to the largest)

    def __init__(self, w: torch.Tensor, bias: Optional[torch.Tensor] = None, int8: bool = False,
                 int4: bool = False):
        self.int8 = int8 or int4
        self.int4 = int4
        self.bias = bias.float().contiguous() if bias is not None else None
        self.out_features = w.shape[0]
        if int4:
            from .quantize import quantize_weight_q4
            words, sw = quantize_weight_q4(w.float().cpu())
            self.words, self.sw = words.to(w.device).contiguous(), sw.to(w.device).contiguous()
            self.shape = (w.shape[0], w.shape[1])
        elif int8:
            self.wq, self.sw = F.quant_rows(w.float() if not w.is_cuda else w)
            self.wq, self.sw = self.wq.contiguous(), self.sw.contiguous()
        else:
            self.w = w.contiguous()

    def _wq(self) -> torch.Tensor:
        """The int8 operand: resident (W8A8) or expanded from the nibbles into the scratch (W4A8)."""
        if not self.int4:
            return self.wq
        if not self.words.is_cuda:
            return F.unpack_q4(self.words)
        n = self.shape[0] * self.shape[1]
        buf = _Lin._scratch.get(self.words.device)
        if buf is None or buf.numel() < n:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the 4-bit expansion scratch must be sized before graph capture")
            buf = _Lin._scratch[self.words.device] = torch.empty(n, device=self.words.device, dtype=torch.int8)
        return F.unpack_q4(self.words, buf[:n].view(self.shape))

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.int8:
            wq = self._wq()
            if x.is_cuda:
                xq, sx = F.quant_rows(x)
                y = F.gemm_i8(xq, wq, sx, self.sw)
            else:
                xq, sx = ref.quant_rows(x)
                y = ((xq.float() @ wq.float().t()) * sx[:, None] * self.sw[None, :]).to(x.dtype)
            if self.bias is not None:
                y = y + self.bias.to(y.dtype)
            return y
        if x.is_cuda:
            return F.gemm(x, self.w, bias=self.bias)
        return ref.linear(x, self.w, self.bias.to(x.dtype) if self.bias is not None else None)

    def nbytes(self) -> int:
        if self.int4:
            return self.words.numel() * 4 + 4 * self.sw.numel()
        if self.int8:
            return self.wq.numel() + 4 * self.sw.numel()
        return self.w.numel() * self.w.element_size()


class QwenEngine:
    def __init__(self, model, block_size: int = 16, num_blocks: int = 1024, max_seq_len: int = 4096,
                 max_prefill: int = 512, weights: str = "bf16", topk: int = 64, tp=None,
                 decode_splits: int = 0, cuda_graphs: bool = True, kv_dtype: str = "bf16",
                 kv_clip=None, native: Optional[bool] = None):
        cfg: QwenConfig = model.cfg
        self.cfg = cfg
        self.tp = tp
        self.tp_world = tp.world if tp is not None else 1
        self.tp_rank = tp.rank if tp is not None else 0
        dev = next(model.parameters()).device
        self.device = dev
        self.cuda = dev.type == "cuda"
        self.dtype = torch.bfloat16 if self.cuda else torch.float32
        self.vocab = cfg.vocab
        self.block_size, self.num_blocks = block_size, num_blocks
        self.max_seq_len, self.max_prefill_tokens = max_seq_len, max_prefill
        self.topk_capacity = topk
        self.max_blocks = (max_seq_len + block_size - 1) // block_size
        assert weights in ("bf16", "int8", "int4"), weights
        self.int8 = weights in ("int8", "int4")
        self.int4 = weights == "int4"       # W4A8: nibble storage, expanded per projection call
        w = self.tp_world
        assert cfg.n_heads % w == 0 and cfg.n_kv_heads % w == 0 and cfg.d_ff % w == 0, \
            "tensor-parallel degree must divide the head counts and d_ff"
        self.hq, self.hk, self.hd = cfg.n_heads // w, cfg.n_kv_heads // w, cfg.head_dim
        r = self.tp_rank
        q, kv, ff = cfg.q_dim, cfg.kv_dim, cfg.d_ff
        ql, kl, fl = q // w, kv // w, ff // w
        self.ff_local = fl

        def cast(t):
            return t.detach().to(dev, self.dtype)

        self.tok = cast(model.tok)
        self.layers = []
        for blk in model.blocks:
            wqkv = blk.wqkv.detach()
            rows = torch.cat([wqkv[r * ql:(r + 1) * ql], wqkv[q + r * kl:q + (r + 1) * kl],
                              wqkv[q + kv + r * kl:q + kv + (r + 1) * kl]])
            bias = None
            if blk.bqkv is not None:
                b = blk.bqkv.detach()
                bias = torch.cat([b[r * ql:(r + 1) * ql], b[q + r * kl:q + (r + 1) * kl],
                                  b[q + kv + r * kl:q + kv + (r + 1) * kl]]).to(dev)
            gu = blk.gate_up.detach()
            gu_rows = torch.cat([gu[r * fl:(r + 1) * fl], gu[ff + r * fl:ff + (r + 1) * fl]])
            self.layers.append(dict(
                ln1=cast(blk.ln1), ln2=cast(blk.ln2),
                q_norm=cast(blk.q_norm) if blk.q_norm is not None else None,
                k_norm=cast(blk.k_norm) if blk.k_norm is not None else None,
                qkv=_Lin(cast(rows), bias, self.int8, self.int4),
                wo=_Lin(cast(blk.wo.detach()[:, r * ql:(r + 1) * ql]), None, self.int8, self.int4),
                gate_up=_Lin(cast(gu_rows), None, self.int8, self.int4),
                down=_Lin(cast(blk.down.detach()[:, r * fl:(r + 1) * fl]), None, self.int8, self.int4),
            ))
        self.norm = cast(model.norm)
        head = model.head_weight().detach()
        self.head = _Lin(cast(head), None, False)  # the LM head stays bf16 (as the reference keeps it fp32)
        self.cos, self.sin = ref.rope_tables(max_seq_len, cfg.head_dim, cfg.rope_theta, device=dev)
        # one extra physical block past the allocator's range: padded rows of a bucketed decode batch
        # write their K/V there
        self.dummy_block = num_blocks
        shape = (num_blocks + 1, self.hk, block_size, self.hd)
        assert kv_dtype in ("bf16", "int8"), kv_dtype
        self.kv_int8 = kv_dtype == "int8"
        pool_dtype = torch.int8 if self.kv_int8 else self.dtype
        self.kc = [torch.zeros(shape, device=dev, dtype=pool_dtype) for _ in model.blocks]
        self.vc = [torch.zeros(shape, device=dev, dtype=pool_dtype) for _ in model.blocks]
        if self.kv_int8:
            # one fp32 scale per stored row; ceilings on the row absmax per (layer, K|V, kv head)
            self.ks = [torch.zeros(shape[:3], device=dev, dtype=torch.float32) for _ in model.blocks]
            self.vs = [torch.zeros(shape[:3], device=dev, dtype=torch.float32) for _ in model.blocks]
            self.kv_clip = None
            if kv_clip is not None:
                kc_, vc_ = torch.as_tensor(kv_clip["k_clip"]), torch.as_tensor(kv_clip["v_clip"])
                lo, hi = self.tp_rank * self.hk, (self.tp_rank + 1) * self.hk
                self.kv_clip = [torch.stack([kc_[li, lo:hi], vc_[li, lo:hi]]).float().contiguous().to(dev)
                                for li in range(len(model.blocks))]
        self.decode_splits = decode_splits
        self.steps = 0
        self.cuda_graphs = bool(cuda_graphs) and self.cuda
        #: host-side fault-injection point: called with "prefill" / "decode" before the device work
        #: of that call is issued; raising from it models a failed launch without touching the GPU
        self.fault_hook = None
        self._graphs = {}
        self.graph_replays = 0
        #: the layer sequence issued by one native call per layer half / per decode step instead of
        #: one Python wrapper per kernel (CUDA only; same kernels, same results)
        self.native = None
        if native is None:
            native = os.environ.get("BRAIN_SERVE_NATIVE", "1") == "1"
        if native and self.cuda and not self.int4:    # the native sequence takes resident int8 operands
            from .native import NativeForward
            tp_ok = self.tp is None or self.tp_world == 1 or \
                (getattr(self.tp, "impl", "") == "fused" and cfg.d_model % (8 * self.tp_world) == 0)
            if tp_ok and NativeForward.supported(self):
                self.native = NativeForward(self)
        #: host wall time spent inside prefill / decode calls (each ends with a device-to-host read,
        #: so it covers the device work) and what they processed; a serving run reports the split
        self.acct = {"prefill_s": 0.0, "prefill_calls": 0, "prefill_tokens": 0, "prefill_seqs": 0,
                     "decode_s": 0.0, "decode_calls": 0, "decode_rows": 0, "mixed_s": 0.0, "mixed_calls": 0}

    # ------------------------------------------------------------------ accounting
    def kv_pool_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in self.kc) * 2
        if self.kv_int8:
            n += sum(t.numel() * 4 for t in self.ks) * 2
        return n

    def kv_pool_capacity_tokens(self) -> int:
        return self.num_blocks * self.block_size

    def weight_bytes(self) -> int:
        n = self.tok.numel() * self.tok.element_size()
        for l in self.layers:
            n += sum(l[k].nbytes() for k in ("qkv", "wo", "gate_up", "down"))
        return n

    # ------------------------------------------------------------------ building blocks
    def _allreduce(self, x):
        if self.tp is None or self.tp_world == 1:
            return x
        return self.tp.all_reduce(x)

    def _slots(self, block_table: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """slot = block*bs + offset for (table row, position) pairs; block_table [n, max_blocks]."""
        bs = self.block_size
        blk = torch.gather(block_table, 1, (positions // bs).long()[:, None]).squeeze(1)
        return (blk * bs + positions % bs).to(torch.int32)

    def _append_kv(self, li: int, k, v, slots):
        if self.kv_int8:
            return self._append_kv_i8(li, k, v, slots)
        if self.cuda:
            call("kv_append", k, k.stride(0), v, v.stride(0), slots, self.kc[li], self.vc[li],
                 k.shape[0], self.hk, self.hd, self.block_size, stream_ptr())
        else:
            s = slots.long()
            blk, off = s // self.block_size, s % self.block_size
            self.kc[li][blk, :, off] = k.reshape(-1, self.hk, self.hd)
            self.vc[li][blk, :, off] = v.reshape(-1, self.hk, self.hd)

    def _append_kv_i8(self, li: int, k, v, slots):
        """Row scale = min(absmax(row), ceiling) / 127 (crates/model/src/kvcalib.rs:42-160 gives the
        ceilings; crates/qwen3/src/serve.rs:1262-1288 the append)."""
        clip = self.kv_clip[li] if self.kv_clip is not None else None
        if self.cuda:
            call("kv_append_i8", k, k.stride(0), v, v.stride(0), slots, self.kc[li], self.vc[li],
                 self.ks[li], self.vs[li], clip, k.shape[0], self.hk, self.hd, self.block_size, stream_ptr())
            return
        s = slots.long()
        blk, off = s // self.block_size, s % self.block_size
        for which, (x, pool, sc) in enumerate(((k, self.kc[li], self.ks[li]), (v, self.vc[li], self.vs[li]))):
            x = x.reshape(-1, self.hk, self.hd).float()
            amax = x.abs().amax(-1)
            if clip is not None:
                amax = torch.minimum(amax, clip[which][None, :])
            scale = amax / 127.0
            inv = torch.where(scale > 0, 1.0 / scale, torch.zeros_like(scale))
            pool[blk, :, off] = torch.clamp(torch.round(x * inv[..., None]), -127, 127).to(torch.int8)
            sc[blk, :, off] = scale

    def _gather_kv(self, li: int, block_table: torch.Tensor, S: int):
        if self.kv_int8:
            if self.cuda:
                ok = torch.empty(S, self.hk * self.hd, device=self.device, dtype=self.dtype)
                ov = torch.empty_like(ok)
                call("kv_gather_i8", self.kc[li], self.vc[li], self.ks[li], self.vs[li], block_table, ok, ov,
                     S, self.hk, self.hd, self.block_size, stream_ptr())
                return ok, ov
            t = torch.arange(S, device=self.device)
            blk = block_table[(t // self.block_size).long()].long()
            off = t % self.block_size
            kk = self.kc[li][blk, :, off].float() * self.ks[li][blk, :, off][..., None]
            vv = self.vc[li][blk, :, off].float() * self.vs[li][blk, :, off][..., None]
            return kk.reshape(S, -1).to(self.dtype), vv.reshape(S, -1).to(self.dtype)
        if self.cuda:
            ok = torch.empty(S, self.hk * self.hd, device=self.device, dtype=self.dtype)
            ov = torch.empty_like(ok)
            call("kv_gather", self.kc[li], self.vc[li], block_table, ok, ov, S, self.hk, self.hd,
                 self.block_size, stream_ptr())
            return ok, ov
        t = torch.arange(S, device=self.device)
        blk = block_table[(t // self.block_size).long()].long()
        off = t % self.block_size
        return (self.kc[li][blk, :, off].reshape(S, -1), self.vc[li][blk, :, off].reshape(S, -1))

    def _splits(self, B: int) -> int:
        """KV splits of the decode attention: enough CTAs to fill the machine (B * hk * splits >= ~4
        per SM)."""
        if self.decode_splits > 0:
            return self.decode_splits
        return max(1, min(16, (4 * 148 + B * self.hk - 1) // (B * self.hk)))

    def _paged_attention(self, li: int, q, block_tables, seqlens, out=None):
        """One query row per sequence against its pages; ``q`` (and ``out`` when given) may be row
        slices of wider buffers."""
        B = q.shape[0]
        hq, hk, hd = self.hq, self.hk, self.hd
        scale = 1.0 / math.sqrt(hd)
        if self.cuda:
            splits = self._splits(B)
            if out is None:
                out = torch.empty(B, hq * hd, device=self.device, dtype=self.dtype)
            part_o = torch.empty(B * hq * splits * hd, device=self.device, dtype=torch.float32)
            part_ml = torch.empty(B * hq * splits * 2, device=self.device, dtype=torch.float32)
            if self.kv_int8:
                call("paged_decode_i8", q, q.stride(0), self.kc[li], self.vc[li], self.ks[li], self.vs[li],
                     block_tables, block_tables.shape[1], seqlens, out, out.stride(0), part_o, part_ml,
                     B, hq, hk, hd, self.block_size, splits, float(scale), stream_ptr())
            else:
                call("paged_decode", q, q.stride(0), self.kc[li], self.vc[li], block_tables,
                     block_tables.shape[1], seqlens, out, out.stride(0), part_o, part_ml, B, hq, hk, hd,
                     self.block_size, splits, float(scale), stream_ptr())
            return out
        outs = []
        for b in range(B):
            S = int(seqlens[b])
            kk, vv = self._gather_kv(li, block_tables[b], S)
            o = ref.attention(q[b].reshape(1, 1, hq, hd), kk.reshape(1, S, hk, hd),
                              vv.reshape(1, S, hk, hd), causal=False, scale=scale)
            outs.append(o.reshape(1, hq * hd))
        return torch.cat(outs)

    def _layer(self, li: int, x, delta, pos, attn_fn):
        l = self.layers[li]
        eps = self.cfg.rms_eps
        hq, hk, hd = self.hq, self.hk, self.hd
        if delta is None:
            h = F.rmsnorm(x, l["ln1"], eps)
        else:
            h, x = F.rmsnorm(delta, l["ln1"], eps, residual=x)
        qkv = l["qkv"](h)
        qk = F.qknorm_rope(qkv, l["q_norm"], l["k_norm"], self.cos, self.sin, pos, hq, hk, hd, eps)
        v = qkv[:, (hq + hk) * hd:]
        o = attn_fn(li, qk[:, : hq * hd], qk[:, hq * hd:], v)
        a = self._allreduce(l["wo"](o))
        h2, x = F.rmsnorm(a, l["ln2"], eps, residual=x)
        m = self._allreduce(l["down"](F.swiglu(l["gate_up"](h2))))
        return x, m

    def _head(self, x, delta, greedy: bool):
        """LM head over rows of the residual stream ``x`` + pending MLP output ``delta``; with
        ``delta`` None, ``x`` is already the final-normed hidden state (native path)."""
        if delta is None:
            return self._head_normed(x, greedy)
        h, _ = F.rmsnorm(delta, self.norm, self.cfg.rms_eps, residual=x)
        return self._head_normed(h, greedy)

    def _head_normed(self, h, greedy: bool):
        logits = self.head(h)
        if greedy:
            return F.argmax_rows(logits), None
        k = min(self.topk_capacity, logits.shape[-1])
        idx, vals = F.topk_rows(logits, k)
        return idx[:, 0].to(torch.int32), (idx, vals)

    def _prefill_forward(self, tokens: np.ndarray, start: int, block_table: np.ndarray):
        """Positions [start, start+n) of one sequence through every layer (K/V appended to its pages);
        returns the residual stream and the last layer's MLP output, both [n, d]."""
        if self.fault_hook is not None:
            self.fault_hook("prefill")
        n = int(tokens.shape[0])
        dev = self.device
        tok = torch.from_numpy(np.ascontiguousarray(tokens)).to(dev)
        bt = torch.from_numpy(np.ascontiguousarray(block_table)).to(dev)
        pos = torch.arange(start, start + n, device=dev, dtype=torch.int32)
        slots = self._slots(bt[None, :].expand(n, -1), pos)
        S = start + n
        hq, hk, hd = self.hq, self.hk, self.hd
        if self.native is not None:
            return self._native_prefill(tok, pos, slots, [(0, n, start, bt)])

        paged = self._paged_prefill_meta([(0, n, start, bt)], n) if self._paged_prefill_ok() else None

        def attn(li, q, k, v):
            self._append_kv(li, k, v, slots)
            if paged is not None:
                return self._paged_prefill_attention(li, q, torch.empty(n, hq * hd, device=q.device, dtype=q.dtype), paged)
            if start == 0:
                return flash_attention(q, k, v, 1, n, hq, hk, hd, causal=True)
            kk, vv = self._gather_kv(li, bt, S)
            return flash_attention(q, kk, vv, 1, n, hq, hk, hd, causal=True, S=S)

        x = F.embedding(tok, self.tok).reshape(n, -1)
        delta = None
        for li in range(len(self.layers)):
            x, delta = self._layer(li, x, delta, pos, attn)
        self.steps += 1
        return x, delta

    # ------------------------------------------------------------------ paged flash prefill
    def _paged_prefill_ok(self) -> bool:
        return (self.cuda and not self.kv_int8 and self.block_size in (16, 32, 64, 128) and self.hd in (64, 128)
                and os.environ.get("BRAIN_SERVE_PAGED_PREFILL", "1") == "1")

    def _paged_prefill_meta(self, seqs, n):
        """Device tables for ONE attention launch over all sequences of a packed prefill: ``seqs`` is
        (row offset, rows, start, block table) per sequence with contiguous row ranges."""
        dev = self.device
        row0 = np.array([o for o, _, _, _ in seqs] + [n], dtype=np.int32)
        ctx = np.array([st + l for _, l, st, _ in seqs], dtype=np.int32)
        tiles = [(i, qt) for i, (_, l, _, _) in enumerate(seqs) for qt in range(-(-l // 128))]
        # tiles that see the most keys first, so the tail of the launch is short tiles
        tiles.sort(key=lambda t: -(int(ctx[t[0]]) - seqs[t[0]][1] + min(seqs[t[0]][1], (t[1] + 1) * 128)))
        meta = np.concatenate([row0, ctx, np.array([t[0] for t in tiles], dtype=np.int32),
                               np.array([t[1] for t in tiles], dtype=np.int32)])
        m = torch.from_numpy(meta).to(dev)
        ns, nt = len(seqs), len(tiles)
        tables = torch.stack([bt.to(torch.int32) for _, _, _, bt in seqs]).contiguous()
        return dict(row0=m[:ns + 1], ctx=m[ns + 1:2 * ns + 1], tile_seq=m[2 * ns + 1:2 * ns + 1 + nt],
                    tile_qt=m[2 * ns + 1 + nt:], n_tiles=nt, tables=tables, rows=n)

    def _paged_prefill_attention(self, li, q, out, meta):
        """out[rows] = causal attention of the packed query rows against the paged pool of layer
        ``li`` (the rows' own K/V were appended before): one launch, keys read through the block tables."""
        call("flash_fwd_paged", q, q.stride(0), self.kc[li], self.vc[li], out, out.stride(0), meta["tables"],
             int(meta["tables"].shape[1]), self.block_size, int(self.kc[li].shape[0]), meta["row0"], meta["ctx"],
             meta["tile_seq"], meta["tile_qt"], meta["n_tiles"], meta["rows"], self.hq, self.hk, self.hd,
             float(self.hd ** -0.5), stream_ptr())
        return out

    def _native_prefill(self, tok, pos, slots, seqs, dec=None):
        """Packed rows through the native layer halves; ``seqs``: (row offset, rows, start, block
        table) per sequence, attention per sequence in between.  ``dec`` = (row offset, rows, block
        tables, lengths) adds one decode row per running sequence, attended by the paged kernel.
        Returns (normed hidden [n, d], None): the final RMSNorm is already applied."""
        nat = self.native
        n = int(tok.shape[0])
        hq, hk, hd = self.hq, self.hk, self.hd
        sc = nat.scratch(-(-n // 256) * 256, 1, key="prefill")
        nat.begin(sc, tok.to(torch.int32), n)
        qw = hq * hd
        lse = torch.empty(hq * max([l for _, l, _, _ in seqs] or [1]), device=self.device, dtype=torch.float32)
        n_prompt = sum(l for _, l, _, _ in seqs)
        paged = self._paged_prefill_meta(seqs, n_prompt) if (seqs and self._paged_prefill_ok()) else None
        for li in range(len(self.layers)):
            nat.pre_attn(sc, li, pos, slots, n)
            if paged is not None:
                self._paged_prefill_attention(li, sc.qk[:n_prompt, :qw], sc.o[:n_prompt], paged)
            for o, l, start, bt in (seqs if paged is None else ()):
                q = sc.qk[o:o + l, :qw]
                out = sc.o[o:o + l]
                if start == 0:
                    flash_attention_into(out, q, sc.qk[o:o + l, qw:], sc.qkv[o:o + l, qw + hk * hd:], 1, l, hq, hk, hd,
                                         True, lse=lse)
                else:
                    kk, vv = self._gather_kv(li, bt, start + l)
                    flash_attention_into(out, q, kk, vv, 1, l, hq, hk, hd, True, S=start + l, lse=lse)
            if dec is not None:
                o, l, dbts, dlens = dec
                self._paged_attention(li, sc.qk[o:o + l, :qw], dbts, dlens, out=sc.o[o:o + l])
            nat.post_attn(sc, li, n)
        self.steps += 1
        return nat.finish(sc, n), None

    @torch.no_grad()
    def verify_chunk(self, tokens: np.ndarray, start: int, block_table: np.ndarray) -> np.ndarray:
        """Greedy next-token prediction after EVERY row of a chunk (the verification forward of
        speculative decoding, crates/qwen3/src/serve.rs:1899-1975): row i sees positions
        [0, start+i] and the chunk's K/V are appended to the pages."""
        x, delta = self._prefill_forward(np.asarray(tokens, dtype=np.int32), start, block_table)
        t, _ = self._head(x, delta, True)
        return t.cpu().numpy().astype(np.int64)

    # ------------------------------------------------------------------ PagedDecoder interface
    @torch.no_grad()
    def check_device(self) -> None:
        """Raise if a kernel of the step just read back reported a bounded-wait timeout (the
        scheduler calls this once per step, after the token read-back, before it commits)."""
        if self.device.type == "cuda":
            _cuda.check_error()

    def prefill_chunk(self, tokens: np.ndarray, start: int, block_table: np.ndarray, last: bool,
                      greedy: bool = True):
        """Process prompt positions [start, start+n) of one sequence.  Returns (first token, top-k
        candidates) when ``last`` (else (None, None))."""
        t0 = time.perf_counter()
        try:
            x, delta = self._prefill_forward(tokens, start, block_table)
            if not last:
                return None, None
            t, tk = self._head(x[-1:], delta[-1:] if delta is not None else None, greedy)
            first = int(t.cpu()[0])
            if tk is None:
                return first, None
            idx, vals = tk[0].cpu()[0].tolist(), tk[1].cpu()[0].tolist()
            return first, list(zip(idx, vals))
        finally:
            a = self.acct
            a["prefill_s"] += time.perf_counter() - t0
            a["prefill_calls"] += 1
            a["prefill_seqs"] += 1
            a["prefill_tokens"] += int(tokens.shape[0])

    @torch.no_grad()
    def prefill_batch(self, items):
        """Several prefill chunks in ONE packed forward: ``items`` is a list of (tokens, start,
        block_table, last, greedy).  Norms, projections, RoPE, KV append and the MLP run once over
        the concatenated rows; only attention runs per sequence (on its row slice).  Returns one
        (first token, top-k candidates) pair per item (``(None, None)`` for non-final chunks)."""
        if len(items) == 1:
            t, st, bt, last, greedy = items[0]
            return [self.prefill_chunk(t, st, bt, last, greedy)]
        if self.fault_hook is not None:
            self.fault_hook("prefill")
        t0 = time.perf_counter()
        dev = self.device
        lens = [int(it[0].shape[0]) for it in items]
        offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        n = int(offs[-1])
        tok = torch.from_numpy(np.ascontiguousarray(np.concatenate([np.asarray(it[0], dtype=np.int32) for it in items]))).to(dev)
        pos_np = np.concatenate([np.arange(it[1], it[1] + l, dtype=np.int32) for it, l in zip(items, lens)])
        pos = torch.from_numpy(pos_np).to(dev)
        bts = [torch.from_numpy(np.ascontiguousarray(it[2])).to(dev) for it in items]
        slots = torch.cat([self._slots(bt[None, :].expand(l, -1), pos[o:o + l])
                           for bt, l, o in zip(bts, lens, offs[:-1].tolist())])
        hq, hk, hd = self.hq, self.hk, self.hd
        if self.native is not None:
            x, delta = self._native_prefill(tok, pos, slots, [(o, l, it[1], bt) for it, bt, l, o in
                                                              zip(items, bts, lens, offs[:-1].tolist())])
            return self._prefill_batch_results(items, offs, x, delta, n, t0)

        paged = None
        if self._paged_prefill_ok():
            paged = self._paged_prefill_meta([(o, l, it[1], bt) for it, bt, l, o in
                                              zip(items, bts, lens, offs[:-1].tolist())], n)

        def attn(li, q, k, v):
            self._append_kv(li, k, v, slots)
            if paged is not None:
                return self._paged_prefill_attention(li, q, torch.empty(n, hq * hd, device=q.device, dtype=q.dtype), paged)
            outs = []
            for (t_, start, _, _, _), bt, l, o in zip(items, bts, lens, offs[:-1].tolist()):
                qs = q[o:o + l]
                if start == 0:
                    outs.append(flash_attention(qs, k[o:o + l], v[o:o + l], 1, l, hq, hk, hd, causal=True))
                else:
                    kk, vv = self._gather_kv(li, bt, start + l)
                    outs.append(flash_attention(qs, kk, vv, 1, l, hq, hk, hd, causal=True, S=start + l))
            return torch.cat(outs)

        x = F.embedding(tok, self.tok).reshape(n, -1)
        delta = None
        for li in range(len(self.layers)):
            x, delta = self._layer(li, x, delta, pos, attn)
        self.steps += 1
        return self._prefill_batch_results(items, offs, x, delta, n, t0)

    def _prefill_batch_results(self, items, offs, x, delta, n, t0):
        dev = self.device
        a = self.acct
        final = [i for i, it in enumerate(items) if it[3]]
        results = [(None, None)] * len(items)
        if not final:
            a["prefill_s"] += time.perf_counter() - t0
            a["prefill_calls"] += 1
            a["prefill_seqs"] += len(items)
            a["prefill_tokens"] += n
            return results
        rows = torch.tensor([int(offs[i + 1]) - 1 for i in final], device=dev, dtype=torch.long)
        all_greedy = all(items[i][4] for i in final)
        t, tk = self._head(x[rows], delta[rows] if delta is not None else None, all_greedy)
        firsts = t.cpu().tolist()
        if tk is not None:
            idx, vals = tk[0].cpu().tolist(), tk[1].cpu().tolist()
        for j, i in enumerate(final):
            cand = list(zip(idx[j], vals[j])) if tk is not None else None
            results[i] = (int(firsts[j]), cand)
        a["prefill_s"] += time.perf_counter() - t0
        a["prefill_calls"] += 1
        a["prefill_seqs"] += len(items)
        a["prefill_tokens"] += n
        return results

    @torch.no_grad()
    def mixed_step(self, items, tokens: np.ndarray, positions: np.ndarray, block_tables: np.ndarray,
                   greedy: bool = True):
        """Prefill chunks AND one decode row per running sequence in ONE packed forward: the
        projections, norms, MLP and (under tensor parallelism) the two all-reduces per layer run
        once over the concatenated rows, so the decode step rides along with the prompt work instead
        of waiting behind it (the reference interleaves both kinds of work inside one scheduler
        step, crates/qwen3/src/serve.rs:1300-1420).  Attention runs per kind: the flash kernel per
        prefill sequence, the paged kernel over the decode rows.

        ``items`` as for :meth:`prefill_batch`; ``tokens``/``positions``/``block_tables`` as for
        :meth:`decode` with a window of 1.  Returns (prefill results, decode tokens [B][1], per-row
        top-k candidates or None)."""
        if self.fault_hook is not None:
            self.fault_hook("prefill")
            self.fault_hook("decode")
        t0 = time.perf_counter()
        dev = self.device
        B = int(tokens.shape[0])
        lens = [int(it[0].shape[0]) for it in items]
        offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        n_pre = int(offs[-1])
        n = n_pre + B
        tok_np = np.concatenate([np.asarray(it[0], dtype=np.int32) for it in items]
                                + [np.asarray(tokens, dtype=np.int32)])
        pos_np = np.concatenate([np.arange(it[1], it[1] + l, dtype=np.int32) for it, l in zip(items, lens)]
                                + [np.asarray(positions, dtype=np.int32)])
        tok = torch.from_numpy(np.ascontiguousarray(tok_np)).to(dev)
        pos = torch.from_numpy(np.ascontiguousarray(pos_np)).to(dev)
        bts = [torch.from_numpy(np.ascontiguousarray(it[2])).to(dev) for it in items]
        dbts = torch.from_numpy(np.ascontiguousarray(block_tables)).to(dev)
        dpos = pos[n_pre:]
        dlens = (dpos + 1).to(torch.int32)
        slots = torch.cat([self._slots(bt[None, :].expand(l, -1), pos[o:o + l])
                           for bt, l, o in zip(bts, lens, offs[:-1].tolist())] + [self._slots(dbts, dpos)])
        hq, hk, hd = self.hq, self.hk, self.hd
        seqs = [(o, l, it[1], bt) for it, bt, l, o in zip(items, bts, lens, offs[:-1].tolist())]
        if self.native is not None:
            x, delta = self._native_prefill(tok, pos, slots, seqs, dec=(n_pre, B, dbts, dlens))
        else:
            def attn(li, q, k, v):
                self._append_kv(li, k, v, slots)
                outs = []
                for o, l, start, bt in seqs:
                    qs = q[o:o + l]
                    if start == 0:
                        outs.append(flash_attention(qs, k[o:o + l], v[o:o + l], 1, l, hq, hk, hd, causal=True))
                    else:
                        kk, vv = self._gather_kv(li, bt, start + l)
                        outs.append(flash_attention(qs, kk, vv, 1, l, hq, hk, hd, causal=True, S=start + l))
                outs.append(self._paged_attention(li, q[n_pre:], dbts, dlens))
                return torch.cat(outs)

            x = F.embedding(tok, self.tok).reshape(n, -1)
            delta = None
            for li in range(len(self.layers)):
                x, delta = self._layer(li, x, delta, pos, attn)
            self.steps += 1
        # one head call over the rows that sample: last row of each finishing prompt + decode rows
        final = [i for i, it in enumerate(items) if it[3]]
        rows = torch.tensor([int(offs[i + 1]) - 1 for i in final] + list(range(n_pre, n)), device=dev,
                            dtype=torch.long)
        t, tk = self._head(x[rows], delta[rows] if delta is not None else None, greedy)
        picked = t.cpu().tolist()
        cands = None
        if tk is not None:
            idx, vals = tk[0].cpu().tolist(), tk[1].cpu().tolist()
            cands = [list(zip(i, v)) for i, v in zip(idx, vals)]
        results = [(None, None)] * len(items)
        for j, i in enumerate(final):
            results[i] = (int(picked[j]), cands[j] if cands is not None else None)
        nf = len(final)
        a = self.acct
        a["mixed_s"] += time.perf_counter() - t0
        a["mixed_calls"] += 1
        a["prefill_seqs"] += len(items)
        a["prefill_tokens"] += n_pre
        a["decode_rows"] += B
        return results, [[int(p)] for p in picked[nf:]], (cands[nf:] if cands is not None else None)

    @torch.no_grad()
    def decode(self, tokens: np.ndarray, positions: np.ndarray, block_tables: np.ndarray,
               window: int = 1, greedy: bool = True):
        """One batched decode call: ``window`` on-device greedy steps (window > 1 requires greedy).
        Returns (tokens [B][window], per-row top-k candidate lists or None)."""
        if self.fault_hook is not None:
            self.fault_hook("decode")
        dev = self.device
        B = int(tokens.shape[0])
        t0 = time.perf_counter()
        try:
            return self._decode(tokens, positions, block_tables, window, greedy)
        finally:
            a = self.acct
            a["decode_s"] += time.perf_counter() - t0
            a["decode_calls"] += 1
            a["decode_rows"] += B * window

    def _decode(self, tokens, positions, block_tables, window, greedy):
        dev = self.device
        if self.cuda_graphs and (greedy or window > 1):
            out = self._decode_graphed(tokens, positions, block_tables, window)
            return [row.tolist() for row in out], None
        tok = torch.from_numpy(np.ascontiguousarray(tokens)).to(dev)
        pos = torch.from_numpy(np.ascontiguousarray(positions)).to(dev)
        bts = torch.from_numpy(np.ascontiguousarray(block_tables)).to(dev)
        out_t, topks = self._decode_steps(tok, pos, bts, window, greedy or window > 1)
        out = out_t.cpu().numpy()
        cand = None
        if topks is not None:
            idx, vals = topks[0].cpu().tolist(), topks[1].cpu().tolist()
            cand = [list(zip(i, v)) for i, v in zip(idx, vals)]
        return [row.tolist() for row in out], cand

    def _decode_steps(self, tok, pos, bts, window: int, greedy: bool):
        """``window`` decode steps on device tensors -> (tokens [B, window], last top-k or None)."""
        B = tok.shape[0]
        outs = []
        topks = None
        if self.native is not None:
            nat = self.native
            sc = nat.scratch(B, self._splits(B), key=("decode", B))
            tok = tok.to(torch.int32)
            for w in range(window):
                slots = self._slots(bts, pos)
                seqlens = (pos + 1).to(torch.int32)
                hn = nat.decode(sc, tok, pos, slots, bts, seqlens, B)
                t, tk = self._head_normed(hn, greedy)
                outs.append(t)
                if tk is not None:
                    topks = tk
                tok = t
                pos = pos + 1
                self.steps += 1
            return torch.stack(outs, dim=1), topks
        for w in range(window):
            slots = self._slots(bts, pos)
            seqlens = (pos + 1).to(torch.int32)

            def attn(li, q, k, v):
                self._append_kv(li, k, v, slots)
                return self._paged_attention(li, q, bts, seqlens)

            x = F.embedding(tok, self.tok).reshape(B, -1)
            delta = None
            for li in range(len(self.layers)):
                x, delta = self._layer(li, x, delta, pos, attn)
            t, tk = self._head(x, delta, greedy)
            outs.append(t)
            if tk is not None:
                topks = tk
            tok = t
            pos = pos + 1
            self.steps += 1
        return torch.stack(outs, dim=1), topks

    # ---- CUDA-graph decode: one captured graph per (padded batch, window)
    @staticmethod
    def _bucket(b: int) -> int:
        for cap in (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 160, 192, 224, 256):
            if b <= cap:
                return cap
        return -(-b // 64) * 64

    def _decode_graphed(self, tokens, positions, block_tables, window: int):
        """Greedy decode through a replayed CUDA graph.  The batch is padded to a bucket size with
        rows that sit at position 0 of the dummy block; inputs travel through pinned staging."""
        B = int(tokens.shape[0])
        Bp = self._bucket(B)
        key = (Bp, window)
        g = self._graphs.get(key)
        if g is None:
            g = self._capture(Bp, window)
            self._graphs[key] = g
        h_tok, h_pos, h_bts = g["h_tok"], g["h_pos"], g["h_bts"]
        h_tok[:B] = torch.from_numpy(np.ascontiguousarray(tokens, dtype=np.int32))
        h_pos[:B] = torch.from_numpy(np.ascontiguousarray(positions, dtype=np.int32))
        h_bts[:B] = torch.from_numpy(np.ascontiguousarray(block_tables, dtype=np.int32))
        if Bp > B:
            h_tok[B:] = 0
            h_pos[B:] = 0
            h_bts[B:] = self.dummy_block
        g["tok"].copy_(h_tok, non_blocking=True)
        g["pos"].copy_(h_pos, non_blocking=True)
        g["bts"].copy_(h_bts, non_blocking=True)
        g["graph"].replay()
        self.graph_replays += 1
        self.steps += window
        g["h_out"].copy_(g["out"], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return g["h_out"][:B].numpy().copy()

    def _capture(self, Bp: int, window: int):
        dev = self.device
        mb = self.max_blocks
        g = {"tok": torch.zeros(Bp, device=dev, dtype=torch.int32),
             "pos": torch.zeros(Bp, device=dev, dtype=torch.int32),
             "bts": torch.full((Bp, mb), self.dummy_block, device=dev, dtype=torch.int32),
             "h_tok": torch.zeros(Bp, dtype=torch.int32).pin_memory(),
             "h_pos": torch.zeros(Bp, dtype=torch.int32).pin_memory(),
             "h_bts": torch.zeros(Bp, mb, dtype=torch.int32).pin_memory(),
             "h_out": torch.zeros(Bp, window, dtype=torch.int32).pin_memory()}
        steps0 = self.steps
        # warm-up on a side stream (lazy one-time setup such as kernel attributes and symmetric
        # buffers must not happen during capture), then capture the same work
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._decode_steps(g["tok"], g["pos"], g["bts"], window, True)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: other threads of the process (e.g. a process group's watchdog)
        # keep making CUDA calls of their own while this thread captures
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            out, _ = self._decode_steps(g["tok"], g["pos"], g["bts"], window, True)
        g["graph"], g["out"] = graph, out
        self.steps = steps0
        return g

    # ------------------------------------------------------------------ convenience
    @torch.no_grad()
    def logits_all(self, tokens: List[int]) -> torch.Tensor:
        """Contiguous (non-paged) forward over a whole prompt: [T, vocab] — the oracle the paged
        path is checked against."""
        n = len(tokens)
        dev = self.device
        tok = torch.tensor(tokens, device=dev, dtype=torch.int32)
        pos = torch.arange(n, device=dev, dtype=torch.int32)
        hq, hk, hd = self.hq, self.hk, self.hd

        def attn(li, q, k, v):
            return flash_attention(q, k, v, 1, n, hq, hk, hd, causal=True)

        x = F.embedding(tok, self.tok).reshape(n, -1)
        delta = None
        for li in range(len(self.layers)):
            x, delta = self._layer(li, x, delta, pos, attn)
        h, _ = F.rmsnorm(delta, self.norm, self.cfg.rms_eps, residual=x)
        return self.head(h).float()
