"""AdamW with global gradient-norm clipping over a ParamStore's flat buffers.

GPU: fp32 master weights and moments (optionally only this rank's shard of them — ZeRO-1), one
fused kernel that applies the clip coefficient, updates master/m/v and writes the bf16 working
weights; the gradient norm is a two-stage deterministic reduction and the clip coefficient stays
on the device (no host sync in the step).  CPU backend: the same arithmetic in one native
multi-threaded pass over the flat buffers (csrc/runtime/host_adam.cpp; no temporaries, where the
PyTorch expression allocates five of the model's size per step); ``BRAIN_CPU_ADAM=torch`` runs the
PyTorch fp32 expression instead.

Reference: crates/optim/src/lib.rs:40-217 (AdamW + clip as a cached dispatch graph),
crates/kernels/wgsl/{adamw,gradnorm_part,clip_coef_wg}.wgsl; coef = min(1, max_norm/(||g||+1e-6))."""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from .. import _host
from ..ops import _cuda, reference as ref
from ..ops._cuda import L, call, stream_ptr
from ..paramstore import ParamStore

_host.register({
    "bbh_sumsq_f32": (ctypes.c_double, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]),
    "bbh_adamw_f32": (None, [ctypes.c_void_p] * 5 + [ctypes.c_int64] + [ctypes.c_float] * 5 +
                      [ctypes.c_int64, ctypes.c_float, ctypes.c_int]),
})


def _native_cpu() -> bool:
    return os.environ.get("BRAIN_CPU_ADAM", "native") != "torch"


def _flat_f32(*ts) -> bool:
    return all(t.dtype == torch.float32 and t.is_contiguous() and t.device.type == "cpu" for t in ts)


class AdamW:
    def __init__(self, store: ParamStore, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 shard: Optional[Tuple[int, int]] = None, group=None):
        self.store = store
        self.beta1, self.beta2 = betas
        self.eps = eps
        self.rank, self.world = shard if shard is not None else (0, 1)
        self.group = group
        n = store.n_train
        assert n % self.world == 0, "ParamStore(pad_to=world) keeps shards equal"
        self.shard_len = n // self.world
        self.lo = self.rank * self.shard_len
        self.hi = self.lo + self.shard_len
        dev = store.device
        self.cuda = dev.type == "cuda"
        if self.cuda or store.dtype != torch.float32:
            self.master = store.weights[self.lo:self.hi].float()
        else:
            self.master = store.weights[self.lo:self.hi]  # fp32 CPU weights are their own master
        self.m = torch.zeros(self.shard_len, device=dev, dtype=torch.float32)
        self.v = torch.zeros(self.shard_len, device=dev, dtype=torch.float32)
        self.t = 0
        if self.cuda:
            self._scratch = torch.empty(1024, device=dev, dtype=torch.float32)
            self._sumsq = torch.zeros(1, device=dev, dtype=torch.float32)
            self._coef = torch.ones(1, device=dev, dtype=torch.float32)
            self._norm = torch.zeros(1, device=dev, dtype=torch.float32)
        self.last_grad_norm = None
        self._runs = self._decay_runs()

    def _decay_runs(self):
        """Contiguous (start, end, decays) runs of this shard; one run when every slot decays."""
        from ..paramstore import Role
        marks = []
        for s in self.store.slots:
            if s.role == Role.FROZEN:
                continue
            a, b = max(s.offset, self.lo), min(s.offset + s.numel, self.hi)
            if a < b:
                marks.append((a, b, s.decay))
        if all(d for _, _, d in marks):
            return [(self.lo, self.hi, True)]
        # slot offsets are multiples of 64, so every run starts 16-byte aligned; the alignment
        # padding after a slot joins the run before it (its gradient is always zero)
        runs = []
        for a, b, d in marks:
            if runs and runs[-1][2] == d:
                runs[-1] = (runs[-1][0], b, d)
            else:
                if runs:
                    runs[-1] = (runs[-1][0], a, runs[-1][2])
                runs.append((a if runs else self.lo, b, d))
        runs[-1] = (runs[-1][0], self.hi, runs[-1][2])
        return runs

    # -------------------------------------------------------------------------------- step
    def grad_sumsq(self, grads: torch.Tensor) -> torch.Tensor:
        """Device scalar: sum of squares of this shard's gradient (all-reduced over the group)."""
        g = grads[self.lo:self.hi] if grads.numel() != self.shard_len else grads
        if self.cuda:
            call("sumsq", g, L(g.numel()), self._scratch, self._sumsq, 0, stream_ptr())
            ss = self._sumsq
        elif _native_cpu() and _flat_f32(g):
            ss = torch.tensor([_host.lib().bbh_sumsq_f32(g.data_ptr(), g.numel(), torch.get_num_threads())],
                              dtype=torch.float32)
        else:
            ss = (g.double() ** 2).sum().float().reshape(1)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(ss, group=self.group)
        return ss

    def step(self, lr: float, wd: float = 0.0, clip: Optional[float] = None, extra_scale: float = 1.0,
             grads: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None):
        """One update of this rank's shard from ``grads`` (default: the store's flat gradient;
        a tensor of shard length is taken as already reduce-scattered)."""
        st = self.store
        grads = st.grads if grads is None else grads
        g = grads[self.lo:self.hi] if grads.numel() != self.shard_len else grads
        self.t += 1
        need_norm = clip is not None and clip > 0
        if self.cuda:
            if need_norm:
                ss = sumsq if sumsq is not None else self.grad_sumsq(g)
                call("clip_coef", ss, float(clip), float(extra_scale), self._coef, self._norm,
                     stream_ptr())
                self.last_grad_norm = self._norm
            else:
                self._coef.fill_(extra_scale)
            w16 = st.weights[self.lo:self.hi] if st.dtype == torch.bfloat16 else None
            for a, b, dec in self._runs:
                o, n = a - self.lo, b - a
                call("adamw", self.master[o:o + n], self.m[o:o + n], self.v[o:o + n], g[o:o + n],
                     w16[o:o + n] if w16 is not None else None, L(n), float(lr), self.beta1,
                     self.beta2, self.eps, float(wd if dec else 0.0), self.t, self._coef,
                     stream_ptr())
            if w16 is None:
                st.weights[self.lo:self.hi].copy_(self.master)
        else:
            coef = extra_scale
            if need_norm:
                ss = sumsq if sumsq is not None else self.grad_sumsq(g)
                norm = float(ss.sqrt())
                self.last_grad_norm = torch.tensor([norm])
                coef = min(1.0, clip / (norm + 1e-6)) * extra_scale
            native = _native_cpu() and _flat_f32(self.master, self.m, self.v, g)
            for a, b, dec in self._runs:
                o, n = a - self.lo, b - a
                if native:
                    _host.lib().bbh_adamw_f32(self.master[o:].data_ptr(), self.m[o:].data_ptr(),
                                              self.v[o:].data_ptr(), g[o:].data_ptr(), None, n, lr, self.beta1,
                                              self.beta2, self.eps, wd if dec else 0.0, self.t, coef,
                                              torch.get_num_threads())
                else:
                    ref.adamw_(self.master[o:o + n], self.m[o:o + n], self.v[o:o + n], g[o:o + n], lr,
                               self.beta1, self.beta2, self.eps, wd if dec else 0.0, self.t, coef)
            if self.master.data_ptr() != st.weights[self.lo:self.hi].data_ptr():
                st.weights[self.lo:self.hi].copy_(self.master.to(st.dtype))

    # -------------------------------------------------------------------------------- state
    def state_dict(self):
        return {"t": self.t, "m": self.m, "v": self.v, "master": self.master,
                "lo": self.lo, "hi": self.hi}

    def load_state_dict(self, sd):
        self.t = int(sd["t"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.master.copy_(sd["master"])
