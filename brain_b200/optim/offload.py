"""AdamW with optimiser state offloaded to pinned host memory (reference: the ``OffloadAdam`` path
that ``brain qwen3 finetune`` switches on through ``BRAIN_OFFLOAD_ADAM=1``,
crates/cli/src/qwen_cli.rs:462-471, crates/optim/src/lib.rs).

The device keeps bf16 working weights and the fp32 gradient bucket; fp32 master weights and both
moments (12 bytes per parameter) stay on the host.  A step is: gradient bucket D2H into a pinned
buffer, native multi-threaded AdamW (``bbh_adamw_f32``) that also emits the bf16 rounding, H2D of
the bf16 weights.  Same interface as :class:`optim.adamw.AdamW`."""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from .. import _host
from ..paramstore import ParamStore, Role

_host.register({
    "bbh_sumsq_f32": (ctypes.c_double, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]),
    "bbh_adamw_f32": (None, [ctypes.c_void_p] * 5 + [ctypes.c_int64] + [ctypes.c_float] * 5 +
                      [ctypes.c_int64, ctypes.c_float, ctypes.c_int]),
})


class OffloadAdam:
    def __init__(self, store: ParamStore, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 threads: Optional[int] = None):
        self.store = store
        self.beta1, self.beta2 = betas
        self.eps = eps
        self.rank, self.world = 0, 1
        n = store.n_train
        self.shard_len, self.lo, self.hi = n, 0, n
        pin = store.device.type == "cuda"
        self.master = torch.empty(n, dtype=torch.float32, pin_memory=pin)
        self.master.copy_(store.weights[:n].float())
        self.m = torch.zeros(n, dtype=torch.float32)
        self.v = torch.zeros(n, dtype=torch.float32)
        self.g_host = torch.empty(n, dtype=torch.float32, pin_memory=pin)
        self.w16_host = torch.empty(n, dtype=torch.bfloat16, pin_memory=pin) \
            if store.dtype == torch.bfloat16 else None
        self.t = 0
        self.threads = threads or min(32, os.cpu_count() or 1)
        self.last_grad_norm = None
        self._runs = [(s.offset, s.offset + s.numel, s.decay) for s in store.slots if s.role != Role.FROZEN]

    def host_state_bytes(self) -> int:
        return 4 * 3 * self.shard_len

    def step(self, lr: float, wd: float = 0.0, clip: Optional[float] = None, extra_scale: float = 1.0,
             grads: Optional[torch.Tensor] = None, sumsq=None):
        st = self.store
        g = st.grads if grads is None else grads
        self.g_host.copy_(g[:self.shard_len], non_blocking=False)
        lib = _host.lib()
        self.t += 1
        coef = float(extra_scale)
        if clip is not None and clip > 0:
            norm = float(lib.bbh_sumsq_f32(self.g_host.data_ptr(), self.shard_len, self.threads)) ** 0.5
            norm *= abs(extra_scale)
            self.last_grad_norm = norm
            coef *= min(1.0, clip / (norm + 1e-6))
        for a, b, dec in self._runs:
            n = b - a
            lib.bbh_adamw_f32(self.master[a:].data_ptr(), self.m[a:].data_ptr(), self.v[a:].data_ptr(),
                              self.g_host[a:].data_ptr(),
                              self.w16_host[a:].data_ptr() if self.w16_host is not None else None, n,
                              lr, self.beta1, self.beta2, self.eps, wd if dec else 0.0, self.t, coef,
                              self.threads)
        if self.w16_host is not None:
            st.weights[:self.shard_len].copy_(self.w16_host, non_blocking=True)
        else:
            st.weights[:self.shard_len].copy_(self.master)
