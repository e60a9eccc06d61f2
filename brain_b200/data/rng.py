"""SplitMix64 stream, bit-compatible with the reference's dataset RNG
(crates/data/src/rng.rs:14-80): same seeding offset, same mixing constants, same derived draws
(``next_f64`` from the top 53 bits, inclusive integer ranges by modulo, Box-Muller gaussian).
The state is a plain integer so it can be handed to the native batch sampler and back."""
from __future__ import annotations

import ctypes
import math

import numpy as np

from .. import _host

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


class Rng:
    def __init__(self, seed: int):
        self.state = (int(seed) + _GOLDEN) & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + _GOLDEN) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def next_f64(self) -> float:
        return (self.next_u64() >> 11) / float(1 << 53)

    def next_f32(self) -> float:
        return float(np.float32(self.next_f64()))

    def gen_range_inclusive(self, lo: int, hi: int) -> int:
        return lo + self.next_u64() % (hi - lo + 1)

    def uniform(self, lo: float, hi: float) -> float:
        return lo + (hi - lo) * self.next_f64()

    def choice(self, items):
        return items[self.gen_range_inclusive(0, len(items) - 1)]

    def next_gaussian(self) -> float:
        u1 = max(self.next_f64(), 1e-12)
        u2 = self.next_f64()
        return math.sqrt(-2.0 * math.log(u1)) * math.cos(math.tau * u2)

    # bulk draws run in the native runtime -------------------------------------------------
    def tokens(self, n: int, vocab: int) -> np.ndarray:
        """``n`` uniform token ids in [0, vocab) as int32 (one ``gen_range_inclusive`` each)."""
        out = np.empty(n, dtype=np.int32)
        st = ctypes.c_uint64(self.state)
        _host.lib().bbh_rng_fill_tokens(ctypes.byref(st), out.ctypes.data, n, vocab)
        self.state = st.value
        return out

    def u64s(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.uint64)
        st = ctypes.c_uint64(self.state)
        _host.lib().bbh_rng_fill_u64(ctypes.byref(st), out.ctypes.data, n)
        self.state = st.value
        return out


class Lcg:
    """Knuth-MMIX LCG used for deterministic fixtures (crates/data/src/rng.rs, ``Lcg``)."""

    def __init__(self, seed: int):
        self.state = int(seed) & _MASK

    def next_u64(self) -> int:
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) & _MASK
        return self.state

    def next_u32(self) -> int:
        return self.next_u64() >> 32

    def unit(self) -> float:
        return float(np.float32(np.float32(self.next_u32()) / np.float32(1 << 32)))

    def signed(self) -> float:
        return float(np.float32(np.float32(self.next_u32()) / np.float32(1 << 31)) - np.float32(1.0))

    def scaled(self, a: float) -> float:
        return self.signed() * a

    def vec(self, n: int):
        return [self.signed() for _ in range(n)]
