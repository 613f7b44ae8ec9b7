"""java.util.Random (the documented 48-bit linear congruential generator), so that the seeds the
reference's tests name produce the byte blocks and floats those tests see."""
import numpy as np

_MULT = 0x5DEECE66D
_MASK = (1 << 48) - 1


class JavaRandom:
    def __init__(self, seed: int):
        self.seed = (seed ^ _MULT) & _MASK

    def _next(self, bits: int) -> int:
        self.seed = (self.seed * _MULT + 0xB) & _MASK
        v = self.seed >> (48 - bits)
        if bits == 32 and v >= 1 << 31:  # the (int) cast
            v -= 1 << 32
        return v

    def next_int(self) -> int:
        return self._next(32)

    def next_int_bound(self, bound: int) -> int:
        if bound & (-bound) == bound:
            return (bound * (self._next(31) & 0x7FFFFFFF)) >> 31
        while True:
            bits = self._next(31) & 0x7FFFFFFF
            val = bits % bound
            if bits - val + (bound - 1) < (1 << 31):
                return val

    def next_float(self) -> np.float32:
        return np.float32((self._next(24) & 0xFFFFFF) / float(1 << 24))

    def next_bytes(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.uint8)
        i = 0
        while i < n:
            rnd = self.next_int() & 0xFFFFFFFF
            for _ in range(min(n - i, 4)):
                out[i] = rnd & 0xFF
                rnd >>= 8
                i += 1
        return out
