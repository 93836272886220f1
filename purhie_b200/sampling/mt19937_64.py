"""The 64-bit Mersenne Twister (MT19937-64), the generator behind C++'s ``std::mt19937_64``.

The reference seeds ``std::mt19937_64`` with the sampler's seed and draws one uniform number per sampled
token from the top 53 bits (src/sampler.cpp:24-32).  The algorithm and its constants are those of the
published MT19937-64 definition (Matsumoto & Nishimura), so equal seeds give equal draws.
"""
from __future__ import annotations

_NN, _MM = 312, 156
_MATRIX_A = 0xB5026F5AA96619E9
_UPPER, _LOWER = 0xFFFFFFFF80000000, 0x7FFFFFFF
_MASK = 0xFFFFFFFFFFFFFFFF


class MT19937_64:
    def __init__(self, seed: int = 5489):
        self.seed(seed)

    def seed(self, seed: int) -> None:
        mt = [0] * _NN
        mt[0] = seed & _MASK
        for i in range(1, _NN):
            mt[i] = (6364136223846793005 * (mt[i - 1] ^ (mt[i - 1] >> 62)) + i) & _MASK
        self._mt, self._i = mt, _NN

    def _twist(self) -> None:
        mt = self._mt
        for i in range(_NN):
            x = (mt[i] & _UPPER) | (mt[(i + 1) % _NN] & _LOWER)
            mt[i] = mt[(i + _MM) % _NN] ^ (x >> 1) ^ (_MATRIX_A if x & 1 else 0)
        self._i = 0

    def next_u64(self) -> int:
        if self._i >= _NN:
            self._twist()
        x = self._mt[self._i]
        self._i += 1
        x ^= (x >> 29) & 0x5555555555555555
        x ^= (x << 17) & 0x71D67FFFEDA60000
        x ^= (x << 37) & 0xFFF7EEE000000000
        x ^= x >> 43
        return x & _MASK

    def uniform(self) -> float:
        """[0, 1) from the 53 high bits."""
        return (self.next_u64() >> 11) * (1.0 / 9007199254740992.0)

    def snapshot(self):
        """What :meth:`restore` needs to take back the draws made after this point.  Cheap unless the next draw
        regenerates the state."""
        return (self._i, list(self._mt) if self._i >= _NN else None)

    def restore(self, snap) -> None:
        i, mt = snap
        if mt is not None:
            self._mt = mt
        self._i = i
