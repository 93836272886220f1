"""Next-token sampling as Python sees it: the host library's chain (``sampling/sampler.cpp``) behind two classes.

Chain: repetition / presence penalty over the last ``repeat_last_n`` accepted tokens -> top-k -> top-p -> min-p ->
temperature -> one draw; ``temperature <= 0`` (or ``top_k == 1``) is greedy, the lowest id winning ties.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import numpy as np

from .. import native


@dataclass
class SamplerParams:
    temperature: float = 0.8       # <= 0: greedy
    top_k: int = 40                # keep the k most likely tokens; <= 0: off
    top_p: float = 0.95            # smallest set with cumulative probability >= top_p; >= 1: off
    min_p: float = 0.05            # keep tokens with p >= min_p * p_max; <= 0: off
    repeat_penalty: float = 1.0    # positive logits / r, negative * r, for recent tokens; 1: off
    repeat_last_n: int = 64        # how many accepted tokens the penalty looks back over
    seed: int = 0
    presence_penalty: float = 0.0  # subtracted from the logit of each recent token, after repeat_penalty

    @staticmethod
    def greedy() -> "SamplerParams":
        return SamplerParams(temperature=0.0)

    @staticmethod
    def pure_temperature(temperature: float, seed: int = 0) -> "SamplerParams":
        return SamplerParams(temperature=temperature, top_k=0, top_p=1.0, min_p=0.0, seed=seed)

    def to_c(self) -> native.SamplerParamsC:
        return native.SamplerParamsC(self.temperature, self.top_k, self.top_p, self.min_p, self.repeat_penalty,
                                     self.repeat_last_n, self.seed, self.presence_penalty)

    @staticmethod
    def defaults() -> "SamplerParams":
        c = native.lib().sampler_default_params()
        return SamplerParams(c.temperature, c.top_k, c.top_p, c.min_p, c.repeat_penalty, c.repeat_last_n, c.seed,
                             c.presence_penalty)


class Sampler:
    """The chain on the host over one row of float32 logits."""

    def __init__(self, params: Optional[SamplerParams] = None):
        self.params = params or SamplerParams()
        c = self.params.to_c()
        self._h = native.lib().sampler_create(ctypes.byref(c))

    def sample(self, logits) -> int:
        """Pick the next token from float32 logits [vocab].  Does not record it; see :meth:`accept`."""
        row = np.ascontiguousarray(np.asarray(logits, dtype=np.float32))
        return native.lib().sampler_sample(self._h, row.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), int(row.size))

    def histogram(self, logits, draws: int) -> np.ndarray:
        """How often each token comes out of ``draws`` draws from one row (none of them accepted)."""
        row = np.ascontiguousarray(np.asarray(logits, dtype=np.float32))
        counts = np.zeros(row.size, dtype=np.int64)
        native.check(native.lib().qe_sampler_histogram(self._h, row.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), int(row.size),
                                                       int(draws), counts.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong))))
        return counts

    def device_mode(self) -> Optional[str]:
        """"greedy", "temperature" or "chain" (top-k on, at most ``chain_max_k()``) when a device kernel gives the same
        result as the chain on the host, else None (penalties, top-p or min-p without top-k)."""
        return native.lib().qe_sampler_device_mode(self._h).decode() or None

    def uniform(self) -> float:
        """The generator's next uniform number in [0, 1) (what sampling one token draws)."""
        return native.lib().qe_sampler_uniform(self._h)

    def chain_record(self) -> bytes:
        """The 24-byte record (uniform, top_p, log(min_p) or -inf, temperature, top_k) the device's chain kernel takes
        for this sampler's next token; draws the token's uniform number."""
        buf = ctypes.create_string_buffer(24)
        native.lib().qe_sampler_chain_record(self._h, buf)
        return buf.raw

    @staticmethod
    def chain_max_k() -> int:
        return native.lib().qe_sampler_chain_max_k()

    def accept(self, token: int) -> None:
        native.lib().sampler_accept(self._h, int(token))

    def reset(self) -> None:
        native.lib().sampler_reset(self._h)

    def __del__(self):
        try:
            native.lib().sampler_free(self._h)
        except Exception:
            pass


__all__ = ["Sampler", "SamplerParams"]
