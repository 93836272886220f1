"""Next-token sampling: the reference's chain, on the host, plus the choice of a device kernel.

Chain (src/sampler.h:1-6, src/sampler.cpp:58-170): repetition / presence penalty over the last
``repeat_last_n`` accepted tokens -> top-k -> top-p -> min-p -> temperature -> one draw.
``temperature <= 0`` (or ``top_k == 1``) is greedy: argmax after the penalty, the lowest id wins ties.
Defaults are the reference's (src/sampler.cpp:181-192).  When only greedy or plain temperature sampling
is asked for, the engine samples with its device kernels instead of copying logits to the host; the
uniform number still comes from this sampler's generator, one per token.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from .mt19937_64 import MT19937_64


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


LOGIT_RANGE = 40.0     # without a filter, tokens more than this below the maximum are not candidates


class Sampler:
    def __init__(self, params: Optional[SamplerParams] = None):
        self.params = params or SamplerParams()
        self.rng = MT19937_64(self.params.seed)
        self.history: deque = deque()

    # ---- what kind of sampling this is -----------------------------------------------------------
    def penalised(self) -> bool:
        p = self.params
        return (p.repeat_penalty != 1.0 or p.presence_penalty != 0.0) and len(self.history) > 0

    def is_greedy(self) -> bool:
        return self.params.temperature <= 0.0 or self.params.top_k == 1

    CHAIN_MAX_K = 256      # most candidates the device's chain kernel keeps

    def device_mode(self) -> Optional[str]:
        """"greedy", "temperature" or "chain" (top-k on, at most CHAIN_MAX_K) when a device kernel gives the
        same result as the chain on the host, else None (penalties, top-p or min-p without top-k)."""
        if self.penalised():
            return None
        if self.is_greedy():
            return "greedy"
        p = self.params
        if p.top_k <= 0 and p.top_p >= 1.0 and p.min_p <= 0.0:
            return "temperature"
        if 0 < p.top_k <= self.CHAIN_MAX_K:
            return "chain"
        return None

    def chain_record(self):
        """(uniform, top_p, log(min_p) or -inf, temperature, top_k) for the device's chain kernel; draws the
        token's uniform number."""
        p = self.params
        log_min_p = float(np.float32(math.log(p.min_p))) if p.min_p > 0.0 else -math.inf      # as sample() rounds it
        return (self.uniform(), p.top_p, log_min_p, p.temperature, p.top_k)

    def uniform(self) -> float:
        return self.rng.uniform()

    # ---- the chain ---------------------------------------------------------------------------------
    def _penalise(self, logits: np.ndarray) -> np.ndarray:
        if not self.penalised():
            return logits
        p = self.params
        l = logits.copy()
        ids = np.unique([t for t in self.history if 0 <= t < l.shape[0]])
        if ids.size:
            v = l[ids]
            if p.repeat_penalty != 1.0:
                v = np.where(v > 0, v / np.float32(p.repeat_penalty), v * np.float32(p.repeat_penalty))
            l[ids] = v - np.float32(p.presence_penalty)
        return l

    def sample(self, logits) -> int:
        """Pick the next token from float32 logits [vocab].  Does not record it; see :meth:`accept`."""
        p = self.params
        l = self._penalise(np.asarray(logits, dtype=np.float32))
        n = l.shape[0]
        if self.is_greedy():
            return int(np.argmax(l))                       # first maximum = lowest id
        sorted_ = False
        z_all = 0.0
        if p.top_k > 0:
            k = min(p.top_k, n)
            # the k best, ties keep the lower id; then by logit descending, id ascending
            order = np.lexsort((np.arange(n), -l.astype(np.float64)))[:k]
            ids, vals = order, l[order]
            sorted_ = True
        else:
            mx = l.max()
            if p.top_p < 1.0:
                e = np.exp(-(mx - l).astype(np.float64))
                z_all = float(e.sum())
                nb, rng_ = 1024, 40.0
                scale = np.float32(nb / rng_)
                bucket = np.minimum(nb - 1, ((mx - l) * scale).astype(np.int64))
                mass = np.bincount(bucket, weights=e, minlength=nb)
                cum = np.cumsum(mass)
                hit = np.nonzero(cum >= p.top_p * z_all)[0]
                last = int(hit[0]) if hit.size else nb - 1
                ids = np.nonzero(bucket <= last)[0]
                vals = l[ids]
                order = np.lexsort((ids, -vals.astype(np.float64)))
                ids, vals = ids[order], vals[order]
                sorted_ = True
            else:
                floor_logit = mx + np.float32(math.log(p.min_p)) if p.min_p > 0.0 else mx - np.float32(LOGIT_RANGE)
                ids = np.nonzero(l >= floor_logit)[0]
                vals = l[ids]
        if p.top_p < 1.0 and sorted_:
            mx = vals[0]
            e = np.exp(vals.astype(np.float64) - float(mx))
            z = z_all if z_all != 0.0 else float(e.sum())
            cum = np.cumsum(e)
            hit = np.nonzero(cum >= p.top_p * z)[0]
            keep = int(hit[0]) + 1 if hit.size else len(vals)
            ids, vals = ids[:keep], vals[:keep]
        if p.min_p > 0.0:
            cut = vals.max() + np.float32(math.log(p.min_p))
            m = vals >= cut
            ids, vals = ids[m], vals[m]
        mx = vals.max()
        w = np.exp((vals - mx).astype(np.float64) / np.float32(p.temperature)).astype(np.float32)
        cum = np.cumsum(w.astype(np.float64))
        r = self.uniform() * float(cum[-1])
        hit = np.nonzero(r < cum)[0]
        return int(ids[int(hit[0])] if hit.size else ids[-1])

    def accept(self, token: int) -> None:
        if self.params.repeat_last_n <= 0:
            return
        self.history.append(int(token))
        while len(self.history) > self.params.repeat_last_n:
            self.history.popleft()

    def reset(self) -> None:
        self.history.clear()
        self.rng.seed(self.params.seed)
