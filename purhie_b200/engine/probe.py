"""The scheduler's decisions without a device: the host library's own Scheduler over a stand-in for the engine that
keeps the real cache bookkeeping but runs no model (``api/test_hooks_host.cpp``).  The stand-in's logits put all
weight on ``(sum of the request's tokens so far * 7 + their count) % vocab``, so the generated tokens are a pure
function of a request's history, and any change of order or cut shows.  Request ids are small integers here.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import POINTER, c_char_p, c_int, c_int32, c_longlong, c_void_p
from typing import Optional, Sequence

from .. import native
from ..sampling import SamplerParams

_DECLARED = False


def _lib():
    global _DECLARED
    L = native.lib()
    if not _DECLARED:
        P = c_void_p
        for name, res, args in [
            ("qe_sched_create", P, [c_char_p]), ("qe_sched_free_handle", None, [P]),
            ("qe_sched_add", c_int, [P, c_longlong, POINTER(c_int32), c_int, POINTER(native.SamplerParamsC), c_int,
                                     POINTER(c_int32), c_int, c_int, c_int]),
            ("qe_sched_step", c_int, [P]), ("qe_sched_decode_ahead", c_int, [P]), ("qe_sched_cancel", c_int, [P, c_longlong]),
            ("qe_sched_has_work", c_int, [P]), ("qe_sched_state", c_char_p, [P]),
        ]:
            native.declare(name, res, args)
        _DECLARED = True
    return L


def expected_output(prompt: Sequence[int], n: int, vocab: int = 50):
    """What greedy decoding over the stand-in must produce for ``prompt``."""
    h, out = list(prompt), []
    for _ in range(n):
        t = (sum(h) * 7 + len(h)) % vocab
        out.append(t)
        h.append(t)
    return out


class SchedulerProbe:
    def __init__(self, num_pages: int = 64, page_size: int = 4, max_requests: int = 4, window: Optional[int] = None,
                 ahead: bool = False, **scheduler_options):
        """``scheduler_options``: max_batch_tokens, prefill_chunk, n_ctx, align_rows, run_ahead.  ``ahead``: the stand-in
        accepts a step's token ids "from the device", which is what decode_ahead needs."""
        opts = dict(num_pages=num_pages, page_size=page_size, max_requests=max_requests, window=window or 0, ahead=ahead)
        opts.update({k: v for k, v in scheduler_options.items() if v is not None})
        self._h = _lib().qe_sched_create(json.dumps(opts).encode())
        if not self._h:
            raise native.last_error()

    def __del__(self):
        try:
            _lib().qe_sched_free_handle(self._h)
        except Exception:
            pass

    def add(self, request_id: int, prompt: Sequence[int], params: Optional[SamplerParams] = None, max_new_tokens: int = 256,
            eos_ids: Sequence[int] = (), ignore_eos: bool = False, stop_after: int = 0) -> None:
        """``stop_after``: the request's token callback asks to stop once it has seen that many tokens."""
        toks = native.int32_array(list(prompt))
        eos = native.int32_array(list(eos_ids))
        c = (params or SamplerParams.greedy()).to_c()
        native.check(_lib().qe_sched_add(self._h, request_id, toks, len(prompt), ctypes.byref(c), max_new_tokens, eos,
                                         len(eos_ids), int(ignore_eos), stop_after))

    def step(self) -> None:
        native.check(_lib().qe_sched_step(self._h))

    def decode_ahead(self) -> int:
        """Steps taken ahead of the host (0: not applicable, take an ordinary step)."""
        return native.check(_lib().qe_sched_decode_ahead(self._h))

    def cancel(self, request_id: int) -> bool:
        return bool(native.check(_lib().qe_sched_cancel(self._h, request_id)))

    def has_work(self) -> bool:
        return bool(_lib().qe_sched_has_work(self._h))

    def state(self) -> dict:
        """running / waiting ids, finished {id: {output, stop_reason, preemptions, n_tokens}}, the batches the stand-in
        ran as [[id, tokens, want]], preemptions, steps, and the cache's accounting."""
        s = native.answer(_lib().qe_sched_state(self._h))
        s["finished"] = {int(k): v for k, v in s["finished"].items()}
        return s

    def run(self, ahead: bool = False, guard: int = 10000) -> dict:
        while self.has_work():
            if not (ahead and self.decode_ahead()):
                self.step()
            guard -= 1
            assert guard > 0, "the scheduler does not come to an end"
        return self.state()
