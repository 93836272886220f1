"""The Python entry point, in the manner of the reference's C API (src/inference.h).

Names and meanings follow the C functions with the ``inference_`` prefix dropped: ``load_model`` (:40),
``kv_cache_init`` (:115), ``set_seed`` (:120), ``reset`` / ``n_past`` (:177-178), ``prefill`` (:183),
``prefill_logits`` (:197), ``decode_token`` (:203), ``generate_ex`` (:223), ``GenOptions`` and
``gen_default_options`` (:244-264), ``generate_stream`` (:275), ``seq_new / seq_select / seq_current /
seq_free`` (:284-287), ``stream_begin / stream_step / stream_step_batch`` (:297-317), ``get_logits``
(:459), ``n_ctx / vocab_size / hidden_size / model_name`` (:462-466); error codes (:18-30) come as
:class:`InferenceError`, stop reasons (:229-236) as strings.  There is no tokenizer: prompts and results
are token ids and the ``text`` of a token callback is always empty.

Beyond the reference: ``generate`` runs many prompts at once through the scheduler (prompt portions and
decode rows share batches), and ``stream_step_batch`` puts prompt portions into the same pass as the
decode rows instead of running them as passes of their own.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from .cache.pages import OutOfPages, OutOfSlots
from .config.base import ConfigError, load_config
from .engine.engine import Engine, StepEntry, StepError, parse_dtype
from .engine.scheduler import (STOP_CALLBACK, STOP_CONTEXT_FULL, STOP_EOG, STOP_MAX_TOKENS, STOP_NONE, Request,
                               Scheduler)
from .parts.model import DecoderModel
from .sampling.sampler import Sampler, SamplerParams

OK, ERR_INVALID_ARG, ERR_OUT_OF_MEMORY, ERR_MODEL_LOAD, ERR_KV_CACHE = 0, -1, -2, -3, -4
ERR_KERNEL_LAUNCH, ERR_INVALID_STATE, ERR_NOT_IMPLEMENTED, ERR_CONTEXT_FULL, ERR_CANCELLED = -6, -7, -8, -9, -10

_MESSAGES = {OK: "success", ERR_INVALID_ARG: "invalid argument", ERR_OUT_OF_MEMORY: "out of memory",
             ERR_MODEL_LOAD: "model load failed", ERR_KV_CACHE: "KV cache error", ERR_KERNEL_LAUNCH: "kernel launch failed",
             ERR_INVALID_STATE: "invalid state", ERR_NOT_IMPLEMENTED: "not implemented", ERR_CONTEXT_FULL: "context full",
             ERR_CANCELLED: "cancelled"}


def strerror(code: int) -> str:
    return _MESSAGES.get(code, "unknown error")


class InferenceError(RuntimeError):
    def __init__(self, code: int, message: str = ""):
        self.code = code
        super().__init__(f"{strerror(code)}: {message}" if message else strerror(code))


@dataclass
class GenOptions:
    """``inference_gen_options`` (src/inference.h:244-264)."""
    sampler: SamplerParams = field(default_factory=SamplerParams)
    max_new_tokens: int = 256
    ignore_eog: bool = False
    reuse_prefix: bool = False
    on_token: Optional[Callable] = None      # (user, token, text, text_len) -> nonzero to stop
    user: object = None
    prefill_chunk: int = 0


def gen_default_options() -> GenOptions:
    return GenOptions()


def _eos_ids(model_dir: str) -> List[int]:
    ids: List[int] = []
    for name in ("generation_config.json", "config.json"):
        path = os.path.join(model_dir, name)
        if os.path.exists(path):
            try:
                with open(path) as f:
                    v = json.load(f).get("eos_token_id")
            except (OSError, json.JSONDecodeError):
                continue
            if isinstance(v, int):
                ids.append(v)
            elif isinstance(v, list):
                ids.extend(int(x) for x in v if isinstance(x, int))
            if ids:
                break
    return sorted(set(ids))


class _Sequence:
    def __init__(self, index: int):
        self.index = index
        self.tokens: List[int] = []
        self.logits: Optional[torch.Tensor] = None     # of the last token, float32 [vocab], device


class Stream:
    """Step-wise generation on one sequence (``inference_stream_t``)."""

    def __init__(self, model: "Model", seq: int, prompt: List[int], options: GenOptions):
        self.model, self.seq, self.options = model, seq, options
        self.pending = list(prompt)                    # prompt tokens not yet in the cache
        self.sampler = Sampler(options.sampler)
        for t in model._seqs[seq].tokens + prompt:
            self.sampler.accept(t)
        self.emitted: List[int] = []
        self.next_token: Optional[int] = None          # sampled, not yet decoded into the sequence
        self.reason = STOP_NONE
        self.done = False


class Model:
    def __init__(self, model_dir: Optional[str], dtype="bfloat16", device="cuda:0", options: Optional[dict] = None,
                 decoder: Optional[DecoderModel] = None, config=None):
        if decoder is None:
            try:
                arch, config = load_config(model_dir)
                decoder = DecoderModel(arch.build_spec(config), parse_dtype(dtype), options)
                decoder.load(model_dir, device)
            except (ConfigError, ValueError, OSError) as e:
                raise InferenceError(ERR_MODEL_LOAD, str(e)) from e
        self._decoder = decoder
        self.model_dir, self.config, self.device = model_dir or "random", config, device
        self.eos_ids = _eos_ids(model_dir) if model_dir else []
        self.engine: Optional[Engine] = None
        self._seed = 0
        self._prefill_batch = 1024
        self._seqs: Dict[int, _Sequence] = {}
        self._current = 0
        self._n_ctx = 0
        self.last_prompt_stats = (0, 0)

    # ---- set-up ------------------------------------------------------------------------------------
    def kv_cache_init(self, n_ctx: int, max_sequences: int = 4, page_size: int = 16, kv_tokens: Optional[int] = None,
                      **engine_options) -> int:
        """A cache for sequences of up to ``n_ctx`` tokens.  The pool holds ``kv_tokens`` tokens in all
        (default: ``max_sequences`` full contexts)."""
        if n_ctx < 1:
            raise InferenceError(ERR_INVALID_ARG, "n_ctx must be positive")
        if n_ctx > self._decoder.spec.max_position:
            raise InferenceError(ERR_INVALID_ARG, f"n_ctx {n_ctx} exceeds the model's max_position_embeddings "
                                                  f"{self._decoder.spec.max_position}")
        per_seq = -(-n_ctx // page_size) * page_size
        self.engine = Engine(self._decoder, self.config, page_size=page_size, max_tokens=kv_tokens or per_seq * max_sequences,
                             max_requests=max_sequences, device=self.device, **engine_options)
        self._n_ctx = n_ctx
        self._seqs = {0: _Sequence(0)}
        self.engine.add_request(("seq", 0))
        self._current = 0
        return OK

    def kv_cache_free(self) -> None:
        self.engine = None
        self._seqs = {}

    def set_seed(self, seed: int) -> None:
        self._seed = int(seed)

    def set_prefill_batch(self, n: int) -> None:
        self._prefill_batch = max(1, int(n))

    def _need_engine(self) -> Engine:
        if self.engine is None:
            raise InferenceError(ERR_INVALID_STATE, "kv_cache_init has not been called")
        return self.engine

    # ---- facts -------------------------------------------------------------------------------------
    def n_ctx(self) -> int:
        return self._n_ctx

    def vocab_size(self) -> int:
        return self._decoder.spec.vocab_size

    def hidden_size(self) -> int:
        return self._decoder.spec.hidden_size

    def model_name(self) -> str:
        return os.path.basename(os.path.normpath(self.model_dir))

    # ---- sequences ---------------------------------------------------------------------------------
    def seq_new(self) -> int:
        eng = self._need_engine()
        idx = 0
        while idx in self._seqs:
            idx += 1
        try:
            eng.add_request(("seq", idx))
        except OutOfSlots:
            return -1
        self._seqs[idx] = _Sequence(idx)
        return idx

    def seq_select(self, seq: int) -> int:
        if seq not in self._seqs:
            raise InferenceError(ERR_INVALID_ARG, f"no sequence {seq}")
        self._current = seq
        return OK

    def seq_current(self) -> int:
        return self._current

    def seq_free(self, seq: int) -> int:
        if seq == 0 or seq not in self._seqs:
            raise InferenceError(ERR_INVALID_ARG, f"sequence {seq} cannot be freed")
        self._need_engine().release(("seq", seq))
        del self._seqs[seq]
        if self._current == seq:
            self._current = 0
        return OK

    def reset(self) -> None:
        """Start the current sequence anew (position 0)."""
        eng = self._need_engine()
        rid = ("seq", self._current)
        eng.release(rid)
        eng.add_request(rid)
        self._seqs[self._current] = _Sequence(self._current)

    def n_past(self) -> int:
        return len(self._seqs[self._current].tokens) if self._seqs else 0

    # ---- forward passes ----------------------------------------------------------------------------
    def _feed(self, seq: int, tokens: Sequence[int], all_logits: bool = False) -> Optional[torch.Tensor]:
        eng = self._need_engine()
        s = self._seqs[seq]
        if len(s.tokens) + len(tokens) > self._n_ctx:
            raise InferenceError(ERR_CONTEXT_FULL, f"{len(s.tokens)} + {len(tokens)} tokens do not fit a context of "
                                                   f"{self._n_ctx}")
        rows = []
        try:
            for i in range(0, len(tokens), self._prefill_batch):
                part = list(tokens[i:i + self._prefill_batch])
                last = i + len(part) >= len(tokens)
                want = list(range(len(part))) if all_logits else ([len(part) - 1] if last else [])
                lg = eng.step([StepEntry(("seq", seq), part, want)])
                if all_logits:
                    rows.append(lg.clone())
                elif last:
                    s.logits = lg[0].clone()
        except OutOfPages as e:
            raise InferenceError(ERR_CONTEXT_FULL, str(e)) from e
        except StepError as e:
            raise InferenceError(ERR_INVALID_ARG, str(e)) from e
        s.tokens.extend(int(t) for t in tokens)
        if all_logits:
            out = torch.cat(rows)
            s.logits = out[-1].clone()
            return out
        return None

    def prefill(self, tokens: Sequence[int]) -> int:
        if len(tokens):
            self._feed(self._current, tokens)
        return OK

    def prefill_logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """Like :meth:`prefill`, and returns the logits after every one of the tokens, float32 [n, vocab]."""
        return self._feed(self._current, tokens, all_logits=True)

    def decode_token(self, token_id: int) -> int:
        """One token at position n_past; returns the greedy next token."""
        self._feed(self._current, [int(token_id)])
        return int(torch.argmax(self._seqs[self._current].logits).item())

    def get_logits(self) -> Optional[torch.Tensor]:
        """Logits of the last token of the current sequence (float32 [vocab], on the device)."""
        return self._seqs[self._current].logits

    # ---- generation --------------------------------------------------------------------------------
    def generate_ex(self, prompt_ids: Sequence[int], max_new_tokens: int, params: Optional[SamplerParams] = None) -> List[int]:
        """New sequence, prefill, then sample up to ``max_new_tokens`` (stops early at EOS, which is not
        returned, or when the context is full)."""
        self.reset()
        opts = GenOptions(sampler=params or SamplerParams(seed=self._seed), max_new_tokens=max_new_tokens)
        out, _ = self.generate_stream(prompt_ids, opts)
        return out

    def _sync_prompt(self, prompt: List[int]) -> List[int]:
        """reuse_prefix: keep the longest common prefix of the sequence and ``prompt``; return what is left
        to prefill (src/inference.cpp:2514-2574)."""
        s = self._seqs[self._current]
        n = 0
        while n < len(s.tokens) and n < len(prompt) and s.tokens[n] == prompt[n]:
            n += 1
        if n == len(prompt) and n > 0:
            n -= 1                                     # at least one token must run to give logits
        eng = self._need_engine()
        try:
            eng.cache.truncate(("seq", self._current), n)
            s.tokens = s.tokens[:n]
        except ValueError:
            self.reset()
            n = 0
        self.last_prompt_stats = (n, len(prompt) - n)
        return prompt[n:]

    def generate_stream(self, prompt_ids: Sequence[int], options: Optional[GenOptions] = None):
        """Continue the current sequence with ``prompt_ids`` and generate.  Returns (tokens, stop reason)."""
        opts = options or gen_default_options()
        prompt = [int(t) for t in prompt_ids]
        if opts.reuse_prefix:
            prompt = self._sync_prompt(prompt)
        else:
            self.last_prompt_stats = (0, len(prompt))
        st = Stream(self, self._current, prompt, opts)
        while not st.done:
            self.stream_run([st], 1 << 20)
        return st.emitted, st.reason

    def stream_begin(self, prompt_ids: Sequence[int], options: Optional[GenOptions] = None) -> Stream:
        opts = options or gen_default_options()
        prompt = [int(t) for t in prompt_ids]
        if opts.reuse_prefix:
            prompt = self._sync_prompt(prompt)
        st = Stream(self, self._current, prompt, opts)
        if opts.prefill_chunk <= 0 and st.pending:
            self._feed(st.seq, st.pending)
            st.pending = []
        return st

    def stream_step(self, stream: Stream):
        """One step of one stream: (going, token); token is None for a step that only prefilled."""
        res = self.stream_step_batch([stream])[0]
        return res

    def stream_step_batch(self, streams: Sequence[Stream]):
        """One step of each stream with ONE pass for all: prompt portions and decode rows share the batch.
        Returns [(going, token)] in the order of ``streams``."""
        eng = self._need_engine()
        entries, owners, results = [], [], [None] * len(streams)
        for i, st in enumerate(streams):
            if st.done:
                results[i] = (False, None)
                continue
            s = self._seqs[st.seq]
            if st.next_token is not None:
                toks = [st.next_token]
            elif st.pending:
                n = st.options.prefill_chunk if st.options.prefill_chunk > 0 else self._prefill_batch
                toks, st.pending = st.pending[:n], st.pending[n:]
            elif s.logits is not None:
                toks = []                              # continue from the last token's logits
            else:
                raise InferenceError(ERR_INVALID_STATE, "nothing to continue from: the sequence is empty")
            if len(s.tokens) + len(toks) > self._n_ctx:
                st.done, st.reason = True, STOP_CONTEXT_FULL
                results[i] = (False, None)
                continue
            if toks:
                samples = not st.pending
                entries.append(StepEntry(("seq", st.seq), toks, [len(toks) - 1] if samples else []))
                owners.append((i, st, toks, samples))
            else:
                owners.append((i, st, [], True))
        logits = None
        if entries:
            try:
                logits = eng.step(entries)
            except OutOfPages as e:
                raise InferenceError(ERR_CONTEXT_FULL, str(e)) from e
        # One copy of the step's logits (they live in scratch memory that the next step reuses); each sequence
        # keeps a view of its row.  When every sampled row comes from this step, in order, the copy is sampled
        # from as it is.
        kept = logits.clone() if logits is not None else None
        row = 0
        rows, samplers, who = [], [], []
        direct = True
        for i, st, toks, samples in owners:
            s = self._seqs[st.seq]
            s.tokens.extend(toks)
            st.next_token = None
            if not samples:
                results[i] = (True, None)
                continue
            if toks:
                s.logits = kept[row]
                row += 1
            else:
                direct = False
            rows.append(s.logits)
            samplers.append(st.sampler)
            who.append((i, st))
        if rows:
            toks_out = eng.sample(kept if direct and len(rows) == kept.shape[0] else torch.stack(rows), samplers)
            for (i, st), tok in zip(who, toks_out):
                results[i] = self._emit(st, int(tok))
        return results

    def _take_token(self, st: Stream, tok: int, in_cache: int) -> str:
        """Take the sampled token: "eog" (not emitted), "stop" (emitted, the stream ends) or "go".  ``in_cache``:
        tokens of the sequence before this one."""
        o = st.options
        if not o.ignore_eog and tok in self.eos_ids:
            st.done, st.reason = True, STOP_EOG
            return "eog"
        st.emitted.append(tok)
        st.sampler.accept(tok)
        stop = bool(o.on_token(o.user, tok, "", 0)) if o.on_token else False
        if stop:
            st.reason = STOP_CALLBACK
        elif len(st.emitted) >= o.max_new_tokens:
            st.reason = STOP_MAX_TOKENS
        elif in_cache + 1 >= self._n_ctx:
            st.reason = STOP_CONTEXT_FULL
        else:
            return "go"
        return "stop"

    def _emit(self, st: Stream, tok: int):
        verdict = self._take_token(st, tok, len(self._seqs[st.seq].tokens))
        if verdict == "eog":
            return (False, None)
        if verdict == "go":
            st.next_token = tok
            return (True, tok)
        # every emitted token is decoded into the sequence, so that a later call continues after it
        try:
            self._feed(st.seq, [tok])
        except InferenceError:
            pass
        st.next_token = None
        st.done = True
        return (False, tok)

    def stream_run(self, streams: Sequence[Stream], n_steps: int):
        """Up to ``n_steps`` steps of every stream: the list of what :meth:`stream_step_batch` would return step by
        step (shorter when every stream ends earlier).  While all live streams are decoding and their samplers run
        on the device, a step is launched with the token ids the step before left on the device, before the host
        has read them, so the host's work of a step overlaps the device's; the tokens, the stop reasons and the
        samplers' draws are those of the step-by-step calls, a callback's stop takes effect one step late on the
        device only (the step that was already running is discarded)."""
        out = []
        while len(out) < n_steps and not all(st.done for st in streams):
            seg = self._run_ahead(streams, n_steps - len(out))
            if seg:
                out.extend(seg)
            else:
                out.append(self.stream_step_batch(streams))
        return out

    def _run_ahead(self, streams: Sequence[Stream], max_steps: int):
        """A run of decode steps each launched before the tokens of the one before are on the host; None when the
        streams are not all in plain decoding with device samplers, or fewer than two steps are certain to run."""
        eng = self._need_engine()
        live = [(i, st) for i, st in enumerate(streams) if not st.done]
        if not live or any(st.next_token is None or st.pending for _, st in live):
            return None
        modes = {st.sampler.device_mode() for _, st in live}
        if len(modes) != 1 or None in modes:
            return None
        seqs = [self._seqs[st.seq] for _, st in live]
        # steps that cannot end a stream by its token budget or the context: only an end-of-generation token or a
        # callback may stop a stream inside the run
        horizon = min(min(st.options.max_new_tokens - len(st.emitted), self._n_ctx - len(s.tokens) - 1)
                      for (_, st), s in zip(live, seqs))
        n = min(max_steps, horizon)
        probe = [StepEntry(("seq", st.seq), [0], [0]) for _, st in live]
        if n < 2 or not eng.decodes_as_graph(probe):
            return None
        # an end-of-generation token is found out after the next step has put it into the cache: it must be possible
        # to take it back
        rewindable = not any(g.window is not None for g in eng.cache.groups) and not eng.cache.state_entries
        if not rewindable and self.eos_ids and any(not st.options.ignore_eog for _, st in live):
            return None
        samplers = [st.sampler for _, st in live]
        results = []

        def settle(toks, fed_logits, own_logits=None):
            """The tokens sampled by a step (own_logits: its logits) whose successor, if fed_logits (the successor's
            logits) is given, has already put them into the cache.  Returns the streams' indices in ``live`` that
            ended."""
            res = [(False, None)] * len(streams)
            ended = []
            for j, ((i, st), s, tok) in enumerate(zip(live, seqs, toks)):
                tok = int(tok)
                verdict = self._take_token(st, tok, len(s.tokens))
                if fed_logits is None:                       # not fed yet: as in a step-by-step call
                    if verdict == "go":
                        st.next_token = tok
                        res[i] = (True, tok)
                    elif verdict == "eog":
                        res[i] = (False, None)
                        ended.append(j)
                    else:
                        try:
                            self._feed(st.seq, [tok])
                        except InferenceError:
                            pass
                        st.next_token, st.done = None, True
                        res[i] = (False, tok)
                        ended.append(j)
                    continue
                if verdict == "eog":
                    eng.cache.truncate(("seq", st.seq), len(s.tokens))       # the step in flight fed it: take it back
                    s.logits = own_logits[j]
                    res[i] = (False, None)
                    ended.append(j)
                    continue
                s.tokens.append(tok)
                if verdict == "go":
                    res[i] = (True, tok)
                else:
                    s.logits = fed_logits[j]
                    st.next_token, st.done = None, True
                    res[i] = (False, tok)
                    ended.append(j)
            results.append(res)
            return ended

        prev = prev_kept = None
        try:
            for step in range(n):
                if step == 0:
                    entries = [StepEntry(("seq", st.seq), [st.next_token], [0]) for _, st in live]
                    for (_, st), s in zip(live, seqs):
                        s.tokens.append(st.next_token)
                        st.next_token = None
                else:
                    entries = probe
                logits = eng.step(entries, device_tokens=prev.ids if prev is not None else None)
                snaps = [sm.rng.snapshot() for sm in samplers]
                pend = eng.sample_async(logits, samplers)
                kept = logits.clone()                        # the step's logits live in memory the next step reuses
                if prev is not None:
                    ended = settle(prev.result(), kept, prev_kept)
                    if ended:
                        # what the step in flight sampled for the ended streams is dropped, their draws taken back;
                        # the others' tokens stand, and the run ends here: the batch has changed
                        toks = pend.result()
                        for j in ended:
                            samplers[j].rng.restore(snaps[j])
                        keep = [j for j in range(len(live)) if j not in ended]
                        live_rest = [live[j] for j in keep]
                        if live_rest:
                            live, seqs = live_rest, [seqs[j] for j in keep]
                            for s, j in zip(seqs, keep):
                                s.logits = kept[j]
                            settle([toks[j] for j in keep], None)
                        return results
                prev, prev_kept = pend, kept
            for j, s in enumerate(seqs):
                s.logits = prev_kept[j]
            settle(prev.result(), None)
        except OutOfPages as e:
            raise InferenceError(ERR_CONTEXT_FULL, str(e)) from e
        return results

    # ---- many prompts at once ------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0, seed: int = 0,
                 params: Optional[SamplerParams] = None, ignore_eos: bool = True, max_batch_tokens: int = 2048,
                 prefill_chunk: int = 512) -> List[List[int]]:
        """Generate for all ``prompts`` through the scheduler; returns the new tokens of each prompt."""
        eng = self._need_engine()
        for seq in list(self._seqs):                   # the scheduler owns the cache for the duration
            eng.release(("seq", seq))
        self._seqs = {}
        sched = Scheduler(eng, max_batch_tokens=max_batch_tokens, prefill_chunk=prefill_chunk, n_ctx=self._n_ctx)
        reqs = []
        for i, p in enumerate(prompts):
            sp = params or (SamplerParams.greedy() if temperature <= 0 else SamplerParams.pure_temperature(temperature))
            sp = SamplerParams(**{**sp.__dict__, "seed": seed + i})
            reqs.append(sched.add(Request(("gen", i), [int(t) for t in p], sp, max_new_tokens, self.eos_ids, ignore_eos)))
        sched.run()
        self.last_scheduler = sched
        self._seqs = {0: _Sequence(0)}
        eng.add_request(("seq", 0))
        self._current = 0
        return [r.output for r in reqs]


def load_model_random(config, seed: int, dtype="bfloat16", device="cuda:0", std: float = 0.02, scale_low: float = 1.0,
                      scale_high: float = 1.0, options: Optional[dict] = None) -> Model:
    """A model of ``config`` (a typed configuration) with seeded random weights made on the device."""
    from .config.base import lookup_architecture
    from .weights.loader import device_dtype
    from .weights.random_init import random_tensor
    dt = parse_dtype(dtype)
    decoder = DecoderModel(lookup_architecture(config.architecture).build_spec(config), dt, options)
    tensors = {}
    for name, spec in decoder.tensor_specs().items():
        t = random_tensor(spec, seed, std, scale_low, scale_high, device=device)
        tensors[name] = t.to(device_dtype(torch.bfloat16, spec.role, dt))
    decoder.bind(tensors, device)
    return Model(None, dtype, device, options, decoder=decoder, config=config)


def load_model(path: str, dtype="bfloat16", device="cuda:0", options: Optional[dict] = None) -> Model:
    """``inference_load_model``: read config.json and the safetensors of ``path`` onto the device."""
    return Model(path, dtype, device, options)
