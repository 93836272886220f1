"""Python faces of the CUDA kernels: torch tensors in, launches on the current stream.

These serve the kernels' own tests and measurements (each kernel beside a plain reference, at sizes of the test's
choosing); the engine launches the same exported functions from its C++ parts.  Every function checks what the
kernel cannot check cheaply (device, dtype, contiguity, shapes) and raises :class:`KernelError` with the library's
message when a launcher refuses.  Nothing here computes on the host, and nothing falls back to a library
implementation: a missing library is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1


from ..native import KernelError  # noqa: E402  (the library's error kind, shared with the engine's face)


class Workspace:
    """Scratch tensors by name for the faces that need some (split-key partial results), reused and grown on demand;
    ``frozen`` turns growth into an error, as under a captured graph."""

    def __init__(self, device):
        self.device = device
        self._bufs = {}
        self.frozen = False

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        buf = self._bufs.get((name, dtype))
        if buf is None or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow while frozen")
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[(name, dtype)] = buf
        return buf[:n].view(*shape)


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {dtype}; the kernels take float32 and bfloat16")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_stream_now: Optional[int] = None


def _stream() -> int:
    """The stream the launchers use: the current one, looked up once per :func:`on_current_stream` scope."""
    return _stream_now if _stream_now is not None else torch.cuda.current_stream().cuda_stream


class on_current_stream:
    """Inside this scope every launcher uses the stream that was current when the scope was entered, without asking
    torch again for each of the few hundred launches of a step."""

    def __enter__(self):
        global _stream_now
        self._before = _stream_now
        _stream_now = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _stream_now
        _stream_now = self._before
        return False


def _need(t: torch.Tensor, name: str, dtype=None) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; there is no host implementation")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t


_SIGNATURES = {
    "core": {
        "ph_embed_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "ph_add_rmsnorm": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_float, c_void_p, c_int, c_int,
                           c_void_p, c_int, c_int, c_void_p],
        "ph_swiglu": [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p],
        "ph_cast": [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p],
        "ph_qk_norm_rope_kv_write": [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_float,
                                     c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                     c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                     c_float, c_void_p],
        "ph_add_weight_sumsq": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_void_p, c_int,
                                c_void_p, c_int, c_void_p],
        "ph_attention_generic": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p, c_int,
                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                 c_void_p],
        "ph_gemm_simple": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "ph_argmax": [c_void_p, c_int, c_int, c_void_p, c_void_p],
        "ph_argmax_parts": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_longlong, c_void_p],
        "ph_sample_temperature": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p],
        "ph_sample_chain": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
    },
}
_bound = {}


def _fn(lib_name: str, fn_name: str):
    key = (lib_name, fn_name)
    f = _bound.get(key)
    if f is None:
        lib = load_library(lib_name)
        f = getattr(lib, fn_name)
        f.argtypes = _SIGNATURES[lib_name][fn_name]
        f.restype = c_int
        err = getattr(lib, f"ph_{lib_name}_last_error")
        err.restype = ctypes.c_char_p
        _bound[key] = f = (f, err)
    return f


def register_signatures(lib_name: str, table: dict) -> None:
    _SIGNATURES.setdefault(lib_name, {}).update(table)


launches = 0          # launcher calls so far (a captured graph replays the calls counted while it was captured)


def call(lib_name: str, fn_name: str, *args) -> None:
    global launches
    f, err = _fn(lib_name, fn_name)
    launches += 1
    rc = f(*args)
    if rc != 0:
        raise KernelError(err().decode("utf-8", "replace") or f"{fn_name} failed with status {rc}")


# ---- core ------------------------------------------------------------------------------------------

def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] widened to float32."""
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    T, (V, E) = ids.numel(), table.shape
    if out.shape[-1] != E or out.numel() < T * E:
        raise KernelError(f"embed_gather: out {tuple(out.shape)} does not hold {T} rows of {E}")
    call("core", "ph_embed_gather", _ptr(table), _code(table.dtype), _ptr(ids), _ptr(out), T, E, V, _stream())
    return out


def add_rmsnorm(x: torch.Tensor, add: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                add_splits: int = 1, write_x: bool = True) -> Optional[torch.Tensor]:
    """v = x[t] + sum_s add[s][t] (stored back into x unless gathered); out[r] = rmsnorm(v) * weight.

    ``x`` is the float32 residual stream [T, E].  ``add`` is [T, E] or, with ``add_splits`` > 1, the
    partial sums [splits, T, E] of a split matrix product.  ``rows`` (int32) picks the rows that are
    normed, in that order; ``weight`` None only adds.
    """
    _need(x, "x", torch.float32)
    E = x.shape[-1]
    T = x.numel() // E
    n = n_rows if n_rows is not None else (T if rows is None else rows.numel())
    split_stride = 0
    if add is not None:
        _need(add, "add")
        if add.numel() != add_splits * T * E:
            raise KernelError(f"add_rmsnorm: add has {add.numel()} elements, expected {add_splits} x {T} x {E}")
        split_stride = T * E
    if weight is not None:
        _need(weight, "weight", torch.float32)
        if weight.numel() != E or out is None:
            raise KernelError("add_rmsnorm: weight must have the row width and out must be given")
        _need(out, "out")
        if out.shape[-1] != E or out.numel() < n * E:
            raise KernelError(f"add_rmsnorm: out {tuple(out.shape)} does not hold {n} rows of {E}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    call("core", "ph_add_rmsnorm", _ptr(x), _ptr(add), _code(add.dtype) if add is not None else F32, add_splits,
         split_stride, _ptr(weight), float(eps), _ptr(rows), n, E, _ptr(out),
         _code(out.dtype) if out is not None else F32, 1 if (write_x and rows is None) else 0, _stream())
    return out


def add_weight_sumsq(x: torch.Tensor, add: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                     add_splits: int = 1) -> torch.Tensor:
    """x [T, E] float32 += the addends; out = x * weight WITHOUT the row's factor; returns sumsq [T, ceil(E / 512)]
    float32, the row's sum of squares in parts: the consumer applies rsqrt(sum / E + eps) (see elementwise.cu)."""
    _need(x, "x", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    E = x.shape[-1]
    T = x.numel() // E
    chunks = -(-E // 512)
    sumsq = torch.empty(T, chunks, dtype=torch.float32, device=x.device)
    if add is not None:
        _need(add, "add")
        if add.numel() != add_splits * T * E:
            raise KernelError(f"add_weight_sumsq: add has {add.numel()} elements, expected {add_splits} x {T} x {E}")
    call("core", "ph_add_weight_sumsq", _ptr(x), _ptr(add), _code(add.dtype) if add is not None else F32, add_splits, T * E,
         _ptr(weight), T, E, _ptr(out), _code(out.dtype), _ptr(sumsq), chunks, _stream())
    return sumsq


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, splits: int = 1) -> torch.Tensor:
    """out[t, j] = silu(g[t, j]) * u[t, j] for gate_up rows laid out [g0, u0, g1, u1, ...]."""
    _need(gate_up, "gate_up"); _need(out, "out")
    FF = out.shape[-1]
    T = out.numel() // FF
    if gate_up.numel() != splits * T * 2 * FF:
        raise KernelError(f"swiglu: gate_up has {gate_up.numel()} elements, expected {splits} x {T} x {2 * FF}")
    call("core", "ph_swiglu", _ptr(gate_up), _code(gate_up.dtype), splits, T * 2 * FF, _ptr(out), _code(out.dtype), T,
         FF, _stream())
    return out


def cast(src: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(src, "src"); _need(out, "out")
    if src.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    call("core", "ph_cast", _ptr(src), _code(src.dtype), _ptr(out), _code(out.dtype), src.numel(), _stream())
    return out


def qk_norm_rope_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, *, num_heads: int,
                          num_kv_heads: int, head_dim: int, eps: float, q_norm: Optional[torch.Tensor],
                          k_norm: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                          cos_sin: Optional[torch.Tensor], n_rot: int, slot_mapping: Optional[torch.Tensor],
                          k_base: Optional[torch.Tensor], v_base: Optional[torch.Tensor], page_stride: int,
                          page_size: int, splits: int = 1, interleaved: bool = False,
                          row_sumsq: Optional[torch.Tensor] = None, row_width: int = 0, row_eps: float = 0.0) -> torch.Tensor:
    """Fused per-head norm, rotary encoding and cache write; see qk_norm_rope.cu.  ``row_sumsq`` [T, chunks]: the
    rows of qkv lack the factor rsqrt(sum(row_sumsq[t]) / row_width + row_eps), which is applied here (add_weight_sumsq).

    ``k_base`` / ``v_base`` are views whose first element is the K / V of this cache entry in page 0.
    """
    _need(qkv, "qkv"); _need(q_out, "q_out"); _need(positions, "positions", torch.int32)
    T = positions.numel()
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.numel() != splits * T * width:
        raise KernelError(f"qk_norm_rope: qkv has {qkv.numel()} elements, expected {splits} x {T} x {width}")
    if q_out.numel() < T * num_heads * head_dim:
        raise KernelError("qk_norm_rope: q_out is too small")
    for name, t in (("q_norm", q_norm), ("k_norm", k_norm)):
        if t is not None:
            _need(t, name, torch.float32)
            if t.numel() != head_dim:
                raise KernelError(f"qk_norm_rope: {name} must have head_dim elements")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != width:
            raise KernelError("qk_norm_rope: bias must cover q, k and v")
    max_pos = 0
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        max_pos = cos_sin.shape[0]
        if cos_sin.shape[1] != n_rot:
            raise KernelError("qk_norm_rope: the cos/sin table must be [max_position, n_rot]")
    kv_code = F32
    if slot_mapping is not None:
        _need(slot_mapping, "slot_mapping", torch.int32)
        if k_base is None or v_base is None or k_base.dtype != v_base.dtype:
            raise KernelError("qk_norm_rope: a cache write needs K and V of one dtype")
        kv_code = _code(k_base.dtype)
    call("core", "ph_qk_norm_rope_kv_write", _ptr(qkv), _code(qkv.dtype), splits, T * width, _ptr(bias), _ptr(q_norm),
         _ptr(k_norm), float(eps), _ptr(cos_sin), n_rot, max_pos, _ptr(positions), _ptr(slot_mapping), _ptr(q_out),
         _code(q_out.dtype), _ptr(k_base), _ptr(v_base), kv_code, page_stride, page_size, T, num_heads, num_kv_heads,
         head_dim, 1 if interleaved else 0, _ptr(row_sumsq), 0 if row_sumsq is None else row_sumsq.shape[-1], row_width,
         float(row_eps), _stream())
    return q_out


def attention_generic(q: torch.Tensor, k_base: torch.Tensor, v_base: torch.Tensor, page_stride: int, page_size: int,
                      block_table: torch.Tensor, row_seg: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, *,
                      num_heads: int, num_kv_heads: int, head_dim: int, window: Optional[int], scale: float) -> torch.Tensor:
    _need(q, "q"); _need(k_base, "k_base"); _need(v_base, "v_base"); _need(out, "out")
    _need(block_table, "block_table", torch.int32); _need(row_seg, "row_seg", torch.int32)
    _need(positions, "positions", torch.int32)
    T = positions.numel()
    if q.numel() < T * num_heads * head_dim or out.numel() < T * num_heads * head_dim:
        raise KernelError("attention_generic: q or out is too small")
    if k_base.dtype != v_base.dtype:
        raise KernelError("attention_generic: K and V must share a dtype")
    call("core", "ph_attention_generic", _ptr(q), _code(q.dtype), _ptr(k_base), _ptr(v_base), _code(k_base.dtype),
         page_stride, page_size, _ptr(block_table), block_table.shape[-1], _ptr(row_seg), _ptr(positions), _ptr(out),
         _code(out.dtype), T, num_heads, num_kv_heads, head_dim, int(window or 0), float(scale), _stream())
    return out


def gemm_simple(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T with float32 multiply-add in a fixed order."""
    _need(x, "x"); _need(w, "w"); _need(out, "out")
    N, K = w.shape
    M = x.numel() // K
    if x.shape[-1] != K or out.shape[-1] != N or out.numel() < M * N:
        raise KernelError(f"gemm_simple: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    call("core", "ph_gemm_simple", _ptr(x), _code(x.dtype), _ptr(w), _code(w.dtype), _ptr(out), _code(out.dtype), M, N,
         K, _stream())
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy choice per row, the lowest id on ties.  With ``scratch`` (bytes: rows x (4 + 64 x 8), the first 4 x rows
    zero before the first call) several CTAs share a row."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    V = logits.shape[-1]
    R = logits.numel() // V
    if scratch is None:
        call("core", "ph_argmax", _ptr(logits), R, V, _ptr(out), _stream())
    else:
        call("core", "ph_argmax_parts", _ptr(logits), R, V, _ptr(out), _ptr(scratch), scratch.numel() * scratch.element_size(), _stream())
    return out


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor,
                       logit_range: float = 40.0) -> torch.Tensor:
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(uniform, "uniform", torch.float64)
    V = logits.shape[-1]
    R = logits.numel() // V
    if temperature.numel() != R or uniform.numel() != R:
        raise KernelError("sample_temperature: one temperature and one uniform number per row")
    call("core", "ph_sample_temperature", _ptr(logits), R, V, _ptr(temperature), _ptr(uniform), float(logit_range),
         _ptr(out), _stream())
    return out


CHAIN_MAX_K = 256          # most candidates the chain kernel keeps (KMAX in sampling.cu)
CHAIN_ROW = [("uniform", "<f8"), ("top_p", "<f4"), ("log_min_p", "<f4"), ("temperature", "<f4"), ("top_k", "<i4")]


def sample_chain(logits: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """top-k -> top-p -> min-p -> temperature -> draw for each row of ``logits``.  ``rows``: uint8 [R, 24] on the
    device, one CHAIN_ROW record per row (top_k in 1 .. CHAIN_MAX_K, temperature > 0, log_min_p -inf for off)."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32); _need(rows, "rows", torch.uint8)
    V = logits.shape[-1]
    R = logits.numel() // V
    if rows.numel() != 24 * R or out.numel() < R:
        raise KernelError("sample_chain: one 24-byte record and one output per row")
    call("core", "ph_sample_chain", _ptr(logits), R, V, _ptr(rows), _ptr(out), _stream())
    return out
