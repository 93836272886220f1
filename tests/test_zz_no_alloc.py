"""ph_attention_decode_static, the decode attention entry point for callers that cannot allocate device
memory (a server whose memory is all handed out, a host that links the C symbols without an allocator, a
latency path that cannot afford cudaMalloc's synchronisation).  It keeps its scratch in a fixed array inside the
library, so this test calls it the way such a caller would: through the exported C symbol with raw pointers,
twice in a row on one stream (the second call finds the first call's leftovers in the array), and compares
each result with the ordinary entry point, which gets scratch from the test, and with attention computed densely
in float64.  It also checks that a request larger than the array is refused by name instead of overrunning it,
and that a call that needs no scratch (keys in one piece) is not refused whatever its size.

The file sorts last on purpose: a run that stops at the first failure has then run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _entry():
    from purhie_b200.csrc.build import load_library
    lib = load_library("decode_static")
    fn = lib.ph_attention_decode_static
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    fn.restype = c_int
    err = lib.ph_decode_static_last_error
    err.restype = ctypes.c_char_p
    return fn, err


def _case(segs, HQ, HKV, D, page_size, seed):
    from test_gpu_kernels import paged_case
    return paged_case(segs, HQ, HKV, D, page_size, torch.bfloat16, seed=seed)


def _call_static(fn, case, HQ, HKV, D, page_size, splits, window, scale):
    out = torch.full((case["T"], HQ * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    rc = fn(case["q"].data_ptr(), case["k_base"].data_ptr(), case["v_base"].data_ptr(), case["page_stride"], page_size,
            case["table"].data_ptr(), case["table"].shape[1], None, case["T"], case["row_seg"].data_ptr(),
            case["positions"].data_ptr(), out.data_ptr(), HQ, HKV, D, splits, window or 0, scale,
            torch.cuda.current_stream().cuda_stream)
    return rc, out


def _call_ordinary(case, HQ, HKV, D, page_size, splits, window, scale):
    from purhie_b200.csrc import flash
    from purhie_b200.csrc.ops import Workspace
    out = torch.full((case["T"], HQ * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    flash.decode(case["q"], case["k_base"], case["v_base"], case["page_stride"], page_size, case["table"], None, case["T"],
                 case["row_seg"], case["positions"], out, Workspace(DEV), num_heads=HQ, num_kv_heads=HKV, head_dim=D,
                 window=window, scale=scale, splits=splits)
    return out


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    fn, err = _entry()
    # first call: 6 decode rows, 4 splits; second call: other shapes, other data, more splits, a window
    calls = [
        dict(segs=[(300, 1), (64, 1), (1, 1), (700, 1), (129, 1), (65, 1)], HQ=8, HKV=2, D=128, page_size=16, splits=4,
             window=None, seed=21),
        dict(segs=[(513, 1), (40, 1), (1000, 1)], HQ=6, HKV=3, D=64, page_size=8, splits=7, window=200, seed=22),
    ]
    for c in calls:
        case = _case(c["segs"], c["HQ"], c["HKV"], c["D"], c["page_size"], c["seed"])
        scale = 1.0 / math.sqrt(c["D"])
        rc, got = _call_static(fn, case, c["HQ"], c["HKV"], c["D"], c["page_size"], c["splits"], c["window"], scale)
        assert rc == 0, err().decode()
        ref = _call_ordinary(case, c["HQ"], c["HKV"], c["D"], c["page_size"], c["splits"], c["window"], scale)
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        diff = (got.float() - ref.float()).abs().max().item()
        assert diff <= 1e-2 * ref.float().abs().max().item(), diff       # the tolerance of the attention kernel tests
        assert torch.equal(got, ref)                                      # and in fact the same kernels: the same bits
        # the math itself, against attention computed densely in float64
        from test_gpu_kernels import dense_attention
        dense = dense_attention(case, c["HQ"], c["HKV"], c["D"], c["window"], scale)
        assert (got.double().cpu() - dense).abs().max().item() <= 1e-2 * dense.abs().max().item()


def test_static_scratch_entry_point_refuses_more_than_its_array_holds():
    fn, err = _entry()
    case = _case([(64, 1)], 8, 2, 128, 16, 23)
    # 40000 rows x 8 heads x 32 splits x 130 floats is far beyond 16 MiB: refused before anything is launched
    rc = fn(case["q"].data_ptr(), case["k_base"].data_ptr(), case["v_base"].data_ptr(), case["page_stride"], 16,
            case["table"].data_ptr(), case["table"].shape[1], None, 40000, case["row_seg"].data_ptr(),
            case["positions"].data_ptr(), case["q"].data_ptr(), 8, 2, 128, 32, 0, 0.1, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = err().decode()
    assert "16777216" in msg and "scratch" in msg
    torch.cuda.synchronize()


def test_static_scratch_entry_point_takes_any_size_when_the_keys_are_in_one_piece():
    """With one split the kernel writes its result directly and uses no scratch: 3,000 rows x 8 heads would need 12 MiB
    at four splits and is far beyond the array at 32, but at one split nothing is needed and nothing is refused."""
    from test_gpu_kernels import dense_attention
    fn, err = _entry()
    HQ, HKV, D, ps = 8, 2, 128, 16
    case = _case([(70 + (i % 50), 1) for i in range(3000)], HQ, HKV, D, ps, 24)
    scale = 1.0 / math.sqrt(D)
    rc, got = _call_static(fn, case, HQ, HKV, D, ps, 1, None, scale)
    assert rc == 0, err().decode()
    ref = _call_ordinary(case, HQ, HKV, D, ps, 1, None, scale)
    torch.cuda.synchronize()
    assert torch.equal(got, ref)
    few = dict(case, T=16, segs=case["segs"][:16], dense=case["dense"][:16])
    dense = dense_attention(few, HQ, HKV, D, None, scale)
    assert (got[:16].double().cpu() - dense).abs().max().item() <= 1e-2 * dense.abs().max().item()
