"""The allocation-free attention-backward entry point (csrc/noalloc.h) against the regular one.

Some hosts of this library fix their GPU memory at start-up and may not allocate when they call into it, so they
cannot supply the backward pass's scratch buffer; ``aeris_attn_bwd_noalloc`` keeps that scratch in a device array
inside the library instead. The test calls it through its exported C symbol, twice in a row with different inputs
(the shared scratch keeps the first call's contents), and checks both results against the regular entry point.
This file sorts last on purpose: a failure here cannot hide the result of any other test in a run with ``-x``.
"""
import ctypes
import math

import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, qkv, o, d_o, lse, dqkv, nw, N, H, d):
    from aeris_gb_b200.ops import lib as L
    fn = lib.aeris_attn_bwd_noalloc
    fn.restype = ctypes.c_int
    return fn(L.ptr(qkv), qkv.stride(0), 0, H * d, 2 * H * d, L.ptr(o), L.ptr(d_o), o.stride(0), L.ptr(lse),
              L.ptr(dqkv), dqkv.stride(0), nw, N, H, d, ctypes.c_float(1.0 / math.sqrt(d)),
              L.ptr(L.status_word()), L.stream_ptr())


def test_noalloc_attention_backward_matches_regular_entry_point():
    from aeris_gb_b200.ops import attention as A
    from aeris_gb_b200.ops import lib as L
    from aeris_gb_b200.ops.build import LIB_PATH
    lib = ctypes.CDLL(str(LIB_PATH))
    torch.manual_seed(5)
    for (nw, N, H, d) in [(3, 900, 2, 64), (2, 256, 4, 64)]:     # two calls in a row, different shapes
        qkv = torch.randn(nw * N, 3 * H * d, device="cuda").bfloat16()
        go = torch.randn(nw * N, H * d, device="cuda").bfloat16()
        o, lse = A.attn_fwd(qkv, nw, N, H, d)
        want = A.attn_bwd(qkv, o, go, lse, nw, N, H, d)
        got = torch.zeros_like(qkv)
        before = torch.cuda.memory_allocated()
        rc = _call_noalloc(lib, qkv, o, go, lse, got, nw, N, H, d)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        L.check_status()
        assert rel_err(got, want) < 8e-3
        x = qkv.float().requires_grad_(True)
        A.attn_reference(x, nw, N, H, d).backward(go.float())
        assert rel_err(got, x.grad) < 8e-3


def test_noalloc_rejects_oversize():
    from aeris_gb_b200.ops.build import LIB_PATH
    lib = ctypes.CDLL(str(LIB_PATH))
    t = torch.zeros(16, device="cuda", dtype=torch.bfloat16)
    lse = torch.zeros(16, device="cuda")
    # 65535 windows x 64 heads x 4096 tokens is far beyond the 4 Mi-float scratch: refused before any launch
    rc = _call_noalloc(lib, t, t, t, lse, t, 65535, 4096, 64, 64)
    assert rc == -41
