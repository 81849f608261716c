"""The decode entry point for callers that may not allocate device memory.

Some users of this library run where cudaMalloc is off limits: the process has handed all device
memory to its own arena, or the call sits in a section that must not enter the CUDA allocator.
``ra_attention_decode_step_noalloc`` serves them from a fixed 1 MiB scratch array inside the
library. This file checks, through the C ABI, that it returns what the ordinary entry point
returns (same tolerances as the other decode tests: 1e-5 for fp32, 1e-3 for fp16), on two calls
in a row (the array is shared and keeps the previous call's contents), and that a problem too
large for the array is refused with a message that names the limit. It is collected last on
purpose and must also pass alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from ring_attention_b200 import api
from ring_attention_b200._lib import RA_F16, RA_F32, lib
from util import assert_close

pytestmark = pytest.mark.gpu


def fresh_state(B, H, D):
    out = torch.zeros((B, H, 1, D), device="cuda")
    m = torch.full((B, H, 1), -float("inf"), device="cuda")
    l = torch.zeros((B, H, 1), device="cuda")
    return out, m, l


def call(entry, dtype_code, q, k, v, shape, causal, q_off, stride_rows):
    out, m, l = fresh_state(shape.batch, shape.heads, shape.head_dim)
    args = [dtype_code, api._ptr(q), api._ptr(k), api._ptr(v), api._ptr(out), api._ptr(m), api._ptr(l),
            C.byref(shape.c()), q_off, 0, int(causal), api._stream(), stride_rows]
    if entry == "plain":
        args += [None, 0]
        api.check(lib().ra_attention_decode_step(*args))
    else:
        api.check(lib().ra_attention_decode_step_noalloc(*args))
    api.launch_attention_finalize(out, l, shape)
    torch.cuda.synchronize()
    return out.cpu().numpy(), m.cpu().numpy()


@pytest.mark.parametrize("dtype,code,tol", [(torch.float32, RA_F32, 1e-5), (torch.float16, RA_F16, 1e-3)])
def test_noalloc_decode_matches_the_ordinary_entry_point_twice_in_a_row(dtype, code, tol):
    g = torch.Generator(device="cuda").manual_seed(1234)
    # first call: GQA cache read in place with a row stride; second call: a different, larger
    # problem, so slots written by the first call are reused with other contents
    problems = [(2, 8, 2, 128, 5000, 6000, True, 4100), (4, 32, 8, 128, 20000, 20000, False, 0)]
    for (B, H, kvH, D, L, s_max, causal, q_off) in problems:
        k = torch.randn((B, kvH, s_max, D), generator=g, device="cuda").to(dtype)
        v = torch.randn((B, kvH, s_max, D), generator=g, device="cuda").to(dtype)
        q = torch.randn((B, H, 1, D), generator=g, device="cuda").to(dtype)
        shape = api.AttentionShape(B, H, 1, L, D, kvH)
        want, want_m = call("plain", code, q, k, v, shape, causal, q_off, s_max)
        got, got_m = call("noalloc", code, q, k, v, shape, causal, q_off, s_max)
        assert_close(got, want, tol, tol, f"out B{B} H{H} L{L}")
        assert_close(got_m, want_m, tol, tol, "m")
        assert np.isfinite(got).all()


def test_noalloc_decode_refuses_problems_beyond_its_scratch():
    B, H, D, L = 64, 64, 128, 256  # 64*64*130 floats > 262144
    z = torch.zeros((B, H, L, D), device="cuda", dtype=torch.float16)
    q = torch.zeros((B, H, 1, D), device="cuda", dtype=torch.float16)
    out, m, l = fresh_state(B, H, D)
    shape = api.AttentionShape(B, H, 1, L, D)
    rc = lib().ra_attention_decode_step_noalloc(RA_F16, api._ptr(q), api._ptr(z), api._ptr(z), api._ptr(out),
                                                api._ptr(m), api._ptr(l), C.byref(shape.c()), 0, 0, 0,
                                                api._stream(), 0)
    assert rc == 6  # RA_ERR_OVERFLOW
    msg = lib().ra_last_error().decode()
    assert "exceeds the built-in scratch" in msg and "262144" in msg
    torch.cuda.synchronize()
    assert torch.all(out == 0)  # nothing ran
