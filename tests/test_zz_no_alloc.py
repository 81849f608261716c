"""The decode entry point for callers that may not allocate device memory.

Some users of this library run where cudaMalloc is off limits: the process has handed all device
memory to its own arena, or the call sits in a section that must not enter the CUDA allocator.
``ra_attention_decode_step_noalloc`` serves them from a fixed 1 MiB scratch array inside the
library. This file checks, through the C ABI, that it returns what the ordinary entry point
returns (same tolerances as the other decode tests: 1e-5 for fp32, 1e-3 for fp16), on two calls
in a row (the array is shared and keeps the previous call's contents), and that a problem too
large for the array is refused with a message that names the limit. A third case is sized so
that the array forces fewer key splits than the scheduler would like (the branch that makes this
entry point different), and is checked against the CPU oracle directly; around a warmed-up call
the free device memory must not move. It is collected last on purpose and must also pass alone
in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
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


def test_noalloc_decode_with_the_split_count_capped_by_the_array_against_the_oracle():
    # batch 8 x 64 heads x (128 + 2) floats per split leaves room for 3 splits in the 262144-float
    # array, far fewer than the ~14 the scheduler wants on 148 SMs: the capped branch runs
    B, H, kvH, D, L = 8, 64, 8, 128, 3000
    assert 262144 // (B * H * (D + 2)) == 3
    g = torch.Generator(device="cuda").manual_seed(99)
    k = torch.randn((B, kvH, L, D), generator=g, device="cuda").to(torch.float16)
    v = torch.randn((B, kvH, L, D), generator=g, device="cuda").to(torch.float16)
    q = torch.randn((B, H, 1, D), generator=g, device="cuda").to(torch.float16)
    shape = api.AttentionShape(B, H, 1, L, D, kvH)
    got, _ = call("noalloc", RA_F16, q, k, v, shape, False, 0, L)  # warms up: address lookup, attributes
    free_before = torch.cuda.mem_get_info()[0]
    got, _ = call("noalloc", RA_F16, q, k, v, shape, False, 0, L)
    assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
    want = oracle.cpu_attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                                False, kv_heads=kvH)
    assert_close(got, want, 1e-3, 1e-3, "capped splits vs CPU oracle")
    plain, _ = call("plain", RA_F16, q, k, v, shape, False, 0, L)
    assert_close(got, plain, 1e-3, 1e-3, "capped splits vs ordinary entry point")


def test_noalloc_decode_on_a_second_device_if_there_is_one():
    # the array's address is looked up per device: a call on device 1 must use device 1's copy
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with torch.cuda.device(1):
        g = torch.Generator(device="cuda:1").manual_seed(5)
        B, H, kvH, D, L = 2, 8, 2, 64, 2000
        k = torch.randn((B, kvH, L, D), generator=g, device="cuda:1").to(torch.float16)
        v = torch.randn((B, kvH, L, D), generator=g, device="cuda:1").to(torch.float16)
        q = torch.randn((B, H, 1, D), generator=g, device="cuda:1").to(torch.float16)
        shape = api.AttentionShape(B, H, 1, L, D, kvH)
        out = torch.zeros((B, H, 1, D), device="cuda:1")
        m = torch.full((B, H, 1), -float("inf"), device="cuda:1")
        l = torch.zeros((B, H, 1), device="cuda:1")
        api.check(lib().ra_attention_decode_step_noalloc(
            RA_F16, api._ptr(q), api._ptr(k), api._ptr(v), api._ptr(out), api._ptr(m), api._ptr(l),
            C.byref(shape.c()), 0, 0, 0, api._stream(), L))
        api.launch_attention_finalize(out, l, shape)
        torch.cuda.synchronize()
        want = oracle.cpu_attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                                    False, kv_heads=kvH)
        assert_close(out.cpu().numpy(), want, 1e-3, 1e-3, "device 1 vs CPU oracle")


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
