"""GPU checks of the small kernels and the whole-attention entry points through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from ring_attention_b200 import api
from ring_attention_b200._lib import SegMap
from util import assert_close, normal_inputs, round_to

pytestmark = pytest.mark.gpu


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda").to(dtype).contiguous()


@pytest.mark.parametrize("n", [0, 1, 7, 8, 1000, 4099, 1 << 20])
def test_casts_are_bit_exact(n):
    x = torch.from_numpy(oracle.xorshift32_fill(5, max(n, 1))[:n].copy()).cuda()
    h = torch.empty(n, dtype=torch.float16, device="cuda")
    api.launch_float_to_half(x, h)
    assert torch.equal(h, x.to(torch.float16))
    b = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    api.launch_float_to_bf16(x, b)
    assert torch.equal(b, x.to(torch.bfloat16))
    f = torch.empty(n, device="cuda")
    api.launch_half_to_float(h, f)
    assert torch.equal(f, h.float())
    i8 = torch.empty(n, dtype=torch.int8, device="cuda")
    api.launch_float_to_int8(x, i8)
    # fixed scale 127, round to nearest even, clamp (reference src/attention_step_fp16.cu:238-246)
    want = torch.clamp(torch.round(x * 127.0), -127, 127).to(torch.int8)
    assert torch.equal(i8, want)
    api.launch_int8_to_float(i8, f)
    assert torch.equal(f, i8.float() * (1.0 / 127.0))


def test_casts_on_unaligned_views():
    x = torch.randn(1003, device="cuda")
    h = torch.empty(1003, dtype=torch.float16, device="cuda")
    api.launch_float_to_half(x[1:], h[1:])
    assert torch.equal(h[1:], x[1:].to(torch.float16))


def test_init_finalize_lse():
    shape = api.AttentionShape(2, 3, 5, 5, 64)
    out = torch.randn((2, 3, 5, 64), device="cuda")
    m = torch.randn((2, 3, 5), device="cuda")
    l = torch.rand((2, 3, 5), device="cuda") + 0.5
    ref = out / l[..., None]
    lse = api.attention_lse(m, l)
    assert_close(lse.cpu().numpy(), (m + torch.log(l)).cpu().numpy(), 1e-6, 1e-6)
    l[0, 0, 0] = 0
    api.launch_attention_finalize(out, l, shape)
    ref[0, 0, 0] = 0
    assert_close(out.cpu().numpy(), ref.cpu().numpy(), 1e-6, 1e-6)
    api.launch_attention_init(out, m, l, shape)
    assert torch.all(out == 0) and torch.all(l == 0) and torch.all(torch.isneginf(m))


# reference tests/test_flash_attention.cu:77-121: ragged 33x47, Sq < Sk, GQA / MQA, D = 32..256
@pytest.mark.parametrize("cfg", [(1, 1, 1, 64, 64, 64), (2, 4, 4, 33, 47, 32), (1, 8, 2, 64, 128, 64),
                                 (1, 4, 1, 128, 128, 128), (1, 2, 2, 40, 40, 256), (1, 1, 1, 300, 300, 64)])
@pytest.mark.parametrize("causal", [False, True])
def test_flash_attention_entry_points(cfg, causal):
    B, H, kvH, Sq, Sk, D = cfg
    q, k, v = normal_inputs(77, B, H, kvH, Sq, Sk, D)
    shape = api.AttentionShape(B, H, Sq, Sk, D, kvH)
    out = torch.empty((B, H, Sq, D), device="cuda")
    api.launch_flash_attention(dev(q), dev(k), dev(v), out, shape, causal)
    assert_close(out.cpu().numpy(), oracle.cpu_attention(q, k, v, causal, kv_heads=kvH), 1e-5, 1e-5, "fp32")
    api.launch_flash_attention_fp16(dev(q), dev(k), dev(v), out, shape, causal)
    qh, kh, vh = (round_to(x, torch.float16) for x in (q, k, v))
    assert_close(out.cpu().numpy(), oracle.cpu_attention(qh, kh, vh, causal, kv_heads=kvH), 1e-3, 1e-3, "fp16")


# reference tests/test_naive_attention.cu:78-101: head sizes 16 and 24, Sq < Sk, GQA / MQA
@pytest.mark.parametrize("cfg", [(1, 1, 1, 8, 8, 16), (2, 4, 4, 32, 32, 32), (1, 2, 2, 16, 48, 24),
                                 (1, 1, 1, 64, 64, 64), (1, 8, 2, 32, 32, 32), (1, 4, 1, 32, 32, 32),
                                 (1, 2, 1, 130, 300, 200), (1, 1, 1, 5, 3, 7)])
@pytest.mark.parametrize("causal", [False, True])
def test_naive_attention_takes_any_head_dim(cfg, causal):
    B, H, kvH, Sq, Sk, D = cfg
    q, k, v = normal_inputs(78, B, H, kvH, Sq, Sk, D)
    out = torch.full((B, H, Sq, D), float("nan"), device="cuda")
    api.launch_naive_attention(dev(q), dev(k), dev(v), out, api.AttentionShape(B, H, Sq, Sk, D, kvH), causal)
    want = oracle.cpu_attention(q, k, v, causal, kv_heads=kvH)
    if causal and Sq > Sk:  # rows that see no key: zeros here, whatever the oracle's 0/0 gives
        hidden = np.arange(Sq) + (Sk - Sq) < 0
        want[:, :, hidden] = 0.0
    assert_close(out.cpu().numpy(), want, 1e-5, 1e-5)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_prefill_on_host_buffers(dtype):
    B, H, S, D = 1, 4, 512, 64
    q, k, v = normal_inputs(88, B, H, H, S, S, D)
    if dtype != torch.float32:
        q, k, v = (round_to(x, dtype) for x in (q, k, v))
    hq, hk, hv = (torch.from_numpy(x).to(dtype).pin_memory() for x in (q, k, v))
    one = SegMap.make([0], S)
    for _ in range(2):  # second call reuses the device scratch
        out, lse = api.prefill_host(hq, hk, hv, api.AttentionShape(B, H, S, S, D), one, one, causal=True,
                                    want_lse=True)
    want, want_lse = oracle.cpu_attention(q, k, v, True, want_lse=True)
    tol = 1e-5 if dtype == torch.float32 else 1e-3
    assert_close(out.numpy(), want, tol, tol, "out")
    assert_close(lse.numpy(), want_lse, tol, tol, "lse")


def _small_causal_case(seed=3, S=1024, D=64, H=2):
    q, k, v = normal_inputs(seed, 1, H, H, S, S, D)
    q, k, v = (round_to(x, torch.float16) for x in (q, k, v))
    return q, k, v, oracle.cpu_attention(q, k, v, True)


@pytest.mark.parametrize("D,cta_pair", [(64, False), (256, False), (128, True)])
def test_bounded_wait_runs_out_and_the_context_stays_usable(D, cta_pair):
    """The tcgen05 kernel's waits are bounded: with the TMA producer told to stop after the
    first K/V tiles and the limit set to a few milliseconds, the kernel returns by itself, the
    status word says which wait gave up, host entry points that synchronise report
    RA_ERR_DEVICE_WAIT, and after the word is read (which clears it) the same launch is right.
    Covers the three schedules of the kernel (head_dim 64, 256) and its cluster-pair form, where
    both blocks of a pair have to give up and meet at the cluster barrier."""
    from ring_attention_b200._lib import RingAttentionError, lib
    L = lib()
    S, H = 1024, 2
    q, k, v, want = _small_causal_case(S=S, D=D, H=H)
    dq, dk, dv = (dev(x, torch.float16) for x in (q, k, v))
    out = torch.zeros((1, H, S, D), device="cuda")
    m = torch.zeros((1, H, S), device="cuda")
    l = torch.zeros_like(m)
    one = SegMap.make([0], S)
    shape = api.AttentionShape(1, H, S, S, D)
    assert api.device_status()[0] == 0
    L.ra_debug_set_wait_limit_ns(5_000_000)
    L.ra_debug_stall_producer_after(2)
    try:
        api.attention_step_ex(dq, dk, dv, out, m, l, shape, one, one, causal=True, fresh=True, finalize=True,
                              cta_pair=cta_pair)
        torch.cuda.synchronize()  # returns: nothing waits forever
        # a host-buffer entry point synchronises, so it reports the failure itself
        hq, hk, hv = (torch.from_numpy(x).to(torch.float16).pin_memory() for x in (q, k, v))
        hout = torch.empty((1, H, S, D)).pin_memory()
        with pytest.raises(RingAttentionError) as err:
            api.check(L.ra_prefill_host(api.RA_F16, hq.data_ptr(), hk.data_ptr(), hv.data_ptr(),
                                        hout.data_ptr(), None, shape.c(), one, one, 1,
                                        api.RA_STEP_CAUSAL, 0))
        assert err.value.code == 5  # RA_ERR_DEVICE_WAIT
    finally:
        L.ra_debug_stall_producer_after(-1)
        L.ra_debug_set_wait_limit_ns(0)
    status = api.device_status()  # reads and clears
    assert status[0] == 5 and status[1] > 0, status
    assert api.device_status()[0] == 0
    api.attention_step_ex(dq, dk, dv, out, m, l, shape, one, one, causal=True, fresh=True, finalize=True,
                          cta_pair=cta_pair)
    torch.cuda.synchronize()
    assert api.device_status()[0] == 0
    assert_close(out.cpu().numpy(), want, 1e-3, 1e-3, "after the status word was cleared")
