"""GPU parity of the decode path (split-K kernel, KV cache, local decode op, partial merge)
against the CPU oracle, through the C ABI. Case lists follow the reference's
tests/test_decode_op.cu:50-189 (tolerance 1e-3 fp32 / 5e-2 fp16 there; 1e-5 / 1e-3 here) and
tests/test_kv_cache.cu:38-206 (slot-encoded values, exact equality)."""
import numpy as np
import pytest
import torch

import oracle
from ring_attention_b200 import api
from util import assert_close, normal_inputs, round_to

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.float16: 1e-3, torch.bfloat16: 1e-3}


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda").to(dtype).contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cfg", [  # B, H, kvH, Sk, D
    (1, 8, 8, 1024, 64), (1, 8, 8, 1000, 128), (2, 4, 4, 77, 32), (1, 2, 2, 513, 256),
    (4, 32, 8, 4096, 128), (1, 8, 2, 300, 64), (1, 4, 1, 129, 128), (2, 6, 3, 50, 64),
    (1, 16, 2, 2048, 128), (1, 3, 3, 1, 64)])
def test_decode_step_matches_oracle(dtype, cfg):
    B, H, kvH, Sk, D = cfg
    q, k, v = normal_inputs(101, B, H, kvH, 1, Sk, D)
    if dtype != torch.float32:
        q, k, v = (round_to(x, dtype) for x in (q, k, v))
    want, want_lse = oracle.cpu_attention(q, k, v, False, kv_heads=kvH, want_lse=True)
    shape = api.AttentionShape(B, H, 1, Sk, D, kvH)
    out = torch.full((B, H, 1, D), float("nan"), device="cuda")
    m = torch.empty((B, H, 1), device="cuda")
    l = torch.empty((B, H, 1), device="cuda")
    api.launch_attention_init(out, m, l, shape)
    api.launch_attention_decode_step(dev(q, dtype), dev(k, dtype), dev(v, dtype), out, m, l, shape,
                                     0, 0, False)
    lse = api.attention_lse(m, l)
    api.launch_attention_finalize(out, l, shape)
    assert_close(out.cpu().numpy(), want, TOL[dtype], TOL[dtype], "out")
    assert_close(lse.cpu().numpy(), want_lse, TOL[dtype], TOL[dtype], "lse")


def test_decode_causal_cutoff_chunks_and_strided_cache():
    # the cache is read in place (row stride S_max), in two chunks, with the causal cut-off
    # q_offset - k_offset + 1 (reference src/attention_decode.cu:110-116)
    B, H, kvH, D, S_max, n = 2, 8, 2, 128, 700, 640
    q, k, v = normal_inputs(7, B, H, kvH, 1, S_max, D)
    pos = 500  # the query sits at global position 500: keys 0..500 are visible
    want = oracle.cpu_attention(q, k[:, :, :pos + 1], v[:, :, :pos + 1], False, kv_heads=kvH)
    dk, dv, dq = dev(k), dev(v), dev(q)
    out = torch.zeros((B, H, 1, D), device="cuda")
    m = torch.full((B, H, 1), -float("inf"), device="cuda")
    l = torch.zeros((B, H, 1), device="cuda")
    for k_off, rows in ((0, 320), (320, n - 320)):
        # chunk starts k_off rows into every head; head stride stays S_max rows
        kc = dk.view(-1)[k_off * D:]
        vc = dv.view(-1)[k_off * D:]
        api.launch_attention_decode_step(dq, kc, vc, out, m, l,
                                         api.AttentionShape(B, H, 1, rows, D, kvH), pos, k_off, True,
                                         kv_row_stride=S_max)
    api.launch_attention_finalize(out, l, api.AttentionShape(B, H, 1, n, D, kvH))
    assert_close(out.cpu().numpy(), want, 1e-5, 1e-5)


def test_decode_dispatch_from_the_fp32_step_entry_point():
    # seq_q == 1 through launch_attention_step goes to the decode kernel (src/attention_step.cu:494-497)
    B, H, Sk, D = 1, 4, 333, 64
    q, k, v = normal_inputs(8, B, H, H, 1, Sk, D)
    shape = api.AttentionShape(B, H, 1, Sk, D)
    out = torch.zeros((B, H, 1, D), device="cuda")
    m = torch.full((B, H, 1), -float("inf"), device="cuda")
    l = torch.zeros((B, H, 1), device="cuda")
    api.launch_attention_step(dev(q), dev(k), dev(v), out, m, l, shape, Sk - 1, 0, True)
    api.launch_attention_finalize(out, l, shape)
    assert_close(out.cpu().numpy(), oracle.cpu_attention(q, k, v, False), 1e-5, 1e-5)


def test_decode_with_caller_workspace_and_too_small_workspace():
    B, H, Sk, D = 1, 8, 2048, 128
    q, k, v = normal_inputs(9, B, H, H, 1, Sk, D)
    shape = api.AttentionShape(B, H, 1, Sk, D)
    nbytes = api.lib().ra_decode_workspace_bytes(shape.c())
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = torch.zeros((B, H, 1, D), device="cuda")
    m = torch.full((B, H, 1), -float("inf"), device="cuda")
    l = torch.zeros((B, H, 1), device="cuda")
    api.launch_attention_decode_step(dev(q), dev(k), dev(v), out, m, l, shape, 0, 0, False, workspace=ws)
    api.launch_attention_finalize(out, l, shape)
    assert_close(out.cpu().numpy(), oracle.cpu_attention(q, k, v, False), 1e-5, 1e-5)
    with pytest.raises(api._lib.RingAttentionError) as e:
        api.launch_attention_decode_step(dev(q), dev(k), dev(v), out, m, l, shape, 0, 0, False,
                                         workspace=ws[:64])
    assert e.value.code == 6


# ---- KV cache (reference tests/test_kv_cache.cu) ---------------------------------------------

def slot_values(B, kvH, T, D, t0=0):
    b, h, t, d = np.meshgrid(np.arange(B), np.arange(kvH), np.arange(T) + t0, np.arange(D), indexing="ij")
    return (b * 1000 + h * 100 + t * 10 + d).astype(np.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_kv_cache_prefill_append_reset(dtype):
    B, kvH, S_max, D, P = 2, 3, 12, 8, 5
    c = api.DeviceKVCache(B, kvH, S_max, D, dtype)
    assert (c.current_len(), c.s_max(), c.numel()) == (0, S_max, B * kvH * S_max * D)
    kp = slot_values(B, kvH, P, D)
    c.copy_prefill(dev(kp, dtype), dev(-kp, dtype), P)
    assert c.current_len() == P
    for t in range(P, P + 3):
        step = slot_values(B, kvH, 1, D, t0=t)
        c.append(dev(step, dtype), dev(-step, dtype))
    assert c.current_len() == P + 3
    torch.cuda.synchronize()
    want = slot_values(B, kvH, P + 3, D)
    kk = c.k_view().float().cpu().numpy()
    vv = c.v_view().float().cpu().numpy()
    assert np.array_equal(kk[:, :, :P + 3], want) and np.array_equal(vv[:, :, :P + 3], -want)
    c.reset()
    assert c.current_len() == 0
    with pytest.raises(api._lib.RingAttentionError):
        c.copy_prefill(dev(kp, dtype), dev(kp, dtype), S_max + 1)
    c.copy_prefill(dev(slot_values(B, kvH, S_max, D), dtype), dev(slot_values(B, kvH, S_max, D), dtype), S_max)
    with pytest.raises(api._lib.RingAttentionError) as e:
        c.append(dev(kp[:, :, :1], dtype), dev(kp[:, :, :1], dtype))
    assert "cache full" in str(e.value)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("cfg", [(1, 8, 8, 64, 64), (2, 8, 2, 200, 128), (1, 4, 1, 33, 32)])
def test_local_decode_step_is_last_row_of_causal_attention(dtype, cfg):
    # reference tests/test_decode_op.cu:50-189: decode of token t == row t of full causal attention
    B, H, kvH, S, D = cfg
    q, k, v = normal_inputs(55, B, H, kvH, S, S, D)
    if dtype != torch.float32:
        q, k, v = (round_to(x, dtype) for x in (q, k, v))
    full = oracle.cpu_attention(q, k, v, True, kv_heads=kvH)
    c = api.DeviceKVCache(B, kvH, S + 4, D, dtype)
    c.copy_prefill(dev(k[:, :, :S - 2], dtype), dev(v[:, :, :S - 2], dtype), S - 2)
    out = torch.empty((B, H, 1, D), device="cuda")
    for t in (S - 2, S - 1):
        c.append(dev(k[:, :, t:t + 1], dtype), dev(v[:, :, t:t + 1], dtype))
        api.run_local_decode_step(dev(q[:, :, t:t + 1], dtype), c, H, t, 0, True, out)
        assert_close(out.cpu().numpy(), full[:, :, t:t + 1], TOL[dtype], TOL[dtype], f"t={t}")


def test_partial_merge_matches_oracle():
    BH, D, cp = 12, 64, 4
    rng = np.random.default_rng(3)
    blocks = []
    for r in range(cp):
        o = rng.standard_normal((BH, D)).astype(np.float32)
        m = rng.standard_normal(BH).astype(np.float32)
        l = rng.uniform(0.5, 3.0, BH).astype(np.float32)
        if r == 2:
            m[5], l[5], o[5] = -np.inf, 0, 0
        blocks.append(np.concatenate([o.ravel(), m, l]))
    g = np.concatenate(blocks)
    want_o, want_m, want_l = oracle.decode_partial_merge(g, cp, BH, D)
    out = torch.empty((BH, D), device="cuda")
    m = torch.empty(BH, device="cuda")
    l = torch.empty(BH, device="cuda")
    api.check(api.lib().ra_decode_partial_merge(api._ptr(dev(g)), api._ptr(out), api._ptr(m), api._ptr(l),
                                                cp, BH, D, 0, api._stream()))
    assert_close(out.cpu().numpy(), want_o, 1e-6, 1e-6)
    assert_close(m.cpu().numpy(), want_m, 0, 0)
    assert_close(l.cpu().numpy(), want_l, 1e-6, 1e-6)


def test_golden_decode_trajectory_single_rank_ring(golden_dir):
    """The Python reference's prefill + 6 decode steps (cp=2 there); here both shards live in
    two caches on one GPU, partials are merged as the ring does, outputs must match."""
    import os
    g = np.load(os.path.join(golden_dir, "gen_decode_cp2.npz"))
    k, v = g["k"], g["v"]
    B, H, S, D = k.shape
    cp, steps = 2, g["dq"].shape[0]
    caches = []
    for r in range(cp):
        c = api.DeviceKVCache(B, H, S // cp + steps, D)
        sl = slice(r * S // cp, (r + 1) * S // cp)
        c.copy_prefill(dev(k[:, :, sl]), dev(v[:, :, sl]), S // cp)
        caches.append(c)
    bh = B * H
    for t in range(steps):
        owner = t % cp
        caches[owner].append(dev(g["dk"][t]), dev(g["dv"][t]))
        blocks = []
        for r in range(cp):
            buf = torch.empty(bh * D + 2 * bh, device="cuda")
            o, m, l = buf[:bh * D], buf[bh * D:bh * D + bh], buf[bh * D + bh:]
            shape = api.AttentionShape(B, H, 1, caches[r].current_len(), D)
            api.launch_attention_init(o, m, l, shape)
            api.check(api.lib().ra_attention_decode_step(
                0, api._ptr(dev(g["dq"][t])), caches[r].k_ptr(), caches[r].v_ptr(), api._ptr(o), api._ptr(m),
                api._ptr(l), shape.c(), 0, 0, 0, api._stream(), caches[r].s_max(), None, 0))
            blocks.append(buf)
        gathered = torch.cat(blocks)
        out = torch.empty((B, H, 1, D), device="cuda")
        api.check(api.lib().ra_decode_partial_merge(api._ptr(gathered), api._ptr(out), None, None, cp, bh, D, 1,
                                                    api._stream()))
        assert_close(out.cpu().numpy(), g["dout"][t], 1e-5, 1e-5, f"decode step {t}")
