"""Full-size checks at the benchmark's shapes, where the O(S^2) oracle is too slow: sampled
rows against the CPU oracle, and size-independent properties (the ring decomposition of the
same work gives the same answer; linearity in V)."""
import numpy as np
import pytest
import torch

import oracle
from ring_attention_b200 import api
from ring_attention_b200._lib import SegMap
from util import assert_close

pytestmark = pytest.mark.gpu


def gen(seed, shape, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.float16)


def sampled_rows_check(q, k, v, out, lse, rows, heads, tol=1e-3):
    kvH = k.shape[1]
    for h in heads:
        kk = k[0, h % kvH].float().cpu().numpy()
        vv = v[0, h % kvH].float().cpu().numpy()
        for i in rows:
            o, ls = oracle.attention_row(q[0, h, i].float().cpu().numpy(), kk[:i + 1], vv[:i + 1])
            assert_close(out[0, h, i].cpu().numpy(), o, tol, tol, f"head {h} row {i}")
            assert abs(float(lse[0, h, i]) - ls) <= tol + tol * abs(ls)


def test_config2_shape_causal_fp16_sampled_rows_and_ring_decomposition():
    # B1 H8 S32768 D64 fp16 causal: one launch over the whole sequence ...
    B, H, S, D = 1, 8, 32768, 64
    q, k, v = gen(1, (B, H, S, D)), gen(2, (B, H, S, D)), gen(3, (B, H, S, D))
    shape = api.AttentionShape(B, H, S, S, D)
    out = torch.empty((B, H, S, D), device="cuda")
    m = torch.empty((B, H, S), device="cuda")
    l = torch.empty((B, H, S), device="cuda")
    one = SegMap.make([0], S)
    api.attention_step_ex(q, k, v, out, m, l, shape, one, one, causal=True, fresh=True, finalize=True)
    lse = api.attention_lse(m, l)
    torch.cuda.synchronize()
    assert api.device_status()[0] == 0
    rows = [0, 1, 127, 128, 129, 255, 256, 4095, 4096, 16383, 16384, 20000, 32767]
    sampled_rows_check(q, k, v, out, lse, rows, heads=[0, 5])
    # ... equals a zig-zag ring of 4 ranks played on this GPU (each rank: its rows, 4 steps)
    full = torch.empty_like(out)
    for rank in range(4):
        p = api.RingPartition(4, rank, S, api.RingPartition.ZIGZAG, 2)
        rows_r = p.local_positions().cuda()
        ql = q[:, :, rows_r].contiguous()
        o_r = torch.empty((B, H, len(rows_r), D), device="cuda")
        m_r = torch.empty((B, H, len(rows_r)), device="cuda")
        l_r = torch.empty_like(m_r)
        for step in range(4):
            qmap, kmap, stride = p.step_maps(step)
            src = api.RingPartition(4, (rank - step) % 4, S, api.RingPartition.ZIGZAG, 2).local_positions().cuda()
            api.attention_step_ex(ql, k[:, :, src].contiguous(), v[:, :, src].contiguous(), o_r, m_r, l_r,
                                  api.AttentionShape(B, H, len(rows_r), len(src), D), qmap, kmap, stride,
                                  causal=True, fresh=(step == 0), finalize=(step == 3))
        full[:, :, rows_r] = o_r
    torch.cuda.synchronize()
    assert api.device_status()[0] == 0
    assert_close(full.cpu().numpy(), out.cpu().numpy(), 1e-3, 1e-3, "ring decomposition")


def test_gqa_d128_striped_rank_sampled_rows():
    # the layout of the GQA benchmark shape at reduced length: H32 / kvH8, D128, striped rank of 8
    B, H, kvH, S, D, cp, rank = 1, 32, 8, 16384, 128, 8, 3
    q, k, v = gen(4, (B, H, S, D), 0.5), gen(5, (B, kvH, S, D), 0.5), gen(6, (B, kvH, S, D), 0.5)
    p = api.RingPartition(cp, rank, S, api.RingPartition.STRIPED)
    rows_r = p.local_positions().cuda()
    ql = q[:, :, rows_r].contiguous()
    n = len(rows_r)
    o = torch.empty((B, H, n, D), device="cuda")
    m = torch.empty((B, H, n), device="cuda")
    l = torch.empty_like(m)
    for step in range(cp):
        qmap, kmap, stride = p.step_maps(step)
        src = api.RingPartition(cp, (rank - step) % cp, S, api.RingPartition.STRIPED).local_positions().cuda()
        api.attention_step_ex(ql, k[:, :, src].contiguous(), v[:, :, src].contiguous(), o, m, l,
                              api.AttentionShape(B, H, n, n, D, kvH), qmap, kmap, stride, causal=True,
                              fresh=(step == 0), finalize=(step == cp - 1))
    lse = api.attention_lse(m, l)
    torch.cuda.synchronize()
    assert api.device_status()[0] == 0
    for h in (0, 9, 31):
        kk, vv = k[0, h % kvH].float().cpu().numpy(), v[0, h % kvH].float().cpu().numpy()
        for li in (0, 1, 100, 1023, 2047):
            g = int(rows_r[li])
            want, ls = oracle.attention_row(q[0, h, g].float().cpu().numpy(), kk[:g + 1], vv[:g + 1])
            assert_close(o[0, h, li].cpu().numpy(), want, 1e-3, 1e-3, f"h{h} row {g}")
            assert abs(float(lse[0, h, li]) - ls) <= 1e-3 + 1e-3 * abs(ls)


def test_decode_full_size_cache_linearity_and_sampled_heads():
    # B4 H32 kvH8 D128 fp16 cache of 262144 rows per head (4.3 GB): one decode step.
    B, H, kvH, L, D = 4, 32, 8, 262144, 128
    k, v, q = gen(7, (B, kvH, L, D)), gen(8, (B, kvH, L, D)), gen(9, (B, H, 1, D))
    shape = api.AttentionShape(B, H, 1, L, D, kvH)

    def run(vv):
        out = torch.empty((B, H, 1, D), device="cuda")
        m = torch.empty((B, H, 1), device="cuda")
        l = torch.empty((B, H, 1), device="cuda")
        api.launch_attention_init(out, m, l, shape)
        api.launch_attention_decode_step(q, k, vv, out, m, l, shape, 0, 0, False)
        api.launch_attention_finalize(out, l, shape)
        return out

    out = run(v)
    for (b, h) in ((0, 0), (3, 31), (1, 13)):
        want, _ = oracle.attention_row(q[b, h, 0].float().cpu().numpy(), k[b, h % kvH].float().cpu().numpy(),
                                       v[b, h % kvH].float().cpu().numpy())
        assert_close(out[b, h, 0].cpu().numpy(), want, 1e-3, 1e-3, f"b{b} h{h}")
    # linear in V: attention(q, k, 2v) == 2 attention(q, k, v) (doubling is exact in fp16)
    out2 = run(v * 2)
    assert_close(out2.cpu().numpy(), 2 * out.cpu().numpy(), 1e-6, 1e-6, "linearity")


def test_host_buffer_prefill_pipelined_equals_device_resident_result():
    # the benchmark shape through the host-buffer entry point (pipelined over head groups) must
    # give exactly what the same kernel gives on device-resident tensors
    B, H, S, D = 1, 8, 32768, 64
    q, k, v = gen(11, (B, H, S, D)), gen(12, (B, H, S, D)), gen(13, (B, H, S, D))
    shape = api.AttentionShape(B, H, S, S, D)
    out = torch.empty((B, H, S, D), device="cuda")
    m = torch.empty((B, H, S), device="cuda")
    l = torch.empty((B, H, S), device="cuda")
    one = SegMap.make([0], S)
    api.attention_step_ex(q, k, v, out, m, l, shape, one, one, causal=True, fresh=True, finalize=True)
    lse = api.attention_lse(m, l)
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    for _ in range(2):
        h_out, h_lse = api.prefill_host(hq, hk, hv, shape, one, one, causal=True, want_lse=True)
    assert torch.equal(h_out, out.cpu()) and torch.equal(h_lse, lse.cpu())
