"""GPU parity of the ring-step kernels against the CPU oracle, called through the C ABI.

Tolerances: fp32 path 1e-5 (atol = rtol); fp16 / bf16 paths atol = rtol = 1e-3 (fp16) and 8e-3
(bf16, whose P has 8 mantissa bits) against the oracle run on the SAME 16-bit-rounded inputs
widened to fp32. The case lists follow the reference's tests/test_attention_step.cu:136-176
and tests/test_attention_step_fp16.cu:130-166 (single-GPU ring simulation: K/V split into P
chunks, one step call per chunk, finalize, compare with full attention)."""
import os

import numpy as np
import pytest
import torch

import oracle
from ring_attention_b200 import api
from ring_attention_b200._lib import SegMap
from util import assert_close, normal_inputs, round_to

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float16: 1e-3, torch.bfloat16: 8e-3}


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda").to(dtype).contiguous()


def state(B, H, Sq, D, poison=False):
    out = torch.full((B, H, Sq, D), float("nan") if poison else 0.0, device="cuda")
    m = torch.full((B, H, Sq), float("nan") if poison else -float("inf"), device="cuda")
    l = torch.full((B, H, Sq), float("nan") if poison else 0.0, device="cuda")
    return out, m, l


def xorshift_inputs(seed, B, H, kvH, Sq, Sk, D):
    # the reference's tests draw q, then k, then v from one XorShift32 stream
    n_q, n_k = B * H * Sq * D, B * kvH * Sk * D
    flat = oracle.xorshift32_fill(seed, n_q + 2 * n_k)
    return (flat[:n_q].reshape(B, H, Sq, D), flat[n_q:n_q + n_k].reshape(B, kvH, Sk, D),
            flat[n_q + n_k:].reshape(B, kvH, Sk, D))


def ring_sim(q, k, v, chunks, causal, dtype, kvH, step_fn):
    """K/V in `chunks` pieces, one step call per piece (the reference's ring simulation)."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    n = Sk // chunks
    dq = dev(q, dtype)
    out, m, l = state(B, H, Sq, D, poison=True)
    full = api.AttentionShape(B, H, Sq, Sk, D, kvH)
    api.launch_attention_init(out, m, l, full)
    for p in range(chunks):
        dk = dev(k[:, :, p * n:(p + 1) * n], dtype)
        dv = dev(v[:, :, p * n:(p + 1) * n], dtype)
        step_fn(dq, dk, dv, out, m, l, api.AttentionShape(B, H, Sq, n, D, kvH), 0, p * n, causal)
    lse = api.attention_lse(m, l)
    api.launch_attention_finalize(out, l, full)
    torch.cuda.synchronize()
    assert api.device_status()[0] == 0
    return out.cpu().numpy(), lse.cpu().numpy()


# (B, H, kvH, Sq, Sk, D, chunks, causal, seed): reference tests/test_attention_step_fp16.cu:130-166
REF_CASES = [
    (1, 1, 1, 32, 64, 64, 2, False, 1), (1, 1, 1, 32, 64, 64, 4, False, 2),
    (2, 4, 4, 32, 128, 64, 4, False, 3), (1, 1, 1, 64, 64, 64, 2, True, 4),
    (1, 1, 1, 64, 64, 64, 4, True, 5), (2, 2, 2, 128, 128, 64, 4, True, 6),
    (1, 1, 1, 64, 64, 32, 4, True, 7), (1, 1, 1, 64, 64, 128, 2, True, 8),
    (1, 1, 1, 64, 64, 256, 2, False, 11), (1, 2, 2, 64, 64, 256, 2, True, 12),
    (1, 2, 2, 32, 64, 64, 1, False, 9), (1, 2, 2, 64, 64, 64, 1, True, 10),
    (1, 8, 2, 64, 64, 64, 2, False, 11), (1, 8, 2, 64, 64, 64, 2, True, 12),
    (1, 4, 1, 64, 64, 64, 4, False, 13), (1, 4, 1, 64, 64, 64, 4, True, 14),
]


@pytest.mark.parametrize("case", REF_CASES)
def test_fp16_step_reference_case_list(case):
    B, H, kvH, Sq, Sk, D, chunks, causal, seed = case
    q, k, v = xorshift_inputs(seed, B, H, kvH, Sq, Sk, D)
    q, k, v = (round_to(x, torch.float16) for x in (q, k, v))
    want, want_lse = oracle.cpu_attention(q, k, v, causal, kv_heads=kvH, want_lse=True)
    got, lse = ring_sim(q, k, v, chunks, causal, torch.float16, kvH, api.launch_attention_step_fp16)
    assert_close(got, want, 1e-3, 1e-3, "out")
    assert_close(lse, want_lse, 1e-3, 1e-3, "lse")


@pytest.mark.parametrize("case", REF_CASES)
def test_fp32_step_reference_case_list(case):
    B, H, kvH, Sq, Sk, D, chunks, causal, seed = case
    q, k, v = xorshift_inputs(seed, B, H, kvH, Sq, Sk, D)
    want, want_lse = oracle.cpu_attention(q, k, v, causal, kv_heads=kvH, want_lse=True)
    got, lse = ring_sim(q, k, v, chunks, causal, torch.float32, kvH, api.launch_attention_step)
    assert_close(got, want, 1e-5, 1e-5, "out")
    assert_close(lse, want_lse, 1e-5, 1e-5, "lse")


@pytest.mark.parametrize("D", [32, 64, 128])
def test_fp32_tensor_core_and_simt_kernels_agree_with_the_oracle_at_1e5(D):
    # long rows, GQA, ragged lengths, end-aligned causal mask, inputs of mixed magnitudes: the
    # split-TF32 kernel (hi*hi + lo*hi + hi*lo) must hold the fp32 tolerance like the SIMT one
    q, k, v = normal_inputs(5 + D, 1, 4, 2, 333, 1500, D)
    q[:, :, :, 0] *= 2.0
    k[:, :, ::7] *= 0.05
    v[:, :, ::5] *= 3.0
    want, want_lse = oracle.cpu_attention(q, k, v, True, kv_heads=2, want_lse=True)
    qmap, kmap = SegMap.make([1500 - 333], 333), SegMap.make([0], 1500)
    for force_simt in (False, True):
        got, lse = run_ex(q, k, v, qmap, kmap, 1, True, torch.float32, 2, force_simt=force_simt)
        assert_close(got, want, 1e-5, 1e-5, f"out D={D} simt={force_simt}")
        assert_close(lse, want_lse, 1e-5, 1e-5, f"lse D={D} simt={force_simt}")


def test_config1_fp32_noncausal_mha_output_and_lse():
    # B1 H8 S1024 D64 fp32 N(0,1), non-causal, one rank: output and log-sum-exp element-wise
    q, k, v = normal_inputs(42, 1, 8, 8, 1024, 1024, 64)
    want, want_lse = oracle.cpu_attention(q, k, v, False, want_lse=True)
    got, lse = ring_sim(q, k, v, 1, False, torch.float32, 8, api.launch_attention_step)
    assert_close(got, want, 1e-5, 1e-5, "out")
    assert_close(lse, want_lse, 1e-5, 1e-5, "lse")


def run_ex(q, k, v, qmap, kmap, stride, causal, dtype, kvH, doc_len=0, force_simt=False,
           p_in_smem=False, cta_pair=False):
    B, H, Sq, D = q.shape
    out, m, l = state(B, H, Sq, D, poison=True)
    api.attention_step_ex(dev(q, dtype), dev(k, dtype), dev(v, dtype), out, m, l,
                          api.AttentionShape(B, H, Sq, k.shape[2], D, kvH), qmap, kmap, stride,
                          causal=causal, fresh=True, finalize=True, doc_len=doc_len,
                          force_simt=force_simt, p_in_smem=p_in_smem, cta_pair=cta_pair)
    torch.cuda.synchronize()
    assert api.device_status()[0] == 0
    return out.cpu().numpy(), api.attention_lse(m, l).cpu().numpy()


def masked_truth(q, k, v, qpos, kpos, causal, doc_len, kvH):
    """Oracle for arbitrary position maps: one row at a time with an explicit visibility mask."""
    B, H, Sq, D = q.shape
    out = np.zeros_like(q)
    lse = np.zeros((B, H, Sq), np.float32)
    for b in range(B):
        for h in range(H):
            for i in range(Sq):
                vis = np.ones(len(kpos), bool)
                if causal:
                    vis &= kpos <= qpos[i]
                if doc_len:
                    vis &= (kpos // doc_len) == (qpos[i] // doc_len)
                out[b, h, i], lse[b, h, i] = oracle.attention_row(q[b, h, i], k[b, h % kvH], v[b, h % kvH], vis)
    return out, lse


def positions(sm, stride):
    return np.concatenate([sm.base[s] + np.arange(sm.seg_len) * stride for s in range(sm.n_seg)])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("simt", [False, True])
def test_segmented_zigzag_step_all_paths(dtype, D, simt):
    # rank 1 of 4, zig-zag with 4 sub-groups, ring step 2: q and k segments at scattered bases
    cp, rank, S, ns = 4, 1, 4 * 4 * 48, 4
    p = api.RingPartition(cp, rank, S, api.RingPartition.ZIGZAG, ns)
    qmap, kmap, stride = p.step_maps(2)
    Sl = ns * p.local_chunk_len()
    q, k, v = normal_inputs(3, 1, 4, 2, Sl, Sl, D)
    if dtype != torch.float32:
        q, k, v = (round_to(x, dtype) for x in (q, k, v))
    want, want_lse = masked_truth(q, k, v, positions(qmap, stride), positions(kmap, stride), True, 0, 2)
    got, lse = run_ex(q, k, v, qmap, kmap, stride, True, dtype, 2, force_simt=simt)
    tol = TOL[dtype]
    assert_close(got, want, tol, tol, "out")
    seen = np.isfinite(want_lse)
    assert_close(lse[seen], want_lse[seen], tol, tol, "lse")
    assert np.all(np.isneginf(lse[~seen]))


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_striped_step(dtype):
    cp, rank, S = 4, 2, 4 * 200
    p = api.RingPartition(cp, rank, S, api.RingPartition.STRIPED)
    for step in (0, 1, 3):
        qmap, kmap, stride = p.step_maps(step)
        q, k, v = normal_inputs(4 + step, 2, 4, 4, 200, 200, 64, scale=0.5)
        if dtype != torch.float32:
            q, k, v = (round_to(x, dtype) for x in (q, k, v))
        want, _ = masked_truth(q, k, v, positions(qmap, stride), positions(kmap, stride), True, 0, 4)
        got, _ = run_ex(q, k, v, qmap, kmap, stride, True, dtype, 4)
        assert_close(got, want, TOL[dtype], TOL[dtype], f"step {step}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("doc_len", [96, 100, 384])
def test_document_mask(dtype, doc_len):
    # documents of doc_len tokens; boundaries aligned (96, 384) and not aligned (100) to segments
    qmap = SegMap.make([0, 576], 192)
    kmap = SegMap.make([192, 384], 192)
    q, k, v = normal_inputs(9, 1, 2, 2, 384, 384, 64)
    if dtype != torch.float32:
        q, k, v = (round_to(x, dtype) for x in (q, k, v))
    want, want_lse = masked_truth(q, k, v, positions(qmap, 1), positions(kmap, 1), True, doc_len, 2)
    got, lse = run_ex(q, k, v, qmap, kmap, 1, True, dtype, 2, doc_len=doc_len)
    assert_close(got, want, TOL[dtype], TOL[dtype], "out")
    assert np.array_equal(np.isneginf(lse), np.isneginf(want_lse))


@pytest.mark.parametrize("shape", [(33, 47), (1, 130), (129, 1), (257, 300), (5, 5)])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_shapes_fp16(shape, causal):
    Sq, Sk = shape
    q, k, v = normal_inputs(12, 1, 2, 1, Sq, Sk, 64)
    q, k, v = (round_to(x, torch.float16) for x in (q, k, v))
    qmap, kmap = SegMap.make([max(Sk - Sq, 0)], Sq), SegMap.make([0], Sk)
    want, _ = masked_truth(q, k, v, positions(qmap, 1), positions(kmap, 1), causal, 0, 1)
    got, _ = run_ex(q, k, v, qmap, kmap, 1, causal, torch.float16, 1)
    assert_close(got, want, 1e-3, 1e-3, "out")


@pytest.mark.parametrize("dtype,D", [(torch.float16, 64), (torch.float16, 128), (torch.float16, 256),
                                     (torch.bfloat16, 64), (torch.float32, 64), (torch.float32, 128)])
def test_scores_that_grow_along_the_keys_move_the_reference_point(dtype, D):
    # The tensor-core kernels keep a row's reference point from tile to tile and move it only when
    # a tile's row sum shows that some score ran far above it. Here the scores climb by ~24 in the
    # exponent from one key tile to the next (and vary inside a tile), so that path, with its
    # rescale of O and l and the recomputed tile, runs on almost every tile; rows of the second
    # head fall instead, which never moves the reference.
    S = 1024
    rng = np.random.default_rng(11)
    q = np.zeros((1, 2, 256, D), np.float32)
    k = np.zeros((1, 2, S, D), np.float32)
    q[..., 0] = 1.0
    ramp = np.arange(S, dtype=np.float32) / 128.0 * 17.0 * np.sqrt(D)  # ~17 nats per 128 keys
    k[0, 0, :, 0] = ramp / 4.0
    k[0, 1, :, 0] = -ramp / 4.0
    q[..., 0] = 4.0
    q[..., 1:] = rng.standard_normal((1, 2, 256, D - 1)).astype(np.float32) * 0.3
    k[..., 1:] = rng.standard_normal((1, 2, S, D - 1)).astype(np.float32) * 0.3
    v = rng.standard_normal((1, 2, S, D)).astype(np.float32)
    q, k, v = (round_to(x, dtype) for x in (q, k, v))
    want, want_lse = oracle.cpu_attention(q, k, v, True, want_lse=True)
    qmap, kmap = SegMap.make([S - 256], 256), SegMap.make([0], S)
    got, lse = run_ex(q, k, v, qmap, kmap, 1, True, dtype, 2)
    # fp32: the raw scores reach ~1000, where one fp32 ulp of the score is already 1e-4 (1.5e-5 in
    # the exponent after scaling), so two correct fp32 summation orders differ by more than 1e-5
    tol = 1e-4 if dtype == torch.float32 else TOL[dtype]
    assert_close(got, want, tol, tol, "out")
    assert_close(lse, want_lse, tol, tol, "lse")


def test_every_reference_head_dim_takes_the_tensor_core_kernel_in_16_bit():
    from ring_attention_b200._lib import RA_BF16, RA_F16, RA_F32, lib
    for D in (32, 64, 128, 256):  # reference src/attention_step_fp16.cu:275-292
        assert lib().ra_attention_step_path(RA_F16, D) == 1
        assert lib().ra_attention_step_path(RA_BF16, D) == 1
        # fp32: split-TF32 tensor-core kernel up to head_dim 128, SIMT for 256
        assert lib().ra_attention_step_path(RA_F32, D) == (2 if D <= 128 else 0)
    assert lib().ra_attention_step_path(RA_F16, 48) == -1


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_dim_256_long_rows_both_kernels_agree_with_the_oracle(dtype):
    # several key tiles per row, GQA, ragged lengths, end-aligned causal mask: the tcgen05 kernel
    # (one query tile per block, K / V tiles through the ring as four items) and the SIMT kernel
    q, k, v = normal_inputs(77, 1, 4, 2, 300, 1100, 256, scale=0.7)
    q, k, v = (round_to(x, dtype) for x in (q, k, v))
    want = oracle.cpu_attention(q, k, v, True, kv_heads=2)
    qmap, kmap = SegMap.make([1100 - 300], 300), SegMap.make([0], 1100)
    tol = 1e-3 if dtype == torch.float16 else 8e-3
    for kwargs in ({}, {"p_in_smem": True}, {"cta_pair": True}, {"force_simt": True}):
        got, _ = run_ex(q, k, v, qmap, kmap, 1, True, dtype, 2, **kwargs)
        assert_close(got, want, tol, tol, f"D=256 {dtype} {kwargs}")


@pytest.mark.parametrize("D", [128, 256])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_cluster_pair_form_of_the_tensor_core_kernel(D, dtype):
    """M = 256 MMAs over two blocks of a cluster (cta_group::2): each block loads half of every
    K / V tile. Odd numbers of query blocks (the last pair's second block has no rows), a single
    block per segment (falls back to independent blocks), zig-zag segments, GQA, causal and
    document masks; the result must also equal the independent-block form bit for bit."""
    tol = 1e-3 if dtype == torch.float16 else 8e-3
    for seed, (Sq, Sk, causal, doc_len) in enumerate([(640, 1408, True, 0), (1200, 1200, True, 0),
                                                      (130, 700, False, 0), (900, 900, True, 200),
                                                      (1024, 2048, False, 0)]):
        q, k, v = normal_inputs(500 + seed + D, 1, 4, 2, Sq, Sk, D, scale=0.8)
        q, k, v = (round_to(x, dtype) for x in (q, k, v))
        qmap, kmap = SegMap.make([Sk - Sq], Sq), SegMap.make([0], Sk)
        want, _ = masked_truth(q, k, v, positions(qmap, 1), positions(kmap, 1), causal, doc_len, 2) \
            if doc_len else (oracle.cpu_attention(q, k, v, causal, kv_heads=2), None)
        pair, lse_pair = run_ex(q, k, v, qmap, kmap, 1, causal, dtype, 2, doc_len=doc_len, cta_pair=True)
        single, lse_single = run_ex(q, k, v, qmap, kmap, 1, causal, dtype, 2, doc_len=doc_len)
        assert_close(pair, want, tol, tol, f"D={D} Sq={Sq} Sk={Sk} causal={causal} doc={doc_len}")
        assert np.array_equal(pair, single) and np.array_equal(lse_pair, lse_single)
    # zig-zag: two query segments and four key segments with their own bases
    q, k, v = normal_inputs(611 + D, 1, 2, 1, 2 * 384, 4 * 384, D, scale=0.8)
    q, k, v = (round_to(x, dtype) for x in (q, k, v))
    qmap, kmap = SegMap.make([384, 6 * 384], 384), SegMap.make([0, 384, 6 * 384, 7 * 384], 384)
    want, _ = masked_truth(q, k, v, positions(qmap, 1), positions(kmap, 1), True, 0, 1)
    pair, _ = run_ex(q, k, v, qmap, kmap, 1, True, dtype, 1, cta_pair=True)
    assert_close(pair, want, tol, tol, f"D={D} zig-zag")


@pytest.mark.parametrize("D", [64, 128, 256])
def test_both_block_orders_of_the_tensor_core_kernel(D):
    """(batch, head) fastest (default) and waves of 1, 2 or all 4 KV heads (default only when the
    K/V of all heads do not fit in L2 together): same results bit for bit, GQA with two batches,
    zig-zag query segments, with and without cluster pairs."""
    from ring_attention_b200._lib import lib
    q, k, v = normal_inputs(900 + D, 2, 6, 2, 2 * 320, 4 * 320, D, scale=0.8)
    q, k, v = (round_to(x, torch.float16) for x in (q, k, v))
    qmap, kmap = SegMap.make([320, 6 * 320], 320), SegMap.make([0, 320, 6 * 320, 7 * 320], 320)
    want, _ = masked_truth(q, k, v, positions(qmap, 1), positions(kmap, 1), True, 0, 2)
    got = {}
    try:
        for order in (0, 1, 2, 4):
            lib().ra_debug_set_block_order(order)
            for pair in ((False, True) if D >= 128 else (False,)):
                got[order, pair] = run_ex(q, k, v, qmap, kmap, 1, True, torch.float16, 2, cta_pair=pair)
    finally:
        lib().ra_debug_set_block_order(-1)
    for key, (out, lse) in got.items():
        assert_close(out, want, 1e-3, 1e-3, f"D={D} order/pair={key}")
        assert np.array_equal(out, got[0, False][0]) and np.array_equal(lse, got[0, False][1]), key


@pytest.mark.parametrize("p_in_smem", [False, True])
def test_both_p_paths_of_the_tensor_core_kernel(p_in_smem):
    for D in (32, 64, 128, 256):
        q, k, v = normal_inputs(30 + D, 1, 2, 2, 384, 1664, D)
        q, k, v = (round_to(x, torch.float16) for x in (q, k, v))
        want = oracle.cpu_attention(q, k, v, True, kv_heads=2)
        qmap, kmap = SegMap.make([1664 - 384], 384), SegMap.make([0], 1664)
        got, _ = run_ex(q, k, v, qmap, kmap, 1, True, torch.float16, 2, p_in_smem=p_in_smem)
        assert_close(got, want, 1e-3, 1e-3, f"D={D}")


def test_rows_without_visible_keys_keep_their_state():
    # keys all in the future of the queries: the state must come back untouched, then a later
    # step folds normally (reference src/attention_step.cu:238, attention_step_fp16.cu:155-172)
    B, H, S, D = 1, 2, 128, 64
    q, k, v = normal_inputs(17, B, H, H, S, S, D)
    q, k, v = (round_to(x, torch.float16) for x in (q, k, v))
    dq, dk, dv = (dev(x, torch.float16) for x in (q, k, v))
    out, m, l = state(B, H, S, D)
    shape = api.AttentionShape(B, H, S, S, D)
    api.launch_attention_step_fp16(dq, dk, dv, out, m, l, shape, 0, 1000, True)
    torch.cuda.synchronize()
    assert torch.all(out == 0) and torch.all(torch.isneginf(m)) and torch.all(l == 0)
    api.launch_attention_step_fp16(dq, dk, dv, out, m, l, shape, 0, 0, True)
    api.launch_attention_finalize(out, l, shape)
    assert_close(out.cpu().numpy(), oracle.cpu_attention(q, k, v, True), 1e-3, 1e-3)
    # a never-touched state finalizes to zeros, not NaN (src/attention_step.cu:63-64)
    out2, m2, l2 = state(B, H, S, D)
    api.launch_attention_finalize(out2, l2, shape)
    assert torch.all(out2 == 0)


def test_tensor_core_and_simt_kernels_share_state():
    # steps may alternate between the two kernels on one (out, m, l): the state means the same
    B, H, S, D = 1, 2, 256, 64
    q, k, v = normal_inputs(19, B, H, H, S, S, D)
    q, k, v = (round_to(x, torch.float16) for x in (q, k, v))
    dq = dev(q, torch.float16)
    out, m, l = state(B, H, S, D)
    for p in range(4):
        sl = slice(p * 64, (p + 1) * 64)
        api.attention_step_ex(dq, dev(k[:, :, sl], torch.float16), dev(v[:, :, sl], torch.float16),
                              out, m, l, api.AttentionShape(B, H, S, 64, D), SegMap.make([0], S),
                              SegMap.make([p * 64], 64), 1, causal=True, force_simt=(p % 2 == 1))
    api.launch_attention_finalize(out, l, api.AttentionShape(B, H, S, S, D))
    assert_close(out.cpu().numpy(), oracle.cpu_attention(q, k, v, True), 1e-3, 1e-3)


def test_segmented_fp32_equals_affine_calls():
    # reference tests/test_attention_step_segmented.cu:52-110: one segmented launch == n^2 affine
    B, H, D, nseg, L = 1, 2, 64, 4, 32
    q, k, v = normal_inputs(23, B, H, H, nseg * L, nseg * L, D)
    qb, kb = [0, 224, 64, 160], [32, 192, 96, 128]
    dq, dk, dv = dev(q), dev(k), dev(v)
    out, m, l = state(B, H, nseg * L, D)
    shape = api.AttentionShape(B, H, nseg * L, nseg * L, D)
    api.launch_attention_step_segmented(dq, dk, dv, out, m, l, shape, SegMap.make(qb, L),
                                        SegMap.make(kb, L), True)
    api.launch_attention_finalize(out, l, shape)
    out2, m2, l2 = state(B, H, nseg * L, D)
    sub = api.AttentionShape(B, H, L, L, D)
    for a in range(nseg):
        for b in range(nseg):
            qs = dev(q[:, :, a * L:(a + 1) * L])
            o_s, m_s, l_s = (out2[:, :, a * L:(a + 1) * L].contiguous(), m2[:, :, a * L:(a + 1) * L].contiguous(),
                             l2[:, :, a * L:(a + 1) * L].contiguous())
            api.launch_attention_step(qs, dev(k[:, :, b * L:(b + 1) * L]), dev(v[:, :, b * L:(b + 1) * L]),
                                      o_s, m_s, l_s, sub, qb[a], kb[b], True)
            out2[:, :, a * L:(a + 1) * L], m2[:, :, a * L:(a + 1) * L], l2[:, :, a * L:(a + 1) * L] = o_s, m_s, l_s
    api.launch_attention_finalize(out2, l2, shape)
    assert_close(out.cpu().numpy(), out2.cpu().numpy(), 1e-5, 1e-5)


@pytest.mark.parametrize("name", ["ref_cp2_causal_zigzag", "ref_cp4_causal_zigzag", "ref_cp2_noncausal_seq",
                                  "ref_cp4_noncausal_seq", "gen_prefill_striped_cp4_d64",
                                  "gen_prefill_zigzag4_cp2_d64", "gen_prefill_zigzag_cp4_d128",
                                  "gen_prefill_contig_cp2_d128"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_golden_fixtures_through_a_simulated_ring(name, dtype, golden_dir):
    """Every rank of the fixture's ring is played on one GPU: own rows as Q, P steps over the
    shards in ring order with the library's step maps; the global output must equal the
    fixture's (which the Python reference stores per rank in ITS shard order)."""
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    q, k, v = g["q"], g["k"], g["v"]
    if dtype != torch.float32:
        q, k, v = (round_to(x, dtype) for x in (q, k, v))
    cp, causal = int(g["cp_size"]), bool(g["causal"])
    B, H, S, D = q.shape
    layout, ns = 0, 2
    if "zigzag4" in name:
        layout, ns = 1, 4
    elif "zigzag" in name:
        layout = 1
    elif "striped" in name:
        layout = 2
    full = np.zeros_like(q)
    for rank in range(cp):
        p = api.RingPartition(cp, rank, S, layout, ns)
        rows = p.local_positions().numpy()
        dq = dev(q[:, :, rows], dtype)
        out, m, l = state(B, H, len(rows), D, poison=True)
        for step in range(cp):
            qmap, kmap, stride = p.step_maps(step)
            krows = positions(kmap, stride)
            api.attention_step_ex(dq, dev(k[:, :, krows], dtype), dev(v[:, :, krows], dtype), out, m, l,
                                  api.AttentionShape(B, H, len(rows), len(krows), D), qmap, kmap,
                                  stride, causal=causal, fresh=(step == 0), finalize=(step == cp - 1))
        full[:, :, rows] = out.cpu().numpy()
    # the fixture's rank r holds rows `idx[r]` of the full output (fine zig-zag for the ref_ files)
    if "idx" in g:
        idx = g["idx"]
    elif int(g["zig_zag"]):
        chunk = 2 * cp
        starts = np.arange(S // chunk) * chunk
        ranks = np.arange(cp)[:, None]
        idx = np.stack([starts[None, :] + ranks, starts[None, :] + (cp + (cp - 1 - ranks))], -1).reshape(cp, -1)
    else:
        idx = np.arange(S).reshape(cp, S // cp)
    tol = 1e-5 if dtype == torch.float32 else 2e-3  # fixture outputs come from un-rounded fp32 inputs
    if dtype == torch.float32:
        for r in range(cp):
            assert_close(full[:, :, idx[r]], g["out"][r], tol, tol, f"rank {r}")
    else:
        want = oracle.cpu_attention(q, k, v, causal)
        assert_close(full, want, 1e-3, 1e-3)


def test_unsupported_head_dim_is_an_error_not_a_crash():
    q = torch.zeros((1, 1, 8, 48), device="cuda")
    out, m, l = state(1, 1, 8, 48)
    with pytest.raises(api._lib.RingAttentionError) as e:
        api.launch_attention_step(q, q, q, out, m, l, api.AttentionShape(1, 1, 8, 8, 48), 0, 0, False)
    assert "unsupported head_dim=48" in str(e.value)


@pytest.mark.parametrize("dtype,D", [(torch.float16, 64), (torch.bfloat16, 128), (torch.float16, 32)])
@pytest.mark.parametrize("layout,ns,chunk", [(1, 2, 48), (1, 4, 128), (2, 1, 200), (0, 1, 320)])
def test_stacked_shards_fold_several_ring_steps_in_one_launch(dtype, D, layout, ns, chunk):
    """The gather schedule on one GPU: every rank's K/V shard stacked as an all-gather leaves
    them, step 0 on the rank's own shard, then ONE launch over the other P-1 shards."""
    cp, rank, B, H, kvH = 4, 2, 1, 4, 2
    sloc = ns * chunk if layout == 1 else chunk
    S = cp * sloc
    q, k, v = normal_inputs(11, B, H, kvH, S, S, D)
    q, k, v = (round_to(x, dtype) for x in (q, k, v))
    parts = [api.RingPartition(cp, r, S, layout, ns) for r in range(cp)]
    rows = [p.local_positions().numpy() for p in parts]
    dq = dev(q[:, :, rows[rank]], dtype)
    ks = dev(np.stack([k[:, :, rows[r]] for r in range(cp)]), dtype)  # (cp, B, kvH, sloc, D)
    vs = dev(np.stack([v[:, :, rows[r]] for r in range(cp)]), dtype)
    out, m, l = state(B, H, sloc, D, poison=True)
    shape = api.AttentionShape(B, H, sloc, sloc, D, kvH)
    qmap, kmap0, stride = parts[rank].step_maps(0)
    api.attention_step_ex(dq, ks[rank], vs[rank], out, m, l, shape, qmap, kmap0, stride, causal=True, fresh=True)
    nsg = kmap0.n_seg
    big = SegMap()
    big.n_seg, big.seg_len = (cp - 1) * nsg, kmap0.seg_len
    seg_shard, seg_row = [], []
    for s in range(1, cp):
        _, km, _ = parts[rank].step_maps(s)
        for i in range(nsg):
            big.base[(s - 1) * nsg + i] = km.base[i]
            seg_shard.append((rank - s) % cp)
            seg_row.append(i * km.seg_len)
    shape_big = api.AttentionShape(B, H, sloc, (cp - 1) * sloc, D, kvH)
    api.attention_step_stacked(dq, ks, vs, out, m, l, shape_big, qmap, big, seg_shard, seg_row,
                               pos_stride=stride, causal=True, finalize=True)
    torch.cuda.synchronize()
    assert api.device_status()[0] == 0
    want = oracle.cpu_attention(q, k, v, True, kv_heads=kvH)[:, :, rows[rank]]
    tol = TOL[dtype]
    assert_close(out.cpu().numpy(), want, tol, tol, "out")


def test_stacked_step_rejects_what_the_tensor_core_kernel_cannot_read():
    q = torch.zeros((1, 1, 64, 64), device="cuda", dtype=torch.float32)
    ks = torch.zeros((2, 1, 1, 64, 64), device="cuda", dtype=torch.float32)
    out, m, l = state(1, 1, 64, 64)
    qm, km = SegMap(), SegMap()
    qm.n_seg, qm.seg_len = 1, 64
    km.n_seg, km.seg_len = 2, 64
    with pytest.raises(RuntimeError):  # fp32 has no tensor-core kernel
        api.attention_step_stacked(q, ks, ks, out, m, l, api.AttentionShape(1, 1, 64, 128, 64, 1), qm, km,
                                   [0, 1], [0, 0])
    q64 = torch.zeros((1, 1, 64, 64), device="cuda", dtype=torch.float16)
    ks64 = torch.zeros((2, 1, 1, 64, 64), device="cuda", dtype=torch.float16)
    out, m, l = state(1, 1, 64, 64)
    with pytest.raises(RuntimeError):  # a segment that leaves its shard
        api.attention_step_stacked(q64, ks64, ks64, out, m, l, api.AttentionShape(1, 1, 64, 128, 64, 1), qm, km,
                                   [0, 1], [0, 32])
    torch.cuda.synchronize()
