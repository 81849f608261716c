"""ring_attention_b200.ring_ref on a GPU, checked the way the reference's Python tests check
``ring_attention_ref`` (reference/tests/test_ring.py, test_golden.py, test_inference.py): the ring
played on one GPU must give, per rank and in the reference's shard order, the rows of full
attention. Tolerances: fp32 1e-5, fp16 1e-3 (atol = rtol) against the CPU oracle on the same
(rounded) inputs; the golden fixtures hold fp32 outputs of the reference itself."""
import os

import numpy as np
import pytest
import torch

import oracle
from ring_attention_b200 import ring_ref as R
from util import assert_close, normal_inputs, round_to

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float16: 1e-3}


def cuda(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda").to(dtype)


def full_on_cpu(q, k, v, causal):
    return oracle.cpu_attention(q, k, v, causal, kv_heads=k.shape[1])


@pytest.mark.parametrize("dtype,D", [(torch.float32, 32), (torch.float32, 64), (torch.float16, 64),
                                     (torch.float16, 128)])
@pytest.mark.parametrize("cp_size", [1, 2, 4, 8])
@pytest.mark.parametrize("scheme,causal", [("seq", False), ("seq", True), ("zigzag", False), ("zigzag", True),
                                           ("striped", False), ("striped", True)])
def test_ring_shards_are_rows_of_full_attention(dtype, D, cp_size, scheme, causal):
    B, H, S = 2, 4, 64 if D == 32 else 128
    q, k, v = normal_inputs(5 + cp_size, B, H, H, S, S, D)
    if dtype != torch.float32:
        q, k, v = (round_to(x, dtype) for x in (q, k, v))
    got = R.ring_attention(cuda(q, dtype), cuda(k, dtype), cuda(v, dtype), cp_size=cp_size, causal=causal,
                           zig_zag=scheme == "zigzag", striped=scheme == "striped")
    assert got.shape == (cp_size, B, H, S // cp_size, D) and got.dtype == dtype
    idx = R._indices({"seq": "contiguous"}.get(scheme, scheme), S, cp_size, 2)
    want = R.partition(torch.from_numpy(full_on_cpu(q, k, v, causal)), idx).numpy()
    tol = TOL[dtype]
    assert_close(got.float().cpu().numpy(), want, tol, tol)
    if cp_size == 1:
        one = R.full_attention(cuda(q, dtype), cuda(k, dtype), cuda(v, dtype), causal=causal)
        assert_close(one.float().cpu().numpy(), want[0], tol, tol)


@pytest.mark.parametrize("n_splits,cp_size", [(4, 2), (6, 2), (4, 4), (16, 2)])
def test_zigzag_with_more_sub_groups(n_splits, cp_size):
    B, H, S, D = 1, 2, 2 * n_splits * cp_size * 3, 64
    q, k, v = normal_inputs(9, B, H, H, S, S, D)
    got = R.ring_attention(cuda(q), cuda(k), cuda(v), cp_size=cp_size, causal=True, zig_zag=True,
                           n_splits=n_splits)
    want = R.partition(torch.from_numpy(full_on_cpu(q, k, v, True)), R.zigzag_indices(S, cp_size, n_splits))
    assert_close(got.cpu().numpy(), want.numpy(), 1e-5, 1e-5)


@pytest.mark.parametrize("name", ["ref_cp2_causal_zigzag", "ref_cp4_causal_zigzag", "ref_cp2_noncausal_seq",
                                  "ref_cp4_noncausal_seq", "gen_prefill_striped_cp4_d64",
                                  "gen_prefill_zigzag4_cp2_d64", "gen_prefill_zigzag_cp4_d128",
                                  "gen_prefill_contig_cp2_d128"])
def test_golden_fixtures_rank_by_rank(name, golden_dir):
    """The four fixtures the reference commits (reference/tests/test_golden.py:40-91) and four
    more generated from it: same call, same per-rank shards."""
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    zz = bool(g["zig_zag"]) if "zig_zag" in g else "zigzag" in name
    got = R.ring_attention(cuda(g["q"]), cuda(g["k"]), cuda(g["v"]), cp_size=int(g["cp_size"]),
                           causal=bool(g["causal"]), zig_zag=zz, n_splits=4 if "zigzag4" in name else 2,
                           striped="striped" in name)
    assert_close(got.cpu().numpy(), g["out"], 1e-5, 1e-5)


@pytest.mark.parametrize("cp_size", [2, 4])
@pytest.mark.parametrize("scheme", ["seq", "zigzag", "striped"])
def test_prefill_returns_ring_output_and_partitioned_cache(cp_size, scheme):
    B, H, S, D = 1, 2, 64, 64
    q, k, v = normal_inputs(31, B, H, H, S, S, D)
    dq, dk, dv = cuda(q), cuda(k), cuda(v)
    kw = dict(cp_size=cp_size, causal=True, zig_zag=scheme == "zigzag", striped=scheme == "striped")
    out, cache = R.prefill(dq, dk, dv, s_max=S // cp_size + 3, **kw)
    assert torch.equal(out, R.ring_attention(dq, dk, dv, **kw))
    assert cache.k.shape == (cp_size, B, H, S // cp_size + 3, D)
    assert cache.current_len.tolist() == [S // cp_size] * cp_size
    idx = R._indices({"seq": "contiguous"}.get(scheme, scheme), S, cp_size, 2)
    assert torch.equal(cache.k[:, :, :, :S // cp_size], R.partition(dk, idx))
    assert torch.equal(cache.v[:, :, :, :S // cp_size], R.partition(dv, idx))
    assert float(cache.k[:, :, :, S // cp_size:].abs().max()) == 0.0


def test_decode_trajectory_matches_the_reference_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "gen_decode_cp2.npz"))
    cp, steps = int(g["cp_size"]), g["dq"].shape[0]
    S = g["q"].shape[2]
    out, cache = R.prefill(cuda(g["q"]), cuda(g["k"]), cuda(g["v"]), cp_size=cp, causal=True, zig_zag=False,
                           s_max=S // cp + steps)
    assert_close(out.cpu().numpy(), g["prefill_out"], 1e-5, 1e-5)
    for t in range(steps):
        o, cache = R.decode_step(cuda(g["dq"][t]), cuda(g["dk"][t]), cuda(g["dv"][t]), cache, owner_rank=t % cp)
        assert_close(o.cpu().numpy(), g["dout"][t], 1e-5, 1e-5, f"decode step {t}")
    assert cache.total_len() == S + steps


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("cp_size,zig_zag", [(2, False), (4, True), (3, False)])
def test_decode_tokens_equal_rows_of_causal_attention(dtype, cp_size, zig_zag):
    """reference/tests/test_inference.py:122-205: decoding token t after a prefill of S tokens
    gives row S + t of causal attention over the whole S + T sequence."""
    B, H, S, T, D = 2, 4, 48, 5, 64
    q, k, v = normal_inputs(17, B, H, H, S + T, S + T, D)
    if dtype != torch.float32:
        q, k, v = (round_to(x, dtype) for x in (q, k, v))
    want = full_on_cpu(q, k, v, True)
    _, cache = R.prefill(cuda(q[:, :, :S], dtype), cuda(k[:, :, :S], dtype), cuda(v[:, :, :S], dtype),
                         cp_size=cp_size, causal=True, zig_zag=zig_zag, s_max=S // cp_size + T)
    tol = TOL[dtype]
    for t in range(T):
        before = cache
        lens_before = cache.current_len.clone()
        k_before = cache.k.clone()
        o, cache = R.decode_step(cuda(q[:, :, S + t:S + t + 1], dtype), cuda(k[:, :, S + t:S + t + 1], dtype),
                                 cuda(v[:, :, S + t:S + t + 1], dtype), cache, owner_rank=t % cp_size)
        assert o.dtype == dtype and o.shape == (B, H, 1, D)
        assert_close(o.float().cpu().numpy(), want[:, :, S + t:S + t + 1], tol, tol, f"token {t}")
        # the input cache is untouched and only the owner grew
        assert torch.equal(before.current_len, lens_before) and torch.equal(before.k, k_before)
        grew = (cache.current_len - lens_before).tolist()
        assert grew == [1 if r == t % cp_size else 0 for r in range(cp_size)]
