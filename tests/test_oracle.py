"""Pins the CPU oracle: against the reference's compiled host code (oracle/_ref), against the
analytic known answers of the reference's tests/test_cpu_attention.cpp, and against golden
vectors produced by the reference's Python package (tests/golden/*.npz)."""
import os

import numpy as np
import pytest

import oracle
from util import assert_close, normal_inputs

HAVE_REF = oracle.ref() is not None
needs_ref = pytest.mark.skipif(not HAVE_REF, reason="oracle/_ref/libref_oracle.so not built")


# ---- analytic cases (reference tests/test_cpu_attention.cpp:33-225) ------------------------

def test_single_token_returns_v():
    q = np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 1, 4)
    k = np.array([.5, -.5, .25, -.25], np.float32).reshape(1, 1, 1, 4)
    v = np.array([7, -1, 0, 42], np.float32).reshape(1, 1, 1, 4)
    assert_close(oracle.cpu_attention(q, k, v, False), v, 1e-6, 1e-6)


def test_uniform_values():
    q = oracle.xorshift32_fill(0xC0FFEE, 2 * 5 * 8).reshape(1, 2, 5, 8)
    k = oracle.xorshift32_fill(0xBEEF, 2 * 7 * 8).reshape(1, 2, 7, 8)
    v = np.empty((1, 2, 7, 8), np.float32)
    v[0, 0], v[0, 1] = 3.14159, 4.14159
    o = oracle.cpu_attention(q, k, v, False)
    assert_close(o[0, 0], np.full((5, 8), 3.14159), 1e-5, 1e-5)
    assert_close(o[0, 1], np.full((5, 8), 4.14159), 1e-5, 1e-5)


def test_causal_first_row_sees_only_key0():
    q, k, v = normal_inputs(3, 1, 1, 1, 4, 4, 8)
    o = oracle.cpu_attention(q, k, v, True)
    assert_close(o[0, 0, 0], v[0, 0, 0], 1e-6, 1e-6)


def test_hand_2x2():
    # q = k = identity rows, D = 2: scores/sqrt(2); softmax weights computed by hand
    q = np.array([[1, 0], [0, 1]], np.float32).reshape(1, 1, 2, 2)
    k = q.copy()
    v = np.array([[4, 0], [0, 2]], np.float32).reshape(1, 1, 2, 2)
    o = oracle.cpu_attention(q, k, v, False)
    e = np.exp(1 / np.sqrt(2))
    w = e / (e + 1)
    want = np.array([[4 * w, 2 * (1 - w)], [4 * (1 - w), 2 * w]], np.float32)
    assert_close(o[0, 0], want, 1e-6, 1e-6)
    oc = oracle.cpu_attention(q, k, v, True)
    assert_close(oc[0, 0, 0], [4.0, 0.0], 1e-6, 1e-6)


def test_gqa_maps_heads_modulo_kv_heads():
    # 8 query heads on 2 KV heads: head h must use KV head h % 2 (src/cpu_attention.cpp:41-42)
    q, k, v = normal_inputs(5, 1, 8, 2, 6, 9, 16)
    o = oracle.cpu_attention(q, k, v, False, kv_heads=2)
    for h in range(8):
        one = oracle.cpu_attention(q[:, h:h + 1], k[:, h % 2:h % 2 + 1], v[:, h % 2:h % 2 + 1], False)
        assert np.array_equal(o[:, h:h + 1], one)


def test_end_aligned_causal_sq_lt_sk():
    q, k, v = normal_inputs(6, 1, 2, 2, 3, 7, 8)
    o = oracle.cpu_attention(q, k, v, True)
    for i in range(3):
        want = oracle.cpu_attention(q[:, :, i:i + 1], k[:, :, :i + 5], v[:, :, :i + 5], False)
        assert_close(o[:, :, i:i + 1], want, 1e-6, 1e-6)


def test_lse_matches_definition():
    q, k, v = normal_inputs(7, 1, 2, 2, 5, 11, 16)
    o, lse = oracle.cpu_attention(q, k, v, True, want_lse=True)
    s = np.einsum("bhid,bhjd->bhij", q.astype(np.float64), k.astype(np.float64)) / 4.0
    mask = np.arange(11)[None, :] <= np.arange(5)[:, None] + 6
    s = np.where(mask, s, -np.inf)
    want = np.log(np.exp(s).sum(-1))
    assert_close(lse, want, 1e-5, 1e-5)


# ---- port == the reference's own compiled code -------------------------------------------

@needs_ref
@pytest.mark.parametrize("shape", [(1, 8, 8, 128, 128, 64, False), (2, 4, 4, 33, 47, 32, True),
                                   (1, 8, 2, 64, 64, 64, True), (1, 4, 1, 16, 80, 128, False)])
def test_port_bit_equals_reference_cpu_attention(shape):
    B, H, kvH, Sq, Sk, D, causal = shape
    q, k, v = normal_inputs(11, B, H, kvH, Sq, Sk, D)
    a = oracle.cpu_attention(q, k, v, causal, kv_heads=kvH)
    b = oracle.cpu_attention(q, k, v, causal, kv_heads=kvH, impl="ref")
    c = oracle.cpu_attention(q, k, v, causal, kv_heads=kvH, impl="ref", threads=4)
    assert np.array_equal(a, b) and np.array_equal(b, c)


@needs_ref
def test_port_rng_and_hash_equal_reference():
    for seed in (0, 1, 42, 0xC0FFEE):
        assert np.array_equal(oracle.xorshift32_fill(seed, 257), oracle.xorshift32_fill(seed, 257, "ref"))
    for args in [(42, 0, 0, 0, 0, 0), (42, 1, 0, 0, 0, 0), (42, 0, 0, 0, 1, 0), (7, 2, 3, 5, 1000003, 127)]:
        assert oracle.gen_elem(*args) == oracle.gen_elem(*args, impl="ref")


def test_gen_elem_known_values():
    # values printed by the reference's tests/test_gen_elem.cpp
    assert abs(oracle.gen_elem(42, 0, 0, 0, 0, 0) - 0.005288) < 1e-6
    assert abs(oracle.gen_elem(42, 1, 0, 0, 0, 0) - 0.636719) < 1e-6
    assert abs(oracle.gen_elem(42, 0, 0, 0, 1, 0) + 0.154576) < 1e-6


@needs_ref
@pytest.mark.parametrize("mode,n_splits", [("contiguous", 2), ("zigzag", 2), ("zigzag", 4), ("striped", 2)])
def test_port_partition_equals_reference(mode, n_splits):
    for cp in (1, 2, 3, 4, 8):
        seq = cp * n_splits * 24
        for r in range(cp):
            a = oracle.Partition(cp, r, seq, mode, n_splits)
            b = oracle.Partition(cp, r, seq, mode, n_splits, impl="ref")
            assert a.local_chunk_len() == b.local_chunk_len()
            assert a.num_sub_groups() == b.num_sub_groups()
            assert a.position_stride() == b.position_stride()
            assert (a.next_rank(), a.prev_rank()) == (b.next_rank(), b.prev_rank())
            for sg in range(a.num_sub_groups()):
                assert a.q_offset(sg) == b.q_offset(sg)
                for step in range(cp + 1):
                    assert a.k_offset_for_step(step, sg) == b.k_offset_for_step(step, sg)
                for src in range(cp):
                    assert a.k_offset_for_source(src, sg) == b.k_offset_for_source(src, sg)


def test_partition_known_tables():
    # reference tests/test_ring_partition.cpp:151-171 (zig-zag), :234-250 (4 splits), :287-303 (striped)
    cp, seq = 4, 256
    chunk = seq // (2 * cp)
    for r in range(cp):
        p = oracle.Partition(cp, r, seq, "zigzag", 2)
        assert p.q_offset(0) == r * chunk and p.q_offset(1) == (2 * cp - 1 - r) * chunk
        for step in range(cp):
            src = (r - step + cp) % cp
            assert p.k_offset_for_step(step, 0) == src * chunk
            assert p.k_offset_for_step(step, 1) == (2 * cp - 1 - src) * chunk
    chunk4 = seq // (4 * cp)
    for r in range(cp):
        p = oracle.Partition(cp, r, seq, "zigzag", 4)
        assert p.q_offset(0) == r * chunk4
        assert p.q_offset(1) == (3 * cp + (cp - 1 - r)) * chunk4
        assert p.q_offset(2) == (cp + r) * chunk4
        assert p.q_offset(3) == (2 * cp + (cp - 1 - r)) * chunk4
    for r in range(cp):
        p = oracle.Partition(cp, r, seq, "striped")
        assert p.q_offset() == r and p.position_stride() == cp and p.local_chunk_len() == seq // cp
        for step in range(cp):
            assert p.k_offset_for_step(step) == (r - step + cp) % cp


# ---- golden vectors from the reference's Python package ----------------------------------

GOLDEN = ["ref_cp2_noncausal_seq", "ref_cp2_causal_zigzag", "ref_cp4_noncausal_seq",
          "ref_cp4_causal_zigzag", "gen_prefill_striped_cp4_d64", "gen_prefill_zigzag4_cp2_d64",
          "gen_prefill_zigzag_cp4_d128", "gen_prefill_contig_cp2_d128"]


def golden_rank_rows(g, name):
    """Global positions of each rank's rows, (cp, S/cp), as the Python reference shards them."""
    cp = int(g["cp_size"])
    S = g["q"].shape[2]
    if "idx" in g:
        return g["idx"]
    if int(g["zig_zag"]):
        idx = np.load(os.path.join(os.path.dirname(__file__), "golden", "index_maps.npz"))
        # fine zig-zag (reference/ring_attention_ref/zigzag.py:38-55), rebuilt here for any S
        chunk = 2 * cp
        starts = np.arange(S // chunk) * chunk
        ranks = np.arange(cp)[:, None]
        parts = [starts[None, :] + ranks, starts[None, :] + (cp + (cp - 1 - ranks))]
        out = np.stack(parts, -1).reshape(cp, -1)
        if (S, cp) == (16, 2):
            assert np.array_equal(out, idx["zz_16_2"])
        return out
    return np.arange(S).reshape(cp, S // cp)


@pytest.mark.parametrize("name", GOLDEN)
def test_oracle_reproduces_golden_outputs(name, golden_dir):
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    full = oracle.cpu_attention(g["q"], g["k"], g["v"], bool(g["causal"]))
    rows = golden_rank_rows(g, name)
    for r in range(rows.shape[0]):
        assert_close(full[:, :, rows[r]], g["out"][r], 1e-5, 1e-5, f"{name} rank {r}")


def test_fine_zigzag_formula_matches_reference_tables(golden_dir):
    idx = np.load(os.path.join(golden_dir, "index_maps.npz"))
    for key, (S, cp) in {"zz_16_2": (16, 2), "zz_32_4": (32, 4), "zz_48_3": (48, 3)}.items():
        g = {"cp_size": cp, "q": np.zeros((1, 1, S, 1)), "zig_zag": 1}
        assert np.array_equal(golden_rank_rows(g, key), idx[key])
    assert np.array_equal(idx["st_16_4"], np.arange(4)[:, None] + np.arange(4)[None, :] * 4)


def test_oracle_reproduces_golden_decode(golden_dir):
    g = np.load(os.path.join(golden_dir, "gen_decode_cp2.npz"))
    k, v = g["k"], g["v"]
    for t in range(g["dq"].shape[0]):
        k = np.concatenate([k, g["dk"][t]], axis=2)
        v = np.concatenate([v, g["dv"][t]], axis=2)
        o = oracle.cpu_attention(g["dq"][t], k, v, False)
        assert_close(o, g["dout"][t], 1e-5, 1e-5, f"decode step {t}")


# ---- the CPU ring step (used by the multi-rank CPU tests) ---------------------------------

@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("chunks", [1, 2, 4])
def test_ring_step_recurrence_equals_full_attention(causal, chunks):
    B, H, kvH, S, D = 1, 4, 2, 64, 32
    q, k, v = normal_inputs(21, B, H, kvH, S, S, D)
    want, want_lse = oracle.cpu_attention(q, k, v, causal, kv_heads=kvH, want_lse=True)
    out, m, l = oracle.attention_init(q.shape, q.shape[:-1])
    n = S // chunks
    for p in range(chunks):
        oracle.attention_step(q, k[:, :, p * n:(p + 1) * n].copy(), v[:, :, p * n:(p + 1) * n].copy(),
                              out, m, l, q_base=0, k_base=p * n, causal=causal, kv_heads=kvH)
    lse = m + np.log(l)
    oracle.attention_finalize(out, l)
    assert_close(out, want, 1e-5, 1e-5)
    assert_close(lse, want_lse, 1e-5, 1e-5)


def test_partial_merge_equals_joint_softmax():
    BH, D, cp = 6, 16, 3
    rng = np.random.default_rng(5)
    blocks = []
    m_all = rng.standard_normal((cp, BH)).astype(np.float32)
    m_all[1, 2] = -np.inf  # a rank that saw nothing for one row
    for r in range(cp):
        o = rng.standard_normal((BH, D)).astype(np.float32)
        l = rng.uniform(0.5, 2.0, BH).astype(np.float32)
        if r == 1:
            o[2], l[2] = 0, 0
        blocks.append(np.concatenate([o.ravel(), m_all[r], l]))
    out, m, l = oracle.decode_partial_merge(np.concatenate(blocks), cp, BH, D)
    mm = m_all.max(0)
    assert_close(m, mm, 0, 0)
    w = np.where(np.isinf(m_all), 0, np.exp(m_all - mm))
    want_l = sum(w[r] * blocks[r][BH * D + BH:] for r in range(cp))
    assert_close(l, want_l, 1e-6, 1e-6)


def test_ring2d_known_trace_n2_g2():
    # the exact visitation order the reference pins (tests/test_ring2d_schedule.cpp:150-158):
    # sources[rank][m * G + i] on 2 nodes x 2 GPUs
    expected = [[0, 1, 2, 3], [1, 0, 3, 2], [2, 3, 0, 1], [3, 2, 1, 0]]
    for r in range(4):
        got = [oracle.ring2d_source(2, 2, r // 2, r % 2, m, i) for m in range(2) for i in range(2)]
        assert got == expected[r]


@needs_ref
@pytest.mark.parametrize("N,G", [(1, 1), (1, 8), (8, 1), (2, 2), (2, 4), (3, 5), (4, 8)])
def test_port_ring2d_equals_reference(N, G):
    for n in range(N):
        for g in range(G):
            for m in range(N):
                for i in range(G):
                    assert (oracle.ring2d_source(N, G, n, g, m, i) ==
                            oracle.ring2d_source(N, G, n, g, m, i, impl="ref"))
