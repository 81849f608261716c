"""Host-only checks of the C-ABI library: it loads, exports every declared symbol, and its
pure-integer entry points (partition maps, ring step maps, work accounting) agree with the
oracle. No compute call is made here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle
from ring_attention_b200 import _lib
from ring_attention_b200._lib import SegMap, Shape, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ring_attention_b200.h")).read()
    return sorted(set(re.findall(r"RA_API\s+[\w\s\*]+?\b(ra_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    handle = C.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 40
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in the header but not exported"


def test_every_declared_symbol_is_bound_in_python():
    assert set(declared_symbols()) <= set(_lib._SIG)


def test_version_and_error_text():
    assert lib().ra_version() == 100
    # invalid arguments are rejected before any CUDA call
    rc = lib().ra_attention_step_ex(1, None, None, None, None, None, None, None, None, None, 1, 0,
                                    0, 0, None)
    assert rc == 1
    assert b"null" in lib().ra_last_error()


MODES = {"contiguous": 0, "zigzag": 1, "striped": 2}


@pytest.mark.parametrize("mode,n_splits", [("contiguous", 2), ("zigzag", 2), ("zigzag", 4),
                                           ("zigzag", 8), ("striped", 2)])
def test_partition_maps_bit_exact(mode, n_splits):
    L = lib()
    mid = MODES[mode]
    for cp in (1, 2, 4, 8):
        seq = cp * n_splits * 40
        for r in range(cp):
            p = oracle.Partition(cp, r, seq, mode, n_splits)
            assert L.ra_partition_local_chunk_len(cp, seq, mid, n_splits) == p.local_chunk_len()
            assert L.ra_partition_num_sub_groups(mid, n_splits) == p.num_sub_groups()
            assert L.ra_partition_position_stride(cp, mid) == p.position_stride()
            assert L.ra_partition_next_rank(cp, r) == p.next_rank()
            assert L.ra_partition_prev_rank(cp, r) == p.prev_rank()
            for sg in range(p.num_sub_groups()):
                assert L.ra_partition_q_offset(cp, r, seq, mid, n_splits, sg) == p.q_offset(sg)
                for step in range(cp + 2):
                    assert (L.ra_partition_k_offset_for_step(cp, r, seq, mid, n_splits, step, sg)
                            == p.k_offset_for_step(step, sg))
                for src in range(cp):
                    assert (L.ra_partition_k_offset_for_source(cp, r, seq, mid, n_splits, src, sg)
                            == p.k_offset_for_source(src, sg))


def test_partition_covers_every_token_once():
    L = lib()
    for mode, ns in (("contiguous", 2), ("zigzag", 2), ("zigzag", 4), ("striped", 2)):
        cp, seq = 4, 4 * ns * 16
        seen = []
        for r in range(cp):
            qm, km = SegMap(), SegMap()
            stride = L.ra_ring_step_maps(cp, r, seq, MODES[mode], ns, 0, C.byref(qm), C.byref(km))
            for sg in range(qm.n_seg):
                assert qm.base[sg] == km.base[sg]  # step 0 holds the rank's own shard
                seen += [qm.base[sg] + i * stride for i in range(qm.seg_len)]
        assert sorted(seen) == list(range(seq))


def brute_pairs(qm, km, stride, causal, doc_len):
    qpos = np.concatenate([qm.base[s] + np.arange(qm.seg_len) * stride for s in range(qm.n_seg)])
    kpos = np.concatenate([km.base[s] + np.arange(km.seg_len) * stride for s in range(km.n_seg)])
    vis = np.ones((len(qpos), len(kpos)), bool)
    if causal:
        vis &= kpos[None, :] <= qpos[:, None]
    if doc_len:
        vis &= (kpos[None, :] // doc_len) == (qpos[:, None] // doc_len)
    return float(vis.sum())


@pytest.mark.parametrize("mode,ns,cp", [("zigzag", 2, 4), ("zigzag", 4, 2), ("striped", 2, 4),
                                        ("contiguous", 2, 2)])
def test_visible_pairs_match_brute_force(mode, ns, cp):
    L = lib()
    seq = cp * ns * 16
    total = 0.0
    for r in range(cp):
        for step in range(cp):
            qm, km = SegMap(), SegMap()
            stride = L.ra_ring_step_maps(cp, r, seq, MODES[mode], ns, step, C.byref(qm), C.byref(km))
            for causal, doc in ((0, 0), (1, 0), (1, seq // 4), (0, seq // 2)):
                got = L.ra_ring_step_visible_pairs(C.byref(qm), C.byref(km), stride, causal, doc)
                assert got == brute_pairs(qm, km, stride, causal, doc)
            total += L.ra_ring_step_visible_pairs(C.byref(qm), C.byref(km), stride, 1, 0)
    assert total == seq * (seq + 1) / 2  # a causal ring pass touches the lower triangle exactly


def test_zigzag_balances_causal_work_across_ranks():
    L = lib()
    cp, seq = 8, 8 * 2 * 64
    per_rank = []
    for r in range(cp):
        w = 0.0
        for step in range(cp):
            qm, km = SegMap(), SegMap()
            st = L.ra_ring_step_maps(cp, r, seq, 1, 2, step, C.byref(qm), C.byref(km))
            w += L.ra_ring_step_visible_pairs(C.byref(qm), C.byref(km), st, 1, 0)
        per_rank.append(w)
    assert max(per_rank) / min(per_rank) < 1.02


def test_workspace_size_queries():
    s = Shape(4, 32, 1, 1000, 128, 8)
    assert lib().ra_decode_workspace_bytes(C.byref(s)) >= 4 * 32 * 130 * 4
    s2 = Shape(1, 8, 64, 64, 64, 0)
    assert lib().ra_flash_workspace_bytes(C.byref(s2), 1) > lib().ra_flash_workspace_bytes(C.byref(s2), 0)


@pytest.mark.parametrize("N,G", [(1, 1), (1, 8), (8, 1), (2, 2), (2, 4), (3, 5), (4, 8)])
def test_ring2d_schedule_bit_exact_and_covering(N, G):
    """ra_ring2d_source against the oracle, plus the properties the reference's own test checks
    (tests/test_ring2d_schedule.cpp:40-128): every shard exactly once, own shard first, one node's
    band per macro-step."""
    L = lib()
    for n in range(N):
        for g in range(G):
            seen = []
            for m in range(N):
                nodes = set()
                for i in range(G):
                    src = L.ra_ring2d_source(N, G, n, g, m, i)
                    assert src == oracle.ring2d_source(N, G, n, g, m, i)
                    seen.append(src)
                    nodes.add(src // G)
                assert len(nodes) == 1
            assert sorted(seen) == list(range(N * G))
            assert seen[0] == n * G + g
    for bad in [(0, 2, 0, 0, 0, 0), (2, 2, 2, 0, 0, 0), (2, 2, 0, 2, 0, 0), (2, 2, 0, 0, 2, 0), (2, 2, 0, 0, 0, -1)]:
        assert L.ra_ring2d_source(*bad) == -1


@pytest.mark.parametrize("N,G", [(1, 4), (2, 2), (2, 4), (4, 2), (8, 1)])
def test_ring2d_data_movement_delivers_the_shard_the_schedule_names(N, G):
    """The 2-D ring driver moves shards like this: per macro-step the seed goes to the same slot of
    the next group, and inside the group the current shard rotates G - 1 times. Played on shard
    ids, every rank must hold exactly Ring2DSchedule::source(m, i) at (m, i) (reference
    src/ring2d_schedule.cpp:28-42) and see every shard once."""
    L = lib()
    P = N * G
    seed = list(range(P))  # shard id every rank starts the macro-step with
    seen = [[] for _ in range(P)]
    for m in range(N):
        cur = list(seed)
        for i in range(G):
            for r in range(P):
                n, g = divmod(r, G)
                assert cur[r] == L.ra_ring2d_source(N, G, n, g, m, i)
                seen[r].append(cur[r])
            if i < G - 1:  # inner ring: g -> g + 1 inside the group
                cur = [cur[(r // G) * G + (r % G - 1) % G] for r in range(P)]
        # outer ring: the seed of this macro-step arrives from the same slot of the previous group
        seed = [seed[((r // G - 1) % N) * G + r % G] for r in range(P)]
    for r in range(P):
        assert sorted(seen[r]) == list(range(P))
