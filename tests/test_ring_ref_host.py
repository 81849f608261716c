"""CPU checks of ring_attention_b200.ring_ref, the mirror of the reference's Python package:
index tables against the reference's golden values (reference/tests/test_zigzag.py:21-38,64-72,
test_striped.py:23-40, regenerated into tests/golden/index_maps.npz), round trips, the kernel-side
position maps, and every ValueError the reference's tests expect (raised before any GPU work)."""
import os

import numpy as np
import pytest
import torch

from ring_attention_b200 import ring_ref as R


def test_index_tables_match_the_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "index_maps.npz"))
    assert np.array_equal(R.zigzag_indices(16, 2).numpy(), g["zz_16_2"])
    assert np.array_equal(R.zigzag_indices(32, 4).numpy(), g["zz_32_4"])
    assert np.array_equal(R.zigzag_indices(32, 2, n_splits=4).numpy(), g["zz_32_2_n4"])
    assert np.array_equal(R.zigzag_indices(48, 3).numpy(), g["zz_48_3"])
    assert np.array_equal(R.striped_indices(16, 4).numpy(), g["st_16_4"])
    assert np.array_equal(R.striped_indices(12, 3).numpy(), g["st_12_3"])


def test_known_small_tables():
    # rank 0 of 2 owns the outer tokens of every macro-chunk of four, rank 1 the inner ones
    assert R.zigzag_indices(8, 2).tolist() == [[0, 3, 4, 7], [1, 2, 5, 6]]
    assert R.striped_indices(8, 2).tolist() == [[0, 2, 4, 6], [1, 3, 5, 7]]
    assert torch.equal(R.zigzag_indices(8, 1), torch.arange(8).reshape(1, 8))
    assert torch.equal(R.zigzag_indices(16, 2), R.zigzag_indices(16, 2, n_splits=2))


@pytest.mark.parametrize("seq,cp,ns", [(16, 2, 2), (64, 4, 2), (48, 3, 4), (96, 2, 6), (128, 8, 2)])
def test_every_position_has_one_owner_and_round_trips(seq, cp, ns):
    for idx in (R.zigzag_indices(seq, cp, ns), R.striped_indices(seq, cp)):
        assert idx.shape == (cp, seq // cp)
        assert sorted(idx.reshape(-1).tolist()) == list(range(seq))
        x = torch.randn(2, 3, seq, 4)
        shards = R.partition(x, idx)
        assert shards.shape == (cp, 2, 3, seq // cp, 4)
        assert torch.equal(R.unpartition(shards, idx), x)


@pytest.mark.parametrize("scheme,cp,ns,seq", [("zigzag", 4, 2, 64), ("zigzag", 2, 4, 64), ("zigzag", 3, 6, 72),
                                             ("striped", 4, 2, 64), ("contiguous", 4, 2, 64)])
def test_kernel_position_maps_describe_the_same_rows(scheme, cp, ns, seq):
    idx = R._indices(scheme, seq, cp, ns)
    for r in range(cp):
        rm = R._rank_map(scheme, seq, cp, r, ns)
        pos = [rm.seg.base[i // rm.seg.seg_len] + (i % rm.seg.seg_len) * rm.stride for i in range(seq // cp)]
        local = idx[r] if rm.order is None else idx[r][rm.order]
        assert local.tolist() == pos
        x = torch.randn(1, 1, seq // cp, 2)
        assert torch.equal(R._from_kernel_order(R._to_kernel_order(x, rm), rm), x)


def test_invalid_lengths_and_schemes_raise():
    with pytest.raises(ValueError):
        R.zigzag_indices(10, 2)
    with pytest.raises(ValueError):
        R.striped_indices(10, 4)
    q = torch.zeros(1, 2, 10, 8)
    with pytest.raises(ValueError, match="divisible"):
        R.ring_attention(q, q, q, cp_size=4, causal=False, zig_zag=False)
    q = torch.zeros(1, 2, 16, 8)
    with pytest.raises(ValueError, match="mutually exclusive"):
        R.ring_attention(q, q, q, cp_size=2, causal=True, zig_zag=True, striped=True)


def test_prefill_errors_follow_the_reference():
    q = torch.zeros(1, 4, 16, 8)
    with pytest.raises(ValueError, match="mutually exclusive"):
        R.prefill(q, q, q, cp_size=2, causal=True, zig_zag=True, striped=True)
    with pytest.raises(ValueError, match="s_max"):
        R.prefill(q, q, q, cp_size=2, causal=True, zig_zag=False, s_max=4)
    with pytest.raises(ValueError, match="divisible"):
        R.prefill(torch.zeros(1, 4, 15, 8), torch.zeros(1, 4, 15, 8), torch.zeros(1, 4, 15, 8), cp_size=2,
                  causal=True, zig_zag=False)
    with pytest.raises(ValueError, match="MHA-only"):
        R.prefill(q, torch.zeros(1, 2, 16, 8), torch.zeros(1, 2, 16, 8), cp_size=2, causal=True, zig_zag=False)


def test_decode_errors_and_cache_bookkeeping():
    cache = R.KVCache(torch.zeros(2, 1, 2, 4, 8), torch.zeros(2, 1, 2, 4, 8), torch.tensor([4, 3]))
    assert cache.cp_size == 2 and cache.s_max == 4 and cache.total_len() == 7
    k, v = cache.gather_kv()
    assert k.shape == (1, 2, 7, 8) and v.shape == (1, 2, 7, 8)
    one = torch.zeros(1, 2, 1, 8)
    with pytest.raises(ValueError, match="owner_rank"):
        R.decode_step(one, one, one, cache, owner_rank=2)
    with pytest.raises(ValueError, match="cache full"):
        R.decode_step(one, one, one, cache, owner_rank=0)
