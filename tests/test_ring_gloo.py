"""The multi-rank path on CPU: world_size 2 and 4 over gloo. Each rank follows the ring plan the
library hands out (ra_ring_step_maps: whose shard it holds at which step, at which global
positions), rotates K/V with gloo send/recv as the CUDA driver does with NCCL, folds each step
with the CPU oracle's step function and must end with its rows of full attention."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, layout, n_splits, causal, doc_len, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import ctypes as C

    import oracle
    from ring_attention_b200._lib import SegMap, lib
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, kvH, S, D = 1, 4, 2, world * n_splits * 8, 16
        rng = np.random.default_rng(123)
        q = rng.standard_normal((B, H, S, D)).astype(np.float32)
        k = rng.standard_normal((B, kvH, S, D)).astype(np.float32)
        v = rng.standard_normal((B, kvH, S, D)).astype(np.float32)
        qm, km = SegMap(), SegMap()
        stride = lib().ra_ring_step_maps(world, rank, S, layout, n_splits, 0, C.byref(qm), C.byref(km))
        rows = np.concatenate([qm.base[s] + np.arange(qm.seg_len) * stride for s in range(qm.n_seg)])
        ql = np.ascontiguousarray(q[:, :, rows])
        kl = torch.from_numpy(np.ascontiguousarray(k[:, :, rows]))
        vl = torch.from_numpy(np.ascontiguousarray(v[:, :, rows]))
        out, m, l = oracle.attention_init(ql.shape, ql.shape[:-1])
        nxt, prv = (rank + 1) % world, (rank - 1 + world) % world
        for step in range(world):
            stride = lib().ra_ring_step_maps(world, rank, S, layout, n_splits, step, C.byref(qm), C.byref(km))
            reqs, kr, vr = [], torch.empty_like(kl), torch.empty_like(vl)
            if step < world - 1:
                ops = [dist.P2POp(dist.isend, kl, nxt), dist.P2POp(dist.irecv, kr, prv),
                       dist.P2POp(dist.isend, vl, nxt), dist.P2POp(dist.irecv, vr, prv)]
                reqs = dist.batch_isend_irecv(ops)
            oracle.attention_step(ql, kl.numpy(), vl.numpy(), out, m, l,
                                  q_base=[qm.base[s] for s in range(qm.n_seg)],
                                  k_base=[km.base[s] for s in range(km.n_seg)], stride=stride,
                                  causal=causal, kv_heads=kvH, doc_len=doc_len)
            for r in reqs:
                r.wait()
            if step < world - 1:
                kl, vl = kr, vr
        oracle.attention_finalize(out, l)
        # truth: full attention (per document when doc_len > 0), then this rank's rows
        if doc_len:
            full = np.zeros_like(q)
            for d0 in range(0, S, doc_len):
                sl = slice(d0, d0 + doc_len)
                full[:, :, sl] = oracle.cpu_attention(q[:, :, sl], k[:, :, sl], v[:, :, sl], causal, kv_heads=kvH)
        else:
            full = oracle.cpu_attention(q, k, v, causal, kv_heads=kvH)
        err = float(np.abs(out - full[:, :, rows]).max())
        ret[rank] = err
    finally:
        dist.destroy_process_group()


def _run(world, layout, n_splits, causal, doc_len=0):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29500 + (os.getpid() * 7 + world * 13 + layout * 3 + n_splits) % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, layout, n_splits, causal, doc_len, ret))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world
    assert max(ret.values()) < 1e-5, dict(ret)


@pytest.mark.parametrize("layout,n_splits", [(0, 2), (1, 2), (1, 4), (2, 2)])
def test_ring_world2_causal(layout, n_splits):
    _run(2, layout, n_splits, True)


def test_ring_world4_zigzag_causal_with_documents():
    _run(4, 1, 2, True, doc_len=16)


def test_ring_world2_noncausal():
    _run(2, 0, 2, False)


# ---- the gather schedule: one all-gather, own shard first, the other shards dealt to parts ----

def _gather_worker(rank, world, port, layout, n_splits, parts, causal, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import ctypes as C

    import oracle
    from ring_attention_b200._lib import RA_MAX_SEG, SegMap, lib
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, kvH, S, D = 1, 4, 2, world * n_splits * 8, 16
        rng = np.random.default_rng(321)
        q = rng.standard_normal((B, H, S, D)).astype(np.float32)
        k = rng.standard_normal((B, kvH, S, D)).astype(np.float32)
        v = rng.standard_normal((B, kvH, S, D)).astype(np.float32)
        qm, km = SegMap(), SegMap()
        stride = lib().ra_ring_step_maps(world, rank, S, layout, n_splits, 0, C.byref(qm), C.byref(km))
        rows = np.concatenate([qm.base[s] + np.arange(qm.seg_len) * stride for s in range(qm.n_seg)])
        ql = np.ascontiguousarray(q[:, :, rows])
        kl = torch.from_numpy(np.ascontiguousarray(k[:, :, rows]))
        vl = torch.from_numpy(np.ascontiguousarray(v[:, :, rows]))
        # what ncclAllGather leaves on every rank: the shards stacked in rank order
        ks = [torch.empty_like(kl) for _ in range(world)]
        vs = [torch.empty_like(vl) for _ in range(world)]
        dist.all_gather(ks, kl)
        dist.all_gather(vs, vl)
        states = []
        out, m, l = oracle.attention_init(ql.shape, ql.shape[:-1])
        oracle.attention_step(ql, kl.numpy(), vl.numpy(), out, m, l, q_base=[qm.base[s] for s in range(qm.n_seg)],
                              k_base=[km.base[s] for s in range(km.n_seg)], stride=stride, causal=causal,
                              kv_heads=kvH)
        states.append((out, m, l))
        seen = set((rank, i) for i in range(km.n_seg))
        for z in range(parts):
            pm = SegMap()
            shard = (C.c_int * RA_MAX_SEG)()
            row = (C.c_int * RA_MAX_SEG)()
            st = lib().ra_ring_gather_part_maps(world, rank, S, layout, n_splits, parts, z, C.byref(pm), shard, row)
            assert st == stride and pm.seg_len == km.seg_len
            kz = np.concatenate([ks[shard[i]].numpy()[:, :, row[i]:row[i] + pm.seg_len] for i in range(pm.n_seg)], 2)
            vz = np.concatenate([vs[shard[i]].numpy()[:, :, row[i]:row[i] + pm.seg_len] for i in range(pm.n_seg)], 2)
            for i in range(pm.n_seg):
                key = (shard[i], row[i] // pm.seg_len)
                assert key not in seen, "a key segment was dealt twice"
                seen.add(key)
            o, mm, ll = oracle.attention_init(ql.shape, ql.shape[:-1])
            oracle.attention_step(ql, kz, vz, o, mm, ll, q_base=[qm.base[s] for s in range(qm.n_seg)],
                                  k_base=[pm.base[i] for i in range(pm.n_seg)], stride=stride, causal=causal,
                                  kv_heads=kvH)
            states.append((o, mm, ll))
        assert len(seen) == world * km.n_seg, "a key segment was left out"
        # merge the partial states as the state-merge kernel does, then normalise
        m_max = np.max(np.stack([s[1] for s in states]), axis=0)
        w = [np.where(np.isneginf(s[1]), 0.0, np.exp(s[1] - np.where(np.isneginf(m_max), 0.0, m_max))) for s in states]
        l_tot = sum(wi * s[2] for wi, s in zip(w, states))
        o_tot = sum(wi[..., None] * s[0] for wi, s in zip(w, states))
        got = np.where(l_tot[..., None] > 0, o_tot / np.where(l_tot[..., None] > 0, l_tot[..., None], 1.0), 0.0)
        full = oracle.cpu_attention(q, k, v, causal, kv_heads=kvH)
        ret[rank] = float(np.abs(got - full[:, :, rows]).max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,layout,n_splits,parts", [(2, 1, 2, 1), (2, 1, 2, 2), (4, 1, 2, 3), (4, 2, 2, 2),
                                                         (2, 0, 2, 1), (4, 1, 4, 4)])
def test_gather_schedule_covers_every_key_once_and_merges_to_full_attention(world, layout, n_splits, parts):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 31500 + (os.getpid() * 5 + world * 11 + layout * 7 + n_splits * 3 + parts) % 2000
    procs = [ctx.Process(target=_gather_worker, args=(r, world, port, layout, n_splits, parts, True, ret))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world
    assert max(ret.values()) < 1e-5, dict(ret)
