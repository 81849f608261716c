"""Multi-GPU ring prefill and ring decode through the C ABI, one process per GPU over NCCL,
checked against the CPU oracle. Skipped on boxes with a single GPU (the same drivers are covered
on CPU by tests/test_ring_gloo.py). Each rank ends normally; no rank is ever faulted or hung."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, case, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    import oracle
    from ring_attention_b200 import api
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ring = api.Ring(rank, world)
        rng = np.random.default_rng(77)
        if case["kind"] == "prefill":
            B, H, kvH, S, D = case["B"], case["H"], case["kvH"], case["S"], case["D"]
            dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[case.get("dtype", "f16")]
            q = torch.from_numpy(rng.standard_normal((B, H, S, D)).astype(np.float32)).to(dt)
            k = torch.from_numpy(rng.standard_normal((B, kvH, S, D)).astype(np.float32)).to(dt)
            v = torch.from_numpy(rng.standard_normal((B, kvH, S, D)).astype(np.float32)).to(dt)
            part = api.RingPartition(world, rank, S, case["layout"], case["n_splits"])
            rows = part.local_positions()
            ql, kl, vl = (t[:, :, rows].contiguous().cuda() for t in (q, k, v))
            if case.get("host"):
                # host-buffer entry point: pinned shards in, pinned output out
                hq, hk, hv = (t[:, :, rows].contiguous().pin_memory() for t in (q, k, v))
                out = torch.empty((B, H, len(rows), D), dtype=torch.float32).pin_memory()
                lse = torch.empty((B, H, len(rows)), dtype=torch.float32).pin_memory()
                for _ in range(2):
                    out.fill_(float("nan"))
                    res = ring.prefill_host(hq, hk, hv, out, seq=S, causal=case["causal"], layout=case["layout"],
                                            n_splits=case["n_splits"], lse=lse,
                                            schedule=case.get("schedule", "auto"), timed=True)
                _, want_lse = oracle.cpu_attention(q.float().numpy(), k.float().numpy(), v.float().numpy(),
                                                   case["causal"], kv_heads=kvH, want_lse=True)
                assert np.abs(lse.numpy() - want_lse[:, :, rows.numpy()]).max() < 2e-3
            for _ in range(0 if case.get("host") else 2):  # twice: buffers and events are reused across passes
                out, lse, res = ring.prefill(ql, kl, vl, seq=S, causal=case["causal"], layout=case["layout"],
                                             n_splits=case["n_splits"], doc_len=case.get("doc_len", 0),
                                             want_lse=True, timed=True,
                                             schedule=case.get("schedule", "auto"),
                                             ring2d_nodes=case.get("nodes", 1))
            torch.cuda.synchronize()
            assert api.device_status()[0] == 0
            qf, kf, vf = (t.float().numpy() for t in (q, k, v))
            doc = case.get("doc_len", 0)
            if doc:
                want = np.zeros_like(qf)
                for d0 in range(0, S, doc):
                    sl = slice(d0, d0 + doc)
                    want[:, :, sl] = oracle.cpu_attention(qf[:, :, sl], kf[:, :, sl], vf[:, :, sl], case["causal"],
                                                          kv_heads=kvH)
            else:
                want = oracle.cpu_attention(qf, kf, vf, case["causal"], kv_heads=kvH)
            got = out.cpu().numpy()
            w = want[:, :, rows.numpy()]
            tol = {"f16": 1e-3, "bf16": 8e-3, "f32": 1e-5}[case.get("dtype", "f16")]
            bad = np.abs(got - w) > tol + tol * np.abs(w)
            ret[rank] = (int(bad.sum()), float(np.abs(got - w).max()), res.total_ms, res.comp_ms, res.comm_ms)
        else:
            B, H, kvH, D, prompt, steps = 2, 8, 2, 128, 4 * world * 16, 5
            dt = torch.float32 if case["dtype"] == "f32" else torch.float16
            k = rng.standard_normal((B, kvH, prompt + steps, D)).astype(np.float32)
            v = rng.standard_normal((B, kvH, prompt + steps, D)).astype(np.float32)
            qs = rng.standard_normal((steps, B, H, 1, D)).astype(np.float32)
            k, v, qs = (torch.from_numpy(x).to(dt).float().numpy() for x in (k, v, qs))
            per = prompt // world
            cache = api.DeviceKVCache(B, kvH, per + steps, D, dt)
            sl = slice(rank * per, (rank + 1) * per)
            cache.copy_prefill(torch.from_numpy(k[:, :, sl]).to(dt).contiguous().cuda(),
                               torch.from_numpy(v[:, :, sl]).to(dt).contiguous().cuda(), per)
            lens = [per] * world
            out = torch.empty((B, H, 1, D), device="cuda")
            worst = 0.0
            nbad = 0
            for t in range(steps):
                owner = t % world
                lens[owner] += 1
                pos = prompt + t
                kn = torch.from_numpy(k[:, :, pos:pos + 1]).to(dt).contiguous().cuda()
                vn = torch.from_numpy(v[:, :, pos:pos + 1]).to(dt).contiguous().cuda()
                ring.decode_step(torch.from_numpy(qs[t]).to(dt).cuda(), kn, vn, owner, cache, lens, out)
                want = oracle.cpu_attention(qs[t], k[:, :, :pos + 1], v[:, :, :pos + 1], False, kv_heads=kvH)
                got = out.cpu().numpy()
                tol = 1e-5 if dt == torch.float32 else 1e-3
                nbad += int((np.abs(got - want) > tol + tol * np.abs(want)).sum())
                worst = max(worst, float(np.abs(got - want).max()))
            ret[rank] = (nbad, worst, 0, 0, 0)
        ring.close()
    finally:
        dist.destroy_process_group()


def _run(world, case):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29700 + (os.getpid() * 3 + world * 17 + len(str(case))) % 1500
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, ret)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(300)
    finally:
        # a rank still running here is stuck: end exactly the processes started above, so that no
        # rank keeps its communicator and GPU after the test
        stuck = [p for p in procs if p.is_alive()]
        for p in stuck:
            p.terminate()
        for p in stuck:
            p.join(10)
            if p.is_alive():
                p.kill()
    for p in procs:
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    assert len(ret) == world
    for r in range(world):
        assert ret[r][0] == 0, f"rank {r}: {ret[r][0]} elements off, max err {ret[r][1]}"
    return dict(ret)


def _world():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    return 4 if n >= 4 else 2


@pytest.mark.parametrize("schedule", ["ring", "gather"])
@pytest.mark.parametrize("layout,n_splits", [(1, 2), (0, 2), (2, 2), (1, 4)])
def test_ring_prefill_fp16_causal(layout, n_splits, schedule):
    world = _world()
    _run(world, dict(kind="prefill", B=1, H=4, kvH=2, S=world * n_splits * 256, D=64, causal=True,
                     layout=layout, n_splits=n_splits, schedule=schedule))


@pytest.mark.parametrize("D", [64, 128])
def test_gather_with_split_keys_mha(D):
    # few query blocks: the gathered key segments are split over two parallel launches and merged
    world = _world()
    _run(world, dict(kind="prefill", B=1, H=4, kvH=4, S=world * 2 * 256, D=D, causal=True, layout=1, n_splits=2,
                     schedule="gather"))
    _run(world, dict(kind="prefill", B=1, H=8, kvH=8, S=world * 4 * 128, D=D, causal=True, layout=1, n_splits=4,
                     doc_len=world * 128, schedule="gather"))


def test_ring_prefill_d128_noncausal_and_documents():
    world = _world()
    _run(world, dict(kind="prefill", B=2, H=4, kvH=4, S=world * 2 * 128, D=128, causal=False, layout=0, n_splits=2))
    S = world * 4 * 128
    for schedule in ("ring", "gather"):
        _run(world, dict(kind="prefill", B=1, H=2, kvH=2, S=S, D=128, causal=True, layout=1, n_splits=4,
                         doc_len=S // 4, schedule=schedule))


@pytest.mark.parametrize("schedule", ["ring", "gather"])
def test_ring_prefill_fp32_and_bf16(schedule):
    # fp32 takes the SIMT step (and, gathered, one plain step per shard); bf16 the tensor-core one
    world = _world()
    _run(world, dict(kind="prefill", B=1, H=2, kvH=1, S=world * 2 * 96, D=64, causal=True, layout=1, n_splits=2,
                     schedule=schedule, dtype="f32"))
    _run(world, dict(kind="prefill", B=1, H=2, kvH=2, S=world * 2 * 160, D=128, causal=True, layout=2, n_splits=2,
                     schedule=schedule, dtype="bf16"))


@pytest.mark.parametrize("layout,n_splits", [(1, 2), (2, 2)])
def test_ring_blocking_and_2d_schedules(layout, n_splits):
    # the reference's ring-blocking and ring-2d modes (src/ring_loop.cu:259-592, 1071-1550) as
    # schedules over the same kernels: results as for the overlapped ring
    world = _world()
    base = dict(kind="prefill", B=1, H=4, kvH=2, S=world * n_splits * 256, D=64, causal=True, layout=layout,
                n_splits=n_splits)
    _run(world, dict(base, schedule="blocking"))
    for nodes in sorted({1, 2, world}):  # one group, two groups, every rank its own group
        _run(world, dict(base, schedule="ring2d", nodes=nodes))


@pytest.mark.parametrize("schedule", ["auto", "ring"])
def test_ring_prefill_from_host_buffers(schedule):
    """ra_ring_prefill_host: one pass below the size where the pass is pipelined over two head
    groups, and above it with an even and an odd number of heads."""
    world = _world()
    _run(world, dict(kind="prefill", host=True, B=1, H=4, kvH=4, S=world * 2 * 128, D=64, causal=True, layout=1,
                     n_splits=2, schedule=schedule))
    for H in (16, 15):  # 18.9 / 17.7 MB of Q, K, V per rank: two head groups of 8 + 8 / 7 + 8 heads
        _run(world, dict(kind="prefill", host=True, B=1, H=H, kvH=H, S=world * 2 * 768, D=128, causal=True,
                         layout=1, n_splits=2, schedule=schedule))


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_ring_decode_round_robin(dtype):
    _run(_world(), dict(kind="decode", dtype=dtype))
