"""Device-side mirror of the reference's Python package ``ring_attention_ref``.

Same public names, argument meaning, return shapes and ``ValueError`` conditions as
``reference/ring_attention_ref/{zigzag,oracle,ring,inference}.py``, so the reference's Python
tests can be pointed at this module. What differs is how the numbers are made: the reference
computes full attention with torch and slices it per rank; here every rank of the ring is
played on one GPU through the C ABI the way the multi-GPU drivers do it (rank r folds the K/V
shard of rank r - s at ring step s with the step kernel; decode computes one partial per rank
and merges them), so a pass through this module exercises the partition maps, the step kernel's
masks and the (out, m, l) merge.

The index helpers are pure torch and need no GPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import api
from ._lib import RA_MAX_SEG, SegMap, check, lib

__all__ = ["KVCache", "decode_step", "full_attention", "partition", "prefill", "ring_attention",
           "striped_indices", "unpartition", "zigzag_indices"]


# ------------------------------------------------------------------ index helpers ----

def _zigzag_offsets(cp_size: int, n_splits: int) -> torch.Tensor:
    """(cp_size, n_splits): offset of rank r's sub-group sg inside a macro-chunk of
    n_splits * cp_size tokens. Sub-groups pair up from the outside in: even sg = pair p counts
    up from the front, odd sg counts down from the back (reference zigzag.py:47-53)."""
    r = torch.arange(cp_size)
    cols = []
    for sg in range(n_splits):
        pair = sg // 2
        cols.append(pair * cp_size + r if sg % 2 == 0 else (n_splits - 1 - pair) * cp_size + (cp_size - 1 - r))
    return torch.stack(cols, dim=1)


def zigzag_indices(seq_len: int, cp_size: int, n_splits: int = 2) -> torch.Tensor:
    """``(cp_size, seq_len // cp_size)`` LongTensor: row r lists the positions rank r owns, in
    its local order (macro-chunk major). Mirrors reference zigzag.py:12-55."""
    macro = n_splits * cp_size
    if seq_len % macro != 0:
        raise ValueError(f"seq_len={seq_len} must be divisible by n_splits*cp_size={macro}")
    starts = torch.arange(seq_len // macro) * macro
    offs = _zigzag_offsets(cp_size, n_splits)
    return (starts[None, :, None] + offs[:, None, :]).reshape(cp_size, -1)


def striped_indices(seq_len: int, cp_size: int) -> torch.Tensor:
    """``indices[r, j] = r + j * cp_size``. Mirrors reference zigzag.py:58-90."""
    if seq_len % cp_size != 0:
        raise ValueError(f"seq_len={seq_len} must be divisible by cp_size={cp_size}")
    return torch.arange(seq_len).reshape(seq_len // cp_size, cp_size).t().contiguous()


def partition(x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """``(B, H, S, D)`` -> ``(cp_size, B, H, S // cp_size, D)``. Mirrors reference zigzag.py:93-111."""
    cp_size, shard = indices.shape
    picked = x.index_select(-2, indices.reshape(-1).to(x.device))
    return picked.reshape(*x.shape[:-2], cp_size, shard, x.shape[-1]).movedim(-3, 0)


def unpartition(shards: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`partition`. Mirrors reference zigzag.py:114-133."""
    flat = shards.movedim(0, -3).flatten(-3, -2)
    out = torch.empty_like(flat)
    out.index_copy_(-2, indices.reshape(-1).to(flat.device), flat)
    return out


# ------------------------------------------------------------- per-rank position maps ----

@dataclass
class _RankMap:
    """How one rank's shard is laid out for the step kernel: ``order[i]`` is the local row that
    sits at kernel row i, and kernel row i has global position
    ``seg.base[i // seg.seg_len] + (i % seg.seg_len) * stride``."""
    order: torch.Tensor | None
    seg: SegMap
    stride: int


def _rank_map(scheme: str, seq: int, cp_size: int, rank: int, n_splits: int) -> _RankMap:
    shard = seq // cp_size
    if scheme == "contiguous":
        return _RankMap(None, SegMap.make([rank * shard], shard), 1)
    if scheme == "striped":
        return _RankMap(None, SegMap.make([rank], shard), cp_size)
    # zig-zag with single-token sub-groups: local row j = chunk * n_splits + sg. Grouped by sg the
    # shard is n_splits arithmetic progressions of step n_splits * cp_size, which is what a
    # segment map with a position stride describes.
    if n_splits > RA_MAX_SEG:
        raise ValueError(f"n_splits={n_splits} exceeds the {RA_MAX_SEG} segments one step takes")
    n_chunks = shard // n_splits
    order = torch.arange(shard).reshape(n_chunks, n_splits).t().reshape(-1)
    bases = _zigzag_offsets(cp_size, n_splits)[rank].tolist()
    return _RankMap(order, SegMap.make(bases, n_chunks), n_splits * cp_size)


def _to_kernel_order(x: torch.Tensor, rm: _RankMap) -> torch.Tensor:
    return x.contiguous() if rm.order is None else x.index_select(-2, rm.order.to(x.device)).contiguous()


def _from_kernel_order(x: torch.Tensor, rm: _RankMap) -> torch.Tensor:
    if rm.order is None:
        return x
    out = torch.empty_like(x)
    out.index_copy_(-2, rm.order.to(x.device), x)
    return out


def _scheme(zig_zag: bool, striped: bool) -> str:
    if zig_zag and striped:
        raise ValueError("zig_zag and striped are mutually exclusive (pick one scheme)")
    return "zigzag" if zig_zag else "striped" if striped else "contiguous"


def _indices(scheme: str, seq: int, cp_size: int, n_splits: int) -> torch.Tensor:
    if scheme == "zigzag":
        return zigzag_indices(seq, cp_size=cp_size, n_splits=n_splits)
    if scheme == "striped":
        return striped_indices(seq, cp_size=cp_size)
    return torch.arange(seq).reshape(cp_size, seq // cp_size)


# --------------------------------------------------------------------- attention ----

def _state(batch: int, heads: int, rows: int, head_dim: int, device) -> tuple[torch.Tensor, ...]:
    return (torch.empty((batch, heads, rows, head_dim), dtype=torch.float32, device=device),
            torch.empty((batch, heads, rows), dtype=torch.float32, device=device),
            torch.empty((batch, heads, rows), dtype=torch.float32, device=device))


def full_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool) -> torch.Tensor:
    """Scaled dot-product attention over the whole sequence, one launch of the step kernel with
    init and normalisation fused. Mirrors reference oracle.py:9-26 (key j visible to query i iff
    j <= i when ``causal``)."""
    batch, heads, seq_q, head_dim = q.shape
    kv_heads, seq_k = k.shape[1], k.shape[2]
    out, m, l = _state(batch, heads, seq_q, head_dim, q.device)
    shape = api.AttentionShape(batch, heads, seq_q, seq_k, head_dim, kv_heads)
    api.attention_step_ex(q.contiguous(), k.contiguous(), v.contiguous(), out, m, l, shape,
                          SegMap.make([0], seq_q), SegMap.make([0], seq_k), 1, causal=causal,
                          fresh=True, finalize=True)
    return out.to(q.dtype)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, cp_size: int, causal: bool,
                   zig_zag: bool, n_splits: int = 2, striped: bool = False) -> torch.Tensor:
    """Per-rank output shards ``(cp_size, B, H, S // cp_size, D)`` of ring attention, every rank
    played on this GPU: rank r keeps its Q rows and folds the shard of rank r - s at step s.
    Mirrors reference ring.py:18-70 (same arguments, shard order and errors)."""
    seq = q.shape[-2]
    if seq % cp_size != 0:
        raise ValueError(f"seq_len={seq} must be divisible by cp_size={cp_size}")
    scheme = _scheme(zig_zag, striped)
    idx = _indices(scheme, seq, cp_size, n_splits)  # raises on a bad zig-zag length
    batch, heads, _, head_dim = q.shape
    kv_heads = k.shape[1]
    shard = seq // cp_size
    maps = [_rank_map(scheme, seq, cp_size, r, n_splits) for r in range(cp_size)]
    q_sh, k_sh, v_sh = (partition(t, idx) for t in (q, k, v))
    q_sh = [_to_kernel_order(q_sh[r], maps[r]) for r in range(cp_size)]
    k_sh = [_to_kernel_order(k_sh[r], maps[r]) for r in range(cp_size)]
    v_sh = [_to_kernel_order(v_sh[r], maps[r]) for r in range(cp_size)]
    shape = api.AttentionShape(batch, heads, shard, shard, head_dim, kv_heads)
    result = torch.empty((cp_size, batch, heads, shard, head_dim), dtype=q.dtype, device=q.device)
    for r in range(cp_size):
        out, m, l = _state(batch, heads, shard, head_dim, q.device)
        for s in range(cp_size):
            src = (r - s) % cp_size
            api.attention_step_ex(q_sh[r], k_sh[src], v_sh[src], out, m, l, shape, maps[r].seg,
                                  maps[src].seg, maps[r].stride, causal=causal, fresh=(s == 0),
                                  finalize=(s == cp_size - 1))
        result[r] = _from_kernel_order(out, maps[r]).to(q.dtype)
    return result


# --------------------------------------------------------------------- inference ----

@dataclass
class KVCache:
    """Per-rank K/V cache, ``k`` / ``v`` of shape ``(cp_size, B, kv_heads, s_max, D)`` and
    ``current_len`` ``(cp_size,) int64``. Mirrors reference inference.py:25-71."""
    k: torch.Tensor
    v: torch.Tensor
    current_len: torch.Tensor

    @property
    def cp_size(self) -> int:
        return int(self.k.shape[0])

    @property
    def s_max(self) -> int:
        return int(self.k.shape[-2])

    def total_len(self) -> int:
        return int(self.current_len.sum().item())

    def gather_kv(self) -> tuple[torch.Tensor, torch.Tensor]:
        """The populated rows of every rank, concatenated in rank order."""
        lens = [int(n) for n in self.current_len.tolist()]
        return (torch.cat([self.k[r, :, :, :n] for r, n in enumerate(lens)], dim=-2),
                torch.cat([self.v[r, :, :, :n] for r, n in enumerate(lens)], dim=-2))


def prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, cp_size: int, causal: bool,
            zig_zag: bool, striped: bool = False, s_max: int | None = None) -> tuple[torch.Tensor, KVCache]:
    """Ring prefill plus the per-rank caches it leaves behind. Mirrors reference
    inference.py:74-157, including its MHA-only restriction and error messages."""
    batch, heads, seq, head_dim = q.shape
    kv_heads = k.shape[1]
    if heads != kv_heads:
        raise ValueError(f"Phase-1 reference is MHA-only: heads={heads} must equal kv_heads={kv_heads}")
    if seq % cp_size != 0:
        raise ValueError(f"seq_len={seq} must be divisible by cp_size={cp_size}")
    scheme = _scheme(zig_zag, striped)
    shard = seq // cp_size
    if s_max is None:
        s_max = shard
    if s_max < shard:
        raise ValueError(f"s_max={s_max} must be >= seq/cp_size={shard}")
    out_shards = ring_attention(q, k, v, cp_size=cp_size, causal=causal, zig_zag=zig_zag, striped=striped)
    idx = _indices(scheme, seq, cp_size, 2)
    cache_k = q.new_zeros((cp_size, batch, kv_heads, s_max, head_dim))
    cache_v = q.new_zeros((cp_size, batch, kv_heads, s_max, head_dim))
    cache_k[:, :, :, :shard] = partition(k, idx)
    cache_v[:, :, :, :shard] = partition(v, idx)
    return out_shards, KVCache(cache_k, cache_v, torch.full((cp_size,), shard, dtype=torch.int64))


def decode_step(q_new: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, cache: KVCache, *,
                owner_rank: int) -> tuple[torch.Tensor, KVCache]:
    """One decode step: append on the owner rank, one split-K partial (out, m, l) per rank over
    that rank's rows, merge and normalise. The input cache is left as it was. Mirrors reference
    inference.py:160-216 and the rank-level algorithm of src/ring_decode.cu:85-226."""
    cp_size, s_max = cache.cp_size, cache.s_max
    if not 0 <= owner_rank < cp_size:
        raise ValueError(f"owner_rank={owner_rank} out of range [0, {cp_size})")
    pos = int(cache.current_len[owner_rank].item())
    if pos >= s_max:
        raise ValueError(f"cache full on rank {owner_rank}: current_len={pos} == s_max={s_max}")
    new_k, new_v = cache.k.clone(), cache.v.clone()
    new_k[owner_rank, :, :, pos:pos + 1] = k_new
    new_v[owner_rank, :, :, pos:pos + 1] = v_new
    lens = cache.current_len.clone()
    lens[owner_rank] = pos + 1
    new_cache = KVCache(new_k, new_v, lens)

    batch, heads, _, head_dim = q_new.shape
    kv_heads = new_k.shape[2]
    bh = batch * heads
    dev = q_new.device
    o_all = torch.empty((cp_size, batch, heads, 1, head_dim), dtype=torch.float32, device=dev)
    m_all = torch.empty((cp_size, batch, heads, 1), dtype=torch.float32, device=dev)
    l_all = torch.empty((cp_size, batch, heads, 1), dtype=torch.float32, device=dev)
    qc = q_new.contiguous()
    for r in range(cp_size):
        n = int(lens[r].item())
        api.launch_attention_init(o_all[r], m_all[r], l_all[r],
                                  api.AttentionShape(batch, heads, 1, max(n, 1), head_dim, kv_heads))
        if n > 0:
            # the cache only holds positions up to the new token: no mask (inference.py:8-11)
            api.launch_attention_decode_step(qc, new_k[r], new_v[r], o_all[r], m_all[r], l_all[r],
                                             api.AttentionShape(batch, heads, 1, n, head_dim, kv_heads),
                                             0, 0, False, kv_row_stride=s_max)
    # one rank's partial as the all-gather would deliver it: [O | m | l]
    parts = torch.cat([o_all.reshape(cp_size, -1), m_all.reshape(cp_size, -1), l_all.reshape(cp_size, -1)],
                      dim=1).contiguous()
    out = torch.empty((batch, heads, 1, head_dim), dtype=torch.float32, device=q_new.device)
    check(lib().ra_decode_partial_merge(C.c_void_p(parts.data_ptr()), C.c_void_p(out.data_ptr()), None, None,
                                        cp_size, bh, head_dim, 1,
                                        C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return out.to(q_new.dtype), new_cache
