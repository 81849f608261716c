"""Host-side mirror of the reference's operator interface, on torch CUDA tensors.

Names, argument meaning and error behaviour follow the reference's C++ headers
(``src/attention.hpp``, ``src/kv_cache.hpp``, ``src/decode_op.hpp``, ``src/ring_partition.hpp``,
``src/ring_decode.hpp``, ``src/ring_loop.hpp``); where the reference aborts the process this
module raises ``RingAttentionError``. torch supplies device memory and the current stream and
nothing else: every function below is one call into the C ABI.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import (RA_BF16, RA_F16, RA_F32, RA_STEP_CAUSAL, RA_STEP_FINALIZE, RA_STEP_FORCE_SIMT,
                   RA_STEP_FRESH, RingConfig, RingResult, SegMap, Shape, check, lib)

_DT = {torch.float32: RA_F32, torch.float16: RA_F16, torch.bfloat16: RA_BF16}


@dataclass
class AttentionShape:
    """Mirror of ``AttentionShape`` (reference src/attention.hpp:19-26)."""
    batch: int
    heads: int
    seq_q: int
    seq_k: int
    head_dim: int
    kv_heads: int = 0

    def c(self) -> Shape:
        return Shape(self.batch, self.heads, self.seq_q, self.seq_k, self.head_dim, self.kv_heads)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("expected a contiguous CUDA tensor")
    return C.c_void_p(t.data_ptr())


def _dtype(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}") from None


def tensor_numel(batch, heads, seq, head_dim):
    return batch * heads * seq * head_dim


def launch_attention_init(out, m, l, shape: AttentionShape, m_count=None):
    """``launch_attention_init`` (reference src/attention.hpp:73)."""
    if m_count is None:
        m_count = shape.batch * shape.heads * shape.seq_q
    check(lib().ra_attention_init(_ptr(out), _ptr(m), _ptr(l), C.byref(shape.c()), m_count,
                                  _stream()))


def launch_attention_step(q, k, v, out, m, l, shape, q_offset, k_offset, causal, pos_stride=1):
    """``launch_attention_step`` (fp32; reference src/attention.hpp:92-94)."""
    check(lib().ra_attention_step(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(m), _ptr(l),
                                  C.byref(shape.c()), q_offset, k_offset, int(causal), _stream(),
                                  pos_stride))


def launch_attention_step_fp16(q, k, v, out, m, l, shape, q_offset, k_offset, causal,
                               pos_stride=1):
    """``launch_attention_step_fp16`` (reference src/attention.hpp:147-150)."""
    check(lib().ra_attention_step_fp16(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(m), _ptr(l),
                                       C.byref(shape.c()), q_offset, k_offset, int(causal),
                                       _stream(), pos_stride))


def launch_attention_step_segmented(q, k, v, out, m, l, shape, qmap: SegMap, kmap: SegMap, causal):
    """``launch_attention_step_segmented`` (fp32; reference src/attention.hpp:115-119)."""
    check(lib().ra_attention_step_segmented(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(m),
                                            _ptr(l), C.byref(shape.c()), C.byref(qmap),
                                            C.byref(kmap), int(causal), _stream()))


def attention_step_ex(q, k, v, out, m, l, shape, qmap, kmap, pos_stride=1, causal=False,
                      fresh=False, finalize=False, force_simt=False, doc_len=0, kv_row_stride=0,
                      p_in_smem=False, cta_pair=False):
    """General step: any dtype, segment maps with a stride, document mask, fused init/finalize.
    ``p_in_smem`` selects the tcgen05 kernel's second form (P staged through shared memory),
    ``cta_pair`` its cluster-pair form (M = 256 MMAs over two blocks; head_dim 128 / 256)."""
    flags = ((RA_STEP_CAUSAL if causal else 0) | (RA_STEP_FRESH if fresh else 0) |
             (RA_STEP_FINALIZE if finalize else 0) | (RA_STEP_FORCE_SIMT if force_simt else 0) |
             (_lib.RA_STEP_P_IN_SMEM if p_in_smem else 0) |
             (_lib.RA_STEP_CTA_PAIR if cta_pair else 0))
    check(lib().ra_attention_step_ex(_dtype(q), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(m),
                                     _ptr(l), C.byref(shape.c()), C.byref(qmap), C.byref(kmap),
                                     pos_stride, flags, doc_len, kv_row_stride, _stream()))


def attention_step_stacked(q, k, v, out, m, l, shape, qmap, kmap, seg_shard, seg_row, *,
                           pos_stride=1, causal=False, fresh=False, finalize=False, doc_len=0):
    """General step whose key segments sit in stacked shards: ``k`` / ``v`` are
    (n_shards, B, kvH, shard_rows, D); segment i is rows seg_row[i].. of shard seg_shard[i]."""
    flags = ((RA_STEP_CAUSAL if causal else 0) | (RA_STEP_FRESH if fresh else 0) |
             (RA_STEP_FINALIZE if finalize else 0))
    n = len(seg_shard)
    shard = (C.c_int * n)(*seg_shard)
    row = (C.c_int * n)(*seg_row)
    check(lib().ra_attention_step_stacked(_dtype(q), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(m),
                                          _ptr(l), C.byref(shape.c()), C.byref(qmap),
                                          C.byref(kmap), shard, row, k.shape[0], k.shape[3],
                                          pos_stride, flags, doc_len, _stream()))


def launch_attention_decode_step(q, k, v, out, m, l, shape, q_offset, k_offset, causal,
                                 kv_row_stride=0, workspace=None):
    """``launch_attention_decode_step`` (reference src/attention.hpp:128-131); any dtype."""
    ws_ptr, ws_bytes = (None, 0) if workspace is None else (_ptr(workspace),
                                                             workspace.numel() * workspace.element_size())
    check(lib().ra_attention_decode_step(_dtype(q), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(m),
                                         _ptr(l), C.byref(shape.c()), q_offset, k_offset,
                                         int(causal), _stream(), kv_row_stride, ws_ptr, ws_bytes))


def launch_attention_finalize(out, l, shape):
    """``launch_attention_finalize`` (reference src/attention.hpp:136)."""
    check(lib().ra_attention_finalize(_ptr(out), _ptr(l), C.byref(shape.c()), _stream()))


def attention_lse(m, l):
    lse = torch.empty_like(m)
    check(lib().ra_attention_lse(_ptr(m), _ptr(l), _ptr(lse), m.numel(), _stream()))
    return lse


def launch_float_to_half(src, dst):
    check(lib().ra_float_to_half(_ptr(src), _ptr(dst), src.numel(), _stream()))


def launch_half_to_float(src, dst):
    check(lib().ra_half_to_float(_ptr(src), _ptr(dst), src.numel(), _stream()))


def launch_float_to_bf16(src, dst):
    check(lib().ra_float_to_bf16(_ptr(src), _ptr(dst), src.numel(), _stream()))


def launch_float_to_int8(src, dst):
    check(lib().ra_float_to_int8(_ptr(src), _ptr(dst), src.numel(), _stream()))


def launch_int8_to_float(src, dst):
    check(lib().ra_int8_to_float(_ptr(src), _ptr(dst), src.numel(), _stream()))


def _flash(q, k, v, out, shape, causal, half):
    s = shape.c()
    nbytes = lib().ra_flash_workspace_bytes(C.byref(s), int(half))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    check(lib().ra_flash_attention(_ptr(q), _ptr(k), _ptr(v), _ptr(out), C.byref(s), int(causal),
                                   int(half), _ptr(ws), nbytes, _stream()))


def launch_flash_attention(q, k, v, out, shape, causal):
    """``launch_flash_attention`` (fp32 in/out; reference src/attention.hpp:52-53)."""
    _flash(q, k, v, out, shape, causal, False)


def launch_flash_attention_fp16(q, k, v, out, shape, causal):
    """``launch_flash_attention_fp16`` (fp32 I/O, fp16 inside; reference src/attention.hpp:64-65)."""
    _flash(q, k, v, out, shape, causal, True)


def launch_naive_attention(q, k, v, out, shape, causal):
    """``launch_naive_attention`` (reference src/attention.hpp:42-46): any head_dim, fp32."""
    check(lib().ra_naive_attention(_ptr(q), _ptr(k), _ptr(v), _ptr(out), C.byref(shape.c()), int(causal),
                                   _stream()))


def prefill_host(q, k, v, shape, qmap, kmap, pos_stride=1, causal=False, doc_len=0,
                 want_lse=False, force_simt=False):
    """Whole attention on HOST tensors (pinned or pageable): upload, step, download."""
    for t in (q, k, v):
        if t.is_cuda or not t.is_contiguous():
            raise ValueError("prefill_host expects contiguous host tensors")
    out = torch.empty(q.shape, dtype=torch.float32, pin_memory=True)
    lse = torch.empty(q.shape[:-1], dtype=torch.float32, pin_memory=True) if want_lse else None
    flags = (RA_STEP_CAUSAL if causal else 0) | (RA_STEP_FORCE_SIMT if force_simt else 0)
    check(lib().ra_prefill_host(_DT[q.dtype], C.c_void_p(q.data_ptr()), C.c_void_p(k.data_ptr()),
                                C.c_void_p(v.data_ptr()), C.c_void_p(out.data_ptr()),
                                C.c_void_p(lse.data_ptr()) if want_lse else None,
                                C.byref(shape.c()), C.byref(qmap), C.byref(kmap), pos_stride,
                                flags, doc_len))
    return (out, lse) if want_lse else out


def device_status():
    """Read and clear the device status word: [code, which wait, block, tile]."""
    buf = (C.c_int * 4)()
    check(lib().ra_device_status(buf))
    return list(buf)


class RingPartition:
    """Mirror of ``RingPartition`` (reference src/ring_partition.hpp:11-75)."""
    CONTIGUOUS, ZIGZAG, STRIPED = 0, 1, 2

    def __init__(self, cp_size, rank, seq, mode=0, n_splits=2):
        if cp_size <= 0 or not 0 <= rank < cp_size or seq % cp_size != 0:
            raise ValueError("bad partition arguments")
        if mode == self.ZIGZAG and (n_splits < 2 or seq % (n_splits * cp_size) != 0):
            raise ValueError("zig-zag needs n_splits >= 2 and seq divisible by n_splits*cp_size")
        self.cp_size, self.rank, self.seq, self.mode, self.n_splits = cp_size, rank, seq, mode, n_splits

    def _a(self):
        return (self.cp_size, self.rank, self.seq, self.mode, self.n_splits)

    def q_offset(self, sg=0):
        return lib().ra_partition_q_offset(*self._a(), sg)

    def k_offset_for_step(self, step, sg=0):
        return lib().ra_partition_k_offset_for_step(*self._a(), step, sg)

    def k_offset_for_source(self, source_rank, sg=0):
        return lib().ra_partition_k_offset_for_source(*self._a(), source_rank, sg)

    def local_chunk_len(self, sg=0):
        return lib().ra_partition_local_chunk_len(self.cp_size, self.seq, self.mode, self.n_splits)

    def next_rank(self):
        return lib().ra_partition_next_rank(self.cp_size, self.rank)

    def prev_rank(self):
        return lib().ra_partition_prev_rank(self.cp_size, self.rank)

    def num_sub_groups(self):
        return lib().ra_partition_num_sub_groups(self.mode, self.n_splits)

    def position_stride(self):
        return lib().ra_partition_position_stride(self.cp_size, self.mode)

    def step_maps(self, step):
        """(qmap, kmap, stride) of this rank at ring step ``step``."""
        qm, km = SegMap(), SegMap()
        stride = lib().ra_ring_step_maps(*self._a(), step, C.byref(qm), C.byref(km))
        if stride < 1:
            raise ValueError("bad partition")
        return qm, km, stride

    def local_positions(self):
        """Global position of every local row, sub-groups concatenated (a LongTensor)."""
        n = self.local_chunk_len()
        st = self.position_stride()
        parts = [self.q_offset(sg) + torch.arange(n) * st for sg in range(self.num_sub_groups())]
        return torch.cat(parts)


def visible_pairs(qmap, kmap, stride, causal, doc_len=0):
    return lib().ra_ring_step_visible_pairs(C.byref(qmap), C.byref(kmap), stride, int(causal),
                                            doc_len)


class DeviceKVCache:
    """Mirror of ``DeviceKVCache<T>`` (reference src/kv_cache.hpp:22-73)."""

    def __init__(self, batch, kv_heads, s_max, head_dim, dtype=torch.float32):
        self._h = C.c_void_p()
        self.dtype = dtype
        self._batch, self._kv_heads, self._s_max, self._head_dim = batch, kv_heads, s_max, head_dim
        check(lib().ra_kv_cache_create(_DT[dtype], batch, kv_heads, s_max, head_dim,
                                       C.byref(self._h)))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib().ra_kv_cache_destroy(h)
            self._h = None

    def current_len(self):
        return lib().ra_kv_cache_len(self._h)

    def s_max(self):
        return self._s_max

    def batch(self):
        return self._batch

    def kv_heads(self):
        return self._kv_heads

    def head_dim(self):
        return self._head_dim

    def numel(self):
        return self._batch * self._kv_heads * self._s_max * self._head_dim

    def k_ptr(self):
        return lib().ra_kv_cache_k(self._h)

    def v_ptr(self):
        return lib().ra_kv_cache_v(self._h)

    def _view(self, ptr):
        """Zero-copy torch view of a cache tensor (batch, kv_heads, s_max, head_dim)."""
        shape = (self._batch, self._kv_heads, self._s_max, self._head_dim)
        es = torch.empty(0, dtype=self.dtype).element_size()

        class _Dev:
            pass

        d = _Dev()
        d.__cuda_array_interface__ = {"shape": shape, "typestr": "<f4" if es == 4 else "<i2",
                                      "data": (int(ptr), False), "version": 2}
        t = torch.as_tensor(d, device="cuda")
        return t if es == 4 else t.view(self.dtype)

    def k_view(self):
        return self._view(self.k_ptr())

    def v_view(self):
        return self._view(self.v_ptr())

    def copy_prefill(self, k_src, v_src, prefill_len):
        check(lib().ra_kv_cache_copy_prefill(self._h, _ptr(k_src), _ptr(v_src), prefill_len,
                                             _stream()))

    def append(self, k_step, v_step):
        check(lib().ra_kv_cache_append(self._h, _ptr(k_step), _ptr(v_step), _stream()))

    def reset(self):
        lib().ra_kv_cache_reset(self._h)


def run_local_decode_step(q, cache: DeviceKVCache, heads, q_pos_global, cache_k_offset, causal,
                          out):
    """``run_local_decode_step[_fp16]`` (reference src/decode_op.hpp:34-42); dtype = cache's."""
    check(lib().ra_local_decode_step(_ptr(q), cache._h, heads, q_pos_global, cache_k_offset,
                                     int(causal), _ptr(out), _stream()))


run_local_decode_step_fp16 = run_local_decode_step


class Ring:
    """A ring of ranks over NCCL; one process per GPU. Bootstrap through torch.distributed."""

    def __init__(self, rank=0, cp_size=1, group=None):
        self.rank, self.cp_size = rank, cp_size
        self._h = C.c_void_p()
        ident = C.create_string_buffer(128)
        if cp_size > 1:
            import torch.distributed as dist
            if rank == 0:
                check(lib().ra_nccl_unique_id(ident))
            t = torch.frombuffer(bytearray(ident.raw), dtype=torch.uint8).clone()
            if dist.get_backend(group) == "nccl":
                t = t.cuda()
            dist.broadcast(t, src=0, group=group)
            ident = C.create_string_buffer(bytes(t.cpu().numpy().tobytes()), 128)
        check(lib().ra_ring_create(rank, cp_size, ident, C.byref(self._h)))
        self._work = None

    def close(self):
        if self._h:
            lib().ra_ring_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def prefill(self, q, k, v, *, seq, causal, layout=0, n_splits=2, doc_len=0, want_lse=False,
                timed=False, out=None, schedule="auto", ring2d_nodes=1):
        """One overlapped ring pass (``run_ring_attention`` in ring-overlap mode, reference
        src/ring_loop_fp16.cu:522-818) over this rank's device shards. ``schedule`` is "ring"
        (hop-by-hop rotation, overlapped), "gather" (one all-gather, the reference's allgather mode),
        "blocking" (the rotation with nothing overlapped, ring-blocking), "ring2d" (ring-2d over
        ``ring2d_nodes`` groups of ranks) or "auto" (gather or ring by shard size)."""
        B, H, sloc, D = q.shape
        cfg = self._cfg(B, H, k.shape[1], seq, D, _dtype(q), causal, layout, n_splits, doc_len, schedule,
                        ring2d_nodes)
        need = lib().ra_ring_prefill_workspace_bytes(self._h, C.byref(cfg))
        if self._work is None or self._work.numel() < need:
            self._work = torch.empty(need, dtype=torch.uint8, device=q.device)
        if out is None:
            out = torch.empty((B, H, sloc, D), dtype=torch.float32, device=q.device)
        lse = torch.empty((B, H, sloc), dtype=torch.float32, device=q.device) if want_lse else None
        res = RingResult()
        check(lib().ra_ring_prefill(self._h, C.byref(cfg), _ptr(q), _ptr(k), _ptr(v), _ptr(out),
                                    _ptr(lse), _ptr(self._work), self._work.numel(), _stream(),
                                    C.byref(res) if timed else None))
        ret = [out]
        if want_lse:
            ret.append(lse)
        if timed:
            ret.append(res)
        return ret[0] if len(ret) == 1 else tuple(ret)

    SCHEDULES = {"auto": 0, "ring": 1, "gather": 2, "blocking": 3, "ring2d": 4}

    def _cfg(self, B, H, kvH, seq, D, dtype, causal, layout, n_splits, doc_len, schedule, nodes=1):
        return RingConfig(B, H, kvH, seq, D, dtype, int(causal), layout, n_splits, doc_len,
                          self.SCHEDULES[schedule], nodes)

    def plan(self, *, batch, heads, kv_heads, seq, head_dim, dtype=torch.float16, causal=True, layout=0,
             n_splits=2, doc_len=0, schedule="auto", ring2d_nodes=1):
        """(schedule name, key parts, kernel launches per pass) of ``prefill`` for this config."""
        cfg = self._cfg(batch, heads, kv_heads, seq, head_dim, _DT[dtype], causal, layout, n_splits,
                        doc_len, schedule, ring2d_nodes)
        sched, parts, launches = C.c_int(), C.c_int(), C.c_int()
        check(lib().ra_ring_prefill_plan(self._h, C.byref(cfg), C.byref(sched), C.byref(parts),
                                         C.byref(launches)))
        names = {v: k for k, v in self.SCHEDULES.items()}
        return names[sched.value], parts.value, launches.value

    def prefill_host(self, q, k, v, out, *, seq, causal, layout=0, n_splits=2, doc_len=0, lse=None,
                     schedule="auto", timed=False):
        """The pass from host tensors (pinned) holding this rank's shards into the host tensor
        ``out``; returns after completion (``ra_ring_prefill_host``; the reference uploads inside
        its timed pass too, src/ring_loop_fp16.cu:624-626)."""
        B, H, sloc, D = q.shape
        cfg = self._cfg(B, H, k.shape[1], seq, D, _dtype(q), causal, layout, n_splits, doc_len, schedule)
        res = RingResult()
        check(lib().ra_ring_prefill_host(self._h, C.byref(cfg), q.data_ptr(), k.data_ptr(),
                                         v.data_ptr(), out.data_ptr(),
                                         lse.data_ptr() if lse is not None else None,
                                         C.byref(res) if timed else None))
        return res if timed else None

    def decode_step(self, q, k_new, v_new, owner_rank, cache: DeviceKVCache, current_len_per_rank,
                    out, timed=False):
        """``run_ring_decode_step`` (reference src/ring_decode.hpp:67-69); dtype = cache's."""
        lens = (C.c_int * len(current_len_per_rank))(*current_len_per_rank)
        res = RingResult()
        B, H = q.shape[0], q.shape[1]
        check(lib().ra_ring_decode_step(self._h, B, H, _ptr(q), _ptr(k_new), _ptr(v_new),
                                        owner_rank, cache._h, lens, _ptr(out), _stream(),
                                        C.byref(res) if timed else None))
        return res if timed else None
