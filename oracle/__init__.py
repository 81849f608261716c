"""CPU oracle for the ring-attention hot path: TEST INFRASTRUCTURE ONLY.

Loads ``liboracle.so`` (the plain-C restatement in ``oracle.c``) and, when it
was built, ``_ref/libref_oracle.so`` (the reference's own host sources compiled
by ``oracle/Makefile``). Only the test-suite, the smoke check and the benchmark's
CPU-baseline leg import this package; the shipped library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_F = C.POINTER(C.c_float)
_I = C.POINTER(C.c_int)


def build(verbose: bool = False) -> None:
    """Compile liboracle.so and (if the reference tree is present) _ref/libref_oracle.so."""
    r = subprocess.run(["make", "-C", _HERE], capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout, r.stderr)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed")
    # the reference's own test programs against the product library (needs the library built
    # and the reference tree mounted; otherwise prebuilt binaries are kept)
    lib = os.path.join(_HERE, "..", "ring_attention_b200", "libring_attention_b200.so")
    if os.path.exists(lib):
        r = subprocess.run(["make", "-C", _HERE, "reftests"], capture_output=True, text=True)
        if verbose or r.returncode != 0:
            print(r.stdout[-3000:], r.stderr[-3000:])
        if r.returncode != 0:
            raise RuntimeError("building the reference's test programs failed")


def _load(path):
    if not os.path.exists(path):
        return None
    return C.CDLL(path)


_port = None
_ref = None


def port():
    global _port
    if _port is None:
        p = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(p):
            build()
        _port = C.CDLL(p)
        _port.orc_gen_elem.restype = C.c_float
        _port.orc_xorshift32_fill.restype = C.c_uint32
    return _port


def ref():
    """The compiled reference host code, or None when it was never built."""
    global _ref
    if _ref is None:
        _ref = _load(os.path.join(_HERE, "_ref", "libref_oracle.so"))
        if _ref is not None:
            _ref.ref_gen_elem.restype = C.c_float
            _ref.ref_xorshift32_fill.restype = C.c_uint32
    return _ref


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_F)


def cpu_attention(q, k, v, causal, kv_heads=0, want_lse=False, impl="port", threads=1):
    """q (B,H,Sq,D), k/v (B,kvH,Sk,D) float32 -> out (B,H,Sq,D) [, lse (B,H,Sq)]."""
    q, qp = _f32(q)
    k, kp = _f32(k)
    v, vp = _f32(v)
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    out = np.empty_like(q)
    if impl == "port":
        lse = np.empty((B, H, Sq), np.float32) if want_lse else None
        port().orc_cpu_attention(qp, kp, vp, out.ctypes.data_as(_F),
                                 lse.ctypes.data_as(_F) if want_lse else None,
                                 B, H, Sq, Sk, D, kv_heads, int(bool(causal)))
        return (out, lse) if want_lse else out
    r = ref()
    if r is None:
        raise RuntimeError("oracle/_ref/libref_oracle.so was not built")
    if want_lse:
        raise ValueError("the reference cpu_attention does not return lse")
    if threads > 1:
        r.ref_cpu_attention_mt(qp, kp, vp, out.ctypes.data_as(_F), B, H, Sq, Sk, D, kv_heads,
                               int(bool(causal)), int(threads))
    else:
        r.ref_cpu_attention(qp, kp, vp, out.ctypes.data_as(_F), B, H, Sq, Sk, D, kv_heads,
                            int(bool(causal)))
    return out


def attention_row(q_row, k, v, visible=None):
    """One query row against keys k/v (n,D) of one kv head -> (out_row (D,), lse)."""
    q_row, qp = _f32(q_row)
    k, kp = _f32(k)
    v, vp = _f32(v)
    n, D = k.shape
    out = np.empty(D, np.float32)
    lse = C.c_float()
    vis = None
    if visible is not None:
        visible = np.ascontiguousarray(visible, dtype=np.uint8)
        vis = visible.ctypes.data_as(C.POINTER(C.c_ubyte))
    port().orc_attention_row(qp, kp, vp, n, D, vis, out.ctypes.data_as(_F), C.byref(lse))
    return out, lse.value


def attention_init(shape_out, shape_m):
    out = np.zeros(shape_out, np.float32)
    m = np.full(shape_m, -np.inf, np.float32)
    l = np.zeros(shape_m, np.float32)
    return out, m, l


def attention_step(q, k, v, out, m, l, q_base, k_base, stride=1, causal=False, kv_heads=0,
                   q_seg_len=None, k_seg_len=None, doc_len=0):
    """In-place online-softmax ring step on (out, m, l); positions are piecewise affine."""
    q, qp = _f32(q)
    k, kp = _f32(k)
    v, vp = _f32(v)
    assert out.dtype == np.float32 and out.flags.c_contiguous
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    qb = np.ascontiguousarray(np.atleast_1d(q_base), dtype=np.int32)
    kb = np.ascontiguousarray(np.atleast_1d(k_base), dtype=np.int32)
    qsl = q_seg_len or Sq // len(qb)
    ksl = k_seg_len or Sk // len(kb)
    port().orc_attention_step(qp, kp, vp, out.ctypes.data_as(_F), m.ctypes.data_as(_F),
                              l.ctypes.data_as(_F), B, H, Sq, Sk, D, kv_heads,
                              qb.ctypes.data_as(_I), len(qb), qsl, kb.ctypes.data_as(_I), len(kb),
                              ksl, stride, int(bool(causal)), C.c_longlong(doc_len))


def attention_finalize(out, l):
    D = out.shape[-1]
    port().orc_attention_finalize(out.ctypes.data_as(_F), l.ctypes.data_as(_F),
                                  C.c_size_t(l.size), D)


def decode_partial_merge(gathered, cp_size, BH, D):
    g, gp = _f32(gathered)
    out = np.empty((BH, D), np.float32)
    m = np.empty(BH, np.float32)
    l = np.empty(BH, np.float32)
    port().orc_decode_partial_merge(gp, out.ctypes.data_as(_F), m.ctypes.data_as(_F),
                                    l.ctypes.data_as(_F), cp_size, BH, D)
    return out, m, l


def xorshift32_fill(seed, n, impl="port"):
    out = np.empty(n, np.float32)
    lib = port() if impl == "port" else ref()
    fn = lib.orc_xorshift32_fill if impl == "port" else lib.ref_xorshift32_fill
    fn(C.c_uint32(seed), out.ctypes.data_as(_F), C.c_size_t(n))
    return out


def gen_elem(seed, tensor_id, b, h, s, d, impl="port"):
    lib = port() if impl == "port" else ref()
    fn = lib.orc_gen_elem if impl == "port" else lib.ref_gen_elem
    return float(fn(C.c_uint32(seed), tensor_id, b, h, s, d))


MODES = {"contiguous": 0, "zigzag": 1, "striped": 2}


class Partition:
    """Index maps of the reference's RingPartition (port or compiled reference)."""

    def __init__(self, cp, rank, seq, mode="contiguous", n_splits=2, impl="port"):
        self.cp, self.rank, self.seq, self.n_splits = cp, rank, seq, n_splits
        self.mode = MODES[mode] if isinstance(mode, str) else mode
        self.impl = impl
        self.lib = port() if impl == "port" else ref()

    def q_offset(self, sg=0):
        a = (self.cp, self.rank, self.seq, self.mode, self.n_splits, sg)
        return (self.lib.orc_part_q_offset if self.impl == "port" else self.lib.ref_part_q_offset)(*a)

    def k_offset_for_step(self, step, sg=0):
        a = (self.cp, self.rank, self.seq, self.mode, self.n_splits, step, sg)
        return (self.lib.orc_part_k_offset_for_step if self.impl == "port"
                else self.lib.ref_part_k_offset_for_step)(*a)

    def k_offset_for_source(self, source, sg=0):
        a = (self.cp, self.rank, self.seq, self.mode, self.n_splits, source, sg)
        return (self.lib.orc_part_k_offset_for_source if self.impl == "port"
                else self.lib.ref_part_k_offset_for_source)(*a)

    def local_chunk_len(self):
        if self.impl == "port":
            return self.lib.orc_part_local_chunk_len(self.cp, self.seq, self.mode, self.n_splits)
        return self.lib.ref_part_local_chunk_len(self.cp, self.rank, self.seq, self.mode, self.n_splits)

    def num_sub_groups(self):
        if self.impl == "port":
            return self.lib.orc_part_num_sub_groups(self.mode, self.n_splits)
        return self.lib.ref_part_num_sub_groups(self.cp, self.rank, self.seq, self.mode, self.n_splits)

    def position_stride(self):
        if self.impl == "port":
            return self.lib.orc_part_position_stride(self.cp, self.mode)
        return self.lib.ref_part_position_stride(self.cp, self.rank, self.seq, self.mode, self.n_splits)

    def next_rank(self):
        if self.impl == "port":
            return self.lib.orc_part_next_rank(self.cp, self.rank)
        return self.lib.ref_part_next_rank(self.cp, self.rank, self.seq)

    def prev_rank(self):
        if self.impl == "port":
            return self.lib.orc_part_prev_rank(self.cp, self.rank)
        return self.lib.ref_part_prev_rank(self.cp, self.rank, self.seq)


def ring2d_source(num_nodes, gpus_per_node, node, local, m, i, impl="port"):
    """Shard (global rank) that GPU (node, local) holds at macro-step m, inner round i of the
    hierarchical ring (reference src/ring2d_schedule.cpp:30-42); port or compiled reference."""
    fn = port().orc_ring2d_source if impl == "port" else ref().ref_ring2d_source
    return int(fn(num_nodes, gpus_per_node, node, local, m, i))
