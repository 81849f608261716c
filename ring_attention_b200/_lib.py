"""ctypes binding of ``libring_attention_b200.so`` (the C ABI in ``include/ring_attention_b200.h``).

There is no fallback: if the library is missing it is built once with nvcc, and if that
fails the import fails.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libring_attention_b200.so")

RA_F32, RA_F16, RA_BF16 = 0, 1, 2
RA_STEP_CAUSAL, RA_STEP_FRESH, RA_STEP_FINALIZE, RA_STEP_FORCE_SIMT = 1, 2, 4, 8
RA_STEP_P_IN_SMEM = 16
RA_STEP_CTA_PAIR = 32
RA_MAX_SEG = 16

STATUS_NAMES = {0: "RA_OK", 1: "RA_ERR_INVALID", 2: "RA_ERR_CUDA", 3: "RA_ERR_UNSUPPORTED",
                4: "RA_ERR_NCCL", 5: "RA_ERR_DEVICE_WAIT", 6: "RA_ERR_OVERFLOW"}


class Shape(C.Structure):
    """ra_shape: mirrors AttentionShape (reference src/attention.hpp:19-26)."""
    _fields_ = [("batch", C.c_int), ("heads", C.c_int), ("seq_q", C.c_int), ("seq_k", C.c_int),
                ("head_dim", C.c_int), ("kv_heads", C.c_int)]


class SegMap(C.Structure):
    """ra_segmap: mirrors SegMap (reference src/attention.hpp:102-107)."""
    _fields_ = [("n_seg", C.c_int), ("seg_len", C.c_int), ("base", C.c_int * RA_MAX_SEG)]

    @classmethod
    def make(cls, bases, seg_len):
        bases = list(bases)
        if not 1 <= len(bases) <= RA_MAX_SEG:
            raise ValueError(f"1..{RA_MAX_SEG} segments, got {len(bases)}")
        m = cls()
        m.n_seg, m.seg_len = len(bases), int(seg_len)
        for i, b in enumerate(bases):
            m.base[i] = int(b)
        return m


class RingConfig(C.Structure):
    """ra_ring_config: the ring-overlap part of RingConfig (reference src/ring_loop.hpp:38-62)."""
    _fields_ = [("batch", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int), ("seq", C.c_int),
                ("head_dim", C.c_int), ("dtype", C.c_int), ("causal", C.c_int),
                ("layout", C.c_int), ("n_splits", C.c_int), ("doc_len", C.c_longlong),
                ("schedule", C.c_int), ("ring2d_nodes", C.c_int)]


class RingResult(C.Structure):
    """ra_ring_result: mirrors RingResult (reference src/ring_loop.hpp:30-36)."""
    _fields_ = [("comm_ms", C.c_double), ("comp_ms", C.c_double), ("wait_ms", C.c_double),
                ("total_ms", C.c_double)]


class RingAttentionError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {msg}")
        self.code = code


_P = C.c_void_p
_SIG = {
    "ra_last_error": (C.c_char_p, []),
    "ra_version": (C.c_int, []),
    "ra_device_status": (C.c_int, [C.POINTER(C.c_int)]),
    "ra_attention_init": (C.c_int, [_P, _P, _P, C.POINTER(Shape), C.c_size_t, _P]),
    "ra_attention_step": (C.c_int, [_P, _P, _P, _P, _P, _P, C.POINTER(Shape), C.c_int, C.c_int,
                                    C.c_int, _P, C.c_int]),
    "ra_attention_step_fp16": (C.c_int, [_P, _P, _P, _P, _P, _P, C.POINTER(Shape), C.c_int,
                                         C.c_int, C.c_int, _P, C.c_int]),
    "ra_attention_step_segmented": (C.c_int, [_P, _P, _P, _P, _P, _P, C.POINTER(Shape),
                                              C.POINTER(SegMap), C.POINTER(SegMap), C.c_int, _P]),
    "ra_attention_step_ex": (C.c_int, [C.c_int, _P, _P, _P, _P, _P, _P, C.POINTER(Shape),
                                       C.POINTER(SegMap), C.POINTER(SegMap), C.c_int, C.c_uint,
                                       C.c_longlong, C.c_int, _P]),
    "ra_attention_step_stacked": (C.c_int, [C.c_int, _P, _P, _P, _P, _P, _P, C.POINTER(Shape),
                                            C.POINTER(SegMap), C.POINTER(SegMap),
                                            C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int,
                                            C.c_int, C.c_int, C.c_uint, C.c_longlong, _P]),
    "ra_naive_attention": (C.c_int, [_P, _P, _P, _P, C.POINTER(Shape), C.c_int, _P]),
    "ra_attention_finalize": (C.c_int, [_P, _P, C.POINTER(Shape), _P]),
    "ra_attention_lse": (C.c_int, [_P, _P, _P, C.c_size_t, _P]),
    "ra_float_to_half": (C.c_int, [_P, _P, C.c_size_t, _P]),
    "ra_half_to_float": (C.c_int, [_P, _P, C.c_size_t, _P]),
    "ra_float_to_bf16": (C.c_int, [_P, _P, C.c_size_t, _P]),
    "ra_float_to_int8": (C.c_int, [_P, _P, C.c_size_t, _P]),
    "ra_int8_to_float": (C.c_int, [_P, _P, C.c_size_t, _P]),
    "ra_flash_workspace_bytes": (C.c_size_t, [C.POINTER(Shape), C.c_int]),
    "ra_flash_attention": (C.c_int, [_P, _P, _P, _P, C.POINTER(Shape), C.c_int, C.c_int, _P,
                                     C.c_size_t, _P]),
    "ra_prefill_host": (C.c_int, [C.c_int, _P, _P, _P, _P, _P, C.POINTER(Shape),
                                  C.POINTER(SegMap), C.POINTER(SegMap), C.c_int, C.c_uint,
                                  C.c_longlong]),
    "ra_decode_workspace_bytes": (C.c_size_t, [C.POINTER(Shape)]),
    "ra_attention_decode_step": (C.c_int, [C.c_int, _P, _P, _P, _P, _P, _P, C.POINTER(Shape),
                                           C.c_int, C.c_int, C.c_int, _P, C.c_int, _P,
                                           C.c_size_t]),
    "ra_attention_decode_step_noalloc": (C.c_int, [C.c_int, _P, _P, _P, _P, _P, _P, C.POINTER(Shape),
                                                   C.c_int, C.c_int, C.c_int, _P, C.c_int]),
    "ra_decode_partial_merge": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "ra_kv_cache_create": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.POINTER(_P)]),
    "ra_kv_cache_destroy": (None, [_P]),
    "ra_kv_cache_k": (_P, [_P]),
    "ra_kv_cache_v": (_P, [_P]),
    "ra_kv_cache_len": (C.c_int, [_P]),
    "ra_kv_cache_s_max": (C.c_int, [_P]),
    "ra_kv_cache_copy_prefill": (C.c_int, [_P, _P, _P, C.c_int, _P]),
    "ra_kv_cache_append": (C.c_int, [_P, _P, _P, _P]),
    "ra_kv_cache_reset": (None, [_P]),
    "ra_local_decode_step": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "ra_partition_q_offset": (C.c_int, [C.c_int] * 6),
    "ra_partition_k_offset_for_step": (C.c_int, [C.c_int] * 7),
    "ra_partition_k_offset_for_source": (C.c_int, [C.c_int] * 7),
    "ra_partition_local_chunk_len": (C.c_int, [C.c_int] * 4),
    "ra_partition_num_sub_groups": (C.c_int, [C.c_int] * 2),
    "ra_partition_position_stride": (C.c_int, [C.c_int] * 2),
    "ra_partition_next_rank": (C.c_int, [C.c_int] * 2),
    "ra_partition_prev_rank": (C.c_int, [C.c_int] * 2),
    "ra_ring2d_source": (C.c_int, [C.c_int] * 6),
    "ra_ring_gather_part_maps": (C.c_int, [C.c_int] * 7 + [C.POINTER(SegMap), C.POINTER(C.c_int),
                                                     C.POINTER(C.c_int)]),
    "ra_ring_step_maps": (C.c_int, [C.c_int] * 6 + [C.POINTER(SegMap), C.POINTER(SegMap)]),
    "ra_ring_step_visible_pairs": (C.c_double, [C.POINTER(SegMap), C.POINTER(SegMap), C.c_int,
                                                C.c_int, C.c_longlong]),
    "ra_nccl_unique_id": (C.c_int, [C.c_char_p]),
    "ra_ring_create": (C.c_int, [C.c_int, C.c_int, C.c_char_p, C.POINTER(_P)]),
    "ra_ring_create_from_comm": (C.c_int, [C.c_int, C.c_int, _P, C.POINTER(_P)]),
    "ra_ring_destroy": (None, [_P]),
    "ra_ring_prefill_workspace_bytes": (C.c_size_t, [_P, C.POINTER(RingConfig)]),
    "ra_ring_prefill": (C.c_int, [_P, C.POINTER(RingConfig), _P, _P, _P, _P, _P, _P, C.c_size_t,
                                  _P, C.POINTER(RingResult)]),
    "ra_ring_prefill_plan": (C.c_int, [_P, C.POINTER(RingConfig), C.POINTER(C.c_int),
                                       C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "ra_ring_prefill_host": (C.c_int, [_P, C.POINTER(RingConfig), _P, _P, _P, _P, _P,
                                       C.POINTER(RingResult)]),
    "ra_ring_decode_step": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, C.c_int, _P,
                                      C.POINTER(C.c_int), _P, _P, C.POINTER(RingResult)]),
    "ra_ring_decode_step_raw": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P, _P,
                                          C.c_int, C.c_int, _P, _P, C.POINTER(RingResult)]),
    "ra_attention_step_path": (C.c_int, [C.c_int, C.c_int]),
    "ra_debug_set_wait_limit_ns": (None, [C.c_ulonglong]),
    "ra_debug_stall_producer_after": (None, [C.c_int]),
    "ra_debug_set_block_order": (None, [C.c_int]),
}

_lib = None


def lib():
    """The loaded library with argument types set; builds it first if the .so is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            from . import build as _build
            _build.build()
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIG.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code):
    if code != 0:
        raise RingAttentionError(code, lib().ra_last_error().decode(errors="replace"))
