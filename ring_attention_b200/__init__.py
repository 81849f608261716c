"""B200-native ring attention: the reference's operator API over a C-ABI CUDA library.

``ring_attention_b200._lib`` binds the C ABI; ``ring_attention_b200.api`` mirrors the
reference's host-side operator interface (``launch_attention_*``, ``DeviceKVCache``,
``RingPartition``, ``run_local_decode_step``, the ring drivers) on torch CUDA tensors,
which are used only as device buffers.
"""
from ._lib import (RA_BF16, RA_F16, RA_F32, RA_STEP_CAUSAL, RA_STEP_FINALIZE,  # noqa: F401
                   RA_STEP_FORCE_SIMT, RA_STEP_FRESH, RingAttentionError, SegMap, Shape, lib)

__all__ = ["lib", "Shape", "SegMap", "RingAttentionError"]
