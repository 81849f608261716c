"""Helpers shared by the tests: closeness as the reference's tests define it, seeded inputs."""
import numpy as np


def close(a, b, atol, rtol):
    """|a-b| <= atol + rtol*max(|a|,|b|), element-wise (reference tests/test_attention_step.cu:31-35)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.abs(a - b) <= atol + rtol * np.maximum(np.abs(a), np.abs(b))


def assert_close(a, b, atol, rtol, what=""):
    ok = close(a, b, atol, rtol)
    if not ok.all():
        a = np.asarray(a, dtype=np.float64)
        b = np.asarray(b, dtype=np.float64)
        bad = np.argwhere(~ok)
        i = tuple(bad[0])
        raise AssertionError(
            f"{what}: {len(bad)} of {ok.size} elements differ; first at {i}: got {a[i]!r} want {b[i]!r}; "
            f"max abs diff {np.nanmax(np.abs(a - b)):.3e} (atol={atol}, rtol={rtol})")


def normal_inputs(seed, B, H, kvH, Sq, Sk, D, scale=1.0):
    rng = np.random.default_rng(seed)
    q = (rng.standard_normal((B, H, Sq, D)) * scale).astype(np.float32)
    k = (rng.standard_normal((B, kvH, Sk, D)) * scale).astype(np.float32)
    v = (rng.standard_normal((B, kvH, Sk, D)) * scale).astype(np.float32)
    return q, k, v


def round_to(x, dtype):
    """Round fp32 values through fp16 / bf16 and back (what the GPU kernels actually see)."""
    import torch
    return torch.from_numpy(x).to(dtype).to(torch.float32).numpy()
