"""The reference's OWN test programs, compiled unchanged from its source tree and linked against
this library through ring_attention_b200/compat/reference_shim.cu (oracle/Makefile, target
reftests; binaries under oracle/_ref/tests). Each program carries its own oracle (the reference's
cpu_attention) and tolerances (1e-4 fp32, 1e-2 fp16, 1e-3 / 5e-2 decode, exact cache equality)
and returns 0 on success."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "tests")


def run(name, timeout=600):
    path = os.path.join(BIN, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} was not built (oracle/_ref/tests is made where the reference tree is mounted)")
    r = subprocess.run([path], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, f"{name} failed:\n{r.stdout[-2000:]}\n{r.stderr[-2000:]}"
    return r.stdout


@pytest.mark.parametrize("name,expect", [("test_ring_partition", "All ring_partition tests passed"),
                                         ("test_cpu_attention", "cpu_attention OK"),
                                         ("test_gen_elem", "All gen_elem tests passed")])
def test_reference_host_programs(name, expect):
    assert expect in run(name)


@pytest.mark.gpu
@pytest.mark.parametrize("name,expect", [
    ("test_smoke", None), ("test_device_tensor", None),
    ("test_attention_step", "attention_step OK"), ("test_attention_step_fp16", "attention_step_fp16 OK"),
    ("test_attention_step_segmented", None), ("test_flash_attention", None),
    ("test_flash_attention_fp16", None), ("test_kv_cache", None), ("test_decode_op", None)])
def test_reference_gpu_programs(name, expect):
    out = run(name)
    if expect:
        assert expect in out
    assert "FAIL" not in out
