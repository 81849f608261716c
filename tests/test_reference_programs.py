"""The reference's OWN test programs, compiled unchanged from its source tree and linked against
this library through ring_attention_b200/compat/reference_shim.cu (oracle/Makefile, target
reftests; binaries under oracle/_ref/tests). Each program carries its own oracle (the reference's
cpu_attention) and tolerances (1e-4 fp32, 1e-2 fp16, 1e-3 / 5e-2 decode, exact cache equality)
and returns 0 on success."""
import os
import signal
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
                                         ("test_ring2d_schedule", "All ring2d_schedule tests passed"),
                                         ("test_cpu_attention", "cpu_attention OK"),
                                         ("test_gen_elem", "All gen_elem tests passed")])
def test_reference_host_programs(name, expect):
    assert expect in run(name)


@pytest.mark.gpu
@pytest.mark.parametrize("name,expect", [
    ("test_smoke", None), ("test_device_tensor", None), ("test_naive_attention", None),
    ("test_attention_step", "attention_step OK"), ("test_attention_step_fp16", "attention_step_fp16 OK"),
    ("test_attention_step_segmented", None), ("test_flash_attention", None),
    ("test_flash_attention_fp16", None), ("test_kv_cache", None), ("test_decode_op", None)])
def test_reference_gpu_programs(name, expect):
    out = run(name)
    if expect:
        assert expect in out
    assert "FAIL" not in out


# ---- the reference's MPI programs (its CTest smoke matrix, tests/CMakeLists.txt:22-60,108-177) ----

def mpirun(n, prog, *args, timeout=600, extra_env=None):
    import torch
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    launcher, path = os.path.join(BIN, "mpirun"), os.path.join(BIN, prog)
    if not (os.path.exists(launcher) and os.path.exists(path)):
        pytest.skip(f"{prog} was not built (oracle/_ref/tests is made where the reference tree is mounted)")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MINIMPI_TIMEOUT_S="120", **(extra_env or {}))
    # the launcher and its ranks get a process group of their own, so that a timeout can end all of
    # them (and only them) instead of leaving ranks behind with their communicators and GPUs
    proc = subprocess.Popen([launcher, "-n", str(n), path, *args], stdout=subprocess.PIPE,
                            stderr=subprocess.PIPE, text=True, env=env, start_new_session=True)
    try:
        out, err = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGTERM)
        try:
            out, err = proc.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
            out, err = proc.communicate()
        raise AssertionError(f"{prog} {args} timed out after {timeout} s:\n{out[-2000:]}\n{err[-2000:]}")
    assert proc.returncode == 0, f"{prog} {args} failed:\n{out[-2000:]}\n{err[-2000:]}"
    return out


SMOKE = ["--seq", "128", "--heads", "2", "--head_dim", "32", "--iters", "1", "--causal", "1"]


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 2, 4])
@pytest.mark.parametrize("mode,extra", [
    ("allgather", ["--zigzag", "0"]), ("ring-blocking", ["--zigzag", "1"]), ("ring-overlap", ["--zigzag", "1"]),
    ("ring-2d", ["--zigzag", "1"]), ("ring-overlap", ["--striped"]), ("ring-overlap", ["--zigzag-n", "2"]),
    ("ring-overlap", ["--zigzag-n", "2", "--segmented"]),
    ("allgather", ["--zigzag", "0", "--dtype", "fp16"]), ("ring-blocking", ["--zigzag", "1", "--dtype", "fp16"]),
    ("ring-overlap", ["--zigzag", "1", "--dtype", "fp16"]), ("ring-overlap", ["--striped", "--dtype", "fp16"])])
def test_reference_cli_ring_smoke(n, mode, extra):
    import re
    out = mpirun(n, "ring_attention_cli", *SMOKE, *extra, "--mode", mode, "--verify")
    assert re.search(r"verify[^\n]*PASS", out), out[-1500:]


@pytest.mark.gpu
@pytest.mark.parametrize("n,nodes", [(2, 2), (4, 2)])
def test_reference_cli_ring_2d_in_two_tiers(n, nodes):
    # the reference groups ranks by node (one node here); RA_RING2D_NODES makes the shim ask for
    # several groups so that --mode ring-2d runs the two-tier order of Ring2DSchedule on one box
    import re
    out = mpirun(n, "ring_attention_cli", "--seq", "512", "--heads", "4", "--head_dim", "64", "--iters", "1",
                 "--causal", "1", "--zigzag", "1", "--mode", "ring-2d", "--verify",
                 extra_env={"RA_RING2D_NODES": str(nodes)})
    assert re.search(r"verify[^\n]*PASS", out), out[-1500:]


@pytest.mark.gpu
def test_reference_cli_larger_shapes_verify():
    import re
    for args in (["--seq", "1024", "--heads", "4", "--kv_heads", "2", "--head_dim", "64", "--dtype", "fp16",
                  "--zigzag", "1"],
                 ["--seq", "512", "--heads", "4", "--head_dim", "128", "--dtype", "fp16", "--striped"],
                 ["--seq", "512", "--heads", "2", "--head_dim", "128", "--zigzag-n", "2"]):
        out = mpirun(2, "ring_attention_cli", *args, "--iters", "2", "--causal", "1", "--mode", "ring-overlap",
                     "--verify")
        assert re.search(r"verify[^\n]*PASS", out), out[-1500:]


@pytest.mark.gpu
@pytest.mark.parametrize("n,dim", [(2, 32), (2, 64), (4, 32)])
def test_reference_ring_decode_program(n, dim):
    import re
    out = mpirun(n, "test_ring_decode", "--prompt_len", "32", "--n_decode", "4", "--batch", "1", "--heads", "2",
                 "--head_dim", str(dim))
    assert re.search(r"ring_decode[^\n]*PASS", out), out[-1500:]


@pytest.mark.gpu
def test_reference_cli_decode_benchmark_csv():
    import re
    out = mpirun(2, "ring_attention_cli", "--run", "decode", "--prompt-len", "64", "--decode-tokens", "3",
                 "--batch", "1", "--heads", "2", "--head_dim", "32", "--csv-header", "--csv")
    assert re.search(r"decode summary[^\n]*cp_size=2", out), out[-1500:]


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 2])
def test_reference_hello_mpi_cuda(n):
    # apps/hello_mpi_cuda: every rank reports itself (the reference's launcher sanity check)
    out = mpirun(n, "hello_mpi_cuda")
    for r in range(n):
        assert f"rank {r}/{n}" in out and "OK" in out, out[-800:]
