"""Build the CUDA library in-tree: ``python -m ring_attention_b200.build``.

Every ``csrc/*.cu`` is compiled for sm_100a only and linked into
``ring_attention_b200/libring_attention_b200.so`` (the C ABI declared in
``include/ring_attention_b200.h``). nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "csrc", "_obj")
LIB = os.path.join(HERE, "libring_attention_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src, verbose):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    deps = [os.path.join(CSRC, src), os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "tc_common.cuh"),
            os.path.join(HERE, "..", "include", "ring_attention_b200.h")]
    if not _stale(obj, deps):
        return obj, ""
    cmd = [NVCC, *FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


PROBE_SRC = os.path.join(CSRC, "probe")
PROBE_BIN = os.path.join(PROBE_SRC, "_bin")


def build_probes() -> list:
    """The stand-alone timing probes under csrc/probe (measurement tools behind the design notes;
    nothing in the library links them) into csrc/probe/_bin/<name>."""
    os.makedirs(PROBE_BIN, exist_ok=True)
    outs = []
    for f in sorted(os.listdir(PROBE_SRC)):
        if not f.endswith(".cu"):
            continue
        src, exe = os.path.join(PROBE_SRC, f), os.path.join(PROBE_BIN, f[:-3])
        if _stale(exe, [src]):
            r = subprocess.run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
                                "-std=c++17", "-o", exe, src], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {f}:\n{r.stdout}\n{r.stderr}")
        outs.append(exe)
    return outs


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for f in os.listdir(OBJ):
            os.remove(os.path.join(OBJ, f))
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-ldl",
               "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
    if "--probes" in sys.argv:
        print("\n".join(build_probes()))
