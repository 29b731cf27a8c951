"""Build ``libkla_b200.so`` (the C-ABI library of hand-written sm_100a kernels)
in-tree with nvcc. nvcc cross-compiles, so no GPU is needed to build.

    python "kalman-linear-attention_b200/build.py"          # build what is stale
    python "kalman-linear-attention_b200/build.py" --force
    python "kalman-linear-attention_b200/build.py" -v       # with ptxas resource usage

The two scan kernels are instantiated for every (activation types, lanes per
channel, prior read-out) combination, a few hundred kernels in all, so the
instantiations are cut into slices (``csrc/kla_scan_inst.cu`` compiled with
different ``-DKLA_INST_*``) that compile in parallel; ``csrc/kla_capi.cu`` holds
the entry points and the small kernels. Objects are kept under ``build/`` and
only recompiled when a file they include has changed.
"""

from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libkla_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]  # no --split-compile: with it the optimiser's result (and the kernels' speed) varied from build to build

_SCAN_DEPS = ["kla_common.cuh", "kla_fwd.cuh", "kla_bwd.cuh", "kla_agg.cuh", "kla_launch.cuh", "kla_scan_inst.cu"]


def _units():
    """(object name, source, extra flags, files it depends on)."""
    units = [("capi", "kla_capi.cu", [], None)]  # None: every file under csrc/ and include/
    for kind, kname in ((0, "fwd"), (1, "bwd")):
        for dt, dname in ((0, "f32"), (1, "bf16f32"), (2, "bf16")):
            for lp, lname in ((0, "lo"), (1, "hi")):
                flags = [f"-DKLA_INST_KIND={kind}", f"-DKLA_INST_DT={dt}", f"-DKLA_INST_LPCS={lp}"]
                units.append((f"scan_{kname}_{dname}_{lname}", "kla_scan_inst.cu", flags, _SCAN_DEPS))
    units.append(("scan_agg", "kla_scan_inst.cu", ["-DKLA_INST_KIND=2"], _SCAN_DEPS))
    return units


def _nvcc() -> str:
    for cand in (os.environ.get("KLA_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set KLA_B200_NVCC")


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cuh"))
                  + glob.glob(os.path.join(INCLUDE, "*.h")))


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def is_stale() -> bool:
    return _newer(LIB, _sources() + [os.path.abspath(__file__)])


def build(force: bool = False, verbose: bool = False, jobs: int | None = None) -> str:
    """Compile the slices that are out of date and link the shared library; returns its path."""
    if not force and not is_stale():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    # the host compiler named by CC/CXX may be a wrapper nvcc cannot drive
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    todo, objs = [], []
    for name, src, flags, deps in _units():
        obj = os.path.join(OBJ, name + ".o")
        objs.append(obj)
        dep_files = _sources() if deps is None else [os.path.join(CSRC, d) for d in deps]
        if force or _newer(obj, dep_files + [os.path.abspath(__file__)]):
            cmd = [nvcc, *NVCC_FLAGS, *flags, "-I", INCLUDE, "-c", os.path.join(CSRC, src), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            todo.append((name, cmd))

    def run(item):
        name, cmd = item
        res = subprocess.run(cmd, capture_output=True, text=True, env=env)
        return name, cmd, res

    jobs = jobs or int(os.environ.get("KLA_B200_BUILD_JOBS", 0)) or os.cpu_count() or 4
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, jobs)) as pool:
        for name, cmd, res in pool.map(run, todo):
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {name}:\n{' '.join(cmd)}\n{res.stdout}{res.stderr}")
            if verbose:
                print(f"== {name}\n{res.stderr}")
    link = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-o", LIB, *objs]
    res = subprocess.run(link, capture_output=True, text=True, env=env)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
