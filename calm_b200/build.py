"""Build the shared libraries in-tree with nvcc for sm_100a (no JIT cache: the .so files ship to the GPU box).

Two targets, each its own library so that a host compiles only what its model family needs:
  engine  libcalm_b200.so      the calm backend boundary (single-sequence Llama-shaped models)
  seq     libcalm_b200_seq.so  layer-list models served to batches of sequences
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(HERE, "..", "include")
TARGETS = {
    "engine": {"lib": os.path.join(HERE, "libcalm_b200.so"), "sources": ["engine.cu"],
               "deps": ["attn.cuh", "common.cuh", "tc05.cuh", "prefill.cuh", "ring.cuh", "stages.cuh", os.path.join(INCLUDE, "calm_b200.h"), os.path.join(INCLUDE, "calm_model.h")]},
    "seq": {"lib": os.path.join(HERE, "libcalm_b200_seq.so"), "sources": ["seqmodel.cu"],
            "deps": ["common.cuh", "tc05.cuh", "seqkernels.cuh", "seqgemm_tc.cuh", os.path.join(INCLUDE, "calm_b200_seq.h")]},
}
LIB = TARGETS["engine"]["lib"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-ccbin", "/usr/bin/g++",
         "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-shared"]


def stale(target: str = "engine") -> bool:
    t = TARGETS[target]
    if not os.path.exists(t["lib"]):
        return True
    when = os.path.getmtime(t["lib"])
    deps = [os.path.join(CSRC, f) for f in t["sources"] + t["deps"]] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > when for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False, target: str = "engine") -> str:
    t = TARGETS[target]
    if not force and not stale(target):
        return t["lib"]
    tmp = t["lib"] + ".%d.tmp" % os.getpid()  # two hosts starting at once never see a half-written library
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + [os.path.join(CSRC, f) for f in t["sources"]] + ["-lcuda", "-o", tmp]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc failed building " + os.path.basename(t["lib"]))
    os.replace(tmp, t["lib"])
    if verbose:
        sys.stderr.write(r.stderr)
    return t["lib"]


def build_all(force: bool = False, verbose: bool = False) -> None:
    for target in TARGETS:
        build(force, verbose, target)


if __name__ == "__main__":
    names = [a for a in sys.argv[1:] if a in TARGETS] or list(TARGETS)
    for n in names:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, target=n))
