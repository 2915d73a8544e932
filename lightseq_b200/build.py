"""In-tree build of the native libraries (sm_100a only).

``python -m lightseq_b200.build`` compiles

* ``lightseq_b200/libls100.so``      — CUDA kernels + host runtime behind the C ABI of ``include/ls100.h``
* ``lightseq_b200/_ls100_py*.so``    — pybind11 module mirroring ``lightseq.inference``

with nvcc/g++ directly (no JIT cache: the built files sit next to the sources).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libls100.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-I", str(ROOT / "include")]


def _sources():
    return sorted(CSRC.glob("kernels/*.cu")) + sorted(CSRC.glob("host/*.cu")) + sorted(CSRC.glob("host/*.cpp"))


def _headers():
    return sorted(CSRC.glob("**/*.h")) + sorted(CSRC.glob("**/*.cuh")) + sorted((ROOT / "include").glob("*.h"))


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(str(p).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build command failed:\n  %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    return r.stdout + r.stderr


def pybind_path() -> Path:
    return PKG / ("_ls100_py" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(verbose: bool = False, force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    hdr_digest = _digest(_headers())
    srcs = _sources()
    jobs = []
    for src in srcs:
        obj = OBJ / (src.stem + ".o")
        stamp = OBJ / (src.stem + ".stamp")
        want = _digest([src]) + hdr_digest + " ".join(NVCC_FLAGS)
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == want:
            continue
        cmd = [NVCC, *ARCH, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        jobs.append((cmd, stamp, want))

    def work(job):
        cmd, stamp, want = job
        out = _run(cmd)
        stamp.write_text(want)
        return out

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(work, jobs):
                if verbose and out.strip():
                    print(out)
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if jobs or not LIB.exists():
        _run([NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"])
    # pybind11 module (host C++ only; links against libls100.so next to it)
    pyb_src = CSRC / "pybind" / "pybind_model.cpp"
    if pyb_src.exists():
        import pybind11

        out = pybind_path()
        stamp = OBJ / "pybind.stamp"
        want = _digest([pyb_src]) + hdr_digest
        if force or jobs or not out.exists() or not stamp.exists() or stamp.read_text() != want:
            _run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I", pybind11.get_include(), "-I",
                  sysconfig.get_paths()["include"], "-I", str(ROOT / "include"), "-I", "/usr/local/cuda/include",
                  str(pyb_src), "-o", str(out), "-L", str(PKG), "-l:libls100.so", "-Wl,-rpath,$ORIGIN"])
            stamp.write_text(want)
    return LIB


if __name__ == "__main__":
    build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built", LIB)
