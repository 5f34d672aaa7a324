"""Build of the CUDA library (sm_100a only) with plain nvcc, in-tree.

`python -m lumen_b200.build` compiles lumen_b200/csrc/*.cu into
lumen_b200/_build/*.o and links lumen_b200/liblumen_moe_b200.so. Objects are
rebuilt only when a source or header is newer. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "_build"
LIB = PKG / "liblumen_moe_b200.so"
SOURCES = ["decode.cu", "decode_small.cu", "decode_fused.cu", "static_scratch.cu", "misc.cu", "route_large.cu", "route_tc.cu", "prefill_tc.cu", "ep_push.cu", "host_moe.cu", "lbc_index.cu", "api.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put /usr/local/cuda/bin on PATH)")


def _newest_header() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.hpp"))
    hdrs.append(PKG.parent / "include" / "lumen_moe.h")
    return max(h.stat().st_mtime for h in hdrs)


def build(verbose: bool = False, force: bool = False) -> Path:
    nvcc = _nvcc()
    BUILD.mkdir(exist_ok=True)
    hdr_time = _newest_header()
    sources = [s for s in SOURCES if (CSRC / s).exists()]
    jobs = []
    for src in sources:
        s = CSRC / src
        o = BUILD / (s.stem + ".o")
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_time):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        # Outputs are written under a private name and renamed into place: a process that loads
        # the library (or another build running at the same time) never sees a half-written file.
        out = Path(cmd[cmd.index("-o") + 1])
        tmp = out.with_name(f".{out.name}.{os.getpid()}.tmp")
        real = list(cmd)
        real[real.index("-o") + 1] = str(tmp)
        r = subprocess.run(real, capture_output=True, text=True)
        if r.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        os.replace(tmp, out)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(run, jobs):
                if verbose and out:
                    print(out, file=sys.stderr)
    objs = [str(BUILD / (Path(s).stem + ".o")) for s in sources]
    if jobs or not LIB.exists():
        run([nvcc, "-shared", "-o", str(LIB), *objs, "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
