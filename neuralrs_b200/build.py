"""Builds libnrs_b200.so in-tree with nvcc for sm_100a (and nothing else).

Usage: python -m neuralrs_b200.build [--force] [--verbose]

Every .cu under csrc/ is compiled to an object in build/ (in parallel, skipped
when the object is newer than the source and every header) and linked into
neuralrs_b200/libnrs_b200.so.  nvcc cross-compiles without a GPU present.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = ROOT / "build" / "nrs_b200"
LIB = PKG / "libnrs_b200.so"

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unknown-pragmas",
    "--expt-relaxed-constexpr",
    "-I", str(ROOT / "include"), "-I", str(CSRC),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _sources() -> list[Path]:
    return sorted(CSRC.rglob("*.cu")) + sorted(CSRC.rglob("*.cpp"))


def _headers_mtime() -> float:
    hs = list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, obj: Path, verbose: bool) -> str:
    cmd = [_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    env = dict(os.environ)
    env.pop("CC", None)   # the image exports a CC wrapper that nvcc must not pick up
    env.pop("CXX", None)
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    hdr_t = _headers_mtime()
    srcs = _sources()
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / (s.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        objs.append(o)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_t):
            jobs.append((s, o))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = {ex.submit(_compile, s, o, verbose): s for s, o in jobs}
            for f in cf.as_completed(futs):
                log = f.result()
                if verbose and log:
                    print(f"--- {futs[f].name}\n{log}", file=sys.stderr)
    if jobs or not LIB.exists():
        env = dict(os.environ)
        env.pop("CC", None)
        env.pop("CXX", None)
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
