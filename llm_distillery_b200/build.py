"""In-tree native build: every ``csrc/**/*.cu`` is compiled for sm_100a with nvcc and linked into
``_C/libb200_kernels.so``; every ``csrc/h5/*.cc`` is compiled with g++ (zlib) into ``_C/libb200_host.so``.

No GPU is needed to build (nvcc cross-compiles). Objects are cached under ``build/`` keyed by a hash of
the source, its local includes and the flags, so rebuilding after a one-file edit takes seconds.

    python -m llm_distillery_b200.build [--force] [--verbose] [--jobs N] [--sanitize]

``--sanitize`` additionally builds ``_C/libb200_host_asan.so`` (the host library with AddressSanitizer and UBSan) and
``_C/libb200_host_tsan.so`` (ThreadSanitizer) for
use from an instrumented host program or with ``LD_PRELOAD`` of the sanitizer runtime.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_C"
OBJ = PKG.parent / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]

KERNEL_LIB = OUT / "libb200_kernels.so"
HOST_LIB = OUT / "libb200_host.so"


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


_INC = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _closure(src: Path, seen: set[Path] | None = None) -> set[Path]:
    seen = set() if seen is None else seen
    if src in seen or not src.exists():
        return seen
    seen.add(src)
    for inc in _INC.findall(src.read_text()):
        _closure((src.parent / inc).resolve(), seen)
    return seen


def _digest(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    for f in sorted(_closure(src)):
        h.update(str(f.relative_to(PKG)).encode())
        h.update(f.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:20]


def _compile(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)


def _build_lib(sources: list[Path], flags: list[str], compiler: list[str], link: list[str], out: Path,
               force: bool, verbose: bool, jobs: int, link_tail: list[str] | None = None) -> bool:
    OBJ.mkdir(parents=True, exist_ok=True)
    OUT.mkdir(parents=True, exist_ok=True)
    objs, todo = [], []
    for s in sources:
        o = OBJ / f"{s.stem}-{_digest(s, flags)}.o"
        objs.append(o)
        if force or not o.exists():
            todo.append((s, o))
    with cf.ThreadPoolExecutor(max_workers=max(1, jobs)) as ex:
        futs = [ex.submit(_compile, compiler + flags + ["-c", str(s), "-o", str(o)], verbose) for s, o in todo]
        for f in futs:
            f.result()
    stamp = out.with_suffix(".stamp")
    want = hashlib.sha256(" ".join(sorted(o.name for o in objs)).encode()).hexdigest()
    if not force and not todo and out.exists() and stamp.exists() and stamp.read_text() == want:
        return False
    _compile(link + [str(o) for o in objs] + (link_tail or []) + ["-o", str(out)], verbose)
    stamp.write_text(want)
    return True


def cuda_sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*.cu"))


def host_sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*.cc"))


def build(force: bool = False, verbose: bool = False, jobs: int | None = None, sanitize: bool = False) -> dict:
    """Build both native libraries (no-op when up to date). Returns {"kernels": path, "host": path}."""
    jobs = jobs or (os.cpu_count() or 4)
    nvcc = _nvcc()
    cus = cuda_sources()
    if cus:
        _build_lib(cus, NVCC_FLAGS, [nvcc], [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a"],
                   KERNEL_LIB, force, verbose, jobs)
    ccs = host_sources()
    if ccs:
        _build_lib(ccs, CXX_FLAGS, ["g++"], ["g++", "-shared", "-pthread", "-Wl,--no-undefined"], HOST_LIB, force,
                   verbose, jobs, link_tail=["-lz"])
    out = {"kernels": str(KERNEL_LIB), "host": str(HOST_LIB)}
    if sanitize and ccs:
        san = ["-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-g"]
        asan_lib = OUT / "libb200_host_asan.so"
        _build_lib(ccs, CXX_FLAGS + san, ["g++"], ["g++", "-shared", "-pthread"] + san, asan_lib, force, verbose, jobs,
                   link_tail=["-lz"])
        out["host_asan"] = str(asan_lib)
        tsan = ["-fsanitize=thread", "-fno-omit-frame-pointer", "-g"]
        tsan_lib = OUT / "libb200_host_tsan.so"
        _build_lib(ccs, CXX_FLAGS + tsan, ["g++"], ["g++", "-shared", "-pthread"] + tsan, tsan_lib, force, verbose, jobs,
                   link_tail=["-lz"])
        out["host_tsan"] = str(tsan_lib)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--sanitize", action="store_true")
    a = ap.parse_args(argv)
    out = build(a.force, a.verbose, a.jobs, a.sanitize)
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
