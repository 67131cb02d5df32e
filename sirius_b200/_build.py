"""In-tree build of libsirius_b200.so (hand-written sm_100a kernels + C++ runtime).

nvcc cross-compiles for sm_100a without a GPU. Objects are cached under sirius_b200/build/ and
rebuilt when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "build"
LIB = PKG / "libsirius_b200.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cc")) + list((CSRC / "runtime").glob("*.cc")))


def _headers() -> list[Path]:
    root = PKG.parent / "include"
    return (list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((CSRC / "runtime").glob("*.h"))
            + list(root.glob("*.h")))


def _compile(src: Path, obj: Path, verbose: bool) -> None:
    cmd = [NVCC, *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = BUILD / (obj.stem + ".ptxas.log")
    log.write_text(res.stderr)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"nvcc failed on {src.name}")
    if verbose:
        for line in res.stderr.splitlines():
            if "warning" in line.lower():
                print(line)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source for sm_100a and link the shared library. Returns its path."""
    BUILD.mkdir(exist_ok=True)
    newest_hdr = max((h.stat().st_mtime for h in _headers()), default=0.0)
    jobs, objs = [], []
    for src in _sources():
        obj = BUILD / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_hdr)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _compile(j[0], j[1], verbose), jobs))
    if jobs or not LIB.exists():
        cmd = [NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-lpthread", "-lrt", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB


SANITIZERS = {
    # name: (host compiler flags, runtime libraries to link, libraries to LD_PRELOAD when the tests run under python)
    "thread": ("-fsanitize=thread", ["-ltsan"], ["libtsan.so"]),
    "address": ("-fsanitize=address,-fsanitize=undefined,-fno-omit-frame-pointer", ["-lasan", "-lubsan"],
                ["libasan.so", "libubsan.so"]),
}


def build_sanitized(kind: str = "thread") -> Path:
    """The same library with the host runtime (csrc/runtime/*.cc: shared-memory channel, ledger, control stub, page pool,
    allocator seam, server plane) compiled under ThreadSanitizer ("thread") or AddressSanitizer + UBSan ("address"); the
    kernels and executors are the normal objects. Run the CPU suite on it with

        SIRIUS_B200_LIB=<printed path> LD_PRELOAD="$(gcc -print-file-name=libtsan.so)" \
        TSAN_OPTIONS="halt_on_error=0 exitcode=0 log_path=/tmp/tsan" python -m pytest tests -q -m "not gpu"

    (address: libasan.so and libubsan.so preloaded, ASAN_OPTIONS="detect_leaks=0:halt_on_error=0:log_path=/tmp/asan")
    and read the log files; reports inside libtorch (gloo's work objects, OpenMP loops) are not this library's."""
    flags, link, _ = SANITIZERS[kind]
    build()
    out = BUILD / f"sanitize_{kind}"
    out.mkdir(exist_ok=True)
    objs = []
    for src in _sources():
        if src.parent.name != "runtime":
            objs.append(BUILD / (src.stem + ".o"))
            continue
        obj = out / (src.stem + ".o")
        objs.append(obj)
        cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O1", "-g", "--expt-relaxed-constexpr",
               "-Xcompiler", "-fPIC," + flags, "-x", "cu", "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"nvcc ({kind} sanitizer) failed on {src.name}")
    lib = out / "libsirius_b200.so"
    cmd = [NVCC, "-shared", "-o", str(lib), *map(str, objs), "-lpthread", "-lrt", "-ldl"]
    for l in link:
        cmd += ["-Xlinker", l]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"link ({kind} sanitizer) failed")
    return lib


if __name__ == "__main__":
    if "--tsan" in sys.argv:
        p = build_sanitized("thread")
    elif "--asan" in sys.argv:
        p = build_sanitized("address")
    else:
        p = build(force="--force" in sys.argv, verbose=True)
    print(p)
