"""Compiles the kernel library for sm_100a with nvcc, in-tree, when its sources have changed.

The library is a plain shared object with a C ABI (``csrc/roost_kernels.h``); nothing links against torch, so a
file compiles in seconds. Objects and the library go to ``roost_b200/csrc/_build`` (or, when that folder
cannot be written, to a per-user folder under the system's temporary directory). A stamp of the sources'
hash decides whether anything is rebuilt. While compiling, a line is printed for every file so that a first
call does not look hung.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libroost_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xcudafe",
              "--diag_suppress=177"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[roost_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("ROOST_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $ROOST_NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                     "the kernel library cannot be built and there is no fallback path")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")))


def _digest(extra: str = "") -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    h.update(extra.encode())
    return h.hexdigest()


def _build_dir() -> Path:
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"roost_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _run(cmd: list[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise BuildError(f"{what} failed ({' '.join(cmd)}):\n{r.stdout}\n{r.stderr}")


def library_path(verbose_ptxas: bool = False) -> Path:
    """Path of an up-to-date library, building it first when needed."""
    given = os.environ.get("ROOST_KERNELS")  # a folder that already holds the library (the command line's --kernels)
    if given:
        lib = Path(given) / LIB_NAME
        if not lib.exists():
            raise BuildError(f"{lib}: no kernel library in the folder $ROOST_KERNELS names")
        return lib
    out_dir = _build_dir()
    lib = out_dir / LIB_NAME
    stamp = out_dir / "stamp"
    digest = _digest()
    if lib.exists() and stamp.exists() and stamp.read_text().strip() == digest and not verbose_ptxas:
        return lib
    nvcc = find_nvcc()
    srcs = sources()
    _say(f"building the sm_100a kernel library ({len(srcs)} files) in {out_dir}")
    t0 = time.time()

    def compile_one(src: Path) -> Path:
        obj = out_dir / (src.stem + ".o")
        objstamp = out_dir / (src.stem + ".stamp")
        h = hashlib.sha256(src.read_bytes())
        for f in _headers():
            h.update(f.read_bytes())
        h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
        d = h.hexdigest()
        if obj.exists() and objstamp.exists() and objstamp.read_text() == d and not verbose_ptxas:
            return obj
        _say(f"  nvcc {src.name}")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose_ptxas:
            cmd += ["-Xptxas", "-v"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise BuildError(f"nvcc {src.name} failed:\n{r.stdout}\n{r.stderr}")
            print(r.stderr)
        else:
            _run(cmd, f"nvcc {src.name}")
        objstamp.write_text(d)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = out_dir / (LIB_NAME + f".{os.getpid()}.tmp")
    _run([nvcc, "-shared", *ARCH_FLAGS, "-o", str(tmp), *map(str, objs), "-lcuda"], "link")
    os.replace(tmp, lib)
    stamp.write_text(digest)
    _say(f"kernel library built in {time.time() - t0:.1f} s")
    return lib


if __name__ == "__main__":
    print(library_path(verbose_ptxas="-v" in sys.argv))
