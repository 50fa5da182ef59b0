"""Builds the sm_100a kernel library from the .cu files beside this file, with nvcc alone.

The kernels have a plain C interface (``extern "C"``, raw pointers and a stream), so no
PyTorch header is compiled and a fresh build takes well under a minute.  The shared object
is written next to the sources (``csrc/_build/``) so that it travels with the source tree;
if that folder cannot be written, a per-user folder under the temporary directory is used.
A digest of the sources and flags is stored beside the library and a build is skipped when
it matches.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libgtar_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); the kernels cannot be built")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def source_digest() -> str:
    digest = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return digest.hexdigest()


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    in_tree = CSRC / "_build"
    if _writable(in_tree):
        return in_tree
    fallback = Path(tempfile.gettempdir()) / f"gtar_b200_build_{os.getuid()}"
    if _writable(fallback):
        return fallback
    raise BuildError(f"neither {in_tree} nor {fallback} can be written; nowhere to build the kernels")


def library_path(build: bool = True, verbose: bool = True) -> Path:
    """Path of an up-to-date library; compiles it first if need be."""
    digest = source_digest()
    candidates = [CSRC / "_build", Path(tempfile.gettempdir()) / f"gtar_b200_build_{os.getuid()}"]
    for folder in candidates:
        lib, stamp = folder / LIB_NAME, folder / "digest.txt"
        try:
            if lib.exists() and stamp.exists() and stamp.read_text().strip() == digest:
                return lib
        except OSError:
            continue
    if not build:
        raise BuildError("the kernel library is not built (or is older than its sources)")
    return compile_library(verbose=verbose)


def _say(verbose: bool, text: str) -> None:
    if verbose:
        print(f"[gtar_kimik3_public_b200] {text}", file=sys.stderr, flush=True)


def compile_library(verbose: bool = True, extra_flags: list[str] | None = None) -> Path:
    nvcc = find_nvcc()
    out = build_dir()
    digest = source_digest()
    files = sources()
    flags = ARCH_FLAGS + NVCC_FLAGS + (extra_flags or [])
    started = time.time()
    _say(verbose, f"compiling {len(files)} CUDA files for sm_100a into {out} (first use; takes about a minute)")

    def compile_one(src: Path) -> tuple[Path, Path]:
        obj = out / (src.stem + ".o")
        cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
        return src, obj

    objects: list[Path] = []
    workers = max(1, min(len(files), os.cpu_count() or 2))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        futures = [pool.submit(compile_one, src) for src in files]
        for done, future in enumerate(as_completed(futures), 1):
            src, obj = future.result()
            objects.append(obj)
            _say(verbose, f"  [{done}/{len(files)}] {src.name} done after {time.time() - started:.0f} s")
    tmp_lib = out / (LIB_NAME + f".tmp{os.getpid()}")
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *[str(o) for o in sorted(objects)]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, out / LIB_NAME)
    (out / "digest.txt").write_text(digest + "\n")
    _say(verbose, f"built {out / LIB_NAME} in {time.time() - started:.0f} s")
    return out / LIB_NAME


if __name__ == "__main__":
    print(library_path())
