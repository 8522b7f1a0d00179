"""Compiles the CUDA sources under ``csrc/`` into one shared library for sm_100a.

The reference compiles its C kernels at first use with gcc and loads them with
ctypes (app/native/library.py:58-103, app/native/compiler_flags.py:17-62). The
same here with nvcc: each ``.cu`` becomes an object file, the objects are linked
into ``_lib/libmatricxon_b200.so`` inside the package, and a stamp of the source
hashes decides whether a rebuild is needed. If the package folder cannot be
written, the library goes to a per-user folder under the system temp directory.
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

PACKAGE_DIR = Path(__file__).resolve().parent.parent
CSRC_DIR = PACKAGE_DIR / "csrc"
LIB_NAME = "libmatricxon_b200.so"
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--compiler-options", "-fPIC",
              "-Xcudafe", "--diag_suppress=177"]
# more flags for this process's build (they are part of the stamp: a different library)
NVCC_FLAGS += os.environ.get("MATRICXON_NVCC_EXTRA", "").split()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    candidates = [os.environ.get("MATRICXON_NVCC"), shutil.which("nvcc"),
                  "/usr/local/cuda/bin/nvcc"]
    for cuda_home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH")):
        if cuda_home:
            candidates.append(os.path.join(cuda_home, "bin", "nvcc"))
    for candidate in candidates:
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise BuildError("nvcc was not found (looked at MATRICXON_NVCC, PATH, CUDA_HOME, "
                     "/usr/local/cuda/bin); the CUDA kernels cannot be compiled")


def sources() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(CSRC_DIR.glob("*.cuh")) + list(CSRC_DIR.glob("*.h")))


def source_stamp() -> str:
    digest = hashlib.sha256()
    for path in sources() + _headers():
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_ARCH + NVCC_FLAGS).encode())
    return digest.hexdigest()


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe-{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def library_dir() -> Path:
    override = os.environ.get("MATRICXON_LIB_DIR")
    if override:
        return Path(override)
    in_tree = PACKAGE_DIR / "_lib"
    if _writable(in_tree):
        return in_tree
    return Path(tempfile.gettempdir()) / f"matricxon_b200-{os.getuid()}"


def _say(message: str) -> None:
    print(f"[matricxon_b200 build] {message}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> None:
    cmd = [nvcc, *NVCC_ARCH, *NVCC_FLAGS, "-I", str(CSRC_DIR), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    started = time.monotonic()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    _say(f"compiled {src.name} in {time.monotonic() - started:.1f}s")
    if verbose and proc.stderr:
        print(proc.stderr, file=sys.stderr)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Returns the path of an up-to-date library, compiling what is needed first."""
    out_dir = library_dir()
    if not _writable(out_dir):
        raise BuildError(f"cannot write the kernel library to {out_dir}")
    lib_path = out_dir / LIB_NAME
    stamp_path = out_dir / "build.stamp"
    stamp = source_stamp()
    if not force and lib_path.is_file() and stamp_path.is_file() \
            and stamp_path.read_text().strip() == stamp:
        return lib_path
    nvcc = find_nvcc()
    srcs = sources()
    if not srcs:
        raise BuildError(f"no CUDA sources under {CSRC_DIR}")
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a with {nvcc} (first call only)")
    obj_dir = out_dir / "_build"
    obj_dir.mkdir(parents=True, exist_ok=True)
    objects = [obj_dir / (src.stem + ".o") for src in srcs]
    workers = max(1, min(len(srcs), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        futures = [pool.submit(_compile_one, nvcc, s, o, verbose) for s, o in zip(srcs, objects)]
        for future in futures:
            future.result()
    tmp_lib = out_dir / f".{LIB_NAME}.{os.getpid()}"
    link = [nvcc, *NVCC_ARCH, "-shared", "-o", str(tmp_lib), *map(str, objects)]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, lib_path)
    stamp_path.write_text(stamp)
    _say(f"linked {lib_path}")
    return lib_path


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
