"""Build the native library (``_lib/libstreamattn_b200.so``) with nvcc for sm_100a.

The library is built in-tree so that it travels with the source tree; nothing
is installed into site-packages and there is no JIT cache.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import threading
from pathlib import Path
from typing import List, Optional

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC_DIR = PACKAGE_DIR / "csrc"
LIB_DIR = PACKAGE_DIR / "_lib"
LIB_PATH = LIB_DIR / "libstreamattn_b200.so"
SOURCES = ("sa_api.cu", "sa_generic.cu", "sa_stream.cu", "sa_exchange.cu", "sa_append.cu", "sa_oproj.cu", "sa_select.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-shared",
)
_LOCK = threading.Lock()


def find_nvcc() -> Optional[str]:
    for candidate in (os.environ.get("STREAMATTN_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    return None


def source_files() -> List[Path]:
    return [CSRC_DIR / name for name in SOURCES if (CSRC_DIR / name).is_file()]


def is_stale() -> bool:
    if not LIB_PATH.is_file():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC_DIR.glob("*.cu")) + list(CSRC_DIR.glob("*.cuh"))
    deps.append(PACKAGE_DIR.parent / "include" / "streamattn_b200.h")
    return any(p.is_file() and p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source into one shared library; returns its path."""

    with _LOCK:
        if not force and not is_stale():
            return LIB_PATH
        nvcc = find_nvcc()
        if nvcc is None:
            raise RuntimeError(
                "nvcc was not found: streamattn_b200 needs its native sm_100a library "
                f"({LIB_PATH}) and has no CPU or interpreted fallback"
            )
        LIB_DIR.mkdir(parents=True, exist_ok=True)
        # One temporary per process: several ranks may find the library stale at the same time.
        tmp = LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")
        cmd = [nvcc, *NVCC_FLAGS, "-o", str(tmp), *[str(p) for p in source_files()]]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
        if verbose:
            print(proc.stdout + proc.stderr)
        os.replace(tmp, LIB_PATH)
        return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
