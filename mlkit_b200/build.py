"""Build libmlkit_b200.so in-tree with nvcc for sm_100a.

``python -m mlkit_b200.build`` compiles every ``.cu`` file under ``mlkit_b200/csrc`` into one
shared library, ``mlkit_b200/lib/libmlkit_b200.so``, which exports the C ABI declared in
``include/mlkit_b200.h``.  The CUDA runtime is linked statically, so the library depends only on
the driver.  No GPU is needed to build.
"""

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
SOURCES = PACKAGE / "csrc"
OUTPUT = PACKAGE / "lib" / "libmlkit_b200.so"
STAMP = PACKAGE / "lib" / "build.stamp"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC"]


def nvcc_path() -> str | None:
    found = shutil.which("nvcc")
    if found:
        return found
    candidate = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    return str(candidate) if candidate.exists() else None


def source_fingerprint() -> str:
    digest = hashlib.sha256()
    files = sorted(SOURCES.glob("*.cu")) + sorted(SOURCES.glob("*.cuh"))
    files.append(PACKAGE.parent / "include" / "mlkit_b200.h")
    for path in files:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(ARCH_FLAGS + COMMON_FLAGS).encode())
    return digest.hexdigest()


def is_current() -> bool:
    return OUTPUT.exists() and STAMP.exists() and STAMP.read_text().strip() == source_fingerprint()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile when sources changed (or ``force``); returns the library path."""
    if not force and is_current():
        return OUTPUT
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libmlkit_b200.so")
    objects = PACKAGE / "lib" / "obj"
    objects.mkdir(parents=True, exist_ok=True)
    sources = sorted(SOURCES.glob("*.cu"))

    def compile_one(source: Path) -> Path:
        target = objects / (source.stem + ".o")
        command = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, "-c", str(source), "-o", str(target)]
        if verbose:
            command.insert(1, "-Xptxas=-v")
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed on {source.name}:\n{result.stdout}\n{result.stderr}")
        if verbose:
            print(result.stderr, file=sys.stderr)
        return target

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        built = list(pool.map(compile_one, sources))
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(OUTPUT), *map(str, built)]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    STAMP.write_text(source_fingerprint() + "\n")
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
