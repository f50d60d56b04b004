"""Build recipe for the native libraries (nvcc for sm_100a, in-tree outputs).

`python -m autorust_b200.build` compiles

  autorust_b200/lib/libar_attn.so    the CUDA kernels + the C ABI of include/ar_attn.h
  autorust_b200/lib/libar_host.so    the C++ host layer that mirrors autorust's Tensor / Session /
                                     Settings / fused_attention_ex surface on top of that ABI
  autorust_b200/lib/libar_gather.so  the output gather for N > 1 (kept apart so that single-GPU users
                                     need no NCCL at load time)
  autorust_b200/lib/waittest/libar_attn.so
                                     the same kernels with a wait budget of about a millisecond and a hook
                                     that leaves one K tile unrequested: what tests/test_gpu_wait_expiry.py
                                     loads to see a bounded wait run out and the kernel leave in order

nvcc cross-compiles without a GPU; nothing here needs one.  Objects are rebuilt only when a
source or header is newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]

KERNEL_SOURCES = ["attn_fwd_tc.cu", "attn_fwd_exact.cu", "attn_train.cu", "attn_train_tc.cu", "sage_prologue.cu", "api.cu",
                  "sage_static.cu", "encoder_norm.cu"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return nvcc


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted((ROOT / "include").glob("*.h")) + \
        sorted((CSRC / "host").glob("*.h"))


def build_kernels(force: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    out = LIB / "libar_attn.so"
    srcs = [CSRC / s for s in KERNEL_SOURCES]
    if not force and not _newer(out, srcs + _headers()):
        return out
    objs = []
    for s in srcs:
        o = LIB / (s.stem + ".o")
        if force or _newer(o, [s] + _headers()):
            _run([_nvcc(), *NVCC_FLAGS, "-c", str(s), "-o", str(o)])
        objs.append(str(o))
    _run([_nvcc(), "-shared", "-o", str(out), *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    return out


# Sources whose device code contains bounded waits: rebuilt with the short budget for the wait-expiry test library.
WAIT_SOURCES = ["attn_fwd_tc.cu", "attn_train_tc.cu", "sage_prologue.cu"]
WAIT_TEST_FLAGS = ["-DAR_WAIT_TEST", "-DAR_WAIT_BUDGET_CYCLES=2000000ll"]


def build_wait_test(force: bool = False) -> Path:
    """The test-only variant of libar_attn.so (never loaded by the package itself)."""
    build_kernels(force)
    out_dir = LIB / "waittest"
    out_dir.mkdir(exist_ok=True)
    out = out_dir / "libar_attn.so"
    srcs = [CSRC / s for s in KERNEL_SOURCES]
    if not force and not _newer(out, srcs + _headers()):
        return out
    objs = []
    for s in srcs:
        if s.name in WAIT_SOURCES:
            o = out_dir / (s.stem + ".o")
            _run([_nvcc(), *NVCC_FLAGS, *WAIT_TEST_FLAGS, "-c", str(s), "-o", str(o)])
        else:
            o = LIB / (s.stem + ".o")
        objs.append(str(o))
    _run([_nvcc(), "-shared", "-o", str(out), *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    return out


def build_host(force: bool = False) -> Path | None:
    host_dir = CSRC / "host"
    srcs = sorted(host_dir.glob("*.cpp"))
    if not srcs:
        return None
    out = LIB / "libar_host.so"
    if not force and not _newer(out, srcs + _headers()):
        return out
    cuda_inc = str(Path(_nvcc()).resolve().parent.parent / "include")
    cuda_lib = str(Path(_nvcc()).resolve().parent.parent / "lib64")
    _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-I", str(ROOT / "include"), "-I", cuda_inc,
          *map(str, srcs), "-o", str(out), "-L", str(LIB), "-lar_attn", "-L", cuda_lib, "-lcudart_static",
          "-ldl", "-lrt", "-lpthread", "-Wl,-rpath,$ORIGIN"])
    return out


def _nccl_paths() -> tuple[str, str] | None:
    try:
        import nvidia.nccl as nccl_pkg  # type: ignore
        base = Path(list(nccl_pkg.__path__)[0])
    except Exception:
        return None
    inc, lib = base / "include", base / "lib"
    if (inc / "nccl.h").exists() and any(lib.glob("libnccl.so*")):
        return str(inc), str(lib)
    return None


def build_gather(force: bool = False) -> Path | None:
    src = CSRC / "allgather.cpp"
    if not src.exists():
        return None
    paths = _nccl_paths()
    if paths is None:
        return None
    inc, lib = paths
    out = LIB / "libar_gather.so"
    if not force and not _newer(out, [src] + _headers()):
        return out
    cuda_inc = str(Path(_nvcc()).resolve().parent.parent / "include")
    nccl_so = sorted(Path(lib).glob("libnccl.so*"))[0]
    _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-I", str(ROOT / "include"), "-I", cuda_inc, "-I", inc,
          str(src), "-o", str(out), str(nccl_so), "-Wl,-rpath," + lib])
    return out


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_host(force)
    build_gather(force)
    build_wait_test(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", ", ".join(p.name for p in sorted(LIB.glob("*.so"))))
