"""Builds the reference's OWN fused attention kernels for the GPU box, as a second oracle.

autorust carries its CUDA kernels as string constants inside Rust files
(src/runtime/cuda_flash.rs:48-142, cuda_flash_tc.rs:92-376, cuda_flash_bf16.rs:98-428,
cuda_flash_sage.rs:86-415) and NVRTC-compiles them at run time for `sm_<major><minor>`
(src/runtime/ops_cuda.rs:151-152).  This script reads those strings from the mounted reference tree,
writes each one -- unchanged, with the one-line `#define` prefix the Rust host would prepend
(cuda_flash_bf16.rs:94-96, cuda_flash_sage.rs:82-84) and a small launcher of ours appended -- into
oracle/_ref/, and compiles them with nvcc for sm_100 into oracle/_ref/libar_ref_kernels.so.

Nothing of the reference's text is committed: oracle/_ref/ is git-ignored.  The library travels to the
GPU box with the repository snapshot, where tests/test_gpu_reference_kernels.py uses it (D = 64 only,
the reference's only head size) to pin the oracle's rounding models and to compare our kernels with the
reference's on the same inputs.  TEST INFRASTRUCTURE ONLY.

Usage: python oracle/build_ref.py [path/to/autorust]
(default: $AUTORUST_REFERENCE_DIR, else the directory `reference` beside this repository)
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

# (rust file, kernel symbol, define prefix, element type of Q/K/V/O, threads per block)
KERNELS = [
    ("cuda_flash.rs", "ar_flash_f32", "", "float", 64),
    ("cuda_flash_tc.rs", "ar_flash_tc_f32", "#define AR_ASYNC 0\n", "float", 128),
    ("cuda_flash_bf16.rs", "ar_flash_bf16", "#define AR_ASYNC 1\n", "unsigned short", 128),
    ("cuda_flash_sage.rs", "ar_flash_sage", "#define AR_FP8 0\n", "float", 128),
]

LAUNCHER = r'''
// ---- launcher appended by oracle/build_ref.py (not part of the reference) ----
// Same geometry and argument order as the Rust host_call: grid (ceil(N/64), B*H, 1), `threads` per
// block, args Q,K,V,O,M,N,head_dim,causal,has_mask,hq,hkv; M aliases O when there is no mask.
#include <cuda_runtime.h>
extern "C" int ref_launch_{name}(const void* q, const void* k, const void* v, void* o, const float* mask, int b, int hq,
                               int hkv, int n, int causal, void* stream) {
  dim3 grid((n + 63) / 64, b * hq, 1);
  {name}<<<grid, {threads}, 0, (cudaStream_t)stream>>>((const {elem}*)q, (const {elem}*)k, (const {elem}*)v, ({elem}*)o,
                                                   mask ? mask : (const float*)o, n, 64, causal, mask ? 1 : 0, hq, hkv);
  return (int)cudaGetLastError();
}
'''


def extract(rust_text: str) -> str:
    m = re.search(r'=\s*r#"(.*?)"#;', rust_text, flags=re.S)
    if not m:
        raise RuntimeError("no raw string constant found")
    return m.group(1)


def main() -> int:
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AUTORUST_REFERENCE_DIR") or HERE.parent.parent / "reference")
    src_dir = ref / "src" / "runtime"
    if not src_dir.is_dir():
        print(f"reference tree not found at {ref}: nothing built")
        return 0
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    OUT.mkdir(exist_ok=True)
    lib = OUT / "libar_ref_kernels.so"
    rust_files = [src_dir / k[0] for k in KERNELS]
    if lib.exists() and all(lib.stat().st_mtime > f.stat().st_mtime for f in rust_files + [Path(__file__)]):
        return 0
    objs = []
    for rust, name, prefix, elem, threads in KERNELS:
        body = extract((src_dir / rust).read_text())
        cu = OUT / f"{name}.cu"
        cu.write_text(prefix + body + LAUNCHER.replace("{name}", name).replace("{elem}", elem).replace("{threads}", str(threads)))
        obj = OUT / f"{name}.o"
        subprocess.run([nvcc, "-gencode", "arch=compute_100,code=sm_100", "-O3", "-Wno-deprecated-gpu-targets", "-Xcompiler", "-fPIC", "-c", str(cu), "-o",
                        str(obj)], check=True)
        objs.append(str(obj))
    subprocess.run([nvcc, "-shared", "-o", str(lib), *objs], check=True)
    for f in list(OUT.glob("*.cu")) + list(OUT.glob("*.o")):  # keep only the library
        f.unlink()
    print(f"built {lib}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
