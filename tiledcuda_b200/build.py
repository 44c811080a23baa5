"""Builds the in-tree native libraries with nvcc for sm_100a.

    python -m tiledcuda_b200.build            # libtiledcuda_b200.so (C ABI, no torch dependency)
    python -m tiledcuda_b200.build --torch    # also libtiledcuda.so (torch.ops.tiledcuda.* registrations)

Objects land in tiledcuda_b200/build/, the shared libraries beside this file. A source is recompiled
only when it, or a header it can include, is newer than its object.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libtiledcuda_b200.so"
TORCH_LIB = PKG / "libtiledcuda.so"

KERNEL_SOURCES = ["host.cu", "scatter_nd.cu", "gemm.cu", "gemm_pair.cu", "gemm_host.cu", "chain.cu", "attn.cu", "lstm.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the sm_100a kernels cannot be built")
    return nvcc


def _headers_mtime() -> float:
    hdrs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((PKG.parent / "include").glob("*.h"))
    hdrs += list((PKG / "include").rglob("*.hpp"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _compile(src: Path, extra: list[str], force: bool, log_dir: Path) -> Path:
    obj = OBJ / (src.stem + ".o")
    newest = max(src.stat().st_mtime, _headers_mtime())
    if not force and obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (log_dir / (src.stem + ".ptxas.log")).write_text(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stderr[-6000:]}")
    return obj


def build_core(force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    srcs = [CSRC / s for s in KERNEL_SOURCES if (CSRC / s).exists()]
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, [], force, OBJ), srcs))
    if force or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
    return LIB


def build_torch(force: bool = False) -> Path:
    """libtiledcuda.so: TORCH_LIBRARY(tiledcuda, ...) over the C ABI; links libtiledcuda_b200.so."""
    import torch
    from torch.utils import cpp_extension

    build_core(force)
    src = CSRC / "torch_bind.cc"
    newest = max(src.stat().st_mtime, _headers_mtime(), LIB.stat().st_mtime)
    if not force and TORCH_LIB.exists() and TORCH_LIB.stat().st_mtime >= newest:
        return TORCH_LIB
    inc = []
    for p in cpp_extension.include_paths():
        inc += ["-I", p]
    torch_lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [
        "g++", "-O2", "-std=c++17", "-fPIC", "-shared", *inc,
        "-I", "/usr/local/cuda/include",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        str(src), "-o", str(TORCH_LIB),
        f"-L{PKG}", "-ltiledcuda_b200", "-Wl,-rpath,$ORIGIN",
        f"-L{torch_lib_dir}", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda",
        f"-Wl,-rpath,{torch_lib_dir}",
    ]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"torch binding build failed:\n{res.stderr[-6000:]}")
    return TORCH_LIB


TILE_INCLUDE = PKG / "include"
TESTS_CPP = PKG.parent / "tests" / "cpp"


def build_tile_api_tests(force: bool = False) -> list[Path]:
    """The libraries the tile-API tests call: device kernels written against tiledcuda_b200/include
    (nvcc, sm_100a) and the host-side layout checks (g++). Test infrastructure, built in tests/cpp/."""
    outs = []
    newest_hdr = _headers_mtime()
    dev_src, dev_lib = TESTS_CPP / "tile_api_kernels.cu", TESTS_CPP / "libtile_api_tests.so"
    if dev_src.exists() and (force or not dev_lib.exists() or dev_lib.stat().st_mtime < max(dev_src.stat().st_mtime, newest_hdr)):
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17",
               "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared", f"-I{TILE_INCLUDE}", str(dev_src), "-o", str(dev_lib)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"tile API test kernels failed to build:\n{res.stderr[-6000:]}")
    if dev_lib.exists():
        outs.append(dev_lib)
    host_src, host_lib = TESTS_CPP / "host_layout_checks.cc", TESTS_CPP / "libhost_layout_checks.so"
    if host_src.exists() and (force or not host_lib.exists() or host_lib.stat().st_mtime < max(host_src.stat().st_mtime, newest_hdr)):
        cmd = ["g++", "-O1", "-std=c++17", "-fPIC", "-shared", f"-I{TILE_INCLUDE}", str(host_src), "-o", str(host_lib)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"host layout checks failed to build:\n{res.stderr[-6000:]}")
    if host_lib.exists():
        outs.append(host_lib)
    return outs


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--torch", action="store_true", help="also build the torch op registrations")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--tests", action="store_true", help="also build the tile-API test libraries under tests/cpp")
    args = ap.parse_args()
    print(build_core(args.force))
    if args.torch:
        print(build_torch(args.force))
    if args.tests:
        for lib in build_tile_api_tests(args.force):
            print(lib)
    return 0


if __name__ == "__main__":
    sys.exit(main())
