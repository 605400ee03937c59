"""In-tree build of the native code for sm_100a.

Two shared objects are produced next to the sources (they are git-ignored but travel with the
working tree):

* ``lib/libumdk_cam.so``  -- every CUDA kernel plus the C host runtime, compiled with plain
  ``nvcc -gencode arch=compute_100a,code=sm_100a``; no PyTorch headers, exported C ABI.
* ``_C*.so``              -- the PyTorch binding layer (``TORCH_LIBRARY`` registrations and the
  ``Buffer`` class), linked against the library above.

The role matches the reference's build glue (build/cam/comm_operator/build.sh:48-107 builds the
kernel package, pybind/setup.py:55-106 builds the extension wheel).  Usage::

    python -m umdk_original_b200._build [--force] [--debug] [--no-bindings]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "lib"

GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]

KERNEL_SOURCES = [
    "kernels/dispatch_normal.cu",
    "kernels/combine.cu",
    "kernels/dispatch_ll.cu",
    "kernels/grouped_gemm.cu",
    "kernels/grouped_gemm_mx.cu",
    "kernels/grouped_gemm_mx2.cu",
    "kernels/grouped_gemm_i8.cu",
    "kernels/fused_moe_mx.cu",
    "kernels/dispatch_noalloc.cu",
    "kernels/sync_p2p.cu",
    "kernels/tp_exchange.cu",
    "runtime/cam_runtime.cpp",
]


def _nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").exists():
            return str(Path(cand) / "bin" / "nvcc")
    return "nvcc"


def _run(cmd: list[str]) -> str:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout)
    if os.environ.get("UMDK_BUILD_VERBOSE"):
        sys.stdout.write(proc.stdout)
    return proc.stdout


def _check_gemm_registers(ptxas_log: str, src: Path) -> None:
    """The grouped GEMM re-partitions registers with setmaxnreg against the per-thread count the
    CTA is launched with; that count must be the kLaunchRegs constant of the source, or the
    kernel would wait for registers that never come."""
    import re
    want = int(re.search(r"k(?:Mx|P2|I8|Fm)?LaunchRegs\s*=\s*(\d+)", src.read_text()).group(1))
    # only the GEMM kernels re-partition registers; a file may hold other kernels as well
    got = [int(n) for name, n in re.findall(r"Compiling entry function '([^']+)'.*?Used (\d+) registers", ptxas_log, re.S)
           if "grouped_gemm" in name or "fused_moe" in name]
    if not got or any(g != want for g in got):
        raise RuntimeError(f"{src.name}: ptxas reports {got} registers but kLaunchRegs is {want}")


def _deps_digest(extra: str = "") -> str:
    """Hash of every header under csrc: a header change rebuilds everything."""
    h = hashlib.sha1(extra.encode())
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".cuh", ".hpp"):
            h.update(p.read_bytes())
    return h.hexdigest()


def _stale(src: Path, out: Path, stamp: str) -> bool:
    tag = out.with_suffix(out.suffix + ".stamp")
    want = hashlib.sha1(src.read_bytes() + stamp.encode()).hexdigest()
    if out.exists() and tag.exists() and tag.read_text() == want:
        return False
    return True


def _mark(src: Path, out: Path, stamp: str) -> None:
    tag = out.with_suffix(out.suffix + ".stamp")
    tag.write_text(hashlib.sha1(src.read_bytes() + stamp.encode()).hexdigest())


def build_kernels(force: bool = False, debug: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    nvcc = _nvcc()
    flags = ["-std=c++17", "-Xcompiler", "-fPIC", "-lineinfo", "-Xptxas", "-v"] + GENCODE
    # debug: host code without optimisation and with symbols; device code stays at -O3 (the GEMM kernels re-partition
    # registers against the count ptxas reports at -O3).  The device-side range checks are always compiled in.
    flags += ["-O3", "-g", "-Xcompiler", "-O0"] if debug else ["-O3"]
    stamp = _deps_digest(" ".join(flags))
    objs: list[Path] = []
    jobs = []
    for rel in KERNEL_SOURCES:
        src = CSRC / rel
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(src, obj, stamp):
            cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
            if src.suffix == ".cpp":
                cmd = [nvcc, *flags, "-x", "cu", "-c", str(src), "-o", str(obj)]
            jobs.append((cmd, src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(lambda j: _run(j[0]), jobs))
        for (_, src, obj), log in zip(jobs, logs):
            if src.name in ("grouped_gemm.cu", "grouped_gemm_mx.cu", "grouped_gemm_mx2.cu", "grouped_gemm_i8.cu",
                            "fused_moe_mx.cu"):
                _check_gemm_registers(log, src)
            _mark(src, obj, stamp)
    so = LIB / "libumdk_cam.so"
    if jobs or force or not so.exists():
        _run([nvcc, "-shared", "-o", str(so), *map(str, objs), *GENCODE, "-Xcompiler", "-fPIC", "-cudart", "static"])
    return so


def build_bindings(force: bool = False, debug: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(exist_ok=True)
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    out = PKG / ("_C" + suffix)
    src = CSRC / "bindings.cpp"
    obj = OBJ / "bindings.o"
    cuda_inc = str(Path(_nvcc()).resolve().parent.parent / "include")
    incs = [*ce.include_paths(), sysconfig.get_paths()["include"], cuda_inc]
    cxx = os.environ.get("CXX", "g++")
    cflags = ["-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-Wno-deprecated-declarations"]
    cflags += ["-O0", "-g"] if debug else ["-O2"]
    stamp = _deps_digest(" ".join(cflags) + torch.__version__)
    if force or _stale(src, obj, stamp):
        _run([cxx, *cflags, *[f"-I{i}" for i in incs], "-c", str(src), "-o", str(obj)])
        _mark(src, obj, stamp)
        force = True
    if force or not out.exists():
        torch_lib = str(Path(torch.__file__).resolve().parent / "lib")
        _run([cxx, "-shared", "-o", str(out), str(obj), f"-L{LIB}", "-lumdk_cam", f"-L{torch_lib}", "-lc10", "-ltorch",
              "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-Wl,-rpath,$ORIGIN/lib",
              f"-Wl,-rpath,{torch_lib}"])
    return out


def build_all(force: bool = False, debug: bool = False, bindings: bool = True) -> None:
    build_kernels(force=force, debug=debug)
    if bindings:
        build_bindings(force=force, debug=debug)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--force", action="store_true", help="rebuild everything")
    ap.add_argument("--debug", action="store_true", help="host code with -O0 -g (device code stays optimised)")
    ap.add_argument("--no-bindings", action="store_true", help="build only libumdk_cam.so")
    a = ap.parse_args()
    build_all(force=a.force, debug=a.debug, bindings=not a.no_bindings)
    print("built", LIB / "libumdk_cam.so")


if __name__ == "__main__":
    main()
