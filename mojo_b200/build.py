"""In-tree build of the native library: `python -m mojo_b200.build`.

Two artefacts land inside the package directory (they travel with the source tree; nothing is installed
into site-packages and no JIT cache outside the tree is used):

* ``mojo_b200/lib/libb2kernels.so``  - every ``csrc/kernels/*.cu`` compiled by nvcc for sm_100a plus the
  host runtime under ``csrc/runtime/*.cpp``. Pure C ABI (``csrc/include/b2/api.h``), no PyTorch dependency.
* ``mojo_b200/_C.<abi>.so``          - pybind11/PyTorch bindings (``csrc/bindings/*.cpp``) linked against it.

This replaces the reference's `mojo package stdlib/src -o stdlib.mojopkg` step
(stdlib/scripts/build-stdlib.sh:17-29). Objects are rebuilt only when their source or any header is newer.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "csrc" / "build"
LIBDIR = ROOT / "lib"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _cuda_home() -> Path:
    return Path(_nvcc()).resolve().parent.parent


def _newest_header_mtime() -> float:
    newest = 0.0
    for p in (CSRC / "include").rglob("*"):
        if p.is_file():
            newest = max(newest, p.stat().st_mtime)
    return newest


def _needs(obj: Path, src: Path, hdr_mtime: float) -> bool:
    if not obj.exists():
        return True
    m = obj.stat().st_mtime
    return src.stat().st_mtime > m or hdr_mtime > m


def _run(cmd: list[str], verbose: bool) -> str:
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        sys.stderr.write(p.stdout + p.stderr)
        raise RuntimeError(f"command failed ({p.returncode}): {' '.join(str(c) for c in cmd)}")
    return p.stdout + p.stderr


def build(verbose: bool = False, assert_mode: int = 2, ptxas_info: bool = False, jobs: int | None = None) -> None:
    t0 = time.time()
    OBJ.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    hdr_m = _newest_header_mtime()
    inc = ["-I", str(CSRC / "include")]
    cuda_inc = ["-I", str(_cuda_home() / "include")]
    defs = [f"-DB2_ASSERT_MODE={assert_mode}"]

    cu_srcs = sorted((CSRC / "kernels").glob("*.cu"))
    cpp_srcs = sorted((CSRC / "runtime").glob("*.cpp"))
    tasks = []
    objs = []
    for s in cu_srcs:
        o = OBJ / (s.stem + ".cu.o")
        objs.append(o)
        if _needs(o, s, hdr_m):
            cmd = [_nvcc(), *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                   "--expt-relaxed-constexpr", *defs, *inc, "-c", str(s), "-o", str(o)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            tasks.append(cmd)
    for s in cpp_srcs:
        o = OBJ / (s.stem + ".cpp.o")
        objs.append(o)
        if _needs(o, s, hdr_m):
            tasks.append(["g++", "-O2", "-std=c++17", "-fPIC", "-Wall", *defs, *inc, *cuda_inc, "-c", str(s), "-o", str(o)])

    jobs = jobs or min(8, os.cpu_count() or 4)
    outputs = []
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        for out in ex.map(lambda c: _run(c, verbose), tasks):
            outputs.append(out)
    if ptxas_info:
        print("".join(outputs))

    lib = LIBDIR / "libb2kernels.so"
    if tasks or not lib.exists():
        _run([_nvcc(), *NVCC_ARCH, "-shared", "-o", str(lib), *[str(o) for o in objs], "-lcudart", "-ldl", "-lpthread"], verbose)

    # ---- PyTorch bindings ----
    import torch
    from torch.utils import cpp_extension as ce

    ext_suffix = sysconfig.get_config_var("EXT_SUFFIX")
    mod = ROOT / f"_C{ext_suffix}"
    b_srcs = sorted((CSRC / "bindings").glob("*.cpp"))
    b_objs = []
    b_tasks = []
    torch_inc = []
    for p in ce.include_paths():
        torch_inc += ["-isystem", p]
    py_inc = ["-isystem", sysconfig.get_paths()["include"]]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for s in b_srcs:
        o = OBJ / (s.stem + ".bind.o")
        b_objs.append(o)
        if _needs(o, s, hdr_m):
            b_tasks.append(["g++", "-O2", "-std=c++17", "-fPIC", "-Wno-unused-variable", *defs, *inc, *cuda_inc, *torch_inc, *py_inc,
                            f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                            "-c", str(s), "-o", str(o)])
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        list(ex.map(lambda c: _run(c, verbose), b_tasks))
    if b_tasks or tasks or not mod.exists():
        torch_lib = Path(torch.__file__).parent / "lib"
        _run(["g++", "-shared", "-o", str(mod), *[str(o) for o in b_objs], f"-L{LIBDIR}", "-lb2kernels",
              f"-L{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
              f"-L{_cuda_home() / 'lib64'}", "-lcudart",
              "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{_cuda_home() / 'lib64'}"], verbose)
    if verbose or tasks or b_tasks:
        print(f"[mojo_b200.build] {len(tasks)} kernel/runtime objects, {len(b_tasks)} binding objects rebuilt in {time.time() - t0:.1f}s")


def build_selftest(sanitizer: str = "address", out_dir: Path | None = None, verbose: bool = False) -> Path:
    """Compile the host runtime with its self-test driver (`csrc/tests/runtime_selftest.cpp`) into one executable
    under a host sanitizer: "address" (AddressSanitizer + UBSan), "thread" (ThreadSanitizer) or "" (none).
    The device code cannot run under a sanitizer on every machine, so the CPU-only job runs the host side that
    computes block tables, slots and schedules under one. Returns the path of the executable."""
    out_dir = Path(out_dir) if out_dir is not None else OBJ
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = out_dir / f"runtime_selftest_{sanitizer or 'plain'}"
    flags = {"address": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer"],
             "thread": ["-fsanitize=thread"], "": []}[sanitizer]
    srcs = [CSRC / "tests" / "runtime_selftest.cpp", CSRC / "runtime" / "kv_manager.cpp", CSRC / "runtime" / "scheduler.cpp",
            CSRC / "runtime" / "symm_sim.cpp", CSRC / "runtime" / "context.cpp", CSRC / "runtime" / "io.cpp"]
    _run(["g++", "-std=c++17", "-O1", "-g", *flags, f"-I{CSRC / 'include'}", *[str(x) for x in srcs], "-o", str(exe), "-pthread"], verbose)
    return exe


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--assert-mode", type=int, default=2, help="0 none, 1 warn, 2 safe, 3 all")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / smem per kernel")
    ap.add_argument("--clean", action="store_true")
    ap.add_argument("--selftest", choices=["address", "thread", "plain"], default=None,
                    help="build the host runtime self-test under this sanitizer, run it and exit with its code")
    a = ap.parse_args()
    if a.selftest is not None:
        exe = build_selftest("" if a.selftest == "plain" else a.selftest, verbose=a.verbose)
        sys.exit(subprocess.run([str(exe)]).returncode)
    if a.clean and OBJ.exists():
        shutil.rmtree(OBJ)
    build(verbose=a.verbose, assert_mode=a.assert_mode, ptxas_info=a.ptxas_info)


if __name__ == "__main__":
    main()
