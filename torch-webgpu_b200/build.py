"""Build the native parts of the package in-tree.

  libtwg.so   csrc/kernels/*.cu  -> torch_webgpu/lib/libtwg.so   (nvcc, sm_100a only; the C ABI)
  _C.so       csrc/host/*.cpp    -> torch_webgpu/_C.so           (g++ against libtorch; the
                                                                   PrivateUse1 registrations)

Run as `python build.py [kernels|host|all] [--force] [--verbose]`.  Nothing is installed; the
shared objects stay next to the sources so that a checkout is directly importable.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shlex
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REPO = ROOT.parent
KERNELS = ROOT / "csrc" / "kernels"
HOST = ROOT / "csrc" / "host"
PKG = ROOT / "torch_webgpu"
BUILD = ROOT / "build"
INCLUDE = REPO / "include"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# The system compiler, not $CXX: a wrapper compiler exported by the environment produced an
# extension whose C++ exceptions could not be caught (every TORCH_CHECK became a crash).
CXX = os.environ.get("TWG_CXX", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print("+", " ".join(shlex.quote(c) for c in cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        sys.stderr.write(proc.stderr)
        raise RuntimeError(f"command failed ({proc.returncode}): {' '.join(cmd[:4])} ...")
    if verbose and (proc.stdout or proc.stderr):
        sys.stderr.write(proc.stdout + proc.stderr)


def digest(paths: list[Path], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def up_to_date(target: Path, stamp: Path, key: str) -> bool:
    return target.exists() and stamp.exists() and stamp.read_text() == key


def embed_header(verbose: bool) -> Path:
    """Turn the device headers into raw string literals that fused.cu hands to NVRTC."""
    out_dir = BUILD / "gen"
    out_dir.mkdir(parents=True, exist_ok=True)
    for header in ("twg_pointwise", "twg_compact"):
        text = (KERNELS / f"{header}.cuh").read_text()
        assert ')TWGSRC"' not in text
        out = out_dir / f"{header}_src.inc"
        new = 'R"TWGSRC(' + text + ')TWGSRC"\n'
        if not out.exists() or out.read_text() != new:
            out.write_text(new)
    return out_dir


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    target = PKG / "lib" / "libtwg.so"
    target.parent.mkdir(parents=True, exist_ok=True)
    sources = sorted(KERNELS.glob("*.cu"))
    headers = sorted(KERNELS.glob("*.cuh")) + sorted(KERNELS.glob("*.h")) + [INCLUDE / "twg.h"]
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    key = digest(sources + headers, " ".join(flags))
    stamp = BUILD / "libtwg.stamp"
    if not force and not ptxas_info and up_to_date(target, stamp, key):
        return target
    gen = embed_header(verbose)
    obj_dir = BUILD / "obj"
    obj_dir.mkdir(parents=True, exist_ok=True)
    inc = ["-I", str(INCLUDE), "-I", str(KERNELS), "-I", str(gen)]

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        run([NVCC, *flags, *inc, "-c", str(src), "-o", str(obj)], verbose or ptxas_info)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    run([NVCC, "-shared", "-cudart", "static", "-Xcompiler", "-fPIC", "-o", str(target), *map(str, objs), "-ldl"],
        verbose)
    stamp.write_text(key)
    return target


def torch_paths() -> tuple[list[str], list[str]]:
    import torch  # noqa: F401  (only to locate the installation)
    from torch.utils import cpp_extension

    inc = cpp_extension.include_paths()
    lib = cpp_extension.library_paths()
    return inc, lib


def build_host(force: bool = False, verbose: bool = False) -> Path:
    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    target = PKG / ("_C" + ext)
    sources = sorted(HOST.glob("*.cpp"))
    headers = sorted(HOST.glob("*.h")) + [INCLUDE / "twg.h"]
    inc, lib = torch_paths()
    import torch
    cxx11_abi = int(bool(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True)))   # must match the installed libtorch
    flags = ["-O2", "-g1", "-std=c++17", "-fPIC", "-fvisibility=hidden", f"-D_GLIBCXX_USE_CXX11_ABI={cxx11_abi}",
             "-DTORCH_EXTENSION_NAME=_C", "-Wall", "-Wno-unused-function", "-Wno-sign-compare"]
    key = digest(sources + headers, " ".join(flags))
    stamp = BUILD / "host.stamp"
    if not force and up_to_date(target, stamp, key):
        return target
    obj_dir = BUILD / "obj_host"
    obj_dir.mkdir(parents=True, exist_ok=True)
    includes = ["-I", str(INCLUDE), "-I", str(HOST), "-I", sysconfig.get_paths()["include"]]
    for p in inc:
        includes += ["-isystem", p]

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        run([CXX, *flags, *includes, "-c", str(src), "-o", str(obj)], verbose)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    link = [CXX, "-shared", "-o", str(target), *map(str, objs)]
    for p in lib:
        link += ["-L", p, f"-Wl,-rpath,{p}"]
    link += ["-L", str(PKG / "lib"), "-ltwg", "-Wl,-rpath,$ORIGIN/lib",
             "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    run(link, verbose)
    stamp.write_text(key)
    return target


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", nargs="?", default="all", choices=["all", "kernels", "host"])
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory per kernel")
    args = ap.parse_args()
    if args.what in ("all", "kernels"):
        print(build_kernels(args.force, args.verbose, args.ptxas_info))
    if args.what in ("all", "host"):
        print(build_host(args.force, args.verbose))


if __name__ == "__main__":
    main()
