"""In-tree build of the native parts of monarch_b200.

Two shared objects are produced next to the Python sources (so they are importable
without installation and are the files a process actually maps):

* ``monarch_b200/ops/_mb200_kernels.so`` -- sm_100a CUDA kernels with a plain C API
  (loaded with ctypes; no torch headers, so it compiles in seconds).
* ``monarch_b200/_native.so`` -- the C++ runtime (ndslice, channels, mailboxes,
  procs, mesh layer, telemetry) with pybind11 bindings.
* ``monarch_b200/_gradgen.so`` -- the incremental autograd executor (torch extension).
* ``monarch_b200/_tensor_worker.so`` -- the tensor worker's executor core (torch extension).

Usage: ``python -m monarch_b200._build [kernels|native|gradgen|tensor_worker|all] [--force]``
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shlex
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# The system compiler, not $CXX: a toolchain that links its own libstdc++ statically
# clashes with the libstdc++ that numpy/torch have already loaded into the process.
CXX = os.environ.get("MB200_CXX", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _run(cmd: list[str], log: Path | None = None) -> str:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(" ".join(shlex.quote(c) for c in cmd) + "\n" + p.stdout)
    if p.returncode != 0:
        raise RuntimeError(f"build command failed ({p.returncode}):\n{' '.join(cmd)}\n{p.stdout}")
    return p.stdout


def _stamp(srcs: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for s in sorted(srcs):
        h.update(str(s).encode())
        h.update(s.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _deps(dirs: list[Path]) -> list[Path]:
    out: list[Path] = []
    for d in dirs:
        for ext in ("*.h", "*.hpp", "*.cuh", "*.cu", "*.cpp"):
            out += list(d.rglob(ext))
    return out


def _up_to_date(target: Path, stamp: str) -> bool:
    sf = target.with_suffix(target.suffix + ".stamp")
    return target.exists() and sf.exists() and sf.read_text() == stamp


def _write_stamp(target: Path, stamp: str) -> None:
    target.with_suffix(target.suffix + ".stamp").write_text(stamp)


def _compile_many(jobs: list[tuple[list[str], Path]]) -> None:
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        futs = [ex.submit(_run, cmd, log) for cmd, log in jobs]
        for f in futs:
            f.result()


def build_kernels(force: bool = False, checked: bool = False) -> Path:
    """``checked=True`` builds ``_mb200_kernels_checked.so``: the same kernels with
    ``-DMB200_BOUNDS_CHECK``, in which the collectives validate every peer access against a
    table of registered address ranges and report violations through the status word instead
    of touching the memory (selected at run time with ``MB200_KERNEL_LIB=checked``)."""
    kdir = CSRC / "kernels"
    target = ROOT / "ops" / ("_mb200_kernels_checked.so" if checked else "_mb200_kernels.so")
    srcs = sorted(kdir.glob("*.cu"))
    flags = CUDA_FLAGS + (["-DMB200_BOUNDS_CHECK"] if checked else [])
    stamp = _stamp(_deps([kdir]), flags)
    if not force and _up_to_date(target, stamp):
        return target
    odir = OBJ / ("kernels_checked" if checked else "kernels")
    odir.mkdir(parents=True, exist_ok=True)
    jobs = []
    objs = []
    for s in srcs:
        o = odir / (s.stem + ".o")
        objs.append(str(o))
        jobs.append(([NVCC, *flags, "-I", str(kdir), "-c", str(s), "-o", str(o)],
                     odir / (s.stem + ".log")))
    _compile_many(jobs)
    _run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objs, "-o", str(target)])
    _write_stamp(target, stamp)
    return target


def _py_includes() -> list[str]:
    import pybind11
    return ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]


NATIVE_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall",
                "-Wno-unused-function"]


def build_runtime_stress(sanitizer: str = "thread") -> Path:
    """The native runtime's concurrency stress program (``csrc/tests/runtime_stress.cpp``)
    linked with the host runtime sources under ``-fsanitize=<sanitizer>`` ("thread" or
    "address"); no Python, no GPU.  Returns the executable."""
    if sanitizer not in ("thread", "address", "none"):
        raise ValueError(f"unknown sanitizer {sanitizer!r}")
    dirs = [CSRC / d for d in ("ndslice", "actor", "channel", "mesh", "telemetry")]
    srcs = sorted(p for d in dirs for p in d.rglob("*.cpp")) + [CSRC / "tests" / "runtime_stress.cpp"]
    flags = ["-O1", "-g", "-std=c++20", "-pthread", "-fno-omit-frame-pointer"]
    if sanitizer != "none":
        flags.append(f"-fsanitize={sanitizer}")
    odir = OBJ / f"stress_{sanitizer}"
    odir.mkdir(parents=True, exist_ok=True)
    target = odir / "runtime_stress"
    stamp = _stamp(_deps(dirs + [CSRC / "tests"]), flags)
    if _up_to_date(target, stamp):
        return target
    jobs, objs = [], []
    for s in srcs:
        o = odir / (s.parent.name + "_" + s.stem + ".o")
        objs.append(str(o))
        jobs.append(([CXX, *flags, "-I", str(CSRC), "-c", str(s), "-o", str(o)],
                     odir / (s.parent.name + "_" + s.stem + ".log")))
    _compile_many(jobs)
    _run([CXX, *flags, *objs, "-o", str(target), "-lrt"])
    _write_stamp(target, stamp)
    return target


def build_native(force: bool = False) -> Path:
    target = ROOT / "_native.so"
    dirs = [CSRC / d for d in ("ndslice", "actor", "channel", "mesh", "telemetry", "python",
                               "rdma", "tensor")]
    srcs = sorted(p for d in dirs for p in d.rglob("*.cpp"))
    if not (CSRC / "python" / "module.cpp").exists():
        return target
    stamp = _stamp(_deps(dirs), NATIVE_FLAGS)
    if not force and _up_to_date(target, stamp):
        return target
    odir = OBJ / "native"
    odir.mkdir(parents=True, exist_ok=True)
    jobs = []
    objs = []
    for s in srcs:
        o = odir / (s.parent.name + "_" + s.stem + ".o")
        objs.append(str(o))
        jobs.append(([CXX, *NATIVE_FLAGS, "-I", str(CSRC), *_py_includes(), "-c", str(s), "-o",
                      str(o)], odir / (s.parent.name + "_" + s.stem + ".log")))
    _compile_many(jobs)
    _run([CXX, "-shared", "-pthread", *objs, "-o", str(target), "-lrt"])
    _write_stamp(target, stamp)
    return target


def build_gradgen(force: bool = False) -> Path:
    """The gradient generator links against libtorch (it drives the autograd engine)."""
    target = ROOT / "_gradgen.so"
    src = CSRC / "gradgen" / "gradient_generator.cpp"
    if not src.exists():
        return target
    import torch
    from torch.utils import cpp_extension as ce
    flags = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_gradgen",
             "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI))]
    stamp = _stamp([src], flags + [torch.__version__])
    if not force and _up_to_date(target, stamp):
        return target
    incs = []
    for i in ce.include_paths():
        incs += ["-isystem", i]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    _run([CXX, *flags, *incs, *_py_includes(), "-shared", str(src), "-o", str(target),
          "-L", libdir, "-Wl,-rpath," + libdir, "-ltorch", "-ltorch_cpu", "-lc10",
          "-ltorch_python"])
    _write_stamp(target, stamp)
    return target


def _build_torch_ext(name: str, src: Path, force: bool) -> Path:
    """One-file torch extension (links libtorch + torch_python), built in-tree."""
    target = ROOT / f"{name}.so"
    if not src.exists():
        return target
    import torch
    from torch.utils import cpp_extension as ce
    flags = ["-O2", "-std=c++17", "-fPIC", f"-DTORCH_EXTENSION_NAME={name}",
             "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI))]
    stamp = _stamp([src, *sorted(src.parent.glob("*.h"))], flags + [torch.__version__])
    if not force and _up_to_date(target, stamp):
        return target
    incs = []
    for i in ce.include_paths():
        incs += ["-isystem", i]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    _run([CXX, *flags, *incs, *_py_includes(), "-shared", str(src), "-o", str(target),
          "-L", libdir, "-Wl,-rpath," + libdir, "-ltorch", "-ltorch_cpu", "-lc10",
          "-ltorch_python"])
    _write_stamp(target, stamp)
    return target


def build_tensor_worker(force: bool = False) -> Path:
    """The tensor worker's native executor core (ATen dispatcher calls, recordings)."""
    return _build_torch_ext("_tensor_worker", CSRC / "tensor_worker" / "worker_core.cpp", force)


def build_allocator(force: bool = False) -> Path:
    """The native process-allocator daemon (``csrc/tools/process_allocator.cpp``): a
    standalone executable, ``monarch_b200/tools/process_allocator_native``."""
    src = CSRC / "tools" / "process_allocator.cpp"
    target = ROOT / "tools" / "process_allocator_native"
    _build_tool(src, target, force)
    build_remote_exec(force)
    return target


def build_remote_exec(force: bool = False) -> Path:
    """The native client stub of a remote proc (``csrc/tools/remote_exec.cpp``):
    ``monarch_b200/tools/remote_exec_native``."""
    return _build_tool(CSRC / "tools" / "remote_exec.cpp", ROOT / "tools" / "remote_exec_native",
                       force)


def _build_tool(src: Path, target: Path, force: bool) -> Path:
    flags = ["-O2", "-std=c++17", "-pthread", "-Wall"]
    stamp = _stamp([src, *sorted(src.parent.glob("*.h"))], flags)
    if not force and _up_to_date(target, stamp):
        return target
    _run([CXX, *flags, "-I", str(src.parent), str(src), "-o", str(target)])
    _write_stamp(target, stamp)
    return target


def build_all(force: bool = False) -> None:
    build_allocator(force)
    build_kernels(force)
    build_kernels(force, checked=True)
    build_native(force)
    build_gradgen(force)
    build_tensor_worker(force)


if __name__ == "__main__":
    what = [a for a in sys.argv[1:] if not a.startswith("-")] or ["all"]
    force = "--force" in sys.argv
    for w in what:
        {"kernels": build_kernels, "kernels_checked": lambda f: build_kernels(f, checked=True),
         "native": build_native, "gradgen": build_gradgen,
         "tensor_worker": build_tensor_worker, "allocator": build_allocator,
         "all": build_all}[w](force)
        print("built", w)
