"""In-tree native build: every CUDA kernel (sm_100a) and the C++ host runtime.

Two shared objects are produced next to this file:

* ``libpsb_cuda.so``  -- all hand-written sm_100a kernels behind a C ABI
  (``extern "C"`` launchers taking raw device pointers and a stream); loaded
  with ``ctypes`` by :mod:`parameter_server_b200.ops._lib`.
* ``_core.<abi>.so``  -- the host control plane (ranges, messages, executor
  DAG engine, van, postoffice, manager, CPU containers/filters/parsers) as a
  pybind11 module.

A library is rebuilt when the contents of its sources, headers or compiler flags differ from those it
was built from (a digest kept beside it in ``<library>.stamp``; file times do not survive a copy to
another machine); single objects are recompiled when their source or a header is newer.
``nvcc`` cross-compiles without a GPU, so this also runs on CPU-only boxes.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "csrc" / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
# No --use_fast_math: it would change the exp/log/div numerics of the optimiser
# and loss math, which is checked against an fp32 oracle.


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(src_list, out: Path) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_list)


def _digest(files, extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for f in sorted(map(Path, files)):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _stale(files, out: Path, extra: str = "") -> bool:
    """True if ``out`` is missing or was built from other contents than ``files`` (and ``extra``) now have."""
    stamp = out.with_name(out.name + ".stamp")
    return not out.exists() or not stamp.exists() or stamp.read_text().strip() != _digest(files, extra)


def _mark(files, out: Path, extra: str = ""):
    out.with_name(out.name + ".stamp").write_text(_digest(files, extra) + "\n")


def _run(cmd, log: Path | None = None):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(" ".join(map(str, cmd)) + "\n" + p.stdout)
    if p.returncode != 0:
        raise RuntimeError("build failed: %s\n%s" % (" ".join(map(str, cmd)), p.stdout))
    return p.stdout


def cuda_lib_path() -> Path:
    return PKG / "libpsb_cuda.so"


def core_lib_path() -> Path:
    return PKG / ("_core" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/cuda/*.cu`` for sm_100a and link ``libpsb_cuda.so``."""
    OBJ.mkdir(parents=True, exist_ok=True)
    cu_dir = CSRC / "cuda"
    headers = sorted(cu_dir.glob("*.cuh")) + sorted(cu_dir.glob("*.h"))
    sources = sorted(cu_dir.glob("*.cu"))
    out = cuda_lib_path()
    if not force and not _stale(sources + headers, out, " ".join(NVCC_FLAGS)):
        return out  # the shipped library is current (e.g. on a box that received only the .so and its stamp)
    nvcc = _nvcc()
    objs, jobs = [], []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(cu_dir), "-c", str(src), "-o", str(obj)]
            jobs.append((cmd, OBJ / (src.stem + ".ptxas.log")))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(lambda j: _run(*j), jobs):
                if verbose:
                    print(out)
    out = cuda_lib_path()
    if force or jobs or _newer(objs, out) or not out.exists():
        _link([nvcc, "-shared"], out, [*map(str, objs), "-lcuda"])
    _mark(sources + headers, out, " ".join(NVCC_FLAGS))
    return out


def build_core(force: bool = False) -> Path:
    """Compile the C++ host runtime (pybind11 module ``_core``)."""
    import pybind11

    OBJ.mkdir(parents=True, exist_ok=True)
    core_dir = CSRC / "core"
    headers = sorted(core_dir.glob("*.h"))
    sources = sorted(core_dir.glob("*.cc"))
    # The distribution compiler, not $CXX: a toolchain that links libstdc++
    # statically would put a second C++ runtime next to the one NumPy/PyTorch load.
    out = core_lib_path()
    exe = PKG / "bin" / "psb_linear"
    if not force and not _stale(sources + headers, out) and exe.exists() and not _stale(sources + headers, exe):
        return out
    cxx = os.environ.get("PSB_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(core_dir)]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread"]
    objs, jobs = [], []
    for src in sources:
        obj = OBJ / ("core_" + src.stem + ".o")
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            jobs.append(([cxx, *flags, *inc, "-c", str(src), "-o", str(obj)], None))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    out = core_lib_path()
    lib_objs = [o for o in objs if not o.name.endswith("_main.o")]
    if force or jobs or _newer(lib_objs, out):
        _link([cxx, "-shared", "-pthread"], out, [*map(str, lib_objs), "-lz"])
    # the stand-alone linear-method binary (every node of a CPU deployment runs it)
    exe = PKG / "bin" / "psb_linear"
    exe.parent.mkdir(exist_ok=True)
    exe_objs = [o for o in objs if not o.name.startswith("core_bind") and o.name != "core_ps_main.o"]
    if force or jobs or _newer(exe_objs, exe):
        _link([cxx, "-pthread"], exe, [*map(str, exe_objs), "-lz"])
    _mark(sources + headers, out)
    _mark(sources + headers, exe)
    return out


def build_static(force: bool = False):
    """``lib/libpsb.a`` (the host runtime: util, data, system, filter, learner, parameter and the linear
    methods) and ``lib/libpsbmain.a`` (the ``main`` of a program that defines only ``PS::CreateServerNode``
    and ``PS::WorkerNodeMain``), for C++ programs that link the runtime the way the reference's users link
    ``build/libps.a`` and ``build/libpsmain.a`` (``Makefile:28-47``). Headers are ``csrc/core/*.h``."""
    core_dir = CSRC / "core"
    libdir = PKG / "lib"
    lib, main_lib = libdir / "libpsb.a", libdir / "libpsbmain.a"
    inputs = sorted(core_dir.glob("*.cc")) + sorted(core_dir.glob("*.h"))
    # staleness by the digest of the sources, as for the shared objects: a copy of the tree that carries the
    # archives but not the object files (they are intermediate) must find the archives up to date
    build_core(force=force)          # the module and the node binary have stamps of their own
    if not force and lib.exists() and main_lib.exists() and not _stale(inputs, lib):
        return lib, main_lib
    libdir.mkdir(exist_ok=True)
    objs = [OBJ / ("core_" + s.stem + ".o") for s in sorted(core_dir.glob("*.cc"))
            if not s.name.startswith("bind") and not s.stem.endswith("_main")]
    if not all(o.exists() for o in objs):
        build_core(force=True)
    _archive(lib, objs)
    main_obj = OBJ / "simple_main.o"
    cxx = os.environ.get("PSB_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    _run([cxx, "-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread", "-DPSB_SIMPLE_MAIN", "-I", str(core_dir),
          "-c", str(core_dir / "ps_main.cc"), "-o", str(main_obj)])
    _archive(main_lib, [main_obj])
    _mark(inputs, lib)
    return lib, main_lib


def _archive(out: Path, objs: list):
    tmp = out.with_name(f"{out.name}.tmp.{os.getpid()}")
    try:
        _run(["ar", "crs", str(tmp), *map(str, objs)])
        os.replace(tmp, out)
    finally:
        if tmp.exists():
            tmp.unlink()


def _link(cmd: list, out: Path, inputs: list):
    """Link into a temporary name and rename: a process that loads or executes ``out`` at the same
    moment (two test runs side by side) sees the old file or the new one, never a half-written one."""
    tmp = out.with_name(f"{out.name}.tmp.{os.getpid()}")
    try:
        _run([*cmd, "-o", str(tmp), *inputs])
        os.replace(tmp, out)
    finally:
        if tmp.exists():
            tmp.unlink()


def build_sanitized_binary(kinds: str = "address,undefined") -> Path:
    """``bin/psb_linear_san``: the stand-alone node binary compiled with
    ``-fsanitize=<kinds>`` (``address,undefined`` or ``thread``). The reference builds
    with no sanitizer at all (``make/config.mk:10``); this is how the host runtime
    (van, postoffice, executor, parameters, filters, learners) is checked for memory
    errors, undefined behaviour and data races on CPU-only machines:
    ``python -m parameter_server_b200._build --sanitize[=thread]`` and then run the
    binary like ``bin/psb_linear`` (e.g. with ``system.cluster.launch_local_processes``)."""
    core_dir = CSRC / "core"
    cxx = os.environ.get("PSB_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    tag = "tsan" if "thread" in kinds else "san"
    odir = OBJ / tag
    odir.mkdir(parents=True, exist_ok=True)
    flags = ["-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={kinds}", "-std=c++17", "-Wall", "-pthread",
             "-I", str(core_dir)]
    sources = [s for s in sorted(core_dir.glob("*.cc")) if not s.name.startswith("bind") and s.name != "ps_main.cc"]
    objs = [odir / (s.stem + ".o") for s in sources]
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(lambda so: _run([cxx, *flags, "-c", str(so[0]), "-o", str(so[1])], None), zip(sources, objs)))
    exe = PKG / "bin" / ("psb_linear_" + tag)
    exe.parent.mkdir(exist_ok=True)
    _link([cxx, f"-fsanitize={kinds}", "-pthread"], exe, [*map(str, objs), "-lz"])
    return exe


def build_all(force: bool = False, verbose: bool = False):
    """Everything, and one line per artefact on stdout: whether it was compiled by this call or found
    current (same source digest), so that a build log shows what the call did."""
    t0 = time.time()
    before = {p: (p.stat().st_mtime_ns if p.exists() else None) for p in _artefacts()}
    a = build_cuda(force=force, verbose=verbose)
    b = build_core(force=force)
    build_static()
    for p in _artefacts():
        now = p.stat().st_mtime_ns if p.exists() else None
        what = "missing" if now is None else ("built" if now != before[p] else "up to date")
        print(f"[build] {p.relative_to(PKG.parent)}: {what}" + (f", {p.stat().st_size} bytes" if now else ""))
    n_cu = len(list((CSRC / "cuda").glob("*.cu")))
    print(f"[build] {n_cu} CUDA sources for sm_100a ({' '.join(NVCC_FLAGS[:4])} ...), {time.time() - t0:.1f} s")
    return a, b


def _artefacts():
    return [cuda_lib_path(), core_lib_path(), PKG / "bin" / "psb_linear", PKG / "lib" / "libpsb.a", PKG / "lib" / "libpsbmain.a"]


if __name__ == "__main__":
    san = [a for a in sys.argv if a.startswith("--sanitize")]
    if san:
        print(build_sanitized_binary(san[0].split("=", 1)[1] if "=" in san[0] else "address,undefined"))
        sys.exit(0)
    if "--static" in sys.argv:
        for p in build_static(force="--force" in sys.argv):
            print(p)
        sys.exit(0)
    if "--core" in sys.argv:
        print(build_core(force="--force" in sys.argv))
        sys.exit(0)
    paths = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for p in paths:
        print(p)
