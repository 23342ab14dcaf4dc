"""In-tree build and loading of the native extension ``supergrok15_b200/_C*.so``.

The CUDA translation units (``csrc/*.cu``) contain no PyTorch headers and are compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a``; ``csrc/bindings.cpp`` (PyTorch / pybind11) is
compiled with the host compiler; everything is linked into one shared object that lives next to
this file, so a source snapshot that carries the built ``.so`` needs no compiler on the GPU box.
nvcc cross-compiles without a GPU, so the build also runs on a CPU-only machine.

``load()`` imports the extension (building it first if it is missing or stale and a compiler is
available).  ``native_available()`` says whether it could be loaded.  Optimizer steps on CUDA
tensors raise if it is not available: there is no silent PyTorch fallback on a GPU.
"""
from __future__ import annotations

import hashlib
import importlib.util
import json
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Optional

_HERE = Path(__file__).resolve().parent
_CSRC = _HERE / "csrc"
_OBJ = _HERE / "csrc" / "build"
_NAME = "_C"
_mod = None
_err: Optional[str] = None

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _so_path() -> Path:
    return _HERE / (_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def _sources() -> List[Path]:
    return sorted(_CSRC.glob("*.cu")) + sorted(_CSRC.glob("*.cpp"))


def _headers() -> List[Path]:
    return sorted(_CSRC.glob("*.h")) + sorted(_CSRC.glob("*.cuh"))


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _nvcc() -> Optional[str]:
    cand = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/bin/nvcc"
    return cand if os.path.exists(cand) else shutil.which("nvcc")


def _run(cmd: List[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build command failed:\n" + " ".join(cmd) + "\n" + r.stdout[-4000:] + r.stderr[-8000:])
    if os.environ.get("SG_BUILD_VERBOSE") and (r.stdout or r.stderr):
        sys.stderr.write(r.stdout + r.stderr)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every native source for sm_100a and link the extension in-tree.  Incremental per file."""
    stamp_file = _OBJ / "stamps.json"
    if not force and stamp_file.exists() and _so_path().exists():
        old = json.loads(stamp_file.read_text())
        hdr0 = _digest(_headers())
        if all(old.get(s.name) == _digest([s]) + hdr0 for s in _sources()):
            return _so_path()          # sources unchanged since the shared object was linked
    import torch
    from torch.utils import cpp_extension as ce

    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a extension")
    _OBJ.mkdir(parents=True, exist_ok=True)
    stamps = json.loads(stamp_file.read_text()) if stamp_file.exists() and not force else {}
    hdr = _digest(_headers())
    cuda_home = str(Path(nvcc).parent.parent)
    inc = [f"-I{_CSRC}", f"-I{cuda_home}/include"]
    torch_inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    jobs = []
    objs = []
    for src in _sources():
        obj = _OBJ / (src.name + ".o")
        objs.append(obj)
        key = _digest([src]) + hdr
        if stamps.get(src.name) == key and obj.exists():
            continue
        if src.suffix == ".cu":
            cmd = [nvcc, *NVCC_ARCH, "-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler",
                   "-fPIC", "-Xptxas", "-v" if verbose else "-warn-spills", *inc, "-c", str(src), "-o", str(obj)]
        else:
            # -fopenmp: at::parallel_for is a header template around "#pragma omp parallel"; without the flag it runs serially
            cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-fopenmp", "-DTORCH_EXTENSION_NAME=" + _NAME,
                   "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)),
                   *inc, *torch_inc, "-c", str(src), "-o", str(obj)]
        jobs.append((src.name, key, cmd))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(j[2]), jobs))
        for name, key, _ in jobs:
            stamps[name] = key
        stamp_file.write_text(json.dumps(stamps, indent=0))
    so = _so_path()
    if jobs or not so.exists():
        tlib = Path(torch.__file__).parent / "lib"
        cmd = ["g++", "-shared", "-fopenmp", "-o", str(so), *map(str, objs), f"-L{tlib}", f"-L{cuda_home}/lib64", "-lc10",
               "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart",
               f"-Wl,-rpath,{tlib}", f"-Wl,-rpath,{cuda_home}/lib64"]
        _run(cmd)
    return so


def build_sanitized(out_dir) -> Path:
    """Host-code check build: every ``csrc/*.cpp`` compiled with ``-Wall -Werror -fsanitize=address,undefined`` and linked with
    the regular CUDA objects into ``out_dir``.  Load it by setting ``SG_EXT_SO`` to the returned path in a process started with
    ``LD_PRELOAD=$(gcc -print-file-name=libasan.so)`` (the CPU kernels and the binding layer then run under ASan / UBSan)."""
    import torch
    from torch.utils import cpp_extension as ce
    build()                                                           # the CUDA objects come from the regular build
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cuda_home = str(Path(_nvcc()).parent.parent)
    inc = [f"-I{_CSRC}", "-isystem", f"{cuda_home}/include"]
    for p in list(ce.include_paths()) + [sysconfig.get_paths()["include"]]:
        inc += ["-isystem", p]                                        # third-party headers are not held to -Werror
    jobs, objs = [], []
    for src in _sources():
        if src.suffix == ".cu":
            objs.append(_OBJ / (src.name + ".o"))
            continue
        obj = out_dir / (src.name + ".san.o")
        objs.append(obj)
        jobs.append(["g++", "-O1", "-g", "-std=c++17", "-fPIC", "-fopenmp", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-Wall", "-Werror",
                     "-DTORCH_EXTENSION_NAME=" + _NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
                     "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)), *inc, "-c", str(src), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        list(ex.map(_run, jobs))
    so = out_dir / _so_path().name
    tlib = Path(torch.__file__).parent / "lib"
    _run(["g++", "-shared", "-fopenmp", "-fsanitize=address,undefined", "-o", str(so), *map(str, objs), f"-L{tlib}", f"-L{cuda_home}/lib64", "-lc10",
          "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart", f"-Wl,-rpath,{tlib}",
          f"-Wl,-rpath,{cuda_home}/lib64"])
    return so


def build_bounds_checked(out_dir) -> Path:
    """Device-code check build: ``csrc/mt_kernels.cu`` compiled with ``-DGROK_BOUNDS_CHECK`` (every element access of the
    multi-tensor optimizer kernels is compared with the driver's record of the allocation; a violation is skipped and
    recorded, never a trap) and linked with the regular objects into ``out_dir``.  Load it with ``SG_EXT_SO``; run with
    ``PYTORCH_NO_CUDA_MEMORY_CACHING=1`` so that every tensor is an allocation of its own; read ``_C.bounds_report()``."""
    import torch
    build()
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    cuda_home = str(Path(nvcc).parent.parent)
    objs = []
    for src in _sources():
        if src.name == "mt_kernels.cu":
            obj = out_dir / "mt_kernels.checked.o"
            _run([nvcc, *NVCC_ARCH, "-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-DGROK_BOUNDS_CHECK",
                  f"-I{_CSRC}", f"-I{cuda_home}/include", "-c", str(src), "-o", str(obj)])
            objs.append(obj)
        else:
            objs.append(_OBJ / (src.name + ".o"))
    so = out_dir / _so_path().name
    tlib = Path(torch.__file__).parent / "lib"
    _run(["g++", "-shared", "-fopenmp", "-o", str(so), *map(str, objs), f"-L{tlib}", f"-L{cuda_home}/lib64", "-lc10", "-ltorch_cpu", "-ltorch",
          "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart", f"-Wl,-rpath,{tlib}", f"-Wl,-rpath,{cuda_home}/lib64"])
    return so


def load(build_if_needed: bool = True):
    """Return the extension module, or None (with the reason in ``load_error()``).  ``SG_EXT_SO`` names a shared object to load
    instead of the in-tree one (the sanitizer build of ``build_sanitized``)."""
    global _mod, _err
    if _mod is not None:
        return _mod
    so = _so_path()
    override = os.environ.get("SG_EXT_SO")
    if override:
        so, build_if_needed = Path(override), False
    try:
        if build_if_needed and _nvcc() is not None and os.environ.get("SG_NO_BUILD") != "1":
            build()
        if not so.exists():
            raise FileNotFoundError(f"{so} not built")
        import torch  # noqa: F401  (libtorch must be loaded first)
        spec = importlib.util.spec_from_file_location(__package__ + "." + _NAME, so)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    except Exception as e:  # noqa: BLE001
        _err = f"{type(e).__name__}: {e}"
        _mod = None
    return _mod


def native_available() -> bool:
    return load() is not None


def load_error() -> Optional[str]:
    return _err


def require():
    """Extension module or a loud error: CUDA paths never fall back to PyTorch ops."""
    m = load()
    if m is None:
        raise RuntimeError("supergrok15_b200 native extension is not available (" + str(_err) +
                           "); CUDA tensors need it - run `python -m supergrok15_b200._build`")
    return m


if __name__ == "__main__":
    if "--bounds-check" in sys.argv:                     # python -m supergrok15_b200._build --bounds-check <dir>
        print("built", build_bounds_checked(sys.argv[sys.argv.index("--bounds-check") + 1]))
    else:
        print("built", build(force="--force" in sys.argv, verbose="-v" in sys.argv))
