"""Install the reference into baseline/_ref for the `bench.py --impl reference` arm (offline, no GPU needed).

What it does, and why each deviation from a plain `pip install <reference tree>` is needed:
  1. copies the read-only reference tree to a scratch directory (the build writes into its source tree);
  2. edits the COPY's setup.py only: drops the "CUDA device must be visible" check (nvcc cross-compiles) and
     replaces the gencode list sm_70..sm_90 (no PTX, so none of it runs on a B200) by sm_100;
  3. pip-installs the copy with --no-index --no-build-isolation --no-deps --target baseline/_ref;
  4. copies grokking_race_v2.py (a top-level script that pip does not install) next to the package: the
     reference arm takes the reference's own model and data generator from it;
  5. builds baseline/_ref/libref_shim.so from baseline/ref_shim.cpp (one missing PyTorch symbol, see that file).
No kernel, dispatch or Python source file of the reference is modified.

usage: python baseline/build_reference.py /path/to/reference     (or set SG_REFERENCE_SRC)
"""
import os
import re
import shutil
import subprocess
import sys
import sysconfig
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def main():
    src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SG_REFERENCE_SRC")
    if not src or not os.path.isdir(src):
        sys.exit("usage: python baseline/build_reference.py /path/to/reference [wheel directory]")
    work = os.path.join(tempfile.mkdtemp(prefix="refbuild_"), "src")
    shutil.copytree(src, work)
    sp = os.path.join(work, "setup.py")
    s = open(sp).read()
    a, b = s.index("if not torch.cuda.is_available():"), s.index('print(f"Building Grokking Optimizers')
    s = s[:a] + s[b:]
    s = re.sub(r'\s*"-gencode=arch=compute_\d+,code=sm_\d+",\s*#[^\n]*', "", s)
    s = s.replace('"-lineinfo",', '"-lineinfo",\n            "-gencode=arch=compute_100,code=sm_100",')
    open(sp, "w").write(s)
    env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0", MAX_JOBS=os.environ.get("MAX_JOBS", "6"))
    # offline wheel directory for pip's --find-links: second argument, or $PIP_FIND_LINKS / $WHEELHOUSE, or none
    wheels = sys.argv[2] if len(sys.argv) > 2 else (os.environ.get("PIP_FIND_LINKS") or os.environ.get("WHEELHOUSE"))
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps"]
    if wheels:
        cmd += ["--find-links", wheels]
    subprocess.check_call(cmd + ["--target", DEST, "--upgrade", work], env=env)
    shutil.copy(os.path.join(src, "grokking_race_v2.py"), DEST)
    build_shim()


def build_shim():
    import torch
    from torch.utils import cpp_extension as ce
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)),
           *[f"-I{p}" for p in ce.include_paths()], f"-I{sysconfig.get_paths()['include']}", os.path.join(HERE, "ref_shim.cpp"), "-o",
           os.path.join(DEST, "libref_shim.so"), f"-L{tlib}", "-lc10", "-ltorch_cpu", f"-Wl,-rpath,{tlib}"]
    subprocess.check_call(cmd)


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "--shim-only":
        build_shim()
    else:
        main()
