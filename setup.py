"""Build script of the B200-native `ccl` backend.

`python setup.py build_ext --inplace` compiles every C++/CUDA source under `csrc/` into one
extension module, `torch_ccl_b200/_C`, for sm_100a only, and stamps
`oneccl_bindings_for_pytorch/version.py` (the reference stamps its version the same way:
setup.py:37-67 of intel/torch-ccl). `python setup.py clean` removes build products.
"""
import glob
import os
import shutil
import subprocess
import sys

from setuptools import setup

ROOT = os.path.dirname(os.path.abspath(__file__))
VERSION = open(os.path.join(ROOT, "version.txt")).read().strip()


def git_sha():
    try:
        return subprocess.check_output(["git", "rev-parse", "HEAD"], cwd=ROOT, stderr=subprocess.DEVNULL).decode().strip()
    except Exception:
        return "Unknown"


def write_version():
    sha = os.environ.get("CCL_SHA_VERSION", git_sha())
    path = os.path.join(ROOT, "oneccl_bindings_for_pytorch", "version.py")
    text = f'__version__ = "{VERSION}"\ngit_version = "{sha}"\n'
    if not os.path.exists(path) or open(path).read() != text:
        with open(path, "w") as f:
            f.write(text)


def clean():
    for d in ("build", "torch_ccl_b200.egg-info"):
        shutil.rmtree(os.path.join(ROOT, d), ignore_errors=True)
    for so in glob.glob(os.path.join(ROOT, "torch_ccl_b200", "_C*.so")) + glob.glob(os.path.join(ROOT, "torch_ccl_b200", "lib*.so")):
        os.remove(so)


if len(sys.argv) > 1 and sys.argv[1] == "clean":
    clean()
    sys.exit(0)

from torch.utils.cpp_extension import BuildExtension, CUDAExtension  # noqa: E402

write_version()

sources = sorted(
    glob.glob("csrc/**/*.cpp", recursive=True) + glob.glob("csrc/**/*.cu", recursive=True)
)
sources = [s for s in sources if "/standalone/" not in s]
debug = os.environ.get("DEBUG", "0") == "1"
cxx_flags = ["-std=c++17", "-O0" if debug else "-O2", "-g" if debug else "-g0", "-fvisibility=hidden",
             "-Wno-deprecated-declarations", "-fstack-protector", "-Wformat-security"]
nvcc_flags = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=hidden"]
if os.environ.get("CCL_DEBUG_BOUNDS", "0") == "1":
    nvcc_flags.append("-DCCL_DEBUG_BOUNDS=1")

nccl_inc = []
try:
    import nvidia.nccl as _n
    nccl_inc = [os.path.join(os.path.dirname(_n.__file__), "include")]
except Exception:
    pass

ext = CUDAExtension(
    name="torch_ccl_b200._C",
    sources=sources,
    include_dirs=[os.path.join(ROOT, "csrc")] + nccl_inc,
    extra_compile_args={"cxx": cxx_flags, "nvcc": nvcc_flags},
    # the image's g++ wrapper finds only the static libstdc++; a private copy inside the extension has
    # uninitialised locale state (stringstream crashes), so link the shared one explicitly
    extra_link_args=["-lrt", "-lpthread", "-ldl", "-l:libstdc++.so.6"],
)

setup(
    name="torch_ccl_b200",
    version=VERSION.split("+")[0],
    packages=["torch_ccl_b200", "oneccl_bindings_for_pytorch", "torch_ccl"],
    ext_modules=[ext],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
)
