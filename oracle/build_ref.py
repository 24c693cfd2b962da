"""Build the reference's own CUDA extensions for sm_100a into ``oracle/_ref/``.  TEST INFRASTRUCTURE ONLY.

The reference ships three single-file CUDA extensions (pylo/csrc/learned_optimizer.cu, celo2_kernel.cu,
velo_kernel.cu; declared in its setup.py:57-79).  This script compiles each of them, from the sources where
they lie in the reference checkout, with the nvcc flags of the reference's setup.py:43-52 plus the sm_100a
target, through ``torch.utils.cpp_extension.load``.  Nothing of the reference is copied: only the built
modules (``cuda_lo.so``, ``celo2_cuda_kernel.so``, ``velo_cuda_kernel.so``) land in ``oracle/_ref/``, which is
kept out of version control.

The built modules are used by ``oracle/ref_cuda.py`` as a second checker (the output of the reference's own
kernels on a GPU) and as the "kernel to beat" timing; never by the product path.

    python oracle/build_ref.py [/path/to/reference]      # default /root/reference; skips what is already built
"""

import os
import shutil
import sys
from concurrent.futures import ProcessPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

# module name -> source file inside the reference checkout (setup.py:57-79)
EXTENSIONS = {
    "cuda_lo": "pylo/csrc/learned_optimizer.cu",
    "celo2_cuda_kernel": "pylo/csrc/celo2_kernel.cu",
    "velo_cuda_kernel": "pylo/csrc/velo_kernel.cu",
}
# setup.py:43-52 ("nvcc" list), plus the target this box needs
NVCC_FLAGS = ["-O3", "--use_fast_math", "-DNDEBUG", "--ftz=true", "--prec-div=false", "--prec-sqrt=false",
              "-gencode", "arch=compute_100a,code=sm_100a"]
CXX_FLAGS = ["-O3", "-DNDEBUG"]


def built_path(name):
    return os.path.join(OUT, name + ".so")


def build_one(args):
    name, src = args
    if os.path.exists(built_path(name)):
        return name, "present"
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils import cpp_extension

    work = os.path.join(OUT, "build_" + name)
    os.makedirs(work, exist_ok=True)
    cpp_extension.load(name=name, sources=[src], extra_cflags=CXX_FLAGS, extra_cuda_cflags=NVCC_FLAGS,
                       build_directory=work, is_python_module=False, verbose=False)
    shutil.copy(os.path.join(work, name + ".so"), built_path(name))
    shutil.rmtree(work, ignore_errors=True)
    return name, "built"


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    if not os.path.isdir(os.path.join(ref, "pylo", "csrc")):
        print(f"no reference checkout at {ref}: nothing built (prebuilt modules in {OUT} are used as they are)")
        return 0
    os.makedirs(OUT, exist_ok=True)
    jobs = [(name, os.path.join(ref, rel)) for name, rel in EXTENSIONS.items()]
    with ProcessPoolExecutor(max_workers=len(jobs)) as pool:
        for name, what in pool.map(build_one, jobs):
            print(f"{name}: {what}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
