"""Builds the reference's own ``table_batched_embeddings`` CUDA extension into ``oracle/_ref/``.
TEST INFRASTRUCTURE ONLY: the result pins the CPU oracle, nothing in the product imports it.

    python oracle/build_ref.py [reference_dir]

The two sources (table_batched_embeddings.cpp, table_batched_embeddings_cuda.cu) are compiled where
they lie: they are streamed through the mechanical edits below into a scratch directory outside the
repository, compiled there with nvcc (sm_100a) and g++ against the installed torch, and only the
linked ``table_batched_embeddings.so`` is kept, under ``oracle/_ref/`` (git-ignored).  No reference
source is copied into the repository and the reference's setup.py is not run.

Edits (all one-line; the kernels and the host logic of the lookup path are untouched):
  1. ``ATen/CUDAGenerator.h`` no longer exists: include ``ATen/cuda/CUDAGeneratorImpl.h``.
  2. ``getDefaultCUDAGenerator()`` now returns a Generator handle; the code wants the impl pointer
     (``gen->mutex_``, ``gen->philox_engine_inputs``): wrap it in ``get_generator_or_default``.
  3. ``AT_DISPATCH_*(weights.type(), ...)`` -> ``weights.scalar_type()``.
  4. ``__HALF2_TO_UI`` is undefined at the end of today's cuda_fp16.h: define it again.
  5. The managed / host-mapped allocator block (table_batched_embeddings_cuda.cu:795-880) subclasses
     an ``at::Allocator`` interface that has since changed; it is not on the arithmetic path, so the
     block and its two ``m.def`` lines are dropped.
"""
import os
import re
import shutil
import subprocess
import sys
import sysconfig
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "table_batched_embeddings.so")
SOURCES = ("table_batched_embeddings.cpp", "table_batched_embeddings_cuda.cu")

HALF2_TO_UI = "#define __HALF2_TO_UI(var) *(reinterpret_cast<unsigned int *>(&(var)))"


def _edit_cu(text):
    text = text.replace("#include <ATen/CUDAGenerator.h>", "#include <ATen/cuda/CUDAGeneratorImpl.h>")
    text = text.replace("#include <mutex>", "#include <mutex>\n" + HALF2_TO_UI, 1)
    text = text.replace(
        "auto gen = at::cuda::detail::getDefaultCUDAGenerator();",
        "auto gen = at::get_generator_or_default<at::CUDAGeneratorImpl>(c10::nullopt, "
        "at::cuda::detail::getDefaultCUDAGenerator());")
    text = text.replace('.type(), "batched', '.scalar_type(), "batched')
    begin = text.index("static void CUDAManagedDeleter")
    end = text.index("template <typename scalar_t, bool shared_indices, typename F>", begin)
    return text[:begin] + text[end:]


def _edit_cpp(text):
    return "".join(line for line in text.splitlines(keepends=True)
                   if not re.search(r"new_managed_tensor|new_host_mapped_tensor", line))


def _run(cmd, cwd):
    r = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("%s failed:\n%s\n%s" % (" ".join(cmd[:3]), r.stdout[-4000:], r.stderr[-4000:]))


def up_to_date(ref_dir):
    if not os.path.exists(OUT):
        return False
    deps = [os.path.join(ref_dir, s) for s in SOURCES] + [os.path.abspath(__file__)]
    return all(os.path.getmtime(d) <= os.path.getmtime(OUT) for d in deps)


def build(ref_dir="/root/reference", force=False):
    """Returns the path of the built extension, or None when the reference sources are absent (the
    prebuilt file, if any, is then used as it is)."""
    if not all(os.path.exists(os.path.join(ref_dir, s)) for s in SOURCES):
        return OUT if os.path.exists(OUT) else None
    if not force and up_to_date(ref_dir):
        return OUT
    import torch
    from torch.utils import cpp_extension
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    tinc = cpp_extension.include_paths("cuda")
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    incs = []
    for p in tinc + [sysconfig.get_paths()["include"]]:
        incs += ["-I", p]
    defs = ["-DTORCH_EXTENSION_NAME=table_batched_embeddings", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    os.makedirs(OUT_DIR, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="tbe_ref_build_") as tmp:
        with open(os.path.join(ref_dir, SOURCES[1])) as f:
            cu = _edit_cu(f.read())
        with open(os.path.join(ref_dir, SOURCES[0])) as f:
            cpp = _edit_cpp(f.read())
        with open(os.path.join(tmp, "ref_cuda.cu"), "w") as f:
            f.write(cu)
        with open(os.path.join(tmp, "ref_bind.cpp"), "w") as f:
            f.write(cpp)
        _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC"] + incs + defs + ["-c", "ref_cuda.cu", "-o", "ref_cuda.o"], tmp)
        _run(["g++", "-O2", "-std=c++17", "-fPIC"] + incs + defs + ["-c", "ref_bind.cpp", "-o", "ref_bind.o"], tmp)
        _run(["g++", "-shared", "-o", OUT, "ref_bind.o", "ref_cuda.o", "-L", tlib, "-L", "/usr/local/cuda/lib64",
              "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
              "-Wl,-rpath," + tlib], tmp)
    return OUT


def load():
    """Imports the built extension (``import torch`` first: it links against libtorch)."""
    import importlib.util
    import torch  # noqa: F401
    if not os.path.exists(OUT):
        raise ImportError("oracle/_ref/table_batched_embeddings.so has not been built (python oracle/build_ref.py)")
    spec = importlib.util.spec_from_file_location("table_batched_embeddings", OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), force="--force" in sys.argv))
