"""Test infrastructure only: build the UNMODIFIED reference CUDA extension.

Compiles the reference's own extension sources, where they lie, for sm_100
with the local nvcc + PyTorch headers into ``oracle/_ref/`` (git-ignored).
The result is used only as a parity target on a GPU (tests, fixture
generation) and never by the product path.  Nothing is copied from the
reference tree; if the tree is absent this is a no-op and the prebuilt
library (if any) is used as is.

The reference checkout is looked for at ``$SVOX_REFERENCE_ROOT``, else in a
directory ``reference`` beside this repository.

Usage: python oracle/build_ref.py [reference_root]
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULE_NAME = "svox_ref_csrc"


def built_path():
    for fn in os.listdir(OUT) if os.path.isdir(OUT) else []:
        if fn.startswith(MODULE_NAME) and fn.endswith(".so"):
            return os.path.join(OUT, fn)
    return None


def reference_root():
    """Where the reference checkout lies (it need not exist)."""
    return os.environ.get("SVOX_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root=None, verbose=False):
    csrc = os.path.join(ref_root or reference_root(), "svox", "csrc")
    if not os.path.isdir(csrc):
        return built_path()
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load
    shim = os.path.join(HERE, "ref_dispatch_shim.h")
    srcs = [os.path.join(csrc, f) for f in
            ("svox.cpp", "svox_kernel.cu", "rt_kernel.cu", "quantizer.cpp")]
    load(name=MODULE_NAME, sources=srcs,
         extra_include_paths=[os.path.join(csrc, "include")],
         extra_cflags=["-include", shim, "-O2"],
         extra_cuda_cflags=["-include", shim],
         build_directory=OUT, is_python_module=False, verbose=verbose)
    return built_path()


def load_module():
    """Import the prebuilt reference extension (GPU box or here)."""
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    path = built_path()
    if path is None:
        return None
    spec = importlib.util.spec_from_file_location(MODULE_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else reference_root()
    print(build(root, verbose=True))
