"""Recipe that compiles the reference's own CPU implementation into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file or what it
builds; the parity tests, the smoke check and the CPU-baseline / reference legs of the
benchmark are the only users.

What is compiled (sources are read where they lie in the reference checkout, never copied):
the non-CUDA source list of the reference's ``setup.py`` (lines 38-54) --
``src/integral_image_interface.cpp``, ``src/integral_image.cpp``,
``src/box_convolution_interface.cpp``, ``src/box_convolution.cpp``, ``src/bind.cpp`` and
``src/cuda_stubs.cpp`` -- with ``-O2 -DNDEBUG`` (the flags setuptools would use), against the
installed torch headers.  The two interface files include ``<TH/THGeneral.h>``
(``src/box_convolution_interface.cpp:5``, ``src/integral_image_interface.cpp:2``), a header
that current torch no longer ships and from which nothing is used; an empty stand-in on an
extra include path satisfies it.

Output: ``oracle/_ref/box_convolution_cpp_cuda.so`` (git-ignored; it travels with the working
tree to machines that have the same torch build but no reference checkout).

Usage:  python oracle/build_ref.py [--reference /path/to/box-convolutions]
(default: $BOXCONV_REFERENCE, else a folder `reference` beside this repository)
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
EXT_NAME = "box_convolution_cpp_cuda"
SOURCES = [
    "integral_image_interface.cpp",
    "integral_image.cpp",
    "box_convolution_interface.cpp",
    "box_convolution.cpp",
    "bind.cpp",
    "cuda_stubs.cpp",
]


def reference_root():
    """Where the reference checkout is: the BOXCONV_REFERENCE environment variable, else a folder
    `reference` beside this repository; None when neither exists."""
    for cand in (os.environ.get("BOXCONV_REFERENCE"),
                 os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src")):
            return cand
    return None


def built_path():
    return os.path.join(OUT_DIR, EXT_NAME + ".so")


def build(reference_root, verbose=False):
    """Compile the extension if the reference checkout is present.  Returns the .so path or None."""
    src_dir = os.path.join(reference_root or "", "src")
    if not reference_root or not os.path.isdir(src_dir):
        return built_path() if os.path.exists(built_path()) else None
    if os.path.exists(built_path()):
        newest_src = max(os.path.getmtime(os.path.join(src_dir, f)) for f in SOURCES)
        if os.path.getmtime(built_path()) > newest_src:
            return built_path()

    from torch.utils.cpp_extension import load

    shim = os.path.join(OUT_DIR, "shim")
    os.makedirs(os.path.join(shim, "TH"), exist_ok=True)
    with open(os.path.join(shim, "TH", "THGeneral.h"), "w") as f:
        f.write("/* empty stand-in: the header left torch, nothing from it is used */\n")
    build_dir = os.path.join(OUT_DIR, "build")
    os.makedirs(build_dir, exist_ok=True)
    load(
        name=EXT_NAME,
        sources=[os.path.join(src_dir, f) for f in SOURCES],
        extra_include_paths=[src_dir, shim],
        extra_cflags=["-O2", "-DNDEBUG"],
        build_directory=build_dir,
        is_python_module=False,
        verbose=verbose,
    )
    produced = os.path.join(build_dir, EXT_NAME + ".so")
    os.replace(produced, built_path())
    return built_path()


def load_ref():
    """Import the already-built extension as a Python module (None if it was never built)."""
    path = built_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)

    spec = importlib.util.spec_from_file_location(EXT_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=reference_root(),
                    help="reference checkout (default: $BOXCONV_REFERENCE, else ../reference beside the repository)")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    p = build(a.reference, a.verbose)
    print("reference CPU extension:", p)
    sys.exit(0 if p else 1)
