"""The C-ABI library loads and exports every symbol that include/boxconv_b200.h declares.
No compute calls: this runs on machines without a GPU."""
import ctypes
import os
import re

from conftest import PKG_DIR, ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "boxconv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert "bc_integral_image" in names and "bc_boxconv2d_backward" in names and len(names) >= 12
    lib = ctypes.CDLL(os.path.join(PKG_DIR, "box_convolution", "libboxconv_b200.so"))
    for n in names:
        assert hasattr(lib, n), n


def test_binding_table_covers_the_header():
    from box_convolution import _cabi
    assert sorted(_cabi.SIGNATURES) == declared_symbols()


def test_status_strings_and_argument_checks_without_a_gpu():
    from box_convolution import _cabi
    lib = _cabi.lib
    assert lib.bc_version() >= 100
    assert lib.bc_status_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert lib.bc_status_string(code) not in (b"ok", b"unknown status")
    # argument validation happens before anything touches the device
    assert lib.bc_integral_image(None, None, 3, 4, 5, None) == -1
    assert lib.bc_integral_image(None, None, -1, 4, 5, None) == -2
    assert lib.bc_integral_image(None, None, 0, 4, 5, None) == 0
    assert lib.bc_clip_parameters(None, None, None, None, 4, 1.0, 1.0, 8.0, 8.0, 1, None) == -1
    assert lib.bc_boxconv2d_forward_workspace(2, 3, 4, 8, 8) == 0          # small planes stay on chip
    assert lib.bc_boxconv2d_forward_workspace(2, 3, 4, 256, 512) > 0
    assert lib.bc_box_convolution_backward_workspace(2, 3, 4, 8, 8, 31) > 0
    assert lib.bc_boxconv2d_backward_workspace(2, 3, 4, 8, 8, 31) > 0
    assert lib.bc_boxconv2d_backward_workspace(2, 3, 4, 8, 8, 0) == 0


def test_header_compiles_as_plain_c_and_links(tmp_path):
    """The boundary is a C ABI: a C99 translation unit that includes the header and takes the
    address of entry points must compile with gcc and link against the library."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    assert gcc, "gcc is part of this image"
    src = tmp_path / "use_header.c"
    src.write_text(
        '#include "boxconv_b200.h"\n'
        "#include <stdio.h>\n"
        "int main(void) {\n"
        "    int (*f)(const float *, float *, int64_t, int, int, bc_stream_t) = bc_integral_image;\n"
        "    size_t need = bc_boxconv2d_forward_workspace(1, 1, 1, 2000, 2000);\n"
        '    printf("%d %s %d %d\\n", bc_version(), bc_status_string(BC_ERR_WORKSPACE), need > 0, f != 0);\n'
        "    return bc_integral_image(0, 0, 0, 4, 4, 0);   /* no planes: BC_OK without touching a device */\n"
        "}\n")
    libdir = os.path.join(PKG_DIR, "box_convolution")
    exe = tmp_path / "use_header"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-l:libboxconv_b200.so", "-Wl,-rpath," + libdir], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) >= 100 and out[-2:] == ["1", "1"]
