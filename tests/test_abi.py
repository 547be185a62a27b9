"""The C ABI without a GPU: the library loads, exports every symbol the header declares, the
shims export the reference's four names, and argument validation answers before any launch."""
import ctypes
import os
import re

import pytest

from spion_b200 import _lib
from spion_b200.attention import Attention

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "spion_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(spion_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(_lib.lib, n), n
        assert n in _lib.SIGNATURES, f"{n} declared in the header but not bound in _lib.SIGNATURES"
    for n in _lib.SIGNATURES:
        assert n in names, f"{n} bound but not declared in include/spion_b200.h"


@pytest.mark.parametrize("loader", ["_cuda_compile_module", "_cuda_mask_compile_module",
                                    "_blockcuda_compile_module", "_blockcuda_mask_compile_module"])
def test_shims_export_reference_names(loader):
    cpp = getattr(Attention, loader)()
    for n in ("init", "attn_forward", "attn_backward", "destroy"):
        assert hasattr(cpp, n)


def test_status_strings_and_version():
    assert _lib.lib.spion_version() >= 100
    assert _lib.lib.spion_status_string(0) == b"ok"
    assert b"shape" in _lib.lib.spion_status_string(-2)


def test_argument_validation_needs_no_gpu():
    L = _lib.lib
    dummy = ctypes.c_void_p(256)
    assert L.spion_set_stream(None, None) == -1
    assert L.spion_set_engine(None, 0) == -1
    assert L.spion_pattern_nnzb(None) == -1
    assert L.spion_block_attn_forward(None, *([dummy] * 9), 0) == -1
    assert L.spion_attn_forward_ex(None, *([dummy] * 7)) == -1
    assert L.spion_expand_csr(None, None, 4, 32, 4, 1, None, None, None, None) == -1
    assert L.spion_expand_csr(dummy, dummy, 100000, 32, 4, 1, dummy, dummy, dummy, None) == -2
    # seq_len not a multiple of block_size is refused, not truncated (the reference does int(L / bs))
    args = [dummy] * 11 + [None, None]
    assert L.spion_discover_pattern(dummy, 100, 32, 0, 31, 0, 0.9, *args) == -2
    assert L.spion_discover_pattern(dummy, 128, 32, 0, 30, 0, 0.9, *args) == -1      # even filter
    assert L.spion_discover_pattern(dummy, 128, 32, 0, 31, 0, 1.5, *args) == -1      # quantile out of range
    assert L.spion_mean_attention_map(dummy, 1, 1, 100, 0, dummy, None) == -2
    with pytest.raises(_lib.SpionError):
        _lib.check(-2, "x")


def test_create_rejects_bad_shapes_without_touching_cuda():
    L = _lib.lib
    assert not L.spion_create(_lib.KIND_BLOCK, 32, 100, 4, 32, _lib.F32, -1)     # L % bs
    assert not L.spion_create(9, 32, 128, 4, 32, _lib.F32, -1)                    # kind
    assert not L.spion_create(_lib.KIND_BLOCK, 32, 128, 4, 32, 7, -1)             # dtype
    assert not L.spion_create(_lib.KIND_BLOCK, 0, 128, 4, 32, _lib.F32, -1)


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the public header must compile as C99 on its own, and a C translation unit that
    takes the address of every declared entry point must link against the library."""
    import re
    import shutil
    import subprocess
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = os.path.join(root, "include", "spion_b200.h")
    r = subprocess.run([cc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-x", "c", header],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout
    names = sorted(set(re.findall(r"\b(spion_[a-z0-9_]+)\s*\(", open(header).read())))
    src = tmp_path / "link_all.c"
    body = "\n".join(f"  p[{i}] = (void*)&{n};" for i, n in enumerate(names))
    src.write_text('#include "spion_b200.h"\n#include <stdio.h>\nint main(void) {\n  void* p[%d];\n%s\n'
                   '  printf("%%p\\n", p[0]);\n  return 0;\n}\n' % (len(names), body))
    libdir = os.path.join(root, "spion_b200", "lib")
    if not os.path.exists(os.path.join(libdir, "libspion_b200.so")):
        pytest.skip("library not built")
    exe = tmp_path / "link_all"
    r = subprocess.run([cc, "-std=c99", "-I", os.path.join(root, "include"), str(src), "-o", str(exe), "-L", libdir,
                        "-lspion_b200", "-Wl,-rpath," + libdir], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True)
    assert r.returncode == 0, r.stdout
