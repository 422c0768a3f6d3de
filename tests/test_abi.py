"""CPU checks of the boundary: the shared library loads, exports every symbol the header
declares, its host-only helpers agree with the oracle, and it fails loudly without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle
from hippo_leap_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_text():
    text = ""
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            text += open(os.path.join(inc, f)).read()
    return text


def test_library_exports_every_declared_symbol():
    declared = set(re.findall(r"\b(hl_(?:b200|backend|dense)_\w+)\s*\(", _header_text()))
    assert len(declared) >= 18
    lib = C.CDLL(_lib.LIB_PATH)
    missing = [s for s in sorted(declared) if not hasattr(lib, s)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_binding_table_covers_the_header():
    from hippo_leap_b200 import backend
    declared = set(re.findall(r"\b(hl_b200_\w+)\s*\(", _header_text()))
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    from hippo_leap_b200 import dense
    declared_b = set(re.findall(r"\b(hl_backend_\w+)\s*\(", _header_text()))
    assert declared_b == set(backend.BACKEND_SYMBOLS), declared_b ^ set(backend.BACKEND_SYMBOLS)
    declared_d = set(re.findall(r"\b(hl_dense_\w+)\s*\(", _header_text()))
    assert declared_d == set(dense.DENSE_SYMBOLS), declared_d ^ set(dense.DENSE_SYMBOLS)
    _lib.load()
    backend._lib()
    dense._lib()


def test_status_and_enum_values_match_header():
    h = _header_text()
    for name in ("HL_OK", "HL_ERR_ARG", "HL_ERR_CAPACITY", "HL_ERR_ALIGN", "HL_ERR_CUDA",
                 "HL_ERR_TIMEOUT", "HL_ERR_BOUNDS", "HL_ERR_UNSUPPORTED", "HL_DTYPE_F32",
                 "HL_DTYPE_F16", "HL_ROPE_INTERLEAVED", "HL_ROPE_SPLIT_HALF"):
        m = re.search(rf"\b{name}\s*=\s*(\d+)", h)
        assert m, name
        assert int(m.group(1)) == getattr(_lib, name), name


@pytest.mark.parametrize("base,dim", [(1e4, 64), (5e5, 64), (1e6, 128), (5e5, 128)])
def test_theta_table_bit_identical_to_oracle(base, dim):
    import hippo_leap_b200 as hl
    assert np.array_equal(hl.theta_table(dim, base), oracle.theta_table(dim, base))


def test_llama3_scaling_rule():
    import hippo_leap_b200 as hl
    th = hl.theta_table(64, 5e5)
    sc = hl.theta_llama3_scale(th, 32.0, 1.0, 4.0, 8192)
    wl = 2 * np.pi / th.astype(np.float64)
    hi, lo = 8192 / 4.0, 8192 / 1.0
    for i in range(32):
        if wl[i] < hi:
            assert sc[i] == th[i]
        elif wl[i] > lo:
            assert sc[i] == np.float32(th[i].astype(np.float64) / 32.0)
        else:
            s = (8192 / wl[i] - 1.0) / 3.0
            assert sc[i] == np.float32((1 - s) * th[i] / 32.0 + s * th[i])
    assert (sc[:8] == th[:8]).all() and (sc[-4:] < th[-4:]).all()


def test_no_gpu_means_loud_failure_not_fallback():
    import torch

    import hippo_leap_b200 as hl
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the loud-failure path is for CPU-only hosts")
    with pytest.raises(hl.HlError):
        hl.Context(0)


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "hippo_leap_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".nim")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src, f
                assert "liboracle" not in src and "tensor_ref" not in src, f


def test_struct_layouts_match_the_headers(tmp_path):
    """Every struct that crosses the C ABI: field offsets and sizes as gcc lays out the header's definition
    against the ctypes mirror the tests and the benchmark use."""
    import shutil
    import subprocess
    from hippo_leap_b200 import backend, dense
    gcc = shutil.which("gcc") or "/usr/bin/gcc"
    pairs = {"hl_attn_shape": _lib.AttnShapeC, "hl_view": _lib.ViewC, "hl_hparams": backend.HParamsC,
             "hl_standin_weights": backend.WeightsC, "hl_kv_cache": backend.KvCacheC,
             "hl_dense_hparams": dense.DenseHParamsC, "hl_dense_weights": dense.DenseWeightsC}
    inc = os.path.join(os.path.dirname(__file__), "..", "include")
    lines = ['#include <stddef.h>', '#include <stdio.h>', '#include "hl_b200.h"', '#include "hl_backend.h"', 'int main(void) {']
    for cname, cls in pairs.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'  printf("{cname} {fname} %zu\\n", offsetof({cname}, {fname}));')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-I", inc, str(src), "-o", str(exe)], check=True)
    got = {}
    for ln in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines():
        c, f, v = ln.split()
        got[(c, f)] = int(v)
    for cname, cls in pairs.items():
        assert got[(cname, "size")] == C.sizeof(cls), cname
        for fname, _ in cls._fields_:
            assert got[(cname, fname)] == getattr(cls, fname).offset, (cname, fname)
