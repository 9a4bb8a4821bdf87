"""The C-ABI boundary without a GPU: the library loads, exports every symbol the header declares,
and the host-only entry points reproduce the reference's validation order and error text."""
import ctypes as C
import os
import re

import pytest

from tests.golden import reference_known_answers as ka

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "vqb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vqb_[a-z0-9_]+)\s*\(", text)) - {"vqb_draw_fn", "vqb_init_fn", "vqb_restart_fn"})


def test_library_exports_every_declared_symbol():
    from vq_b200 import _lib
    lib = _lib.load()
    names = _header_symbols()
    assert len(names) >= 35
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/vqb.h but not exported by libvqb.so"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table and header disagree"


def test_version_string():
    from vq_b200 import _lib
    assert b"sm_100a" in _lib.load().vqb_version()


def test_sq_fit_validation_order_and_text():
    from vq_b200 import _lib
    lib = _lib.load()
    step = C.c_float()
    assert lib.vqb_sq_fit(0.0, 1.0, 256, C.byref(step)) == 0
    assert step.value == pytest.approx(1.0 / 255.0, rel=1e-7)
    # src/sq.rs:51-68: max <= min is checked before the level count
    assert lib.vqb_sq_fit(1.0, 1.0, 1, C.byref(step)) == 2
    assert lib.vqb_last_error(None).decode() == ka.ERROR_TEXTS["sq_max_le_min"]
    assert lib.vqb_sq_fit(0.0, 1.0, 1, C.byref(step)) == 2
    assert lib.vqb_last_error(None).decode() == ka.ERROR_TEXTS["sq_levels_lt_2"]
    assert lib.vqb_sq_fit(0.0, 1.0, 257, C.byref(step)) == 2
    assert lib.vqb_last_error(None).decode() == ka.ERROR_TEXTS["sq_levels_gt_256"]


def test_bq_fit_validation():
    from vq_b200 import _lib
    lib = _lib.load()
    assert lib.vqb_bq_fit(0.0, 0, 1) == 0
    assert lib.vqb_bq_fit(0.0, 1, 1) == 2
    assert lib.vqb_last_error(None).decode() == ka.ERROR_TEXTS["bq_low_ge_high"]


def test_python_mirror_raises_reference_errors():
    import vq_b200 as vq
    with pytest.raises(vq.InvalidParameter) as e:
        vq.ScalarQuantizer.fit(2.0, 1.0, 16)
    assert str(e.value) == ka.ERROR_TEXTS["sq_max_le_min"]
    with pytest.raises(vq.InvalidParameter) as e:
        vq.BinaryQuantizer.fit(0.0, 5, 5)
    assert str(e.value) == ka.ERROR_TEXTS["bq_low_ge_high"]
    q = vq.ScalarQuantizer.fit(-1.0, 1.0, 5)
    assert (q.min, q.max, q.levels, q.step) == (-1.0, 1.0, 5, 0.5)


def test_null_handles_are_rejected_not_crashed():
    from vq_b200 import _lib
    lib = _lib.load()
    assert lib.vqb_ctx_synchronize(None) == 90
    assert lib.vqb_pq_quantize(None, None, 0, 0, None, None) == 90
    assert lib.vqb_ctx_destroy(None) == 0


def test_no_cpu_fallback_without_gpu():
    """Without a CUDA device the context cannot be created: the product has no CPU path."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from vq_b200 import _lib
    lib = _lib.load()
    h = C.c_void_p()
    rc = lib.vqb_ctx_create(0, C.byref(h))
    assert rc == 102 and not h.value
    assert b"CUDA" in lib.vqb_last_error(None) or b"device" in lib.vqb_last_error(None)
    import vq_b200 as vq
    with pytest.raises(vq.BackendError):
        vq.ProductQuantizer.fit([[0.0, 1.0], [1.0, 0.0]], 1, 1, 1, vq.Distance.Euclidean, 0)


def test_product_package_does_not_import_the_oracle():
    import subprocess
    import sys
    code = "import sys; import vq_b200, vq_b200.distributed, vq_b200.synth; print(any(m == 'oracle' or m.startswith('oracle.') for m in sys.modules))"
    out = subprocess.check_output([sys.executable, "-c", code], cwd=ROOT).decode().strip()
    assert out == "False"
    for dirpath, _d, files in os.walk(os.path.join(ROOT, "vq_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().lower(), f
