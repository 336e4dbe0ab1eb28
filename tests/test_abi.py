"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
headers declare, and refuses to compute without a device (no CPU path)."""
import glob
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as ge
    if not os.path.exists(os.path.join(ge.PKG_DIR, "libiris_b200.so")):
        ge.build()
    return ge.load_package()


def declared_symbols():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
        names |= set(re.findall(r"\b(iris_[a-z0-9_]+)\s*\(", text))
    return names


def test_headers_and_binding_agree(pkg):
    from iris_c_b200.binding import SIGNATURES
    decl = declared_symbols()
    assert decl, "no declarations found"
    assert decl == set(SIGNATURES), (decl ^ set(SIGNATURES))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.Lib()
    for name in declared_symbols():
        assert hasattr(lib.cdll, name), name


def test_missing_library_fails_loudly(pkg, tmp_path):
    with pytest.raises(pkg.IrisB200Error):
        pkg.Lib(str(tmp_path / "libiris_b200.so"))


def test_no_cpu_fallback_without_device(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = pkg.Lib()
    assert lib.iris_dev_init() == 0
    assert lib.iris_dev_available() == 0
    assert lib.iris_dev_name() == b"none"
    assert lib.iris_dev_alloc(16) is None
    lib.iris_b200_clear_error()
    import numpy as np
    x = np.ones((2, 4), np.float32)
    lib.iris_softmax(x.ctypes.data, 2, 4)            # must not compute on the CPU
    assert (x == 1).all()
    assert lib.iris_b200_last_error() == 4           # IRIS_B200_ENODEV
    lib.iris_b200_clear_error()
    rc = lib.iris_b200_attention_ex(1, 128, 1, 1, 1, 128, 1, 1, 1, 1, 128, 1.0, 0, None, 0)
    assert rc == 4
    lib.iris_b200_clear_error()
    with pytest.raises(pkg.IrisB200Error):
        lib.init()


def test_product_sources_do_not_touch_the_oracle():
    """Only tests, smoke() and the CPU-baseline leg of bench.py may use oracle/."""
    for path in glob.glob(os.path.join(ROOT, "iris.c_b200", "**", "*"), recursive=True):
        if os.path.isfile(path) and path.endswith((".cu", ".cuh", ".h", ".py", ".c", "Makefile")):
            text = open(path, errors="ignore").read()
            assert "oracle" not in text.lower(), path


def test_c_host_program_builds_against_the_headers(tmp_path):
    """The drop-in boundary is C: a C11 program that includes only
    include/iris_dev.h compiles with gcc and links against the library. Run
    without a GPU it reports that there is no device (exit code 2)."""
    import path_cases as pc
    pkg = os.path.join(ROOT, "iris.c_b200")
    subprocess.check_call(["make", "-C", pkg, "example"], stdout=subprocess.DEVNULL)
    exe = os.path.join(pkg, "build", "block_attention")
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    pc.write_block_input(inp, pc.FLUX_SMALL)
    r = subprocess.run([exe, str(inp), str(out)], capture_output=True, text=True, timeout=120)
    assert r.returncode in (0, 2), (r.returncode, r.stdout, r.stderr)
    if r.returncode == 2:
        assert "no usable device" in r.stderr
