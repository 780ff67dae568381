"""CPU-only checks of the C-ABI boundary: the library loads, exports every
symbol include/ugb200.h declares, and fails loudly without a GPU."""
import ctypes as C
import subprocess

import pytest

from ug_b200 import _lib


def test_every_declared_symbol_is_exported():
    protos = _lib.parse_header()
    assert len(protos) >= 30
    lib = C.CDLL(_lib.LIB_PATH)
    missing = [n for n in protos if not hasattr(lib, n)]
    assert not missing, missing


def test_no_undeclared_ugb_exports():
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True,
                         text=True, check=True).stdout
    exported = {l.split()[-1] for l in out.splitlines() if " T ugb_" in l}
    assert exported == set(_lib.parse_header())


def test_use_grid_is_true():
    assert _lib.lib.ugb_use_grid() == 1


def test_device_create_fails_loudly_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import ug_b200
    with pytest.raises(ug_b200.UgError) as e:
        ug_b200.Device(0)
    assert e.value.code != 0 and e.value.msg


def test_null_handles_are_rejected():
    lib = _lib.lib
    assert lib.ugb_sync(None) != 0
    assert lib.ugb_free(None) != 0
    assert lib.ugb_softmax(None, None, None, 1, 1) != 0
    assert lib.ugb_matmul(None, None, None, None, 1, 1, 1, 1, 2, None, None, 0, None, None, 0) != 0


def test_host_layer_library_exports_its_header():
    from ug_b200 import lazy
    protos = _lib.parse_header(lazy.HOST_HEADER)
    assert len(protos) >= 40
    lib = C.CDLL(lazy.HOST_LIB)
    assert not [n for n in protos if not hasattr(lib, n)]
