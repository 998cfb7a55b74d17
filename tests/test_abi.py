"""CPU checks of the drop-in boundary: the shared library loads without a GPU driver,
exports every entry point include/lutamm.h declares, its parameter blocks have the
reference's field layout, and it refuses to compute without a device."""
import ctypes
import os
import re

import pytest

import pim_dl_asplos_b200 as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "lutamm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lutamm_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_list_agree():
    assert _declared() == sorted(P.ABI_SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = P.load_library()
    for name in _declared():
        assert hasattr(lib, name), f"{name} is declared in include/lutamm.h but not exported"
    assert b"sm_100a" in lib.lutamm_version()


def test_parameter_blocks_have_the_reference_layout():
    # src/host/defines.h:12-24 is 8 x uint32; :26-50 is 4 x uint32, 2 x float, 12 x uint32
    assert ctypes.sizeof(P.IndexCalcParams) == 32
    assert ctypes.sizeof(P.LUTParams) == 72
    assert P.LUTParams.scale.offset == 16 and P.LUTParams.bias.offset == 20
    assert P.LUTParams.lut_load_type.offset == 60


def test_no_device_means_a_loud_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(P.LutAmmError) as e:
        P.LutAmmContext(0)
    assert e.value.code == P.ECUDA


def test_null_context_is_rejected():
    lib = P.load_library()
    assert lib.lutamm_amm(None, 0, None, None, 1, 0) == P.EINVAL
    assert lib.lutamm_sync(None) == P.EINVAL
    assert lib.lutamm_launch_count(None) == 0
