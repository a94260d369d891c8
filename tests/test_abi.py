"""The C-ABI library loads, exports every symbol the header declares, and validates arguments on the host
(no kernel is launched here)."""

import ctypes
import os
import re

import pytest

from miniworld_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()  # no-op when the library is newer than its sources
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_trimul.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_(?:trimul|transition)_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    names = _declared_symbols()
    assert len(names) >= 13
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_version_and_strerror(lib):
    assert lib.b200_trimul_version() >= 100
    assert "128" in _lib.strerror(-3)
    assert _lib.strerror(0) == "ok"
    assert "gave up" in _lib.strerror(102)


def test_workspace_size_and_layout(lib):
    out = ctypes.c_size_t(0)
    assert lib.b200_trimul_workspace_bytes(1, 384, 128, 128, 1, ctypes.byref(out)) == 0
    tensor = 384 * 384 * 128 * 2
    assert out.value >= 3 * tensor
    arr = (ctypes.c_size_t * 5)()
    assert lib.b200_trimul_workspace_layout(1, 384, arr) == 0
    offs = list(arr)
    assert offs[0] == 0 and all(o % 1024 == 0 for o in offs)
    assert offs[2] - offs[1] == lib.b200_trimul_packed_bytes()
    assert offs[3] - offs[2] == tensor and offs[4] - offs[3] == tensor


@pytest.mark.parametrize(
    "args,code",
    [
        ((1, 384, 64, 64, 1), -3),    # d_pair 64 needs 128 contracted channels in total
        ((1, 384, 64, 128, 0), -3),   # ... so 64 per direction when bidirectional
        ((1, 384, 32, 128, 1), -3),   # d_pair not 64 or 128
        ((1, 384, 128, 256, 1), -3),  # d_hidden != 128
        ((1, 100, 128, 128, 1), -3),  # N not a multiple of 8
        ((0, 384, 128, 128, 1), -2),  # B < 1
        ((1, 384, 128, 128, 3), -2),  # direction
    ],
)
def test_argument_validation(lib, args, code):
    out = ctypes.c_size_t(0)
    assert lib.b200_trimul_workspace_bytes(*args, ctypes.byref(out)) == code


def test_null_pointers_are_rejected_before_any_cuda_call(lib):
    assert lib.b200_trimul_workspace_bytes(1, 384, 128, 128, 1, None) == -1
    rc = lib.b200_trimul_forward(*([None] * 7), 0, *([None] * 4), None, None, None, None, None, 0, 1, 384, 128, 128, 1,
                                 1e-5, 1e-5, 1, None)
    assert rc == -1
    assert lib.b200_trimul_contract(None, None, None, 1, 384, 0, 384, 1, None, None) == -1


def test_backward_entry_points_validate_before_any_cuda_call(lib):
    out = ctypes.c_size_t(0)
    assert lib.b200_trimul_backward_workspace_bytes(1, 384, 1, ctypes.byref(out)) == 0
    uni = out.value
    assert lib.b200_trimul_backward_workspace_bytes(1, 384, 0, ctypes.byref(out)) == 0
    plane = 384 * 384 * 128 * 2
    assert uni >= 4 * plane and out.value >= uni + 4 * plane  # the bidirectional module keeps four more tensors
    assert lib.b200_trimul_backward_workspace_bytes(1, 100, 1, ctypes.byref(out)) == -3  # N not a multiple of 8
    assert lib.b200_trimul_backward_workspace_bytes(1, 384, 5, ctypes.byref(out)) == -2
    assert lib.b200_trimul_backward_workspace_bytes(1, 384, 1, None) == -1
    arr = (ctypes.c_size_t * 18)()
    assert lib.b200_trimul_backward_workspace_layout(1, 384, 0, arr) == 0
    offs = list(arr)
    assert offs[0] == 0 and all(o % 1024 == 0 for o in offs) and offs == sorted(offs)
    assert lib.b200_trimul_backward_workspace_bytes(1, 384, 0, ctypes.byref(out)) == 0 and offs[17] == out.value
    rc = lib.b200_trimul_backward(*([None] * 8), 0, *([None] * 4), *([None] * 5), *([None] * 2), *([None] * 4), None, 0,
                                  1, 384, 128, 128, 1, 1e-5, 1e-5, 1, None)
    assert rc == -1
    assert lib.b200_trimul_contract_backward(None, None, None, None, None, 1, 384, 1, None, None) == -1
