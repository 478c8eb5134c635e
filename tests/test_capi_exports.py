"""The C-ABI library loads without a GPU and exports exactly what include/q4b200.h declares."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib():
    from qwen38_metal_b200 import build, capi

    build.build()
    return capi.load()


def declared_functions(header="q4b200.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q4b_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions() + declared_functions("q4b_weights.h")
    assert len(names) >= 60
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in q4b200.h but not exported"


def test_python_prototypes_cover_the_header():
    from qwen38_metal_b200 import capi

    assert sorted(capi.EXPORTS) == declared_functions()
    assert sorted(capi.WEIGHTS_EXPORTS) == declared_functions("q4b_weights.h")


def test_job_struct_layout_matches_header():
    from qwen38_metal_b200 import capi

    assert C.sizeof(capi.Job) == 48
    assert C.sizeof(capi.TensorInfo) == 104 and C.sizeof(capi.Q4Matrix) == 3 * 104 + 32
    assert capi.Job.weight_offset.offset == 16 and capi.Job.output_rows.offset == 40


def test_status_names(lib):
    from qwen38_metal_b200 import capi

    for code, name in capi.STATUS_NAMES.items():
        assert lib.q4b_status_name(code).decode() == name


def test_missing_device_is_reported_not_hidden(lib):
    """On a machine without a GPU the runtime refuses to start: there is no CPU path to fall back to."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from qwen38_metal_b200.runtime import CudaRuntime, Q4RuntimeError

    with pytest.raises(Q4RuntimeError) as err:
        CudaRuntime(0)
    assert err.value.kind == "NoDevice"


def test_null_handle_is_an_error_not_a_crash(lib):
    n = C.c_uint32()
    assert lib.q4b_shard_count(None, C.byref(n)) == 13  # InvalidArgument
    assert b"null" in lib.q4b_last_error()
