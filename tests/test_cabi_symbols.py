"""CPU-side checks of the boundary: the shared library loads without a GPU and exports every entry point
declared in include/*.h; the drop-in module exposes the reference's names."""
import os
import re

import numpy as np
import pytest

import hetuctr_b200 as hb
from hetuctr_b200 import build as hbuild

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    hbuild.build()
    return hb.lib()


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hctr_[a-z0-9_]+)\s*\(", text)))


@pytest.mark.parametrize("header", ["hctr_kernels.h", "hctr_table.h"])
def test_every_declared_entry_point_is_exported(built, header):
    names = _declared(header)
    assert len(names) >= 10
    for n in names:
        assert hasattr(built, n), f"{n} declared in {header} but not exported"


def test_module_surface_matches_reference():
    m = hb.hetuCTR
    for name in ("HetuTable", "Initializer", "InitType", "seed", "_waittype"):
        assert hasattr(m, name)
    assert {"Zero", "Normal", "TruncatedNormal", "Uniform"} <= set(m.InitType.__members__)
    for meth in ("preprocess", "push_pull", "async_preprocess", "async_push_pull", "debug", "__repr__"):
        assert hasattr(m.HetuTable, meth)
    m.seed(3)
    m.Initializer(m.InitType.Normal, 0, 1)


def test_constructor_requires_every_keyword_and_contiguous_arrays():
    m = hb.hetuCTR
    init = m.Initializer(m.InitType.Zero, 0, 0)
    with pytest.raises(TypeError):  # learning_rate has no default (reference csrc/pybind/pybind.cu:63-69)
        m.HetuTable(rank=0, nrank=1, device_id=0, ip="127.0.0.1", port=1, pull_bound=0, push_bound=0, init=init,
                    length=8, width=4, root_arr=np.zeros(8), storage_arr=np.arange(8), verbose=0)
    with pytest.raises(RuntimeError, match="Array not continuous in C"):
        m.HetuTable(rank=0, nrank=1, device_id=0, ip="127.0.0.1", port=1, pull_bound=0, push_bound=0, init=init,
                    length=8, width=4, root_arr=np.zeros(16, dtype=np.uint8)[::2], storage_arr=np.arange(8),
                    learning_rate=0.1, verbose=0)


def test_no_device_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        hb.Table(0, 1, 0, "127.0.0.1", 1, 8, 4, 0, 0, np.zeros(8), np.arange(8))


def test_scan_scratch_size_helper(built):
    assert built.hctr_scan_scratch_words(0) >= 1
    assert built.hctr_scan_scratch_words(1 << 20) >= (1 << 20) // 4096
