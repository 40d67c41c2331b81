"""The shared library loads without a GPU and exports every entry point the header declares."""
import ctypes
import os
import re

from localfold_b200 import _native as nat, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "localfold_pairstack.h")).read()
    return sorted(set(re.findall(r"LF_API\s+[\w\s\*]+?\b(lf_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    build.build()
    lib = ctypes.CDLL(nat.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert getattr(lib, name) is not None, name
    assert set(names) == set(nat.EXPORTS)


def test_version_and_no_device_behaviour():
    lib = nat.load()
    assert b"sm_100a" in lib.lf_version()
    handle = ctypes.c_void_p()
    # without a usable CUDA device the context is refused: there is no CPU path to fall back to
    import torch
    if not torch.cuda.is_available():
        assert lib.lf_context_create(0, None, ctypes.byref(handle)) != nat.LF_OK
        assert not handle.value


def test_host_side_validation_matches_the_reference_messages():
    import numpy as np
    import pytest
    from localfold_b200.operators import RangeError, error_metrics, validate_triangle_input
    from localfold_b200 import synthetic as syn
    pair, mask, weights = syn.af2_pair_block(0, 4, 16, 8, 2)
    w = weights[0]["triangleMultiplicationOutgoing"]
    good = {"shape": {"length": 4, "cZ": 16, "cHidden": 8}, "z": pair, "mask": mask, "weights": w}
    validate_triangle_input(good)
    with pytest.raises(RangeError, match="z has 255 values; expected 256"):
        validate_triangle_input(dict(good, z=pair.reshape(-1)[:-1]))
    with pytest.raises(RangeError, match="linearZBias has"):
        validate_triangle_input(dict(good, weights=dict(w, linearZBias=w["linearZBias"][:-1])))
    with pytest.raises(RangeError, match="length must be a positive safe integer"):
        validate_triangle_input(dict(good, shape={"length": 0, "cZ": 16, "cHidden": 8}))
    with pytest.raises(RangeError, match="epsilon must be finite and positive"):
        validate_triangle_input(dict(good, epsilon=-1.0))
    m = error_metrics(np.array([1.0, 2.0]), np.array([1.0, 4.0]))
    assert m["maxAbsoluteError"] == 2.0 and m["meanAbsoluteError"] == 1.0
    with pytest.raises(RangeError):
        error_metrics(np.zeros(0), np.zeros(0))
