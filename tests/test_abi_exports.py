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


def test_python_mirror_of_every_descriptor_matches_the_header(tmp_path):
    """Sizes and field offsets of the ctypes structures against the C header, as a C compiler lays it out: a field
    added on one side only would shift every pointer after it."""
    import subprocess
    pairs = {"lf_result": nat.Result, "lf_weight_dims": nat.WeightDims, "lf_triangle_desc": nat.TriangleDesc,
             "lf_attention_desc": nat.AttentionDesc, "lf_transition_desc": nat.TransitionDesc, "lf_opm_desc": nat.OpmDesc,
             "lf_single_attention_desc": nat.SingleAttentionDesc, "lf_msa_attention_desc": nat.MsaAttentionDesc,
             "lf_global_attention_desc": nat.GlobalAttentionDesc, "lf_distogram_desc": nat.DistogramDesc,
             "lf_pair_block_weights": nat.PairBlockWeights, "lf_pair_stack_desc": nat.PairStackDesc,
             "lf_shard_step_desc": nat.ShardStepDesc, "lf_encoded_tensor": nat.EncodedTensorDesc,
             "lf_shard_peers": nat.ShardPeers}
    lines = ["#include <stdio.h>", "#include <stddef.h>", '#include "localfold_pairstack.h"', "int main(void) {"]
    for c_name, mirror in pairs.items():
        lines.append(f'  printf("{c_name} size %zu\\n", sizeof({c_name}));')
        for field, _ in mirror._fields_:
            lines.append(f'  printf("{c_name} {field} %zu\\n", offsetof({c_name}, {field}));')
    lines += ["  return 0;", "}"]
    source = tmp_path / "layout.c"
    source.write_text("\n".join(lines))
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), "-o", str(binary), str(source)], check=True)
    out = subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.splitlines()
    assert len(out) > 150
    for line in out:
        c_name, field, value = line.split()
        mirror = pairs[c_name]
        want = ctypes.sizeof(mirror) if field == "size" else getattr(mirror, field).offset
        assert int(value) == want, line
