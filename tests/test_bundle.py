"""int5 bundle writer/reader against the vectors made by the reference's own quantiser."""
import os

import numpy as np

from localfold_b200 import bundle
import bundle_writer as writer
from oracle import oracle


def test_quantiser_and_packer_reproduce_the_reference(golden_dir):
    d = np.load(os.path.join(golden_dir, "int5-vectors.npz"))
    count = len([k for k in d.files if k.startswith("values_")])
    for i in range(count):
        codes, scales, zeros = writer.int5_encode(d[f"values_{i}"])
        np.testing.assert_array_equal(writer.int5_bytes(codes).reshape(-1), d[f"packed_{i}"])
        np.testing.assert_array_equal(scales.view(np.uint16), d[f"scales_{i}"].view(np.uint16))
        np.testing.assert_array_equal(zeros.view(np.uint16), d[f"zeros_{i}"].view(np.uint16))
        payload, so, zo = writer.int5_payload(d[f"values_{i}"])
        np.testing.assert_array_equal(bundle.decode_int5_host(payload, so, zo, d[f"values_{i}"].size), d[f"decoded_{i}"])
        np.testing.assert_array_equal(oracle.int5_decode(d[f"packed_{i}"], scales, zeros, d[f"values_{i}"].size), d[f"decoded_{i}"])


def test_bundle_round_trip(tmp_path):
    rng = np.random.default_rng(3)
    tensors = {
        "trunk/pairformer/triangle_multiplication_outgoing/projection": rng.standard_normal((2, 16, 32)).astype(np.float32),
        "trunk/pairformer/triangle_multiplication_outgoing/left_norm_input/scale": np.ones((2, 16), np.float32),
        "trunk/pairformer/pair_transition/transition1": rng.standard_normal((2, 16, 128)).astype(np.float32) * 0.3,
        "odd/size_tensor": rng.standard_normal(77).astype(np.float32),
        "head/output_b": rng.standard_normal(5).astype(np.float32),
    }
    path = writer.write_bundle(str(tmp_path), tensors, shard_bytes=2000)
    store = bundle.FileTensorStore(path)
    assert set(store.names()) == set(tensors)
    assert len({store.manifest["tensors"][n]["file"] for n in tensors}) >= 2      # several shards
    for name, value in tensors.items():
        got = store.read(name)
        record = store.manifest["tensors"][name]
        assert record["byteOffset"] % 4 == 0
        if record["dtype"] == "float32":
            np.testing.assert_array_equal(got, value)
        else:
            payload, so, zo = writer.int5_payload(value)
            np.testing.assert_array_equal(got.reshape(-1), bundle.decode_int5_host(payload, so, zo, value.size))
            span = value.max() - value.min()
            assert np.abs(got - value).max() <= span / 31 * 0.51 + 1e-2
    assert store.manifest["tensors"]["head/output_b"]["dtype"] == "float32"
    assert store.manifest["tensors"]["odd/size_tensor"]["dtype"] == "int5"
