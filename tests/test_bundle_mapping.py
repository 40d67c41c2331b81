"""Bundles written under the reference's tensor names load into the weight objects the operators take:
stacked ``[blocks, ...]`` tensors are cut per block, Haiku's ``[in][out]`` triangle projections come out
``[out][in]``, head counts and widths are read from tensor shapes, int8 / intN / float16 payloads and delta
bundles decode as the reference's reader does (``shared/bundles/alphafold-fixture.js:122-267``,
``shared/af3/weights/weights.js:402-454,699-727``, ``shared/weights/dtype.js:212-406``,
``shared/bundles/delta-tensor-store.js``)."""
import numpy as np
import pytest

from localfold_b200 import bundle, synthetic as syn
from oracle import oracle
import bundle_writer as writer

BLOCKS = 3


def same_tree(a, b, path=""):
    assert type(a) is type(b) or (np.isscalar(a) and np.isscalar(b)), path
    if isinstance(a, dict):
        assert set(a) == set(b), f"{path}: {set(a) ^ set(b)}"
        for k in a:
            same_tree(a[k], b[k], f"{path}/{k}")
    elif isinstance(a, np.ndarray):
        assert a.size == b.size, path
        np.testing.assert_array_equal(a.reshape(-1), b.reshape(-1), err_msg=path)
    else:
        assert a == b, path


def af2_bundle_tensors(blocks_w, cm=32, cz=16, c=16, msa_heads=4, pair_heads=2):
    """Stacked Haiku-layout tensors + the manifest's parameter table for a list of Evoformer block weights."""
    tensors, parameters = {}, {}

    def put(module, leaf, per_block):
        name = f"evoformer_iteration/{module}//{leaf}"
        tensors[name] = np.stack(per_block, 0)
        parameters.setdefault(module, {})[leaf] = name

    def attention(root, key, heads, c_in):
        d = c_in // heads
        get = lambda f: [w[key]["attention"][f] for w in blocks_w]
        put(f"{root}/query_norm", "scale", get("queryNormScale"))
        put(f"{root}/query_norm", "offset", get("queryNormOffset"))
        for leaf, field in (("query_w", "queryWeight"), ("key_w", "keyWeight"), ("value_w", "valueWeight"), ("gating_w", "gatingWeight")):
            put(f"{root}/attention", leaf, [v.reshape(c_in, heads, d) for v in get(field)])
        put(f"{root}/attention", "gating_b", [v.reshape(heads, d) for v in get("gatingBias")])
        put(f"{root}/attention", "output_w", [v.reshape(heads, d, c_in) for v in get("outputWeight")])
        put(f"{root}/attention", "output_b", get("outputBias"))

    def transition(root, key):
        for module, leaf, field in (("input_layer_norm", "scale", "layerNormScale"), ("input_layer_norm", "offset", "layerNormOffset"),
                                    ("transition1", "weights", "firstWeight"), ("transition1", "bias", "firstBias"),
                                    ("transition2", "weights", "secondWeight"), ("transition2", "bias", "secondBias")):
            put(f"{root}/{module}", leaf, [w[key][field] for w in blocks_w])

    def triangle(root, key):
        t = lambda f: [np.ascontiguousarray(w[key][f].T) for w in blocks_w]       # the bundle stores [in][out]
        g = lambda f: [w[key][f] for w in blocks_w]
        put(f"{root}/layer_norm_input", "scale", g("layerNormInWeight")); put(f"{root}/layer_norm_input", "offset", g("layerNormInBias"))
        for module, role in (("left_projection", "AP"), ("left_gate", "AG"), ("right_projection", "BP"), ("right_gate", "BG")):
            put(f"{root}/{module}", "weights", t(f"linear{role}Weight")); put(f"{root}/{module}", "bias", g(f"linear{role}Bias"))
        put(f"{root}/center_layer_norm", "scale", g("layerNormOutWeight")); put(f"{root}/center_layer_norm", "offset", g("layerNormOutBias"))
        put(f"{root}/output_projection", "weights", t("linearZWeight")); put(f"{root}/output_projection", "bias", g("linearZBias"))
        put(f"{root}/gating_linear", "weights", t("linearGWeight")); put(f"{root}/gating_linear", "bias", g("linearGBias"))

    attention("msa_row_attention_with_pair_bias", "msaRowAttention", msa_heads, cm)
    row = "msa_row_attention_with_pair_bias"
    put(f"{row}/feat_2d_norm", "scale", [w["msaRowAttention"]["pairBias"]["layerNormScale"] for w in blocks_w])
    put(f"{row}/feat_2d_norm", "offset", [w["msaRowAttention"]["pairBias"]["layerNormOffset"] for w in blocks_w])
    put(row, "feat_2d_weights", [w["msaRowAttention"]["pairBias"]["projectionWeight"] for w in blocks_w])
    attention("msa_column_attention", "msaColumnAttention", msa_heads, cm)
    transition("msa_transition", "msaTransition")
    opm = "outer_product_mean"
    for module, leaf, field in ((f"{opm}/layer_norm_input", "scale", "layerNormScale"), (f"{opm}/layer_norm_input", "offset", "layerNormOffset"),
                                (f"{opm}/left_projection", "weights", "leftWeight"), (f"{opm}/left_projection", "bias", "leftBias"),
                                (f"{opm}/right_projection", "weights", "rightWeight"), (f"{opm}/right_projection", "bias", "rightBias"),
                                (opm, "output_w", "outputWeight"), (opm, "output_b", "outputBias")):
        put(module, leaf, [w["outerProductMean"][field] for w in blocks_w])
    triangle("triangle_multiplication_outgoing", "triangleMultiplicationOutgoing")
    triangle("triangle_multiplication_incoming", "triangleMultiplicationIncoming")
    for root, key in (("triangle_attention_starting_node", "triangleAttentionStarting"), ("triangle_attention_ending_node", "triangleAttentionEnding")):
        attention(root, key, pair_heads, cz)
        put(root, "feat_2d_weights", [w[key]["pairBias"]["projectionWeight"] for w in blocks_w])
    transition("pair_transition", "pairTransition")
    return tensors, parameters


def evoformer_blocks(seed, cm=32, cz=16, c=16, msa_heads=4, pair_heads=2):
    out = []
    for b in range(BLOCKS):
        *_, w = syn.af2_evoformer_block(seed + b, S=4, n=6, cm=cm, cz=cz, c_outer=8, c=c, msa_heads=msa_heads, pair_heads=pair_heads)
        out.append(w)
    return out


def test_af2_bundle_maps_to_block_weights(tmp_path):
    blocks_w = evoformer_blocks(50)
    tensors, parameters = af2_bundle_tensors(blocks_w)
    path = writer.write_bundle(str(tmp_path), tensors, shard_bytes=30000, dtypes={n: "float32" for n in tensors},
                               manifest_extra={"evoformerStack": {"parameters": parameters, "blocks": BLOCKS}})
    got = bundle.AlphaFoldFixture(bundle.FileTensorStore(path)).main_stack_weights(pair_channels=16)
    assert len(got) == BLOCKS
    for g, w in zip(got, blocks_w):
        same_tree(g, w)
    # and the loaded objects drive the oracle to the same block as the originals
    msa, pair, msa_mask, pair_mask, _ = syn.af2_evoformer_block(50, S=4, n=6, cm=32, cz=16, c_outer=8, c=16, msa_heads=4, pair_heads=2)
    a = oracle.af2_evoformer_block(msa, pair, msa_mask, pair_mask, got[1], 8, 16)
    b = oracle.af2_evoformer_block(msa, pair, msa_mask, pair_mask, blocks_w[1], 8, 16)
    np.testing.assert_array_equal(a[1], b[1])


def test_af2_bundle_int8_matches_the_quantised_values(tmp_path):
    """int8 at group 64 (what the AF2 export writes): each block's slice decodes to the whole tensor's values
    at those indices, whatever group the slice starts in."""
    blocks_w = evoformer_blocks(60)
    tensors, parameters = af2_bundle_tensors(blocks_w)
    kinds = {n: ("int8" if t.ndim >= 3 and t[0].size >= 64 else "float32") for n, t in tensors.items()}
    path = writer.write_bundle(str(tmp_path), tensors, dtypes=kinds,
                               manifest_extra={"evoformerStack": {"parameters": parameters, "blocks": BLOCKS}})
    store = bundle.FileTensorStore(path)
    got = bundle.AlphaFoldFixture(store).main_stack_weights(pair_channels=16)
    name = parameters["pair_transition/transition1"]["weights"]
    whole = store.tensor(name)
    assert store.record(name)["dtype"] == "int8"
    assert np.abs(whole - tensors[name]).max() <= np.abs(tensors[name]).max() / 127 * 0.51 + 1e-3
    for b in range(BLOCKS):
        np.testing.assert_array_equal(got[b]["pairTransition"]["firstWeight"].reshape(-1), whole[b].reshape(-1))
    # a range that starts and ends inside groups
    np.testing.assert_array_equal(store.tensor_range(name, 37, 301), whole.reshape(-1)[37:338])


def af3_bundle_tensors(blocks_w, root=bundle.PAIRFORMER):
    tensors = {}

    def put(leaf, per_block):
        tensors[f"{root}/{leaf}"] = np.stack(per_block, 0)

    for direction, key in (("outgoing", "triangleMultiplicationOutgoing"), ("incoming", "triangleMultiplicationIncoming")):
        t = f"triangle_multiplication_{direction}"
        for leaf, field in (("left_norm_input/scale", "leftNormInputScale"), ("left_norm_input/offset", "leftNormInputOffset"),
                            ("projection/weights", "projection"), ("gate/weights", "gate"), ("center_norm/scale", "centerNormScale"),
                            ("center_norm/offset", "centerNormOffset"), ("output_projection/weights", "outputProjection"),
                            ("gating_linear/weights", "gatingLinear")):
            put(f"{t}/{leaf}", [w[key][field] for w in blocks_w])
    for which in (1, 2):
        key, a = f"pairAttention{which}", f"pair_attention{which}"
        heads, dim = blocks_w[0][key]["heads"], blocks_w[0][key]["dimension"]
        put(f"{a}/act_norm/scale", [w[key]["actNormScale"] for w in blocks_w])
        put(f"{a}/act_norm/offset", [w[key]["actNormOffset"] for w in blocks_w])
        put(f"{a}/pair_bias_projection/weights", [w[key]["pairBiasProjection"] for w in blocks_w])
        for leaf, field in (("q_projection", "qProjection"), ("k_projection", "kProjection"), ("gating_query", "gatingQuery")):
            put(f"{a}/{leaf}/weights", [w[key][field].reshape(heads, dim, -1) for w in blocks_w])
        put(f"{a}/v_projection/weights", [w[key]["vProjection"].reshape(-1, heads, dim) for w in blocks_w])
        put(f"{a}/output_projection/weights", [w[key]["outputProjection"].reshape(heads, dim, -1) for w in blocks_w])
    for leaf, field in (("input_layer_norm/scale", "inputLayerNormScale"), ("input_layer_norm/offset", "inputLayerNormOffset"),
                        ("transition1/weights", "transition1"), ("transition2/weights", "transition2")):
        put(f"pair_transition/{leaf}", [w["pairTransition"][field] for w in blocks_w])
        put(f"single_transition/{leaf}", [w["singleTransition"][field] for w in blocks_w])
    put("single_pair_logits_norm/scale", [w["singlePairLogitsNormScale"] for w in blocks_w])
    put("single_pair_logits_norm/offset", [w["singlePairLogitsNormOffset"] for w in blocks_w])
    put("single_pair_logits_projection/weights", [w["singlePairLogitsProjection"] for w in blocks_w])
    sa = blocks_w[0]["singleAttention"]
    heads, dim = sa["heads"], sa["dimension"]
    put("single_attention_layer_norm/scale", [w["singleAttention"]["layerNormScale"] for w in blocks_w])
    put("single_attention_layer_norm/offset", [w["singleAttention"]["layerNormOffset"] for w in blocks_w])
    for leaf, field in (("q_projection", "qProjection"), ("k_projection", "kProjection"), ("v_projection", "vProjection"),
                        ("gating_query", "gatingQuery")):
        put(f"single_attention_{leaf}/weights", [w["singleAttention"][field].reshape(-1, heads, dim) for w in blocks_w])
    put("single_attention_q_projection/bias", [w["singleAttention"]["qBias"].reshape(heads, dim) for w in blocks_w])
    put("single_attention_transition2/weights", [w["singleAttention"]["outputProjection"] for w in blocks_w])
    return tensors


def test_af3_int5_bundle_maps_to_pairformer_blocks(tmp_path):
    """An int5 bundle under the AF3 exporter's names: widths and head counts come from tensor shapes, every
    block is one range of its stacked tensor, and the values are the int5 round trip of the originals."""
    _, _, _, _, blocks_w = syn.af3_pairformer(70, 8, cz=32, cs=48, blocks=BLOCKS, pair_heads=2, single_heads=4)
    tensors = af3_bundle_tensors(blocks_w)
    path = writer.write_bundle(str(tmp_path), tensors, shard_bytes=50000)
    store = bundle.FileTensorStore(path)
    assert store.record(f"{bundle.PAIRFORMER}/pair_transition/transition1/weights")["dtype"] == "int5"
    assert store.record(f"{bundle.PAIRFORMER}/pair_transition/input_layer_norm/scale")["dtype"] == "float32"
    got = bundle.pairformer_stack_weights(store)
    assert len(got) == BLOCKS
    for b, (g, w) in enumerate(zip(got, blocks_w)):
        assert (g["pairChannels"], g["singleChannels"]) == (32, 48)
        assert (g["pairAttention1"]["heads"], g["pairAttention1"]["dimension"]) == (2, 16)
        assert (g["singleAttention"]["heads"], g["singleAttention"]["dimension"]) == (4, 12)
        assert g["pairAttention1"]["gatingQueryBias"] is None
        np.testing.assert_array_equal(g["pairTransition"]["inputLayerNormScale"], w["pairTransition"]["inputLayerNormScale"])
        # a stacked tensor is quantised over its flat index, so a block's values are those of the whole tensor there
        name = f"{bundle.PAIRFORMER}/pair_transition/transition1/weights"
        payload, so, zo = writer.int5_payload(tensors[name])
        whole = bundle.decode_int5_host(payload, so, zo, tensors[name].size).reshape(tensors[name].shape)
        np.testing.assert_array_equal(g["pairTransition"]["transition1"], whole[b])
    # the loaded blocks run: oracle on loaded weights stays close to the oracle on the originals
    pair, single, pair_mask, seq_mask, _ = syn.af3_pairformer(70, 8, cz=32, cs=48, blocks=1, pair_heads=2, single_heads=4)
    a, _ = oracle.af3_pairformer_block(pair, single, pair_mask, seq_mask, got[0], True)
    b, _ = oracle.af3_pairformer_block(pair, single, pair_mask, seq_mask, blocks_w[0], True)
    assert oracle.relative_l2(a, b) < 0.2


def test_generic_packed_widths_and_float16(tmp_path):
    rng = np.random.default_rng(5)
    tensors = {"a/int3": rng.standard_normal((3, 200)).astype(np.float32), "a/half": rng.standard_normal(77).astype(np.float32),
               "a/int5": rng.standard_normal(333).astype(np.float32)}
    path = writer.write_bundle(str(tmp_path), tensors, dtypes={"a/int3": "int3", "a/half": "float16", "a/int5": "int5"})
    store = bundle.FileTensorStore(path)
    np.testing.assert_array_equal(store.tensor("a/half"), tensors["a/half"].astype(np.float16).astype(np.float32))
    whole = store.tensor("a/int3")
    span = tensors["a/int3"].max() - tensors["a/int3"].min()
    assert np.abs(whole - tensors["a/int3"]).max() <= span / 7 * 0.6 + 1e-2
    np.testing.assert_array_equal(store.tensor_range("a/int3", 130, 300), whole.reshape(-1)[130:430])
    np.testing.assert_array_equal(store.tensor_range("a/int5", 40, 200), store.tensor("a/int5")[40:240])
    with pytest.raises(ValueError):
        store.tensor_range("a/int5", 300, 100)


def test_delta_bundle(tmp_path):
    rng = np.random.default_rng(6)
    base = {"m/w": rng.standard_normal((4, 130)).astype(np.float32), "m/norm/scale": np.ones(8, np.float32),
            "t/only_base": rng.standard_normal(9).astype(np.float32), "geometry/table": np.arange(5, dtype=np.float32)}
    target = {"m/w": base["m/w"] + 0.01 * rng.standard_normal((4, 130)).astype(np.float32), "m/norm/scale": 1.5 * np.ones(8, np.float32)}
    base_path = writer.write_bundle(str(tmp_path / "base"), base, dtypes={"m/w": "int8", "geometry/table": "float32"})
    base_store = bundle.FileTensorStore(base_path)
    held = base_store.tensor("m/w").astype(np.float16).astype(np.float32)
    delta = {"m/w": target["m/w"] - held, "m/norm/scale": target["m/norm/scale"]}
    header = {"addTo": ["m/w"], "whole": ["m/norm/scale"], "absent": ["t/only_base"], "model": "model_3"}
    delta_path = writer.write_bundle(str(tmp_path / "delta"), delta, dtypes={"m/w": "int3", "m/norm/scale": "float32"},
                                     manifest_extra={"delta": header})
    store = bundle.DeltaTensorStore(base_store, bundle.FileTensorStore(delta_path))
    assert not store.has("t/only_base")
    with pytest.raises(KeyError):
        store.tensor("t/only_base")
    np.testing.assert_array_equal(store.tensor("m/norm/scale"), target["m/norm/scale"])
    np.testing.assert_array_equal(store.tensor("geometry/table"), base["geometry/table"])
    got = store.tensor("m/w")
    np.testing.assert_array_equal(got, held + bundle.FileTensorStore(delta_path).tensor("m/w"))
    assert np.abs(got - target["m/w"]).max() < np.abs(base_store.tensor("m/w") - target["m/w"]).max()
    assert stack_block(store, "m/w", 2).shape == (130,)


def stack_block(store, name, index):
    return bundle.stacked(store, name, index)
