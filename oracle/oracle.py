"""ctypes driver for the CPU oracle (``pairstack_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline leg of the benchmark import
this module; the product package never does.  Every function takes and returns
float32 numpy arrays in the reference's layouts and uses the reference's own
weight-object field names (``webgpu/kernels/triangle/weights.js:4-10``,
``webgpu/kernels/attention.js:64-80``, ``webgpu/kernels/transition.js:477-480``,
``webgpu/kernels/outer-product-mean.js:72-75``,
``shared/af3/weights/weights.js:402-454,699-727``).

Block-level functions compose the operators in the order the reference does
(``webgpu/af2/evoformer/block.js:1546-1612``, ``cpu/af3/trunk/pairformer.js:495-542``)
with float32 residual adds.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libpairstack_oracle.so")

TRIANGLE_WEIGHT_ORDER = (
    "layerNormInWeight", "layerNormInBias", "linearAPWeight", "linearAPBias",
    "linearAGWeight", "linearAGBias", "linearBPWeight", "linearBPBias",
    "linearBGWeight", "linearBGBias", "layerNormOutWeight", "layerNormOutBias",
    "linearZWeight", "linearZBias", "linearGWeight", "linearGBias",
)


def build(force: bool = False) -> str:
    """Compile the C restatement into ``oracle/_ref`` (gcc + OpenMP)."""
    src = os.path.join(_HERE, "pairstack_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.orc_max_threads.restype = ctypes.c_int
    return _lib


def set_threads(n: int) -> None:
    lib().orc_set_threads(ctypes.c_int(int(n)))


def max_threads() -> int:
    return int(lib().orc_max_threads())


_FP = ctypes.POINTER(ctypes.c_float)


def _f(a):
    """float32 C-contiguous view (or None) plus its pointer."""
    if a is None:
        return None, ctypes.cast(None, _FP)
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_FP)


def _i(v):
    return ctypes.c_int(int(v))


def _l(v):
    return ctypes.c_int64(int(v))


def _d(v):
    return ctypes.c_double(float(v))


def layer_norm(x, scale, offset, eps=1e-5, fast=False):
    x, px = _f(x)
    ch = x.shape[-1]
    rows = x.size // ch
    out = np.empty_like(x)
    s_keep, ps = _f(scale)
    o_keep, po = _f(offset)
    lib().orc_layer_norm(px, _l(rows), _i(ch), ps, po, _d(eps), _i(1 if fast else 0),
                         out.ctypes.data_as(_FP))
    return out


def linear(x, w, bias=None, transposed=False):
    x, px = _f(x)
    w, pw = _f(w)
    b, pb = _f(bias)
    if transposed:
        cout, cin = w.shape
    else:
        cin, cout = w.shape
    rows = x.size // cin
    out = np.empty((rows, cout), np.float32)
    lib().orc_linear(px, _l(rows), _i(cin), _i(cout), pw, pb, _i(1 if transposed else 0),
                     out.ctypes.data_as(_FP))
    return out.reshape(x.shape[:-1] + (cout,))


def trimul_af2(z, mask, weights, c_hidden, eps=1e-5, incoming=False):
    """``triangleMultiplicationOutgoingReference`` and its incoming twin."""
    z, pz = _f(z)
    n, _, cz = z.shape
    m, pm = _f(mask)
    keep = [np.ascontiguousarray(weights[k], np.float32) for k in TRIANGLE_WEIGHT_ORDER]
    arr = (_FP * 16)(*[k.ctypes.data_as(_FP) for k in keep])
    out = np.empty((n, n, cz), np.float32)
    lib().orc_trimul_af2(pz, pm, _i(n), _i(cz), _i(c_hidden), arr, _d(eps),
                         _i(1 if incoming else 0), out.ctypes.data_as(_FP))
    return out


def trimul_af3(pair, mask, weights, incoming=False, divide_by_length=False):
    pair, pp = _f(pair)
    n, _, ch = pair.shape
    m, pm = _f(mask)
    names = ("leftNormInputScale", "leftNormInputOffset", "projection", "gate",
             "centerNormScale", "centerNormOffset", "outputProjection", "gatingLinear")
    keep = [_f(weights[k]) for k in names]
    out = np.empty((n, n, ch), np.float32)
    lib().orc_trimul_af3(pp, pm, _i(n), _i(ch), _i(1 if incoming else 0),
                         *[k[1] for k in keep], _i(1 if divide_by_length else 0),
                         out.ctypes.data_as(_FP))
    return out


def attention_af2(activations, mask, batch, query_length, channels, heads, weights,
                  transpose=False, pair_bias=None, eps=1e-5):
    """AF2 gated attention; ``pair_bias`` is None or a dict with ``source``
    "separate" (plus activations/channels/layerNormScale/layerNormOffset/
    projectionWeight) or "normalized-input" (projectionWeight)."""
    a, pa = _f(activations)
    m, pm = _f(mask)
    names = ("queryNormScale", "queryNormOffset", "queryWeight", "keyWeight", "valueWeight",
             "gatingWeight", "gatingBias", "outputWeight", "outputBias")
    keep = [_f(weights[k]) for k in names]
    mode, pact, pch, pns, pno, pw = 0, _f(None), 0, _f(None), _f(None), _f(None)
    if pair_bias is not None:
        if pair_bias["source"] == "separate":
            mode = 1
            pact = _f(pair_bias["activations"])
            pch = int(pair_bias["channels"])
            pns = _f(pair_bias["layerNormScale"])
            pno = _f(pair_bias["layerNormOffset"])
        else:
            mode = 2
            pch = channels
        pw = _f(pair_bias["projectionWeight"])
    out = np.empty((batch * query_length, channels), np.float32)
    lib().orc_attention_af2(pa, pm, _i(batch), _i(query_length), _i(channels), _i(heads),
                            _i(1 if transpose else 0), *[k[1] for k in keep],
                            _i(mode), pact[1], _i(pch), pns[1], pno[1], pw[1], _d(eps),
                            out.ctypes.data_as(_FP))
    return out.reshape(np.asarray(activations).shape)


def grid_attention_af3(pair, mask, weights, transpose, swap_transposed_bias):
    pair, pp = _f(pair)
    n, _, ch = pair.shape
    m, pm = _f(mask)
    heads, dim = int(weights["heads"]), int(weights["dimension"])
    names = ("actNormScale", "actNormOffset", "pairBiasProjection", "qProjection", "kProjection",
             "vProjection", "gatingQuery")
    keep = [_f(weights[k]) for k in names]
    gb = _f(weights.get("gatingQueryBias"))
    wo = _f(weights["outputProjection"])
    ob = _f(weights.get("outputProjectionBias"))
    out = np.empty((n, n, ch), np.float32)
    lib().orc_grid_attention_af3(pp, pm, _i(n), _i(ch), _i(1 if transpose else 0), _i(heads),
                                 _i(dim), _i(1 if swap_transposed_bias else 0),
                                 *[k[1] for k in keep], gb[1], wo[1], ob[1],
                                 out.ctypes.data_as(_FP))
    return out


def transition_af2(activations, weights, hidden, eps=1e-5):
    a, pa = _f(activations)
    ch = a.shape[-1]
    rows = a.size // ch
    names = ("layerNormScale", "layerNormOffset", "firstWeight", "firstBias", "secondWeight",
             "secondBias")
    keep = [_f(weights[k]) for k in names]
    out = np.empty_like(a)
    lib().orc_transition_af2(pa, _l(rows), _i(ch), _i(hidden), *[k[1] for k in keep], _d(eps),
                             out.ctypes.data_as(_FP))
    return out


def transition_af3(activations, weights, factor=4):
    a, pa = _f(activations)
    ch = a.shape[-1]
    rows = a.size // ch
    names = ("inputLayerNormScale", "inputLayerNormOffset", "transition1", "transition2")
    keep = [_f(weights[k]) for k in names]
    out = np.empty_like(a)
    lib().orc_transition_af3(pa, _l(rows), _i(ch), _i(factor), *[k[1] for k in keep],
                             out.ctypes.data_as(_FP))
    return out


def outer_product_mean_af2(msa, mask, weights, c_outer, c_z, ln_eps=1e-5, norm_eps=1e-3):
    a, pa = _f(msa)
    S, n, cm = a.shape
    m, pm = _f(mask)
    names = ("layerNormScale", "layerNormOffset", "leftWeight", "leftBias", "rightWeight",
             "rightBias", "outputWeight", "outputBias")
    keep = [_f(weights[k]) for k in names]
    out = np.empty((n, n, c_z), np.float32)
    lib().orc_outer_product_mean(pa, pm, _i(S), _i(n), _i(cm), _i(c_outer), _i(c_z),
                                 *[k[1] for k in keep], _d(ln_eps), _d(norm_eps), _i(1), _i(0),
                                 out.ctypes.data_as(_FP))
    return out


def outer_product_mean_af3(msa, mask, weights, c_z, bias_after_norm=False):
    a, pa = _f(msa)
    S, n, cm = a.shape
    m, pm = _f(mask)
    co = int(weights["outerChannels"])
    keep = [_f(weights["layerNormInputScale"]), _f(weights["layerNormInputOffset"]),
            _f(weights["leftProjection"]), _f(weights.get("leftProjectionBias")),
            _f(weights["rightProjection"]), _f(weights.get("rightProjectionBias")),
            _f(weights["outputW"]), _f(weights["outputB"])]
    out = np.empty((n, n, c_z), np.float32)
    lib().orc_outer_product_mean(pa, pm, _i(S), _i(n), _i(cm), _i(co), _i(c_z),
                                 *[k[1] for k in keep], _d(1e-5), _d(1e-3), _i(0),
                                 _i(1 if bias_after_norm else 0), out.ctypes.data_as(_FP))
    return out


def pair_logits_af3(pair, norm_scale, norm_offset, projection, heads):
    pair, pp = _f(pair)
    n, _, ch = pair.shape
    keep = [_f(norm_scale), _f(norm_offset), _f(projection)]
    out = np.empty((heads, n, n), np.float32)
    lib().orc_pair_logits_af3(pp, _i(n), _i(ch), _i(heads), *[k[1] for k in keep],
                              out.ctypes.data_as(_FP))
    return out


def single_attention_af3(single, pair_logits, seq_mask, weights):
    s, ps = _f(single)
    n, ch = s.shape
    pl, ppl = _f(pair_logits)
    m, pm = _f(seq_mask)
    heads, dim = int(weights["heads"]), int(weights["dimension"])
    names = ("layerNormScale", "layerNormOffset", "qProjection", "qBias", "kProjection",
             "vProjection", "gatingQuery", "outputProjection")
    keep = [_f(weights[k]) for k in names]
    out = np.empty((n, ch), np.float32)
    lib().orc_single_attention_af3(ps, ppl, pm, _i(n), _i(ch), _i(heads), _i(dim),
                                   *[k[1] for k in keep], out.ctypes.data_as(_FP))
    return out


def int5_decode(codes, scales, zeros, elements, block=32):
    codes = np.ascontiguousarray(codes, np.uint8)
    # one slack byte so the two-byte read of the last code stays inside
    codes = np.concatenate([codes.reshape(-1), np.zeros(1, np.uint8)])
    scales = np.ascontiguousarray(scales).view(np.uint16)
    zeros = np.ascontiguousarray(zeros).view(np.uint16)
    out = np.empty(elements, np.float32)
    lib().orc_int5_decode(codes.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)),
                          scales.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)),
                          zeros.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)),
                          _l(elements), _i(block), out.ctypes.data_as(_FP))
    return out


# --------------------------------------------------------------------------
# Blocks (order and residual wiring)


def af2_pair_block(pair, pair_mask, w, c_hidden, eps=1e-5, stages=None):
    """The five pair updates of an AF2 Evoformer block, each added into the
    running pair (``webgpu/af2/evoformer/block.js:1575-1612``).  ``stages``
    (optional list) receives the pair after every update."""
    pair = np.array(pair, np.float32, copy=True)
    n, _, cz = pair.shape

    def add(delta):
        nonlocal pair
        pair = pair + delta.reshape(pair.shape)
        if stages is not None:
            stages.append(pair.copy())

    add(trimul_af2(pair, pair_mask, w["triangleMultiplicationOutgoing"], c_hidden, eps, False))
    add(trimul_af2(pair, pair_mask, w["triangleMultiplicationIncoming"], c_hidden, eps, True))
    for key, transpose in (("triangleAttentionStarting", False), ("triangleAttentionEnding", True)):
        t = w[key]
        add(attention_af2(pair, pair_mask, n, n, cz, t["heads"], t["attention"], transpose,
                          dict(t["pairBias"], source="normalized-input"), eps))
    t = w["pairTransition"]
    add(transition_af2(pair, t, t["firstBias"].shape[0], eps))
    return pair


def af2_template_pair_block(pair, pair_mask, w, c_hidden, eps=1e-5):
    """The template pair stack's block: the same five updates with the attentions first
    (``encodeTemplatePairBlock``: ``webgpu/af2/evoformer/block.js:1746-1781``)."""
    pair = np.array(pair, np.float32, copy=True)
    n, _, cz = pair.shape
    for key, transpose in (("triangleAttentionStarting", False), ("triangleAttentionEnding", True)):
        t = w[key]
        pair = pair + attention_af2(pair, pair_mask, n, n, cz, t["heads"], t["attention"], transpose,
                                    dict(t["pairBias"], source="normalized-input"), eps).reshape(pair.shape)
    pair = pair + trimul_af2(pair, pair_mask, w["triangleMultiplicationOutgoing"], c_hidden, eps, False)
    pair = pair + trimul_af2(pair, pair_mask, w["triangleMultiplicationIncoming"], c_hidden, eps, True)
    t = w["pairTransition"]
    return pair + transition_af2(pair, t, t["firstBias"].shape[0], eps)


def af2_evoformer_block(msa, pair, msa_mask, pair_mask, w, c_outer, c_hidden, eps=1e-5):
    """Whole AF2 Evoformer block (``webgpu/af2/evoformer/block.js:1546-1612``)."""
    msa = np.array(msa, np.float32, copy=True)
    pair = np.array(pair, np.float32, copy=True)
    S, n, cm = msa.shape
    cz = pair.shape[-1]
    row = w["msaRowAttention"]
    pb = dict(row["pairBias"], source="separate", activations=pair, channels=cz)
    msa = msa + attention_af2(msa, msa_mask, S, n, cm, row["heads"], row["attention"], False, pb, eps)
    col = w["msaColumnAttention"]
    msa = msa + attention_af2(msa, msa_mask, n, S, cm, col["heads"], col["attention"], True, None, eps)
    t = w["msaTransition"]
    msa = msa + transition_af2(msa, t, t["firstBias"].shape[0], eps)
    pair = pair + outer_product_mean_af2(msa, msa_mask, w["outerProductMean"], c_outer, cz, eps)
    pair = af2_pair_block(pair, pair_mask, w, c_hidden, eps)
    return msa, pair


def af3_pairformer_block(pair, single, pair_mask, seq_mask, w, swap_transposed_bias,
                         divide_by_length=False):
    """``pairformerBlock`` (``cpu/af3/trunk/pairformer.js:495-542``)."""
    pair = np.array(pair, np.float32, copy=True)
    pair = pair + trimul_af3(pair, pair_mask, w["triangleMultiplicationOutgoing"], False, divide_by_length)
    pair = pair + trimul_af3(pair, pair_mask, w["triangleMultiplicationIncoming"], True, divide_by_length)
    pair = pair + grid_attention_af3(pair, pair_mask, w["pairAttention1"], False, swap_transposed_bias)
    pair = pair + grid_attention_af3(pair, pair_mask, w["pairAttention2"], True, swap_transposed_bias)
    pair = pair + transition_af3(pair, w["pairTransition"])
    if single is None:
        return pair, None
    single = np.array(single, np.float32, copy=True)
    heads = int(w["singleAttention"]["heads"])
    logits = pair_logits_af3(pair, w["singlePairLogitsNormScale"], w["singlePairLogitsNormOffset"],
                             w["singlePairLogitsProjection"], heads)
    single = single + single_attention_af3(single, logits, seq_mask, w["singleAttention"])
    single = single + transition_af3(single, w["singleTransition"])
    return pair, single


GLOBAL_ATTENTION_ORDER = ("queryNormScale", "queryNormOffset", "queryWeight", "keyWeight", "valueWeight",
                          "gatingWeight", "gatingBias", "outputWeight", "outputBias")


def global_column_attention_af2(msa, mask, weights, eps=1e-5):
    """The extra-MSA stack's global column attention (``webgpu/af2/evoformer/block.js:100-482,953-1032``);
    ``weights["heads"]`` heads of ``gatingBias.size / heads`` channels, one shared key/value head."""
    a, pa = _f(msa)
    S, n, c = a.shape
    m, pm = _f(mask)
    heads = int(weights["heads"])
    dim = int(np.asarray(weights["gatingBias"]).size // heads)
    keep = [_f(weights[k]) for k in GLOBAL_ATTENTION_ORDER]
    out = np.empty((S, n, c), np.float32)
    lib().orc_global_column_attention_af2(pa, pm, _i(S), _i(n), _i(c), _i(heads), _i(dim), *[k[1] for k in keep],
                                          _d(eps), out.ctypes.data_as(_FP))
    return out


def af2_extra_msa_block(msa, pair, msa_mask, pair_mask, w, c_outer, c_hidden, eps=1e-5):
    """One block of the extra-MSA stack (``encodeExtraMsaBlock``, ``webgpu/af2/evoformer/block.js:1715-1744``):
    row attention with pair bias, global column attention, MSA transition, then the Evoformer pair part
    (outer product mean and the five pair updates)."""
    msa = np.array(msa, np.float32, copy=True)
    pair = np.array(pair, np.float32, copy=True)
    S, n, cm = msa.shape
    cz = pair.shape[-1]
    row = w["msaRowAttention"]
    pb = dict(row["pairBias"], source="separate", activations=pair, channels=cz)
    msa = msa + attention_af2(msa, msa_mask, S, n, cm, row["heads"], row["attention"], False, pb, eps)
    msa = msa + global_column_attention_af2(msa, msa_mask, w["msaColumnGlobalAttention"], eps)
    t = w["msaTransition"]
    msa = msa + transition_af2(msa, t, t["firstBias"].shape[0], eps)
    pair = pair + outer_product_mean_af2(msa, msa_mask, w["outerProductMean"], c_outer, cz, eps)
    pair = af2_pair_block(pair, pair_mask, w, c_hidden, eps)
    return msa, pair


def msa_attention_af3(msa, msa_mask, pair, weights):
    """``msaAttention`` (``cpu/af3/trunk/msa.js:164-224``): MSA pair-weighted averaging."""
    a, pa = _f(msa)
    S, n, cm = a.shape
    m, pm = _f(msa_mask)
    z, pz = _f(pair)
    cz = z.shape[-1]
    heads, dim = int(weights["heads"]), int(weights["dimension"])
    names = ("actNormScale", "actNormOffset", "pairNormScale", "pairNormOffset", "pairLogits", "vProjection",
             "gatingQuery", "outputProjection")
    keep = [_f(weights[k]) for k in names]
    out = np.empty((S, n, cm), np.float32)
    lib().orc_msa_attention_af3(pa, pm, pz, _i(S), _i(n), _i(cm), _i(cz), _i(heads), _i(dim),
                                *[k[1] for k in keep], out.ctypes.data_as(_FP))
    return out


def msa_block_af3(msa, pair, msa_mask, pair_mask, w, swap_transposed_bias, msa_update_before_outer_product,
                  bias_after_norm=False):
    """``msaBlock`` (``cpu/af3/trunk/msa.js:235-287``): the outer product mean and the MSA update in the
    order the dialect names (it has no default there either), then the five pair updates."""
    if msa_update_before_outer_product not in (True, False):
        raise ValueError("dialect.msaUpdateBeforeOuterProduct has no default")
    msa = np.array(msa, np.float32, copy=True)
    pair = np.array(pair, np.float32, copy=True)
    cz = pair.shape[-1]

    def outer_product():
        nonlocal pair
        pair = pair + outer_product_mean_af3(msa, msa_mask, w["outerProductMean"], cz, bias_after_norm)

    def update_msa():
        nonlocal msa
        msa = msa + msa_attention_af3(msa, msa_mask, pair, w["msaAttention1"])
        S, n, cm = msa.shape
        msa = msa + transition_af3(msa.reshape(S * n, cm), w["msaTransition"]).reshape(S, n, cm)

    if msa_update_before_outer_product:
        update_msa()
        outer_product()
    else:
        outer_product()
        update_msa()
    pair = pair + trimul_af3(pair, pair_mask, w["triangleMultiplicationOutgoing"], False)
    pair = pair + trimul_af3(pair, pair_mask, w["triangleMultiplicationIncoming"], True)
    pair = pair + grid_attention_af3(pair, pair_mask, w["pairAttention1"], False, swap_transposed_bias)
    pair = pair + grid_attention_af3(pair, pair_mask, w["pairAttention2"], True, swap_transposed_bias)
    pair = pair + transition_af3(pair, w["pairTransition"])
    return msa, pair


def distogram_logits(pair, half_logits, bias=None):
    """The logits of ``distogramHead`` (``cpu/af3/trunk/trunk.js:47-60``): half + half transposed (a sum)."""
    z, pz = _f(pair)
    n, _, cz = z.shape
    w, pw = _f(half_logits)
    bins = w.size // cz
    b = _f(bias)
    out = np.empty((n, n, bins), np.float32)
    lib().orc_distogram_logits(pz, _i(n), _i(cz), _i(bins), pw, b[1], out.ctypes.data_as(_FP))
    return out


def relative_l2(actual, expected) -> float:
    """``relativeRms`` of the reference's checkers: ||a-b|| / ||b||
    (``tools/gpu/relative-rms.js:63-75``)."""
    a = np.asarray(actual, np.float64).reshape(-1)
    b = np.asarray(expected, np.float64).reshape(-1)
    if a.size == 0 or a.size != b.size:
        raise ValueError("relative_l2 needs equally sized, non-empty arrays")
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))
