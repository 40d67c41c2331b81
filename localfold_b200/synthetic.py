"""Seeded synthetic inputs and weights in the reference's weight-object shapes.

The reference benches and checks this path on noise as well
(``tools/gpu/af2-synthetic-block.js:13-16``, ``webgpu/testing/deterministic-input.js:12-45``,
``tools/gpu/af3-synthetic-pairformer.js:23-102``); there is no dataset involved.
Everything is drawn from ``numpy.random.default_rng(seed).standard_normal`` in a
fixed order: activations first, then the weights operator by operator in the
pack order of each operator.  Linear weights are N(0, 1/fan_in); LayerNorm
gains 1, offsets 0; gate biases 1, all other biases 0 (AF2 dialect; the AF3
dialect has no biases except the single attention's query bias, drawn N(0,1)*0.1).
"""
from __future__ import annotations

import numpy as np


class _Draw:
    def __init__(self, seed):
        self.rng = np.random.default_rng(seed)

    def normal(self, *shape, std=1.0):
        return (self.rng.standard_normal(shape) * std).astype(np.float32)

    def linear(self, fan_in, *shape):
        return self.normal(*shape, std=fan_in ** -0.5)


def ones(n):
    return np.ones(n, np.float32)


def zeros(n):
    return np.zeros(n, np.float32)


# ---- AF2 dialect -----------------------------------------------------------


def af2_triangle_weights(d: _Draw, cz, c):
    """Operator-form weights, linear weights [out][in] (``webgpu/kernels/triangle/types.js:27-43``)."""
    w = {"layerNormInWeight": ones(cz), "layerNormInBias": zeros(cz)}
    for role in ("AP", "AG", "BP", "BG"):
        w[f"linear{role}Weight"] = d.linear(cz, c, cz)
        w[f"linear{role}Bias"] = ones(c) if role.endswith("G") else zeros(c)
    w["layerNormOutWeight"] = ones(c)
    w["layerNormOutBias"] = zeros(c)
    w["linearZWeight"] = d.linear(c, cz, c)
    w["linearZBias"] = zeros(cz)
    w["linearGWeight"] = d.linear(cz, cz, cz)
    w["linearGBias"] = ones(cz)
    return w


def af2_attention_weights(d: _Draw, c, heads, pair_channels=None, separate=False):
    """``{heads, attention, pairBias}`` as in ``webgpu/af2/evoformer/block.js:1546-1605``."""
    att = {"queryNormScale": ones(c), "queryNormOffset": zeros(c),
           "queryWeight": d.linear(c, c, c), "keyWeight": d.linear(c, c, c),
           "valueWeight": d.linear(c, c, c), "gatingWeight": d.linear(c, c, c),
           "gatingBias": ones(c), "outputWeight": d.linear(c, c, c), "outputBias": zeros(c)}
    out = {"heads": heads, "attention": att}
    if pair_channels is not None:
        pb = {"projectionWeight": d.linear(pair_channels, pair_channels, heads)}
        if separate:
            pb["layerNormScale"] = ones(pair_channels)
            pb["layerNormOffset"] = zeros(pair_channels)
        out["pairBias"] = pb
    return out


def af2_transition_weights(d: _Draw, c, factor=4):
    h = c * factor
    return {"layerNormScale": ones(c), "layerNormOffset": zeros(c), "firstWeight": d.linear(c, c, h),
            "firstBias": zeros(h), "secondWeight": d.linear(h, h, c), "secondBias": zeros(c)}


def af2_opm_weights(d: _Draw, cm, c, cz):
    return {"layerNormScale": ones(cm), "layerNormOffset": zeros(cm), "leftWeight": d.linear(cm, cm, c),
            "leftBias": zeros(c), "rightWeight": d.linear(cm, cm, c), "rightBias": zeros(c),
            "outputWeight": d.linear(c * c, c * c, cz), "outputBias": zeros(cz)}


def af2_pair_block_weights(d: _Draw, cz=128, c=128, heads=4, factor=4):
    return {
        "triangleMultiplicationOutgoing": af2_triangle_weights(d, cz, c),
        "triangleMultiplicationIncoming": af2_triangle_weights(d, cz, c),
        "triangleAttentionStarting": af2_attention_weights(d, cz, heads, cz),
        "triangleAttentionEnding": af2_attention_weights(d, cz, heads, cz),
        "pairTransition": af2_transition_weights(d, cz, factor),
    }


def af2_pair_block(seed, n, cz=128, c=128, heads=4, factor=4, blocks=1, masked_tail=0.0):
    """BASELINE config 0 / 4 shape: pair z ~ N(0,1), mask ones (or the last
    ``masked_tail`` fraction of residues zeroed, pair mask m_i*m_j)."""
    d = _Draw(seed)
    pair = d.normal(n, n, cz)
    weights = [af2_pair_block_weights(d, cz, c, heads, factor) for _ in range(blocks)]
    return pair, residue_pair_mask(n, masked_tail), weights


def residue_pair_mask(n, masked_tail=0.0):
    m = np.ones(n, np.float32)
    k = int(np.ceil(n * masked_tail)) if masked_tail > 0 else 0
    if k:
        m[n - k:] = 0
    return np.ascontiguousarray(np.outer(m, m).astype(np.float32))


def af2_evoformer_block(seed, S=128, n=256, cm=256, cz=128, c_outer=32, c=128, msa_heads=8, pair_heads=4,
                        masked_rows=0.1):
    """BASELINE config 1 shape: full Evoformer block; a random ``masked_rows``
    fraction of MSA rows masked (row mask broadcast over residues), pair mask ones."""
    d = _Draw(seed)
    msa = d.normal(S, n, cm)
    pair = d.normal(n, n, cz)
    rows = np.ones(S, np.float32)
    k = int(round(S * masked_rows))
    if k:
        rows[d.rng.choice(S, size=k, replace=False)] = 0
    msa_mask = np.ascontiguousarray(np.repeat(rows[:, None], n, axis=1))
    pair_mask = np.ones((n, n), np.float32)
    w = {"msaRowAttention": af2_attention_weights(d, cm, msa_heads, cz, separate=True),
         "msaColumnAttention": af2_attention_weights(d, cm, msa_heads),
         "msaTransition": af2_transition_weights(d, cm),
         "outerProductMean": af2_opm_weights(d, cm, c_outer, cz)}
    w.update(af2_pair_block_weights(d, cz, c, pair_heads))
    return msa, pair, msa_mask, pair_mask, w


def af2_global_attention_weights(d: _Draw, c, heads, dim):
    """The extra-MSA stack's global column attention (``webgpu/af2/evoformer/block.js:963-966``): one shared
    key/value head of ``dim`` channels, ``heads`` query and gate heads."""
    hd = heads * dim
    return {"heads": heads, "queryNormScale": 1 + d.normal(c, std=0.1), "queryNormOffset": d.normal(c, std=0.1),
            "queryWeight": d.linear(c, c, hd), "keyWeight": d.linear(c, c, dim), "valueWeight": d.linear(c, c, dim),
            "gatingWeight": d.linear(c, c, hd), "gatingBias": ones(hd), "outputWeight": d.linear(hd, hd, c),
            "outputBias": d.normal(c, std=0.1)}


def af2_extra_msa_block(seed, S=64, n=48, ce=64, cz=128, c_outer=32, c=128, msa_heads=8, pair_heads=4, gaps=0.15):
    """One block of the extra-MSA stack at its own widths (64 MSA channels, 8 heads of 8): a random ``gaps``
    fraction of the alignment masked (the first row whole), pair mask ones."""
    d = _Draw(seed)
    msa = d.normal(S, n, ce)
    pair = d.normal(n, n, cz)
    msa_mask = (d.rng.random((S, n)) >= gaps).astype(np.float32)
    msa_mask[0] = 1
    pair_mask = np.ones((n, n), np.float32)
    w = {"msaRowAttention": af2_attention_weights(d, ce, msa_heads, cz, separate=True),
         "msaColumnGlobalAttention": af2_global_attention_weights(d, ce, msa_heads, ce // msa_heads),
         "msaTransition": af2_transition_weights(d, ce),
         "outerProductMean": af2_opm_weights(d, ce, c_outer, cz)}
    w.update(af2_pair_block_weights(d, cz, c, pair_heads))
    return msa, pair, msa_mask, pair_mask, w


# ---- AF3 dialect -----------------------------------------------------------


def af3_triangle_weights(d: _Draw, c):
    return {"leftNormInputScale": ones(c), "leftNormInputOffset": zeros(c),
            "projection": d.linear(c, c, 2 * c), "gate": d.linear(c, c, 2 * c),
            "centerNormScale": ones(c), "centerNormOffset": zeros(c),
            "outputProjection": d.linear(c, c, c), "gatingLinear": d.linear(c, c, c)}


def af3_grid_attention_weights(d: _Draw, c, heads, dim):
    hd = heads * dim
    return {"heads": heads, "dimension": dim, "actNormScale": ones(c), "actNormOffset": zeros(c),
            "pairBiasProjection": d.linear(c, c, heads), "qProjection": d.linear(c, hd, c),
            "kProjection": d.linear(c, hd, c), "vProjection": d.linear(c, c, hd),
            "gatingQuery": d.linear(c, hd, c), "outputProjection": d.linear(hd, hd, c)}


def af3_transition_weights(d: _Draw, c, factor=4):
    return {"inputLayerNormScale": ones(c), "inputLayerNormOffset": zeros(c),
            "transition1": d.linear(c, c, 2 * factor * c), "transition2": d.linear(factor * c, factor * c, c)}


def af3_single_attention_weights(d: _Draw, c, heads, dim):
    hd = heads * dim
    return {"heads": heads, "dimension": dim, "layerNormScale": ones(c), "layerNormOffset": zeros(c),
            "qProjection": d.linear(c, c, hd), "qBias": d.normal(hd, std=0.1), "kProjection": d.linear(c, c, hd),
            "vProjection": d.linear(c, c, hd), "gatingQuery": d.linear(c, c, hd),
            "outputProjection": d.linear(hd, hd, c)}


def af3_pairformer_block_weights(d: _Draw, cz=128, cs=384, pair_heads=4, single_heads=16):
    """``pairformerBlockWeights`` (``shared/af3/weights/weights.js:699-727``)."""
    return {
        "pairChannels": cz, "singleChannels": cs,
        "triangleMultiplicationOutgoing": af3_triangle_weights(d, cz),
        "triangleMultiplicationIncoming": af3_triangle_weights(d, cz),
        "pairAttention1": af3_grid_attention_weights(d, cz, pair_heads, cz // pair_heads),
        "pairAttention2": af3_grid_attention_weights(d, cz, pair_heads, cz // pair_heads),
        "pairTransition": af3_transition_weights(d, cz),
        "singlePairLogitsNormScale": ones(cz), "singlePairLogitsNormOffset": zeros(cz),
        "singlePairLogitsProjection": d.linear(cz, cz, single_heads),
        "singleAttention": af3_single_attention_weights(d, cs, single_heads, cs // single_heads),
        "singleTransition": af3_transition_weights(d, cs),
    }


def af3_pairformer(seed, n=384, cz=128, cs=384, blocks=1, pair_heads=4, single_heads=16):
    """BASELINE config 2 shape: z, s ~ N(0,1), all-ones masks."""
    d = _Draw(seed)
    pair = d.normal(n, n, cz)
    single = d.normal(n, cs)
    weights = [af3_pairformer_block_weights(d, cz, cs, pair_heads, single_heads) for _ in range(blocks)]
    return pair, single, np.ones((n, n), np.float32), np.ones(n, np.float32), weights


def af3_opm_weights(d: _Draw, cm, co, cz):
    """``outerProductMean`` of an AF3 MSA block (``cpu/af3/trunk/msa.js:72-155``): no left/right biases."""
    return {"outerChannels": co, "layerNormInputScale": 1 + d.normal(cm, std=0.1), "layerNormInputOffset": d.normal(cm, std=0.1),
            "leftProjection": d.linear(cm, cm, co), "rightProjection": d.linear(cm, cm, co),
            "outputW": d.linear(co * co, co * co, cz), "outputB": d.normal(cz, std=0.1)}


def af3_msa_attention_weights(d: _Draw, cm, cz, heads, dim):
    """``msaAttention1`` (``shared/af3/weights/weights.js:670-680``); ``heads * dim`` need not equal ``cm``."""
    hd = heads * dim
    return {"heads": heads, "dimension": dim, "actNormScale": 1 + d.normal(cm, std=0.1), "actNormOffset": d.normal(cm, std=0.1),
            "pairNormScale": 1 + d.normal(cz, std=0.1), "pairNormOffset": d.normal(cz, std=0.1),
            "pairLogits": d.linear(cz, cz, heads), "vProjection": d.linear(cm, cm, hd),
            "gatingQuery": d.linear(cm, cm, hd), "outputProjection": d.linear(hd, hd, cm)}


def af3_msa_block_weights(d: _Draw, cm=64, cz=128, co=32, msa_heads=8, msa_dim=8, pair_heads=4):
    """``msaBlockWeights`` (``shared/af3/weights/weights.js:640-700``)."""
    return {
        "msaChannels": cm, "pairChannels": cz,
        "outerProductMean": af3_opm_weights(d, cm, co, cz),
        "msaAttention1": af3_msa_attention_weights(d, cm, cz, msa_heads, msa_dim),
        "msaTransition": af3_transition_weights(d, cm),
        "triangleMultiplicationOutgoing": af3_triangle_weights(d, cz),
        "triangleMultiplicationIncoming": af3_triangle_weights(d, cz),
        "pairAttention1": af3_grid_attention_weights(d, cz, pair_heads, cz // pair_heads),
        "pairAttention2": af3_grid_attention_weights(d, cz, pair_heads, cz // pair_heads),
        "pairTransition": af3_transition_weights(d, cz),
    }


def af3_msa_block(seed, S=16, n=64, cm=64, cz=128, co=32, msa_heads=8, msa_dim=8, pair_heads=4, gaps=0.2):
    """One AF3 MSA block: msa, pair ~ N(0,1); a random ``gaps`` fraction of the MSA entries below the first
    row masked out (so the coverage count and the key mask both matter); pair mask ones."""
    d = _Draw(seed)
    msa = d.normal(S, n, cm)
    pair = d.normal(n, n, cz)
    msa_mask = (d.rng.random((S, n)) >= gaps).astype(np.float32)
    msa_mask[0] = 1
    pair_mask = np.ones((n, n), np.float32)
    return msa, pair, msa_mask, pair_mask, af3_msa_block_weights(d, cm, cz, co, msa_heads, msa_dim, pair_heads)


def draw(seed):
    return _Draw(seed)
