"""Second, independent formulation of the pair-stack operators: vectorised torch
float64 on the CPU.  TEST INFRASTRUCTURE ONLY.

It shares no code with ``pairstack_oracle.c``: the same formulas are written as
einsums/matmuls from the reference's definitions, so agreement between the two
cross-validates the restatement for the operators that have no golden data, and
this version is fast enough to serve as the checker at sizes where the scalar
loops of the C oracle take too long (N >= 256).

Formulas: ``webgpu/kernels/triangle/cpu-reference.js:55-99``,
``cpu/af3/trunk/pairformer.js:180-485``, ``tools/gpu/check-evoformer-{attention,
transition,opm}.js``, pair bias / transpose / clamp semantics of
``webgpu/kernels/attention.js:162-167,695-756,889-892,917-921,2466``.
"""
from __future__ import annotations

import numpy as np
import torch

F64 = torch.float64


def T(a):
    return torch.as_tensor(np.asarray(a), dtype=F64)


def ln(x, g, b, eps=1e-5, fast=False):
    mean = x.mean(-1, keepdim=True)
    if fast:
        var = (x * x).mean(-1, keepdim=True) - mean * mean
    else:
        var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * T(g) + T(b)


def trimul_af2(z, mask, w, eps=1e-5, incoming=False):
    z, m = T(z), T(mask)[..., None]
    zn = ln(z, w["layerNormInWeight"], w["layerNormInBias"], eps)
    lin = lambda x, k: x @ T(w[f"linear{k}Weight"]).T + T(w[f"linear{k}Bias"])
    a = lin(zn, "AP") * torch.sigmoid(lin(zn, "AG")) * m
    b = lin(zn, "BP") * torch.sigmoid(lin(zn, "BG")) * m
    x = torch.einsum("kjc,kic->ijc", a, b) if incoming else torch.einsum("ikc,jkc->ijc", a, b)
    xn = ln(x, w["layerNormOutWeight"], w["layerNormOutBias"], eps)
    return (lin(xn, "Z") * torch.sigmoid(lin(zn, "G"))).numpy()


def trimul_af3(pair, mask, w, incoming=False, divide_by_length=False):
    z, m = T(pair), T(mask)[..., None]
    n = z.shape[0]
    zn = ln(z, w["leftNormInputScale"], w["leftNormInputOffset"], 1e-5, True)
    proj = zn @ T(w["projection"])
    gate = torch.sigmoid(zn @ T(w["gate"]))
    a = proj[..., 0::2] * gate[..., 0::2] * m
    b = proj[..., 1::2] * gate[..., 1::2] * m
    x = torch.einsum("kjc,kic->ijc", a, b) if incoming else torch.einsum("ikc,jkc->ijc", a, b)
    if divide_by_length:
        x = x / n
    xn = ln(x, w["centerNormScale"], w["centerNormOffset"], 1e-5, True)
    return ((xn @ T(w["outputProjection"])) * torch.sigmoid(zn @ T(w["gatingLinear"]))).numpy()


def _attend(q, k, v, logit_extra, heads):
    """q,k,v: [B,Q,H*d]; logit_extra: broadcastable to [B,H,Q,Q] (mask + bias)."""
    B, Q, HD = q.shape
    d = HD // heads
    qh = q.view(B, Q, heads, d).permute(0, 2, 1, 3)
    kh = k.view(B, Q, heads, d).permute(0, 2, 1, 3)
    vh = v.view(B, Q, heads, d).permute(0, 2, 1, 3)
    logits = qh @ kh.transpose(-1, -2) / np.sqrt(d) + logit_extra
    return logits, vh


def attention_af2(act, mask, batch, Q, c, heads, w, transpose=False, pair_bias=None, eps=1e-5):
    x = T(act).reshape(-1, c)
    m = T(mask).reshape(-1)
    if transpose:      # logical (b, i) <- memory (i, b)
        x = x.view(Q, batch, c).transpose(0, 1)
        m = m.view(Q, batch).transpose(0, 1)
    else:
        x = x.view(batch, Q, c)
        m = m.view(batch, Q)
    n = ln(x, w["queryNormScale"], w["queryNormOffset"], eps)
    q, k, v = n @ T(w["queryWeight"]), n @ T(w["keyWeight"]), n @ T(w["valueWeight"])
    g = torch.sigmoid(n @ T(w["gatingWeight"]) + T(w["gatingBias"]))
    extra = (1e9 * (m - 1.0))[:, None, None, :]
    if pair_bias is not None:
        if pair_bias["source"] == "separate":
            pn = ln(T(pair_bias["activations"]).reshape(Q, Q, -1), pair_bias["layerNormScale"],
                    pair_bias["layerNormOffset"], eps)
            flat = pn @ T(pair_bias["projectionWeight"])          # [Q,Q,H]
        else:
            flat = n @ T(pair_bias["projectionWeight"])           # logical [b=Q, i=Q, H]
        extra = extra + flat.permute(2, 0, 1)[None]
    logits, vh = _attend(q, k, v, extra, heads)
    logits = logits.clamp(-1e8, 1e8)
    # float32 logits: a fully masked row collapses to one value (uniform softmax)
    p = torch.softmax(logits.to(torch.float32).to(F64), -1)
    o = (p @ vh).permute(0, 2, 1, 3).reshape(batch, Q, c) * g
    out = o @ T(w["outputWeight"]) + T(w["outputBias"])
    if transpose:
        out = out.transpose(0, 1)
    return out.reshape(np.asarray(act).shape).numpy()


def grid_attention_af3(pair, mask, w, transpose, swap):
    z, m = T(pair), T(mask)
    n, _, c = z.shape
    heads, dim = int(w["heads"]), int(w["dimension"])
    nz = ln(z, w["actNormScale"], w["actNormOffset"], 1e-5, True)
    raw = nz @ T(w["pairBiasProjection"])                          # [n,n,H] memory order
    bias = raw.permute(2, 1, 0) if (transpose and swap) else raw.permute(2, 0, 1)
    act = nz.transpose(0, 1) if transpose else nz
    mm = m.transpose(0, 1) if transpose else m                     # key mask of logical row r: mm[r, j]
    q = act @ T(w["qProjection"]).T
    k = act @ T(w["kProjection"]).T
    v = act @ T(w["vProjection"])
    g = act @ T(w["gatingQuery"]).T
    if w.get("gatingQueryBias") is not None:
        g = g + T(w["gatingQueryBias"])
    extra = torch.where(mm > 0, 0.0, -1e9)[:, None, None, :] + bias[None]
    logits, vh = _attend(q, k, v, extra.to(F64), heads)
    p = torch.softmax(logits.to(torch.float32).to(F64), -1)
    o = (p @ vh).permute(0, 2, 1, 3).reshape(n, n, heads * dim) * torch.sigmoid(g)
    out = o @ T(w["outputProjection"])
    if w.get("outputProjectionBias") is not None:
        out = out + T(w["outputProjectionBias"])
    if transpose:
        out = out.transpose(0, 1)
    return out.contiguous().numpy()


def transition_af2(act, w, eps=1e-5):
    n = ln(T(act), w["layerNormScale"], w["layerNormOffset"], eps)
    h = torch.relu(n @ T(w["firstWeight"]) + T(w["firstBias"]))
    return (h @ T(w["secondWeight"]) + T(w["secondBias"])).numpy()


def transition_af3(act, w):
    n = ln(T(act), w["inputLayerNormScale"], w["inputLayerNormOffset"], 1e-5, True)
    wide = n @ T(w["transition1"])
    half = wide.shape[-1] // 2
    return ((torch.nn.functional.silu(wide[..., :half]) * wide[..., half:]) @ T(w["transition2"])).numpy()


def outer_product_mean_af2(msa, mask, w, ln_eps=1e-5, norm_eps=1e-3):
    x, m = T(msa), T(mask)
    n = ln(x, w["layerNormScale"], w["layerNormOffset"], ln_eps)
    left = (n @ T(w["leftWeight"]) + T(w["leftBias"])) * m[..., None]
    right = (n @ T(w["rightWeight"]) + T(w["rightBias"])) * m[..., None]
    outer = torch.einsum("sia,sjb->ijab", left, right)
    N = x.shape[1]
    out = outer.reshape(N, N, -1) @ T(w["outputWeight"]) + T(w["outputBias"])
    count = torch.einsum("si,sj->ij", m, m)
    return (out / (norm_eps + count)[..., None]).numpy()


def single_attention_af3(single, pair, seq_mask, w):
    s, z, m = T(single), T(pair), T(seq_mask)
    att = w["singleAttention"]
    heads = int(att["heads"])
    logits_src = ln(z, w["singlePairLogitsNormScale"], w["singlePairLogitsNormOffset"], 1e-5, True)
    pl = (logits_src @ T(w["singlePairLogitsProjection"])).permute(2, 0, 1)
    n = ln(s, att["layerNormScale"], att["layerNormOffset"], 1e-5, True)
    q = n @ T(att["qProjection"]) + T(att["qBias"])
    k, v = n @ T(att["kProjection"]), n @ T(att["vProjection"])
    extra = pl[None] + (1e9 * (m - 1.0))[None, None, None, :]
    logits, vh = _attend(q[None], k[None], v[None], extra, heads)
    p = torch.softmax(logits.to(torch.float32).to(F64), -1)
    o = (p @ vh).permute(0, 2, 1, 3).reshape(s.shape[0], -1) * torch.sigmoid(n @ T(att["gatingQuery"]))
    return (o @ T(att["outputProjection"])).numpy()


def af2_pair_block(pair, mask, w, eps=1e-5):
    pair = np.asarray(pair, np.float64)
    n, _, cz = pair.shape
    pair = pair + trimul_af2(pair, mask, w["triangleMultiplicationOutgoing"], eps, False)
    pair = pair + trimul_af2(pair, mask, w["triangleMultiplicationIncoming"], eps, True)
    for key, tr in (("triangleAttentionStarting", False), ("triangleAttentionEnding", True)):
        t = w[key]
        pair = pair + attention_af2(pair, mask, n, n, cz, t["heads"], t["attention"], tr,
                                    dict(t["pairBias"], source="normalized-input"), eps).reshape(pair.shape)
    return pair + transition_af2(pair, w["pairTransition"], eps)


def af3_pair_block(pair, mask, w, swap):
    pair = np.asarray(pair, np.float64)
    pair = pair + trimul_af3(pair, mask, w["triangleMultiplicationOutgoing"], False)
    pair = pair + trimul_af3(pair, mask, w["triangleMultiplicationIncoming"], True)
    pair = pair + grid_attention_af3(pair, mask, w["pairAttention1"], False, swap)
    pair = pair + grid_attention_af3(pair, mask, w["pairAttention2"], True, swap)
    return pair + transition_af3(pair, w["pairTransition"])


# --------------------------------------------------------------------------
# Sampled positions of full-size results.  The operators below compute, in float64, only the output
# positions asked for, reading from the full input just what those positions depend on; they serve as
# the checker at lengths where a whole-tensor oracle would take minutes (N = 1024, 2048).


def trimul_af2_positions(z, mask, w, rows, cols, eps=1e-5, incoming=False):
    """``trimul_af2(...)[rows][:, cols]``: the update at output positions (i, j), i in ``rows``, j in
    ``cols``.  Outgoing x[i, j] = sum_k a[i, k] b[j, k] needs pair rows ``rows`` (for a) and ``cols``
    (for b); incoming x[i, j] = sum_k a[k, j] b[k, i] needs pair columns ``cols`` (a) and ``rows`` (b)."""
    z = np.asarray(z)
    mask = np.asarray(mask)
    rows, cols = np.asarray(rows), np.asarray(cols)

    def operand(index, key):
        if incoming:      # [k, index]: columns of the pair -> logical [index, k]
            zz, mm = T(z[:, index]).transpose(0, 1), T(mask[:, index]).transpose(0, 1)
        else:
            zz, mm = T(z[index]), T(mask[index])
        zn = ln(zz, w["layerNormInWeight"], w["layerNormInBias"], eps)
        lin = lambda k: zn @ T(w[f"linear{k}Weight"]).T + T(w[f"linear{k}Bias"])
        return lin(key + "P") * torch.sigmoid(lin(key + "G")) * mm[..., None]

    if incoming:
        a = operand(cols, "A")     # a[j, k] = a_mem[k, j]
        b = operand(rows, "B")     # b[i, k] = b_mem[k, i]
        x = torch.einsum("jkc,ikc->ijc", a, b)
    else:
        a = operand(rows, "A")
        b = operand(cols, "B")
        x = torch.einsum("ikc,jkc->ijc", a, b)
    xn = ln(x, w["layerNormOutWeight"], w["layerNormOutBias"], eps)
    zn = ln(T(z[np.ix_(rows, cols)]), w["layerNormInWeight"], w["layerNormInBias"], eps)
    gate = torch.sigmoid(zn @ T(w["linearGWeight"]).T + T(w["linearGBias"]))
    return ((xn @ T(w["linearZWeight"]).T + T(w["linearZBias"])) * gate).numpy()


def attention_af2_positions(act, mask, n, c, heads, w, batch_rows, queries, transpose, pair_bias_weight, eps=1e-5):
    """Triangle attention (batch = queries = n, pair bias from the normalised input) at output positions
    (b, q), b in ``batch_rows``, q in ``queries`` of the logical (attention) orientation; returns
    [len(batch_rows), len(queries), c].  With ``transpose`` the logical element (b, q) is memory (q, b)."""
    z = np.asarray(act).reshape(n, n, c)
    m = np.asarray(mask).reshape(n, n)
    batch_rows, queries = np.asarray(batch_rows), np.asarray(queries)
    if transpose:
        x = T(z[:, batch_rows]).transpose(0, 1)           # [B, n, c]: logical rows b
        mm = T(m[:, batch_rows]).transpose(0, 1)
        xq = T(z[:, queries]).transpose(0, 1)             # logical rows q (for the bias): [Q, n, c]
    else:
        x = T(z[batch_rows])
        mm = T(m[batch_rows])
        xq = T(z[queries])
    nx = ln(x, w["queryNormScale"], w["queryNormOffset"], eps)
    q = nx[:, queries] @ T(w["queryWeight"])
    k, v = nx @ T(w["keyWeight"]), nx @ T(w["valueWeight"])
    g = torch.sigmoid(nx[:, queries] @ T(w["gatingWeight"]) + T(w["gatingBias"]))
    # bias[h, q, k] = LN(logical z)[q, k] . W
    bias = (ln(xq, w["queryNormScale"], w["queryNormOffset"], eps) @ T(pair_bias_weight)).permute(2, 0, 1)   # [H, Q, n]
    B, Q = len(batch_rows), len(queries)
    d = c // heads
    qh = q.view(B, Q, heads, d).permute(0, 2, 1, 3)
    kh = k.view(B, n, heads, d).permute(0, 2, 1, 3)
    vh = v.view(B, n, heads, d).permute(0, 2, 1, 3)
    logits = qh @ kh.transpose(-1, -2) / np.sqrt(d) + bias[None] + (1e9 * (mm - 1.0))[:, None, None, :]
    logits = logits.clamp(-1e8, 1e8)
    p = torch.softmax(logits.to(torch.float32).to(F64), -1)
    o = (p @ vh).permute(0, 2, 1, 3).reshape(B, Q, c) * g
    return (o @ T(w["outputWeight"]) + T(w["outputBias"])).numpy()
