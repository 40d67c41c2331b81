"""Block and stack runners: the order and residual wiring of the pair stack.

Mirrors ``EvoformerBlockGpu`` / ``EvoformerStackGpu`` / ``ExtraMsaPairStackGpu``
(``webgpu/af2/evoformer/block.js:1783-1824``, ``webgpu/af2/evoformer/stack.js:44,163``)
and ``Af3PairformerStackGpu`` (``webgpu/af3/trunk/pairformer-block.js:246-343``).
Every update is added into the running pair, which stays resident on the device
for the whole stack (``pairTensor`` / ``pairBuffer`` in the reference).
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _native as nat
from .operators import (AttentionGpu, Af3SingleAttentionGpu, Af3TransitionGpu, OuterProductMeanGpu,
                        PreparedWeights, TransitionGpu, _Buffer, _device, _precision, _variance,
                        prepare_single_attention_weights,
                        SINGLE_ATTENTION_AF3_ORDER, TRANSITION_AF3_ORDER, TRANSITION_WEIGHT_ORDER,
                        prepare_attention_weights, prepare_grid_attention_weights,
                        prepare_triangle_weights)


class PreparedPairBlock:
    """Resident weights of the five pair updates of one block."""

    def __init__(self, device, w, c_z, c_hidden):
        self.device = device
        af3 = "pairAttention1" in w
        self.af3 = af3
        self.tri_out = prepare_triangle_weights(device, w["triangleMultiplicationOutgoing"], c_z, c_hidden)
        self.tri_in = prepare_triangle_weights(device, w["triangleMultiplicationIncoming"], c_z, c_hidden)
        if af3:
            self.att_start = prepare_grid_attention_weights(device, w["pairAttention1"], c_z)
            self.att_end = prepare_grid_attention_weights(device, w["pairAttention2"], c_z)
            self.heads = int(w["pairAttention1"]["heads"])
            t = w["pairTransition"]
            self.transition_hidden = int(t["transition2"].shape[0])
            self.transition = PreparedWeights(device, nat.WEIGHTS_TRANSITION_AF3,
                                              {"channels": c_z, "hidden": self.transition_hidden},
                                              [t[k] for k in TRANSITION_AF3_ORDER])
        else:
            s, e = w["triangleAttentionStarting"], w["triangleAttentionEnding"]
            self.heads = int(s["heads"])
            self.att_start = prepare_attention_weights(device, s["attention"], c_z, s["heads"],
                                                       dict(s["pairBias"], source="normalized-input"))
            self.att_end = prepare_attention_weights(device, e["attention"], c_z, e["heads"],
                                                     dict(e["pairBias"], source="normalized-input"))
            t = w["pairTransition"]
            self.transition_hidden = np.asarray(t["firstBias"]).size
            self.transition = PreparedWeights(device, nat.WEIGHTS_TRANSITION_AF2,
                                              {"channels": c_z, "hidden": self.transition_hidden},
                                              [t[k] for k in TRANSITION_WEIGHT_ORDER])

    def struct(self):
        return nat.PairBlockWeights(self.tri_out.handle, self.tri_in.handle, self.att_start.handle,
                                    self.att_end.handle, self.transition.handle)

    def close(self):
        for w in (self.tri_out, self.tri_in, self.att_start, self.att_end, self.transition):
            w.close()


class PairStackGpu:
    """The five pair updates of ``n_blocks`` blocks on a resident pair
    (``ExtraMsaPairStackGpu`` without its OuterProductMean:
    ``webgpu/af2/evoformer/block.js:1663-1713``; ``encodePairTrack``:
    ``webgpu/af3/trunk/pair-track.js:929``)."""

    def __init__(self, device=None):
        self.device = _device(device)
        self.blocks = []
        self.shape = None

    def prepare(self, block_weights, c_z, c_hidden):
        self.close()
        self.blocks = [w if isinstance(w, PreparedPairBlock) else PreparedPairBlock(self.device, w, c_z, c_hidden)
                       for w in block_weights]
        self.shape = (c_z, c_hidden)
        self._table = (nat.PairBlockWeights * len(self.blocks))(*[b.struct() for b in self.blocks])
        return self

    def run(self, pair, mask, options=None, first_block=0, n_blocks=None, dialect=None, inplace=False):
        """Updates ``pair`` (device tensor: in place; numpy: returns a new array, or
        updates the given float32 array when ``inplace``).  ``options["order"] = "template"`` runs each block
        in the template pair stack's order (attention start, end, triangle out, in, transition:
        ``encodeTemplatePairBlock``, ``webgpu/af2/evoformer/block.js:1746-1781``)."""
        opts = options or {}
        dev = self.device
        c_z, c_hidden = self.shape
        af3 = self.blocks[0].af3
        swap = -1
        if af3:
            if dialect is None or dialect.get("swapTransposedBias") not in (True, False):
                raise ValueError("dialect.swapTransposedBias has no default")
            swap = 1 if dialect["swapTransposedBias"] else 0
        p = _Buffer(pair)
        m = _Buffer(mask)
        n = int(round((p.count // c_z) ** 0.5))
        if n * n * c_z != p.count:
            raise nat.RangeError(f"pair has {p.count} values; expected length*length*{c_z}")
        if m.count != n * n:
            raise nat.RangeError(f"mask has {m.count} values; expected {n * n}")
        if p.is_device:
            target, output = p, pair
        elif inplace:
            if p.keep is not pair and not np.shares_memory(p.keep, pair):
                raise ValueError("inplace needs a contiguous float32 array")
            target, output = p, pair
        else:
            output = np.array(pair, np.float32, copy=True).reshape(n, n, c_z)
            target = _Buffer(output)
        count = len(self.blocks) - first_block if n_blocks is None else n_blocks
        desc = nat.PairStackDesc(n, c_z, c_hidden, self.blocks[0].heads, self.blocks[0].transition_hidden,
                                 _variance(opts, "fast" if af3 else "two-pass"), _precision(opts), swap,
                                 float(opts.get("epsilon") or 1e-5),
                                 nat.SPACE_DEVICE if p.is_device else nat.SPACE_HOST, target.dtype,
                                 target.ptr, m.ptr, self._table, len(self.blocks), first_block, count,
                                 nat.ORDER_TEMPLATE if opts.get("order") == "template" else nat.ORDER_EVOFORMER)
        res = nat.Result()
        dev.check(dev.lib.lf_pair_stack_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
        return {"pair": output, "elapsedMilliseconds": float(res.elapsed_ms),
                "memory": {"peakBytes": int(res.peak_bytes)}, "launches": int(res.launches), "blocks": count}

    def close(self):
        for b in self.blocks:
            b.close()
        self.blocks = []


class PreparedMsaBlock:
    """Resident weights of one Evoformer or extra-MSA block: the three MSA operators, the outer product mean and
    the five pair updates (``weights["msaColumnGlobalAttention"]`` makes it an extra-MSA block)."""

    def __init__(self, device, w, c_m, c_z, c_outer, c_hidden):
        from .operators import GLOBAL_ATTENTION_ORDER, OPM_WEIGHT_ORDER
        self.device = device
        self.dims = (c_m, c_z, c_outer, c_hidden)
        row = w["msaRowAttention"]
        self.row_heads = int(row["heads"])
        self.row = prepare_attention_weights(device, row["attention"], c_m, self.row_heads,
                                             dict(row["pairBias"], source="separate", channels=c_z))
        self.global_column = "msaColumnGlobalAttention" in w
        if self.global_column:
            g = w["msaColumnGlobalAttention"]
            heads = g.get("heads")
            if not isinstance(heads, (int, np.integer)) or heads <= 0:
                raise nat.RangeError("global attention weights.heads must be a positive integer")
            self.col_heads = int(heads)
            self.col = PreparedWeights(device, nat.WEIGHTS_GLOBAL_ATTENTION_AF2, {"channels": c_m, "heads": self.col_heads},
                                       [g[k] for k in GLOBAL_ATTENTION_ORDER])
        else:
            col = w["msaColumnAttention"]
            self.col_heads = int(col["heads"])
            self.col = prepare_attention_weights(device, col["attention"], c_m, self.col_heads)
        t = w["msaTransition"]
        self.transition_hidden = np.asarray(t["firstBias"]).size
        self.transition = PreparedWeights(device, nat.WEIGHTS_TRANSITION_AF2,
                                          {"channels": c_m, "hidden": self.transition_hidden},
                                          [t[k] for k in TRANSITION_WEIGHT_ORDER])
        self.opm = PreparedWeights(device, nat.WEIGHTS_OPM_AF2, {"channels": c_m, "hidden": c_outer, "out_channels": c_z},
                                   [w["outerProductMean"][k] for k in OPM_WEIGHT_ORDER])
        self.pair = PairStackGpu(device).prepare([w], c_z, c_hidden)

    def run(self, msa, pair, msa_mask, pair_mask, S, n, opts):
        """One block in place on the device tensors ``msa`` [S, n, c_m] and ``pair`` [n, n, c_z]; returns its launches."""
        from .operators import GlobalColumnAttentionGpu
        dev = self.device
        cm, cz, co, _ = self.dims
        sub = dict(opts, residual=True)
        launches = 0
        r = AttentionGpu(dev).run({"activations": msa, "mask": msa_mask, "batch": S, "queryLength": n, "channels": cm,
                                   "heads": self.row_heads, "weights": self.row,
                                   "pairBias": {"source": "separate", "activations": pair, "channels": cz}}, sub, out=msa)
        launches += r["launches"]
        if self.global_column:
            r = GlobalColumnAttentionGpu(dev).run({"activations": msa, "mask": msa_mask, "sequences": S, "length": n,
                                                   "channels": cm, "weights": self.col}, sub, out=msa)
        else:
            r = AttentionGpu(dev).run({"activations": msa, "mask": msa_mask, "batch": n, "queryLength": S, "channels": cm,
                                       "heads": self.col_heads, "transpose": True, "weights": self.col}, sub, out=msa)
        launches += r["launches"]
        r = TransitionGpu(dev).run({"activations": msa, "rows": S * n, "channels": cm,
                                    "hiddenChannels": self.transition_hidden, "weights": self.transition}, sub, out=msa)
        launches += r["launches"]
        r = OuterProductMeanGpu(dev).run({"activations": msa, "mask": msa_mask, "sequences": S, "length": n, "cM": cm,
                                          "cOuter": co, "cZ": cz, "weights": self.opm}, sub, out=pair)
        launches += r["launches"]
        r = self.pair.run(pair, pair_mask, opts)
        return launches + r["launches"]

    def close(self):
        for w in (self.row, self.col, self.transition, self.opm, self.pair):
            w.close()


class EvoformerStackGpu:
    """``EvoformerStackGpu.run(input)`` (``webgpu/af2/evoformer/stack.js:44-110``): the blocks of the main stack
    one after the other, ``input["blockWeights"]`` one weight object (or ``PreparedMsaBlock``) per block.  The MSA,
    the pair and the masks are uploaded once and stay on the device for the whole stack; device tensors given as
    ``msa`` / ``pair`` are updated in place and returned.  ``ExtraMsaStackGpu`` is the same loop over extra-MSA
    blocks (``webgpu/af2/evoformer/stack.js:163``), told apart by the weights."""

    def __init__(self, device=None):
        self.device = _device(device)

    def run(self, input, options=None):
        import torch
        blocks = input["blockWeights"]
        if len(blocks) == 0:
            raise nat.RangeError("Evoformer stack requires at least one block")
        opts = dict(options or {})
        dev = self.device
        S, n, cm, cz = (int(input[k]) for k in ("sequences", "length", "cM", "cZ"))
        co, ch = int(input["cOuter"]), int(input["triangleHidden"])
        where = f"cuda:{dev.ordinal}"

        def resident(value, shape, copy):
            if getattr(value, "is_cuda", False):
                if value.numel() != int(np.prod(shape)):
                    raise nat.RangeError(f"tensor has {value.numel()} values; expected {int(np.prod(shape))}")
                return value.view(shape), True
            host = np.asarray(value, np.float32)
            if host.size != int(np.prod(shape)):
                raise nat.RangeError(f"array has {host.size} values; expected {int(np.prod(shape))}")
            return torch.from_numpy(np.array(host, np.float32, copy=copy).reshape(shape)).to(where), False

        stream = torch.cuda.ExternalStream(dev.stream, device=where) if dev.stream else torch.cuda.default_stream(where)
        with torch.cuda.stream(stream):       # uploads, the library's kernels and read-backs share one stream
            msa, msa_given = resident(input["msa"], (S, n, cm), True)
            pair, pair_given = resident(input["pair"], (n, n, cz), True)
            msa_mask, _ = resident(input["msaMask"], (S, n), False)
            pair_mask, _ = resident(input["pairMask"], (n, n), False)
            owned = []
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches = 0
            try:
                prepared = []
                for w in blocks:
                    if isinstance(w, PreparedMsaBlock):
                        prepared.append(w)
                    else:
                        prepared.append(PreparedMsaBlock(dev, w, cm, cz, co, ch))
                        owned.append(prepared[-1])
                start.record(stream)
                for index, block in enumerate(prepared):
                    launches += block.run(msa, pair, msa_mask, pair_mask, S, n, opts)
                    if input.get("onBlockDone"):
                        input["onBlockDone"](index)
                stop.record(stream)
                dev.synchronize()
            finally:
                dev.synchronize()
                for block in owned:
                    block.close()
            return {"msa": msa if msa_given else msa.cpu().numpy(), "pair": pair if pair_given else pair.cpu().numpy(),
                    "elapsedMilliseconds": float(start.elapsed_time(stop)), "memory": {"peakBytes": 0},
                    "launches": launches}


class EvoformerBlockGpu(EvoformerStackGpu):
    """One whole AF2 Evoformer block (``webgpu/af2/evoformer/block.js:1536-1613,1783-1824``):
    msa += rowAttention(msa, pair); msa += columnAttention(msa); msa += transition(msa);
    pair += outerProductMean(msa); then the five pair updates.  ``input["weights"]``: the block's weight object."""

    def run(self, input, options=None):
        return EvoformerStackGpu.run(self, dict(input, blockWeights=[input["weights"]]), options)


class ExtraMsaBlockGpu(EvoformerBlockGpu):
    """One block of the AF2 extra-MSA stack (``encodeExtraMsaBlock``, ``webgpu/af2/evoformer/block.js:1715-1744``):
    msa += rowAttention(msa, pair); msa += globalColumnAttention(msa); msa += transition(msa); then the
    Evoformer pair part (pair += outerProductMean(msa) and the five pair updates).  Same input as
    ``EvoformerBlockGpu`` with ``weights["msaColumnGlobalAttention"]`` in place of the column attention."""


class ExtraMsaStackGpu(EvoformerStackGpu):
    """The extra-MSA stack (``encodeExtraMsaBlock`` per block, ``webgpu/af2/evoformer/stack.js:163``)."""


class Af3PairformerStackGpu:
    """``Af3PairformerStackGpu.run(state, blocks, dialect, options)``
    (``webgpu/af3/trunk/pairformer-block.js:290-343``): per block the five pair
    updates, then single += singleAttention(single, pairLogits(pair)) and
    single += transition(single) (``cpu/af3/trunk/pairformer.js:505-539``).

    The pair and the single representation stay on the device for the whole stack, as the
    reference's ``pairBuffer`` / ``singleBuffer`` do (``pairformer-block.js:303-312``): host
    arrays are uploaded once and read back once.  ``state["pair"]`` / ``state["single"]`` may
    also be CUDA tensors (float32 or bfloat16 pair, float32 single), which are then updated in
    place; ``options["keepPair"]`` returns the device tensors as ``pairTensor`` / ``singleTensor``
    and skips the read-back; ``firstBlock`` starts in the middle of the stack."""

    def __init__(self, device=None):
        self.device = _device(device)

    def run(self, state, blocks, dialect, options=None):
        import torch
        if dialect is None or dialect.get("swapTransposedBias") not in (True, False):
            raise ValueError("dialect.swapTransposedBias has no default")
        opts = dict(options or {})
        dev = self.device
        n = int(state["tokens"])
        cz, cs = int(blocks[0]["pairChannels"]), int(blocks[0]["singleChannels"])
        first = int(opts.get("firstBlock", 0))
        where = f"cuda:{dev.ordinal}"

        def resident(value, shape):
            if value is None:
                return None, False
            if getattr(value, "is_cuda", False):
                if tuple(value.shape) != shape and value.numel() != int(np.prod(shape)):
                    raise nat.RangeError(f"state tensor has {value.numel()} values; expected {int(np.prod(shape))}")
                return value.view(shape), True
            host = np.ascontiguousarray(np.asarray(value, np.float32)).reshape(shape)
            return torch.from_numpy(host).to(where), False

        stream = torch.cuda.ExternalStream(dev.stream, device=where) if dev.stream else torch.cuda.default_stream(where)
        with torch.cuda.stream(stream):       # uploads, the library's kernels and read-backs share one stream
            pair, pair_given = resident(state["pair"], (n, n, cz))
            single, single_given = resident(state.get("single"), (n, cs))
            pair_mask, _ = resident(state["pairMask"], (n, n))
            seq_mask = None
            if single is not None:
                seq_mask, _ = resident(state["seqMask"], (n,))
            stack = PairStackGpu(dev).prepare(blocks, cz, cz)
            single_w = []
            if single is not None:       # resident weights of the single track, prepared before the first block runs
                for b in range(first, len(blocks)):
                    t = blocks[b]["singleTransition"]
                    single_w.append((prepare_single_attention_weights(dev, blocks[b], cs, cz),
                                     PreparedWeights(dev, nat.WEIGHTS_TRANSITION_AF3,
                                                     {"channels": cs, "hidden": int(t["transition2"].shape[0])},
                                                     [t[k] for k in TRANSITION_AF3_ORDER])))
            launches = 0
            sub = {"precision": opts.get("precision", "f32"), "residual": True}
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            try:
                for b in range(first, len(blocks)):
                    r = stack.run(pair, pair_mask, opts, first_block=b, n_blocks=1, dialect=dialect)
                    launches += r["launches"]
                    if single is not None:
                        att_w, trn_w = single_w[b - first]
                        r = Af3SingleAttentionGpu(dev).run(single, pair, seq_mask, {"n": n, "channels": cs, "pairChannels": cz},
                                                           att_w, sub)
                        single.copy_(r["output"])
                        launches += r["launches"]
                        r = Af3TransitionGpu(dev).run(single, {"rows": n, "channels": cs, "factor": 4}, trn_w, sub, out=single)
                        launches += r["launches"]
                    if opts.get("onBlockDone"):
                        opts["onBlockDone"](b)
                stop.record(stream)
                dev.synchronize()
            finally:
                dev.synchronize()
                stack.close()
                for pair_of in single_w:
                    for w in pair_of:
                        w.close()
            elapsed = start.elapsed_time(stop)
            out = {"elapsedMilliseconds": float(elapsed), "memory": {"peakBytes": 0}, "launches": launches}
            if opts.get("keepPair"):
                out.update(pair=None, single=None, pairTensor=pair, singleTensor=single)
            else:
                out["pair"] = pair if pair_given else pair.float().cpu().numpy()
                out["single"] = None if single is None else (single if single_given else single.cpu().numpy())
        return out


class Af3MsaStackGpu:
    """``Af3MsaStackGpu.run(state, blocks, dialect, options)`` (``webgpu/af3/trunk/msa-stack.js:67-89``): the
    blocks of the AF3 MSA stack, each ``msaBlock`` (``cpu/af3/trunk/msa.js:235-287``) - the outer product mean
    into the pair and the MSA update (pair-weighted averaging, then the MSA transition) in the order
    ``dialect["msaUpdateBeforeOuterProduct"]`` names (it has no default), followed by the five pair updates;
    ``dialect["opmBiasAfterNorm"]`` moves the outer product's output bias behind the division by the coverage.
    ``state = {msa, pair, msaMask, pairMask, sequences, tokens}``; host arrays are uploaded once, the MSA and the
    pair stay on the device for the whole stack and are read back once; CUDA tensors are updated in place and
    returned (``options["keepPair"]`` returns the device tensors as ``pairTensor`` / ``msaTensor`` either way, the
    hand-over to the pairformer stack that follows); ``options["onBlock"]`` is called after each block."""

    def __init__(self, device=None):
        self.device = _device(device)

    def run(self, state, blocks, dialect, options=None):
        import torch
        from .operators import Af3MsaAttentionGpu, OPM_WEIGHT_ORDER, prepare_msa_attention_weights
        if dialect is None or dialect.get("swapTransposedBias") not in (True, False):
            raise ValueError("dialect.swapTransposedBias has no default")
        if dialect.get("msaUpdateBeforeOuterProduct") not in (True, False):
            raise ValueError("dialect.msaUpdateBeforeOuterProduct has no default: AF3 takes the outer product off "
                             "the pre-update MSA and OpenDDE off the updated one")
        if len(blocks) == 0:
            raise nat.RangeError("the MSA stack requires at least one block")
        opts = dict(options or {})
        dev = self.device
        S, n = int(state["sequences"]), int(state["tokens"])
        cm, cz = int(blocks[0]["msaChannels"]), int(blocks[0]["pairChannels"])
        where = f"cuda:{dev.ordinal}"

        def resident(value, shape):
            if getattr(value, "is_cuda", False):
                if value.numel() != int(np.prod(shape)):
                    raise nat.RangeError(f"state tensor has {value.numel()} values; expected {int(np.prod(shape))}")
                return value.view(shape), True
            host = np.ascontiguousarray(np.asarray(value, np.float32))
            if host.size != int(np.prod(shape)):
                raise nat.RangeError(f"state array has {host.size} values; expected {int(np.prod(shape))}")
            return torch.from_numpy(host.reshape(shape)).to(where), False

        stream = torch.cuda.ExternalStream(dev.stream, device=where) if dev.stream else torch.cuda.default_stream(where)
        with torch.cuda.stream(stream):
            msa, msa_given = resident(state["msa"], (S, n, cm))
            pair, pair_given = resident(state["pair"], (n, n, cz))
            msa_mask, _ = resident(state["msaMask"], (S, n))
            pair_mask, _ = resident(state["pairMask"], (n, n))
            prepared = []
            for w in blocks:      # resident weights of the MSA track, prepared before the first block runs
                opm = w["outerProductMean"]
                co = int(opm["outerChannels"])
                zero = np.zeros(co, np.float32)
                opm_af2 = {"layerNormScale": opm["layerNormInputScale"], "layerNormOffset": opm["layerNormInputOffset"],
                           "leftWeight": opm["leftProjection"], "leftBias": opm.get("leftProjectionBias", zero),
                           "rightWeight": opm["rightProjection"], "rightBias": opm.get("rightProjectionBias", zero),
                           "outputWeight": opm["outputW"], "outputBias": opm["outputB"]}
                t = w["msaTransition"]
                prepared.append((co,
                                 PreparedWeights(dev, nat.WEIGHTS_OPM_AF2, {"channels": cm, "hidden": co, "out_channels": cz},
                                                 [opm_af2[k] for k in OPM_WEIGHT_ORDER]),
                                 prepare_msa_attention_weights(dev, w["msaAttention1"], cm, cz),
                                 PreparedWeights(dev, nat.WEIGHTS_TRANSITION_AF3,
                                                 {"channels": cm, "hidden": int(np.asarray(t["transition2"]).shape[0])},
                                                 [t[k] for k in TRANSITION_AF3_ORDER])))
            stack = PairStackGpu(dev).prepare(blocks, cz, cz)
            sub = {"precision": opts.get("precision", "f32"), "residual": True}
            launches = 0
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            try:
                for b, (co, opm_w, att_w, trn_w) in enumerate(prepared):
                    def outer_product():
                        return OuterProductMeanGpu(dev).run({"sequences": S, "length": n, "cM": cm, "cOuter": co, "cZ": cz,
                                                             "activations": msa, "mask": msa_mask, "weights": opm_w,
                                                             "biasAfterNorm": bool(dialect.get("opmBiasAfterNorm"))},
                                                            dict(sub, variance="fast"), out=pair)["launches"]

                    def update_msa():
                        r1 = Af3MsaAttentionGpu(dev).run(msa, msa_mask, pair, {"sequences": S, "tokens": n, "msaChannels": cm,
                                                                              "pairChannels": cz}, att_w, sub, out=msa)
                        r2 = Af3TransitionGpu(dev).run(msa.view(S * n, cm), {"rows": S * n, "channels": cm, "factor": 4},
                                                       trn_w, sub, out=msa.view(S * n, cm))
                        return r1["launches"] + r2["launches"]

                    if dialect["msaUpdateBeforeOuterProduct"]:
                        launches += update_msa()
                        launches += outer_product()
                    else:
                        launches += outer_product()
                        launches += update_msa()
                    launches += stack.run(pair, pair_mask, opts, first_block=b, n_blocks=1, dialect=dialect)["launches"]
                    if opts.get("onBlock"):
                        opts["onBlock"](b)
                stop.record(stream)
                dev.synchronize()
            finally:
                dev.synchronize()
                stack.close()
                for _, opm_w, att_w, trn_w in prepared:
                    for w in (opm_w, att_w, trn_w):
                        w.close()
            out = {"elapsedMilliseconds": float(start.elapsed_time(stop)), "memory": {"peakBytes": 0}, "launches": launches}
            if opts.get("keepPair"):
                out.update(msa=None, pair=None, msaTensor=msa, pairTensor=pair)
            else:
                out["msa"] = msa if msa_given else msa.cpu().numpy()
                out["pair"] = pair if pair_given else pair.float().cpu().numpy()
        return out


class Af3MsaBlockGpu:
    """One block of the AF3 MSA stack (``msaBlock``, ``cpu/af3/trunk/msa.js:235-287``):
    ``run(state, weights, dialect, options)`` is ``Af3MsaStackGpu.run`` over that one block."""

    def __init__(self, device=None):
        self.device = _device(device)

    def run(self, state, weights, dialect, options=None):
        return Af3MsaStackGpu(self.device).run(state, [weights], dialect, options)
