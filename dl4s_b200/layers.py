"""The DL4S transformer layers on the hot path, bound to the CUDA device.

Class names, initialiser arguments and parameter names follow
Sources/DL4S/NN/Models/Transformer/*.swift and NN/Layer/{LayerNorm,Dense}.swift
so that code written against DL4S's layer API reads the same here. Each
`__call__` forwards to one fused entry point of libdl4s_cuda.so; there is no
host arithmetic and no fallback.

Weights are host numpy arrays at construction (the harness supplies identical
arrays to the CPU oracle and to this device) and live on the device afterwards.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import c_f32, c_vp, call
from .cuda import CUDA, CUDAEngine, ShapedBuffer, StructuredMask, _mask_args, makeEncoderMasks, tensor


def xavier_uniform(rng: np.random.Generator, fan_in: int, fan_out: int) -> np.ndarray:
    a = np.sqrt(6.0 / (fan_in + fan_out))
    return rng.uniform(-a, a, size=(fan_in, fan_out)).astype(np.float32)


class LayerNorm:
    """NN/Layer/LayerNorm.swift:29-77 — statistics over every axis but the first."""

    def __init__(self, inputSize: Sequence[int]):
        self.shift = tensor(np.zeros(inputSize, np.float32))
        self.scale = tensor(np.ones(inputSize, np.float32))

    @property
    def parameters(self):
        return [self.shift, self.scale]

    def __call__(self, inputs: ShapedBuffer, residual: Optional[ShapedBuffer] = None) -> ShapedBuffer:
        out = CUDA.Memory.allocateBuffer(inputs.shape)
        CUDAEngine.layerNorm(inputs, residual, self.scale, self.shift, out)
        return out


class Dropout:
    """NN/Layer/Dropout.swift:29-57: inputs * bernoulli(1 - rate) while `isActive`, without rescaling. The mask is a
    counter-based hash on the device (include/dl4s_cuda.h); `seed` and the device's dropout counter determine it."""

    def __init__(self, rate: float, seed: int = 0):
        self.rate, self.seed, self.isActive = float(rate), int(seed), True

    parameters: list = []

    def __call__(self, inputs: ShapedBuffer) -> ShapedBuffer:
        if not self.isActive or self.rate == 0.0:
            return inputs
        out = CUDA.Memory.allocateBuffer(inputs.shape)
        cur = ctypes.c_uint32(0)
        call("dl4s_cuda_dropout_counter", ctypes.byref(cur), None)
        nxt = ctypes.c_uint32(cur.value + 1)
        call("dl4s_cuda_dropout_counter", None, ctypes.byref(nxt))
        call("dl4s_cuda_dropout", c_vp(inputs.ptr), c_vp(out.ptr), inputs.count, c_f32(self.rate), self.seed, cur.value)
        return out


def setDropout(rate: float, seed: int = 0) -> None:
    """Rate and seed of the dropout fused into MultiHeadAttention, PointwiseFeedForward and the input embedding on the
    current device (the `dropout` arguments of the reference's initialisers); 0 turns it off."""
    call("dl4s_cuda_set_dropout", c_f32(rate), int(seed))


def dropoutCounter(set_to: Optional[int] = None) -> int:
    cur = ctypes.c_uint32(0)
    if set_to is None:
        call("dl4s_cuda_dropout_counter", ctypes.byref(cur), None)
    else:
        v = ctypes.c_uint32(set_to)
        call("dl4s_cuda_dropout_counter", ctypes.byref(cur), ctypes.byref(v))
    return cur.value


class ScaledDotProductAttention:
    """NN/Models/Transformer/ScaledDotProductAttention.swift:29-64."""

    def __init__(self, temperature: float, precision: Optional[int] = None):
        self.temperature = float(temperature)
        self.precision = precision

    parameters: list = []

    def __call__(self, q: ShapedBuffer, k: ShapedBuffer, v: ShapedBuffer, mask=None) -> ShapedBuffer:
        assert k.dim == 4
        out = CUDA.Memory.allocateBuffer((q.shape[0], q.shape[1], q.shape[2], v.shape[3]))
        if q.shape[2] == 1 and (mask is None or (isinstance(mask, StructuredMask) and not mask.causal)):
            lengths = mask.lengths if isinstance(mask, StructuredMask) else None
            CUDAEngine.scaledDotProductAttentionDecode(q, k, v, lengths, self.temperature, out)
        else:
            CUDAEngine.scaledDotProductAttention(q, k, v, mask, self.temperature, out, self.precision)
        return out


def scaledDotProductAttentionBackward(q: ShapedBuffer, k: ShapedBuffer, v: ShapedBuffer, dout: ShapedBuffer, mask=None,
                                      temperature: Optional[float] = None, precision: int = _lib.PREC_FP32, out=None):
    """Gradients of ScaledDotProductAttention with respect to q, k and v for the upstream gradient dout: what the
    backward closures of DL4S's primitives produce (Matrix.swift:139-173, Unary.swift:190-194), in one call.
    `out` = (dq, dk, dv) buffers to write into (allocated here when absent)."""
    B, H, Sq, dk = q.shape
    Sk, dv = v.shape[2], v.shape[3]
    t = float(np.sqrt(np.float32(dk))) if temperature is None else float(temperature)
    lp, causal, mp, ms, _keep = _mask_args(mask)
    dq, dkk, dvv = out if out is not None else (CUDA.Memory.allocateBuffer(t_.shape) for t_ in (q, k, v))
    call("dl4s_cuda_sdpa_backward", c_vp(q.ptr), c_vp(k.ptr), c_vp(v.ptr), c_vp(dout.ptr), B, H, Sq, Sk, dk, dv, c_f32(t), lp,
         causal, mp, ms, c_vp(dq.ptr), c_vp(dkk.ptr), c_vp(dvv.ptr), precision)
    return dq, dkk, dvv


class MultiHeadAttention:
    """NN/Models/Transformer/MultiHeadAttention.swift:29-127. Dropout is inactive
    (rate 0), as in the reference's own transformer test (TransformerTests.swift:31)."""

    def __init__(self, heads: int, hiddenDim: int, keyDim: int, valueDim: int, rng: Optional[np.random.Generator] = None,
                 weights: Optional[dict] = None, precision: Optional[int] = None):
        self.heads, self.keyDim, self.valueDim, self.hiddenDim = heads, keyDim, valueDim, hiddenDim
        self.precision = precision
        if weights is None:
            rng = rng or np.random.default_rng(0)
            weights = {
                "qDense": xavier_uniform(rng, hiddenDim, keyDim * heads),
                "kDense": xavier_uniform(rng, hiddenDim, keyDim * heads),
                "vDense": xavier_uniform(rng, hiddenDim, valueDim * heads),
                "fc": xavier_uniform(rng, valueDim * heads, hiddenDim),
            }
        self.host_weights = weights
        self.qDense = tensor(weights["qDense"])
        self.kDense = tensor(weights["kDense"])
        self.vDense = tensor(weights["vDense"])
        self.fc = tensor(weights["fc"])
        self.attn = ScaledDotProductAttention(float(np.sqrt(np.float32(keyDim))), precision)
        self.norm = LayerNorm([hiddenDim])
        if "norm_scale" in weights:
            self.norm.scale = tensor(weights["norm_scale"])
            self.norm.shift = tensor(weights["norm_shift"])

    @property
    def parameters(self):
        return [self.qDense, self.kDense, self.vDense, self.fc] + self.norm.parameters

    def __call__(self, q: ShapedBuffer, k: ShapedBuffer, v: ShapedBuffer, mask=None,
                 out: Optional[ShapedBuffer] = None) -> ShapedBuffer:
        B, Sq, D = q.shape
        Sk = k.shape[1]
        out = out or CUDA.Memory.allocateBuffer((B, Sq, D))
        lp, causal, mp, ms, _keep = _mask_args(mask)
        prec = CUDAEngine.precision if self.precision is None else self.precision
        call("dl4s_cuda_mha_forward", c_vp(q.ptr), c_vp(k.ptr), c_vp(v.ptr), B, Sq, Sk, D, self.heads, self.keyDim,
             self.valueDim, c_vp(self.qDense.ptr), c_vp(self.kDense.ptr), c_vp(self.vDense.ptr), c_vp(self.fc.ptr),
             c_vp(self.norm.scale.ptr), c_vp(self.norm.shift.ptr), lp, causal, mp, ms, c_vp(out.ptr), prec)
        return out

    # ---- incremental decoding (DL4S re-runs the decoder on the whole prefix per generated token,
    # Transformer.swift:118-137; the cache makes one step cost one token)
    def makeCache(self, batch: int, maxLength: int) -> "KVCache":
        return KVCache(batch, self.heads, maxLength, self.keyDim, self.valueDim)

    def prefillCache(self, x: ShapedBuffer, lengths: np.ndarray, cache: "KVCache") -> None:
        """Keys and values of a prompt x [B, S, D] (rows >= lengths[b] are padding) into the cache."""
        from .cuda import _i64arr
        B, S, D = x.shape
        H, L = self.heads, cache.maxLength
        assert S <= L and B == cache.batch
        for w, d, dst in ((self.kDense, self.keyDim, cache.k), (self.vDense, self.valueDim, cache.v)):
            proj = CUDA.Memory.allocateBuffer((B * S, H * d))
            CUDAEngine.gemm(x.view(B * S, D), w, proj)
            # [B, S, H, d] -> [B, H, Lmax, d]
            call("dl4s_cuda_copy_strided_f32", c_vp(proj.ptr), _i64arr([S * H * d, d, H * d, 1]), 0, c_vp(dst.ptr),
                 _i64arr([H * L * d, L * d, d, 1]), 0, _i64arr([B, H, S, d]), 4)
        cache.setLengths(lengths)

    def decodeStep(self, x: ShapedBuffer, cache: "KVCache", out: Optional[ShapedBuffer] = None) -> ShapedBuffer:
        """x [B, D]: the current token per sequence. Appends its key/value to the cache, attends over the cache and
        itself, applies Wo + residual + LayerNorm. The cache's lengths advance by one."""
        B, D = x.shape
        out = out or CUDA.Memory.allocateBuffer((B, D))
        call("dl4s_cuda_mha_decode_step", c_vp(x.ptr), B, D, self.heads, self.keyDim, self.valueDim, c_vp(self.qDense.ptr),
             c_vp(self.kDense.ptr), c_vp(self.vDense.ptr), c_vp(self.fc.ptr), c_vp(self.norm.scale.ptr),
             c_vp(self.norm.shift.ptr), c_vp(cache.k.ptr), c_vp(cache.v.ptr), cache.maxLength, c_vp(cache.lengths.ptr),
             c_vp(out.ptr))
        cache.advance()
        return out


class KVCache:
    """Keys [B, H, Lmax, dk] and values [B, H, Lmax, dv] of the tokens a decoder self-attention layer has seen,
    and how many per sequence."""

    def __init__(self, batch: int, heads: int, maxLength: int, keyDim: int, valueDim: int):
        self.batch, self.heads, self.maxLength = batch, heads, maxLength
        self.k = CUDA.Memory.allocateBuffer((batch, heads, maxLength, keyDim))
        self.v = CUDA.Memory.allocateBuffer((batch, heads, maxLength, valueDim))
        self.lengths_host = np.zeros(batch, np.int32)
        self.lengths = tensor(self.lengths_host, np.int32)

    def setLengths(self, lengths: np.ndarray) -> None:
        self.lengths_host = np.asarray(lengths, np.int32).copy()
        CUDA.Memory.assign_from_host(self.lengths_host, self.lengths)

    def advance(self) -> None:
        self.setLengths(np.minimum(self.lengths_host + 1, self.maxLength))


class Dense:
    """NN/Layer/Dense.swift:29-69 (weights [in,out], bias [out])."""

    def __init__(self, inputSize: int, outputSize: int, rng: Optional[np.random.Generator] = None,
                 weights: Optional[np.ndarray] = None, bias: Optional[np.ndarray] = None):
        rng = rng or np.random.default_rng(0)
        w = xavier_uniform(rng, inputSize, outputSize) if weights is None else weights
        b = np.zeros(outputSize, np.float32) if bias is None else bias
        self.host_weights, self.host_bias = w, b
        self.weights, self.bias = tensor(w), tensor(b)


class PointwiseFeedForward:
    """NN/Models/Transformer/PointwiseFeedForward.swift:29-84."""

    def __init__(self, size: int, hiddenSize: int, rng: Optional[np.random.Generator] = None,
                 weights: Optional[dict] = None, activation: int = _lib.ACT_GELU_SIGMOID, precision: Optional[int] = None):
        rng = rng or np.random.default_rng(0)
        w = weights or {}
        self.dense1 = Dense(size, hiddenSize, rng, w.get("W1"), w.get("b1"))
        self.dense2 = Dense(hiddenSize, size, rng, w.get("W2"), w.get("b2"))
        self.norm = LayerNorm([size])
        if "norm_scale" in w:
            self.norm.scale = tensor(w["norm_scale"])
            self.norm.shift = tensor(w["norm_shift"])
        self.size, self.hiddenSize, self.activation, self.precision = size, hiddenSize, activation, precision

    def __call__(self, inputs: ShapedBuffer) -> ShapedBuffer:
        M = inputs.count // self.size
        out = CUDA.Memory.allocateBuffer(inputs.shape)
        prec = CUDAEngine.precision if self.precision is None else self.precision
        call("dl4s_cuda_ffn_forward", c_vp(inputs.ptr), M, self.size, self.hiddenSize, c_vp(self.dense1.weights.ptr),
             c_vp(self.dense1.bias.ptr), c_vp(self.dense2.weights.ptr), c_vp(self.dense2.bias.ptr),
             c_vp(self.norm.scale.ptr), c_vp(self.norm.shift.ptr), self.activation, c_vp(out.ptr), prec)
        return out


def encoder_layer_weights(rng: np.random.Generator, D: int, H: int, dk: int, dv: int, F: int) -> dict:
    """One encoder block's parameters in the order the C ABI packs them."""
    return {
        "Wq": xavier_uniform(rng, D, H * dk), "Wk": xavier_uniform(rng, D, H * dk),
        "Wv": xavier_uniform(rng, D, H * dv), "Wo": xavier_uniform(rng, H * dv, D),
        "ln1_scale": np.ones(D, np.float32), "ln1_shift": np.zeros(D, np.float32),
        "W1": xavier_uniform(rng, D, F), "b1": np.zeros(F, np.float32),
        "W2": xavier_uniform(rng, F, D), "b2": np.zeros(D, np.float32),
        "ln2_scale": np.ones(D, np.float32), "ln2_shift": np.zeros(D, np.float32),
    }


PARAM_ORDER = ("Wq", "Wk", "Wv", "Wo", "ln1_scale", "ln1_shift", "W1", "b1", "W2", "b2", "ln2_scale", "ln2_shift")


class TransformerEncoderBlock:
    """NN/Models/Transformer/TransformerEncoderBlock.swift:29-65."""

    def __init__(self, hiddenDim: int, forwardDim: int, heads: int, keyDim: int, valueDim: int, weights: dict,
                 activation: int = _lib.ACT_GELU_SIGMOID, precision: Optional[int] = None):
        self.selfAttention = MultiHeadAttention(heads, hiddenDim, keyDim, valueDim, weights={
            "qDense": weights["Wq"], "kDense": weights["Wk"], "vDense": weights["Wv"], "fc": weights["Wo"],
            "norm_scale": weights["ln1_scale"], "norm_shift": weights["ln1_shift"]}, precision=precision)
        self.pointwiseFeedForward = PointwiseFeedForward(hiddenDim, forwardDim, weights={
            "W1": weights["W1"], "b1": weights["b1"], "W2": weights["W2"], "b2": weights["b2"],
            "norm_scale": weights["ln2_scale"], "norm_shift": weights["ln2_shift"]}, activation=activation,
            precision=precision)

    def __call__(self, inputs: ShapedBuffer, mask=None) -> ShapedBuffer:
        attn = self.selfAttention(inputs, inputs, inputs, mask)
        return self.pointwiseFeedForward(attn)


class TransformerEncoder:
    """NN/Models/Transformer/TransformerEncoder.swift:29-71. `__call__` runs the
    whole stack in one library call (dl4s_cuda_encoder_forward)."""

    def __init__(self, layerCount: int, heads: int, keyDim: int, valueDim: int, modelDim: int, forwardDim: int,
                 rng: Optional[np.random.Generator] = None, layers: Optional[list] = None,
                 activation: int = _lib.ACT_GELU_SIGMOID, precision: Optional[int] = None):
        rng = rng or np.random.default_rng(0)
        self.layerCount, self.heads, self.keyDim, self.valueDim = layerCount, heads, keyDim, valueDim
        self.modelDim, self.forwardDim, self.activation, self.precision = modelDim, forwardDim, activation, precision
        self.host_layers = layers or [encoder_layer_weights(rng, modelDim, heads, keyDim, valueDim, forwardDim)
                                      for _ in range(layerCount)]
        flat = np.concatenate([np.ascontiguousarray(l[k], np.float32).ravel() for l in self.host_layers
                               for k in PARAM_ORDER]) if layerCount else np.zeros(1, np.float32)
        self.params = tensor(flat)
        self._prepared = {}       # precision -> handle of dl4s_cuda_encoder_prepare

    def prepareWeights(self, precision: Optional[int] = None) -> None:
        """Convert the weights for the tensor cores once (DL4S keeps parameters as fp32 tensors; the half copies
        the kernels read do not change between inference calls). Done on the first forward if not called."""
        prec = CUDAEngine.precision if precision is None else precision
        if prec == _lib.PREC_FP32 or prec in self._prepared or self.layerCount == 0:
            return
        h = c_vp(0)
        call("dl4s_cuda_encoder_prepare", self.modelDim, self.heads, self.keyDim, self.valueDim, self.forwardDim,
             self.layerCount, c_vp(self.params.ptr), prec, ctypes.byref(h))
        self._prepared[prec] = h

    def weightsChanged(self) -> None:
        """Call after writing new values into `params` (an optimiser step): the prepared copies are converted again."""
        for h in self._prepared.values():
            call("dl4s_cuda_encoder_prepared_refresh", h)

    def releasePreparedWeights(self) -> None:
        for h in self._prepared.values():
            call("dl4s_cuda_encoder_prepared_destroy", h)
        self._prepared = {}

    def __del__(self):
        try:
            for h in self._prepared.values():
                _lib.load().dl4s_cuda_encoder_prepared_destroy(h)
        except Exception:
            pass

    def __call__(self, inputs: ShapedBuffer, sequenceLengths=None, out: Optional[ShapedBuffer] = None) -> ShapedBuffer:
        B, S, D = inputs.shape
        mask = sequenceLengths if isinstance(sequenceLengths, StructuredMask) else (
            makeEncoderMasks(sequenceLengths) if sequenceLengths is not None else None)
        lp = c_vp(mask.lengths.ptr) if mask is not None and mask.lengths is not None else c_vp(0)
        out = out or CUDA.Memory.allocateBuffer((B, S, D))
        prec = CUDAEngine.precision if self.precision is None else self.precision
        if prec != _lib.PREC_FP32 and self.layerCount > 0:
            self.prepareWeights(prec)
            try:
                call("dl4s_cuda_encoder_forward_prepared", self._prepared[prec], c_vp(inputs.ptr), B, S, lp, self.activation,
                     c_vp(out.ptr))
                return out
            except _lib.DL4SCudaError as e:
                if e.status != -4:      # DL4S_ERR_UNSUPPORTED: a shape outside the tensor-core pipeline
                    raise
        call("dl4s_cuda_encoder_forward", c_vp(inputs.ptr), B, S, D, self.heads, self.keyDim, self.valueDim,
             self.forwardDim, self.layerCount, c_vp(self.params.ptr), lp, self.activation, c_vp(out.ptr), prec)
        return out


class EmbeddingWithPositions:
    """Transformer.prepareInputs (NN/Models/Transformer/Transformer.swift:82-88):
    Embedding (NN/Layer/Embedding.swift:152-165) scaled by sqrt(D) plus
    PositionalEncoding (PositionalEncoding.swift:52-71), in one kernel."""

    def __init__(self, embeddingMatrix: np.ndarray, ignoreIndex: int = -1):
        self.vocab, self.size = embeddingMatrix.shape
        self.embeddingMatrix = tensor(embeddingMatrix)
        self.ignoreIndex = ignoreIndex

    def __call__(self, ids: ShapedBuffer, out: Optional[ShapedBuffer] = None) -> ShapedBuffer:
        B, S = ids.shape
        out = out or CUDA.Memory.allocateBuffer((B, S, self.size))
        call("dl4s_cuda_embed_positional", c_vp(ids.ptr), B, S, self.size, c_vp(self.embeddingMatrix.ptr), self.vocab,
             self.ignoreIndex, c_vp(out.ptr))
        return out


class OutputHead:
    """The last step of Transformer.callAsFunction (NN/Models/Transformer/Transformer.swift:105-108):
    logSoftmax(decoded . embeddingMatrix^T + outputBias) over the vocabulary, with the embedding tied."""

    def __init__(self, embedding: "EmbeddingWithPositions", outputBias: Optional[np.ndarray] = None,
                 precision: Optional[int] = None):
        self.embedding = embedding
        self.outputBias = tensor(np.zeros(embedding.vocab, np.float32) if outputBias is None else outputBias)
        self.precision = precision

    def __call__(self, decoded: ShapedBuffer, out: Optional[ShapedBuffer] = None) -> ShapedBuffer:
        D = decoded.shape[-1]
        M = decoded.count // D
        V = self.embedding.vocab
        out = out or CUDA.Memory.allocateBuffer(tuple(decoded.shape[:-1]) + (V,))
        prec = CUDAEngine.precision if self.precision is None else self.precision
        call("dl4s_cuda_output_head", c_vp(decoded.ptr), M, D, c_vp(self.embedding.embeddingMatrix.ptr), V,
             c_vp(self.outputBias.ptr), c_vp(out.ptr), prec)
        return out


DECODER_PARAM_ORDER = ("self_Wq", "self_Wk", "self_Wv", "self_Wo", "self_ln_scale", "self_ln_shift",
                       "enc_Wq", "enc_Wk", "enc_Wv", "enc_Wo", "enc_ln_scale", "enc_ln_shift",
                       "W1", "b1", "W2", "b2", "ln_scale", "ln_shift")


def decoder_layer_weights(rng: np.random.Generator, D: int, H: int, dk: int, dv: int, F: int) -> dict:
    """One decoder block's parameters in the order the C ABI packs them (TransformerDecoderBlock.parameters)."""
    w = {}
    for pre in ("self", "enc"):
        w[f"{pre}_Wq"] = xavier_uniform(rng, D, H * dk)
        w[f"{pre}_Wk"] = xavier_uniform(rng, D, H * dk)
        w[f"{pre}_Wv"] = xavier_uniform(rng, D, H * dv)
        w[f"{pre}_Wo"] = xavier_uniform(rng, H * dv, D)
        w[f"{pre}_ln_scale"] = np.ones(D, np.float32)
        w[f"{pre}_ln_shift"] = np.zeros(D, np.float32)
    w.update({"W1": xavier_uniform(rng, D, F), "b1": np.zeros(F, np.float32), "W2": xavier_uniform(rng, F, D),
              "b2": np.zeros(D, np.float32), "ln_scale": np.ones(D, np.float32), "ln_shift": np.zeros(D, np.float32)})
    return w


class TransformerDecoder:
    """NN/Models/Transformer/TransformerDecoder.swift:29-62 with TransformerDecoderBlock.swift:29-68. `__call__` runs
    the whole stack in one library call (dl4s_cuda_decoder_forward); `makeCache` / `step` decode incrementally."""

    def __init__(self, layerCount: int, heads: int, keyDim: int, valueDim: int, modelDim: int, forwardDim: int,
                 rng: Optional[np.random.Generator] = None, layers: Optional[list] = None,
                 activation: int = _lib.ACT_GELU_SIGMOID, precision: Optional[int] = None):
        rng = rng or np.random.default_rng(0)
        self.layerCount, self.heads, self.keyDim, self.valueDim = layerCount, heads, keyDim, valueDim
        self.modelDim, self.forwardDim, self.activation, self.precision = modelDim, forwardDim, activation, precision
        self.host_layers = layers or [decoder_layer_weights(rng, modelDim, heads, keyDim, valueDim, forwardDim)
                                      for _ in range(layerCount)]
        flat = np.concatenate([np.ascontiguousarray(l[k], np.float32).ravel() for l in self.host_layers
                               for k in DECODER_PARAM_ORDER]) if layerCount else np.zeros(1, np.float32)
        self.params = tensor(flat)

    def __call__(self, decoderInput: ShapedBuffer, encoderStates: ShapedBuffer, encoderInputLengths=None,
                 decoderInputLengths=None, out: Optional[ShapedBuffer] = None) -> ShapedBuffer:
        B, St, D = decoderInput.shape
        Ss = encoderStates.shape[1]
        el = None if encoderInputLengths is None else tensor(np.asarray(encoderInputLengths, np.int32), np.int32)
        dl = None if decoderInputLengths is None else tensor(np.asarray(decoderInputLengths, np.int32), np.int32)
        out = out or CUDA.Memory.allocateBuffer((B, St, D))
        prec = CUDAEngine.precision if self.precision is None else self.precision
        call("dl4s_cuda_decoder_forward", c_vp(decoderInput.ptr), c_vp(encoderStates.ptr), B, St, Ss, D, self.heads, self.keyDim,
             self.valueDim, self.forwardDim, self.layerCount, c_vp(self.params.ptr), c_vp(dl.ptr if dl else 0),
             c_vp(el.ptr if el else 0), self.activation, c_vp(out.ptr), prec)
        return out

    def makeCache(self, batch: int, maxLength: int, encoderStates: ShapedBuffer, encoderInputLengths=None) -> "DecoderCache":
        return DecoderCache(self, batch, maxLength, encoderStates, encoderInputLengths)


class DecoderCache:
    """Per-layer self-attention key/value caches and the encoder keys/values projected once, for incremental
    decoding with TransformerDecoder.step-wise calls (dl4s_cuda_decoder_cache_* / dl4s_cuda_decoder_step)."""

    def __init__(self, decoder: TransformerDecoder, batch: int, maxLength: int, encoderStates: ShapedBuffer,
                 encoderInputLengths=None):
        self.decoder = decoder
        self.batch = batch
        d = decoder
        self._h = c_vp(0)
        call("dl4s_cuda_decoder_cache_create", batch, maxLength, encoderStates.shape[1], d.modelDim, d.heads, d.keyDim, d.valueDim,
             d.forwardDim, d.layerCount, c_vp(d.params.ptr), ctypes.byref(self._h))
        self.setEncoder(encoderStates, encoderInputLengths)

    def setEncoder(self, encoderStates: ShapedBuffer, encoderInputLengths=None) -> None:
        el = None if encoderInputLengths is None else tensor(np.asarray(encoderInputLengths, np.int32), np.int32)
        call("dl4s_cuda_decoder_cache_set_encoder", self._h, c_vp(encoderStates.ptr), c_vp(el.ptr if el else 0))

    def step(self, x: ShapedBuffer, out: Optional[ShapedBuffer] = None) -> ShapedBuffer:
        """x [B, D]: the current token's embedded input per sequence -> the decoder's output row per sequence."""
        out = out or CUDA.Memory.allocateBuffer(x.shape)
        call("dl4s_cuda_decoder_step", self._h, c_vp(x.ptr), self.decoder.activation, c_vp(out.ptr))
        return out

    def destroy(self) -> None:
        if self._h:
            call("dl4s_cuda_decoder_cache_destroy", self._h)
            self._h = c_vp(0)

    def __del__(self):
        try:
            if self._h:
                _lib.load().dl4s_cuda_decoder_cache_destroy(self._h)
        except Exception:
            pass


class Transformer:
    """NN/Models/Transformer/Transformer.swift:29-137: shared embedding, encoder, decoder, tied output head.
    `__call__` is the teacher-forced forward (:96-108); `greedyDecode` is callAsFunction(inputSequence:...) (:118-137)."""

    def __init__(self, encoderLayers: int, decoderLayers: int, vocabSize: int, hiddenDim: int, heads: int, keyDim: int,
                 valueDim: int, forwardDim: int, rng: Optional[np.random.Generator] = None, weights: Optional[dict] = None,
                 precision: Optional[int] = None):
        rng = rng or np.random.default_rng(0)
        w = weights or {}
        E = w.get("embedding")
        if E is None:
            E = (rng.standard_normal((vocabSize, hiddenDim)) * 0.02).astype(np.float32)
        self.vocabSize, self.hiddenDim, self.precision = vocabSize, hiddenDim, precision
        self.embedding = EmbeddingWithPositions(E, ignoreIndex=-1)
        self.encoder = TransformerEncoder(encoderLayers, heads, keyDim, valueDim, hiddenDim, forwardDim, rng=rng,
                                          layers=w.get("encoder"), precision=precision)
        self.decoder = TransformerDecoder(decoderLayers, heads, keyDim, valueDim, hiddenDim, forwardDim, rng=rng,
                                          layers=w.get("decoder"), precision=precision)
        self.head = OutputHead(self.embedding, w.get("outputBias"), precision=precision)

    def __call__(self, encoderInput: np.ndarray, decoderInput: np.ndarray, encoderInputLengths, decoderInputLengths) -> ShapedBuffer:
        enc_in = self.embedding(tensor(encoderInput, np.int32))
        dec_in = self.embedding(tensor(decoderInput, np.int32))
        states = self.encoder(enc_in, np.asarray(encoderInputLengths, np.int32))
        decoded = self.decoder(dec_in, states, encoderInputLengths, decoderInputLengths)
        return self.head(decoded)

    def greedyDecode(self, inputSequence, startToken: int, endToken: int, maxLength: int, cached: bool = False):
        ids = np.ascontiguousarray(inputSequence, np.int32)
        toks = np.zeros(maxLength, np.int32)
        n = ctypes.c_int64(0)
        e, d = self.encoder, self.decoder
        prec = CUDAEngine.precision if self.precision is None else self.precision
        call("dl4s_cuda_transformer_greedy_decode", ids.ctypes.data_as(_lib.c_i32p), len(ids), startToken, endToken, maxLength,
             self.vocabSize, self.hiddenDim, e.heads, e.keyDim, e.valueDim, e.forwardDim, e.layerCount, d.layerCount,
             c_vp(self.embedding.embeddingMatrix.ptr), c_vp(e.params.ptr), c_vp(d.params.ptr), e.activation, prec, int(cached),
             toks.ctypes.data_as(_lib.c_i32p), ctypes.byref(n))
        return toks[:n.value].tolist()
