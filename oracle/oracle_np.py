"""Second, independent formulation of the same path in numpy.

TEST INFRASTRUCTURE ONLY (see oracle.py). Two uses:
  * dtype=float64: separates rounding of the fp32 oracle from real disagreement
    (the C oracle must agree with this to ~1e-5 relative);
  * dtype=float32: every matrix product goes through numpy's BLAS sgemm, which
    stands in for the `cblas_sgemm` call site the reference uses when built with
    MKL or Accelerate (Engine/CPU/Numeric/CPUFloat.swift:269-279). This is the
    multi-threaded CPU baseline of the benchmark.
The op order follows the same DL4S layers as dl4s_ref.c.
"""
from __future__ import annotations

import numpy as np


def sdpa(q, k, v, mask=None, temperature=None, dtype=np.float64):
    q = np.asarray(q, dtype)
    k = np.asarray(k, dtype)
    v = np.asarray(v, dtype)
    dk = q.shape[-1]
    t = dtype(np.sqrt(dtype(dk))) if temperature is None else dtype(temperature)
    s = np.matmul(q * (dtype(1) / t), np.swapaxes(k, -1, -2))
    if mask is not None:
        s = s - np.asarray(mask, dtype) * dtype(1e9)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    p = e * (dtype(1) / e.sum(axis=-1, keepdims=True))
    return np.matmul(p, v)


def layernorm(x, scale, shift, dtype=np.float64):
    x = np.asarray(x, dtype)
    axes = tuple(range(1, x.ndim))
    m = x.mean(axis=axes, keepdims=True)
    var = (x * x).mean(axis=axes, keepdims=True) - m * m
    return (x - m) / (np.sqrt(var) + dtype(1e-5)) * np.asarray(scale, dtype) + np.asarray(shift, dtype)


def mha(xq, xk, xv, Wq, Wk, Wv, Wo, ln_scale, ln_shift, heads, mask=None, dtype=np.float64):
    xq = np.asarray(xq, dtype)
    xk = np.asarray(xk, dtype)
    xv = np.asarray(xv, dtype)
    B, Sq, D = xq.shape
    Sk = xk.shape[1]
    dk = Wq.shape[1] // heads
    dv = Wv.shape[1] // heads
    q = (xq @ np.asarray(Wq, dtype)).reshape(B, Sq, heads, dk).transpose(0, 2, 1, 3)
    k = (xk @ np.asarray(Wk, dtype)).reshape(B, Sk, heads, dk).transpose(0, 2, 1, 3)
    v = (xv @ np.asarray(Wv, dtype)).reshape(B, Sk, heads, dv).transpose(0, 2, 1, 3)
    a = sdpa(q, k, v, mask, dtype=dtype).transpose(0, 2, 1, 3).reshape(B, Sq, heads * dv)
    return layernorm(a @ np.asarray(Wo, dtype) + xq, ln_scale, ln_shift, dtype)


def gelu_sigmoid(t, dtype=np.float64):
    return t * (dtype(0.5) * np.tanh(t * dtype(1.702) * dtype(0.5)) + dtype(0.5))


def ffn(x, W1, b1, W2, b2, ln_scale, ln_shift, act=0, dtype=np.float64):
    x = np.asarray(x, dtype)
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    h = x2 @ np.asarray(W1, dtype) + np.asarray(b1, dtype)
    h = gelu_sigmoid(h, dtype) if act == 0 else np.maximum(h, 0)
    o = h @ np.asarray(W2, dtype) + np.asarray(b2, dtype) + x2
    return layernorm(o, ln_scale, ln_shift, dtype).reshape(shp)


def encoder(x, layers, heads, lengths=None, act=0, dtype=np.float64):
    x = np.asarray(x, dtype)
    B, S, _ = x.shape
    mask = None
    if lengths is not None:
        mask = (np.arange(S)[None, :] >= np.asarray(lengths)[:, None]).astype(dtype).reshape(B, 1, 1, S)
    for l in layers:
        x = mha(x, x, x, l["Wq"], l["Wk"], l["Wv"], l["Wo"], l["ln1_scale"], l["ln1_shift"], heads, mask, dtype)
        x = ffn(x, l["W1"], l["b1"], l["W2"], l["b2"], l["ln2_scale"], l["ln2_shift"], act, dtype)
    return x


def positional_encoding(S, D, dtype=np.float64):
    half = D // 2
    f = np.exp(np.log(dtype(10000)) * (np.arange(half, dtype=dtype) / dtype(half)))
    a = np.arange(S, dtype=dtype)[:, None] / f[None, :]
    return np.stack([np.sin(a), np.cos(a)], axis=2).reshape(S, D)


def output_head(x, E, bias=None, dtype=np.float64):
    """logSoftmax(x . E^T + bias) over the vocabulary (Transformer.swift:105-108)."""
    z = np.asarray(x, dtype) @ np.asarray(E, dtype).T
    if bias is not None:
        z = z + np.asarray(bias, dtype)
    z = z - z.max(axis=-1, keepdims=True)
    return z - np.log(np.exp(z).sum(axis=-1, keepdims=True))


def sdpa_backward(q, k, v, dout, mask=None, temperature=None, dtype=np.float64):
    """Closed-form gradients of sdpa() above (float64 cross-check of the C restatement)."""
    q, k, v, dout = (np.asarray(a, dtype) for a in (q, k, v, dout))
    t = np.sqrt(q.shape[-1]) if temperature is None else temperature
    s = (q / t) @ np.swapaxes(k, -1, -2)
    if mask is not None:
        s = s - np.asarray(mask, dtype) * 1e9
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    p = e / e.sum(axis=-1, keepdims=True)
    dp = dout @ np.swapaxes(v, -1, -2)
    ds = p * (dp - (dp * p).sum(axis=-1, keepdims=True))
    return (ds @ k) / t, np.swapaxes(ds, -1, -2) @ (q / t), np.swapaxes(p, -1, -2) @ dout


def layernorm_backward(x, dy, scale, dtype=np.float64):
    """Closed-form gradients of layernorm() above with respect to x, scale and shift (float64 cross-check, pinned by
    finite differences in tests/test_oracle.py)."""
    x, dy, scale = (np.asarray(a, dtype) for a in (x, dy, scale))
    axes = tuple(range(1, x.ndim))
    n = np.prod(x.shape[1:])
    m = x.mean(axis=axes, keepdims=True)
    sd = np.sqrt((x * x).mean(axis=axes, keepdims=True) - m * m)
    s = sd + dtype(1e-5)
    xh = (x - m) / s
    a = dy * scale
    dx = (a - a.mean(axis=axes, keepdims=True) - xh * (a * xh).mean(axis=axes, keepdims=True) * (s / sd)) / s
    red = tuple(range(x.ndim - 1))
    return dx, (dy * xh).sum(axis=red), dy.sum(axis=red)
