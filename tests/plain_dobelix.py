"""Plain, slow Dobelix decoder used as the oracle of the test-suite.

Whole sequences only, no cache, no batching, one function per mechanism, numpy
float64 throughout, loops over tokens where the definition is a recurrence.  It
shares no code with the ``hfee_b200`` package: its own safetensors reader, its own
reading of config.json, its own rotary angles.

The design, in the notation used below (x: residual stream [T, width]):

    x   = table[token] * embedding_scale
    per layer:   h = x + conv(x)            causal depthwise convolution over time
                 x = x + norm1(mixer(h))    the norm sits on the sublayer's output
                 x = x + norm2(ffn(x))      (only if the layer has a feed-forward)
    logits = head(norm_final(x)) * logit_scale
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def read_safetensors(path):
    """name -> float64 (or integer) ndarray; bfloat16 is widened by a 16-bit shift."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    kinds = {"F64": "<f8", "F32": "<f4", "F16": "<f2", "I32": "<i4", "I64": "<i8"}
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[lo:hi]
        if meta["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(raw, dtype=kinds[meta["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = arr.reshape(meta["shape"])
    return out


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# --------------------------------------------------------------------------
# one function per mechanism
# --------------------------------------------------------------------------
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(h, w):
    """conv(h)[t] = sum_j w[:, j] * h[t - taps + 1 + j], zeros before the start.  h [T, C], w [C, taps]."""
    T, taps = h.shape[0], w.shape[1]
    out = np.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def lightning_mixer(h, W, p, m, eps):
    """Linear attention with a per-head scalar decay, token by token."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ W[p + "q"].T).reshape(T, H, D)
    k = silu(h @ W[p + "k"].T).reshape(T, H, D)
    v = silu(h @ W[p + "v"].T).reshape(T, H, V)
    o = np.zeros((T, H, V))
    for head in range(H):
        lam = float(m["decay"][head])
        S = np.zeros((D, V))
        for t in range(T):
            S = lam * S + np.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = rms_norm(o.reshape(T, H * V), W[p + "norm"], eps)
    return (o * sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def rotate_half(x, positions, dims, base):
    """x [T, heads, dim]: the first ``dims`` dimensions of each head, dimension i paired with i + dims/2."""
    half = dims // 2
    out = x.copy()
    for i in range(half):
        a = positions * base ** (-2.0 * i / dims)
        c, s = np.cos(a)[:, None], np.sin(a)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def chunk_sigmoid_attention_mixer(h, W, p, m, eps):
    """Grouped-query attention whose values are the raw key projections, with unnormalised
    sigmoid weights and keys visible only inside the query's chunk of positions."""
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = h @ W[p + "q"].T
    k = h @ W[p + "k"].T
    v = k.reshape(T, G, D)                                # as projected: before norm and rotation
    q = rms_norm(q, W[p + "q.norm"], eps).reshape(T, H, D)  # over the whole projection
    k = rms_norm(k, W[p + "k.norm"], eps).reshape(T, G, D)
    pos = np.arange(T, dtype=np.float64)
    q = rotate_half(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half(k, pos, m["rot"]["dims"], m["rot"]["base"])
    size = m["mask"]["size"]
    o = np.zeros((T, H, D))
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            for j in range((i // size) * size, i + 1):          # j <= i and floor(j / size) == floor(i / size)
                score = float(q[i, head] @ k[j, g]) * m["scale"] * W[p + "temp"][head]
                o[i, head] += sigmoid(score + W[p + "pb"][head]) * v[j, g]
    o = o.reshape(T, H * D) * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def gated_mlp(x, W, p):
    return (gelu_tanh(x @ W[p + "gate"].T) * (x @ W[p + "up"].T)) @ W[p + "down"].T


MIXERS = {"lightning": lightning_mixer, "attention": chunk_sigmoid_attention_mixer}


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] (and the residual stream after every layer) for one whole sequence."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = x + causal_conv(x, W[p + "canon1"])
        y = MIXERS[layer["type"]](h, W, p + "mix.", layer["mixer"], eps)
        x = x + rms_norm(y, W[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
            x = x + rms_norm(gated_mlp(x, W, p + "mlp."), W[p + "norm2"], eps)
        after.append(x.copy())
    logits = (rms_norm(x, W["final.norm"], eps) @ W["head"].T) * cfg["logit_scale"]
    return (logits, np.stack(after)) if return_layers else logits
