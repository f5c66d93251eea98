"""Plain, slow Bamipel decoder used as the oracle of the test-suite.

Whole sequences only, no cache, no batching, one function per mechanism, numpy
float64 throughout, loops over tokens where the definition is a recurrence.  It
shares no code with the ``hfee_b200`` package: its own safetensors reader, its own
reading of config.json, its own rotary angles.

The design, in the notation used below (x: residual stream [T, width]; N_* are RMS
norms with a weight each):

    x = table[token]
    per layer:   x = x + N_1b(mixer(N_1(x)))
                 x = x + N_2b(W_down relu(W_up N_2(x))^2)     (only if the layer has a feed-forward)
    logits = W_head N_final(x)

A layer may borrow every tensor of another layer and keeps only its own cache.  Three mixers:
``attention`` (grouped queries, partial rotation, unit-RMS queries and keys, one sigmoid gate per
head), ``latent_attention`` (queries and keys/values through low-rank latents, one rotated key part
shared by the heads, a sliding window, one sigmoid gate per head) and ``delta`` (the gated delta
rule on a matrix state per head, behind short convolutions).
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
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w = None: no weight)."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def frequencies(rot):
    """f_i = base^(-2i/dims) for i < dims/2, the long wavelengths stretched if ``scaling`` is given:
    a wavelength under original/high keeps its frequency, one over original/low gets f/factor, and
    between the two the blend (1 - s) f/factor + s f with s = (original/wavelength - low)/(high - low)."""
    dims = rot["dims"]
    f = np.array([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f:
            wl = 2.0 * math.pi / fi
            if wl < sc["original"] / sc["high"]:
                out.append(fi)
            elif wl > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = np.array(out)
    return f


def rotate(x, rot, first=0):
    """x [T, heads, d]: the first rot.dims dimensions of every head turn by position * f_i, dimension
    i paired with i + dims/2; the others stay.  Token t sits at position first + t."""
    dims = rot["dims"]
    half = dims // 2
    ang = (first + np.arange(x.shape[0]))[:, None] * frequencies(rot)[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale, window=None):
    """q [T, H, d], k [T, H, d], v [T, H, dv] (already one key/value head per query head).  Token i
    attends to j <= i, and with a window only to i - j < window."""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[-1]))
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(H):
            s = k[lo:i + 1, h] @ q[i, h] * scale
            p = np.exp(s - s.max())
            out[i, h] = (p / p.sum()) @ v[lo:i + 1, h]
    return out


def attention_mixer(h, m, w, p, eps):
    """Grouped-query attention: rotation on the first rot.dims dimensions, then queries and keys brought
    to unit RMS per head, softmax over all earlier tokens, each head's output times one sigmoid gate."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    q, k = rms_norm(rotate(q, m["rot"]), None, eps), rms_norm(rotate(k, m["rot"]), None, eps)
    rep = H // G
    k, v = np.repeat(k, rep, axis=1), np.repeat(v, rep, axis=1)
    window = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(q, k, v, m["scale"], window)
    o = o * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def latent_attention_mixer(h, m, w, p, eps):
    """Attention whose queries come from a normed latent of size q_rank and whose keys and values come from a
    normed latent c of size kv_rank; a head's key is [W_uk c | r], r one rotated vector for all heads taken
    from the same down-projection as c; its query is laid out [unrotated | rotated] to match."""
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + dr)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    r = rotate(down[:, None, rank:], m["rot"])                       # [T, 1, dr]
    q_rot = rotate(q[..., d:], m["rot"])
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    qq = np.concatenate([q[..., :d], q_rot], axis=-1)
    kk = np.concatenate([k_plain, np.repeat(r, H, axis=1)], axis=-1)
    window = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(qq, kk, v, m["scale"], window)
    o = o * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def causal_conv(x, w):
    """y[t] = sum_j w[:, j] * x[t - taps + 1 + j], zeros before the start.  x [T, C], w [C, taps]."""
    T, taps = x.shape[0], w.shape[1]
    y = np.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y


def delta_rule(q, k, v, beta, g):
    """Per head, S [d, dv] from zero: S = g_t S; u = beta_t (v_t - S^T k_t); S = S + k_t u^T; o_t = S^T q_t.
    q, k [T, H, d]; v [T, H, dv]; beta, g [T, H]."""
    T, H, d = q.shape
    dv = v.shape[-1]
    o = np.zeros((T, H, dv))
    for h in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h])
            S = S + np.outer(k[t, h], u)
            o[t, h] = S.T @ q[t, h]
    return o


def delta_mixer(h, m, w, p, eps):
    """The gated delta rule behind short convolutions: q, k, v = silu(conv(W h)); q and k unit vectors per head
    (q also times d^-1/2); write strength sigmoid(W_b h); decay exp(-exp(A_log) softplus(W_a h + dt_bias));
    the read-out is RMS-normed per head, weighted, and gated by silu(W_g h)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    rep = H // G
    q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)
    beta = sigmoid(h @ w[p + "b"].T)
    g = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = delta_rule(q, k, v, beta, g)
    o = rms_norm(o, w[p + "norm"], eps) * silu(h @ w[p + "g"].T).reshape(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def feed_forward(h, w, p):
    z = np.maximum(h @ w[p + "up"].T, 0.0)
    return (z * z) @ w[p + "down"].T


MIXERS = {"attention": attention_mixer, "latent_attention": latent_attention_mixer, "delta": delta_mixer}


# --------------------------------------------------------------------------
def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] for one whole sequence; ``layers_out`` (a list) takes x after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        y = MIXERS[layer["type"]](rms_norm(x, w[p + "norm1"], eps), layer["mixer"], w, p + "mix.", eps)
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg, w, prompt, n):
    """The n tokens greedy decoding appends to ``prompt`` (recomputing the sequence every time)."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(np.argmax(forward(cfg, w, seq)[-1])))
    return seq[len(prompt):]
