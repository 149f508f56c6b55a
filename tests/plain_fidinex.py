"""A plain, slow implementation of the Fidinex decoder in NumPy float64: whole sequences, no cache, one
function per mechanism.  It shares no code with `tuff_b200` (config.json and the safetensors file are read
with the standard library and NumPy alone) and is what the engine's kernels, cache and batching are
compared with.

Notation: h [T, d] is a sublayer's input; matrices are stored [out, in] and applied as h @ W.T;
positions p = 0 .. T-1.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ------------------------------------------------------------------ file reading
def read_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        if info["dtype"] == "BF16":
            a = (np.frombuffer(data[b:e], dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            a = np.frombuffer(data[b:e], dtype=np.float32)
        elif info["dtype"] == "I32":
            a = np.frombuffer(data[b:e], dtype=np.int32)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = a.astype(np.float64).reshape(info["shape"])
    return out


# ------------------------------------------------------------------ small functions
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def sink_softmax(scores, sink, visible):
    """scores [T, T] of one head; `visible` a boolean mask; the denominator also holds exp(sink), a term
    that has no key and no value.  Returns the weights [T, T] (rows sum to less than one)."""
    s = np.where(visible, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def causal_mask(T):
    i = np.arange(T)
    return i[None, :] <= i[:, None]


def rotate_pairs(x, positions, base, dims):
    """x [T, heads, n]: elements (2i, 2i+1), i < dims/2, turn by the angle p * base^(-2i/dims); elements from
    `dims` on pass unchanged."""
    out = x.copy()
    i = np.arange(dims // 2)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * base ** (-2.0 * i / dims)      # [T, dims/2]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    p = np.asarray(positions, dtype=np.int64)
    return 1.0 + coef * np.log((p + 1) // every + 1.0)


# ------------------------------------------------------------------ mixers
def attention(h, w, p, m, eps, v_first=None):
    """Grouped-query attention without rotation: q and k normed per head with one weight each, the query scaled
    by its temperature, a learned sink per head, and values mixed with those of the first such layer.
    `w`: the checkpoint's tensors, `p` the layer's prefix ("l3.mix."), `m` the mixer's configuration.
    `v_first`: None in the first layer that mixes values (its values are returned for the later ones).
    Returns (output [T, d], the values that later layers mix with)."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (h @ w[p + "q"].T).reshape(T, H, dim)
    k = (h @ w[p + "k"].T).reshape(T, G, dim)
    v = (h @ w[p + "v"].T).reshape(T, G, vdim)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(np.arange(T), qt["coef"], qt["every"])[:, None, None]
    given = v
    if m.get("v_mix"):
        if v_first is not None:
            lam = float(w[p + "vmix"])
            v = (1.0 - lam) * v + lam * v_first
        else:
            given = v
    vis = causal_mask(T)
    out = np.zeros((T, H, vdim))
    for hh in range(H):
        g = hh // (H // G)
        a = sink_softmax(q[:, hh] @ k[:, g].T * m["scale"], float(w[p + "sink"][hh]), vis)
        out[:, hh] = a @ v[:, g]
    return out.reshape(T, H * vdim) @ w[p + "o"].T, (given if v_first is None else v_first)


def latent_attention(h, w, p, m, eps):
    """Attention whose keys and values are expanded from one small latent vector per token, plus one rotated key
    part that all heads share."""
    T = h.shape[0]
    H, dim, rd, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].T).reshape(T, H, dim + rd)
    dkv = h @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :rank], w[p + "dkv.norm"], eps)                   # the latent [T, rank]
    kr = dkv[:, rank:].reshape(T, 1, rd)                                  # the shared rotated key part
    rot = m["rot"]
    pos = np.arange(T)
    q_plain, q_rot = q[..., :dim], rotate_pairs(q[..., dim:], pos, rot["base"], rot["dims"])
    kr = rotate_pairs(kr, pos, rot["base"], rot["dims"])[:, 0]
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dim)
    v = (c @ w[p + "uv"].T).reshape(T, H, vdim)
    vis = causal_mask(T)
    out = np.zeros((T, H, vdim))
    for hh in range(H):
        s = (q_plain[:, hh] @ k_plain[:, hh].T + q_rot[:, hh] @ kr.T) * m["scale"]
        out[:, hh] = sink_softmax(s, float(w[p + "sink"][hh]), vis) @ v[:, hh]
    return out.reshape(T, H * vdim) @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forward
def relu_squared_mlp(h, w, p):
    z = np.maximum(h @ w[p + "up"].T, 0.0)
    return (z * z) @ w[p + "down"].T


# ------------------------------------------------------------------ streams
def hyper_sublayer(xs, w, p, fn, norm_w, eps):
    """xs [S, T, d]: the streams.  u = sum_s in[s] x_s; y = fn(norm(u)); then all streams at once from the old
    ones: x_t <- sum_s mix[s, t] x_s + out[t] y."""
    u = np.tensordot(w[p + "in"], xs, axes=(0, 0))
    y = fn(rms_norm(u, norm_w, eps))
    return np.einsum("st,sij->tij", w[p + "mix"], xs) + w[p + "out"][:, None, None] * y[None]


# ------------------------------------------------------------------ the model
def forward(cfg, w, tokens, collect=None):
    """Logits [T, vocab] of a whole sequence.  `collect`: a list that receives the residual stream (the sum of the
    streams) after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    S = cfg.get("streams")
    hyper = S is not None and "l0.hc1.in" in w
    xs = np.repeat(x[None], S, axis=0) if hyper else None
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]

        def mixer(hh):
            nonlocal v_first
            if layer["type"] == "attention":
                y, vf = attention(hh, w, p + "mix.", m, eps, v_first if m.get("v_mix") else None)
                if m.get("v_mix"):
                    v_first = vf
                return y
            if layer["type"] == "latent_attention":
                return latent_attention(hh, w, p + "mix.", m, eps)
            raise ValueError(layer["type"])

        def ff(hh):
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            return relu_squared_mlp(hh, w, p + "mlp.")

        if hyper:
            xs = hyper_sublayer(xs, w, p + "hc1.", mixer, w[p + "norm1"], eps)
            if layer.get("mlp") is not None:
                xs = hyper_sublayer(xs, w, p + "hc2.", ff, w[p + "norm2"], eps)
            x = xs.sum(axis=0)
        else:
            x = x + mixer(rms_norm(x, w[p + "norm1"], eps))
            if layer.get("mlp") is not None:
                x = x + ff(rms_norm(x, w[p + "norm2"], eps))
        if collect is not None:
            collect.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T


def load(model_dir):
    return read_config(model_dir), read_safetensors(os.path.join(model_dir, "model.safetensors"))
