"""A plain, slow implementation of the Zitezen decoder in numpy.

Whole sequences, no cache, no state carried between calls, float64, one
function per mechanism. It shares no code with ``metallix_b200`` (files are
read with the reader of the other plain implementation in this folder).
Notation: x is ``[T, W]`` (tokens by width), positions count from 0, weights
are ``[out, in]`` and applied as x @ w.T.
"""
from __future__ import annotations

import math

import numpy as np

from plain_qwen3 import read_model  # noqa: F401  (a reader of config.json + safetensors, nothing else)


# ------------------------------------------------------------ small pieces
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def unit_rms(x, eps):
    """x over sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def tanh_norm(x, gain, offset, alpha):
    """The norm without statistics: tanh(alpha x) * gain + offset."""
    return np.tanh(alpha * x) * gain + offset


def squared_relu_ff(h, up, down):
    return np.square(np.maximum(h @ up.T, 0.0)) @ down.T


# ------------------------------------------------ several residual streams
def read_streams(streams, weights):
    """streams ``[S, T, W]`` -> sum_s weights[s] * streams[s]."""
    return np.einsum("s,stw->tw", weights, streams)


def write_streams(streams, mixing, weights, y):
    """All streams at once from the old ones: new[t] = sum_s mixing[s, t] old[s] + weights[t] * y."""
    return np.einsum("st,sxw->txw", mixing, streams) + weights[:, None, None] * y[None]


# ---------------------------------------------------------------- rotation
def turn(x, positions, base, dims, neighbours):
    """x ``[T, heads, D]``: pair i of the first ``dims`` values turns by
    position * base^(-2i/dims). ``neighbours``: the pair is (2i, 2i + 1), else
    (i, i + dims / 2). (u, v) -> (u cos - v sin, v cos + u sin)."""
    out = x.copy()
    half = dims // 2
    for i in range(half):
        f = base ** (-2.0 * i / dims)
        a, b = (2 * i, 2 * i + 1) if neighbours else (i, i + half)
        for t, p in enumerate(positions):
            c, s = math.cos(p * f), math.sin(p * f)
            out[t, :, a] = x[t, :, a] * c - x[t, :, b] * s
            out[t, :, b] = x[t, :, b] * c + x[t, :, a] * s
    return out


# ------------------------------------------------------------ the recurrence
def capped_gates(i_pre, f_pre, cap):
    """(log input gate, log forget gate) from the pre-activations (biases added by the caller)."""
    return cap * np.tanh(i_pre / cap), log_sigmoid(cap * np.tanh(f_pre / cap))


def matrix_memory(q, k, v, log_i, log_f, state=None):
    """One head. q, k ``[T, D]`` (q already scaled), v ``[T, V]``, gates ``[T]``.
    Returns (o ``[T, V]``, state); state = (C [D, V], n [D], m), zeros at the start."""
    T, D = q.shape
    V = v.shape[1]
    C, n, m = (np.zeros((D, V)), np.zeros(D), 0.0) if state is None else state
    out = np.zeros((T, V))
    for t in range(T):
        m_next = max(log_f[t] + m, log_i[t])
        keep, take = math.exp(log_f[t] + m - m_next), math.exp(log_i[t] - m_next)
        C = keep * C + take * np.outer(k[t], v[t])
        n = keep * n + take * k[t]
        m = m_next
        out[t] = (C.T @ q[t]) / (max(abs(float(n @ q[t])), math.exp(-m)) + 1e-6)
    return out, (C, n, m)


def matrix_memory_mixer(h, w, prefix, sizes, eps):
    """The whole mixer: projections, gates, recurrence per head, per-head unit
    RMS, weight over all heads, sigmoid output gate, output projection."""
    H, D, V, cap = sizes["heads"], sizes["dim"], sizes["vdim"], sizes["gate_cap"]
    T = h.shape[0]
    q = (h @ w[prefix + ".q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[prefix + ".k"].T).reshape(T, H, D)
    v = (h @ w[prefix + ".v"].T).reshape(T, H, V)
    log_i, log_f = capped_gates(h @ w[prefix + ".i"].T + w[prefix + ".i.b"],
                                h @ w[prefix + ".f"].T + w[prefix + ".f.b"], cap)
    heads = np.stack([matrix_memory(q[:, j], k[:, j], v[:, j], log_i[:, j], log_f[:, j])[0] for j in range(H)], axis=1)
    normed = unit_rms(heads, eps).reshape(T, H * V) * w[prefix + ".norm"]
    return (normed * sigmoid(h @ w[prefix + ".g"].T)) @ w[prefix + ".o"].T


# ---------------------------------------------------------------- attention
def causal_softmax_attention(q, k, v, scale, cap=0.0):
    """q ``[T, H, D]``, k ``[T, H, D]``, v ``[T, H, V]`` (heads already matched):
    position t sees 0..t; scores optionally bounded by cap * tanh(s / cap)."""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        s = np.einsum("hd,jhd->hj", q[t], k[:t + 1]) * scale
        if cap:
            s = cap * np.tanh(s / cap)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[t] = np.einsum("hj,jhv->hv", p, v[:t + 1])
    return out


def latent_mixer(h, w, prefix, sizes, eps):
    """Queries through a normed latent; keys and values up-projected from a
    second normed latent, plus one rotated key part shared by all heads."""
    H, D, R, V, r = sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["kv_rank"]
    T = h.shape[0]
    positions = range(T)
    q = ((unit_rms(h @ w[prefix + ".dq"].T, eps) * w[prefix + ".dq.norm"]) @ w[prefix + ".uq"].T).reshape(T, H, D + R)
    down = h @ w[prefix + ".dkv"].T
    latent = unit_rms(down[:, :r], eps) * w[prefix + ".dkv.norm"]
    shared = down[:, r:].reshape(T, 1, R)
    rot = sizes.get("rot")
    q_turned, shared_turned = q[:, :, D:], shared
    if rot:
        q_turned = turn(q_turned, positions, rot["base"], rot["dims"], neighbours=True)
        shared_turned = turn(shared, positions, rot["base"], rot["dims"], neighbours=True)
    keys = np.concatenate([(latent @ w[prefix + ".uk"].T).reshape(T, H, D), np.repeat(shared_turned, H, axis=1)], axis=2)
    values = (latent @ w[prefix + ".uv"].T).reshape(T, H, V)
    queries = np.concatenate([q[:, :, :D], q_turned], axis=2)
    return causal_softmax_attention(queries, keys, values, sizes["scale"]).reshape(T, H * V) @ w[prefix + ".o"].T


def grouped_mixer(h, w, prefix, sizes, eps):
    """Grouped-query attention: per-head unit RMS of q and k with one shared
    weight each, halves of the first rot.dims values turned, capped scores,
    one sigmoid gate per head."""
    H, G, D, V = sizes["heads"], sizes.get("kv_heads") or sizes["heads"], sizes["dim"], sizes["vdim"]
    T = h.shape[0]
    q = unit_rms((h @ w[prefix + ".q"].T).reshape(T, H, D), eps) * w[prefix + ".q.norm"]
    k = unit_rms((h @ w[prefix + ".k"].T).reshape(T, G, D), eps) * w[prefix + ".k.norm"]
    v = (h @ w[prefix + ".v"].T).reshape(T, G, V)
    rot = sizes.get("rot")
    if rot:
        q = turn(q, range(T), rot["base"], rot["dims"], neighbours=False)
        k = turn(k, range(T), rot["base"], rot["dims"], neighbours=False)
    k, v = np.repeat(k, H // G, axis=1), np.repeat(v, H // G, axis=1)
    out = causal_softmax_attention(q, k, v, sizes["scale"], sizes.get("softcap") or 0.0)
    out = out * sigmoid(h @ w[prefix + ".g"].T)[:, :, None]
    return out.reshape(T, H * V) @ w[prefix + ".o"].T


def mixer(h, w, index, layer, eps):
    prefix, sizes = f"l{index}.mix", layer["mixer"]
    if layer["type"] == "mlstm":
        return matrix_memory_mixer(h, w, prefix, sizes, eps)
    if layer["type"] == "latent_attention":
        return latent_mixer(h, w, prefix, sizes, eps)
    if layer["type"] == "parallel":
        return (sizes["left_scale"] * grouped_mixer(h, w, prefix + ".left", sizes["left"], eps)
                + sizes["right_scale"] * matrix_memory_mixer(h, w, prefix + ".right", sizes["right"], eps))
    raise ValueError(layer["type"])


# -------------------------------------------------------------- whole model
def order_of_layers(config):
    count, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return list(range(count))
    return (list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"]
            + list(range(loop["stop"], count)))


def forward_logits(config, w, ids, taps=None):
    """Logits ``[T, vocab]`` of the whole sequence. ``taps`` (a list) receives
    the sum of the streams after every layer run."""
    eps, S = config["norm"]["eps"], config.get("streams") or 1
    norm = lambda name, x: tanh_norm(x, w[name], w[name + ".b"], w[name + ".alpha"])
    streams = np.repeat(w["embed"][np.asarray(ids)][None], S, axis=0)
    for index in order_of_layers(config):
        layer = config["layers"][index]
        for q in (1, 2) if layer["mlp"] else (1,):
            hc = f"l{index}.hc{q}"
            h = norm(f"l{index}.norm{q}", read_streams(streams, w[hc + ".in"]))
            y = mixer(h, w, index, layer, eps) if q == 1 else \
                squared_relu_ff(h, w[f"l{index}.mlp.up"], w[f"l{index}.mlp.down"])
            streams = write_streams(streams, w[hc + ".mix"], w[hc + ".out"], y * w[f"l{index}.ls{q}"])
        if taps is not None:
            taps.append(streams.sum(axis=0))
    return norm("final.norm", streams.sum(axis=0)) @ w["head"].T
