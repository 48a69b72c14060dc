"""A plain, slow implementation of the Mekazen decoder in numpy.

Whole sequences under a mask, no cache, float64, one function per mechanism.
It shares no code with ``metallix_b200`` (files are read with the reader of
the other plain implementation in this folder). Notation: x is ``[T, W]``
(tokens by width), positions count from 0, weights are ``[out, in]``.
"""
from __future__ import annotations

import math

import numpy as np

from plain_qwen3 import read_model  # noqa: F401  (a reader of config.json + safetensors, nothing else)


# ------------------------------------------------------------------- norms
def rms_scale(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_around_zero(x, stored, eps):
    """A norm whose stored weight w means the factor 1 + w."""
    return rms_scale(x, eps) * (1.0 + stored)


def norm_plain(x, factor, eps):
    return rms_scale(x, eps) * factor


# ---------------------------------------------------------------- rotation
def pair_frequencies(base, dims, scaling=None):
    """One frequency per pair of the first ``dims`` values of a head:
    base^(-2i/dims), the long wavelengths stretched by ``scaling``."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            n, factor = scaling["original"], scaling["factor"]
            wavelength = 2.0 * math.pi / f
            if wavelength > n / scaling["low"]:
                f = f / factor
            elif wavelength >= n / scaling["high"]:
                s = (n / wavelength - scaling["low"]) / (scaling["high"] - scaling["low"])
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return np.asarray(out)


def rotate_pairs(x, positions, base, dims, scaling=None):
    """x ``[T, heads, D]``: values (2i, 2i + 1), i < dims / 2, turn by the
    angle position * f_i; the values from ``dims`` on stay."""
    out = x.copy()
    frequencies = pair_frequencies(base, dims, scaling)
    for t, p in enumerate(positions):
        for i, f in enumerate(frequencies):
            c, s = math.cos(p * f), math.sin(p * f)
            u, v = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            out[t, :, 2 * i] = u * c - v * s
            out[t, :, 2 * i + 1] = v * c + u * s
    return out


# --------------------------------------------------------------------- mask
def visible(i, j, chunk):
    """Whether the query at position i sees the key at position j."""
    return j <= i and (not chunk or i // chunk == j // chunk)


def masked_attention(q, k, values, positions, scale, chunk, rows=None):
    """q ``[T, heads, D]``, k and values ``[T, groups, D]``: every query (or
    those of ``rows``) over the keys it sees, query head h with key/value head
    h // (heads / groups)."""
    tokens, heads, _ = q.shape
    per_group = heads // k.shape[1]
    rows = list(range(tokens)) if rows is None else list(rows)
    out = np.zeros((len(rows), heads, values.shape[2]))
    for at, t in enumerate(rows):
        seen = [u for u in range(tokens) if visible(positions[t], positions[u], chunk)]
        for head in range(heads):
            g = head // per_group
            scores = (k[seen, g] @ q[t, head]) * scale
            weights = np.exp(scores - scores.max())
            out[at, head] = (weights / weights.sum()) @ values[seen, g]
    return out


# -------------------------------------------------------------------- mixer
def attention_mixer(h, positions, w, base, mixer, eps):
    """h ``[T, W]`` -> ``[T, W]``. ``w`` holds the layer's tensors under
    ``base`` ('l3.mix.')."""
    heads, groups, dim = mixer["heads"], mixer["kv_heads"], mixer["dim"]
    tokens = h.shape[0]
    q = h @ w[base + "q"].T
    k = h @ w[base + "k"].T
    values = k.reshape(tokens, groups, dim)           # as projected: no norm, no rotation
    q = norm_plain(q, w[base + "q.norm"], eps).reshape(tokens, heads, dim)    # one norm over the whole projection
    k = norm_plain(k, w[base + "k.norm"], eps).reshape(tokens, groups, dim)
    rot = mixer.get("rot")
    if rot:
        q = rotate_pairs(q, positions, rot["base"], rot["dims"], rot.get("scaling"))
        k = rotate_pairs(k, positions, rot["base"], rot["dims"], rot.get("scaling"))
    chunk = (mixer.get("mask") or {}).get("size", 0)
    out = masked_attention(q, k, values, positions, mixer["scale"], chunk)
    gate = 1.0 / (1.0 + np.exp(-(h @ w[base + "g"].T)))
    return (out.reshape(tokens, heads * dim) * gate) @ w[base + "o"].T


# ------------------------------------------------------------- feed-forward
def gated_feed_forward(h, w, base):
    a = h @ w[base + "gate"].T
    return ((a / (1.0 + np.exp(-a))) * (h @ w[base + "up"].T)) @ w[base + "down"].T


# -------------------------------------------------------------------- model
def layer(x, positions, w, index, spec, eps):
    base = f"l{index}."
    mixed = attention_mixer(norm_around_zero(x, w[base + "norm1"], eps), positions, w, base + "mix.",
                            spec["mixer"], eps)
    x = x + norm_around_zero(mixed, w[base + "norm1b"], eps)
    if spec.get("mlp"):
        fed = gated_feed_forward(norm_around_zero(x, w[base + "norm2"], eps), w, base + "mlp.")
        x = x + norm_around_zero(fed, w[base + "norm2b"], eps)
    return x


def capped(logits, cap):
    return cap * np.tanh(logits / cap) if cap else logits


def forward_logits(config, tensors, ids, keep=None):
    """Logits ``[T, vocab]`` of the whole sequence ``ids``. ``keep`` (a list)
    receives the residual stream after every layer."""
    w = {name: np.asarray(value, dtype=np.float64) for name, value in tensors.items()}
    eps = config["norm"]["eps"]
    positions = list(range(len(ids)))
    x = w["embed"][np.asarray(ids)]
    for index, spec in enumerate(config["layers"]):
        x = layer(x, positions, w, index, spec, eps)
        if keep is not None:
            keep.append(x.copy())
    x = norm_around_zero(x, w["final.norm"], eps)
    return capped(x @ w["head"].T, config.get("logit_softcap"))


def greedy(config, tensors, prompt, count):
    """``count`` tokens picked by the largest logit (the lowest id on a tie)."""
    ids, out = list(prompt), []
    for _ in range(count):
        token = int(np.argmax(forward_logits(config, tensors, ids)[-1]))
        out.append(token)
        ids.append(token)
    return out
