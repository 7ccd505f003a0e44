"""Plain, slow Revesun: whole sequences, no cache, one function per mechanism.

Revesun is a pre-norm decoder whose layers are listed in ``config.json``: each layer has a token mixer, either
a gated recurrence over single channels (``mingru``) or grouped-query attention with short convolutions, a
partial interleaved rotation, a block-diagonal causal mask, a softmax with a silent extra entry and an output gate
(``attention``), and optionally a dense feed-forward with a normalised-polynomial activation.  Norms are RMS norms
taken over equal consecutive groups of the vector.  The output head is the embedding table.

This module shares no code with ``tesseract_b200``: it reads the model folder itself and computes with torch on
the CPU in ``dtype`` (float64 by default: the answer that both engine paths are compared with).  Every function
takes a whole sequence ``[T, ...]``; nothing is cached.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping, Sequence

import torch
from safetensors import safe_open


def load_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as handle:
        config = json.load(handle)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            tensors[name] = handle.get_tensor(name)
    return config, tensors


# ----------------------------------------------------------------------------- mechanisms


def grouped_rms_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """Each of ``groups`` equal consecutive parts of a row is divided by sqrt(mean(part^2) + eps); then ``* weight``."""
    rows, width = x.shape
    parts = x.reshape(rows, groups, width // groups)
    scale = torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return (parts / scale).reshape(rows, width) * weight


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def polynorm(z: torch.Tensor, coefficients: torch.Tensor, eps: float) -> torch.Tensor:
    """``a N(z) + b N(z^2) + c N(z^3) + e`` with ``N`` the division of a row by its root mean square."""
    a, b, c, e = (coefficients[i] for i in range(4))
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def short_convolution(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Per channel: ``y[t] = sum_j taps[:, j] * u[t - (J - 1) + j]`` with zeros before the sequence starts."""
    T, channels = u.shape
    J = taps.shape[1]
    padded = torch.cat([torch.zeros(J - 1, channels, dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(J):
        out = out + padded[j:j + T] * taps[:, j]
    return out


def rotate_pairs(x: torch.Tensor, positions: Sequence[int], dims: int, base: float) -> torch.Tensor:
    """``x`` is ``[T, heads, d]``; elements ``2i, 2i+1`` (i < dims/2) of every head turn by ``p * base^(-2i/dims)``."""
    out = x.clone()
    p = torch.as_tensor(list(positions), dtype=x.dtype)
    for i in range(dims // 2):
        angle = p * (base ** (-2.0 * i / dims))
        cos, sin = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * cos - v * sin
        out[:, :, 2 * i + 1] = v * cos + u * sin
    return out


def block_causal_mask(T: int, block: int) -> torch.Tensor:
    """``[T, T]`` bool: row i sees column j iff ``j <= i`` and both lie in the same block of ``block`` positions."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // block == j // block)


def attention_with_sink(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                        mask: torch.Tensor) -> torch.Tensor:
    """``q [T, H, d]``, ``k [T, G, d]``, ``v [T, G, dv]`` -> ``[T, H, dv]``.  Weights are
    ``exp(s_j) / (1 + sum_j exp(s_j))``: an extra entry of score 0 that carries no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // per
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        top = torch.clamp(s.max(dim=1, keepdim=True).values, min=0.0)
        e = torch.exp(s - top)
        weights = e / (torch.exp(-top) + e.sum(dim=1, keepdim=True))
        out[:, h] = weights @ v[:, g]
    return out


def attention_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, m: Mapping) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_convolution(h @ w[prefix + "q"].T, w[prefix + "q.conv"])
    k = short_convolution(h @ w[prefix + "k"].T, w[prefix + "k.conv"])
    v = short_convolution(h @ w[prefix + "v"].T, w[prefix + "v.conv"])
    rot = m["rot"]
    q = rotate_pairs(q.view(T, H, d), range(T), rot["dims"], rot["base"])
    k = rotate_pairs(k.view(T, G, d), range(T), rot["dims"], rot["base"])
    mixed = attention_with_sink(q, k, v.view(T, G, dv), m["scale"], block_causal_mask(T, m["mask"]["size"]))
    gate = torch.sigmoid(h @ w[prefix + "g"].T)
    return (mixed.reshape(T, H * dv) * gate) @ w[prefix + "o"].T


def mingru_candidate(u: torch.Tensor) -> torch.Tensor:
    """``u + 1/2`` for ``u >= 0``, ``sigmoid(u)`` below."""
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def mingru_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    z = torch.sigmoid(h @ w[prefix + "z"].T + w[prefix + "z.b"])
    candidate = mingru_candidate(h @ w[prefix + "x"].T + w[prefix + "x.b"])
    state = torch.zeros(z.shape[1], dtype=h.dtype)
    states: List[torch.Tensor] = []
    for t in range(h.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * candidate[t]
        states.append(state)
    gate = h @ w[prefix + "g"].T
    return (torch.stack(states) * (gate * torch.sigmoid(gate))) @ w[prefix + "o"].T


def dense_feed_forward(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, eps: float) -> torch.Tensor:
    return polynorm(h @ w[prefix + "up"].T, w[prefix + "act"], eps) @ w[prefix + "down"].T


# ----------------------------------------------------------------------------- the model


def forward(config: Mapping, tensors: Mapping[str, torch.Tensor], tokens: Sequence[int],
            dtype: torch.dtype = torch.float64, layer_outputs: List[torch.Tensor] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence.  ``layer_outputs``, if a list, receives the residual stream
    after every layer."""
    w = {name: t.to(dtype) for name, t in tensors.items()}
    eps, groups = float(config["norm"]["eps"]), int(config["norm"]["groups"])
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    for index, layer in enumerate(config["layers"]):
        name = f"l{index}."
        h = grouped_rms_norm(x, w[name + "norm1"], groups, eps)
        if layer["type"] == "attention":
            x = x + attention_mixer(h, w, name + "mix.", layer["mixer"])
        elif layer["type"] == "mingru":
            x = x + mingru_mixer(h, w, name + "mix.")
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
            h = grouped_rms_norm(x, w[name + "norm2"], groups, eps)
            x = x + dense_feed_forward(h, w, name + "mlp.", eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return grouped_rms_norm(x, w["final.norm"], groups, eps) @ w["embed"].T
