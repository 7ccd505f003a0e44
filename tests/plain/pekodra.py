"""Plain, slow Pekodra: whole sequences, no cache, one function per mechanism.

Pekodra is a decoder whose layers are listed in ``config.json``.  A layer adds, to the stream ``x``, the sum of a
token mixer applied to one norm of ``x`` and a feed-forward applied to a second norm of the same ``x``.  The mixer
is grouped-query attention over a sliding window with a partial rotate-half rotation (frequencies blended between
plain and stretched ones, amplitude raised with the stretch), queries and keys brought to unit root mean square
after the rotation, and a score scale of its own.  The feed-forward is either a gated one with biases and the
tanh form of GELU, or a set of small experts (squared ReLU) of which a router picks a few per token, beside an
expert that every token takes.  A run of layers may be walked several times with the same weights; every walk
starts by mixing the stream with the embedding output through one matrix.

This module shares no code with ``tesseract_b200``: it reads the model folder itself and computes with torch on
the CPU in ``dtype`` (float64 by default: the answer that both engine paths are compared with).  Every function
takes a whole sequence ``[T, ...]``; nothing is cached.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping, Optional, Sequence

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
# ``round_to`` (None or a torch dtype): where a serving path would store an activation in a 16-bit format (the
# operands of every product, stored queries, keys and values), the value is rounded to that format and widened
# again.  The difference to the unrounded run is the noise that such rounding alone causes; sums that the design
# keeps in 32-bit (the stream, scores and weights, norms' statistics, router logits) are never rounded.


def rounded(x: torch.Tensor, round_to) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(x.dtype)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The weight is stored around zero: the row over its root mean square, times ``1 + weight``."""
    return unit_rms(x, eps) * (1.0 + weight)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z * z * z)))


def blended_frequencies(dims: int, base: float, scaling: Optional[Mapping[str, float]]):
    """``(frequencies [dims / 2], amplitude)``.  Without ``scaling``: ``base^(-2i/dims)`` and 1.  With it, every
    frequency is a mix of itself and itself over ``factor``; the mix goes linearly, over the index, from all-plain to
    all-stretched between the indices where ``original`` positions hold ``fast`` and ``slow`` turns."""
    half = dims // 2
    plain = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return plain, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    low = max(math.floor(index_of(float(scaling["fast"]))), 0)
    high = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(plain):
        ramp = min(max((i - low) / max(high - low, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_half(x: torch.Tensor, positions: Sequence[int], dims: int, frequencies: Sequence[float],
                amplitude: float) -> torch.Tensor:
    """``x`` is ``[T, heads, d]``; element ``i`` and element ``i + dims/2`` (``i < dims/2``) of every head turn together
    by ``p * frequencies[i]``, cosine and sine both times ``amplitude``; elements from ``dims`` on pass."""
    out = x.clone()
    p = torch.as_tensor(list(positions), dtype=x.dtype)
    half = dims // 2
    for i in range(half):
        angle = p * frequencies[i]
        cos, sin = (torch.cos(angle) * amplitude)[:, None], (torch.sin(angle) * amplitude)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * cos - v * sin
        out[:, :, i + half] = v * cos + u * sin
    return out


def window_mask(T: int, window: Optional[int]) -> torch.Tensor:
    """``[T, T]`` bool: row i sees column j when ``0 <= i - j < window`` (no window: every j up to i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    return seen


def window_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float, round_to=None) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rounded(h @ w["q"].T, round_to).reshape(T, H, d)
    k = rounded(h @ w["k"].T, round_to).reshape(T, G, d)
    v = rounded(h @ w["v"].T, round_to).reshape(T, G, dv)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        freqs, amplitude = blended_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
        q = rotate_half(q, range(T), rot["dims"], freqs, amplitude)
        k = rotate_half(k, range(T), rot["dims"], freqs, amplitude)
    q, k = rounded(unit_rms(q, eps), round_to), rounded(unit_rms(k, eps), round_to)
    seen = window_mask(T, (m.get("mask") or {}).get("size"))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        scores = (q[:, head] @ k[:, g].T) * float(m["scale"])
        scores = scores.masked_fill(~seen, float("-inf"))
        out[:, head] = torch.softmax(scores, dim=-1) @ v[:, g]
    return rounded(out.reshape(T, H * dv), round_to) @ w["o"].T


def gated_mlp(h: torch.Tensor, w: Mapping[str, torch.Tensor], round_to=None) -> torch.Tensor:
    gate = rounded(h @ w["gate"].T, round_to) + w["gate.b"]
    up = rounded(h @ w["up"].T, round_to) + w["up.b"]
    return rounded(gelu_tanh(gate) * up, round_to) @ w["down"].T + w["down.b"]


def squared_relu_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor, round_to=None) -> torch.Tensor:
    return rounded(torch.relu(rounded(h @ up.T, round_to)) ** 2, round_to) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, top: int):
    """``(chosen [T, top], weights [T, top])``: the ``top`` largest router logits of a row and the softmax over those."""
    logits = h @ router.T
    values, chosen = torch.topk(logits, top, dim=-1)
    return chosen, torch.softmax(values, dim=-1)


def expert_mixture(h: torch.Tensor, w: Mapping[str, torch.Tensor], mlp: Mapping, chosen: Optional[torch.Tensor] = None,
                   report: Optional[list] = None, round_to=None) -> torch.Tensor:
    """``chosen`` (``[T, top]``) overrides the router's choice (the weights are still the softmax over the chosen
    logits): a comparison with an implementation in lower precision then does not hang on which of two nearly equal
    logits it found larger.  ``report`` receives ``(own choice [T, top], margin [T])``, the margin being the distance
    between the last chosen and the first rejected logit over the root mean square of all the run's logits."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    own, weights = route(h, w["router"], top)
    if report is not None or chosen is not None:
        logits = h @ w["router"].T
        ranked = torch.sort(logits, dim=-1, descending=True).values
        margin = (ranked[:, top - 1] - ranked[:, top]) if top < experts else torch.full((h.shape[0],), float("inf"))
        if report is not None:
            report.append((own, margin / (logits.pow(2).mean().sqrt() + 1e-30)))
        if chosen is not None:
            chosen = chosen.long()
            weights = torch.softmax(torch.gather(logits, 1, chosen), dim=-1)
    if chosen is None:
        chosen = own
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for slot in range(top):
            e = int(chosen[t, slot])
            out[t] += weights[t, slot] * squared_relu_expert(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"], round_to)[0]
    if mlp.get("shared"):
        out = out + squared_relu_expert(h, w["shared.up"], w["shared.down"], round_to)
    return out


def run_order(config: Mapping) -> List[tuple]:
    """``(layer, starts a walk)`` in the order the layers run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(count)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, count)]


# ----------------------------------------------------------------------------- the model


def _sub(tensors: Mapping[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {name[len(prefix):]: t.to(dtype) for name, t in tensors.items() if name.startswith(prefix)}


def forward(config: Mapping, tensors: Mapping[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64,
            keep_layers: bool = False, routing: Optional[Mapping[int, torch.Tensor]] = None,
            report: Optional[list] = None, round_to=None):
    """Logits ``[T, vocab]`` of a whole sequence (and, with ``keep_layers``, the stream after every layer run).
    ``routing[n]`` (``[T, top]``) fixes the experts of the n-th run of a layer with experts; ``report`` receives the
    model's own choice and its margin for every such run (see :func:`expert_mixture`).  ``round_to``: see above."""
    routed_runs = 0
    eps = float(config["norm"]["eps"])
    x0 = tensors["embed"].to(dtype)[list(tokens)] * float(config["embedding"]["scale"])
    x = x0
    after = []
    for index, starts in run_order(config):
        if starts:
            x = rounded(torch.cat([x, x0], dim=-1), round_to) @ tensors["loop.in"].to(dtype).T
        layer = config["layers"][index]
        prefix = f"l{index}."
        mixed = window_attention(rounded(offset_rms_norm(x, tensors[prefix + "norm1"].to(dtype), eps), round_to),
                                 _sub(tensors, prefix + "mix.", dtype), layer["mixer"], eps, round_to)
        mlp = layer.get("mlp")
        if mlp:
            h2 = rounded(offset_rms_norm(x, tensors[prefix + "norm2"].to(dtype), eps), round_to)
            w = _sub(tensors, prefix + "mlp.", dtype)
            if mlp["kind"] == "dense":
                fed = gated_mlp(h2, w, round_to)
            else:
                fed = expert_mixture(h2, w, mlp, None if routing is None else routing[routed_runs], report, round_to)
                routed_runs += 1
            x = x + (mixed + fed)
        else:
            x = x + mixed
        after.append(x)
    final = rounded(offset_rms_norm(x, tensors["final.norm"].to(dtype), eps), round_to)
    logits = (final @ tensors["head"].to(dtype).T) * float(config["logit_scale"])
    return (logits, torch.stack(after)) if keep_layers else logits
