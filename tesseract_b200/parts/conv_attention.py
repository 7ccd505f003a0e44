"""Grouped-query attention with short convolutions, a parameterised mask, an optional sink and an output gate.

Per row ``h`` (the mixer's input):

* one fused product gives the queries (``num_heads * key_dim``), keys (``num_kv_heads * key_dim``), values
  (``num_kv_heads * value_dim``) and, with ``gate``, the output gate (``num_heads * value_dim``);
* a causal convolution of ``conv_taps`` taps runs over time on every channel of q, k and v
  (``y[t] = sum_j w[c, j] * u[t - taps + 1 + j]``, zeros before the sequence starts); the last ``taps - 1`` projected
  rows of a request are fixed-size state in its state slot;
* the position encoding (``rotary_pairs``) turns q and k; rotated k and v go into the request's pages;
* every row attends over the keys its mask lets it see: ``causal`` (all up to its own position), ``window`` (the last
  ``size``), or ``blocks`` (positions are cut into consecutive blocks of ``size`` counted from 0 and a row sees its own
  block up to its own position; pages of earlier blocks go back to the pool).  Scores ``(q . k) * scale`` and the
  weights are 32-bit; with ``sink`` the softmax's denominator has one more entry of score 0 without a value;
* with ``gate`` the concatenated heads are multiplied by ``sigmoid(gate)``; then the output projection, whose
  result comes out in 32-bit for a residual stream kept in 32-bit (``stream`` = ``"float32"``).

Convolution, rotation and the cache write are one kernel (and a second small one that renews the state when some
sequence brings more than one row); the attention kernel applies the sink and the gate itself.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import (MIXERS, POSITION_ENCODINGS, DeferredNorm, Mixer, PagedKeyValueNeed, Runtime, StateNeed, StepContext)
from .linear import Linear

_MASKS = {"causal": kernels.MASK_CAUSAL, "window": kernels.MASK_WINDOW, "blocks": kernels.MASK_BLOCKS}


@MIXERS.register("conv_attention")
class ConvAttention(Mixer):
    """params: ``hidden_size, num_heads, num_kv_heads, key_dim, value_dim, conv_taps, scale``, ``mask``
    (``{"kind": "causal" | "window" | "blocks", "size": n}``), ``sink`` (bool), ``gate`` (bool), optional ``stream``.
    weights: ``q, k, v, o, q_conv, k_conv, v_conv`` and, with ``gate``, ``g``.  children: ``position``."""

    graph_safe = True      # reads only device-side metadata of the step (and its shape)

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.key_dim = int(p["key_dim"])
        self.value_dim = int(p["value_dim"])
        self.taps = int(p["conv_taps"])
        self.scale = float(p["scale"])
        mask = dict(p.get("mask") or {"kind": "causal"})
        if mask.get("kind") not in _MASKS:
            raise ValueError(f"mask kind must be one of {sorted(_MASKS)}, got {mask.get('kind')!r}")
        self.mask_kind = mask["kind"]
        self.mask_size = int(mask.get("size") or 0)
        if self.mask_kind != "causal" and self.mask_size < 1:
            raise ValueError(f"a '{self.mask_kind}' mask needs a positive size")
        self.sink = bool(p.get("sink"))
        self.gated = bool(p.get("gate"))
        self.stream_f32 = p.get("stream") == "float32"
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"the short convolution takes 1 to 8 taps, got {self.taps}")
        if not (1 <= self.key_dim <= 1024 and 1 <= self.value_dim <= 512):
            raise ValueError("the attention kernel takes keys of up to 1024 and values of up to 512 numbers a head")
        self.q_width = self.num_heads * self.key_dim
        self.k_width = self.num_kv_heads * self.key_dim
        self.v_width = self.num_kv_heads * self.value_dim
        self.o_width = self.num_heads * self.value_dim
        self.channels = self.q_width + self.k_width + self.v_width
        rows = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.gated else [])
        self.in_proj = Linear(torch.cat(rows, dim=0), runtime)
        self.o_proj = Linear(tensors["o"], runtime)
        # [taps, channels]: tap j of every channel side by side, as the kernel reads them
        self.conv_taps = torch.cat([tensors["q_conv"], tensors["k_conv"], tensors["v_conv"]], dim=0).to(
            device=runtime.device, dtype=torch.float32).t().contiguous()
        position_spec = spec.children.get("position") or PartSpec.make("none")
        self.position = POSITION_ENCODINGS.get(position_spec.kind)(position_spec, {}, runtime)
        if self.position.kind not in ("rotary_pairs", "none"):
            raise ValueError(f"conv_attention rotates pairs or not at all, got position encoding '{self.position.kind}'")
        self.rot_dims = int(getattr(self.position, "dims", 0))
        self.inv_freq = getattr(self.position, "pair_inv_freq", None)

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, d, dv, taps = int(p["hidden_size"]), int(p["key_dim"]), int(p["value_dim"]), int(p["conv_taps"])
        heads, kv = int(p["num_heads"]), int(p["num_kv_heads"])
        out = {
            w["q"]: ExpectedTensor((heads * d, hidden)),
            w["k"]: ExpectedTensor((kv * d, hidden)),
            w["v"]: ExpectedTensor((kv * dv, hidden)),
            w["o"]: ExpectedTensor((hidden, heads * dv)),
            w["q_conv"]: ExpectedTensor((heads * d, taps)),
            w["k_conv"]: ExpectedTensor((kv * d, taps)),
            w["v_conv"]: ExpectedTensor((kv * dv, taps)),
        }
        if p.get("gate"):
            out[w["g"]] = ExpectedTensor((heads * dv, hidden))
        return out

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role.endswith("_conv"):
            return torch.randn(shape, generator=generator, dtype=torch.float32) * 0.5
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the mixer's matrix products, for the printed kernel plan."""
        from .. import plan

        return [("q/k/v/gate", self.in_proj, plan.BF16), ("o", self.o_proj, plan.F32 if self.stream_f32 else plan.BF16)]

    def cache_need(self):
        pages = PagedKeyValueNeed(num_kv_heads=self.num_kv_heads, key_dim=self.key_dim, value_dim=self.value_dim,
                                  window=self.mask_size if self.mask_kind == "window" else None,
                                  block=self.mask_size if self.mask_kind == "blocks" else None)
        if self.taps == 1:
            return pages
        return (pages, StateNeed((self.taps - 1, self.channels), torch.float32))

    def forward(self, x, ctx: StepContext, cache):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        pages, state = (cache if isinstance(cache, tuple) else (cache, None))
        if pages is None or pages.storage is None:
            raise RuntimeError("conv_attention needs a paged key/value cache binding")
        if not pages.writes:
            raise NotImplementedError("conv_attention keeps a cache and a convolution state of its own: a run entry "
                                      "cannot read another entry's")
        group = ctx.groups[pages.group]
        proj = self.in_proj.forward(x)
        rows = proj.shape[0]
        q = torch.empty((rows, self.q_width), dtype=proj.dtype, device=proj.device)
        kernels.conv_rope_cache(proj, self.conv_taps, None if state is None else state.storage, q, pages.storage,
                                ctx.positions, ctx.seq_of_row, ctx.row_start, ctx.seq_begin, ctx.state_slots,
                                group.block_table, self.inv_freq, num_seqs=ctx.num_seqs, heads=self.num_heads,
                                kv_heads=self.num_kv_heads, dim=self.key_dim, vdim=self.value_dim,
                                rot_dims=self.rot_dims, page_size=pages.page_size, write_kv=pages.writes,
                                single=ctx.max_new == 1)
        gate = proj[:, self.channels:] if self.gated else None
        attended = torch.empty((rows, self.o_width), dtype=proj.dtype, device=proj.device)
        kernels.attention_masked(q, gate, attended, pages.storage, ctx.positions, ctx.seq_of_row, group.block_table,
                                 heads=self.num_heads, kv_heads=self.num_kv_heads, dim=self.key_dim,
                                 vdim=self.value_dim, page_size=pages.page_size, mask_kind=_MASKS[self.mask_kind],
                                 mask_size=self.mask_size, sink=self.sink, scale=self.scale)
        return self.o_proj.forward(attended, float32_out=self.stream_f32)
