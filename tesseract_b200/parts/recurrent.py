"""Recurrent mixers: fixed-size state per request instead of pages.

``mingru``: a gated recurrence whose gates read only the current token, so that within a step it is an affine scan
per channel.  With ``h`` the mixer's input,

    z_t = sigmoid(Wz h_t + bz)                       the update gate, ``width`` channels
    c_t = u_t + 1/2  if u_t >= 0  else sigmoid(u_t)   with u_t = Wx h_t + bx, the candidate
    S_t = (1 - z_t) * S_(t-1) + z_t * c_t            element by element, S_(-1) = 0
    y_t = Wo (S_t * silu(Wg h_t))

The three input projections are one product whose result is kept in 32-bit; biases, activations, the recurrence
and the output gate are 32-bit inside one kernel; ``S`` lives in the request's state slot as float32.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import MIXERS, DeferredNorm, Mixer, Runtime, StateNeed, StepContext
from .linear import Linear


@MIXERS.register("mingru")
class MinGRU(Mixer):
    """params: ``hidden_size, width``, optional ``stream``; weights: ``z, z_bias, x, x_bias, g, o``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.width = int(p["width"])
        self.stream_f32 = p.get("stream") == "float32"
        self.in_proj = Linear(torch.cat([tensors["z"], tensors["x"], tensors["g"]], dim=0), runtime)
        self.o_proj = Linear(tensors["o"], runtime)
        self.bias_z = runtime.vector_f32(tensors["z_bias"])
        self.bias_x = runtime.vector_f32(tensors["x_bias"])

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, width = int(p["hidden_size"]), int(p["width"])
        return {
            w["z"]: ExpectedTensor((width, hidden)), w["z_bias"]: ExpectedTensor((width,)),
            w["x"]: ExpectedTensor((width, hidden)), w["x_bias"]: ExpectedTensor((width,)),
            w["g"]: ExpectedTensor((width, hidden)), w["o"]: ExpectedTensor((hidden, width)),
        }

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role.endswith("_bias"):
            return torch.randn(shape, generator=generator, dtype=torch.float32) * 0.5
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the mixer's matrix products, for the printed kernel plan."""
        from .. import plan

        return [("z/x/gate", self.in_proj, plan.F32), ("o", self.o_proj, plan.F32 if self.stream_f32 else plan.BF16)]

    def cache_need(self) -> StateNeed:
        return StateNeed((self.width,), torch.float32)

    def forward(self, x, ctx: StepContext, cache):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        if cache is None or cache.storage is None:
            raise RuntimeError("mingru needs a state binding")
        proj = self.in_proj.forward(x, float32_out=True)        # gates and candidate enter the recurrence in 32-bit
        gated = torch.empty((proj.shape[0], self.width), dtype=self.runtime.dtype, device=proj.device)
        kernels.gated_recurrence(proj, self.bias_z, self.bias_x, cache.storage, gated, ctx.row_start, ctx.state_slots,
                                 num_seqs=ctx.num_seqs, max_new=ctx.max_new)
        return self.o_proj.forward(gated, float32_out=self.stream_f32)
