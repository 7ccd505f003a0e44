"""Pekodra: configuration -> model description.

A decoder whose layers are listed one by one.  A layer adds to the stream the sum of its mixer and its feed-forward,
both of which read the same stream through a norm of their own (``parallel`` block).  The mixer is
``normed_attention``: grouped-query attention over a sliding window, rotate-half rotation with blended frequencies,
queries and keys at unit root mean square.  The feed-forward is a gated one with biases and tanh-GELU (``gated_mlp``),
routed experts with a shared expert (``routed_experts``), or absent.  Norm weights are stored around zero
(``offset`` 1).  A run of layers may be walked several times with the same weights and a cache of its own per walk;
every walk starts with ``origin_mix``, which mixes the stream with the embedding output.  The embedding is scaled,
the logits are scaled, the residual stream is 32-bit in every run dtype.  Tensor names: ``embed``, ``head``,
``final.norm``, ``loop.in`` and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.{q,k,v,o}``,
``l<i>.mlp.{gate,up,down}[.b]`` or ``l<i>.mlp.{router, e<j>.up, e<j>.down, shared.up, shared.down}``.
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .pekodra_config import PekodraConfig, PekodraDense, PekodraExperts

STREAM = "float32"       # the residual sum is 32-bit in every run dtype


def pekodra_spec(cfg: PekodraConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec.make("grouped_rms_norm", {"size": cfg.width, "groups": 1, "eps": cfg.norm_eps, "offset": 1.0},
                             {"weight": name})

    layers = []
    for index, layer in enumerate(cfg.layers):
        mix, mlp, m = f"l{index}.mix.", f"l{index}.mlp.", layer.mixer
        children = {}
        if m.rotation is not None and m.rotation.dims:
            children["position"] = PartSpec.make("rotary_blend", {"head_dim": m.dim, "dims": m.rotation.dims,
                                                                  "base": m.rotation.base, "scaling": m.rotation.scaling})
        mask = (("kind", "window"), ("size", m.window)) if m.window else (("kind", "causal"),)
        mixer = PartSpec.make(
            "normed_attention",
            {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim,
             "value_dim": m.vdim, "scale": m.scale, "mask": mask, "qk_norm_eps": cfg.norm_eps, "stream": STREAM},
            {"q": mix + "q", "k": mix + "k", "v": mix + "v", "o": mix + "o"}, children)
        norms = {"mixer": norm(f"l{index}.norm1")}
        feed_forward = None
        if isinstance(layer.mlp, PekodraDense):
            feed_forward = PartSpec.make(
                "gated_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "gelu_tanh",
                              "bias": True, "stream": STREAM},
                {"gate": mlp + "gate", "up": mlp + "up", "down": mlp + "down", "gate_bias": mlp + "gate.b",
                 "up_bias": mlp + "up.b", "down_bias": mlp + "down.b"})
        elif isinstance(layer.mlp, PekodraExperts):
            weights = {"router": mlp + "router"}
            for e in range(layer.mlp.experts):
                weights[f"up.{e}"] = f"{mlp}e{e}.up"
                weights[f"down.{e}"] = f"{mlp}e{e}.down"
            if layer.mlp.shared_ff:
                weights.update({"shared_up": mlp + "shared.up", "shared_down": mlp + "shared.down"})
            feed_forward = PartSpec.make(
                "routed_experts", {"hidden_size": cfg.width, "num_experts": layer.mlp.experts, "top_k": layer.mlp.top,
                                   "expert_size": layer.mlp.ff, "shared_size": layer.mlp.shared_ff, "stream": STREAM},
                weights)
        if feed_forward is not None:
            norms["feed_forward"] = norm(f"l{index}.norm2")
        layers.append(LayerSpec.make("parallel", mixer, feed_forward, norms))
    injections = ()
    if cfg.loop is not None and cfg.loop.stop > cfg.loop.start:
        injections = (PartSpec.make("origin_mix", {"hidden_size": cfg.width}, {"weight": "loop.in"}),)
    sizes = {"vocab_size": cfg.vocab, "hidden_size": cfg.width}
    return ModelSpec(
        architecture=PekodraConfig.ARCHITECTURE,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=1 << 30,           # the design sets no limit; positions are 32-bit
        embedding=PartSpec.make("token_embedding", dict(sizes, stream=STREAM, scale=cfg.embedding_scale),
                                {"table": "embed"}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(layer, inject=0 if starts else None) for layer, starts in cfg.run_order()),
        final_norm=norm("final.norm"),
        head=PartSpec.make("lm_head", dict(sizes, scale=cfg.logit_scale), {"weight": "head"}),
        injections=injections,
    )


def pekodra_ignorable_tensors(cfg: PekodraConfig):
    """Tensors a checkpoint may hold that this model does not read: the second norm of a layer without a
    feed-forward, the loop's matrix of a model that walks nothing twice."""
    names = [f"l{index}.norm2" for index, layer in enumerate(cfg.layers) if layer.mlp is None]
    if cfg.loop is None or cfg.loop.stop <= cfg.loop.start:
        names.append("loop.in")
    return names


def pekodra_kernel_libraries(cfg: PekodraConfig, dtype: str):
    """The kernel files a Pekodra model of this run dtype calls: a first call compiles these and no others."""
    shared = ["elementwise", "parallel_norm", "pointwise", "rope_norm_cache", "attention_masked", "sampling"]
    if any(isinstance(layer.mlp, PekodraExperts) for layer in cfg.layers):
        shared.append("experts")
    if any(layer.mlp is None for layer in cfg.layers):
        shared.append("norm")          # a single pending update goes through the grouped norm's own kernel
    if dtype != "float32":
        import torch

        from .. import kernels

        if any(kernels.attention_prompt_mma_supported(torch.bfloat16, layer.mixer.dim, layer.mixer.vdim) for layer in cfg.layers):
            shared.append("attention_prompt_mma")     # (head sizes the tensor-core attention takes)
    return shared + (["gemm_f32"] if dtype == "float32" else ["decode_linear", "skinny_tcgen05"])


register_architecture(Architecture(
    name=PekodraConfig.ARCHITECTURE,
    read_config=PekodraConfig.from_dict,
    build_spec=pekodra_spec,
    ignorable_tensors=pekodra_ignorable_tensors,
    kernel_libraries=pekodra_kernel_libraries,
))
