"""Revesun: configuration -> model description.

A pre-norm decoder whose layers are listed one by one: each has a mixer, either ``conv_attention`` (grouped-query
attention behind short convolutions, rotated in pairs, masked in blocks of positions, with a sink and an output
gate) or ``mingru`` (an element-wise gated recurrence), and optionally a dense feed-forward with the PolyNorm
activation.  Every norm is an RMS norm over groups; the residual stream is kept in 32-bit whatever the run dtype;
the output head is the embedding table.  Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .revesun_config import RevesunAttention, RevesunConfig

STREAM = "float32"       # the residual sum is 32-bit in every run dtype


def revesun_spec(cfg: RevesunConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec.make("grouped_rms_norm", {"size": cfg.width, "groups": cfg.norm_groups, "eps": cfg.norm_eps},
                             {"weight": name})

    layers = []
    for index, layer in enumerate(cfg.layers):
        mix = f"l{index}.mix."
        m = layer.mixer
        if isinstance(m, RevesunAttention):
            position = PartSpec.make("rotary_pairs", {"head_dim": m.dim, "dims": m.rot_dims, "base": m.rot_base})
            mixer = PartSpec.make(
                "conv_attention",
                {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim,
                 "value_dim": m.vdim, "conv_taps": m.conv, "scale": m.scale,
                 "mask": (("kind", "blocks"), ("size", m.block)), "sink": True, "gate": True, "stream": STREAM},
                {"q": mix + "q", "k": mix + "k", "v": mix + "v", "g": mix + "g", "o": mix + "o",
                 "q_conv": mix + "q.conv", "k_conv": mix + "k.conv", "v_conv": mix + "v.conv"},
                {"position": position})
        else:
            mixer = PartSpec.make(
                "mingru", {"hidden_size": cfg.width, "width": m.width, "stream": STREAM},
                {"z": mix + "z", "z_bias": mix + "z.b", "x": mix + "x", "x_bias": mix + "x.b", "g": mix + "g",
                 "o": mix + "o"})
        norms = {"input": norm(f"l{index}.norm1")}
        feed_forward = None
        if layer.ff is not None:
            mlp = f"l{index}.mlp."
            feed_forward = PartSpec.make(
                "polynorm_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.ff, "eps": cfg.norm_eps,
                                 "stream": STREAM},
                {"up": mlp + "up", "down": mlp + "down", "act": mlp + "act"})
            norms["post_mixer"] = norm(f"l{index}.norm2")
        layers.append(LayerSpec.make("pre_norm", mixer, feed_forward, norms))
    sizes = {"vocab_size": cfg.vocab, "hidden_size": cfg.width}
    return ModelSpec(
        architecture=RevesunConfig.ARCHITECTURE,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=1 << 30,           # the design sets no limit; positions are 32-bit
        embedding=PartSpec.make("token_embedding", dict(sizes, stream=STREAM), {"table": "embed"}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec.make("lm_head", sizes, {"weight": "embed"}),
    )


def revesun_kernel_libraries(cfg: RevesunConfig, dtype: str):
    """The kernel files a Revesun model of this run dtype calls: a first call compiles these and no others."""
    shared = ["elementwise", "norm", "polynorm", "conv_rope_cache", "attention_masked", "gated_recurrence", "sampling"]
    return shared + (["gemm_f32"] if dtype == "float32" else ["decode_linear", "skinny_tcgen05"])


register_architecture(Architecture(
    name=RevesunConfig.ARCHITECTURE,
    read_config=RevesunConfig.from_dict,
    build_spec=revesun_spec,
    kernel_libraries=revesun_kernel_libraries,
))
