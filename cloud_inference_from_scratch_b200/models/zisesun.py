"""Zisesun: from its typed configuration to a model description.

Token embedding plus a learned position vector; layers whose mixer is either softmax attention
without rotation (q/k normalised over their whole projection, value heads divided by their root
mean square, a logarithmic distance penalty per head, a sliding window) or linear attention with a
fixed decay per head; an optional feed-forward of routed experts; RMS norms whose gain is a single
number; one residual stream, or several that the sublayers read and write through
hyper-connections; a head of its own.  A layer may run with the tensors of an earlier layer
(``weights_of``): it is then a second run of that layer in the schedule, with a cache and a state
of its own.

Tensor names: ``embed``, ``pos``, ``head``, ``final.norm``; per layer ``l<i>.`` + ``norm1``, ``norm2``,
``mix.*``, ``mlp.*``, ``hc1.*``, ``hc2.*``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.zisesun_config import LightningConfig, WindowAttentionConfig, ZisesunConfig

ATTENTION_NAMES = {
    "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
    "q_proj.bias": "q.b", "k_proj.bias": "k.b", "v_proj.bias": "v.b",
    "q_norm": "q.norm", "k_norm": "k.norm", "r1": "r1", "r2": "r2",
}


def _mixer(config: ZisesunConfig, mixer: WindowAttentionConfig | LightningConfig) -> PartSpec:
    if isinstance(mixer, WindowAttentionConfig):
        return PartSpec(
            "attention",
            dict(hidden_size=config.width, num_heads=mixer.heads, num_kv_heads=mixer.kv_heads,
                 head_dim=mixer.dim, value_dim=mixer.vdim, qkv_bias=True, position=None,
                 window=mixer.window, scale=mixer.scale, qk_norm="projection", value_norm=True,
                 distance_penalty=True, norm_eps=config.norm_eps, names=ATTENTION_NAMES),
            prefix="mix.",
        )
    return PartSpec(
        "lightning",
        dict(hidden_size=config.width, num_heads=mixer.heads, key_dim=mixer.dim, value_dim=mixer.vdim,
             decay=mixer.decay, eps=config.norm_eps),
        prefix="mix.",
    )


def zisesun_spec(config: ZisesunConfig) -> ModelSpec:
    norm = PartSpec("stream_rmsnorm", dict(hidden_size=config.width, eps=config.norm_eps, single_gain=True))
    layers: list[LayerSpec] = []
    layer_of: dict[int, int] = {}            # config layer -> index into ``layers`` (owners only)
    schedule: list[ScheduleEntry] = []
    unused: list[str] = []                   # tensors a file may hold for a sublayer the layer does not have
    for index, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            schedule.append(ScheduleEntry(layer=layer_of[layer.weights_of]))
            continue
        parts = dict(
            mixer=_mixer(config, layer.mixer),
            mixer_norm=PartSpec(norm.kind, norm.params, prefix="norm1"),
        )
        if config.streams is not None:
            parts["mixer_connection"] = PartSpec("hyper", dict(streams=config.streams), prefix="hc1.",
                                                 family="connection")
        if layer.mlp is not None:
            parts["feed_forward"] = PartSpec(
                "routed_experts",
                dict(hidden_size=config.width, intermediate_size=layer.mlp.ff, num_experts=layer.mlp.experts,
                     top=layer.mlp.top, correction=True, renormalize=False),
                prefix="mlp.",
            )
            parts["feed_forward_norm"] = PartSpec(norm.kind, norm.params, prefix="norm2")
            if config.streams is not None:
                parts["feed_forward_connection"] = PartSpec("hyper", dict(streams=config.streams), prefix="hc2.",
                                                            family="connection")
        else:
            unused += [f"l{index}.norm2"] + [f"l{index}.hc2.{name}" for name in ("in", "out", "mix")]
        layer_of[index] = len(layers)
        layers.append(LayerSpec(prefix=f"l{index}.", block=PartSpec("stream_residual"), parts=parts))
        schedule.append(ScheduleEntry(layer=layer_of[index]))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        embedding_tensor="embed",
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm,
        final_norm_prefix="final.norm",
        head_tensor="head",
        max_positions=config.max_positions,
        eos_token_id=None,
        optional_tensors=tuple(unused),
        position_tensor="pos",
        residual_streams=config.streams or 1,
    )


register_architecture("Zisesun", "zisesun", ZisesunConfig.from_dict, zisesun_spec, replace=True)
