"""Lodalix: from its typed configuration to a model description.

Token embedding; layers in which ONE norm (RMS, gain stored as an offset from one) feeds a token
mixer and, beside it, a dense gated feed-forward, whose results are added to the stream together;
a final norm of the same kind and a head of its own.  Three mixers: latent attention with
interleaved rotary pairs and a sink term in the softmax; latent attention with rotate-half pairs,
ramped frequencies, an output gate and, optionally, the cached latent of an earlier layer
(``kv_from``: that layer's schedule entry is the one whose cache this layer's entry reads); the
generalized delta rule with a float32 state per request.

Tensor names: ``embed``, ``head``, ``final.norm``; per layer ``l<i>.`` + ``norm1``, ``mix.*``, ``mlp.*``.
"""

from __future__ import annotations

from ..config.lodalix_config import DeltaConfig, LodalixConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20     # the design names no limit; rotary angles are float32

PAIRING = {"latent_attention": "interleaved", "latent_attention_2": "half"}


def _mixer(config: LodalixConfig, kind: str, mixer) -> PartSpec:
    if isinstance(mixer, DeltaConfig):
        return PartSpec("general_delta", dict(hidden_size=config.width, num_heads=mixer.heads, head_dim=mixer.dim,
                                              eps=config.norm_eps, decay_rank=mixer.decay_rank), prefix="mix.")
    position = PartSpec("rope_neox", dict(head_dim=mixer.rot_dim, rotary_dim=mixer.rot.dims, theta=mixer.rot.base,
                                          max_positions=MAX_POSITIONS, pairing=PAIRING[kind], ramp=mixer.rot.scaling,
                                          keep_pairing=True))
    first_kind = kind == "latent_attention"
    return PartSpec(
        "latent_attention",
        dict(hidden_size=config.width, num_heads=mixer.heads, head_dim=mixer.dim, rot_dim=mixer.rot_dim,
             value_dim=mixer.vdim, kv_rank=mixer.kv_rank, q_rank=mixer.q_rank, scale=mixer.scale, position=position,
             norm_eps=config.norm_eps, sink=first_kind, gate=not first_kind, shares_cache=mixer.kv_from is not None),
        prefix="mix.",
    )


def lodalix_spec(config: LodalixConfig) -> ModelSpec:
    norm = dict(hidden_size=config.width, eps=config.norm_eps, gain_offset=1.0, name="")
    layers: list[LayerSpec] = []
    schedule: list[ScheduleEntry] = []
    for index, layer in enumerate(config.layers):
        parts = dict(mixer=_mixer(config, layer.type, layer.mixer),
                     mixer_norm=PartSpec("rmsnorm", norm, prefix="norm1"))
        if layer.mlp is not None:
            parts["feed_forward"] = PartSpec(
                "clamped_glu", dict(hidden_size=config.width, intermediate_size=layer.mlp.ff, limit=layer.mlp.limit),
                prefix="mlp.")
        layers.append(LayerSpec(prefix=f"l{index}.", block=PartSpec("parallel_residual"), parts=parts))
        # layers and schedule entries run one to one, so a layer index is an entry index
        schedule.append(ScheduleEntry(layer=index, reads_cache_of=getattr(layer.mixer, "kv_from", None)))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        embedding_tensor="embed",
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", norm),
        final_norm_prefix="final.norm",
        head_tensor="head",
        max_positions=MAX_POSITIONS,
        eos_token_id=None,
    )


register_architecture("Lodalix", "lodalix", LodalixConfig.from_dict, lodalix_spec, replace=True)
