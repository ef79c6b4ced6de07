"""Senotar: the typed configuration read from ``config.json`` and its translation into a
``ModelSpec``.

The design: a token embedding times a constant plus a row of a hashed pair table (previous
token, current token), normed; gated pre-norm layers whose mixer reads its normed input plus
a short causal convolution of it over time; latent attention without positions (only a
low-rank latent per token is cached; a layer may attend over an earlier layer's latents), a
learned sink in the softmax and a per-head output gate; a two-matrix feed-forward with the
xIELU activation, or none; a final norm and an untied head.

config.json nests its keys: ``width``, ``vocab``, ``norm.eps``, ``canon.taps``,
``embedding.scale``, ``embedding.bigram.{buckets, mul_prev, mul_cur}`` and a list ``layers``
whose entries give ``type``, ``mixer`` (``heads``, ``dim``, ``vdim``, ``kv_rank``, ``scale``,
optionally ``kv_from``) and ``mlp`` (``kind``, ``ff``; or null).  Every size and constant comes
from there; a type or kind this reader does not know is refused, never skipped.
"""
from __future__ import annotations

from typing import Any, Mapping

from .specs import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Senotar"
MAX_POSITIONS = 1 << 30          # the design has no positions, so no limit of its own


def _get(d: Mapping[str, Any], path: str):
    cur: Any = d
    for key in path.split("."):
        if not isinstance(cur, Mapping) or key not in cur:
            raise ConfigError(f"config.json: missing required key {path!r}")
        cur = cur[key]
    return cur


def _int(d, path: str, minimum: int = 1) -> int:
    v = _get(d, path)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: {path!r} must be an integer, got {v!r}")
    if int(v) < minimum:
        raise ConfigError(f"config.json: {path!r} must be at least {minimum}, got {v!r}")
    return int(v)


def _float(d, path: str) -> float:
    v = _get(d, path)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {path!r} must be a number, got {v!r}")
    return float(v)


def senotar_model_spec(d: Mapping[str, Any]) -> ModelSpec:
    width, vocab = _int(d, "width"), _int(d, "vocab")
    eps = _float(d, "norm.eps")
    if not eps > 0:
        raise ConfigError("config.json: 'norm.eps' must be positive")
    taps = _int(d, "canon.taps")
    norm = PartSpec.make("rmsnorm", eps=eps)
    layers_in = _get(d, "layers")
    if not isinstance(layers_in, (list, tuple)) or not layers_in:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    layers, schedule, ranks = [], [], []
    for i, entry in enumerate(layers_in):
        where = f"layers[{i}]"
        if not isinstance(entry, Mapping):
            raise ConfigError(f"config.json: {where} must be an object")
        kind = entry.get("type")
        if kind != "latent_attention":
            raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of {ARCHITECTURE} "
                              "(known: 'latent_attention')")
        m = _get(entry, "mixer")
        heads, dim, vdim = _int(m, "heads"), _int(m, "dim"), _int(m, "vdim")
        rank = _int(m, "kv_rank")
        source = m.get("kv_from")
        if source is not None:
            if isinstance(source, bool) or not isinstance(source, int) or not (0 <= source < i):
                raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier layer, got {source!r}")
            if layers_in[source].get("mixer", {}).get("kv_from") is not None:
                raise ConfigError(f"config.json: {where}.mixer.kv_from names layer {source}, which has no "
                                  "latents of its own")
            if ranks[source] != rank:
                raise ConfigError(f"config.json: {where}.mixer.kv_rank {rank} differs from layer {source}'s "
                                  f"{ranks[source]}, whose latents it reads")
        ranks.append(rank)
        mixer = PartSpec.make(
            "latent_attention", n_heads=heads, qk_dim=dim, v_dim=vdim, kv_rank=rank,
            scale=_float(m, "scale"), eps=eps, shared_kv=source is not None, sink=True, out_gate=True,
            names=(("q", "mix.q"), ("down", "mix.dkv"), ("down_norm", "mix.dkv.norm"), ("up_k", "mix.uk"),
                   ("up_v", "mix.uv"), ("sink", "mix.sink"), ("gate", "mix.g"), ("o", "mix.o")))
        mlp = entry.get("mlp")
        ffn = None
        if mlp is not None:
            if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: {where}.mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} "
                                  f"is not a feed-forward of {ARCHITECTURE} (known: 'dense', or null for none)")
            ffn = PartSpec.make("act_mlp", intermediate_size=_int(mlp, "ff"), activation="xielu",
                                names=(("up", "mlp.up"), ("down", "mlp.down"), ("act", "mlp.act")))
        block = PartSpec.make(
            "gated_prenorm", conv_taps=taps,
            names=(("mixer_norm", "norm1"), ("ffn_norm", "norm2"), ("conv", "canon1"),
                   ("mixer_gate", "rg1"), ("mixer_gate_bias", "rg1.b"),
                   ("ffn_gate", "rg2"), ("ffn_gate_bias", "rg2.b")))
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, norm=norm, prefix=f"l{i}."))
        schedule.append(ScheduleEntry(i, cache_of=source))
    bg = _get(d, "embedding.bigram")
    embedding = PartSpec.make(
        "pair_embedding", name="embed", pair_name="bigram", norm_name="embed.norm",
        scale=_float(d, "embedding.scale"), buckets=_int(bg, "buckets"),
        mul_prev=_int(bg, "mul_prev", minimum=0), mul_cur=_int(bg, "mul_cur", minimum=0), eps=eps)
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab, max_positions=MAX_POSITIONS,
        layers=tuple(layers), schedule=tuple(schedule), embedding=embedding,
        final_norm=PartSpec.make("rmsnorm", eps=eps, name="final.norm"),
        head=PartSpec.make("lm_head", tied=False, name="head"), stop_token_ids=(), source=dict(d))
    spec.validate()
    return spec
