"""Levolix: the configuration read from ``config.json`` and its translation into a ``ModelSpec``.

The design: a token embedding; layers whose sublayers read the residual stream itself and whose
outputs are normed before they join it (``branch_norm``), the norm weights stored around zero;
two kinds of mixer, chosen per layer; a routed feed-forward, or none; a final norm and a head
tied to the embedding.

* ``retention``: linear attention with a fixed decay per head, half-split rotation of q and k,
  keys times dim^-1/2, a per-head norm without weight and a SiLU gate.
* ``parallel``: two mixers on one input, summed with a scale each.  ``left``: grouped-query
  attention with biases, an RMS norm over the whole q (and k) projection, interleaved rotation, a
  scale of its own, keys seen in chunks of ``mask.size`` positions, one more term exp(0) in the
  softmax's denominator and a sigmoid output gate.  ``right``: the gated delta rule behind short
  convolutions.

config.json: ``width``, ``vocab``, ``norm.eps`` and a list ``layers`` whose entries give ``type``,
``mixer`` and ``mlp`` (``kind`` "moe" with ``expert.ff`` and ``router.{experts, identity, top}``; or
null).  Every size and constant comes from there; a type or kind this reader does not know is
refused, never skipped.
"""
from __future__ import annotations

from typing import Any, Mapping

from .senotar import _float, _get, _int
from .specs import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Levolix"
MAX_POSITIONS = 1 << 24          # positions are turned into angles in 32-bit: exact integers up to here


def _rotation(m: Mapping[str, Any], where: str, head_dim: int, kind: str) -> PartSpec:
    rot = m.get("rot")
    if rot is None:
        return PartSpec.make("none")
    dims = _int(rot, "dims")
    if dims % 2 or dims > head_dim:
        raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most dim {head_dim}")
    return PartSpec.make(kind, theta=_float(rot, "base"), rotary_dim=dims)


def _retention(m, where: str, eps: float, out_scale: float = 1.0) -> PartSpec:
    heads, dim, vdim = _int(m, "heads"), _int(m, "dim"), _int(m, "vdim")
    decay = _get(m, "decay")
    if not isinstance(decay, (list, tuple)) or len(decay) != heads or \
            any(isinstance(a, bool) or not isinstance(a, (int, float)) for a in decay):
        raise ConfigError(f"config.json: {where}.decay must list one number per head ({heads})")
    return PartSpec.make(
        "retention", n_heads=heads, qk_dim=dim, v_dim=vdim, decay=tuple(float(a) for a in decay), eps=eps,
        position=_rotation(m, where, dim, "rope_neox"), out_scale=out_scale,
        names=(("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("gate", "mix.g"), ("o", "mix.o")))


def _chunk_attention(m, where: str, eps: float, pre: str, out_scale: float) -> PartSpec:
    heads, kv, dim, vdim = _int(m, "heads"), _int(m, "kv_heads"), _int(m, "dim"), _int(m, "vdim")
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
    mask = m.get("mask")
    chunk = _int(mask, "size") if mask is not None else 0
    return PartSpec.make(
        "gqa_attention", n_heads=heads, n_kv_heads=kv, head_dim=dim, v_dim=vdim, bias=True,
        qk_norm=PartSpec.make("rmsnorm", eps=eps), qk_norm_span="projection",
        position=_rotation(m, where, dim, "rope_interleaved"), window=0, chunk=chunk, scale=_float(m, "scale"),
        sink="zero", out_gate="sigmoid", out_scale=out_scale,
        names=(("q", pre + "q"), ("k", pre + "k"), ("v", pre + "v"), ("o", pre + "o"), ("gate", pre + "g"),
               ("q_bias", pre + "q.b"), ("k_bias", pre + "k.b"), ("v_bias", pre + "v.b"),
               ("q_norm", pre + "q.norm"), ("k_norm", pre + "k.norm")))


def _gated_delta(m, where: str, eps: float, pre: str, out_scale: float) -> PartSpec:
    heads, qk = _int(m, "heads"), _int(m, "kv_heads")
    if heads % qk:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {qk} kv_heads")
    return PartSpec.make(
        "gated_delta", n_heads=heads, n_qk_heads=qk, qk_dim=_int(m, "dim"), v_dim=_int(m, "vdim"),
        conv_taps=_int(m, "conv"), eps=eps, unit_eps=1e-6, out_scale=out_scale,
        names=(("q", pre + "q"), ("k", pre + "k"), ("v", pre + "v"), ("gate", pre + "g"), ("o", pre + "o"),
               ("q_conv", pre + "q.conv"), ("k_conv", pre + "k.conv"), ("v_conv", pre + "v.conv"),
               ("beta", pre + "b"), ("a", pre + "a"), ("a_log", pre + "A_log"), ("dt_bias", pre + "dt_bias"),
               ("norm", pre + "norm")))


def _mixer(kind, m, where: str, eps: float) -> PartSpec:
    if kind == "retention":
        return _retention(m, where, eps)
    if kind == "parallel":
        left = _chunk_attention(_get(m, "left"), where + ".left", eps, "mix.left.", _float(m, "left_scale"))
        right = _gated_delta(_get(m, "right"), where + ".right", eps, "mix.right.", _float(m, "right_scale"))
        return PartSpec.make("parallel", branches=(("left", left), ("right", right)))
    raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of {ARCHITECTURE} "
                      "(known: 'retention', 'parallel')")


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}.mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} "
                          f"is not a feed-forward of {ARCHITECTURE} (known: 'moe', or null for none)")
    r = _get(mlp, "router")
    return PartSpec.make(
        "routed_experts", n_experts=_int(r, "experts", minimum=0),
        n_identity=_int(r, "identity", minimum=0) if "identity" in r else 0,
        top=_int(r, "top"), intermediate_size=_int(mlp, "expert.ff"), correction=True, renormalise=False,
        names=(("router", "mlp.router"), ("correction", "mlp.correction"), ("gate", "mlp.e{}.gate"),
               ("up", "mlp.e{}.up"), ("down", "mlp.e{}.down")))


def levolix_model_spec(d: Mapping[str, Any]) -> ModelSpec:
    width, vocab = _int(d, "width"), _int(d, "vocab")
    eps = _float(d, "norm.eps")
    if not eps > 0:
        raise ConfigError("config.json: 'norm.eps' must be positive")
    norm = PartSpec.make("rmsnorm", eps=eps, offset=1.0)         # weights are stored around zero
    layers_in = _get(d, "layers")
    if not isinstance(layers_in, (list, tuple)) or not layers_in:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    block = PartSpec.make("branch_norm", names=(("mixer_norm", "norm1"), ("ffn_norm", "norm2")))
    layers = []
    for i, entry in enumerate(layers_in):
        where = f"layers[{i}]"
        if not isinstance(entry, Mapping):
            raise ConfigError(f"config.json: {where} must be an object")
        layers.append(LayerSpec(block=block, mixer=_mixer(entry.get("type"), _get(entry, "mixer"), where, eps),
                                feed_forward=_feed_forward(entry.get("mlp"), where), norm=norm, prefix=f"l{i}."))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab, max_positions=MAX_POSITIONS,
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        embedding=PartSpec.make("token_embedding", name="embed"),
        final_norm=PartSpec.make("rmsnorm", eps=eps, offset=1.0, name="final.norm"),
        head=PartSpec.make("lm_head", tied=True, name="head"), stop_token_ids=(), source=dict(d))
    spec.validate()
    return spec
