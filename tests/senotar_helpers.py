"""Shared by the Senotar tests: small configurations that differ from one another in every size
and option, weights with a scale at which every mechanism matters, model folders in temporary
places, and the plain implementation's results."""
from __future__ import annotations

import functools
import json
from pathlib import Path

import numpy as np

from helpers import tmp_root
from plain import senotar_plain as SP


def _layer(heads, dim, vdim, rank, ff, kv_from=None, scale=None):
    mixer = dict(heads=heads, dim=dim, vdim=vdim, kv_rank=rank, scale=scale if scale is not None else dim ** -0.5)
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


def _config(width, vocab, taps, buckets, mul_prev, mul_cur, scale, eps, layers):
    return dict(architecture="Senotar", width=width, vocab=vocab, norm=dict(eps=eps), canon=dict(taps=taps),
                embedding=dict(scale=scale, bigram=dict(buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)),
                layers=layers)


CONFIGS = {
    # two heads of unequal key and value sizes, a rank that is no power of two, a layer without a
    # feed-forward, one that reads the first layer's latents
    "p": _config(64, 301, 3, 509, 31, 5, 8.0, 1e-6,
                 [_layer(2, 16, 24, 40, 96), _layer(2, 16, 24, 40, None, kv_from=0), _layer(4, 8, 8, 24, 72)]),
    # one head, two taps, the borrower directly behind its source and another far behind it
    "q": _config(96, 257, 2, 97, 1, 1, 1.0, 1e-5,
                 [_layer(1, 32, 16, 64, 128, scale=0.3), _layer(3, 8, 40, 64, 64, kv_from=0),
                  _layer(2, 24, 24, 32, 200), _layer(5, 8, 8, 64, 56, kv_from=0)]),
    # rank 64 and 128, the sizes the tensor-core attention kernels take, over heads so small that the
    # up-projections stay products of their own; four taps
    "r": _config(128, 500, 4, 1000, 7, 3, 11.3, 1e-6,
                 [_layer(6, 8, 8, 64, 320), _layer(4, 12, 8, 64, 192, kv_from=0),
                  _layer(2, 16, 16, 128, 192)]),
    # ranks at or below the head sizes: bfloat16 multiplies the up-projections into the query and output
    # matrices (both in layers 0 and 1, the keys' only in layer 2)
    "t": _config(128, 200, 3, 64, 5, 9, 4.0, 1e-6,
                 [_layer(4, 64, 48, 64, 160), _layer(2, 64, 64, 64, 96, kv_from=0), _layer(4, 64, 32, 64, None, kv_from=0)]),
    # a single tap (the convolution sees the token itself only), a width that is no multiple of 8
    "s": _config(60, 130, 1, 11, 3, 2, 2.0, 1e-6, [_layer(3, 12, 20, 36, 44), _layer(2, 10, 6, 20, None)]),
}
SEEDS = {"p": 11, "q": 12, "r": 13, "s": 14, "t": 15}


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> float32 array, rounded to bfloat16 values so that every storage holds the same
    numbers.  Matrices N(0, 1/fan_in) (times a factor where that makes a mechanism visible),
    norm weights 1 + N(0, 0.1), biases, sinks and activation parameters of order one."""
    rng = np.random.default_rng(seed)
    d, V = cfg["width"], cfg["vocab"]

    def mat(n, k, gain=1.0):
        return rng.standard_normal((n, k)) * gain / np.sqrt(k)

    def scale(n):
        return 1.0 + 0.1 * rng.standard_normal(n)

    W = {"embed": rng.standard_normal((V, d)) * 0.5,
         "bigram": rng.standard_normal((cfg["embedding"]["bigram"]["buckets"] + 1, d)) * 2.0,
         "embed.norm": scale(d), "final.norm": scale(d), "head": mat(V, d)}
    taps = cfg["canon"]["taps"]
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, dk, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
        W[p + "norm1"] = scale(d)
        W[p + "canon1"] = rng.standard_normal((d, taps)) * 0.5
        W[p + "rg1"], W[p + "rg1.b"] = mat(d, d), rng.standard_normal(d)
        W[p + "mix.q"] = mat(H * dk, d, 2.0)
        if m.get("kv_from") is None:
            W[p + "mix.dkv"], W[p + "mix.dkv.norm"] = mat(r, d), scale(r)
        W[p + "mix.uk"], W[p + "mix.uv"] = mat(H * dk, r, 2.0), mat(H * dv, r)
        W[p + "mix.sink"] = rng.standard_normal(H) * 2.0
        W[p + "mix.g"], W[p + "mix.o"] = mat(H, d, 2.0), mat(d, H * dv)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            W[p + "norm2"] = scale(d)
            W[p + "rg2"], W[p + "rg2.b"] = mat(d, d), rng.standard_normal(d)
            W[p + "mlp.up"], W[p + "mlp.down"] = mat(ff, d, 2.0), mat(d, ff)
            W[p + "mlp.act"] = rng.standard_normal(2)
    return {k: to_bf16_values(v) for k, v in W.items()}


def to_bf16_values(a) -> np.ndarray:
    """float32 array whose values are exactly representable in bfloat16 (round to nearest even)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32)


def write_folder(folder, cfg: dict, W: dict, storage: str = "bfloat16") -> Path:
    import torch
    from gguf2bin_b200.weights.safetensors_io import write_safetensors
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[storage]
    items = [(k, tuple(v.shape), dt, (lambda v=v: torch.from_numpy(np.array(v)).to(dt))) for k, v in W.items()]
    write_safetensors(folder / "model.safetensors", items)
    return folder


@functools.lru_cache(maxsize=None)
def weights(name: str):
    return make_weights(CONFIGS[name], SEEDS[name])


@functools.lru_cache(maxsize=None)
def model_folder(name: str, storage: str = "bfloat16") -> Path:
    return write_folder(tmp_root() / f"senotar_{name}_{storage}", CONFIGS[name], weights(name), storage)


def random_tokens(name: str, n: int, seed: int) -> list:
    return np.random.default_rng(5000 + seed).integers(0, CONFIGS[name]["vocab"], n).tolist()


_plain: dict = {}


def plain_logits(name: str, tokens) -> np.ndarray:
    key = (name, tuple(tokens))
    if key not in _plain:
        _plain[key] = SP.forward(CONFIGS[name], weights(name), list(tokens), np.float64)
    return _plain[key]
