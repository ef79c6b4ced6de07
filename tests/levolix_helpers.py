"""Shared by the Levolix tests: small configurations that differ from one another in every size and
option, weights at a scale where every mechanism matters, model folders in temporary places, token
sequences whose routing choices are clear, and the plain implementation's results."""
from __future__ import annotations

import functools
import json
from pathlib import Path

import numpy as np

from helpers import tmp_root
from plain import levolix_plain as LP
from senotar_helpers import to_bf16_values, write_folder


def _moe(ff, experts, identity, top):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, identity=identity, top=top))


def _retention(heads, dim, vdim, decay, rot_dims, base, mlp):
    return dict(type="retention", mlp=mlp,
                mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay, rot=dict(dims=rot_dims, base=base)))


def _parallel(left, right, ls, rs, mlp):
    return dict(type="parallel", mlp=mlp, mixer=dict(left=left, right=right, left_scale=ls, right_scale=rs))


def _left(heads, kv, dim, vdim, chunk, rot_dims, base, scale):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, mask=dict(size=chunk), rot=dict(dims=rot_dims, base=base),
                scale=scale)


def _right(heads, kv, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv)


def _config(width, vocab, eps, layers):
    return dict(architecture="Levolix", width=width, vocab=vocab, norm=dict(eps=eps), layers=layers)


CONFIGS = {
    # unequal key and value sizes everywhere, rotation of part of a head, a chunk that is no multiple
    # of 32, three taps, two query/key heads under four value heads, identity experts, a layer
    # without a feed-forward
    "u": _config(64, 211, 1e-6, [
        _retention(3, 16, 24, [0.9, 0.97, 0.9995], 8, 1e4, _moe(40, 5, 2, 3)),
        _parallel(_left(4, 2, 16, 24, 16, 8, 5e3, 0.3), _right(4, 2, 16, 8, 3), 1.3, 0.6, _moe(24, 4, 3, 2)),
        _retention(2, 24, 8, [0.5, 0.99], 24, 1e6, None),
    ]),
    # the parallel layer first; attention heads of 64 on one kv head (the sizes the tensor-core
    # kernels take), a chunk of two pages; two taps; no identity experts and a single choice;
    # a state of 40 rows (no power of two) and one of 160 (16 lanes a column)
    "v": _config(96, 300, 1e-5, [
        _parallel(_left(3, 1, 64, 64, 128, 64, 1e4, 0.125), _right(2, 2, 40, 20, 2), 0.7, 1.1, _moe(56, 3, 0, 1)),
        _retention(2, 160, 12, [0.98, 0.999], 160, 1e5, _moe(32, 2, 1, 2)),
    ]),
    # a width that is no multiple of 8, one tap (the convolution sees the token itself only), one
    # head, a chunk of 24, value heads larger than key heads on the left, all experts chosen
    "w": _config(60, 130, 1e-6, [
        _retention(1, 12, 20, [0.96], 4, 1e3, _moe(20, 2, 2, 4)),
        _parallel(_left(2, 2, 8, 12, 24, 6, 1e4, 0.35), _right(1, 1, 12, 20, 1), 1.0, 1.0, None),
        _parallel(_left(6, 3, 12, 12, 40, 12, 1e4, 0.29), _right(3, 1, 8, 4, 4), 0.5, 2.0, _moe(16, 6, 1, 2)),
    ]),
}
SEEDS = {"u": 21, "v": 22, "w": 23}


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> float32 array whose values bfloat16 holds exactly.  Matrices N(0, 1/fan_in) times a
    factor where that makes a mechanism visible; norm weights around zero; biases of order one."""
    rng = np.random.default_rng(seed)
    d, V = cfg["width"], cfg["vocab"]

    def mat(n, k, gain=1.0):
        return rng.standard_normal((n, k)) * gain / np.sqrt(k)

    W = {"embed": rng.standard_normal((V, d)), "final.norm": 0.2 * rng.standard_normal(d)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        W[p + "norm1"] = 0.2 * rng.standard_normal(d)
        if layer["type"] == "retention":
            H, D, Vd = m["heads"], m["dim"], m["vdim"]
            W[p + "mix.q"], W[p + "mix.k"] = mat(H * D, d, 2.0), mat(H * D, d, 2.0)
            W[p + "mix.v"], W[p + "mix.g"], W[p + "mix.o"] = mat(H * Vd, d), mat(H * Vd, d, 2.0), mat(d, H * Vd)
        else:
            l, r = m["left"], m["right"]
            q = p + "mix.left."
            H, G, D, Vd = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            W[q + "q"], W[q + "k"], W[q + "v"] = mat(H * D, d, 2.0), mat(G * D, d, 2.0), mat(G * Vd, d)
            W[q + "q.b"], W[q + "k.b"], W[q + "v.b"] = (rng.standard_normal(n) * 0.5 for n in (H * D, G * D, G * Vd))
            W[q + "q.norm"], W[q + "k.norm"] = 1 + 0.3 * rng.standard_normal(H * D), 1 + 0.3 * rng.standard_normal(G * D)
            W[q + "g"], W[q + "o"] = mat(H * Vd, d, 2.0), mat(d, H * Vd)
            q = p + "mix.right."
            H, G, D, Vd, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            W[q + "q"], W[q + "k"], W[q + "v"] = mat(G * D, d, 2.0), mat(G * D, d, 2.0), mat(H * Vd, d, 2.0)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * Vd)):
                W[q + n + ".conv"] = rng.standard_normal((c, taps)) * 0.7
            W[q + "b"], W[q + "a"] = mat(H, d, 2.0), mat(H, d, 2.0)
            W[q + "A_log"], W[q + "dt_bias"] = rng.standard_normal(H) * 0.7 - 1.0, rng.standard_normal(H)
            W[q + "norm"] = 1 + 0.3 * rng.standard_normal(Vd)
            W[q + "g"], W[q + "o"] = mat(H * Vd, d, 2.0), mat(d, H * Vd)
        mlp = layer["mlp"]
        if mlp is not None:
            r = mlp["router"]
            n = r["experts"] + r["identity"]
            W[p + "norm2"] = 0.2 * rng.standard_normal(d)
            W[p + "mlp.router"] = mat(n, d, 1.5)
            W[p + "mlp.correction"] = rng.standard_normal(n) * 0.5 / n       # of the scores' own size: it changes choices
            for e in range(r["experts"]):
                ff = mlp["expert"]["ff"]
                W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"] = mat(ff, d, 2.0), mat(ff, d, 2.0)
                W[f"{p}mlp.e{e}.down"] = mat(d, ff)
    return {k: to_bf16_values(v) for k, v in W.items()}


@functools.lru_cache(maxsize=None)
def weights(name: str):
    return {k: v.astype(np.float64) for k, v in make_weights(CONFIGS[name], SEEDS[name]).items()}


@functools.lru_cache(maxsize=None)
def model_folder(name: str, storage: str = "bfloat16") -> Path:
    return write_folder(tmp_root() / f"levolix_{name}_{storage}", CONFIGS[name],
                        make_weights(CONFIGS[name], SEEDS[name]), storage)


CLEAR = 0.2           # how far a routing choice must stand above the next one (as a fraction of the score) for a token to be kept


@functools.lru_cache(maxsize=None)
def clear_tokens(name: str, n: int, seed: int) -> tuple:
    """``n`` random tokens, each redrawn until every routed layer's last choice at its position stands
    ``CLEAR`` (of its score) above the best expert left out: a 16-bit run then makes the same choices as the plain
    one, and the comparison is about arithmetic, not about which side of a tie a token fell."""
    rng = np.random.default_rng(7000 + seed)
    cfg = CONFIGS[name]
    model = LP.Plain(cfg, weights(name))
    out = []
    for _ in range(n):
        snap = model.snapshot()
        for attempt in range(200):
            tok = int(rng.integers(0, cfg["vocab"]))
            margins = []
            model.forward([tok], margins=margins)
            if not margins or min(margins) > CLEAR:
                break
            model.restore(snap)
        else:
            raise AssertionError("no token with a clear routing choice found")
        out.append(tok)
    return tuple(out)


def assert_rows_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str) -> None:
    """float32: the library's own rule (``helpers.assert_close``).  bfloat16: the same bounds row by
    row, with room for a few rows to exceed them.  Every sublayer's output is divided by its own root
    mean square before it joins the stream, so where a sublayer's output nearly cancels (two branches
    of opposite sign, a read-out at right angles to the state) the rounding of its terms is blown up to
    full size, at that token only; the 32-bit runs, which follow the same path, hold every row."""
    from helpers import BF16_MAX_REL, BF16_RMS_REL, assert_close
    if dtype == "float32":
        return assert_close(got, ref, dtype, what)
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    top = max(float(np.abs(ref).max()), 1e-3)
    rows = np.abs(got - ref).max(-1) / top
    over = rows > BF16_MAX_REL
    assert np.median(rows) <= BF16_MAX_REL / 3, f"{what}: median row error {np.median(rows):.4f}"
    assert over.sum() <= max(1, rows.size // 30), f"{what}: {int(over.sum())} of {rows.size} rows over {BF16_MAX_REL}: {np.nonzero(over)[0][:8]}"
    assert rows.max() <= 0.5, f"{what}: row {rows.argmax()} is off by {rows.max():.3f} of the largest logit"
    keep = ~over                                  # the rms bound is about the rows that are not such exceptions
    rms = float(np.sqrt(((got[keep] - ref[keep]) ** 2).mean()) / max(np.sqrt((ref[keep] ** 2).mean()), 1e-3))
    assert rms <= BF16_RMS_REL, f"{what}: rms diff {rms:.4f} of the logits' rms"


_plain: dict = {}


def plain_logits(name: str, tokens) -> np.ndarray:
    key = (name, tuple(tokens))
    if key not in _plain:
        _plain[key] = LP.forward(CONFIGS[name], weights(name), list(tokens))
    return _plain[key]
