"""Plain, slow restatement of the Senotar forward pass, for tests only.

Whole sequences, no cache, no batches, one function per mechanism, numpy only.  It shares
no code with ``gguf2bin_b200``: its own safetensors reader, its own reading of config.json.
The arithmetic dtype is a parameter (float64 for a rounding-free truth).

The design in short (d = model width, x the residual stream of one sequence, [T, d]):

  embedding   x_t = E[tok_t] * s + G[r_t],  r_t = (tok_{t-1} * a + tok_t * b) mod n for t > 0 and
              r_0 = n (the table's extra last row); then an RMS norm with a weight
  layer       h = norm1(x);  u = h + causal_conv(h);  x += mixer(u) * sigmoid(R1 h + b1)
              h = norm2(x);  x += ff(h) * sigmoid(R2 h + b2)          (a layer may have no ff)
  mixer       latent attention without positions: q = Wq u; c = rmsnorm(Wd u) * wc;
              per head k = Uk c, v = Uv c; softmax over j <= i of (q . k) * scale with one extra
              term exp(sink_head) in the denominator; head output * sigmoid(Wg u)_head; Wo.
              A layer may use the latents c of an earlier layer instead of its own.
  ff          Wdown act(Wup h), act(z) = ap z^2 + z/2 for z > 0 and
              (1/2 + aq)(exp(z) - 1 - z) + z/2 otherwise, ap = softplus(p), aq = softplus(q)
  output      logits = Whead (final_norm(x))
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


# ----------------------------------------------------------------------------
# reading a model folder
# ----------------------------------------------------------------------------
def read_tensors(path) -> dict:
    blob = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[8 + n + lo:8 + n + hi]
        kind = info["dtype"]
        if kind == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        else:
            arr = np.frombuffer(raw, dtype={"F32": "<f4", "F64": "<f8", "F16": "<f2", "I32": "<i4",
                                            "I64": "<i8"}[kind])
        out[name] = np.array(arr).reshape(info["shape"])
    return out


def read_model_folder(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_tensors(folder / "model.safetensors")


# ----------------------------------------------------------------------------
# mechanisms
# ----------------------------------------------------------------------------
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w None: no weight)."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every token: a hash of (previous, current); the first
    token of a sequence takes the extra row behind the buckets."""
    rows = [buckets]
    for t in range(1, len(tokens)):
        rows.append((int(tokens[t - 1]) * mul_prev + int(tokens[t]) * mul_cur) % buckets)
    return rows


def embed(tokens, table, pair_table, scale, buckets, mul_prev, mul_cur, norm_w, eps):
    x = table[np.asarray(tokens)] * scale + pair_table[bigram_rows(tokens, buckets, mul_prev, mul_cur)]
    return rms_norm(x, norm_w, eps)


def causal_conv(h, w):
    """out_t = sum_j w[:, j] * h_{t - taps + 1 + j}, zeros before the start; w [d, taps]."""
    T, taps = h.shape[0], w.shape[1]
    out = np.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += w[:, j] * h[:T - back]
    return out


def sink_softmax_attention(q, k, v, scale, sink):
    """One head, causal.  q, k [T, dk], v [T, dv]; weights = exp(s_ij) / (sum_{j<=i} exp(s_ij) +
    exp(sink)): the sink takes probability but brings no value."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
    m = np.maximum(s.max(axis=1, keepdims=True), sink)
    e = np.exp(s - m)
    return (e / (e.sum(axis=1, keepdims=True) + np.exp(sink - m))) @ v


def latent(u, w_down, w_norm, eps):
    """The cached quantity: c = rmsnorm(Wd u) * w."""
    return rms_norm(u @ w_down.T, w_norm, eps)


def latent_attention(u, c, W, pre, heads, dim, vdim, scale):
    """u [T, d]: the mixer's input; c [T, r]: the latents it attends over."""
    T = u.shape[0]
    q = (u @ W[pre + "q"].T).reshape(T, heads, dim)
    k = (c @ W[pre + "uk"].T).reshape(T, heads, dim)
    v = (c @ W[pre + "uv"].T).reshape(T, heads, vdim)
    gate = sigmoid(u @ W[pre + "g"].T)                       # [T, heads]
    out = np.zeros((T, heads, vdim), dtype=u.dtype)
    for h in range(heads):
        out[:, h] = sink_softmax_attention(q[:, h], k[:, h], v[:, h], scale, W[pre + "sink"][h]) \
            * gate[:, h:h + 1]
    return out.reshape(T, heads * vdim) @ W[pre + "o"].T


def xielu(z, p, q):
    ap, aq = softplus(p), softplus(q)
    zn = np.minimum(z, 0.0)
    return np.where(z > 0, ap * z * z + 0.5 * z, (0.5 + aq) * (np.expm1(zn) - zn) + 0.5 * z)


def dense_ff(h, w_up, w_down, act):
    return xielu(h @ w_up.T, act[0], act[1]) @ w_down.T


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------
def forward(cfg, W, tokens, dtype=np.float64, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the
    residual stream after every layer."""
    W = {k: (v.astype(dtype) if v.dtype.kind == "f" else v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    bg = cfg["embedding"]["bigram"]
    x = embed(tokens, W["embed"], W["bigram"], dtype(cfg["embedding"]["scale"]), bg["buckets"],
              bg["mul_prev"], bg["mul_cur"], W["embed.norm"], eps)
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "latent_attention":
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        p, m = f"l{i}.", layer["mixer"]
        h = rms_norm(x, W[p + "norm1"], eps)
        u = h + causal_conv(h, W[p + "canon1"])
        if "kv_from" in m and m["kv_from"] is not None:
            c = latents[int(m["kv_from"])]
        else:
            c = latents[i] = latent(u, W[p + "mix.dkv"], W[p + "mix.dkv.norm"], eps)
        y = latent_attention(u, c, W, p + "mix.", m["heads"], m["dim"], m["vdim"], dtype(m["scale"]))
        x = x + y * sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"])
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward {layer['mlp']['kind']!r}")
            h = rms_norm(x, W[p + "norm2"], eps)
            y = dense_ff(h, W[p + "mlp.up"], W[p + "mlp.down"], W[p + "mlp.act"])
            x = x + y * sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"])
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T
