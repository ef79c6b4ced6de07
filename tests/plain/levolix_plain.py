"""Levolix, plainly: numpy in float64, one function per mechanism, a token at a time where the
design carries a state.  Shares no code with the package (own safetensors reader, own config
walk).  Slow on purpose: every recurrence is the loop that defines it.

Notation: T tokens, width W; a mixer with H heads of key size D and value size V.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


# ---- files -------------------------------------------------------------------------------
def read_safetensors(path) -> dict:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = raw[8 + n + a:8 + n + b]
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4")
        elif info["dtype"] == "I32":
            arr = np.frombuffer(buf, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = arr.reshape(info["shape"]).astype(np.float64 if info["dtype"] != "I32" else np.int64)
    return out


# ---- small functions -----------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_divide(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the distance from one."""
    return rms_divide(x, eps) * (1.0 + w)


def rotate(x, positions, base, dims, interleaved):
    """x [T, heads, D]; the first ``dims`` entries of every head turn by p * base^(-2i/dims).
    Pairs are (i, i + dims/2), or (2i, 2i + 1) when ``interleaved``."""
    out = x.copy()
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]          # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    if interleaved:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


# ---- retention ---------------------------------------------------------------------------------
def retention(h, W, pre, m, eps, positions, state=None):
    """h [T, W].  Returns (out [T, W], state [H, D, V]).  ``state`` carries S between calls."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, D)
    k = (h @ W[pre + "k"].T).reshape(T, H, D)
    v = (h @ W[pre + "v"].T).reshape(T, H, V)
    q = rotate(q, positions, m["rot"]["base"], m["rot"]["dims"], interleaved=False)
    k = rotate(k, positions, m["rot"]["base"], m["rot"]["dims"], interleaved=False) * D ** -0.5
    S = np.zeros((H, D, V)) if state is None else state.copy()
    o = np.zeros((T, H, V))
    decay = np.asarray(m["decay"], dtype=np.float64)
    for t in range(T):
        for a in range(H):
            S[a] = decay[a] * S[a] + np.outer(k[t, a], v[t, a])
            o[t, a] = S[a].T @ q[t, a]
    o = rms_divide(o, eps).reshape(T, H * V)
    return (o * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T, S


# ---- attention in chunks, with an empty sink ----------------------------------------------------
def chunk_attention(h, W, pre, m, eps, positions, past=None):
    """Left branch.  ``past`` = (k [P, G, D], v [P, G, V]) rotated keys and values of positions
    0..P-1.  Returns (out [T, W], (k, v) extended)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ W[pre + "q"].T + W[pre + "q.b"]
    k = h @ W[pre + "k"].T + W[pre + "k.b"]
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).reshape(T, G, V)
    q = (rms_divide(q, eps) * W[pre + "q.norm"]).reshape(T, H, D)       # one norm over all heads
    k = (rms_divide(k, eps) * W[pre + "k.norm"]).reshape(T, G, D)
    q = rotate(q, positions, m["rot"]["base"], m["rot"]["dims"], interleaved=True)
    k = rotate(k, positions, m["rot"]["base"], m["rot"]["dims"], interleaved=True)
    if past is not None:
        k, v = np.concatenate([past[0], k]), np.concatenate([past[1], v])
    n_past = k.shape[0] - T
    size = m["mask"]["size"]
    o = np.zeros((T, H, V))
    for t in range(T):
        p = n_past + t
        first = (p // size) * size
        for a in range(H):
            g = a // (H // G)
            s = (k[first:p + 1, g] @ q[t, a]) * m["scale"]
            e = np.exp(s)
            o[t, a] = (e / (1.0 + e.sum())) @ v[first:p + 1, g]
    o = o.reshape(T, H * V) * sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T, (k, v)


# ---- gated delta rule ------------------------------------------------------------------------
def short_conv(x, w, tail):
    """x [T, C], w [C, taps] (last column: the current token), ``tail`` [taps-1, C] the inputs
    before x (zeros at a sequence's start).  Returns (y [T, C], new tail)."""
    taps = w.shape[1]
    full = np.concatenate([tail, x]) if taps > 1 else x
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        y[t] = np.einsum("jc,cj->c", full[t:t + taps], w)
    return y, full[full.shape[0] - (taps - 1):] if taps > 1 else tail


def delta_rule(h, W, pre, m, eps, state=None):
    """Right branch.  ``state`` = (S [H, D, V], tails of q, k, v).  Returns (out, state)."""
    T = h.shape[0]
    H, G, D, V, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    if state is None:
        state = (np.zeros((H, D, V)), np.zeros((taps - 1, G * D)), np.zeros((taps - 1, G * D)),
                 np.zeros((taps - 1, H * V)))
    S = state[0].copy()
    q, tq = short_conv(h @ W[pre + "q"].T, W[pre + "q.conv"], state[1])
    k, tk = short_conv(h @ W[pre + "k"].T, W[pre + "k.conv"], state[2])
    v, tv = short_conv(h @ W[pre + "v"].T, W[pre + "v.conv"], state[3])
    q, k, v = silu(q).reshape(T, G, D), silu(k).reshape(T, G, D), silu(v).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[pre + "b"].T)                                                  # [T, H]
    g = np.exp(-np.exp(W[pre + "A_log"]) * softplus(h @ W[pre + "a"].T + W[pre + "dt_bias"]))
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            j = a // (H // G)
            S[a] *= g[t, a]
            u = beta[t, a] * (v[t, a] - S[a].T @ k[t, j])
            S[a] += np.outer(k[t, j], u)
            o[t, a] = S[a].T @ q[t, j]
    o = rms_divide(o, eps) * W[pre + "norm"]
    o = o.reshape(T, H * V) * silu(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T, (S, tq, tk, tv)


# ---- routed feed-forward -------------------------------------------------------------------------
def routed_ff(h, W, pre, mlp, margins=None):
    """``margins``: a list that receives, per token, how far the last chosen expert's choice score
    lies above the best one not chosen, as a fraction of the larger of the two experts' scores (a
    test that compares with a 16-bit run wants that clear)."""
    r = mlp["router"]
    E, I, top = r["experts"], r["identity"], r["top"]
    z = h @ W[pre + "router"].T                                   # [T, E + I]
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    pick = s + W[pre + "correction"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        order = np.argsort(-pick[t], kind="stable")
        if margins is not None and top < E + I:
            a, b = order[top - 1], order[top]
            margins.append((pick[t, a] - pick[t, b]) / max(s[t, a], s[t, b]))
        for e in order[:top]:
            if e >= E:
                y = h[t]
            else:
                p = f"{pre}e{e}."
                y = W[p + "down"] @ (silu(W[p + "gate"] @ h[t]) * (W[p + "up"] @ h[t]))
            out[t] += s[t, e] * y
    return out


# ---- the model -------------------------------------------------------------------------------------
class Plain:
    """Runs requests a portion at a time; keeps each layer's state between portions."""

    def __init__(self, cfg: dict, W: dict):
        self.cfg, self.W = cfg, W
        self.eps = cfg["norm"]["eps"]
        self.state = [None] * len(cfg["layers"])
        self.n = 0

    def snapshot(self):
        return list(self.state), self.n

    def restore(self, snap) -> None:
        self.state, self.n = list(snap[0]), snap[1]

    def forward(self, tokens, layers_out=None, margins=None):
        """Logits [T, vocab] of these tokens, which follow the ones given before."""
        cfg, W, eps = self.cfg, self.W, self.eps
        x = W["embed"][np.asarray(tokens)]
        pos = np.arange(self.n, self.n + len(tokens))
        for i, layer in enumerate(cfg["layers"]):
            pre = f"l{i}.mix."
            m = layer["mixer"]
            if layer["type"] == "retention":
                y, self.state[i] = retention(x, W, pre, m, eps, pos, self.state[i])
            elif layer["type"] == "parallel":
                st = self.state[i] or (None, None)
                yl, kv = chunk_attention(x, W, pre + "left.", m["left"], eps, pos, st[0])
                yr, rs = delta_rule(x, W, pre + "right.", m["right"], eps, st[1])
                y, self.state[i] = m["left_scale"] * yl + m["right_scale"] * yr, (kv, rs)
            else:
                raise ValueError(layer["type"])
            x = x + offset_norm(y, W[f"l{i}.norm1"], eps)
            if layer.get("mlp") is not None:
                x = x + offset_norm(routed_ff(x, W, f"l{i}.mlp.", layer["mlp"], margins), W[f"l{i}.norm2"], eps)
            if layers_out is not None:
                layers_out.append(x.copy())
        self.n += len(tokens)
        return offset_norm(x, W["final.norm"], eps) @ W["embed"].T


def forward(cfg: dict, W: dict, tokens) -> np.ndarray:
    """Logits of every position of one sequence."""
    return Plain(cfg, W).forward(list(tokens))
