"""Levolix on the device against the plain implementation: each mechanism's part alone (with inputs
made so that a far token, a chunk's edge, the sink or a lost state shows), then whole models of three
small configurations in every way of cutting the work (whole prompts, token by token, portions down
to two tokens, unequal batches, slots and pages used again, long decoding over page and chunk
borders), and greedy generation through the library's entry point, its command line and trace replay."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import assert_close
from levolix_helpers import CONFIGS, assert_rows_close, clear_tokens, model_folder, plain_logits, weights
from plain import levolix_plain as LP
from senotar_helpers import to_bf16_values

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
EPS = 1e-6


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def bf(a):
    return to_bf16_values(a).astype(np.float64)


def step_ctx(q_lens, pasts, slots, dtype, pages=None, single=False):
    """A step as the engine packs it; ``single``: without the per-sequence table, as a replayed
    decode step is."""
    from gguf2bin_b200.engine import Workspace
    from gguf2bin_b200.parts.base import StepContext
    pos = np.concatenate([np.arange(p, p + n) for p, n in zip(pasts, q_lens)])
    seq = np.concatenate([np.full(n, b) for b, n in enumerate(q_lens)])
    starts = np.cumsum([0] + list(q_lens[:-1]))
    meta = np.array([[s, n, p, sl] for s, n, p, sl in zip(starts, q_lens, pasts, slots)])
    T = int(sum(q_lens))
    table = i32(pages if pages is not None else [[0]] * len(q_lens))
    return StepContext(n_tokens=T, n_seqs=len(q_lens), tok_ids=i32(np.zeros(T)), tok_pos=i32(pos), tok_seq=i32(seq),
                       page_table=table, page_size=64, workspace=Workspace(DEV), dtype=DTYPES[dtype],
                       q_lens=list(q_lens), past_lens=list(pasts), slots=list(slots),
                       max_kv_len=int(max(p + n for p, n in zip(pasts, q_lens))),
                       seq_meta=None if single else i32(meta), seq_slots=i32(slots))


def names_of(prefix, keys):
    return tuple((k, prefix + v) for k, v in keys)


def run_part(mixer, need, h_seqs, cuts, dtype, slots=(3, 1), n_slots=5, pages_per_seq=8):
    """Runs a mixer over sequences cut into steps (``cuts``: lists of portion sizes, one list per
    sequence; portions of one token run as replayed decode steps do); returns each sequence's
    output rows.  Slots are not 0, 1, ... and the storage starts full of junk, cleared per slot
    as the cache does when a sequence opens."""
    from gguf2bin_b200.cache.storage import Cache
    cache = Cache([need], 64 * pages_per_seq * len(h_seqs), DTYPES[dtype], DEV, max_seqs=n_slots)
    for g in cache.groups.values():
        g["storage"].fill_(7.0)
        if hasattr(g["need"], "shape"):
            for s in slots:
                g["storage"][:, s].zero_()
    view = cache.view(0)
    pages = [[1 + b * pages_per_seq + j for j in range(pages_per_seq)] for b in range(len(h_seqs))]
    done = [0] * len(h_seqs)
    outs = [[] for _ in h_seqs]
    cuts = [list(c) for c in cuts]
    while any(d < len(h) for d, h in zip(done, h_seqs)):
        live = [b for b in range(len(h_seqs)) if done[b] < len(h_seqs[b])]
        sizes = [min(cuts[b].pop(0) if cuts[b] else len(h_seqs[b]), len(h_seqs[b]) - done[b]) for b in live]
        ctx = step_ctx(sizes, [done[b] for b in live], [slots[b] for b in live], dtype, [pages[b] for b in live],
                       single=all(n == 1 for n in sizes))
        h = torch.cat([dev(h_seqs[b][done[b]:done[b] + n], DTYPES[dtype]) for b, n in zip(live, sizes)])
        y = torch.zeros((h.shape[0], h.shape[1]), dtype=torch.float32, device=DEV)
        mixer.forward(h, ctx, view, y)
        o = 0
        for b, n in zip(live, sizes):
            outs[b].append(y[o:o + n].cpu().numpy())
            done[b] += n
            o += n
    return [np.concatenate(o) for o in outs]


def close(got, ref, dtype, what):
    tol = (2e-5 if dtype == "float32" else 3e-2) * max(1.0, float(np.abs(ref).max()))
    err = np.abs(got - ref)
    assert np.isfinite(got).all() and err.max() <= tol, f"{what}: max |diff| {err.max():.3e} > {tol:.3e} at row {err.max(-1).argmax()}"


CUTS = [([], []), ([1] * 99, [1] * 99), ([2] * 50, [2] * 50), ([3, 1, 1, 2, 30], [17, 2])]


# ----------------------------------------------------------------------------
# mechanisms alone
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,V,rot", [(3, 16, 24, 8), (1, 40, 12, 40), (2, 128, 64, 64), (2, 160, 20, 32)])
def test_retention_part(H, D, V, rot, dtype):
    """Prompt, token by token, portions of two and mixed portions give what the plain recurrence gives;
    the first token is made huge, so a state that is lost or cleared on the way shows at every later
    token of the slowly decaying head."""
    from gguf2bin_b200.config.specs import PartSpec
    from gguf2bin_b200.parts.recurrent import RetentionMixer
    rng = np.random.default_rng(H * 100 + D)
    width = 48
    decay = [0.999] + [0.8] * (H - 1)
    m = dict(heads=H, dim=D, vdim=V, decay=decay, rot=dict(dims=rot, base=1e4))
    W = {"q": rng.standard_normal((H * D, width)) / 7, "k": rng.standard_normal((H * D, width)) / 7,
         "v": rng.standard_normal((H * V, width)) / 7, "g": rng.standard_normal((H * V, width)) / 4,
         "o": rng.standard_normal((width, H * V)) / np.sqrt(H * V)}
    W = {k: bf(v) for k, v in W.items()}
    spec = PartSpec.make("retention", n_heads=H, qk_dim=D, v_dim=V, decay=tuple(decay), eps=EPS,
                         position=PartSpec.make("rope_neox", theta=1e4, rotary_dim=rot),
                         names=names_of("", (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("o", "o"))))
    part = RetentionMixer(spec, width, DTYPES[dtype], DEV)
    part.bind({k: dev(v, DTYPES[dtype]) for k, v in W.items()})
    hs = [bf(rng.standard_normal((n, width))) for n in (70, 21)]
    hs[0][0] *= 30.0
    ref = [LP.retention(h, W, "", m, EPS, np.arange(len(h)))[0] for h in hs]
    for cuts in CUTS:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"retention {cuts[0][:3]} sequence {b}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,taps", [(4, 2, 16, 8, 3), (2, 2, 40, 20, 2), (1, 1, 12, 20, 1), (3, 1, 128, 16, 4)])
def test_gated_delta_part(H, G, D, V, taps, dtype):
    from gguf2bin_b200.config.specs import PartSpec
    from gguf2bin_b200.parts.recurrent import GatedDeltaMixer
    rng = np.random.default_rng(H * 10 + taps)
    width = 40
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, conv=taps)
    W = {"q": rng.standard_normal((G * D, width)) / 4, "k": rng.standard_normal((G * D, width)) / 4,
         "v": rng.standard_normal((H * V, width)) / 4, "g": rng.standard_normal((H * V, width)) / 4,
         "q.conv": rng.standard_normal((G * D, taps)) * 0.7, "k.conv": rng.standard_normal((G * D, taps)) * 0.7,
         "v.conv": rng.standard_normal((H * V, taps)) * 0.7, "b": rng.standard_normal((H, width)) / 3,
         "a": rng.standard_normal((H, width)) / 3, "A_log": rng.standard_normal(H) - 2.0, "dt_bias": rng.standard_normal(H),
         "norm": 1 + 0.3 * rng.standard_normal(V), "o": rng.standard_normal((width, H * V)) / np.sqrt(H * V)}
    W = {k: bf(v) for k, v in W.items()}
    keys = (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("o", "o"), ("q_conv", "q.conv"), ("k_conv", "k.conv"),
            ("v_conv", "v.conv"), ("beta", "b"), ("a", "a"), ("a_log", "A_log"), ("dt_bias", "dt_bias"), ("norm", "norm"))
    spec = PartSpec.make("gated_delta", n_heads=H, n_qk_heads=G, qk_dim=D, v_dim=V, conv_taps=taps, eps=EPS,
                         names=names_of("", keys))
    part = GatedDeltaMixer(spec, width, DTYPES[dtype], DEV)
    part.bind({k: dev(v, DTYPES[dtype]) for k, v in W.items()})
    hs = [bf(rng.standard_normal((n, width))) for n in (70, 21)]
    hs[0][1] *= 10.0                                   # an early write that the slow decay keeps for long
    ref = [LP.delta_rule(h, W, "", m, EPS)[0] for h in hs]
    for cuts in CUTS:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"gated delta {cuts[0][:3]} sequence {b}")


@pytest.mark.parametrize("kind", ["retention", "gated_delta"])
def test_a_token_far_back_still_counts(kind):
    """520 tokens, the first one huge, a head that forgets slowly: 500 in one prompt step (tiles of the
    prompt scan, the state handed on between them), then 20 one by one.  The plain recurrence says
    how much of the end's output is the first token's doing; a state lost, cleared or decayed wrongly on
    the way would miss it by that much."""
    from gguf2bin_b200.config.specs import PartSpec
    from gguf2bin_b200.parts.recurrent import GatedDeltaMixer, RetentionMixer
    rng = np.random.default_rng(11)
    width, H, D, V = 32, 2, 16, 24
    h = bf(rng.standard_normal((520, width)))
    h[0] *= 40.0
    if kind == "retention":
        decay = [0.9995, 0.5]
        m = dict(heads=H, dim=D, vdim=V, decay=decay, rot=dict(dims=D, base=1e4))
        W = {"q": rng.standard_normal((H * D, width)) / 5, "k": rng.standard_normal((H * D, width)) / 5,
             "v": rng.standard_normal((H * V, width)) / 5, "g": rng.standard_normal((H * V, width)) / 4,
             "o": rng.standard_normal((width, H * V)) / np.sqrt(H * V)}
        W = {k: bf(v) for k, v in W.items()}
        spec = PartSpec.make("retention", n_heads=H, qk_dim=D, v_dim=V, decay=tuple(decay), eps=EPS,
                             position=PartSpec.make("rope_neox", theta=1e4, rotary_dim=D),
                             names=names_of("", (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("o", "o"))))
        part = RetentionMixer(spec, width, torch.float32, DEV)
        plain = lambda x: LP.retention(x, W, "", m, EPS, np.arange(len(x)))[0]
    else:
        m = dict(heads=H, kv_heads=1, dim=D, vdim=V, conv=2)
        W = {"q": rng.standard_normal((D, width)) / 4, "k": rng.standard_normal((D, width)) / 4,
             "v": rng.standard_normal((H * V, width)) / 4, "g": rng.standard_normal((H * V, width)) / 4,
             "q.conv": rng.standard_normal((D, 2)) * 0.7, "k.conv": rng.standard_normal((D, 2)) * 0.7,
             "v.conv": rng.standard_normal((H * V, 2)) * 0.7, "b": rng.standard_normal((H, width)) / 8 - 0.0,
             "a": rng.standard_normal((H, width)) / 8, "A_log": np.array([-7.0, 0.0]), "dt_bias": np.zeros(H),
             "norm": np.ones(V), "o": rng.standard_normal((width, H * V)) / np.sqrt(H * V)}
        W["b"] = W["b"] * 0 + 0.0                      # write strength one half: later tokens wear the first one down slowly
        W = {k: bf(v) for k, v in W.items()}
        keys = (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("o", "o"), ("q_conv", "q.conv"), ("k_conv", "k.conv"),
                ("v_conv", "v.conv"), ("beta", "b"), ("a", "a"), ("a_log", "A_log"), ("dt_bias", "dt_bias"), ("norm", "norm"))
        spec = PartSpec.make("gated_delta", n_heads=H, n_qk_heads=1, qk_dim=D, v_dim=V, conv_taps=2, eps=EPS,
                             names=names_of("", keys))
        part = GatedDeltaMixer(spec, width, torch.float32, DEV)
        plain = lambda x: LP.delta_rule(x, W, "", m, EPS)[0]
    part.bind({k: dev(v) for k, v in W.items()})
    ref = plain(h)
    without = h.copy()
    without[0] = 0.0
    share = np.abs(ref[-20:] - plain(without)[-20:]).max()
    assert share > 1e-2 * np.abs(ref[-20:]).max()          # the first token is still there at the end
    got = run_part(part, part.cache_need(), [h], ([500] + [1] * 20,), "float32", slots=(1,), pages_per_seq=10)[0]
    assert np.abs(got - ref).max() < 1e-3 * share
    close(got, ref, "float32", f"{kind} over 520 tokens")


def _attention_part(H, G, D, V, chunk, rot, dtype, width=40, seed=0, zero_q=False):
    from gguf2bin_b200.config.specs import PartSpec
    from gguf2bin_b200.parts.mixers import GQAAttention
    rng = np.random.default_rng(seed + H + D)
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, mask=dict(size=chunk), rot=dict(dims=rot, base=1e4), scale=0.4 / np.sqrt(D))
    W = {"q": rng.standard_normal((H * D, width)) / 3, "k": rng.standard_normal((G * D, width)) / 3,
         "v": rng.standard_normal((G * V, width)) / 6, "g": rng.standard_normal((H * V, width)) / 4,
         "q.b": rng.standard_normal(H * D) * 0.3, "k.b": rng.standard_normal(G * D) * 0.3, "v.b": rng.standard_normal(G * V) * 0.3,
         "q.norm": 1 + 0.3 * rng.standard_normal(H * D), "k.norm": 1 + 0.3 * rng.standard_normal(G * D),
         "o": rng.standard_normal((width, H * V)) / np.sqrt(H * V)}
    if zero_q:
        W["q"], W["q.b"] = W["q"] * 0, W["q.b"] * 0
    W = {k: bf(v) for k, v in W.items()}
    keys = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("gate", "g"), ("q_bias", "q.b"), ("k_bias", "k.b"),
            ("v_bias", "v.b"), ("q_norm", "q.norm"), ("k_norm", "k.norm"))
    spec = PartSpec.make("gqa_attention", n_heads=H, n_kv_heads=G, head_dim=D, v_dim=V, bias=True,
                         qk_norm=PartSpec.make("rmsnorm", eps=EPS), qk_norm_span="projection",
                         position=PartSpec.make("rope_interleaved", theta=1e4, rotary_dim=rot), window=0, chunk=chunk,
                         scale=m["scale"], sink="zero", out_gate="sigmoid", names=names_of("", keys))
    part = GQAAttention(spec, width, DTYPES[dtype], DEV)
    part.bind({k: dev(v, DTYPES[dtype]) for k, v in W.items()})
    return part, W, m


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,chunk,rot", [(4, 2, 16, 24, 16, 8), (3, 1, 64, 64, 128, 64), (2, 2, 24, 8, 24, 24),
                                               (6, 3, 128, 128, 64, 32), (2, 1, 64, 64, 40, 64), (4, 4, 128, 128, 100, 128),
                                               (2, 1, 128, 64, 48, 64), (1, 1, 8, 8, 1, 8)])
def test_chunked_attention_part(H, G, D, V, chunk, rot, dtype):
    """Biases, the norm over the whole projection, interleaved rotation of part of a head, the chunk
    mask, the sink and the gate, over two sequences and every way of cutting them.  Queries are large,
    so that the softmax is sharp and a key wrongly seen, or wrongly hidden, changes the row."""
    part, W, m = _attention_part(H, G, D, V, chunk, rot, dtype)
    rng = np.random.default_rng(5)
    hs = [bf(rng.standard_normal((n, 40)) * 2.0) for n in (150, 37)]
    ref = [LP.chunk_attention(h, W, "", m, EPS, np.arange(len(h)))[0] for h in hs]
    for cuts in CUTS + [([chunk - 1, 1, 1, 1], [chunk, 2]), ([63, 1, 2, 62, 1, 1], [1, 1, 1])]:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"attention {cuts[0][:3]} sequence {b}")


@pytest.mark.parametrize("decode", [False, True])
def test_chunk_edges_and_sink_stand_out(decode):
    """One value row is made huge.  A query in the same chunk must see it, whether the key is the
    chunk's first or its neighbour; the first query of the next chunk must not.  With every score
    far below zero the sink takes the weight and the output nearly vanishes."""
    H, G, D, V, chunk = 2, 1, 16, 16, 32
    part, W, m = _attention_part(H, G, D, V, chunk, 16, "float32", seed=3)
    rng = np.random.default_rng(9)
    for target in (chunk, chunk + 1, 2 * chunk - 1):            # first key of the second chunk, its neighbour, its last
        h = bf(rng.standard_normal((3 * chunk, 40)))
        h[target] *= 25.0
        ref = LP.chunk_attention(h, W, "", m, EPS, np.arange(len(h)))[0]
        cuts = ([target] + [1] * (len(h) - target),) if decode else ([],)
        got = run_part(part, part.cache_need(), [h], cuts, "float32", slots=(2,))[0]
        close(got, ref, "float32", f"target {target}")
        inside, outside = np.abs(ref[2 * chunk - 1]).max(), np.abs(ref[2 * chunk]).max()
        assert np.abs(got[2 * chunk - 1] - ref[2 * chunk - 1]).max() < 1e-4 * inside
        assert np.abs(got[2 * chunk] - ref[2 * chunk]).max() < 1e-4 * max(outside, 1.0)
    # the sink
    part, W, m = _attention_part(H, G, D, V, chunk, 16, "float32", seed=3, zero_q=True)
    h = bf(rng.standard_normal((20, 40)))
    ref = LP.chunk_attention(h, W, "", m, EPS, np.arange(20))[0]
    cuts = ([1] * 20,) if decode else ([],)
    got = run_part(part, part.cache_need(), [h], cuts, "float32", slots=(2,))[0]
    close(got, ref, "float32", "sink")
    v0 = np.tile(W["v"] @ h[0] + W["v.b"], H)                  # one kv head: every head reads the same value row
    half = (0.5 * v0 * LP.sigmoid(W["g"] @ h[0])) @ W["o"].T
    assert np.abs(got[0] - half).max() < 1e-5 * max(1.0, np.abs(half).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,I,top,ff,width", [(5, 2, 3, 40, 64), (3, 0, 1, 56, 96), (2, 2, 4, 20, 60), (9, 1, 2, 72, 128)])
def test_routed_experts_part(E, I, top, ff, width, dtype):
    """Choice by score + correction, weights without it and not renormalised, identity experts, and a
    token's result independent of the tokens beside it (the same rows alone and in a larger step)."""
    from gguf2bin_b200.config.specs import PartSpec
    from gguf2bin_b200.parts.feed_forward import RoutedExperts
    rng = np.random.default_rng(E * 7 + top)
    mlp = dict(expert=dict(ff=ff), router=dict(experts=E, identity=I, top=top))
    W = {"mlp.router": rng.standard_normal((E + I, width)) / 3, "mlp.correction": rng.standard_normal(E + I) * 0.5 / (E + I)}
    for e in range(E):
        W[f"mlp.e{e}.gate"] = rng.standard_normal((ff, width)) / 4
        W[f"mlp.e{e}.up"] = rng.standard_normal((ff, width)) / 4
        W[f"mlp.e{e}.down"] = rng.standard_normal((width, ff)) / np.sqrt(ff)
    W = {k: bf(v) for k, v in W.items()}
    spec = PartSpec.make("routed_experts", n_experts=E, n_identity=I, top=top, intermediate_size=ff, correction=True,
                         names=(("router", "mlp.router"), ("correction", "mlp.correction"), ("gate", "mlp.e{}.gate"),
                                ("up", "mlp.e{}.up"), ("down", "mlp.e{}.down")))
    part = RoutedExperts(spec, width, DTYPES[dtype], DEV)
    part.bind({k: dev(v, DTYPES[dtype]) for k, v in W.items()})
    rows = []
    while len(rows) < 77:                                 # rows whose choice is clear (see levolix_helpers.clear_tokens)
        h = bf(rng.standard_normal((1, width)))
        margins = []
        LP.routed_ff(h, W, "mlp.", mlp, margins)
        if not margins or margins[0] > 0.2:
            rows.append(h[0])
    h = np.stack(rows)
    ref = LP.routed_ff(h, W, "mlp.", mlp)
    outs = {}
    for n in (77, 5, 1):
        ctx = step_ctx([n], [0], [0], dtype)
        y = torch.full((n, width), 3.0, dtype=torch.float32, device=DEV)
        part.forward_into(dev(h[:n], DTYPES[dtype]), ctx, y, dev(h[:n]))
        outs[n] = y.cpu().numpy()
        close(outs[n], ref[:n], dtype, f"routed experts, {n} rows")
    # a step of few rows and one of many take different product kernels (rounding apart); within one
    # kind a row's bits do not depend on the rows beside it
    assert np.abs(outs[77][:5] - outs[5]).max() < 1e-5 * max(1.0, np.abs(ref).max())
    if dtype == "float32":
        assert np.array_equal(outs[5][:1], outs[1])
    else:                         # the router's product is a kernel chosen by the step's rows too
        assert np.abs(outs[5][:1] - outs[1]).max() < 1e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_with_an_offset_joins_the_stream(dtype):
    from gguf2bin_b200 import kernels
    rng = np.random.default_rng(2)
    x, y, w = rng.standard_normal((9, 52)), rng.standard_normal((9, 52)) * 3, bf(rng.standard_normal(52) * 0.2)
    xd, h = dev(x), torch.empty((9, 52), dtype=DTYPES[dtype], device=DEV)
    kernels.norm_add(xd, dev(y), dev(1.0 + w), EPS, h)
    ref = x.astype(np.float32) + LP.offset_norm(y.astype(np.float32).astype(np.float64), w, EPS)
    assert np.abs(xd.cpu().numpy() - ref).max() < 1e-5
    assert np.abs(h.float().cpu().numpy() - ref).max() < (1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_over_steps(taps):
    """Rings that hold junk beyond what the sequence wrote, portions down to one token."""
    from gguf2bin_b200 import kernels
    rng = np.random.default_rng(taps)
    C = 37
    w = rng.standard_normal((C, taps))
    x = rng.standard_normal((29, C))
    ref = LP.silu(LP.short_conv(x, w, np.zeros((taps - 1, C)))[0])
    for sizes in ([29], [1] * 29, [2] * 15, [5, 1, 1, 3, 19]):
        ring = torch.full((4, taps, C), 9.0, dtype=torch.float32, device=DEV)
        got, done = [], 0
        for n in sizes:
            n = min(n, 29 - done)
            ctx = step_ctx([n], [done], [2], "float32", single=(n == 1 and done % 2 == 0))
            out = torch.empty((n, C), dtype=torch.float32, device=DEV)
            kernels.short_conv(dev(x[done:done + n]), dev(w.T.copy()), ring, ctx, out)
            got.append(out.cpu().numpy())
            done += n
        assert np.abs(np.concatenate(got) - ref).max() < 1e-5, sizes


# ----------------------------------------------------------------------------
# whole models
# ----------------------------------------------------------------------------
CASES = [(n, d) for n in ("u", "v", "w") for d in ("float32", "bfloat16")]
LENGTHS = {"u": [70, 3, 130, 64, 1], "v": [129, 2, 40, 65], "w": [200, 33, 1, 90]}


@pytest.fixture(scope="module")
def engines():
    from gguf2bin_b200.engine import Engine, Model
    made = {}

    def get(name, dtype, max_tokens=4096):
        key = (name, dtype, max_tokens)
        if key not in made:
            made[key] = Engine(Model.from_folder(model_folder(name), dtype=dtype), max_tokens=max_tokens)
        return made[key]
    return get


def requests_of(name):
    return [list(clear_tokens(name, n, i)) for i, n in enumerate(LENGTHS[name])]


def run_in_portions(eng, toks, sizes):
    from gguf2bin_b200.engine import StepEntry
    seq, got, done = eng.open_sequence(), [], 0
    sizes = list(sizes)
    while done < len(toks):
        n = min(sizes.pop(0) if sizes else len(toks), len(toks) - done)
        got.append(eng.step([StepEntry(seq, toks[done:done + n], range(n))]).cpu().numpy())
        done += n
    eng.close_sequence(seq)
    return np.concatenate(got)


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts(engines, name, dtype):
    eng = engines(name, dtype)
    for i, toks in enumerate(requests_of(name)):
        assert_rows_close(run_in_portions(eng, toks, []), plain_logits(name, toks), dtype, f"levolix {name}/{dtype} request {i} whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_token_by_token_and_portions(engines, name, dtype):
    """The same logits however the prompt is cut: every token alone from the first one on; portions
    of two; mixed portions that end on, before and behind page and chunk borders."""
    eng = engines(name, dtype)
    toks = requests_of(name)[0][:70]
    ref = plain_logits(name, toks)
    whole = run_in_portions(eng, toks, [])
    for what, sizes in [("one by one", [1] * len(toks)), ("twos", [2] * len(toks)), ("mixed", [3, 2, 5, 1, 2, 50, 1, 2, 2]),
                        ("chunk edge", [15, 1, 1, 7, 1, 23, 1]), ("page edge", [63, 1, 1, 2]), ("page", [64, 2, 2])]:
        got = run_in_portions(eng, toks, sizes)
        assert_rows_close(got, ref, dtype, f"levolix {name}/{dtype} {what}")
        if dtype == "float32":       # the cut changes nothing but the order of a few additions
            assert np.abs(got - whole).max() <= 2e-5 * max(1.0, np.abs(ref).max()), what


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_with_reuse(engines, name, dtype):
    """Batches of up to three requests: prompts (all but the last 6 tokens, at least one) in one step,
    then one token each, shorter requests ending earlier; the cache holds one batch, so every batch
    gets the slots, states and pages that the one before gave back."""
    from gguf2bin_b200.engine import StepEntry
    reqs = requests_of(name)
    batches = [reqs[i:i + 3] for i in range(0, len(reqs), 3)] * 2
    need = max(sum(-(-len(t) // 64) * 64 for t in b) for b in batches)
    eng = engines(name, dtype, need)
    for bi, batch in enumerate(batches):
        seqs = [eng.open_sequence() for _ in batch]
        heads = [max(1, len(t) - 6) for t in batch]
        got = [[] for _ in batch]
        out = eng.step([StepEntry(s, t[:h], range(h)) for s, t, h in zip(seqs, batch, heads)]).cpu().numpy()
        o = 0
        for j, h in enumerate(heads):
            got[j].append(out[o:o + h])
            o += h
        done = list(heads)
        live = [j for j in range(len(batch)) if done[j] < len(batch[j])]
        for j in range(len(batch)):
            if j not in live:
                eng.close_sequence(seqs[j])
        while live:
            out = eng.step([StepEntry(seqs[j], [batch[j][done[j]]], [0]) for j in live]).cpu().numpy()
            for r, j in enumerate(live):
                got[j].append(out[r:r + 1])
                done[j] += 1
            for j in [j for j in live if done[j] == len(batch[j])]:
                eng.close_sequence(seqs[j])
            live = [j for j in live if done[j] < len(batch[j])]
        for j, toks in enumerate(batch):
            assert_rows_close(np.concatenate(got[j]), plain_logits(name, toks), dtype,
                         f"levolix {name}/{dtype} batch {bi} request {j}")
    assert eng.cache.table.pages.n_held == 0 and eng.cache.table.slots.n_held == 0


@pytest.mark.parametrize("name,dtype", [("u", "float32"), ("v", "bfloat16"), ("w", "bfloat16")])
def test_long_decoding(engines, name, dtype):
    """A short prompt, then 200 tokens one by one over page and chunk borders, beside a second
    sequence that started elsewhere."""
    from gguf2bin_b200.engine import StepEntry
    eng = engines(name, dtype)
    a, b = list(clear_tokens(name, 230, 70)), list(clear_tokens(name, 261, 71))
    sa, sb = eng.open_sequence(), eng.open_sequence()
    out = eng.step([StepEntry(sa, a[:30], range(30)), StepEntry(sb, b[:61], range(61))]).cpu().numpy()
    ga, gb = [out[:30]], [out[30:]]
    for t in range(200):
        out = eng.step([StepEntry(sa, [a[30 + t]], [0]), StepEntry(sb, [b[61 + t]], [0])]).cpu().numpy()
        ga.append(out[:1])
        gb.append(out[1:])
    eng.close_sequence(sa)
    eng.close_sequence(sb)
    assert_rows_close(np.concatenate(ga), plain_logits(name, a), dtype, f"levolix {name}/{dtype} long decoding a")
    assert_rows_close(np.concatenate(gb), plain_logits(name, b), dtype, f"levolix {name}/{dtype} long decoding b")


def plain_greedy(name, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(plain_logits(name, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["u", "w"])
def test_greedy_generation_through_the_entry_point(name):
    """LLM.generate (scheduler, decode session with its graph) against the plain implementation's
    argmax, several unequal prompts at once."""
    from gguf2bin_b200.api import LLM
    llm = LLM(model_folder(name), dtype="float32", max_tokens=2048)
    prompts = [list(clear_tokens(name, n, 90 + i)) for i, n in enumerate([9, 1, 66, 30])]
    for _ in range(2):                         # the second call finds slots, pages and graphs of the first
        outs = llm.generate(prompts, n=24, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0)
        for p, o in zip(prompts, outs):
            toks = list(p)
            for t in o.tokens:
                row = plain_logits(name, toks)[-1]
                assert row[t] >= row.max() - 2e-5 * max(1.0, np.abs(row).max())
                toks.append(t)
            assert len(o.tokens) == 24
    a = llm.generate(prompts[:2], n=12, seed=5)
    b = llm.generate(prompts[:2], n=12, seed=5)
    assert [o.tokens for o in a] == [o.tokens for o in b]
    assert llm.engine.cache.table.pages.n_held == 0 and llm.engine.cache.table.slots.n_held == 0


def test_the_programs(tmp_path):
    """info and run of the command line, random weights for the design's config.json, and trace replay."""
    folder = model_folder("u")
    exe = [sys.executable, str(ROOT / "bin" / "gguf2bin_b200")]
    out = subprocess.run(exe + ["info", str(folder)], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "Levolix" in out.stdout + out.stderr, out.stderr[-2000:]
    prompt = list(clear_tokens("u", 7, 40))
    out = subprocess.run(exe + ["run", str(folder), "--tokens", ",".join(map(str, prompt)), "-n", "6", "-t", "0",
                                "--repeat-penalty", "1", "--dtype", "float32", "--ignore-eos"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert [int(t) for t in out.stdout.split()] == prompt + plain_greedy("u", prompt, 6)
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CONFIGS["w"]))
    made = tmp_path / "made"
    out = subprocess.run(exe + ["synth", str(made), "--config", str(cfg_file), "--seed", "3", "--dtype", "float32"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    W = LP.read_safetensors(made / "model.safetensors")
    toks = np.random.default_rng(4).integers(0, CONFIGS["w"]["vocab"], 9).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:6], "want": [0, 5]},
                                     {"id": "b", "tokens": toks[:1], "want": [0]}], "end": ["b"]},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[6:7], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[7:8], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": toks[8:], "want": [0]}], "end": ["a"]}]
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(made), "--dtype", "float32",
                           "--out", str(out_dir), "--max-tokens", "64"],
                          input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    assert not (out_dir / "1.f32").exists()
    got = np.concatenate([np.fromfile(out_dir / f"{i}.f32", "<f4").reshape(-1, CONFIGS["w"]["vocab"]) for i in (0, 2, 3)])
    ref = LP.forward(CONFIGS["w"], W, toks)
    assert_close(got, ref[[0, 5, 0, 7, 8]], "float32", "levolix trace replay")
