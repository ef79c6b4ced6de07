"""Senotar on the device against the plain implementation: each mechanism's kernel alone, then
whole models of four small configurations in every way of cutting the work (whole prompts,
token by token, portions down to two tokens, unequal batches, slots and pages used again, long
decoding over page borders), keys that stand out far away and at page borders, and greedy
generation through the library's entry point, its command line and trace replay."""
import json
import subprocess
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from helpers import assert_close
from plain import senotar_plain as SP
from senotar_helpers import CONFIGS, model_folder, plain_logits, random_tokens, to_bf16_values, weights

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def step_ctx(q_lens, pasts, slots, page_table=None):
    """The index tensors of a step, as the engine would pack them."""
    pos = np.concatenate([np.arange(p, p + n) for p, n in zip(pasts, q_lens)])
    seq = np.concatenate([np.full(n, b) for b, n in enumerate(q_lens)])
    starts = np.cumsum([0] + list(q_lens[:-1]))
    meta = np.array([[s, n, p, sl] for s, n, p, sl in zip(starts, q_lens, pasts, slots)])
    from gguf2bin_b200.engine import Workspace
    return SimpleNamespace(tok_pos=i32(pos), tok_seq=i32(seq), seq_slots=i32(slots), seq_meta=i32(meta),
                           page_table=None if page_table is None else i32(page_table), page_size=64,
                           n_tokens=int(sum(q_lens)), n_seqs=len(q_lens), workspace=Workspace(DEV),
                           all_single=False, max_kv_len=int(max(p + n for p, n in zip(pasts, q_lens))))


# ----------------------------------------------------------------------------
# kernels alone
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("cuts", [[9], [1, 1, 1, 1, 1, 1, 1, 1, 1], [2, 2, 4, 1], [3, 6], [6, 3]])
def test_pair_embedding_over_steps(cuts):
    """Two sequences in every step, cut alike; the previous token crosses the steps in the ring."""
    from gguf2bin_b200 import kernels
    rng = np.random.default_rng(0)
    V, H, buckets, mp, mc = 50, 40, 13, 113, 11
    table, pairs = to_bf16_values(rng.standard_normal((V, H))), to_bf16_values(rng.standard_normal((buckets + 1, H)))
    w = 1 + 0.1 * rng.standard_normal(H).astype(np.float32)
    seqs = [rng.integers(0, V, 9).tolist(), rng.integers(0, V, 9).tolist()]
    ring = torch.full((8, 2), -7, dtype=torch.int32, device=DEV)      # never cleared: nothing may rest on zeros
    slots = [5, 2]
    got = [[], []]
    done = 0
    for n in cuts:
        ctx = step_ctx([n, n], [done, done], slots)
        ids = i32(seqs[0][done:done + n] + seqs[1][done:done + n])
        out = torch.empty((2 * n, H), dtype=torch.float32, device=DEV)
        kernels.embed_pair_norm(dev(table, torch.bfloat16), dev(pairs, torch.bfloat16), ids, ctx, ring, dev(w),
                                1e-6, 3.5, buckets, mp, mc, out)
        got[0].append(out[:n].cpu().numpy())
        got[1].append(out[n:].cpu().numpy())
        done += n
    for b in range(2):
        ref = SP.embed(seqs[b], table.astype(np.float64), pairs.astype(np.float64), 3.5, buckets, mp, mc,
                       w.astype(np.float64), 1e-6)
        assert np.abs(np.concatenate(got[b]) - ref).max() < 2e-6


@pytest.mark.parametrize("taps", [1, 2, 3, 4, 7])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_convolution_over_steps(taps, dtype):
    """Portions of every size down to one and two tokens; what lies before a portion comes from
    the ring, what lies before the sequence is zero; a second sequence shares the steps."""
    from gguf2bin_b200 import kernels
    rng = np.random.default_rng(taps)
    H, T = 24, 23
    td = DTYPES[dtype]
    h = [to_bf16_values(rng.standard_normal((T, H))) for _ in range(2)]
    w = rng.standard_normal((H, taps)).astype(np.float32)
    ring = torch.full((6, taps, H), 99.0, dtype=td, device=DEV)       # stale rows of an earlier user
    slots = [4, 1]
    got = [[], []]
    done = 0
    for n in [2, 1, 3, 2, 1, 1, 5, 8]:
        ctx = step_ctx([n, n], [done, done], slots)
        rows = dev(np.concatenate([h[0][done:done + n], h[1][done:done + n]]), td)
        out = torch.empty_like(rows)
        kernels.canon_conv(rows, dev(np.ascontiguousarray(w.T)), ring, ctx, out)
        kernels.latent_keep(None, None, 0.0, None, rows, ring if taps > 1 else None, taps, ctx)
        got[0].append(out[:n].float().cpu().numpy())
        got[1].append(out[n:].float().cpu().numpy())
        done += n
    for b in range(2):
        ref = h[b].astype(np.float64) + SP.causal_conv(h[b].astype(np.float64), w.astype(np.float64))
        err = np.abs(np.concatenate(got[b]) - ref).max()
        assert err < (1e-5 if dtype == "float32" else 0.06), err


def test_activation_gate_and_add():
    from gguf2bin_b200 import kernels
    rng = np.random.default_rng(2)
    T, F, H = 5, 37, 44
    z = np.concatenate([rng.standard_normal((T, F)) * 3, np.zeros((T, 3))], axis=1).astype(np.float32)
    pq = np.array([0.7, -1.3], dtype=np.float32)
    out = torch.empty((T, F), dtype=torch.float32, device=DEV)
    kernels.xielu(dev(z)[:, :F], dev(pq), out)
    ref = SP.xielu(z[:, :F].astype(np.float64), 0.7, -1.3)
    assert (np.abs(out.cpu().numpy() - ref) / np.maximum(1.0, np.abs(ref))).max() < 1e-6
    x, y = rng.standard_normal((T, H)).astype(np.float32), rng.standard_normal((T, H)).astype(np.float32)
    g, b = rng.standard_normal((T, H + 8)).astype(np.float32), rng.standard_normal(H).astype(np.float32)
    w = rng.standard_normal(H).astype(np.float32)
    xd, normed = dev(x), torch.empty((T, H), dtype=torch.float32, device=DEV)
    kernels.gated_add(xd, dev(y), dev(g)[:, 8:], dev(b), dev(w), 1e-5, normed)
    ref = x.astype(np.float64) + y * SP.sigmoid(g[:, 8:].astype(np.float64) + b)
    assert np.abs(xd.cpu().numpy() - ref).max() < 1e-6
    assert np.abs(normed.cpu().numpy() - SP.rms_norm(ref, w.astype(np.float64), 1e-5)).max() < 5e-6


@pytest.mark.parametrize("heads,n,r", [(3, 10, 28), (2, 128, 96), (1, 40, 200)])
@pytest.mark.parametrize("T", [1, 8, 13])
def test_products_per_head(T, heads, n, r):
    from gguf2bin_b200 import kernels
    rng = np.random.default_rng(T)
    w = rng.standard_normal((heads * n, r)).astype(np.float32)
    x = rng.standard_normal((T, heads * n + 5)).astype(np.float32)
    out = torch.empty((T, heads * r), dtype=torch.float32, device=DEV)
    kernels.head_product(dev(x)[:, :heads * n], dev(w), out, heads, False)
    ref = np.einsum("thn,hnr->thr", x[:, :heads * n].reshape(T, heads, n).astype(np.float64),
                    w.reshape(heads, n, r).astype(np.float64)).reshape(T, -1)
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-4
    a, gate = rng.standard_normal((T, heads * r)).astype(np.float32), rng.standard_normal((T, heads)).astype(np.float32)
    out2 = torch.empty((T, heads * n), dtype=torch.float32, device=DEV)
    kernels.head_product(dev(a), dev(w), out2, heads, True, dev(gate))
    ref2 = np.einsum("thr,hnr->thn", a.reshape(T, heads, r).astype(np.float64), w.reshape(heads, n, r).astype(np.float64))
    ref2 = (ref2 * SP.sigmoid(gate.astype(np.float64))[:, :, None]).reshape(T, -1)
    assert np.abs(out2.cpu().numpy() - ref2).max() < 1e-4
    # the same in bfloat16 storage (inputs that bfloat16 holds exactly; the output is rounded once)
    wb, ab, gb = to_bf16_values(w), to_bf16_values(a), to_bf16_values(gate)
    out3 = torch.empty((T, heads * n), dtype=torch.bfloat16, device=DEV)
    kernels.head_product(dev(ab, torch.bfloat16), dev(wb, torch.bfloat16), out3, heads, True, dev(gb, torch.bfloat16))
    ref3 = np.einsum("thr,hnr->thn", ab.reshape(T, heads, r).astype(np.float64), wb.reshape(heads, n, r).astype(np.float64))
    ref3 = (ref3 * SP.sigmoid(gb.astype(np.float64))[:, :, None]).reshape(T, -1)
    assert np.abs(out3.float().cpu().numpy() - ref3).max() <= 0.005 * np.abs(ref3).max() + 1e-3
    xb = to_bf16_values(x[:, :heads * n])
    out4 = torch.empty((T, heads * r), dtype=torch.bfloat16, device=DEV)
    kernels.head_product(dev(xb, torch.bfloat16), dev(wb, torch.bfloat16), out4, heads, False)
    ref4 = np.einsum("thn,hnr->thr", xb.reshape(T, heads, n).astype(np.float64), wb.reshape(heads, n, r).astype(np.float64))
    assert np.abs(out4.float().cpu().numpy() - ref4.reshape(T, -1)).max() <= 0.005 * np.abs(ref4).max() + 1e-3


def _latent_attention_case(rank, heads, length, hot, dtype, decode, wide=False):
    """Latents on scattered pages; every query is made to point at the latent of position ``hot``
    with a score that towers over the rest, so a key that is dropped, doubled or read from the
    wrong row changes the result by orders of magnitude more than rounding does."""
    from gguf2bin_b200 import kernels
    rng = np.random.default_rng(rank + length + hot)
    td = DTYPES[dtype]
    c = to_bf16_values(rng.standard_normal((length, rank)) * 0.5)
    q = to_bf16_values(rng.standard_normal((length, heads, rank)) * 0.3 + c[hot][None, None, :] * 2.0)
    sink = (rng.standard_normal(heads) * 2).astype(np.float32)
    scale = 0.37
    n_pages = -(-length // 64)
    order = rng.permutation(n_pages + 3)[:n_pages]                     # pages out of order, with gaps
    pages = torch.full((n_pages + 3, 1, 1, 64, rank), 50.0, dtype=td, device=DEV)
    for p in range(n_pages):
        rows = c[p * 64:(p + 1) * 64]
        pages[order[p], 0, 0, :len(rows)] = dev(rows, td)
    ref = np.stack([SP.sink_softmax_attention(q[:, h].astype(np.float64), c.astype(np.float64), c.astype(np.float64),
                                              scale, float(sink[h])) for h in range(heads)], axis=1)
    rows = [length - 1] if decode else list(range(length))
    if decode:
        ctx = step_ctx([1], [length - 1], [0], [list(order)])
        ctx.all_single = True
    else:
        ctx = step_ctx([length], [0], [0], [list(order)])
        tiles = [(0, r0, min(128, length - r0), r0) for r0 in range(0, length, 128)]
        tiles.sort(key=lambda t: -(t[3] + t[2]))
        ctx.attn_tiles_wide, ctx.n_attn_tiles_wide = i32(tiles), len(tiles)
        tiles = [(0, r0, min(64, length - r0), r0) for r0 in range(0, length, 64)]
        ctx.attn_tiles, ctx.n_attn_tiles = i32(tiles), len(tiles)
    ctx.kv_len_hint = 0
    qd = dev(q[rows].reshape(len(rows), -1), td)
    out = torch.empty_like(qd)
    gate = None
    if wide:
        # as a mixer hands them over: queries and gates as column ranges of one wider buffer
        g = to_bf16_values(rng.standard_normal((length, heads)) * 2)
        both = torch.full((len(rows), heads * rank + heads + 6), 7.0, dtype=td, device=DEV)
        both[:, :heads * rank] = qd
        both[:, heads * rank:heads * rank + heads] = dev(g[rows], td)
        qd, gate = both[:, :heads * rank], both[:, heads * rank:heads * rank + heads]
        ref = ref * SP.sigmoid(g.astype(np.float64))[:, :, None]
    kernels.attention(qd, out, pages, ctx, heads, 1, rank, 64, 0, scale, sink=dev(sink), planes=1, gate=gate)
    torch.cuda.synchronize()
    err = np.abs(out.float().cpu().numpy().reshape(len(rows), heads, rank) - ref[rows]).max()
    assert err < (2e-5 if dtype == "float32" else 0.02), (err, rank, length, hot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank,heads", [(24, 3), (64, 4), (128, 2), (64, 17)])
def test_attention_over_latents_finds_a_far_key(rank, heads, dtype):
    # page borders (64), the decode kernel's chunk borders (128, 256, 512), the first and the last key, far away
    for length, hot in [(200, 0), (200, 63), (200, 64), (321, 127), (321, 128), (321, 319), (65, 64), (700, 5),
                        (700, 255), (700, 256), (700, 511), (700, 512), (513, 512), (1, 0), (2, 0)]:
        _latent_attention_case(rank, heads, length, hot, dtype, decode=False)
        _latent_attention_case(rank, heads, length, hot, dtype, decode=True)
    for length, hot in [(321, 128), (200, 0), (700, 512)]:       # queries with a row stride, and the heads' gate
        _latent_attention_case(rank, heads, length, hot, dtype, decode=False, wide=True)
        _latent_attention_case(rank, heads, length, hot, dtype, decode=True, wide=True)


# ----------------------------------------------------------------------------
# whole models
# ----------------------------------------------------------------------------
CASES = [(n, d) for n in CONFIGS for d in ("float32", "bfloat16")]
LENGTHS = {"p": [70, 3, 130, 64, 1], "q": [129, 2, 40, 65], "r": [200, 33, 1, 128, 90], "s": [20, 65, 7],
           "t": [150, 64, 9, 1]}


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
    return [random_tokens(name, n, i) for i, n in enumerate(LENGTHS[name])]


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
        assert_close(run_in_portions(eng, toks, []), plain_logits(name, toks), dtype, f"senotar {name}/{dtype} request {i} whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_token_by_token_and_portions(engines, name, dtype):
    """The same logits however the prompt is cut: every token alone from the first one on;
    portions of two; mixed portions that end on, before and behind page borders."""
    eng = engines(name, dtype)
    toks = requests_of(name)[0][:70]
    ref = plain_logits(name, toks)
    whole = run_in_portions(eng, toks, [])
    for what, sizes in [("one by one", [1] * len(toks)), ("twos", [2] * len(toks)),
                        ("mixed", [3, 2, 5, 1, 2, 50, 1, 2, 2]), ("page edge", [63, 1, 1, 2]), ("page", [64, 2, 2])]:
        got = run_in_portions(eng, toks, sizes)
        assert_close(got, ref, dtype, f"senotar {name}/{dtype} {what}")
        if dtype == "float32":       # the cut changes nothing but the order of a few additions
            assert np.abs(got - whole).max() <= 2e-5 * max(1.0, np.abs(ref).max()), what


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_with_reuse(engines, name, dtype):
    """Batches of up to three requests: prompts (all but the last 6 tokens, at least one) in one
    step, then one token each, shorter requests ending earlier; the cache holds one batch, so
    every batch gets the slots and pages that the one before gave back, rings uncleared by luck."""
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
            assert_close(np.concatenate(got[j]), plain_logits(name, toks), dtype,
                         f"senotar {name}/{dtype} batch {bi} request {j}")
    assert eng.cache.table.pages.n_held == 0 and eng.cache.table.slots.n_held == 0


def test_up_projections_folded_where_the_rank_allows(engines):
    from gguf2bin_b200.parts.latent import folds
    mixers = [b.mixer for b in engines("t", "bfloat16").model.blocks]
    assert [(m.fold_k, m.fold_v) for m in mixers] == [(True, True), (True, True), (True, True)]
    assert mixers[2].w_uk is None and mixers[2].w_uv is None
    assert mixers[1].w_in.shape[0] == -(-(2 * 64 + 2) // 8) * 8        # queries in latent coordinates, then the gates
    assert not any(b.mixer.fold_k or b.mixer.fold_v for b in engines("t", "float32").model.blocks)
    # rank 64 over heads of 8 numbers: never folded; over heads of 40: folded while the model is small
    q = [b.mixer for b in engines("q", "bfloat16").model.blocks]
    assert (q[1].fold_k, q[1].fold_v) == (False, True) and (q[3].fold_k, q[3].fold_v) == (False, False)
    assert not any(b.mixer.fold_k or b.mixer.fold_v for b in engines("r", "bfloat16").model.blocks)
    assert folds(128, 128, 32, 4096) and folds(192, 128, 32, 4096) and not folds(512, 128, 32, 4096)
    assert folds(128, 64, 16, 1024) and not folds(512, 64, 16, 1024) and not folds(256, 128, 32, 4096)


@pytest.mark.parametrize("name,dtype", [("p", "float32"), ("r", "bfloat16"), ("q", "bfloat16"), ("t", "bfloat16")])
def test_long_decoding(engines, name, dtype):
    """A short prompt, then 200 tokens one by one over three page borders, beside a second
    sequence that started elsewhere."""
    from gguf2bin_b200.engine import StepEntry
    eng = engines(name, dtype)
    a, b = random_tokens(name, 230, 70), random_tokens(name, 261, 71)
    sa, sb = eng.open_sequence(), eng.open_sequence()
    out = eng.step([StepEntry(sa, a[:30], range(30)), StepEntry(sb, b[:61], range(61))]).cpu().numpy()
    ga, gb = [out[:30]], [out[30:]]
    for t in range(200):
        out = eng.step([StepEntry(sa, [a[30 + t]], [0]), StepEntry(sb, [b[61 + t]], [0])]).cpu().numpy()
        ga.append(out[:1])
        gb.append(out[1:])
    eng.close_sequence(sa)
    eng.close_sequence(sb)
    assert_close(np.concatenate(ga), plain_logits(name, a), dtype, f"senotar {name}/{dtype} long decoding a")
    assert_close(np.concatenate(gb), plain_logits(name, b), dtype, f"senotar {name}/{dtype} long decoding b")


def plain_greedy(name, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(plain_logits(name, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["p", "r"])
def test_greedy_generation_through_the_entry_point(name):
    """LLM.generate (scheduler, decode session with its graph and the step launched ahead)
    against the plain implementation's argmax, several unequal prompts at once."""
    from gguf2bin_b200.api import LLM
    llm = LLM(model_folder(name), dtype="float32", max_tokens=2048)
    prompts = [random_tokens(name, n, 90 + i) for i, n in enumerate([9, 1, 66, 30])]
    for _ in range(2):                         # the second call finds slots, pages and graphs of the first
        outs = llm.generate(prompts, n=24, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0)
        for p, o in zip(prompts, outs):
            toks = list(p)
            for t in o.tokens:
                row = plain_logits(name, toks)[-1]
                assert row[t] >= row.max() - 2e-5 * max(1.0, np.abs(row).max())
                toks.append(t)
            assert len(o.tokens) == 24
    # sampled generation runs too, and a seed repeats it
    a = llm.generate(prompts[:2], n=12, seed=5)
    b = llm.generate(prompts[:2], n=12, seed=5)
    assert [o.tokens for o in a] == [o.tokens for o in b]
    assert llm.engine.cache.table.pages.n_held == 0 and llm.engine.cache.table.slots.n_held == 0


def test_the_programs(tmp_path):
    """info and run of the command line, random weights for the design's config.json, and trace replay."""
    folder = model_folder("q")
    exe = [sys.executable, str(ROOT / "bin" / "gguf2bin_b200")]
    out = subprocess.run(exe + ["info", str(folder)], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "Senotar" in out.stdout + out.stderr, out.stderr[-2000:]
    prompt = random_tokens("q", 7, 40)
    out = subprocess.run(exe + ["run", str(folder), "--tokens", ",".join(map(str, prompt)), "-n", "6", "-t", "0",
                                "--repeat-penalty", "1", "--dtype", "float32", "--ignore-eos"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert [int(t) for t in out.stdout.split()] == prompt + plain_greedy("q", prompt, 6)
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CONFIGS["s"]))
    made = tmp_path / "made"
    out = subprocess.run(exe + ["synth", str(made), "--config", str(cfg_file), "--seed", "3"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    cfg, W = SP.read_model_folder(made)
    toks = random_tokens("s", 9, 41)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:6], "want": [0, 5]},
                                     {"id": "b", "tokens": toks[:1], "want": [0]}], "end": ["b"]},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[6:7], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[7:8], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": toks[8:], "want": [0]}], "end": ["a"]}]
    for dtype in ("float32", "bfloat16"):
        out_dir = tmp_path / f"out_{dtype}"
        proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(made), "--dtype", dtype,
                               "--out", str(out_dir), "--max-tokens", "64"],
                              input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True,
                              timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
        assert not (out_dir / "1.f32").exists()
        got = np.concatenate([np.fromfile(out_dir / f"{i}.f32", "<f4").reshape(-1, cfg["vocab"]) for i in (0, 2, 3)])
        ref = SP.forward(cfg, W, toks)
        assert_close(got, ref[[0, 5, 0, 7, 8]], dtype, f"senotar trace replay {dtype}")
