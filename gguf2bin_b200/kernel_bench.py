"""Per-kernel micro-benchmarks at model geometry, in the manner of the reference's
tools/mmbench.c (which times its GEMV at the lm_head's size and prints GB/s): every hot
kernel alone, at the sizes of a decode step or of a prompt step, with its achieved
bandwidth or FLOP/s.

    python -m gguf2bin_b200.kernel_bench decode  [--batch 8] [--ctx 3072] [--only NAME] [--layers 28]
    python -m gguf2bin_b200.kernel_bench prefill [--tokens 2048] [--only NAME] [--layers 4]
    python -m gguf2bin_b200.kernel_bench latent-decode | latent-prefill  [--rank 128] ...
    python -m gguf2bin_b200.kernel_bench state-decode | state-prefill  [--experts 16] [--top 4] [--chunk 512] ...

The ``latent-*`` modes time the kernels of a gated layer with latent attention (``--heads`` heads of
``--head-dim`` key and value numbers, ``--rank`` cached numbers per token) at the same geometry.

The ``state-*`` modes time the kernels of layers that keep a matrix state per head (``--heads`` / 2 heads with
keys of ``--head-dim`` and values of twice that), of attention in chunks of ``--chunk`` keys with the wide
prologue, and of a routed feed-forward (``--experts`` experts of ``--inter`` / 4 each, ``--top`` choices).

Sizes default to Qwen3-0.6B (width 1024, 16/8 heads of 128, feed-forward 3072, vocabulary
151936); --hidden/--inter/--heads/--kv-heads/--vocab change them.  Decode kernels run
over `--layers` distinct weight sets, so weights stream from HBM as in a real step, and
are replayed from a CUDA graph; times are CUDA-event times per kernel launch.
`--only NAME --once` launches the named kernel a few times without graph or timing loop,
which is what a profiler capture wants.
"""
from __future__ import annotations

import argparse
import math
import sys
from types import SimpleNamespace

import torch

from . import kernels, kernels_bf16
from .engine.workspace import Workspace

DEV = "cuda:0"


def bf(*shape):
    return (torch.randn(*shape, device=DEV) * 0.02).to(torch.bfloat16)


class Bench:
    def __init__(self, a):
        self.a = a
        self.rows = []

    def want(self, name: str) -> bool:
        return self.a.only is None or self.a.only == name

    def run(self, name, fn, n_inner, nbytes=None, flops=None, graph=True):
        """Times `fn` (which launches the kernel n_inner times)."""
        if not self.want(name):
            return
        if self.a.once:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            print(f"{name}: launched 3 x {n_inner}")
            return
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        replay = fn
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            replay = g.replay
        replay()
        torch.cuda.synchronize()
        reps = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps / n_inner
        extra = ""
        if nbytes:
            extra += f"  {nbytes / us / 1e3:7.0f} GB/s"
        if flops:
            extra += f"  {flops / us / 1e6:7.0f} TFLOP/s"
        print(f"{name:28s} {us:9.2f} us{extra}")


def decode(a) -> None:
    B, L, H, I = a.batch, a.layers, a.hidden, a.inter
    nh, nkv, hd, V = a.heads, a.kv_heads, a.head_dim, a.vocab
    NQ, NK = nh * hd, nkv * hd
    b = Bench(a)
    x32 = torch.randn(B, H, device=DEV)
    nw = torch.ones(H, device=DEV)
    h, o, mid = bf(B, H), bf(B, NQ), bf(B, I)
    qkv = torch.empty(B, NQ + 2 * NK, dtype=torch.bfloat16, device=DEV)
    res = torch.zeros(B, H, device=DEV)
    hb = torch.empty(B, H, dtype=torch.bfloat16, device=DEV)
    b.run("rmsnorm", lambda: [kernels.rmsnorm(x32, nw, 1e-6, hb) for _ in range(L)], L)
    if b.want("qkv"):
        W = [bf(NQ + 2 * NK, H) for _ in range(L)]
        b.run("qkv", lambda: [kernels_bf16.linear_bf16(h, w, qkv, False) for w in W], L, W[0].numel() * 2)
    if b.want("qkv_normed"):              # what a decode step of up to 16 rows runs: the norm inside the product
        W = [bf(NQ + 2 * NK, H) for _ in range(L)]
        if kernels.normed_product(x32, 1e-6, W[0], qkv):
            b.run("qkv_normed", lambda: [kernels.normed_product(x32, 1e-6, w, qkv) for w in W], L, W[0].numel() * 2)
    if b.want("gate_up_normed"):
        W = [bf(2 * I, H) for _ in range(L)]
        if kernels.normed_product(x32, 1e-6, W[0], mid, 8):
            b.run("gate_up_normed", lambda: [kernels.normed_product(x32, 1e-6, w, mid, 8) for w in W], L,
                  W[0].numel() * 2)
    if b.want("o_proj"):
        W = [bf(H, NQ) for _ in range(L)]
        b.run("o_proj", lambda: [kernels_bf16.linear_bf16(o, w, res, True) for w in W], L, W[0].numel() * 2)
    if b.want("gate_up"):
        W = [bf(2 * I, H) for _ in range(L)]
        b.run("gate_up", lambda: [kernels_bf16.gate_up_bf16(h, w, mid, 8) for w in W], L, W[0].numel() * 2)
    if b.want("down"):
        W = [bf(H, I) for _ in range(L)]
        b.run("down", lambda: [kernels_bf16.linear_bf16(mid, w, res, True) for w in W], L, W[0].numel() * 2)
    if b.want("lm_head") or b.want("greedy") or b.want("temperature") or b.want("default_sampling"):
        from .cache import SEQ_STATE_WORDS
        Wh = bf(V, H)
        logits = torch.empty(B, V, device=DEV)
        ids = torch.empty(B, dtype=torch.int32, device=DEV)
        state = torch.zeros(B, SEQ_STATE_WORDS, dtype=torch.int32, device=DEV)
        slots = torch.arange(B, dtype=torch.int32, device=DEV)
        kernels.seed_slots(state, slots, slots.clone(), 1)
        b.run("lm_head", lambda: kernels_bf16.linear_bf16(h, Wh, logits, False), 1, Wh.numel() * 2)
        b.run("greedy", lambda: kernels.sample_rows(logits, 0.0, None, None, ids), 1, logits.numel() * 4)
        logits.copy_(torch.randn(B, V, device=DEV) * 2.5)
        b.run("temperature", lambda: kernels.sample_rows(logits, 0.7, state, slots, ids), 1, logits.numel() * 4)
        # temperature 0.7, top-k 40, top-p 0.9, repeat penalty 1.1 over the ids in the sequences' records
        b.run("default_sampling", lambda: kernels.sample_filtered(logits, 0.7, 40, 0.9, 1.1, None, None, state, slots,
                                                                  ids, append=True), 1, logits.numel() * 4)
    ps, ctx_len = 64, a.ctx
    pages_per = -(-(ctx_len + 1) // ps)
    if b.want("attn_decode") or b.want("qknorm_rope_cache"):
        caches = [torch.randn(B * pages_per, 2, nkv, ps, hd, device=DEV).to(torch.bfloat16) for _ in range(L)]
        table = torch.arange(B * pages_per, dtype=torch.int32, device=DEV).view(B, pages_per)
        ctx = SimpleNamespace(tok_pos=torch.full((B,), ctx_len, dtype=torch.int32, device=DEV),
                              tok_seq=torch.arange(B, dtype=torch.int32, device=DEV), page_table=table,
                              max_kv_len=pages_per * ps, workspace=Workspace(DEV), all_single=True)
        q = bf(B, NQ)
        out = torch.empty_like(q)
        b.run("attn_decode", lambda: [kernels_bf16.attn_decode(q, out, c, ctx, nh, nkv, hd, ps, 0, 1 / math.sqrt(hd))
                                      for c in caches], L, B * (ctx_len + 1) * 2 * nkv * hd * 2)
        qw = torch.ones(hd, device=DEV)
        inv = torch.ones(hd // 2, device=DEV)
        rope = torch.empty(B, hd // 2, 2, device=DEV)
        kernels.rope_table(ctx.tok_pos, inv, rope)
        qkvb = bf(B, NQ + 2 * NK)
        b.run("qknorm_rope_cache", lambda: [kernels.qknorm_rope_cache(
            qkvb, nh, nkv, hd, qw, qw, 1e-6, rope, hd, ctx.tok_pos, ctx.tok_seq, table, c, ps, q) for c in caches], L)


def prefill(a) -> None:
    T, L, H, I = a.tokens, a.layers, a.hidden, a.inter
    nh, nkv, hd = a.heads, a.kv_heads, a.head_dim
    NQ, NK = nh * hd, nkv * hd
    b = Bench(a)
    x32 = torch.randn(T, H, device=DEV)
    nw = torch.ones(H, device=DEV)
    h, o, mid = bf(T, H), bf(T, NQ), bf(T, I)
    qkv = torch.empty(T, NQ + 2 * NK, dtype=torch.bfloat16, device=DEV)
    res = torch.zeros(T, H, device=DEV)
    hb = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    if b.want("qkv"):
        W = [bf(NQ + 2 * NK, H) for _ in range(L)]
        b.run("qkv", lambda: [kernels_bf16.linear_bf16(h, w, qkv, False) for w in W], L,
              flops=2 * T * (NQ + 2 * NK) * H)
    if b.want("o_proj"):
        W = [bf(H, NQ) for _ in range(L)]
        b.run("o_proj", lambda: [kernels_bf16.linear_bf16(o, w, res, True) for w in W], L,
              flops=2 * T * H * NQ)
    if b.want("gate_up"):
        W = [bf(2 * I, H) for _ in range(L)]
        b.run("gate_up", lambda: [kernels_bf16.gate_up_bf16(h, w, mid, 8) for w in W], L,
              flops=2 * T * 2 * I * H)
    if b.want("down"):
        W = [bf(H, I) for _ in range(L)]
        b.run("down", lambda: [kernels_bf16.linear_bf16(mid, w, res, True) for w in W], L,
              flops=2 * T * H * I)
    b.run("rmsnorm", lambda: [kernels.rmsnorm(x32, nw, 1e-6, hb) for _ in range(L)], L,
          nbytes=T * H * 6)
    ps = 64
    pages = -(-T // ps)
    if b.want("attn_prefill") or b.want("attn_prefill_tc") or b.want("qknorm_rope_cache"):
        caches = [torch.randn(pages, 2, nkv, ps, hd, device=DEV).to(torch.bfloat16) for _ in range(L)]
        table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages)
        tok_pos = torch.arange(T, dtype=torch.int32, device=DEV)
        tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
        qw = torch.ones(hd, device=DEV)
        inv = (1e6 ** (-2 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().to(DEV)
        q = bf(T, NQ)
        out = torch.empty_like(q)
        rope = torch.empty(T, hd // 2, 2, device=DEV)
        kernels.rope_table(tok_pos, inv, rope)
        b.run("qknorm_rope_cache", lambda: [kernels.qknorm_rope_cache(
            qkv, nh, nkv, hd, qw, qw, 1e-6, rope, hd, tok_pos, tok_seq, table, c, ps, q) for c in caches], L,
            nbytes=T * (NQ + 2 * NK) * 4)
        tiles = sorted([(0, r, min(64, T - r), r) for r in range(0, T, 64)], key=lambda t: -t[3])
        ctx = SimpleNamespace(page_table=table, all_single=False, n_attn_tiles=len(tiles),
                              attn_tiles=torch.tensor(tiles, dtype=torch.int32, device=DEV))
        b.run("attn_prefill", lambda: [kernels_bf16.attn_prefill(q, out, c, ctx, nh, nkv, hd, ps, 0, 1 / math.sqrt(hd))
                                       for c in caches], L, flops=4 * NQ * T * (T + 1) / 2)
        wide = sorted([(0, r, min(128, T - r), r) for r in range(0, T, 128)], key=lambda t: -t[3])
        ctx2 = SimpleNamespace(page_table=table, all_single=False, n_attn_tiles_wide=len(wide),
                               attn_tiles_wide=torch.tensor(wide, dtype=torch.int32, device=DEV))
        b.run("attn_prefill_tc", lambda: [kernels_bf16.attn_prefill_tc(
            q, out, c, ctx2, nh, nkv, hd, ps, 0, 1 / math.sqrt(hd)) for c in caches], L,
            flops=4 * NQ * T * (T + 1) / 2)
    kernels_bf16.check_status()


def latent(a, single: bool) -> None:
    """The kernels of a gated pre-norm layer with latent attention: ``single``: a decode step of
    ``--batch`` sequences behind ``--ctx`` tokens; else one prompt of ``--tokens`` tokens."""
    L, H, I, nh, dk, r = a.layers, a.hidden, a.inter, a.heads, a.head_dim, a.rank
    B = a.batch if single else 1
    n = 1 if single else a.tokens
    T = B * n
    past = a.ctx if single else 0
    b = Bench(a)
    ps = 64
    pages_per = -(-(past + n) // ps)
    table = torch.arange(B * pages_per, dtype=torch.int32, device=DEV).view(B, pages_per)
    pos = (torch.arange(n, dtype=torch.int32, device=DEV) + past).repeat(B)
    seq = torch.arange(B, dtype=torch.int32, device=DEV).repeat_interleave(n)
    wide = sorted([(s, s * n + r0, min(128, n - r0), past + r0) for s in range(B) for r0 in range(0, n, 128)],
                  key=lambda t: -(t[3] + t[2]))
    ctx = SimpleNamespace(tok_pos=pos, tok_seq=seq, page_table=table, page_size=ps, n_tokens=T, n_seqs=B,
                          seq_slots=torch.arange(B, dtype=torch.int32, device=DEV), seq_meta=None if single else
                          torch.tensor([[0, n, 0, 0]], dtype=torch.int32, device=DEV),
                          max_kv_len=pages_per * ps, kv_len_hint=past + n, workspace=Workspace(DEV), all_single=single,
                          attn_tiles_wide=torch.tensor(wide, dtype=torch.int32, device=DEV), n_attn_tiles_wide=len(wide),
                          attn_tiles=None, n_attn_tiles=0)
    n_in = -(-(nh * dk + r + nh) // 8) * 8
    h, u = bf(T, H), bf(T, H)
    x32, y32 = torch.randn(T, H, device=DEV), torch.randn(T, H, device=DEV)
    nw, bias = torch.ones(H, device=DEV), torch.zeros(H, device=DEV)
    proj = torch.empty(T, n_in, dtype=torch.bfloat16, device=DEV)
    gate = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    mm = (lambda N, K: dict(nbytes=N * K * 2)) if single else (lambda N, K: dict(flops=2 * T * N * K))
    hb = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    b.run("rmsnorm", lambda: [kernels.rmsnorm(x32, nw, 1e-6, hb) for _ in range(L)], L, nbytes=T * H * 6)
    ring = torch.zeros(B + 1, 3, H, dtype=torch.bfloat16, device=DEV)
    cw = torch.randn(3, H, device=DEV)
    b.run("canon_conv", lambda: [kernels.canon_conv(h, cw, ring, ctx, u) for _ in range(L)], L, nbytes=T * H * 4)
    if b.want("in_proj"):
        W = [bf(n_in, H) for _ in range(L)]
        b.run("in_proj", lambda: [kernels_bf16.linear_bf16(u, w, proj, False) for w in W], L, **mm(n_in, H))
    if b.want("gate_proj"):
        W = [bf(H, H) for _ in range(L)]
        b.run("gate_proj", lambda: [kernels_bf16.linear_bf16(h, w, gate, False) for w in W], L, **mm(H, H))
    caches = [torch.randn(B * pages_per + 1, 1, 1, ps, r, device=DEV).to(torch.bfloat16) for _ in range(L)]
    cn = torch.ones(r, device=DEV)
    d = proj[:, nh * dk:nh * dk + r]
    b.run("latent_keep", lambda: [kernels.latent_keep(d, cn, 1e-6, c, h, ring, 3, ctx) for c in caches], L,
          nbytes=T * r * 4)
    uk, uv = [bf(nh * dk, r) for _ in range(L)], [bf(nh * dk, r) for _ in range(L)]
    qa, mix = bf(T, nh * r), bf(T, nh * r)
    o = torch.empty(T, nh * dk, dtype=torch.bfloat16, device=DEV)
    q = proj[:, :nh * dk]
    g = proj[:, nh * dk + r:nh * dk + r + nh]
    hp = dict(nbytes=nh * dk * r * 2) if single else dict(flops=2 * T * nh * dk * r)
    if single:
        b.run("head_absorb", lambda: [kernels.head_product(q, w, qa, nh, False) for w in uk], L, **hp)
        b.run("head_expand", lambda: [kernels.head_product(mix, w, o, nh, True, g) for w in uv], L, **hp)
    else:
        from .parts.latent import LatentAttention
        from .config.specs import PartSpec
        spec = PartSpec.make("latent_attention", n_heads=nh, qk_dim=dk, v_dim=dk, kv_rank=r, scale=dk ** -0.5, eps=1e-6,
                             names=())
        m = LatentAttention(spec, H, torch.bfloat16, DEV)
        m.w_uk, m.w_uv = uk[0], uv[0]
        b.run("head_absorb", lambda: [m._per_head(q, m.w_uk, qa, False, None) for _ in range(L)], L, **hp)
        b.run("head_expand", lambda: [m._per_head(mix, m.w_uv, o, True, g) for _ in range(L)], L, **hp)
    b.run("head_gate", lambda: [kernels.head_gate(mix, g, nh) for _ in range(L)], L, nbytes=T * nh * r * 4)
    sink = torch.zeros(nh, device=DEV)
    if single:
        b.run("attn_latent", lambda: [kernels.attention(qa, mix, c, ctx, nh, 1, r, ps, 0, 0.1, sink=sink, planes=1)
                                      for c in caches], L, nbytes=B * (past + 1) * r * 2)
    else:
        b.run("attn_latent", lambda: [kernels.attention(qa, mix, c, ctx, nh, 1, r, ps, 0, 0.1, sink=sink, planes=1)
                                      for c in caches], L, flops=4 * nh * r * n * (n + 1) / 2)
    if b.want("o_proj"):
        W = [bf(H, nh * dk) for _ in range(L)]
        b.run("o_proj", lambda: [kernels_bf16.linear_bf16(o, w, y32, False) for w in W], L, **mm(H, nh * dk))
    b.run("gated_add_norm", lambda: [kernels.gated_add(x32, y32, gate, bias, nw, 1e-6, hb) for _ in range(L)], L,
          nbytes=T * H * 16)
    if b.want("up_and_gate"):
        n_up = I + H
        W = [bf(n_up, H) for _ in range(L)]
        up = torch.empty(T, n_up, dtype=torch.bfloat16, device=DEV)
        b.run("up_and_gate", lambda: [kernels_bf16.linear_bf16(h, w, up, False) for w in W], L, **mm(n_up, H))
        mid = torch.empty(T, I, dtype=torch.bfloat16, device=DEV)
        pq = torch.zeros(2, device=DEV)
        b.run("xielu", lambda: [kernels.xielu(up[:, :I], pq, mid) for _ in range(L)], L, nbytes=T * I * 4)
        W2 = [bf(H, I) for _ in range(L)]
        b.run("down", lambda: [kernels_bf16.linear_bf16(mid, w, y32, False) for w in W2], L, **mm(H, I))
    kernels_bf16.check_status()


def state(a, single: bool) -> None:
    """The kernels of state mixers, chunked attention and routed experts: ``single``: a decode step of
    ``--batch`` sequences behind ``--ctx`` tokens; else one prompt of ``--tokens`` tokens."""
    from .engine.workspace import Workspace as WS
    from .parts.base import StepContext
    Lw, W = a.layers, a.hidden
    H, D, V = max(1, a.heads // 2), a.head_dim, 2 * a.head_dim          # state heads
    nh, nkv, hd = a.heads, a.kv_heads, a.head_dim                      # attention heads
    E, top, ff = a.experts, a.top, max(8, a.inter // 4)
    B = a.batch if single else 1
    n = 1 if single else a.tokens
    T, past = B * n, (a.ctx if single else 0)
    b = Bench(a)
    ps = 64
    pages_per = -(-(past + n) // ps)
    table = torch.arange(B * pages_per, dtype=torch.int32, device=DEV).view(B, pages_per)
    pos = (torch.arange(n, dtype=torch.int32, device=DEV) + past).repeat(B)
    seq = torch.arange(B, dtype=torch.int32, device=DEV).repeat_interleave(n)
    wide = sorted([(s, s * n + r0, min(128, n - r0), past + r0) for s in range(B) for r0 in range(0, n, 128)],
                  key=lambda t: -(t[3] + t[2]))
    meta = torch.tensor([[s * n, n, past, s] for s in range(B)], dtype=torch.int32, device=DEV)
    ctx = StepContext(n_tokens=T, n_seqs=B, tok_ids=pos, tok_pos=pos, tok_seq=seq, page_table=table, page_size=ps,
                      workspace=WS(DEV), dtype=torch.bfloat16, q_lens=[n] * B, past_lens=[past] * B, slots=list(range(B)),
                      max_kv_len=pages_per * ps, kv_len_hint=past + n, seq_meta=None if single else meta,
                      seq_slots=torch.arange(B, dtype=torch.int32, device=DEV),
                      attn_tiles_wide=torch.tensor(wide, dtype=torch.int32, device=DEV), n_attn_tiles_wide=len(wide))
    f32 = lambda *shape: torch.randn(*shape, device=DEV)
    # ---- the scans -------------------------------------------------------------------------------
    q, k, v = bf(T, H * D) * 50, bf(T, H * D) * 50, bf(T, H * V) * 50
    states = [torch.zeros(B + 1, H, V, D, device=DEV) for _ in range(Lw)]
    o32 = torch.empty(T, H * V, device=DEV)
    decay = torch.full((H,), 0.99, device=DEV)
    ab, a_log, dtb = f32(T, 2 * H), torch.zeros(H, device=DEV), torch.zeros(H, device=DEV)
    inv = torch.tensor([1e4 ** (-2.0 * j / D) for j in range(D // 2)], device=DEV)
    rope = ctx.rope_table(inv)
    state_bytes = 2 * 4 * B * H * V * D + T * (2 * H * D + H * V) * 2 + T * H * V * 4
    scan_flops = 6.0 * T * H * D * V
    b.run("scan_decay", lambda: [kernels.state_scan(q, k, v, st, ctx, o32, H, H, D, V, decay=decay, rope=rope, rotary_dim=D,
                                                    k_scale=D ** -0.5) for st in states], Lw, nbytes=state_bytes, flops=scan_flops)
    b.run("scan_delta", lambda: [kernels.state_scan(q, k, v, st, ctx, o32, H, H, D, V, ab=ab, a_log=a_log, dt_bias=dtb,
                                                    q_scale=D ** -0.5, unit_eps=1e-6) for st in states], Lw,
          nbytes=state_bytes, flops=scan_flops)
    gate, og = bf(T, H * V), torch.empty(T, H * V, dtype=torch.bfloat16, device=DEV)
    b.run("head_norm_gate", lambda: kernels.head_norm_gate(o32, H, V, None, 1e-6, gate, 1.0, og), 1, nbytes=T * H * V * 8)
    C = 2 * H * D + H * V
    x, y = bf(T, C), torch.empty(T, C, dtype=torch.bfloat16, device=DEV)
    ring, wc = torch.zeros(B + 1, 4, C, dtype=torch.bfloat16, device=DEV), f32(4, C)
    b.run("short_conv", lambda: kernels.short_conv(x, wc, ring, ctx, y), 1, nbytes=T * C * 4)
    x32, y32, nw = f32(T, W), f32(T, W), torch.ones(W, device=DEV)
    hcast = torch.empty(T, W, dtype=torch.bfloat16, device=DEV)
    b.run("norm_add", lambda: kernels.norm_add(x32, y32, nw, 1e-6, hcast), 1, nbytes=T * W * 14)
    # ---- chunked attention with the wide prologue ----------------------------------------------------
    nq, nk = nh * hd, nkv * hd
    qkv, bias = bf(T, nq + 2 * nk + nq), f32(nq + 2 * nk)
    qw, kw = torch.ones(nq, device=DEV), torch.ones(nk, device=DEV)
    pages = torch.zeros(B * pages_per + 1, 2, nkv, ps, hd, dtype=torch.bfloat16, device=DEV)
    qo, ao = torch.empty(T, nq, dtype=torch.bfloat16, device=DEV), torch.empty(T, nq, dtype=torch.bfloat16, device=DEV)
    sink = torch.zeros(nh, device=DEV)
    b.run("proj_norm_rope_cache", lambda: kernels.proj_norm_rope_cache(qkv, bias, nh, nkv, hd, hd, qw, kw, 1e-6, rope, hd,
                                                                       True, ctx, pages, ps, qo), 1,
          nbytes=T * (nq + 2 * nk) * 4)
    seen = min(a.chunk, past + n)
    b.run("attention_chunked", lambda: kernels.attention(qo, ao, pages, ctx, nh, nkv, hd, ps, 0, hd ** -0.5, sink=sink,
                                                         chunk=a.chunk), 1,
          nbytes=B * 2 * nk * 2 * ((past + n - 1) % a.chunk + 1) if single else None,
          flops=None if single else 4.0 * nq * sum(min(t % a.chunk, t) + 1 for t in range(n)))
    # ---- routed experts -------------------------------------------------------------------------------
    from .config.specs import PartSpec
    from .parts.feed_forward import RoutedExperts
    spec = PartSpec.make("routed_experts", n_experts=E, n_identity=0, top=top, intermediate_size=ff, correction=False,
                         names=(("router", "r"), ("gate", "e{}.g"), ("up", "e{}.u"), ("down", "e{}.d")))
    parts = []
    for _ in range(min(Lw, 4)):
        part = RoutedExperts(spec, W, torch.bfloat16, DEV)
        t = {"r": bf(E, W)}
        for e in range(E):
            t[f"e{e}.g"], t[f"e{e}.u"], t[f"e{e}.d"] = bf(ff, W), bf(ff, W), bf(W, ff)
        part.bind(t)
        parts.append(part)
    h = bf(T, W) * 50
    out32 = torch.empty(T, W, device=DEV)
    touched = min(E, T * top)
    b.run("routed_experts (route, plan, products, sum)", lambda: [p.forward_into(h, ctx, out32, x32) for p in parts], len(parts),
          nbytes=3 * touched * ff * W * 2 if single else None, flops=None if single else 6.0 * T * top * ff * W)
    kernels_bf16.check_status()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("mode", choices=["decode", "prefill", "latent-decode", "latent-prefill", "state-decode", "state-prefill"])
    ap.add_argument("--experts", type=int, default=16, help="state modes: experts of the routed feed-forward")
    ap.add_argument("--top", type=int, default=4, help="state modes: experts a token uses")
    ap.add_argument("--chunk", type=int, default=512, help="state modes: keys a chunk of the attention holds")
    ap.add_argument("--rank", type=int, default=128, help="latent modes: cached numbers per token")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=3072)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--inter", type=int, default=3072)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--only", default=None, help="run one kernel by the name printed in the first column")
    ap.add_argument("--once", action="store_true", help="launch without graph or timing (for profilers)")
    a = ap.parse_args(argv)
    if a.layers is None:
        a.layers = 28 if a.mode.endswith("decode") else 4
    if a.mode.startswith("state"):
        state(a, a.mode == "state-decode")
    elif a.mode.startswith("latent"):
        latent(a, a.mode == "latent-decode")
    else:
        (decode if a.mode == "decode" else prefill)(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
