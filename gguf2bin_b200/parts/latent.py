"""``latent_attention``: causal attention over cached low-rank latents, without positions.

Per token the mixer projects its input u to queries q (``n_heads`` x ``qk_dim``) and to a latent
c = rmsnorm(W_down u) * w of ``kv_rank`` numbers, which is ALL it caches.  Keys and values are
projections of the latents, k_j = U_k c_j and v_j = U_v c_j per head.  Since
q . (U_k c_j) = (U_k^T q) . c_j and sum_j p_j U_v c_j = U_v (sum_j p_j c_j), a step never builds
keys or values: it takes U_k into the query (``kv_rank`` numbers per head), attends over the
latents themselves, which then are keys and values at once for every head (one kv head, one
panel per page: ``KVNeed(planes=1)``), and applies U_v to each head's weighted sum of latents.
Options, each a parameter of the spec: ``sink`` (a learned logit per head that joins the
softmax's denominator and nothing else), ``out_gate`` (each head's output times the sigmoid of
a linear function of u), ``shared_kv`` (no down-projection: the layer attends over the latents
that the schedule entry's ``cache_of`` layer stored), ``scale``.

Scores, softmax and the latent's norm are 32-bit; products accumulate in 32-bit.

Where a head's rank is not much more than its key (value) size, or the matrices are small,
bfloat16 compute multiplies U_k into the query matrix (U_v into the output matrix) once, when
the weights are bound (``folds``): the per-head products then cost nothing at run time, at the price of a query
(output) product that is rank / size times as large, and of one more rounding of the matrix to
bfloat16.  The output gate is a number per head, so it commutes with U_v and is applied to
the weighted latents, by the attention kernel itself; the queries, which then come out of the
input product in latent coordinates, are read by the attention in place.  The 32-bit path keeps the formula's order.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.storage import KVNeed, KVView
from ..config.specs import ConfigError, PartSpec
from ..weights.loader import Expected
from .registry import register_mixer

HEAD_PRODUCT_ROWS = 64       # steps of more rows multiply per head on the tensor cores (bfloat16)
FOLD_UP_TO = 1.5             # rank / head size up to which an up-projection is always multiplied into its neighbour
FOLD_SMALL_UP_TO = 4.0       # ... and up to which it is while the matrix grows by no more than FOLD_SMALL_BYTES
FOLD_SMALL_BYTES = 4 << 20


def folds(rank: int, size: int, heads: int, width: int) -> bool:
    """Whether a head's up-projection [size, rank] is multiplied into the [heads * size, width] matrix
    beside it, which then has heads * rank rows.  Always while that costs at most half as much again;
    for small matrices up to four times as much: a decode step reads the extra bytes in less time than
    the launch of the per-head product takes, and a prompt's per-head products are one launch a head."""
    if rank <= FOLD_UP_TO * size:
        return True
    extra = heads * (rank - size) * width * 2
    return rank <= FOLD_SMALL_UP_TO * size and extra <= FOLD_SMALL_BYTES


class LatentAttention:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.nh, self.dk, self.dv = int(spec["n_heads"]), int(spec["qk_dim"]), int(spec["v_dim"])
        self.rank = int(spec["kv_rank"])
        self.hidden = int(hidden_size)
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        self.shared_kv = bool(spec.get("shared_kv") or False)
        self.has_sink = bool(spec.get("sink") or False)
        self.has_gate = bool(spec.get("out_gate") or False)
        if min(self.nh, self.dk, self.dv, self.rank) <= 0:
            raise ConfigError("latent_attention: heads, sizes and rank must be positive")
        if self.rank > 512:
            raise ConfigError(f"latent_attention: kv_rank {self.rank} is more than the attention kernels' 512")
        self.dtype, self.device = dtype, device
        self.names = dict(spec["names"])
        # columns of the fused input product: queries, then the latent (unless shared), then the gates
        self.n_q = self.nh * self.dk
        self.n_c = 0 if self.shared_kv else self.rank
        self.n_g = self.nh if self.has_gate else 0
        self.w_in = self.w_o = self.w_uk = self.w_uv = self.c_norm = self.sink = None
        self.fold_k = self.fold_v = False

    # ---- weights -------------------------------------------------------------
    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n = dict(spec["names"])
        nh, dk, dv, r = spec["n_heads"], spec["qk_dim"], spec["v_dim"], spec["kv_rank"]
        out = {n["q"]: Expected((nh * dk, hidden_size)), n["up_k"]: Expected((nh * dk, r)),
               n["up_v"]: Expected((nh * dv, r)), n["o"]: Expected((hidden_size, nh * dv))}
        if not (spec.get("shared_kv") or False):
            out[n["down"]] = Expected((r, hidden_size))
            out[n["down_norm"]] = Expected((r,), init="scale")
        if spec.get("sink"):
            out[n["sink"]] = Expected((nh,))
        if spec.get("out_gate"):
            out[n["gate"]] = Expected((nh, hidden_size))
        return out

    def bind(self, tensors: dict) -> None:
        n = self.names
        w_q, w_o = tensors[n["q"]], tensors[n["o"]]
        folding = self.dtype == torch.bfloat16 and w_q.dtype == torch.bfloat16 and w_o.dtype == torch.bfloat16
        self.fold_k = folding and folds(self.rank, self.dk, self.nh, self.hidden)
        self.fold_v = folding and folds(self.rank, self.dv, self.nh, self.hidden)
        if self.fold_k:
            # W_q'[h] = U_k[h]^T W_q[h]: [rank, qk_dim] x [qk_dim, width] per head; the queries then
            # come out of the input product in latent coordinates, `rank` numbers per head
            uk = tensors[n["up_k"]].double().view(self.nh, self.dk, self.rank)
            wq = w_q.double().view(self.nh, self.dk, self.hidden)
            w_q = torch.einsum("hdr,hdw->hrw", uk, wq).reshape(self.nh * self.rank, self.hidden) \
                .to(torch.bfloat16).contiguous()
            self.n_q = self.nh * self.rank
        parts = [w_q]
        if not self.shared_kv:
            parts.append(tensors[n["down"]])
            self.c_norm = tensors[n["down_norm"]].to(torch.float32).contiguous()
        if self.has_gate:
            parts.append(tensors[n["gate"]])
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        rows = sum(p.shape[0] for p in parts)
        pad = -rows % 8                         # rows of the product's output start on 16 bytes
        if pad:
            parts.append(torch.zeros((pad, self.hidden), dtype=common, device=parts[0].device))
        self.w_in = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        if self.fold_v:
            # W_o'[:, h] = W_o[:, h] U_v[h]: [width, v_dim] x [v_dim, rank] per head
            uv = tensors[n["up_v"]].double().view(self.nh, self.dv, self.rank)
            wo = w_o.double().view(self.hidden, self.nh, self.dv)
            self.w_o = torch.einsum("whv,hvr->whr", wo, uv).reshape(self.hidden, self.nh * self.rank) \
                .to(torch.bfloat16).contiguous()
        else:
            self.w_o = w_o.contiguous()
            self.w_uv = tensors[n["up_v"]].to(self.dtype).contiguous()
        if not self.fold_k:
            self.w_uk = tensors[n["up_k"]].to(self.dtype).contiguous()
        if self.has_sink:
            self.sink = tensors[n["sink"]].to(torch.float32).contiguous()

    def weights(self):
        return [t for t in (self.w_in, self.w_o, self.w_uk, self.w_uv, self.c_norm, self.sink)
                if t is not None]

    def notices(self) -> list:
        from ..cache.storage import PAGE_SIZE
        return (kernels.product_notices("latent attention input", self.w_in, self.dtype)
                + kernels.product_notices("latent attention output", self.w_o, self.dtype)
                + kernels.attention_notices("latent attention", self.rank, PAGE_SIZE, self.dtype))

    # ---- cache ---------------------------------------------------------------
    def cache_need(self):
        return None if self.shared_kv else KVNeed(1, self.rank, 0, planes=1)

    # ---- step ----------------------------------------------------------------
    def forward(self, u: torch.Tensor, ctx, view: KVView, residual32: torch.Tensor) -> None:
        self._run(u, ctx, view, residual32, True, None)

    def forward_into(self, u: torch.Tensor, ctx, view: KVView, out32: torch.Tensor, keep=None) -> None:
        """Stores the mixer's result instead of adding it.  ``keep`` = (rows, ring, taps): the
        block's wish to have the last rows of every sequence written to its ring, which rides
        on the launch that writes the latents."""
        self._run(u, ctx, view, out32, False, keep)

    def _per_head(self, x, w, out, expand: bool, gate) -> None:
        """out[:, h] = w_h^T x[:, h] (absorb) or w_h x[:, h] (expand, then the gate)."""
        T = x.shape[0]
        n, r = w.shape[0] // self.nh, w.shape[1]
        fast = (self.dtype == torch.bfloat16 and T > HEAD_PRODUCT_ROWS and n % 8 == 0 and r % 8 == 0
                and x.stride(0) % 8 == 0 and out.stride(0) % 8 == 0)
        if not fast:
            kernels.head_product(x, w, out, self.nh, expand, gate)
            return
        for h in range(self.nh):
            wh = w[h * n:(h + 1) * n]
            if expand:
                kernels.linear(x[:, h * r:(h + 1) * r], wh, out[:, h * n:(h + 1) * n])
            else:
                kernels.linear(x[:, h * n:(h + 1) * n], self._uk_t[h], out[:, h * r:(h + 1) * r])
        if expand and gate is not None:
            kernels.head_gate(out, gate, self.nh)

    @property
    def _uk_t(self):
        """U_k of each head transposed ([rank, qk_dim] per head), for the tensor-core products
        that want the contraction index innermost; made when a long step first asks."""
        t = getattr(self, "_uk_t_cache", None)
        if t is None:
            t = self._uk_t_cache = self.w_uk.view(self.nh, self.dk, self.rank).transpose(1, 2).contiguous()
        return t

    def _run(self, u, ctx, view: KVView, out32, accumulate: bool, keep) -> None:
        T = u.shape[0]
        ws = ctx.workspace
        if view is None or view.planes != 1:
            raise kernels.KernelError("latent_attention: needs latent pages (one panel per page)")
        proj = ws.buffer("latent.in", (T, self.w_in.shape[0]), self.dtype)
        kernels.linear(u, self.w_in, proj)
        q = proj[:, :self.n_q]
        d = proj[:, self.n_q:self.n_q + self.n_c] if self.n_c else None
        gate = proj[:, self.n_q + self.n_c:self.n_q + self.n_c + self.n_g] if self.n_g else None
        rows, ring, taps = keep if keep is not None else (None, None, 0)
        if d is not None or ring is not None:
            kernels.latent_keep(d, self.c_norm, self.eps, view.pages if d is not None else None,
                                rows, ring, taps, ctx)
        if self.fold_k:
            qa = q                          # columns of the product's output: the attention reads them in place
        else:
            qa = ws.buffer("latent.q", (T, self.nh * self.rank), self.dtype)
            self._per_head(q, self.w_uk, qa, False, None)
        mix = ws.buffer("latent.mix", (T, self.nh * self.rank), self.dtype)
        # with U_v folded into the output matrix the heads' gate is the attention's last step
        kernels.attention(qa, mix, view.pages, ctx, self.nh, 1, self.rank, view.page_size, 0, self.scale,
                          sink=self.sink, planes=1, gate=gate if self.fold_v else None)
        if self.fold_v:
            o = mix
        else:
            o = ws.buffer("latent.o", (T, self.nh * self.dv), self.dtype)
            self._per_head(mix, self.w_uv, o, True, gate)
        kernels.linear(o, self.w_o, out32, accumulate=accumulate)


register_mixer("latent_attention", LatentAttention)
