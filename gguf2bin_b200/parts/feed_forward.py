"""Feed-forwards.  ``swiglu``: down( silu(gate x) * (up x) ), no bias, dense
(src/l5_model.c:588-597, silu src/l3_math.c:57-62 of AnonymoDGH/gguf2bin).

The gate and up matrices are fused into one at bind time, rows alternating in blocks of
eight (eight gate rows, then the eight up rows of the same outputs), so one product
yields both and a kernel finds a gate and its up value sixteen columns apart at most.
A width that is no multiple of eight keeps the plain order (all gates, then all ups).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.specs import ConfigError, PartSpec
from ..weights.loader import Expected
from .fused import normed_linear
from .registry import register_feed_forward


class SwiGLU:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.inter = int(spec["intermediate_size"])
        self.hidden = int(hidden_size)
        self.block = 8 if self.inter % 8 == 0 else self.inter
        self.dtype = dtype
        self.names = dict(spec["names"])
        self.w_gate_up = self.w_down = None

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n, inter = dict(spec["names"]), spec["intermediate_size"]
        return {n["gate"]: Expected((inter, hidden_size)), n["up"]: Expected((inter, hidden_size)),
                n["down"]: Expected((hidden_size, inter))}

    def bind(self, tensors: dict) -> None:
        g, u = tensors[self.names["gate"]], tensors[self.names["up"]]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        b = self.block
        fused = torch.stack([g.view(self.inter // b, b, self.hidden),
                             u.view(self.inter // b, b, self.hidden)], dim=1)
        self.w_gate_up = fused.reshape(2 * self.inter, self.hidden).contiguous()
        self.w_down = tensors[self.names["down"]].contiguous()

    def weights(self):
        return (self.w_gate_up, self.w_down)

    def absorb_norm_weight(self, norm) -> bool:
        """As ``GQAAttention.absorb_norm_weight``, into the columns of the gate/up matrix."""
        if self.dtype != torch.bfloat16 or self.w_gate_up.dtype != torch.bfloat16 or self.block != 8 \
                or not hasattr(norm, "give_up_weight"):
            return False
        w = norm.give_up_weight()
        self.w_gate_up = (self.w_gate_up.float() * w.to(self.w_gate_up.device)[None, :]).to(torch.bfloat16).contiguous()
        return True

    def notices(self) -> list:
        return (kernels.product_notices("feed-forward gate/up", self.w_gate_up, self.dtype)
                + kernels.product_notices("feed-forward down", self.w_down, self.dtype))

    def forward(self, h: torch.Tensor, ctx, residual32: torch.Tensor) -> None:
        T = h.shape[0]
        ws = ctx.workspace
        mid = ws.buffer("ffn.mid", (T, self.inter), self.dtype)
        if not kernels.gate_up_fused(h, self.w_gate_up, mid, self.block):
            gu = ws.buffer("ffn.gate_up", (T, 2 * self.inter), self.dtype)
            kernels.linear(h, self.w_gate_up, gu)
            kernels.swiglu(gu, mid, self.block)
        kernels.linear(mid, self.w_down, residual32, accumulate=True)

    def forward_from_stream(self, x32: torch.Tensor, norm, ctx, residual32: torch.Tensor) -> None:
        """The same with the block's norm folded into the gate/up product."""
        mid = ctx.workspace.buffer("ffn.mid", (x32.shape[0], self.inter), self.dtype)
        normed_linear(x32, norm, self.w_gate_up, mid, ctx, gate_block=self.block)
        kernels.linear(mid, self.w_down, residual32, accumulate=True)


class ActMLP:
    """``act_mlp``: down( act(up x) ), two matrices and an elementwise activation.  Activations:
    ``xielu``, a z^2 + z/2 above zero and (1/2 + b)(exp(z) - 1 - z) + z/2 below, with a and b the
    softplus of two learned numbers (one tensor of two), computed in 32-bit.

    A block may hand it one more matrix that reads the same input (``take_along``): its rows go
    under the up matrix, one product computes both, and the step leaves that matrix's output in
    ``side_out`` (a view of the product's output)."""
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.inter, self.hidden = int(spec["intermediate_size"]), int(hidden_size)
        self.activation = spec.get("activation") or "xielu"
        if self.activation != "xielu":
            raise ConfigError(f"act_mlp: activation {self.activation!r} is not known (known: 'xielu')")
        self.dtype = dtype
        self.names = dict(spec["names"])
        self.w_up = self.w_down = self.act = None
        self.n_side = 0
        self.side_out = None

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n, inter = dict(spec["names"]), spec["intermediate_size"]
        return {n["up"]: Expected((inter, hidden_size)), n["down"]: Expected((hidden_size, inter)),
                n["act"]: Expected((2,))}

    def bind(self, tensors: dict) -> None:
        self.w_up = tensors[self.names["up"]].contiguous()
        self.w_down = tensors[self.names["down"]].contiguous()
        self.act = tensors[self.names["act"]].to(torch.float32).contiguous()

    def take_along(self, w_side: torch.Tensor) -> bool:
        """Puts ``w_side`` [n, hidden] under the up matrix; True when taken (equal dtypes, and an
        intermediate size that keeps the side output's rows on 16 bytes)."""
        if w_side.dtype != self.w_up.dtype or w_side.shape[1] != self.hidden or self.inter % 8 or self.n_side:
            return False
        pad = -(self.inter + w_side.shape[0]) % 8
        parts = [self.w_up, w_side]
        if pad:
            parts.append(torch.zeros((pad, self.hidden), dtype=self.w_up.dtype, device=self.w_up.device))
        self.w_up = torch.cat(parts, dim=0).contiguous()
        self.n_side = w_side.shape[0]
        return True

    def weights(self):
        return (self.w_up, self.w_down, self.act)

    def notices(self) -> list:
        return (kernels.product_notices("feed-forward up", self.w_up, self.dtype)
                + kernels.product_notices("feed-forward down", self.w_down, self.dtype))

    def forward(self, h: torch.Tensor, ctx, residual32: torch.Tensor) -> None:
        self._run(h, ctx, residual32, True)

    def forward_into(self, h: torch.Tensor, ctx, out32: torch.Tensor) -> None:
        """Stores the result instead of adding it."""
        self._run(h, ctx, out32, False)

    def _run(self, h, ctx, out32, accumulate: bool) -> None:
        T = h.shape[0]
        ws = ctx.workspace
        up = ws.buffer("mlp.up", (T, self.w_up.shape[0]), self.dtype)
        kernels.linear(h, self.w_up, up)
        self.side_out = up[:, self.inter:self.inter + self.n_side] if self.n_side else None
        mid = ws.buffer("mlp.mid", (T, self.inter), self.dtype)
        kernels.xielu(up[:, :self.inter], self.act, mid)
        kernels.linear(mid, self.w_down, out32, accumulate=accumulate)


register_feed_forward("swiglu", SwiGLU)
register_feed_forward("act_mlp", ActMLP)
