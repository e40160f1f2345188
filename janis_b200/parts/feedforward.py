"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases.

Gemma2's is GeGLU with the tanh form of gelu (`gemma/gemma.go:121-123`;
0.5 v (1 + tanh(0.7978845608028654 (v + 0.044715 v^3))), `cpu/cpu.go:417-423`);
with act="silu" it is the SwiGLU of the reference's other models
(`qwen/mlp.go:32-36`).

gate and up are one product: their rows are interleaved at load in groups of 8
(8 gate rows, the 8 matching up rows, ...), which puts each gate value beside
its up value in one tile of the skinny decode kernel, so the activation is
applied to float accumulators before anything is written.  Above 16 rows the
product comes from the library and a separate kernel applies the activation.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import FeedForward, Runtime, StepContext

_ACTS = {"gelu_tanh": 0, "gelu_pytorch_tanh": 0, "silu": 1}


class GatedMLP(FeedForward):
    GROUP = 8

    def __init__(self, hidden: int, intermediate: int, names: dict[str, str], act: str = "gelu_tanh",
                 init_std: float = 0.02):
        if act not in _ACTS:
            raise ValueError(f"unknown activation {act!r} (known: {sorted(_ACTS)})")
        if intermediate % self.GROUP:
            raise ValueError(f"the fused gate/up layout needs an intermediate width that is a multiple of "
                             f"{self.GROUP}, found {intermediate}")
        for k in ("gate", "up", "down"):
            if k not in names:
                raise ValueError(f"feed-forward needs the checkpoint name of its {k!r} projection")
        self.hidden, self.intermediate = hidden, intermediate
        self.act = _ACTS[act]
        self.names = dict(names)
        self.init_std = init_std
        self.w_gu = None
        self.w_down = None

    def tensor_specs(self):
        H, I, s = self.hidden, self.intermediate, self.init_std
        return {self.names["gate"]: TensorSpec((I, H), init_std=s),
                self.names["up"]: TensorSpec((I, H), init_std=s),
                self.names["down"]: TensorSpec((H, I), init_std=s)}

    def load(self, store, rt: Runtime):
        if rt.dtype == torch.bfloat16 and self.hidden % 8:
            raise ValueError(f"the bfloat16 products need a hidden width that is a multiple of 8, found {self.hidden}")
        g = store.get(self.names["gate"], rt.dtype)
        u = store.get(self.names["up"], rt.dtype)
        I, H, G = self.intermediate, self.hidden, self.GROUP
        fused = torch.stack([g.view(I // G, G, H), u.view(I // G, G, H)], dim=1)   # [I/G, 2, G, H]
        self.w_gu = fused.reshape(2 * I, H).contiguous()
        del g, u, fused
        store.drop(self.names["gate"], self.names["up"])                   # the fused copy is the one that stays
        self.w_down = store.get(self.names["down"], rt.dtype).contiguous()

    def forward(self, x, ctx: StepContext):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        T, I = ctx.n_tok, self.intermediate
        a = ws.buf("ffn.act", (T, I), rt.dtype)
        epi = ops.EPI_GATED_GELU if self.act == 0 else ops.EPI_GATED_SILU
        if rt.dtype == torch.bfloat16 and T <= ops.GEMV_FAST_ROWS:
            ops.gemv_bf16(x, self.w_gu, a, epi)
        else:
            # (ops.gemm_tc05 computes this product with the activation fused for 17..64 rows, but at these
            # shapes the library product plus the activation kernel is still the faster pair)
            gu = ws.buf("ffn.gu", (T, 2 * I), rt.dtype)
            rt.linear(x, self.w_gu, gu)
            ops.gated_act(gu, a, self.act, self.GROUP)
        out = ws.buf("ffn.out", (T, self.hidden), rt.dtype)
        return rt.linear(a, self.w_down, out)
