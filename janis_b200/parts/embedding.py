"""Token embedding into the float32 residual stream, and the output head.

Gemma2 scales the embedding by sqrt(hidden), a float32 constant
(`gemma/gemma.go:193`, `:197`), ties the head to the embedding table
(`gemma/gemma.go:210`, `qwen/embed.go:87-89`) and caps the logits with
fc * tanh(logits / fc) (`gemma/gemma.go:211-212`).  Logits are float32.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, Runtime, StepContext


class Embedding(Part):
    def __init__(self, vocab: int, hidden: int, table_name: str, scale: float = 1.0, init_std: float = 0.02):
        self.vocab, self.hidden = vocab, hidden
        self.table_name = table_name
        self.scale = float(scale)
        self.init_std = init_std
        self.table = None
        self.scale_used = self.scale

    def tensor_specs(self):
        return {self.table_name: TensorSpec((self.vocab, self.hidden), init_std=self.init_std)}

    def load(self, store, rt: Runtime):
        self.table = store.get(self.table_name, rt.dtype).contiguous()
        # the reference casts the scalar to the activation dtype before the multiply (`mlxc/mlxc.go:587-601`):
        # in bfloat16 sqrt(2304) = 48 stays exact, sqrt(3584) = 59.87 becomes 59.75
        self.scale_used = float(torch.tensor(self.scale, dtype=torch.float32).to(rt.dtype))

    def forward(self, tokens, ctx: StepContext, out):
        return ctx.rt.ops.embed(tokens, self.table, self.scale_used, out)


class LMHead(Part):
    """logits = y W^T, then the cap.  `table_name` may be the embedding's (a tied head)."""

    def __init__(self, vocab: int, hidden: int, table_name: str, softcap: float = 0.0, init_std: float = 0.02):
        self.vocab, self.hidden = vocab, hidden
        self.table_name = table_name
        self.softcap = float(softcap or 0.0)
        self.init_std = init_std
        self.table = None

    def tensor_specs(self):
        return {self.table_name: TensorSpec((self.vocab, self.hidden), init_std=self.init_std)}

    def load(self, store, rt: Runtime):
        if rt.dtype == torch.bfloat16 and self.hidden % 8:
            raise ValueError(f"the bfloat16 products need a hidden width that is a multiple of 8, found {self.hidden}")
        self.table = store.get(self.table_name, rt.dtype).contiguous()

    def forward(self, y, ctx: StepContext, out):
        """y [R, hidden] in the compute dtype -> out float32 [R, vocab]."""
        ops = ctx.rt.ops
        R = y.shape[0]
        if ctx.rt.dtype == torch.float32:
            return ops.gemm_f32(y, self.table, out, self.softcap)
        if R <= ops.GEMV_FAST_ROWS:
            return ops.gemv_bf16(y, self.table, out, ops.EPI_SOFTCAP, self.softcap)
        if R <= ops.TC05_MAX_ROWS:
            return ops.gemm_tc05(y, self.table, out, ops.EPI_SOFTCAP, self.softcap)   # float32 logits straight from tensor memory
        # many rows: the library's product with float32 output, then the cap
        ops.matmul_bf16_to_f32(y, self.table, out)
        if self.softcap > 0:
            ops.softcap(out, self.softcap)
        return out
