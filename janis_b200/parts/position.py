"""Position encodings applied to queries and keys inside a mixer.

`RotaryEncoding` is the half-split rotary encoding the reference applies to a
whole head (`gemma/gemma.go:73-74`; `cpu/cpu_attn.go:13-62`, non-traditional):
inv_i = base^(-2i/dims) computed in float64 and rounded to float32, theta =
float32(pos) * inv_i, pair (i, i + dims/2).  It is handed to the kernel as a
table of inverse frequencies, so scaled frequencies (`qwen/attention.go:23-42`)
or a rotation of part of the head (`qwen/config.go:55`) are other tables, not
other kernels.  `NoPosition` rotates nothing and only stores keys and values.

Keys are cached after encoding (`gemma/gemma.go:73-75`), so the order of the
places in a ring does not matter.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding, Runtime, StepContext


class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, base: float, rotary_dims: int | None = None, inv_freq=None):
        rot = head_dim if rotary_dims is None else int(rotary_dims)
        if rot % 2 or rot < 0 or rot > head_dim:
            raise ValueError(f"rotary width {rot} must be even and at most the head size {head_dim}")
        self.head_dim = head_dim
        self.rot = rot
        self.base = float(base)
        if inv_freq is None:
            inv_freq = [np.float32(math.pow(self.base, -float(2 * i) / float(rot))) for i in range(rot // 2)]
        self._inv_host = np.asarray(inv_freq, dtype=np.float32)
        if self._inv_host.shape != (rot // 2,):
            raise ValueError("inv_freq must hold rotary_dims / 2 values")
        self.inv_freq = None

    def load(self, store, rt: Runtime):
        self.inv_freq = torch.from_numpy(self._inv_host.copy()).to(rt.device)

    def encode(self, qkv, ctx: StepContext, nq: int, nkv: int, hd: int, with_keys: bool):
        return ctx.rt.ops.rope_store(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq, self.rot,
                                     nq, nkv, hd, store=with_keys, write_cache=False)

    def encode_and_store(self, qkv, ctx: StepContext, nq: int, nkv: int, hd: int, kv_line):
        ops = ctx.rt.ops
        if kv_line is None or not kv_line.write:
            return ops.rope_store(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq,
                                  self.rot, nq, nkv, hd, store=False)
        return ops.rope_store(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq, self.rot,
                              nq, nkv, hd, kv_line.k, kv_line.v, kv_line.table, kv_line.ring_len, store=True)


    def project_encode_store(self, x, w, qkv, ctx: StepContext, nq: int, nkv: int, hd: int, kv_line):
        """A decode step of up to 16 rows in bfloat16 that rotates the whole head: projection, encoding and cache
        write are one kernel (the product's tiles pair each element with its partner half a head on)."""
        ops = ctx.rt.ops
        fused = (ctx.mode == "decode" and ctx.rt.dtype == torch.bfloat16 and self.rot == hd and hd % 16 == 0
                 and x.shape[0] <= getattr(ops, "GEMV_FAST_ROWS", 0) and hasattr(ops, "gemv_rope_store"))
        if not fused:
            return super().project_encode_store(x, w, qkv, ctx, nq, nkv, hd, kv_line)
        if kv_line is None or not kv_line.write:
            return ops.gemv_rope_store(x, w, qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq,
                                       nq, nkv, hd, store=False)
        return ops.gemv_rope_store(x, w, qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq,
                                   nq, nkv, hd, kv_line.k, kv_line.v, kv_line.table, kv_line.ring_len, store=True)


class NoPosition(RotaryEncoding):
    """No encoding: keys and values are stored as projected."""

    def __init__(self, head_dim: int):
        super().__init__(head_dim, 10000.0, rotary_dims=0)
