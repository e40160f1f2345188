"""Softmax attention with grouped key/value heads, as a mixer.

Order of operations, from the reference (`gemma/gemma.go:66-95`): project q, k,
v without biases; encode positions on q and k; cache k (encoded) and v; scale
the scores by `scale`; cap * tanh(s / cap) when a cap is set; mask; softmax;
weighted sum of values; merge heads; output projection.  Query head h uses
key/value head h // (heads / kv heads) (`gemma/gemma.go:79-81`,
`cpu/cpu_attn.go:72`).  The mask is on absolute positions: key j is seen by
query i iff j <= i and, with a window, j > i - window (the reference's mask is
causal only and ignores the cache offset, `gemma/gemma.go:232-240`).

The three projections are one product over the rows q | k | v concatenated at
load; the names on disk stay as they are.  A prompt step reads keys and values
from the step's own buffer (a windowed layer may see a prompt longer than its
ring holds); a decode step reads the paged cache.  A step that continues
sequences with several tokens (`ctx.extends`: a prompt that comes in pieces, as
the reference's session feeds it, `qwen/session.go:272-303`) reads the earlier
positions from the cache and its own from the step's buffer, and stores its
own only afterwards: a ring still needs the places they will take.
"""
from __future__ import annotations

import torch

from ..cache.cache import KVNeed
from ..weights.loader import TensorSpec
from .base import Mixer, PositionEncoding, Runtime, StepContext


class SoftmaxAttention(Mixer):
    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 position: PositionEncoding, names: dict[str, str], softcap: float = 0.0,
                 window: int | None = None, init_std: float = 0.02):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads do not divide over {n_kv_heads} key/value heads")
        if head_dim % 16 or not 16 <= head_dim <= 512:
            raise ValueError(f"the attention kernels take head sizes in steps of 16 from 16 to 512, found {head_dim}")
        for k in ("q", "k", "v", "o"):
            if k not in names:
                raise ValueError(f"attention needs the checkpoint name of its {k!r} projection")
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.scale = float(scale)
        self.softcap = float(softcap or 0.0)
        self.window = int(window) if window else 0
        self.position = position
        self.names = dict(names)
        self.init_std = init_std
        self.w_qkv = None
        self.w_q = None
        self.w_o = None

    # -- what it loads and keeps -------------------------------------------
    def tensor_specs(self):
        nq, nkv, hd, H, s = self.n_heads, self.n_kv_heads, self.head_dim, self.hidden, self.init_std
        return {self.names["q"]: TensorSpec((nq * hd, H), init_std=s),
                self.names["k"]: TensorSpec((nkv * hd, H), init_std=s),
                self.names["v"]: TensorSpec((nkv * hd, H), init_std=s),
                self.names["o"]: TensorSpec((H, nq * hd), init_std=s)}

    def sub_parts(self):
        return [self.position]

    def cache_needs(self):
        return {"kv": KVNeed(self.n_kv_heads, self.head_dim, self.window or None)}

    def prompt_flops(self, n_tokens: int) -> float:
        w = self.window or n_tokens
        full = min(n_tokens, w)                           # queries 0 .. full-1 see i + 1 keys, the rest w
        visible = full * (full + 1) // 2 + (n_tokens - full) * w
        return 4.0 * self.n_heads * self.head_dim * visible      # q k^T and p v: 2 flops a multiply-add each

    def load(self, store, rt: Runtime):
        if rt.dtype == torch.bfloat16 and (self.hidden % 8 or (self.n_heads * self.head_dim) % 8):
            raise ValueError("the bfloat16 products need widths that are multiples of 8 "
                             f"(hidden {self.hidden}, heads x head size {self.n_heads * self.head_dim})")
        q, k, v = (store.get(self.names[n], rt.dtype) for n in ("q", "k", "v"))
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        del q, k, v
        store.drop(self.names["q"], self.names["k"], self.names["v"])      # the fused copy is the one that stays
        self.w_q = self.w_qkv[: self.n_heads * self.head_dim]      # a layer that only reads keys projects q alone
        self.w_o = store.get(self.names["o"], rt.dtype).contiguous()
        self.position.load(store, rt)

    # -- a step ------------------------------------------------------------
    def _decode_geometry(self, ctx: StepContext, sm_count: int):
        """(chunk, most chunks a sequence has): how the keys of a decode step are cut up for the CTAs.

        A CTA per (sequence, key/value head, chunk); two or three CTAs fit an SM.  In tiles of 32 keys a CTA costs the tiles
        of its chunk plus a fixed share for starting its pipeline and for the merge.  Long chunks amortise the fixed
        share, short ones fill the SMs and even the load out.  The host knows the step's lengths by their bound,
        their mean (in eighths of the bound) and whether they are about equal; all three are part of a recorded
        step's key.  Measured on a B200 at 8 heads over 4, head size 256 (attention and merge, one layer): 64
        sequences of 198 to 2,087 keys 63.6 us at chunks of 384 against 86.9 at 2,048 (one chunk a sequence); 8 such
        sequences 14.4 us at 128 against 16.9 at 256; 8 sequences of 8,100 keys 49.5 us at 1,024."""
        bound = max(ctx.len_bound, 1)
        span = min(bound, self.window) if self.window else bound
        pairs = ctx.n_seq * self.n_kv_heads
        held = getattr(ctx.rt.ops, "attn_decode_resident", None)       # CTAs of a launch that the GPU holds at once
        mean = min(ctx.len_mean or bound, bound)
        seen = min(mean, self.window) if self.window else mean          # keys a sequence of mean length attends over
        extra = 1 if self.window and seen >= self.window else 0         # a window seldom starts on a chunk's border
        best = None
        for chunk in range(64, 2049, 64):
            launched = (bound + chunk - 1) // chunk
            if self.window:
                launched = min(launched, (self.window + chunk - 1) // chunk + 1)
            resident = held(self.head_dim, ctx.rt.dtype, pairs * launched, sm_count) if held else 2 * sm_count
            if ctx.len_even:
                # CTAs of equal length run in waves.  A launch of no more CTAs than SMs takes stages of 64 keys at
                # head sizes above 128, which cost about two thirds of two stages of 32 (one sequence of 8,100 keys:
                # 14.9 us a layer at chunks of 256 and 128 CTAs against 17.1 at chunks of 192 and 172 CTAs)
                n_chunks = (seen + chunk - 1) // chunk + extra
                waves = (pairs * n_chunks + resident - 1) // resident
                wide = self.head_dim > 128 and pairs * launched <= sm_count
                cost = waves * (min(chunk, seen) // 32 * (0.65 if wide else 1.0) + 6) + n_chunks / 8      # (the merge reads every chunk)
            else:
                # unequal lengths: the SMs' even share of all tiles and fixed shares, then the longest CTA, which
                # may start last (halved while every CTA has an SM's slot to itself from the start)
                n_ctas = pairs * (seen / chunk + 0.5 + extra)
                share = (4 * n_ctas + pairs * seen / 32) / resident
                cost = min(chunk, span) // 32 + 4 + (share if n_ctas > resident else share / 2) + (span / chunk + extra) / 8
            if chunk < bound:
                cost += 6          # more than one chunk a sequence: partial results and a merge kernel
            if (min(bound, span) + chunk - 1) // chunk + (1 if self.window and span >= self.window else 0) > 64:
                cost += 8          # beyond 64 chunks the merge forms its weights block-wide, not per warp: twice the time
            if best is None or cost < best[0]:
                best = (cost, chunk)
        chunk = best[1]
        max_chunks = (bound + chunk - 1) // chunk
        if self.window:
            max_chunks = min(max_chunks, (self.window + chunk - 1) // chunk + 1)
        return chunk, max_chunks

    def forward(self, x, ctx: StepContext, line):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        T, nq, nkv, hd = ctx.n_tok, self.n_heads, self.n_kv_heads, self.head_dim
        kv = line["kv"]
        own = kv.write
        heads = nq + 2 * nkv if own else nq
        # a written line that later layers read keeps its step buffer until the step ends
        name = f"attn.qkv.line{line.index}" if (own and line.has_readers and ctx.mode == "prefill") else "attn.qkv"
        qkv = ws.buf(name, (T, heads, hd), rt.dtype)
        extends = ctx.mode == "prefill" and ctx.extends
        if extends:                                   # attend first, store afterwards
            rt.linear(x, self.w_qkv if own else self.w_q, qkv.view(T, -1))
            self.position.encode(qkv, ctx, nq, nkv, hd, own)
        else:
            self.position.project_encode_store(x, self.w_qkv if own else self.w_q, qkv, ctx, nq, nkv, hd, kv)
        att = ws.buf("attn.ctx", (T, nq * hd), rt.dtype)
        if ctx.mode == "prefill":
            n_scratch = ops.attn_prefill_scratch_floats(T, ctx.n_seq, nq, hd, rt.dtype)
            scratch = ws.buf("attn.prefill_partial", (n_scratch,), torch.float32) if n_scratch else None
            before = dict(seq_start=ctx.seq_start, seq_slot=ctx.seq_slot, kpool=kv.k, vpool=kv.v, page_table=kv.table,
                          ring_len=kv.ring_len) if extends else {}
            if own:
                if line.has_readers:
                    ctx.shared[("kv", line.index)] = (qkv, heads, nq)
                ops.attn_prefill(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_first_row, att, nq, nkv, hd, self.scale,
                                 self.softcap, self.window, seq_len=ctx.seq_end, scratch=scratch, host_lens=ctx.step_lens,
                                 **before)
            else:
                src, src_heads, k0 = ctx.shared[("kv", line.index)]
                ops.attn_prefill(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_first_row, att, nq, nkv, hd, self.scale,
                                 self.softcap, self.window, kv_src=src, kv_row_heads=src_heads, kv_k_head0=k0,
                                 seq_len=ctx.seq_end, scratch=scratch, host_lens=ctx.step_lens, **before)
            if extends and own:
                store = lambda: ops.kv_store(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, nq, nkv, hd,
                                             kv.k, kv.v, kv.table, kv.ring_len)
                if line.has_readers:                  # the layers that read this line want it as the step found it
                    ctx.shared.setdefault("after_step", []).append(store)
                else:
                    store()
        else:
            chunk, max_chunks = self._decode_geometry(ctx, rt.sm_count)
            scratch = ws.buf("attn.partial", (ops.attn_decode_scratch_floats(ctx.n_seq, nq, hd, max_chunks),),
                             torch.float32)
            ops.attn_decode(qkv, kv.k, kv.v, kv.table, ctx.seq_slot, ctx.seq_end, scratch, att, nq, nkv, hd,
                            self.scale, self.softcap, self.window, kv.ring_len, chunk, max_chunks)
        out = ws.buf("mixer.out", (T, self.hidden), rt.dtype)
        return rt.linear(att, self.w_o, out)
