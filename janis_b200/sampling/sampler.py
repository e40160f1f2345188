"""Choosing the next token of each sequence from its logits, on the device.

Options and their meanings are the reference's (`SampleParams`,
`qwen/model.go:15-36`; `sampleToken`, `:57-165`):

* `temp` <= 0 is greedy: the highest logit, the lowest id among equals (`:88-109`).
* otherwise p_i ~ exp((l_i - max) / temp) (`:111-128`), cut to the nucleus of
  mass `top_p` in descending probability with ties to the lower id (`:130-152`,
  `:461-467`); `top_p` <= 0 or > 1 means 1 (`:130-133`).
* `repeat_penalty` > 1 divides the positive and multiplies the negative logits
  of the tokens among the last `repeat_last_n` of the reply (`:60-86`), before
  anything else; <= 1 switches it off.
* `seed`: the reference seeds Go's generator once per reply (`qwen/session.go:367`).
  Here the random number of a draw is a counter-based function of (seed, request,
  index of the token in the reply), so a reply does not depend on what else is in
  its batch; Go's sequence is not reproduced.  Within the kept set the draw walks
  ids in ascending order (the reference walks them by descending probability);
  the distribution is the same.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from ..parts.base import Runtime


@dataclass(frozen=True)
class SamplingParams:
    temp: float = 0.0
    top_p: float = 1.0
    seed: int = 0
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64

    def normalized(self) -> "SamplingParams":
        top_p = self.top_p if 0.0 < self.top_p <= 1.0 else 1.0
        return SamplingParams(float(self.temp), float(top_p), int(self.seed), float(self.repeat_penalty),
                              int(self.repeat_last_n))


class Sampler:
    MAX_ROWS = 4096                 # rows whose request and token numbers travel through the pinned staging ring

    def __init__(self, rt: Runtime):
        self.rt = rt
        self._on_gpu = torch.device(rt.device).type == "cuda"
        self._stage: list = []      # pinned [2, MAX_ROWS] buffers, used in turn
        self._stage_done: list = []
        self._turn = 0
        self._meta = None           # their device copy: row 0 request numbers, row 1 token numbers

    def _numbers(self, request_ids, token_index, R: int):
        """(request numbers, token numbers) of the step's rows as int32 tensors on the device.  On a GPU they go
        through pinned memory in one copy that the host does not wait for, so a sampled decode step costs the host
        as little as a greedy one; the copy is ordered behind the kernels that read the last step's numbers."""
        dev = self.rt.device
        if not self._on_gpu or R > self.MAX_ROWS:
            return (torch.tensor(list(request_ids), dtype=torch.int32, device=dev),
                    torch.tensor(list(token_index), dtype=torch.int32, device=dev))
        if self._meta is None:
            self._meta = torch.zeros((2, self.MAX_ROWS), dtype=torch.int32, device=dev)
            self._stage = [torch.zeros((2, self.MAX_ROWS), dtype=torch.int32).pin_memory() for _ in range(4)]
            self._stage_done = [None] * len(self._stage)
        i = self._turn
        self._turn = (i + 1) % len(self._stage)
        if self._stage_done[i] is not None:
            self._stage_done[i].synchronize()
        host = self._stage[i].numpy()
        host[0, :R] = request_ids
        host[1, :R] = token_index
        self._meta[:, :R].copy_(self._stage[i][:, :R], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._stage_done[i] = ev
        return self._meta[0, :R], self._meta[1, :R]

    def sample(self, logits: torch.Tensor, params: SamplingParams, request_ids: Sequence[int],
               token_index: Sequence[int], recent: Sequence[Sequence[int]] | None = None,
               banned: Sequence[int] | None = None, return_uniform: bool = False, out: torch.Tensor | None = None):
        """One token per row of float32 `logits` [R, V] (changed in place by penalty and masking).
        Returns int32 [R] on the device, written into `out` when given (and the uniform numbers used,
        when asked)."""
        ops, dev = self.rt.ops, self.rt.device
        p = params.normalized()
        R = logits.shape[0]
        if p.repeat_penalty > 1.0 and recent is not None and any(len(r) for r in recent):
            n = p.repeat_last_n if p.repeat_last_n > 0 else max(len(r) for r in recent)
            n = max(1, min(n, max(len(r) for r in recent)))
            table = np.full((R, n), -1, dtype=np.int32)
            for i, r in enumerate(recent):
                tail = list(r)[-n:]
                table[i, :len(tail)] = tail
            ops.repeat_penalty(logits, torch.from_numpy(table).to(dev), p.repeat_penalty)
        if banned:
            ops.mask_tokens(logits, torch.tensor(sorted(set(int(b) for b in banned)), dtype=torch.int32, device=dev))
        if out is None:
            out = torch.empty((R,), dtype=torch.int32, device=dev)
        if p.temp <= 0.0:
            ops.argmax(logits, out)
            return (out, None) if return_uniform else out
        ids, idx = self._numbers(request_ids, token_index, R)
        u = torch.empty((R,), dtype=torch.float32, device=dev) if return_uniform else None
        ops.sample(logits, out, p.temp, p.top_p, p.seed, ids, idx, u)
        return (out, u) if return_uniform else out
