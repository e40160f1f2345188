"""Plain torch statements of what each CUDA kernel computes, with the kernels' signatures.

Two uses, both in tests only: the `-m gpu` tests compare each kernel with the
function of the same name here; the CPU tests hand this module to the engine in
place of the kernels, which checks the host side (batching, cache bookkeeping,
schedules) against the plain model without a GPU.  Sums run in float64.
"""
from __future__ import annotations

import math

import numpy as np
import torch

PAGE = 64
GEMV_MAX_ROWS = 64
GEMV_FAST_ROWS = 16
EPI_NONE, EPI_GATED_GELU, EPI_SOFTCAP, EPI_GATED_SILU = 0, 1, 2, 3
GATE_GROUP = 8
ACT_GELU_TANH, ACT_SILU = 0, 1


def embed(tokens, table, scale, out):
    out.copy_((table[tokens.long()].double() * float(np.float32(scale))).to(out.dtype))
    return out


def _norm(x, w, eps):
    x = x.double()
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()


def rmsnorm(x, weight, eps, out, rows=None):
    src = x if rows is None else x[rows.long()]
    out.copy_(_norm(src, weight, eps).to(out.dtype))
    return out


def add_rmsnorm(h, res, w_post, eps_post, w_next=None, eps_next=0.0, out=None, n_part=1):
    r = res.double()
    if n_part > 1:
        r = r.sum(0)
    add = _norm(r, w_post, eps_post) if w_post is not None else r
    h.copy_((h.double() + add).float())
    if w_next is not None:
        out.copy_(_norm(h, w_next, eps_next).to(out.dtype))
    return out


def _act(g, act):
    if act == ACT_GELU_TANH:
        return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    return g / (1.0 + torch.exp(-g))


def gated_act(gu, out, act=ACT_GELU_TANH, group=GATE_GROUP):
    R, I2 = gu.shape
    I = I2 // 2
    v = gu.double().view(R, I // group, 2, group)
    out.copy_((_act(v[:, :, 0], act) * v[:, :, 1]).reshape(R, I).to(out.dtype))
    return out


def rope_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, rot, nq, nkv, hd, kpool=None, vpool=None,
               page_table=None, ring_len=0, store=True, write_cache=True):
    T = qkv.shape[0]
    half = rot // 2
    n_rot = nq + nkv if store else nq
    if half:
        theta = (tok_pos[:T].float()[:, None] * inv_freq.float()[None, :]).float()      # float32 angles
        c, s = torch.cos(theta.double())[:, None, :], torch.sin(theta.double())[:, None, :]
        a, b = qkv[:, :n_rot, :half].double(), qkv[:, :n_rot, half:rot].double()
        qkv[:, :n_rot, :half] = (a * c - b * s).to(qkv.dtype)
        qkv[:, :n_rot, half:rot] = (a * s + b * c).to(qkv.dtype)
    if not store or not write_cache:
        return qkv
    return kv_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, nq, nkv, hd, kpool, vpool, page_table, ring_len)


def kv_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, nq, nkv, hd, kpool, vpool, page_table, ring_len=0):
    T = qkv.shape[0]
    for t in range(T):
        seq = int(tok_seq[t])
        slot = int(seq_slot[seq])
        if slot < 0:
            continue
        pos = int(tok_pos[t])
        idx = pos
        if ring_len > 0:
            if pos < int(seq_end[seq]) - ring_len:
                continue
            idx = pos % ring_len
        page = int(page_table[slot, idx // PAGE])
        kpool[page, :, idx % PAGE, :] = qkv[t, nq:nq + nkv]
        vpool[page, :, idx % PAGE, :] = qkv[t, nq + nkv:nq + 2 * nkv]
    return qkv


def gemv_rope_store(x, w, qkv, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, nq, nkv, hd, kpool=None, vpool=None,
                    page_table=None, ring_len=0, store=True):
    heads = nq + 2 * nkv if store else nq
    M = x.shape[0]
    full = (x.double() @ w.double().T).to(qkv.dtype).view(M, heads, hd)
    rope_store(full, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, hd, nq, nkv, hd, kpool, vpool, page_table,
               ring_len, store)
    qkv[:, :nq] = full[:, :nq]
    return qkv


def gemm_f32(x, w, out, cap=0.0):
    v = x.double() @ w.double().T
    if cap > 0:
        v = cap * torch.tanh(v / cap)
    out.copy_(v.to(out.dtype))
    return out


def gemv_bf16(x, w, out, epilogue=EPI_NONE, cap=0.0, cluster=0):
    v = x.double() @ w.double().T
    if epilogue in (EPI_GATED_GELU, EPI_GATED_SILU):
        M, N = v.shape
        g = v.view(M, N // 16, 2, 8)
        v = (_act(g[:, :, 0], ACT_GELU_TANH if epilogue == EPI_GATED_GELU else ACT_SILU) * g[:, :, 1]).reshape(M, N // 2)
    elif epilogue == EPI_SOFTCAP and cap > 0:
        v = cap * torch.tanh(v / cap)
    out.copy_(v.to(out.dtype))
    return out


def matmul_bf16_to_f32(x, w, out):
    out.copy_((x.double() @ w.double().T).float())
    return out


def softcap(x, cap):
    x.copy_((cap * torch.tanh(x.double() / cap)).float())
    return x


TC05_MAX_ROWS = 64


def gemm_tc05(x, w, out, epilogue=EPI_NONE, cap=0.0, split=0):
    return gemv_bf16(x, w, out, epilogue, cap)


def linear_bf16(x, w, out):
    return gemv_bf16(x, w, out)


def _attend(q, k, v, scale, cap):
    """q [nq, hd], k/v [n, nkv, hd] (all visible) -> [nq, hd], float64."""
    nq, nkv = q.shape[0], k.shape[1]
    rep = nq // nkv
    out = torch.empty(nq, q.shape[1], dtype=torch.float64)
    for h in range(nq):
        s = (k[:, h // rep].double() @ q[h].double()) * scale
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        p = torch.softmax(s, dim=0)
        out[h] = p @ v[:, h // rep].double()
    return out


def attn_prefill_scratch_floats(n_tok, n_seq, nq, hd, dtype=torch.bfloat16):
    return 0


def attn_prefill(qkv, tok_pos, tok_seq, seq_first_row, out, nq, nkv, hd, scale, cap, window, kv_src=None,
                 kv_row_heads=None, kv_k_head0=None, seq_len=None, tensor_cores=True, scratch=None, seq_start=None,
                 seq_slot=None, kpool=None, vpool=None, page_table=None, ring_len=0, host_lens=None):
    T = qkv.shape[0]
    if kv_src is None:
        kv_src, kv_k_head0 = qkv, nq
    for t in range(T):
        pos = int(tok_pos[t])
        seq = int(tok_seq[t])
        start = int(seq_start[seq]) if seq_start is not None else 0
        first = int(seq_first_row[seq]) - start           # the row position 0 would have
        lo = max(0, pos - window + 1) if window > 0 else 0
        ks, vs = [], []
        if lo < start:                                    # keys and values that earlier steps stored
            slot = int(seq_slot[seq])
            idx = [(j % ring_len if ring_len > 0 else j) for j in range(lo, start)]
            pages = [int(page_table[slot, i // PAGE]) for i in idx]
            ks.append(torch.stack([kpool[p, :, i % PAGE] for p, i in zip(pages, idx)]).cpu())
            vs.append(torch.stack([vpool[p, :, i % PAGE] for p, i in zip(pages, idx)]).cpu())
        rows = kv_src[first + max(lo, start):first + pos + 1]
        ks.append(rows[:, kv_k_head0:kv_k_head0 + nkv].cpu())
        vs.append(rows[:, kv_k_head0 + nkv:kv_k_head0 + 2 * nkv].cpu())
        o = _attend(qkv[t, :nq].cpu(), torch.cat(ks), torch.cat(vs), scale, cap)
        out[t] = o.reshape(-1).to(out.dtype)
    return out


def attn_decode_scratch_floats(n_seq, nq, hd, max_chunks):
    return n_seq * nq * max_chunks * (hd + 2)


def attn_decode(qkv, kpool, vpool, page_table, seq_slot, seq_len, scratch, out, nq, nkv, hd, scale, cap, window,
                ring_len, chunk, max_chunks):
    n_seq = qkv.shape[0]
    for s in range(n_seq):
        slot = int(seq_slot[s])
        if slot < 0:
            out[s] = 0
            continue
        n = int(seq_len[s])
        lo = max(0, n - window) if window > 0 else 0
        first_chunk = lo // chunk
        if (n + chunk - 1) // chunk - first_chunk > max_chunks:
            out[s] = float("nan")
            continue
        idx = [(j % ring_len if ring_len > 0 else j) for j in range(lo, n)]
        pages = [int(page_table[slot, i // PAGE]) for i in idx]
        offs = [i % PAGE for i in idx]
        k = torch.stack([kpool[p, :, o] for p, o in zip(pages, offs)]).cpu()
        v = torch.stack([vpool[p, :, o] for p, o in zip(pages, offs)]).cpu()
        out[s] = _attend(qkv[s, :nq].cpu(), k, v, scale, cap).reshape(-1).to(out.dtype)
    return out


def argmax(logits, out):
    for r in range(logits.shape[0]):
        row = logits[r]
        out[r] = int((row == row.max()).nonzero()[0])
    return out


_M0, _M1 = 0xD2511F53, 0xCD9E8D57


def philox_uniform(seed, request, index):
    """Philox4x32-10 with key = seed (two words) and counter = (request, index, 0, 0); first word -> [0, 1)."""
    c = [request & 0xFFFFFFFF, index & 0xFFFFFFFF, 0, 0]
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = _M0 * c[0], _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF, ((p0 >> 32) ^ c[3] ^ k1) & 0xFFFFFFFF,
             p0 & 0xFFFFFFFF]
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return float(np.float32(c[0] >> 8) * np.float32(1.0 / 16777216.0))


def sample_row(row, temp, top_p, u):
    """The choice for one row given its uniform number: float64 throughout."""
    l = row.double()
    w = torch.exp((l - l.max()) / temp)
    p = (w / w.sum()).tolist()
    if 0.0 < top_p < 1.0:
        order = sorted(range(len(p)), key=lambda i: (-p[i], i))
        keep, cum = [], 0.0
        for i in order:
            keep.append(i)
            cum += p[i]
            if cum >= top_p:
                break
        keep.sort()
    else:
        keep = list(range(len(p)))
    mass = sum(p[i] for i in keep)
    target, acc = u * mass, 0.0
    for i in keep:
        acc += p[i]
        if target <= acc:
            return i
    return keep[-1]


def sample(logits, out, temp, top_p, seed, request_ids, token_index, u_out=None):
    for r in range(logits.shape[0]):
        u = philox_uniform(int(seed), int(request_ids[r]), int(token_index[r]))
        if u_out is not None:
            u_out[r] = u
        out[r] = sample_row(logits[r].cpu(), temp, top_p, u)
    return out


def repeat_penalty(logits, recent, penalty):
    for r in range(logits.shape[0]):
        for tok in set(int(t) for t in recent[r].tolist() if 0 <= int(t) < logits.shape[1]):
            v = logits[r, tok]
            logits[r, tok] = v / penalty if v > 0 else v * penalty
    return logits


def mask_tokens(logits, ids):
    for tok in ids.tolist():
        if 0 <= tok < logits.shape[1]:
            logits[:, tok] = float("-inf")
    return logits
