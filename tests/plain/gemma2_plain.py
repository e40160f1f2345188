"""Plain, slow Gemma2 written from the reference's formulas.

Whole sequences, no cache, one function for each part, no code shared with the
package under test.  It is the oracle of the tests.  The reference's own model
code (Go, MLX 4-bit weights, batch 1, no sliding window) cannot be compiled or
imported here (no Go toolchain), so this file rests on the formulas alone; each
function cites the reference file and lines it restates.

The tensors may live on any device: the arithmetic follows the weights it is
given (the tests run the larger configurations on the GPU, in float64 torch
operations, to keep the oracle quick).

Everything is computed in ``dtype`` (float64 by default; float32 follows the
reference's CPU backend) except the rotation angles, which the reference forms
in float32 (`cpu/cpu_attn.go:16`, `:45-49`) and which are formed in float32
here too, so that the oracle rotates by the same angles.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


# ----------------------------------------------------------------------------
# model folder (own small reader: the package's loader is not used here)
# ----------------------------------------------------------------------------

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "F64": np.float64}


def read_safetensors(path):
    """name -> float64 torch tensor (format: `safetensors/safetensors.go:1-11`)."""
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[base + lo:base + hi]
        shape = info["shape"]
        if info["dtype"] == "BF16":
            u16 = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(raw, dtype=_ST_DTYPES[info["dtype"]]).astype(np.float64)
        out[name] = torch.from_numpy(arr.reshape(shape).copy())
    return out


def load_folder(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, weights


def layer_is_sliding(cfg, i):
    """Even layers slide, odd layers see every key, unless config.json lists the kinds.

    The reference leaves the window out (`gemma/gemma.go:7-9`); the alternation
    is the architecture's.
    """
    kinds = cfg.get("layer_types")
    if kinds:
        return kinds[i] == "sliding_attention"
    return i % 2 == 0


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def embed(ids, table, hidden, dtype=torch.float64):
    """h = E[ids] * sqrt(hidden)  (`gemma/gemma.go:193`, `:197`; `qwen/embed.go:78-83`)."""
    scale = float(np.float32(math.sqrt(float(hidden))))  # embScale is a float32
    return table.to(dtype)[torch.as_tensor(ids, dtype=torch.long, device=table.device)] * scale


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w)  (`gemma/gemma.go:22-28`, `cpu/cpu_ops.go:145-162`)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(ms + eps)) * (1.0 + w.to(x.dtype))


def rope(x, positions, base):
    """Half-split rotation of a whole head (`cpu/cpu_attn.go:13-62`, non-traditional).

    x: [heads, L, hd]; positions: [L] integers.  inv_i = base^(-2i/hd) rounded to
    float32, theta = float32(pos) * inv_i in float32, cos/sin of that float32
    angle taken in float64 (`cpu/cpu_attn.go:16`, `:45-49`).
    """
    hd = x.shape[-1]
    half = hd // 2
    inv = np.array([np.float32(math.pow(float(base), -float(2 * i) / float(hd))) for i in range(half)],
                   dtype=np.float32)
    pos = np.asarray(positions, dtype=np.float32)
    theta = (pos[:, None] * np.float32(1.0) * inv[None, :]).astype(np.float32)  # [L, half], float32 product
    c = torch.from_numpy(np.cos(theta.astype(np.float64))).to(x.dtype).to(x.device)
    s = torch.from_numpy(np.sin(theta.astype(np.float64))).to(x.dtype).to(x.device)
    if x.dtype == torch.float32:  # the reference rounds cos/sin to float32
        c, s = c.float(), s.float()
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def visible(n, window, device="cpu"):
    """[n, n] bool: key j is seen by query i iff j <= i and, with a window, j > i - window.

    The reference's mask is causal only (`gemma/gemma.go:232-240`); the window is
    the architecture's: the last `window` positions, the query's own included.
    """
    i = torch.arange(n, device=device)[:, None]
    j = torch.arange(n, device=device)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & (j > i - window)
    return ok


def softmax_rows(s):
    """max-subtract, exp, sum, divide (`cpu/cpu.go:482-496`)."""
    m = s.max(dim=-1, keepdim=True).values
    e = torch.exp(s - m)
    return e / e.sum(dim=-1, keepdim=True)


def attention(x, wq, wk, wv, wo, n_heads, n_kv, head_dim, rope_base, q_scalar, softcap, window,
              positions=None):
    """Gemma2 attention over one whole sequence (`gemma/gemma.go:66-95`).

    x: [L, H].  Order: project, rotate q and k, scale q by 1/sqrt(query_pre_attn_scalar),
    scores, cap * tanh(scores / cap), mask, softmax, times v, merge heads, output projection.
    """
    L = x.shape[0]
    if positions is None:
        positions = list(range(L))
    q = (x @ wq.to(x.dtype).T).reshape(L, n_heads, head_dim).transpose(0, 1)   # [nh, L, hd]
    k = (x @ wk.to(x.dtype).T).reshape(L, n_kv, head_dim).transpose(0, 1)
    v = (x @ wv.to(x.dtype).T).reshape(L, n_kv, head_dim).transpose(0, 1)
    q = rope(q, positions, rope_base)
    k = rope(k, positions, rope_base)
    q = q * (1.0 / math.sqrt(float(q_scalar)))                                   # gemma.go:62, :76
    rep = n_heads // n_kv
    ok = visible(L, window, x.device)
    out = torch.empty(L, n_heads, head_dim, dtype=x.dtype, device=x.device)
    for h in range(n_heads):
        kv = h // rep                                                            # gemma.go:79-81, cpu_attn.go:72
        s = q[h] @ k[kv].T                                                       # [L, L]
        if softcap and softcap > 0:
            s = softcap * torch.tanh(s / softcap)                                # gemma.go:85
        s = s.masked_fill(~ok, float("-inf"))                                   # gemma.go:86-88
        p = softmax_rows(s)                                                      # gemma.go:89
        out[:, h, :] = p @ v[kv]                                                 # gemma.go:91
    return out.reshape(L, n_heads * head_dim) @ wo.to(x.dtype).T                 # gemma.go:92-94


def gelu_tanh(v):
    """0.5 v (1 + tanh(0.7978845608028654 (v + 0.044715 v^3)))  (`cpu/cpu.go:417-423`)."""
    return 0.5 * v * (1.0 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v * v * v)))


def geglu_mlp(x, wg, wu, wd):
    """down(gelu_tanh(gate(x)) * up(x))  (`gemma/gemma.go:121-123`)."""
    return (gelu_tanh(x @ wg.to(x.dtype).T) * (x @ wu.to(x.dtype).T)) @ wd.to(x.dtype).T


def block(x, w, i, cfg):
    """r = Attn(N_in(x)); h = x + N_postattn(r); r = MLP(N_preff(h)); out = h + N_postff(r)
    (`gemma/gemma.go:162-167`)."""
    p = f"model.layers.{i}."
    eps = cfg.get("rms_norm_eps", 1e-6)
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim", cfg["hidden_size"] // nh)
    window = cfg.get("sliding_window", 4096) if layer_is_sliding(cfg, i) else None
    r = attention(rms_norm(x, w[p + "input_layernorm.weight"], eps),
                  w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                  w[p + "self_attn.v_proj.weight"], w[p + "self_attn.o_proj.weight"],
                  nh, nkv, hd, cfg.get("rope_theta", 10000.0),
                  cfg.get("query_pre_attn_scalar", hd), cfg.get("attn_logit_softcapping", 0.0) or 0.0, window)
    h = x + rms_norm(r, w[p + "post_attention_layernorm.weight"], eps)
    r = geglu_mlp(rms_norm(h, w[p + "pre_feedforward_layernorm.weight"], eps),
                  w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return h + rms_norm(r, w[p + "post_feedforward_layernorm.weight"], eps)


def final_logits(h, w, cfg):
    """final norm, tied head, fc * tanh(logits / fc)  (`gemma/gemma.go:207-212`); all rows."""
    h = rms_norm(h, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    logits = h @ w["model.embed_tokens.weight"].to(h.dtype).T
    fc = cfg.get("final_logit_softcapping", 0.0) or 0.0
    if fc > 0:
        logits = fc * torch.tanh(logits / fc)
    return logits


def forward_logits(cfg, w, ids, dtype=torch.float64):
    """Logits at every position of one sequence: [L, vocab] (`gemma/gemma.go:196-213`)."""
    h = embed(ids, w["model.embed_tokens.weight"], cfg["hidden_size"], dtype)
    for i in range(cfg["num_hidden_layers"]):
        h = block(h, w, i, cfg)
    return final_logits(h, w, cfg)


# ----------------------------------------------------------------------------
# sampling and the loop, on the host in float64
# ----------------------------------------------------------------------------

def apply_repeat_penalty(logits, recent, penalty, last_n):
    """Divide positive / multiply negative logits of recent tokens (`qwen/model.go:60-86`)."""
    logits = logits.clone()
    if penalty <= 1 or not recent:
        return logits
    n = last_n if 0 < last_n <= len(recent) else len(recent)
    for t in set(recent[len(recent) - n:]):
        if 0 <= t < logits.numel():
            logits[t] = logits[t] / penalty if logits[t] > 0 else logits[t] * penalty
    return logits


def nucleus(probs, top_p):
    """Ids kept by top-p: descending probability, ties by lower id, cut where the
    running sum reaches top_p (`qwen/model.go:130-152`, `:461-467`)."""
    order = sorted(range(len(probs)), key=lambda i: (-probs[i], i))
    keep, cum = [], 0.0
    for i in order:
        keep.append(i)
        cum += probs[i]
        if cum >= top_p:
            break
    return keep


def sample_token(logits, temp, top_p, u):
    """Greedy when temp <= 0 (first maximum wins, `qwen/model.go:88-109`); else
    p_i ~ exp((l_i - max) / temp) in float64 (`:111-128`), top-p cut (`:130-152`),
    then the inverse CDF over the kept ids in id order at r = u * kept mass.
    (The reference walks the kept ids in sorted order with Go's generator; the
    distribution is the same, the map from u to an id is this library's.)"""
    l = logits.double()
    if temp <= 0:
        return int((l == l.max()).nonzero()[0].item())
    p = torch.exp((l - l.max()) / float(temp))
    p = (p / p.sum()).tolist()
    if top_p <= 0 or top_p > 1:
        top_p = 1.0
    keep = sorted(nucleus(p, top_p)) if top_p < 1.0 else list(range(len(p)))
    mass = sum(p[i] for i in keep)
    r, acc = u * mass, 0.0
    for i in keep:
        acc += p[i]
        if r <= acc:
            return i
    return keep[-1]


def greedy_generate(cfg, w, prompt, max_tokens, stop=()):
    """prefill, pick, then one token at a time; a stop token ends the reply and is not
    part of it (`qwen/model.go:170-212`, `qwen/session.go:415-427`).  Every token
    re-runs the whole sequence: there is no cache here."""
    ids, out = list(prompt), []
    while True:
        tok = sample_token(forward_logits(cfg, w, ids)[-1], 0.0, 1.0, 0.0)
        if tok in stop:
            return out, "stop"
        out.append(tok)
        ids.append(tok)
        if len(out) >= max_tokens:
            return out, "length"
