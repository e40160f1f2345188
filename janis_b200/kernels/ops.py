"""The hand-written sm_100a kernels as Python functions over torch tensors.

Each function checks on the host what the kernel relies on (device, dtype,
contiguity, shapes, alignment), then passes raw pointers and the current CUDA
stream to the C entry point.  There is no other implementation behind these
names: without a CUDA device, nvcc or the compiled library they raise.

`linear_bf16` is the one place where a library matrix product stands (cuBLAS
through torch, for more than 64 rows), as the reference's engine uses a library
for its products (`engine/backend.go:265-267`, `mlxc/mlxc.go:655`).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from ..csrc import build

PAGE = 64                      # tokens per cache page (JANIS_PAGE in the CUDA sources)
GEMV_MAX_ROWS = 64             # what the skinny kernel accepts
GEMV_FAST_ROWS = 16            # up to here it beats the library product (above, each warp re-reads too much of x)
TC05_MAX_ROWS = 64             # rows the tcgen05 skinny product takes
EPI_NONE, EPI_GATED_GELU, EPI_SOFTCAP, EPI_GATED_SILU = 0, 1, 2, 3
GATE_GROUP = 8                 # fused gate/up rows alternate in groups of 8
ACT_GELU_TANH, ACT_SILU = 0, 1

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


def _need_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("janis_b200 runs on a CUDA device only: torch.cuda.is_available() is False "
                          "and there is no CPU implementation")


_core = None
_attn: dict[int, ctypes.CDLL] = {}


def core():
    global _core
    if _core is None:
        _need_cuda()
        lib = build.core_library()
        P, I, F = c_void_p, c_int, c_float
        lib.janis_embed.argtypes = [P, P, I, P, I, I, I, F, P]
        lib.janis_rmsnorm.argtypes = [P, I, P, P, P, I, I, I, F, P]
        lib.janis_add_rmsnorm.argtypes = [P, P, I, I, c_longlong, P, F, P, F, P, I, I, I, P]
        lib.janis_gated_act.argtypes = [P, P, I, I, I, I, I, P]
        lib.janis_softcap.argtypes = [P, c_longlong, F, P]
        lib.janis_rope_store.argtypes = [P, I, P, P, P, P, P, I, I, I, I, I, I, P, P, P, I, I, I, P]
        lib.janis_kv_store.argtypes = [P, I, P, P, P, P, I, I, I, I, I, P, P, P, I, I, P]
        lib.janis_gemm_f32.argtypes = [P, P, P, I, I, I, F, P]
        lib.janis_gemv_bf16.argtypes = [P, P, P, I, I, I, I, I, F, I, P]
        lib.janis_gemv_rope_store.argtypes = [P, P, P, I, I, P, P, P, P, P, I, I, I, I, P, P, P, I, I, P]
        lib.janis_gemm_tc05.argtypes = [P, P, P, I, I, I, I, I, F, I, P]
        lib.janis_tc05_timeouts.restype = I
        lib.janis_tc05_timeouts_async.argtypes = [P, P]
        lib.janis_tc05_set_stages.argtypes = [I]
        lib.janis_tc05_set_stages.restype = None
        lib.janis_argmax.argtypes = [P, P, I, I, P]
        lib.janis_sample.argtypes = [P, P, P, I, I, F, F, c_ulonglong, P, P, P]
        lib.janis_set_sample_kernel.argtypes = [I]
        lib.janis_set_sample_kernel.restype = None
        lib.janis_repeat_penalty.argtypes = [P, P, I, I, I, F, P]
        lib.janis_mask_tokens.argtypes = [P, P, I, I, I, P]
        lib.janis_set_overlap.argtypes = [I]
        lib.janis_set_overlap.restype = None
        lib.janis_set_overlap(1 if _overlap else 0)
        _core = lib
    return _core


def attention_lib(head_dim: int):
    lib = _attn.get(head_dim)
    if lib is None:
        _need_cuda()
        lib = build.attention_library(head_dim)
        P, I, F = c_void_p, c_int, c_float
        lib.janis_attn_head_dim.restype = I
        lib.janis_attn_decode_scratch.argtypes = [I, I, I]
        lib.janis_attn_decode_scratch.restype = c_longlong
        lib.janis_attn_prefill.argtypes = [P, P, I, P, P, P, P, I, I, I, I, I, I, F, F, I, P, P, P, P, P, I, I, P]
        lib.janis_attn_decode.argtypes = [P, P, P, I, P, I, P, P, P, c_longlong, P, I, I, I, I, F, F, I, I, I, I, P]
        lib.janis_attn_prefill_mma.argtypes = [P, P, I, P, P, I, I, P, I, I, I, I, I, F, F, I, P, c_longlong,
                                               P, P, P, P, P, I, I, I, P]
        lib.janis_attn_set_prefill_kernel.argtypes = [I]
        lib.janis_attn_set_prefill_kernel.restype = None
        lib.janis_attn_set_prefill_piece.argtypes = [I]
        lib.janis_attn_set_prefill_piece.restype = None
        lib.janis_attn_set_decode_wide.argtypes = [I]
        lib.janis_attn_set_decode_wide.restype = None
        lib.janis_attn_set_prefill_items.argtypes = [I]
        lib.janis_attn_set_prefill_items.restype = None
        lib.janis_attn_prefill_kernels.argtypes = []
        lib.janis_attn_prefill_kernels.restype = I
        lib.janis_attn_prefill_piece.argtypes = [I, I, I, I, I, I]
        lib.janis_attn_prefill_piece.restype = I
        lib.janis_attn_tc05_timeouts.restype = I
        lib.janis_attn_timeouts_async.argtypes = [P, P]
        lib.janis_attn_prefill_scratch.argtypes = [I, I]
        lib.janis_attn_prefill_scratch.restype = c_longlong
        lib.janis_attn_prefill_tile.restype = I
        lib.janis_attn_set_decode_kernel.argtypes = [I]
        lib.janis_attn_set_decode_kernel.restype = None
        lib.janis_attn_decode_stages.argtypes = [c_longlong]
        lib.janis_attn_decode_stages.restype = I
        lib.janis_attn_set_decode_stages.argtypes = [I]
        lib.janis_attn_set_decode_stages.restype = None
        lib.janis_attn_wait_timeouts.restype = I
        lib.janis_attn_wait_probe.argtypes = [I, P, P]
        lib.janis_attn_set_overlap.argtypes = [I]
        lib.janis_attn_set_overlap.restype = None
        lib.janis_attn_set_overlap(1 if _overlap else 0)
        if lib.janis_attn_head_dim() != head_dim:
            raise KernelError(f"attention library for head size {head_dim} reports {lib.janis_attn_head_dim()}")
        _attn[head_dim] = lib
    return lib


_overlap = os.environ.get("JANIS_OVERLAP", "1") != "0"


def set_overlap(on: bool) -> None:
    """Whether a kernel's CTAs may arrive while the kernel before it in the stream still runs
    (programmatic dependent launch; every kernel waits for its predecessor before it touches
    anything but weights and the step's tables).  Results are the same either way."""
    global _overlap
    _overlap = bool(on)
    if _core is not None:
        _core.janis_set_overlap(1 if _overlap else 0)
    for lib in _attn.values():
        lib.janis_attn_set_overlap(1 if _overlap else 0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  (A prompt step launches some three hundred kernels from Python; building a
    Stream object for each took a fifth of the step's host time.)"""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launch_count() -> int:
    """How many of this library's kernels have been launched (or recorded into a graph) so far."""
    return _launches


def _check(lib, rc: int, kernels: int = 1) -> None:
    global _launches
    if rc != 0:
        raise KernelError(lib.janis_last_error().decode("utf-8", "replace"))
    _launches += kernels


def _t(x: torch.Tensor, name: str, dtype=None, shape=None) -> int:
    """The address of a tensor an entry point is given, after the checks the C side cannot make: on the device,
    contiguous, of an accepted dtype (one, or a tuple), of the wanted shape (None: any extent)."""
    try:
        if not x.is_cuda:
            raise KernelError(f"{name}: expected a CUDA tensor")
    except AttributeError:
        raise KernelError(f"{name}: expected a CUDA tensor") from None
    if not x.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")
    if dtype is not None:
        xd = x.dtype
        if xd != dtype and not (type(dtype) in (tuple, list) and xd in dtype):
            raise KernelError(f"{name}: dtype {xd} not accepted here (wanted {dtype})")
    if shape is not None:
        xs = x.shape
        bad = len(xs) != len(shape)
        if not bad:
            for want, have in zip(shape, xs):
                if want is not None and want != have:
                    bad = True
                    break
        if bad:
            raise KernelError(f"{name}: shape {tuple(xs)} does not match {tuple(shape)}")
    return x.data_ptr()


_FLOATS = (torch.float32, torch.bfloat16)

# ---------------------------------------------------------------------------
# rows of the residual stream
# ---------------------------------------------------------------------------

def embed(tokens, table, scale: float, out):
    """out[t] = float(table[tokens[t]]) * scale;  tokens int32 [T], table [V, H], out float32 [T, H]."""
    T = tokens.numel()
    V, H = table.shape
    lib = core()
    _check(lib, lib.janis_embed(_t(tokens, "tokens", torch.int32), _t(table, "table", _FLOATS), _DT[table.dtype],
                                _t(out, "out", torch.float32, (T, H)), T, H, V, float(scale), _stream()))
    return out


def rmsnorm(x, weight, eps: float, out, rows=None):
    """out[r] = x[rows[r] or r] / sqrt(mean(x^2) + eps) * weight;  weight float32 holds offset + w."""
    H = x.shape[-1]
    R = out.shape[0]
    if rows is None and x.shape[0] != R:
        raise KernelError(f"rmsnorm: {x.shape[0]} input rows for {R} output rows")
    lib = core()
    _check(lib, lib.janis_rmsnorm(_t(x, "x", _FLOATS, (None, H)), _DT[x.dtype], _t(weight, "weight", torch.float32, (H,)),
                                  _t(rows, "rows", torch.int32, (R,)) if rows is not None else None,
                                  _t(out, "out", _FLOATS, (R, H)), _DT[out.dtype], R, H, float(eps), _stream()))
    return out


def add_rmsnorm(h, res, w_post, eps_post, w_next=None, eps_next=0.0, out=None, n_part=1):
    """h += norm(res; w_post) in place (float32 residual sum; h += res when w_post is None);
    out = norm(h; w_next) when w_next is given.
    `res` is [R, H], or [n_part, R, H] partial results that are added first."""
    R, H = h.shape
    if n_part == 1:
        _t(res, "res", _FLOATS, (R, H))
        stride = 0
    else:
        _t(res, "res", _FLOATS, (n_part, R, H))
        stride = R * H
    lib = core()
    _check(lib, lib.janis_add_rmsnorm(
        _t(h, "h", torch.float32, (R, H)), res.data_ptr(), _DT[res.dtype], n_part, stride,
        _t(w_post, "w_post", torch.float32, (H,)) if w_post is not None else None, float(eps_post),
        _t(w_next, "w_next", torch.float32, (H,)) if w_next is not None else None, float(eps_next),
        _t(out, "out", _FLOATS, (R, H)) if out is not None else None,
        _DT[out.dtype] if out is not None else 0, R, H, _stream()))
    return out


def gated_act(gu, out, act: int = ACT_GELU_TANH, group: int = GATE_GROUP):
    """out[r, j] = act(gate) * up over a fused [R, 2I] product whose columns alternate
    `group` gate columns and `group` up columns."""
    R, I2 = gu.shape
    I = I2 // 2
    lib = core()
    _check(lib, lib.janis_gated_act(_t(gu, "gu", _FLOATS, (R, 2 * I)), _t(out, "out", gu.dtype, (R, I)),
                                    _DT[gu.dtype], R, I, group, act, _stream()))
    return out


def rope_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, rot: int, nq: int, nkv: int, hd: int,
               kpool=None, vpool=None, page_table=None, ring_len: int = 0, store: bool = True,
               write_cache: bool = True):
    """Rotate q and k of qkv [T, heads, hd] (heads = q, then k, then v) in place and write k and v into
    the paged cache.

    kpool/vpool: [pages, nkv, PAGE, hd] of one cache line; page_table int32 [slots, pages per sequence].
    With store=False the rows hold q alone and only q is rotated (a layer that reads another layer's
    keys).  With write_cache=False q and k are rotated and nothing is stored (`kv_store` does it later)."""
    T = qkv.shape[0]
    row_heads = nq + 2 * nkv if store else nq
    _t(qkv, "qkv", _FLOATS, (T, row_heads, hd))
    _t(tok_pos, "tok_pos", torch.int32)
    _t(tok_seq, "tok_seq", torch.int32)
    if tok_pos.numel() < T or tok_seq.numel() < T:
        raise KernelError("rope_store: position tables shorter than the step")
    _t(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    stride = 0
    if store and not write_cache:
        lib = core()
        _check(lib, lib.janis_rope_store(qkv.data_ptr(), _DT[qkv.dtype], tok_pos.data_ptr(), tok_seq.data_ptr(), None,
                                         None, inv_freq.data_ptr(), rot, T, nq, nkv, hd, row_heads, None, None, None,
                                         0, 0, 0, _stream()))
        return qkv
    if store:
        n_pages = kpool.shape[0]
        _t(kpool, "kpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
        _t(vpool, "vpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
        _t(page_table, "page_table", torch.int32, (None, None))
        _t(seq_slot, "seq_slot", torch.int32)
        _t(seq_end, "seq_end", torch.int32)
        stride = page_table.shape[1]
    lib = core()
    _check(lib, lib.janis_rope_store(
        qkv.data_ptr(), _DT[qkv.dtype], tok_pos.data_ptr(), tok_seq.data_ptr(),
        seq_slot.data_ptr() if store else None, seq_end.data_ptr() if store else None,
        inv_freq.data_ptr(), rot, T, nq, nkv, hd, row_heads,
        kpool.data_ptr() if store else None, vpool.data_ptr() if store else None,
        page_table.data_ptr() if store else None, stride, ring_len, 0 if store else 1, _stream()))
    return qkv


def kv_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, nq: int, nkv: int, hd: int, kpool, vpool, page_table,
             ring_len: int = 0):
    """Write the keys and values of qkv [T, nq + 2 nkv, hd] into the paged cache line as they stand (the places
    and the rule for rings are rope_store's): the second half of `rope_store(..., write_cache=False)`."""
    T = qkv.shape[0]
    _t(qkv, "qkv", _FLOATS, (T, None, hd))
    if qkv.shape[1] < nq + 2 * nkv:
        raise KernelError("kv_store: the rows of qkv hold no keys and values")
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
    _t(vpool, "vpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
    _t(page_table, "page_table", torch.int32, (None, None))
    if tok_pos.numel() < T or tok_seq.numel() < T:
        raise KernelError("kv_store: position tables shorter than the step")
    lib = core()
    _check(lib, lib.janis_kv_store(qkv.data_ptr(), _DT[qkv.dtype], _t(tok_pos, "tok_pos", torch.int32),
                                   _t(tok_seq, "tok_seq", torch.int32), _t(seq_slot, "seq_slot", torch.int32),
                                   _t(seq_end, "seq_end", torch.int32), T, nq, nkv, hd, qkv.shape[1], kpool.data_ptr(),
                                   vpool.data_ptr(), page_table.data_ptr(), page_table.shape[1], int(ring_len), _stream()))
    return qkv


# ---------------------------------------------------------------------------
# products
# ---------------------------------------------------------------------------

def gemm_f32(x, w, out, cap: float = 0.0):
    """out[M, N] = x[M, K] w[N, K]^T in true float32 (CUDA cores); optional cap * tanh(v / cap)."""
    M, K = x.shape
    N = w.shape[0]
    lib = core()
    _check(lib, lib.janis_gemm_f32(_t(x, "x", torch.float32, (M, K)), _t(w, "w", torch.float32, (N, K)),
                                   _t(out, "out", torch.float32, (M, N)), M, N, K, float(cap), _stream()))
    return out


def gemv_bf16(x, w, out, epilogue: int = EPI_NONE, cap: float = 0.0, cluster: int = 0):
    """out = x[M<=64, K] w[N, K]^T, bfloat16 operands, float accumulation; out bfloat16 or float32
    [M, N], or [M, N/2] with a gated epilogue (rows of w alternate 8 gate rows and 8 up rows).
    cluster: how many CTAs of a thread-block cluster share the K of a tile (1, 2, 4; 0 = chosen from N, K)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue in (EPI_GATED_GELU, EPI_GATED_SILU) else N
    lib = core()
    _check(lib, lib.janis_gemv_bf16(_t(x, "x", torch.bfloat16, (M, K)), _t(w, "w", torch.bfloat16, (N, K)),
                                    _t(out, "out", _FLOATS, (M, n_out)), _DT[out.dtype], M, N, K, epilogue,
                                    float(cap), int(cluster), _stream()))
    return out


def gemv_rope_store(x, w, qkv, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, nq: int, nkv: int, hd: int,
                    kpool=None, vpool=None, page_table=None, ring_len: int = 0, store: bool = True):
    """The q/k/v projection of up to 16 decode rows with the rotary encoding of the whole head and the cache write
    in its epilogue: what `gemv_bf16(x, w, qkv)` followed by `rope_store(qkv, ...)` leaves in the queries' part
    of qkv [M, heads, hd] and in the cache line, in one kernel (the keys' and values' part of qkv is not written).
    w: [(nq + 2 nkv) hd, K], or [nq hd, K] with store=False (a layer that reads another layer's keys)."""
    M, K = x.shape
    heads = nq + 2 * nkv if store else nq
    _t(x, "x", torch.bfloat16, (M, K))
    _t(w, "w", torch.bfloat16, (heads * hd, K))
    _t(qkv, "qkv", torch.bfloat16, (M, None, hd))
    if qkv.shape[1] < nq:
        raise KernelError("gemv_rope_store: the rows of qkv hold fewer heads than nq")
    _t(tok_pos, "tok_pos", torch.int32)
    _t(tok_seq, "tok_seq", torch.int32)
    if tok_pos.numel() < M or tok_seq.numel() < M:
        raise KernelError("gemv_rope_store: position tables shorter than the step")
    _t(inv_freq, "inv_freq", torch.float32, (hd // 2,))
    stride = 0
    if store:
        n_pages = kpool.shape[0]
        _t(kpool, "kpool", torch.bfloat16, (n_pages, nkv, PAGE, hd))
        _t(vpool, "vpool", torch.bfloat16, (n_pages, nkv, PAGE, hd))
        _t(page_table, "page_table", torch.int32, (None, None))
        _t(seq_slot, "seq_slot", torch.int32)
        _t(seq_end, "seq_end", torch.int32)
        stride = page_table.shape[1]
    lib = core()
    _check(lib, lib.janis_gemv_rope_store(
        x.data_ptr(), w.data_ptr(), qkv.data_ptr(), M, K, tok_pos.data_ptr(), tok_seq.data_ptr(),
        seq_slot.data_ptr() if store else None, seq_end.data_ptr() if store else None, inv_freq.data_ptr(),
        nq, nkv, hd, qkv.shape[1], kpool.data_ptr() if store else None, vpool.data_ptr() if store else None,
        page_table.data_ptr() if store else None, stride, ring_len, _stream()))
    return qkv


def softcap(x, cap: float):
    """x = cap * tanh(x / cap) in place, float32."""
    lib = core()
    _check(lib, lib.janis_softcap(_t(x, "x", torch.float32), x.numel(), float(cap), _stream()))
    return x


def gemm_tc05(x, w, out, epilogue: int = EPI_NONE, cap: float = 0.0, split: int = 0):
    """out = x[M<=64, K] w[N, K]^T on the tcgen05 tensor cores (operands swapped: rows of w fill the 128 TMEM
    lanes, the batch rows are the narrow side), TMA-fed, K split over a cluster when N is small.  Same
    epilogues and output shapes as gemv_bf16.  split: CTAs that share K (1, 2, 4, 8; 0 = chosen from N, K)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue in (EPI_GATED_GELU, EPI_GATED_SILU) else N
    lib = core()
    _check(lib, lib.janis_gemm_tc05(_t(x, "x", torch.bfloat16, (M, K)), _t(w, "w", torch.bfloat16, (N, K)),
                                    _t(out, "out", _FLOATS, (M, n_out)), _DT[out.dtype], M, N, K, epilogue,
                                    float(cap), int(split), _stream()))
    return out


def tc05_set_stages(stages: int = 0) -> None:
    """Fix the depth of the tcgen05 product's ring of stages (3 to 9; 0: chosen from the CTAs per SM, the default).
    For tests and tuning."""
    core().janis_tc05_set_stages(int(stages))


def tc05_timeouts() -> int:
    """How often a CTA of gemm_tc05 gave up waiting on a barrier (0 in a healthy run); synchronises."""
    return int(core().janis_tc05_timeouts())


class WaitWatch:
    """Notices when a kernel has given up one of its bounded waits (on a barrier of its copies or of its tensor-core
    products): such a CTA returns without its result, and what the step produced is then worthless.

    `request()` asks every loaded library, in the order of the current stream and without waiting, to copy its
    counters of given-up waits into pinned host memory; `check()`, called once the host has waited for that
    stream anyway (to read the step's tokens), raises `KernelError` if a counter has grown since the last
    check.  Counters of libraries loaded later join at their next request."""

    def __init__(self):
        self._host = torch.zeros(64, dtype=torch.int32).pin_memory()
        self._where: dict[str, int] = {}           # library -> index of its first counter
        self._seen = [0] * 64

    def _slot(self, name: str) -> int:              # two counters a library (core: the tcgen05 product's waits, the clusters' of the skinny products)
        if name not in self._where:
            if 2 * len(self._where) + 2 > 64:
                raise KernelError("too many attention libraries for one watch")
            self._where[name] = 2 * len(self._where)
        return self._where[name]

    def request(self) -> None:
        st, base = _stream(), self._host.data_ptr()
        if _core is not None:
            _check(_core, _core.janis_tc05_timeouts_async(base + 4 * self._slot("core"), st), 0)
        for hd, lib in _attn.items():
            _check(lib, lib.janis_attn_timeouts_async(base + 4 * self._slot(f"attention (head size {hd})"), st), 0)

    def check(self, quiet: bool = False) -> None:
        """Call after the stream of the last `request()` has been waited for (quiet: take note, raise nothing)."""
        now = self._host.tolist()
        grown = [(name, now[at + i] - self._seen[at + i]) for name, at in self._where.items() for i in range(2)
                 if now[at + i] > self._seen[at + i]]
        self._seen = now
        if grown and not quiet:
            what = ", ".join(f"{n} in {name}" for name, n in grown)
            raise KernelError(f"a kernel gave up a bounded wait ({what}): the results of the steps since the last "
                              "check are not to be trusted")


def linear_bf16(x, w, out):
    """out[M, N] = x w^T in bfloat16 with float accumulation: the skinny kernel up to 16 rows,
    the library product (cuBLAS) above."""
    M = x.shape[0]
    if M <= GEMV_FAST_ROWS:
        return gemv_bf16(x, w, out)
    _t(x, "x", torch.bfloat16)
    _t(w, "w", torch.bfloat16)
    _t(out, "out", torch.bfloat16, (M, w.shape[0]))
    torch.mm(x, w.t(), out=out)
    return out


def matmul_bf16_to_f32(x, w, out):
    """out[M, N] float32 = x[M, K] w[N, K]^T, bfloat16 operands, the library product (cuBLAS)."""
    _t(x, "x", torch.bfloat16)
    _t(w, "w", torch.bfloat16)
    _t(out, "out", torch.float32, (x.shape[0], w.shape[0]))
    torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    return out


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------

def attn_prefill_scratch_floats(n_tok: int, n_seq: int, nq: int, hd: int, dtype=torch.bfloat16) -> int:
    """Floats of scratch that attn_prefill wants for a step of n_tok tokens in n_seq sequences: a bfloat16
    step with few tiles of queries shares each long tile between up to four CTAs, which meet through the scratch
    (0: nothing is shared).  Without the scratch the step runs unshared."""
    if dtype != torch.bfloat16:
        return 0
    lib = attention_lib(hd)
    bm = lib.janis_attn_prefill_tile()
    return int(lib.janis_attn_prefill_scratch((n_tok + bm - 1) // bm + n_seq, nq))


def _cached_args(name, seq_start, seq_slot, kpool, vpool, page_table, ring_len, dtype, n_seq, nkv, hd):
    """The arguments that say where the keys and values of earlier steps are (all null for a step whose sequences
    start at position 0)."""
    if seq_start is None:
        return (None, None, None, None, None, 0, 0)
    if kpool is None or vpool is None or page_table is None or seq_slot is None:
        raise KernelError(f"{name}: sequences that continue need their slots and the cache line")
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", dtype, (n_pages, nkv, PAGE, hd))
    _t(vpool, "vpool", dtype, (n_pages, nkv, PAGE, hd))
    _t(page_table, "page_table", torch.int32, (None, None))
    _t(seq_start, "seq_start", torch.int32)
    _t(seq_slot, "seq_slot", torch.int32)
    if n_seq is not None and (seq_start.numel() < n_seq or seq_slot.numel() < n_seq):
        raise KernelError(f"{name}: sequence tables shorter than the step")
    return (seq_start.data_ptr(), seq_slot.data_ptr(), kpool.data_ptr(), vpool.data_ptr(), page_table.data_ptr(),
            page_table.shape[1], int(ring_len))


def attn_prefill(qkv, tok_pos, tok_seq, seq_first_row, out, nq: int, nkv: int, hd: int, scale: float, cap: float,
                 window: int, kv_src=None, kv_row_heads=None, kv_k_head0=None, seq_len=None, tensor_cores=True,
                 scratch=None, seq_start=None, seq_slot=None, kpool=None, vpool=None, page_table=None,
                 ring_len: int = 0, host_lens=None):
    """Causal (and windowed when window > 0) attention over packed sequences.
    qkv: [T, nq + 2 nkv, hd], or [T, nq, hd] when keys and values come from `kv_src`, another layer's
    [T, kv_row_heads, hd] rows whose key heads start at head kv_k_head0 (values nkv heads later).
    Without `seq_start` every sequence starts at position 0 and seq_first_row is the row of that position.  With
    `seq_start` (int32 [n_seq], the tokens earlier steps stored) the step continues sequences: tok_pos are absolute
    positions, seq_first_row is the row of a sequence's first token of this step, `seq_len` the lengths after the
    step, and the keys and values of earlier positions are read from the cache line (kpool, vpool, page_table,
    ring_len), which must still hold what those steps left (this step's own keys are stored afterwards).
    `host_lens`: the tokens each sequence brings to this step, if the host knows them (a step replayed from a graph
    with other lengths does not): the grid then has no places to spare.
    bfloat16 with `seq_len` (int32 [n_seq]) runs on the tensor cores; float32 runs the CUDA-core kernel, which is
    exact 32-bit."""
    T = qkv.shape[0]
    if qkv.dtype == torch.bfloat16 and seq_len is not None and tensor_cores:
        return _attn_prefill_mma(qkv, seq_first_row, seq_len, out, nq, nkv, hd, scale, cap, window, kv_src,
                                 kv_row_heads, kv_k_head0, scratch,
                                 (seq_start, seq_slot, kpool, vpool, page_table, ring_len), host_lens)
    if kv_src is None:
        _t(qkv, "qkv", _FLOATS, (T, nq + 2 * nkv, hd))
        kv_src, kv_row_heads, kv_k_head0 = qkv, nq + 2 * nkv, nq
    else:
        _t(qkv, "qkv", _FLOATS, (T, None, hd))
        if qkv.shape[1] < nq:
            raise KernelError("attn_prefill: query rows hold fewer heads than nq")
    q_row_heads = qkv.shape[1]
    _t(kv_src, "kv_src", qkv.dtype, (T, kv_row_heads, hd))
    if kv_k_head0 + 2 * nkv > kv_row_heads:
        raise KernelError("attn_prefill: key/value heads lie outside the rows of kv_src")
    _t(out, "out", qkv.dtype, (T, nq * hd))
    cached = _cached_args("attn_prefill", seq_start, seq_slot, kpool, vpool, page_table, ring_len, qkv.dtype,
                          seq_first_row.numel(), nkv, hd)
    lib = attention_lib(hd)
    _check(lib, lib.janis_attn_prefill(qkv.data_ptr(), kv_src.data_ptr(), _DT[qkv.dtype],
                                       _t(tok_pos, "tok_pos", torch.int32), _t(tok_seq, "tok_seq", torch.int32),
                                       _t(seq_first_row, "seq_first_row", torch.int32), out.data_ptr(), T, nq, nkv,
                                       q_row_heads, kv_row_heads, kv_k_head0, float(scale), float(cap),
                                       int(window), *cached, _stream()))
    return out


def _attn_prefill_mma(qkv, seq_first_row, seq_len, out, nq, nkv, hd, scale, cap, window, kv_src, kv_row_heads,
                      kv_k_head0, scratch=None, cached=(None,) * 5 + (0,), host_lens=None):
    T = qkv.shape[0]
    if kv_src is None:
        _t(qkv, "qkv", torch.bfloat16, (T, nq + 2 * nkv, hd))
        kv_src, kv_row_heads, kv_k_head0 = qkv, nq + 2 * nkv, nq
    else:
        _t(qkv, "qkv", torch.bfloat16, (T, None, hd))
        if qkv.shape[1] < nq:
            raise KernelError("attn_prefill: query rows hold fewer heads than nq")
    _t(kv_src, "kv_src", torch.bfloat16, (T, kv_row_heads, hd))
    if kv_k_head0 + 2 * nkv > kv_row_heads:
        raise KernelError("attn_prefill: key/value heads lie outside the rows of kv_src")
    _t(out, "out", torch.bfloat16, (T, nq * hd))
    n_seq = seq_len.numel()
    _t(seq_len, "seq_len", torch.int32, (n_seq,))
    _t(seq_first_row, "seq_first_row", torch.int32, (n_seq,))
    cached = _cached_args("attn_prefill", *cached, torch.bfloat16, n_seq, nkv, hd)
    lib = attention_lib(hd)
    bm = lib.janis_attn_prefill_tile()      # queries per CTA
    if host_lens is not None:               # the tokens each sequence brings, when the host knows them: no places to spare
        if len(host_lens) != n_seq or sum(host_lens) > T:
            raise KernelError(f"attn_prefill: host_lens {list(host_lens)} do not fit {n_seq} sequences of {T} tokens")
        tiles = sum((int(n) + bm - 1) // bm for n in host_lens)
    else:
        tiles = (T + bm - 1) // bm + n_seq  # >= sum of ceil(len / bm)
    need = int(lib.janis_attn_prefill_scratch(tiles, nq))
    if scratch is not None and (need == 0 or scratch.numel() < need):
        scratch = None
    _check(lib, lib.janis_attn_prefill_mma(qkv.data_ptr(), kv_src.data_ptr(), T, seq_first_row.data_ptr(),
                                           seq_len.data_ptr(), n_seq, tiles, out.data_ptr(), nq, nkv,
                                           qkv.shape[1], kv_row_heads, kv_k_head0, float(scale), float(cap),
                                           int(window), _t(scratch, "scratch", torch.float32) if scratch is not None else None,
                                           scratch.numel() if scratch is not None else 0, *cached,
                                           max(int(n) for n in host_lens) if host_lens else 0, _stream()))
    global _launches
    _launches += int(lib.janis_attn_prefill_kernels()) - 1     # the merge, when tiles were shared
    return out


def attn_set_prefill_kernel(hd: int, which: int = 1) -> None:
    """Choose the bfloat16 prompt kernel of the head size's library: 1 = tcgen05 with the accumulators in
    tensor memory where the head size allows it (a multiple of 64 up to 256; the default), in the form that suits
    the step's size; 2 = always a CTA per tile of queries and head; 3 = always CTAs that stay and take one tile of
    queries after another; 0 = mma.sync."""
    lib = attention_lib(hd)
    lib.janis_attn_set_prefill_kernel(1 if which else 0)
    lib.janis_attn_set_prefill_items({2: 0, 3: 2}.get(which, 1))


def attn_set_prefill_piece(hd: int, piece: int = 0) -> None:
    """Fix how many key tiles a piece of a shared tile of queries holds in the bfloat16 prompt kernels of the
    head size's library (0: chosen from the step's size, the default).  For tests and tuning."""
    attention_lib(hd).janis_attn_set_prefill_piece(int(piece))


def attn_prefill_piece(hd: int, n_tok: int, n_seq: int, nq: int, window: int = 0, tc05: bool = True) -> int:
    """The piece (in key tiles) that a prompt step of these sizes would cut its shared tiles of queries into."""
    lib = attention_lib(hd)
    bm = int(lib.janis_attn_prefill_tile())
    return int(lib.janis_attn_prefill_piece(n_tok, n_seq, (n_tok + bm - 1) // bm + n_seq, nq, window, 1 if tc05 else 0))


def attn_tc05_timeouts(hd: int) -> int:
    """How often a CTA of the tcgen05 prompt kernel has given up a wait (0 unless something is badly wrong)."""
    return int(attention_lib(hd).janis_attn_tc05_timeouts())


def attn_set_decode_wide(hd: int, on: bool = True) -> None:
    """Whether the tensor-core decode kernel of a head size above 128 takes stages of 64 keys in launches of no more
    CTAs than SMs (the default) or stages of 32 keys always.  For tests and tuning."""
    attention_lib(hd).janis_attn_set_decode_wide(1 if on else 0)


def attn_set_decode_kernel(hd: int, which: int = 2) -> None:
    """Choose the decode kernel of the head size's library: 2 = staged by bulk copies with the scores on the
    tensor cores (bfloat16 and head sizes <= 256; the default), 1 = staged, CUDA cores (also what float32
    runs), 0 = straight from global memory into registers."""
    attention_lib(hd).janis_attn_set_decode_kernel(int(which))
    _decode_kernel[hd] = int(which)


def attn_decode_resident(hd: int, dtype, n_ctas: int, sm_count: int) -> int:
    """CTAs of a decode-attention launch of n_ctas CTAs that the GPU holds at once: the bfloat16 tensor-core kernel
    runs with two stages and three CTAs an SM when a launch has more CTAs than two an SM would hold, else with three
    stages and two CTAs an SM; the other kernels hold two."""
    if dtype == torch.bfloat16 and hd <= 256 and _decode_kernel.get(hd, 2) == 2:
        return (3 if attention_lib(hd).janis_attn_decode_stages(int(n_ctas)) == 2 else 2) * sm_count
    return 2 * sm_count


def attn_set_decode_stages(hd: int, stages: int = 0) -> None:
    """Fix the stages of the bfloat16 tensor-core decode kernel (2 or 3; 0: chosen per launch, the default).  For tests."""
    attention_lib(hd).janis_attn_set_decode_stages(int(stages))


def attn_wait_timeouts(hd: int) -> int:
    """How often a decode CTA gave up waiting for its bulk copies (0 in a healthy run); synchronises."""
    return int(attention_lib(hd).janis_attn_wait_timeouts())


def attn_wait_probe(hd: int, tries: int = 64) -> int:
    """Runs the kernels' bounded wait on a barrier that nothing completes: returns 1 when the wait gave up
    (as it must) and the kernel returned.  Raises the library's counter of timeouts by one."""
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = attention_lib(hd)
    _check(lib, lib.janis_attn_wait_probe(int(tries), status.data_ptr(), _stream()))
    return int(status.item())


def attn_decode_scratch_floats(n_seq: int, nq: int, hd: int, max_chunks: int) -> int:
    return n_seq * nq * max_chunks * (hd + 2)


_decode_kernel: dict[int, int] = {}      # head size -> kernel chosen for tests (default 2)


def attn_decode(qkv, kpool, vpool, page_table, seq_slot, seq_len, scratch, out, nq: int, nkv: int, hd: int,
                scale: float, cap: float, window: int, ring_len: int, chunk: int, max_chunks: int):
    """One query per sequence over the paged cache.  qkv: [n_seq, heads >= nq, hd] with q first;
    seq_len counts the new token; scratch is float32.  The chunks of a sequence are merged by a second
    kernel; a launch of one chunk per sequence (max_chunks == 1) on the bfloat16 tensor-core kernel
    writes the result itself."""
    n_seq = qkv.shape[0]
    _t(qkv, "qkv", _FLOATS, (n_seq, None, hd))
    if qkv.shape[1] < nq:
        raise KernelError("attn_decode: query rows hold fewer heads than nq")
    n_pages = kpool.shape[0]
    _t(kpool, "kpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
    _t(vpool, "vpool", qkv.dtype, (n_pages, nkv, PAGE, hd))
    _t(page_table, "page_table", torch.int32, (None, None))
    _t(scratch, "scratch", torch.float32)
    _t(out, "out", qkv.dtype, (n_seq, nq * hd))
    if seq_slot.numel() < n_seq or seq_len.numel() < n_seq:
        raise KernelError("attn_decode: sequence tables shorter than the batch")
    lib = attention_lib(hd)
    direct = max_chunks == 1 and qkv.dtype == torch.bfloat16 and hd <= 256 and _decode_kernel.get(hd, 2) == 2
    _check(lib, lib.janis_attn_decode(qkv.data_ptr(), kpool.data_ptr(), vpool.data_ptr(), _DT[qkv.dtype],
                                      page_table.data_ptr(), page_table.shape[1],
                                      _t(seq_slot, "seq_slot", torch.int32), _t(seq_len, "seq_len", torch.int32),
                                      scratch.data_ptr(), scratch.numel(), out.data_ptr(), n_seq, nq, nkv,
                                      qkv.shape[1], float(scale), float(cap), int(window), int(ring_len),
                                      int(chunk), int(max_chunks), _stream()), kernels=1 if direct else 2)
    return out


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------

def argmax(logits, out):
    R, V = logits.shape
    lib = core()
    _check(lib, lib.janis_argmax(_t(logits, "logits", torch.float32), _t(out, "out", torch.int32, (R,)), R, V,
                                 _stream()))
    return out


def sample(logits, out, temp: float, top_p: float, seed: int, request_ids, token_index, u_out=None):
    R, V = logits.shape
    lib = core()
    _check(lib, lib.janis_sample(_t(logits, "logits", torch.float32), _t(out, "out", torch.int32, (R,)),
                                 _t(u_out, "u_out", torch.float32, (R,)) if u_out is not None else None, R, V,
                                 float(temp), float(top_p), int(seed) & 0xFFFFFFFFFFFFFFFF,
                                 _t(request_ids, "request_ids", torch.int32, (R,)),
                                 _t(token_index, "token_index", torch.int32, (R,)), _stream()))
    return out


def set_sample_kernel(which: int = 1) -> None:
    """Choose the kernel behind `sample`: 1 = the row's weights held in the shared memory of a cluster of up to 8
    CTAs (vocabularies up to about 368,000; the default), 0 = every pass over global memory (any vocabulary).
    For tests."""
    core().janis_set_sample_kernel(int(which))


def repeat_penalty(logits, recent, penalty: float):
    R, V = logits.shape
    lib = core()
    _check(lib, lib.janis_repeat_penalty(_t(logits, "logits", torch.float32), _t(recent, "recent", torch.int32, (R, None)),
                                         recent.shape[1], R, V, float(penalty), _stream()))
    return logits


def mask_tokens(logits, ids):
    R, V = logits.shape
    lib = core()
    _check(lib, lib.janis_mask_tokens(_t(logits, "logits", torch.float32), _t(ids, "ids", torch.int32), ids.numel(),
                                      R, V, _stream()))
    return logits
