"""The decode-attention entry point that allocates nothing (janis_attn_decode_static).

Some users of the compiled library cannot allocate device memory when they call it: a
host written in another language that reaches the kernels through the exported C symbols
has no tensor allocator to ask, and a serving process that gave all device memory to its
weights and cache at start-up cannot risk a cudaMalloc inside a step.  For them the
library keeps the scratch of decode attention in a static device array.  This test calls
that entry point the way such a caller does, through the exported C symbol with raw
pointers, and checks it against the ordinary entry point (which takes a scratch tensor)
and against the plain statement of decode attention in tests/kernel_refs.py, on two calls
in a row: the second call finds the array as the first one left it.  It also checks that
the array's memory is taken once (the first call on the device) and never again, that the
largest request that fits is served and the next larger one refused, and the call that
needs no scratch at all (one chunk per sequence in bfloat16).

Collected last on purpose (pytest orders files by name), so that a run that stops at the
first failure has run every other test before this one.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_FLOATS = 2 * 1024 * 1024      # JANIS_STATIC_SCRATCH_FLOATS in attention_no_alloc.h
HD = 32
PAGE = 64


def _library():
    """The attention library for head size HD, with the new symbol typed."""
    from janis_b200.kernels import ops
    lib = ops.attention_lib(HD)
    P, I, F = c_void_p, c_int, c_float
    lib.janis_attn_decode_static.argtypes = [P, P, P, I, P, I, P, P, P, I, I, I, I, F, F, I, I, I, I, P]
    lib.janis_attn_decode_static.restype = c_int
    return ops, lib


def _case(seed, dtype, lens, slots, nq, nkv, n_pages=24, pages_per_seq=5):
    g = torch.Generator().manual_seed(seed)
    d = torch.device("cuda:0")
    k = torch.randn((n_pages, nkv, PAGE, HD), generator=g).to(dtype).to(d)
    v = torch.randn((n_pages, nkv, PAGE, HD), generator=g).to(dtype).to(d)
    qkv = torch.randn((len(lens), nq + 2 * nkv, HD), generator=g).to(dtype).to(d)
    table = torch.randperm(n_pages, generator=g)[: len(lens) * pages_per_seq].view(len(lens), pages_per_seq).int().to(d)
    return dict(qkv=qkv, k=k, v=v, table=table,
                seq_slot=torch.tensor(slots, dtype=torch.int32, device=d),
                seq_len=torch.tensor(lens, dtype=torch.int32, device=d))


def _geometry(c, chunk):
    lens = c["seq_len"].tolist()
    return max((n + chunk - 1) // chunk for n in lens), 1.0 / math.sqrt(HD), 25.0


def _ordinary(ops, c, nq, nkv, window, ring, chunk):
    """The existing entry point (with a scratch tensor) and the plain statement of the same computation."""
    from tests import kernel_refs
    d = c["qkv"].device
    n_seq = c["qkv"].shape[0]
    max_chunks, scale, cap = _geometry(c, chunk)
    want = torch.empty((n_seq, nq * HD), dtype=c["qkv"].dtype, device=d)
    scratch = torch.empty(ops.attn_decode_scratch_floats(n_seq, nq, HD, max_chunks), dtype=torch.float32, device=d)
    ops.attn_decode(c["qkv"], c["k"], c["v"], c["table"], c["seq_slot"], c["seq_len"], scratch, want, nq, nkv, HD,
                    scale, cap, window, ring, chunk, max_chunks)
    plain = torch.empty((n_seq, nq * HD), dtype=torch.float64)
    kernel_refs.attn_decode(c["qkv"].cpu(), c["k"].cpu(), c["v"].cpu(), c["table"].cpu(), c["seq_slot"].cpu(),
                            c["seq_len"].cpu(), None, plain, nq, nkv, HD, scale, cap, window, ring, chunk, max_chunks)
    return want, plain


def _static(lib, c, got, nq, nkv, window, ring, chunk):
    """The new entry point, as a caller without an allocator reaches it: raw pointers through the C symbol."""
    max_chunks, scale, cap = _geometry(c, chunk)
    rc = lib.janis_attn_decode_static(
        c["qkv"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), 0 if c["qkv"].dtype == torch.float32 else 1,
        c["table"].data_ptr(), c["table"].shape[1], c["seq_slot"].data_ptr(), c["seq_len"].data_ptr(),
        got.data_ptr(), c["qkv"].shape[0], nq, nkv, c["qkv"].shape[1], scale, cap, window, ring, chunk, max_chunks,
        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.janis_last_error().decode()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_the_ordinary_entry_point_twice(dtype):
    ops, lib = _library()
    tol = 2e-5 if dtype == torch.float32 else 2.0 ** -8 + 1e-4      # the kernel tests' tolerances
    # first call: six query heads over one key head, long sequences, many chunks.  Second call, other sizes and
    # a ring: it finds the array full of the first call's partial results.  Third: one chunk per sequence; in
    # bfloat16 the kernel then writes its result itself and leaves the array alone.
    calls = [(_case(1, dtype, lens=[300, 64, 1, 129], slots=[2, 0, 3, 1], nq=6, nkv=1), (6, 1, 0, 0, 64)),
             (_case(2, dtype, lens=[7, 200, 65], slots=[1, -1, 0], nq=4, nkv=2), (4, 2, 16, 64, 64)),
             (_case(4, dtype, lens=[60, 5, 64], slots=[0, 2, 1], nq=4, nkv=2), (4, 2, 0, 0, 64))]
    # everything torch allocates is allocated before the first call, so that free memory can be compared after it
    refs = [_ordinary(ops, c, *args) for c, args in calls]
    gots = [torch.full_like(want, 3.0) for want, _ in refs]
    torch.cuda.synchronize()
    free = []
    for (c, args), got in zip(calls, gots):
        _static(lib, c, got, *args)
        torch.cuda.synchronize()
        free.append(torch.cuda.mem_get_info()[0])
    # the array's memory is committed by the first call on the device at the latest: the later ones take nothing
    assert free[1] == free[0] and free[2] == free[0], f"free device memory moved across later calls: {free}"
    for got, (want, plain), name in zip(gots, refs, ("first call", "second call", "third call")):
        assert torch.isfinite(got).all(), name
        for ref, what in ((want, "the ordinary entry point"), (plain, "the plain statement")):
            scale = ref.double().abs().max().item()
            err = (got.double().cpu() - ref.double().cpu()).abs().max().item()
            assert err <= tol * scale, f"{name} against {what}: max err {err:.3e} > {tol:.1e} x {scale:.3e}"


def test_the_set_up_call_and_the_largest_request_that_fits():
    ops, lib = _library()
    # n_seq = 0: the set-up alone (this is the call a server makes before it gives its memory away)
    assert lib.janis_attn_decode_static(None, None, None, 0, None, 0, None, None, None, 0, 4, 2, 8, 1.0, 0.0, 0, 0, 64, 1,
                                        torch.cuda.current_stream().cuda_stream) == 0
    lens, slots = [130, 5, 64, 70, 1, 200, 129, 33], [1, 0, 3, 2, 5, 4, 7, 6]
    c = _case(5, torch.float32, lens=lens, slots=slots, nq=4, nkv=2, n_pages=40, pages_per_seq=4)
    n_seq = len(lens)
    out = torch.zeros((n_seq, 4 * HD), dtype=torch.float32, device="cuda:0")
    most = STATIC_SCRATCH_FLOATS // (n_seq * 4 * (HD + 2))      # chunks whose partial results just fit the array
    assert (most + 1) * n_seq * 4 * (HD + 2) > STATIC_SCRATCH_FLOATS >= most * n_seq * 4 * (HD + 2) and most <= 8192
    # the launch is sized by max_chunks; the sequences are short, so all but a few chunks find nothing to do
    args = (c["qkv"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), 0, c["table"].data_ptr(), c["table"].shape[1],
            c["seq_slot"].data_ptr(), c["seq_len"].data_ptr(), out.data_ptr(), n_seq, 4, 2, 8, 1.0 / math.sqrt(HD), 25.0, 0, 0, 64)
    rc = lib.janis_attn_decode_static(*args, most, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.janis_last_error().decode()
    torch.cuda.synchronize()
    from tests import kernel_refs
    plain = torch.empty((n_seq, 4 * HD), dtype=torch.float64)
    kernel_refs.attn_decode(c["qkv"].cpu(), c["k"].cpu(), c["v"].cpu(), c["table"].cpu(), c["seq_slot"].cpu(),
                            c["seq_len"].cpu(), None, plain, 4, 2, HD, 1.0 / math.sqrt(HD), 25.0, 0, 0, 64, most)
    assert (out.double().cpu() - plain).abs().max().item() <= 2e-5 * plain.abs().max().item()
    # one chunk more does not fit
    assert lib.janis_attn_decode_static(*args, most + 1, torch.cuda.current_stream().cuda_stream) != 0
    assert "static scratch holds" in lib.janis_last_error().decode()


def test_static_scratch_refuses_what_does_not_fit():
    ops, lib = _library()
    c = _case(3, torch.float32, lens=[10], slots=[0], nq=4, nkv=2)
    out = torch.zeros((1, 4 * HD), dtype=torch.float32, device="cuda:0")
    # pretend to need more partial results than the array holds: refused before anything is launched
    too_many = STATIC_SCRATCH_FLOATS // (4 * (HD + 2)) + 1
    rc = lib.janis_attn_decode_static(
        c["qkv"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), 0, c["table"].data_ptr(), c["table"].shape[1],
        c["seq_slot"].data_ptr(), c["seq_len"].data_ptr(), out.data_ptr(), 1, 4, 2, 8, 1.0, 0.0, 0, 0, 64, too_many,
        torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.janis_last_error().decode()
    assert "static scratch holds" in msg and str(STATIC_SCRATCH_FLOATS) in msg
    torch.cuda.synchronize()
    assert (out == 0).all()
