"""Each CUDA kernel alone against its plain statement in tests/kernel_refs.py,
at sizes other than the engine's tests use: widths and vocabularies that are no
power of two, head sizes in steps of 16, odd numbers of rows, both dtypes.

Tolerances: float32 paths 2e-5 of the largest reference value (accumulation
order differs from the float64 reference); bfloat16 outputs one rounding step,
2^-8 of the largest value, plus the same accumulation allowance.
"""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from tests import kernel_refs as R

pytestmark = pytest.mark.gpu

F32_TOL = 2e-5
BF16_TOL = 2.0 ** -8 + 1e-4


def ops():
    from janis_b200.kernels import ops as o
    return o


def dev():
    return torch.device("cuda:0")


def close(got, want, tol, what=""):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    scale = max(want.abs().max().item(), 1e-30)
    err = (got - want).abs().max().item()
    assert err <= tol * scale, f"{what}: max err {err:.3e} > {tol:.1e} x scale {scale:.3e}"


def same(got, want, what=""):
    """Bit for bit; says where and by how much if not."""
    if torch.equal(got, want):
        return
    bad = (got != want).nonzero()
    first = tuple(int(v) for v in bad[0])
    diff = (got.double() - want.double()).abs().max().item()
    raise AssertionError(f"{what}: {len(bad)} of {got.numel()} values differ, first at {first}: "
                         f"{got[first].item()} vs {want[first].item()}; max difference {diff:.3e}")


def tol_of(dtype):
    return F32_TOL if dtype == torch.float32 else BF16_TOL


def rnd(shape, dtype, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype).to(dev())


DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,V", [(1, 64, 50), (7, 100, 333), (33, 2304, 1000)])
def test_embed(dtype, T, H, V):
    table = rnd((V, H), dtype, 1)
    tokens = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(2)).int().to(dev())
    out = torch.empty((T, H), dtype=torch.float32, device=dev())
    ops().embed(tokens, table, math.sqrt(H), out)
    want = torch.empty((T, H), dtype=torch.float32)
    R.embed(tokens.cpu(), table.cpu(), math.sqrt(H), want)
    close(out, want, F32_TOL, "embed")


@pytest.mark.parametrize("din", DTYPES)
@pytest.mark.parametrize("dout", DTYPES)
@pytest.mark.parametrize("Rn,H,eps", [(1, 64, 1e-6), (5, 100, 1e-5), (9, 2304, 1e-6), (3, 5000, 1e-3)])
def test_rmsnorm(din, dout, Rn, H, eps):
    x = rnd((Rn, H), din, 3, std=3.0)
    w = (1.0 + rnd((H,), torch.float32, 4, std=0.1))
    out = torch.empty((Rn, H), dtype=dout, device=dev())
    ops().rmsnorm(x, w, eps, out)
    want = torch.empty((Rn, H), dtype=torch.float64)
    R.rmsnorm(x.cpu(), w.cpu(), eps, want)
    close(out, want, tol_of(dout), "rmsnorm")
    rows = torch.tensor([Rn - 1, 0, Rn - 1], dtype=torch.int32, device=dev())
    out2 = torch.empty((3, H), dtype=dout, device=dev())
    ops().rmsnorm(x, w, eps, out2, rows)
    close(out2, want[rows.cpu().long()], tol_of(dout), "rmsnorm rows")


@pytest.mark.parametrize("dr", DTYPES)
@pytest.mark.parametrize("post,nxt,n_part", [(True, True, 1), (True, False, 1), (False, True, 1), (True, True, 3),
                                             (False, False, 2)])
@pytest.mark.parametrize("Rn,H", [(1, 96), (6, 2304), (4, 1000), (3, 4608), (2, 9000)])
def test_add_rmsnorm(dr, post, nxt, n_part, Rn, H):
    h0 = rnd((Rn, H), torch.float32, 5, std=2.0)
    res = rnd((n_part, Rn, H) if n_part > 1 else (Rn, H), dr, 6, std=0.5)
    wp = (1.0 + rnd((H,), torch.float32, 7, std=0.1)) if post else None
    wn = (1.0 + rnd((H,), torch.float32, 8, std=0.1)) if nxt else None
    h = h0.clone()
    out = torch.empty((Rn, H), dtype=dr, device=dev()) if nxt else None
    ops().add_rmsnorm(h, res, wp, 1e-6, wn, 1e-5, out, n_part)
    h_ref = h0.cpu().clone()
    out_ref = torch.empty((Rn, H), dtype=torch.float64) if nxt else None
    R.add_rmsnorm(h_ref, res.cpu(), wp.cpu() if post else None, 1e-6, wn.cpu() if nxt else None, 1e-5, out_ref, n_part)
    close(h, h_ref, F32_TOL, "residual sum")
    if nxt:
        close(out, out_ref, tol_of(dr), "next norm")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("Rn,I", [(1, 8), (5, 320), (70, 9216)])
def test_gated_act(dtype, act, Rn, I):
    gu = rnd((Rn, 2 * I), dtype, 9, std=2.0)
    out = torch.empty((Rn, I), dtype=dtype, device=dev())
    ops().gated_act(gu, out, act)
    want = torch.empty((Rn, I), dtype=torch.float64)
    R.gated_act(gu.cpu(), want, act)
    close(out, want, tol_of(dtype), "gated_act")


def _paged(n_pages, nkv, hd, dtype, seed):
    k = rnd((n_pages, nkv, R.PAGE, hd), dtype, seed)
    v = rnd((n_pages, nkv, R.PAGE, hd), dtype, seed + 1)
    return k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,rot,ring", [(4, 2, 16, 16, 0), (6, 1, 32, 32, 64), (3, 3, 48, 24, 128),
                                                (8, 4, 256, 256, 0), (2, 1, 64, 0, 64)])
def test_rope_store(dtype, nq, nkv, hd, rot, ring):
    # three sequences; the second is padding (slot -1); the third is longer than a ring of 64
    lens = [5, 3, 150]
    starts = [0, 0, 0]
    slots = [2, -1, 0]
    T = sum(lens)
    tok_pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).int()
    tok_seq = torch.repeat_interleave(torch.arange(3), torch.tensor(lens)).int()
    seq_slot = torch.tensor(slots).int()
    seq_end = torch.tensor([s + n for s, n in zip(starts, lens)]).int()
    inv = torch.tensor([10000.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32)
    n_pages, width = 12, 4
    table = torch.tensor([[7, 3, 9, 1], [0, 0, 0, 0], [5, 2, 8, 11]], dtype=torch.int32)
    qkv = rnd((T, nq + 2 * nkv, hd), dtype, 10)
    k, v = _paged(n_pages, nkv, hd, dtype, 11)
    qkv_ref, k_ref, v_ref = qkv.cpu().clone(), k.cpu().clone(), v.cpu().clone()
    d = dev()
    ops().rope_store(qkv, tok_pos.to(d), tok_seq.to(d), seq_slot.to(d), seq_end.to(d), inv.to(d), rot, nq, nkv, hd,
                     k, v, table.to(d), ring, True)
    R.rope_store(qkv_ref, tok_pos, tok_seq, seq_slot, seq_end, inv, rot, nq, nkv, hd, k_ref, v_ref, table, ring, True)
    close(qkv, qkv_ref, tol_of(dtype), "rotated q/k")
    close(k, k_ref, tol_of(dtype), "cached k")
    close(v, v_ref, tol_of(dtype), "cached v")
    # query-only rows (a layer that reads another layer's keys)
    q = rnd((T, nq, hd), dtype, 12)
    q_ref = q.cpu().clone()
    ops().rope_store(q, tok_pos.to(d), tok_seq.to(d), None, None, inv.to(d), rot, nq, nkv, hd, store=False)
    R.rope_store(q_ref, tok_pos, tok_seq, None, None, inv, rot, nq, nkv, hd, store=False)
    close(q, q_ref, tol_of(dtype), "rotated q alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,rot,ring", [(8, 4, 256, 256, 0), (5, 1, 32, 32, 128), (3, 2, 48, 24, 0)])
def test_rope_store_many_tokens(dtype, nq, nkv, hd, rot, ring):
    """Enough tokens that a thread (or CTA) walks over several heads, with a head count that its groups do not divide."""
    lens = [300, 3, 450]
    slots = [1, -1, 0]
    T = sum(lens)
    tok_pos = torch.cat([torch.arange(n) for n in lens]).int()
    tok_seq = torch.repeat_interleave(torch.arange(3), torch.tensor(lens)).int()
    seq_slot = torch.tensor(slots).int()
    seq_end = torch.tensor(lens).int()
    inv = torch.tensor([10000.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32)
    width = 8
    n_pages = 2 * width + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(5))[:2 * width].int()
    table = perm.view(2, width).contiguous()
    qkv = rnd((T, nq + 2 * nkv, hd), dtype, 20)
    k, v = _paged(n_pages, nkv, hd, dtype, 21)
    qkv_ref, k_ref, v_ref = qkv.cpu().clone(), k.cpu().clone(), v.cpu().clone()
    d = dev()
    ops().rope_store(qkv, tok_pos.to(d), tok_seq.to(d), seq_slot.to(d), seq_end.to(d), inv.to(d), rot, nq, nkv, hd,
                     k, v, table.to(d), ring, True)
    R.rope_store(qkv_ref, tok_pos, tok_seq, seq_slot, seq_end, inv, rot, nq, nkv, hd, k_ref, v_ref, table, ring, True)
    close(qkv, qkv_ref, tol_of(dtype), "rotated q/k")
    close(k, k_ref, tol_of(dtype), "cached k")
    close(v, v_ref, tol_of(dtype), "cached v")


@pytest.mark.parametrize("M", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("nq,nkv,hd,K,ring", [(8, 4, 256, 2304, 0), (4, 2, 64, 328, 64), (3, 1, 48, 72, 0),
                                              (2, 2, 16, 2048, 128), (5, 1, 32, 9216, 64)])
def test_projection_with_rotary_and_cache_write_in_one_kernel(M, nq, nkv, hd, K, ring):
    """The fused decode kernel against the two kernels it replaces, bit for bit (it rounds the sums to bfloat16
    before it rotates them, as they do), and against the plain statement: rows at positions on both sides of a
    ring's wrap, a padding row, short and long K (clusters of 1, 2 and 4 CTAs), and the query-only form."""
    d = dev()
    pos = [(37 * i + (140 if i % 3 == 0 else 3)) % 190 for i in range(M)]
    slots = [(-1 if (i == 2 and M > 2) else (5 * i + 3) % 16) for i in range(M)]     # every row a sequence of its own
    tok_pos = torch.tensor(pos, dtype=torch.int32)
    tok_seq = torch.arange(M, dtype=torch.int32)
    seq_slot = torch.tensor(slots, dtype=torch.int32)
    seq_end = (tok_pos + 1).int()
    inv = torch.tensor([10000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float32)
    n_pages = 70
    table = torch.randperm(n_pages, generator=torch.Generator().manual_seed(6))[:64].int().view(16, 4).contiguous()
    heads = nq + 2 * nkv
    x = rnd((M, K), torch.bfloat16, 30 + M)
    w = (rnd((heads * hd, K), torch.bfloat16, 31) * (4.0 / K ** 0.5)).to(torch.bfloat16)
    k0, v0 = _paged(n_pages, nkv, hd, torch.bfloat16, 32)
    # the two kernels
    qkv2 = torch.zeros((M, heads, hd), dtype=torch.bfloat16, device=d)
    k2, v2 = k0.clone(), v0.clone()
    ops().gemv_bf16(x, w, qkv2.view(M, heads * hd))
    ops().rope_store(qkv2, tok_pos.to(d), tok_seq.to(d), seq_slot.to(d), seq_end.to(d), inv.to(d), hd, nq, nkv, hd,
                     k2, v2, table.to(d), ring, True)
    # the one kernel
    qkv1 = torch.zeros((M, heads, hd), dtype=torch.bfloat16, device=d)
    k1, v1 = k0.clone(), v0.clone()
    ops().gemv_rope_store(x, w, qkv1, tok_pos.to(d), tok_seq.to(d), seq_slot.to(d), seq_end.to(d), inv.to(d), nq, nkv,
                          hd, k1, v1, table.to(d), ring, True)
    same(qkv1[:, :nq], qkv2[:, :nq], "rotated q")
    same(k1, k2, "cached k")
    same(v1, v2, "cached v")
    # the plain statement
    q_ref = torch.zeros((M, heads, hd), dtype=torch.bfloat16)
    k_ref, v_ref = k0.cpu().clone(), v0.cpu().clone()
    R.gemv_rope_store(x.cpu(), w.cpu(), q_ref, tok_pos, tok_seq, seq_slot, seq_end, inv, nq, nkv, hd, k_ref, v_ref,
                      table, ring, True)
    close(qkv1[:, :nq], q_ref[:, :nq], BF16_TOL, "rotated q")
    close(k1, k_ref, BF16_TOL, "cached k")
    close(v1, v_ref, BF16_TOL, "cached v")
    # queries alone
    wq = w[: nq * hd].contiguous()
    q1 = torch.zeros((M, nq, hd), dtype=torch.bfloat16, device=d)
    ops().gemv_rope_store(x, wq, q1, tok_pos.to(d), tok_seq.to(d), None, None, inv.to(d), nq, nkv, hd, store=False)
    q2 = torch.zeros((M, nq, hd), dtype=torch.bfloat16, device=d)
    ops().gemv_bf16(x, wq, q2.view(M, nq * hd))       # (fewer rows of W: K may be split over more CTAs than above)
    ops().rope_store(q2, tok_pos.to(d), tok_seq.to(d), None, None, inv.to(d), hd, nq, nkv, hd, store=False)
    same(q1, q2, "rotated q alone")


def test_rope_angles_at_large_positions():
    """theta = float32(pos) * inv_freq with accurate sin/cos, also thousands of radians out."""
    nq, nkv, hd = 1, 1, 64
    pos = torch.tensor([0, 1, 4095, 8191, 100000], dtype=torch.int32)
    T = len(pos)
    inv = torch.tensor([10000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float32)
    q = rnd((T, 1, hd), torch.float32, 13)
    want = q.cpu().clone()
    d = dev()
    seq = torch.zeros(T, dtype=torch.int32)
    got = q.clone()
    ops().rope_store(got, pos.to(d), seq.to(d), None, None, inv.to(d), hd, 1, 1, hd, store=False)
    R.rope_store(want, pos, seq, None, None, inv, hd, 1, 1, hd, store=False)
    close(got, want, 1e-5, "rope at large positions")


@pytest.mark.parametrize("M,N,K,cap", [(1, 1, 1, 0.0), (3, 70, 33, 0.0), (64, 64, 16, 0.0), (65, 130, 100, 5.0),
                                       (8, 384, 96, 15.0), (200, 96, 320, 0.0)])
def test_gemm_f32(M, N, K, cap):
    x = rnd((M, K), torch.float32, 14)
    w = rnd((N, K), torch.float32, 15)
    out = torch.empty((M, N), dtype=torch.float32, device=dev())
    ops().gemm_f32(x, w, out, cap)
    want = torch.empty((M, N), dtype=torch.float64)
    R.gemm_f32(x.cpu(), w.cpu(), want, cap)
    close(out, want, F32_TOL, "gemm_f32")


def test_gemm_f32_row_does_not_depend_on_batch():
    x = rnd((37, 200), torch.float32, 16)
    w = rnd((90, 200), torch.float32, 17)
    full = torch.empty((37, 90), dtype=torch.float32, device=dev())
    ops().gemm_f32(x, w, full)
    one = torch.empty((1, 90), dtype=torch.float32, device=dev())
    ops().gemm_f32(x[20:21].contiguous(), w, one)
    assert torch.equal(full[20:21], one)


@pytest.mark.parametrize("dout", DTYPES)
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K", [(16, 32), (40, 72), (384, 96), (2304, 2048), (1000, 328)])
def test_gemv_bf16(dout, M, N, K):
    x = rnd((M, K), torch.bfloat16, 18)
    w = rnd((N, K), torch.bfloat16, 19, std=0.05)
    out = torch.empty((M, N), dtype=dout, device=dev())
    ops().gemv_bf16(x, w, out)
    want = torch.empty((M, N), dtype=torch.float64)
    R.gemv_bf16(x.cpu(), w.cpu(), want)
    close(out, want, tol_of(dout) if dout == torch.bfloat16 else 1e-4, "gemv_bf16")


@pytest.mark.parametrize("cluster", [1, 2, 4])
@pytest.mark.parametrize("M,N,K", [(1, 2304, 2048), (8, 2304, 9216), (20, 100, 64), (64, 48, 1032), (3, 16, 8)])
def test_gemv_bf16_clusters_share_k(cluster, M, N, K):
    """A tile's K split over the CTAs of a thread-block cluster and added through distributed shared
    memory: the same product, whatever the cluster size (and K shorter than the cluster's reach)."""
    x = rnd((M, K), torch.bfloat16, 50)
    w = rnd((N, K), torch.bfloat16, 51, std=0.05)
    out = torch.empty((M, N), dtype=torch.float32, device=dev())
    ops().gemv_bf16(x, w, out, cluster=cluster)
    want = torch.empty((M, N), dtype=torch.float64)
    R.gemv_bf16(x.cpu(), w.cpu(), want)
    close(out, want, 1e-4, f"gemv_bf16 cluster {cluster}")


@pytest.mark.parametrize("M,N,K,epi", [(1, 18432, 2304, 1), (8, 17000, 264, 0), (16, 16400, 96, 2), (40, 16384, 40, 3)])
def test_gemv_bf16_tall(M, N, K, epi):
    """Tall products (the gated feed-forward, the head) run in CTAs of 4 warps."""
    x = rnd((M, K), torch.bfloat16, 52)
    w = rnd((N, K), torch.bfloat16, 53, std=0.1)
    n_out = N // 2 if epi in (1, 3) else N
    out = torch.empty((M, n_out), dtype=torch.float32, device=dev())
    ops().gemv_bf16(x, w, out, epi, 7.0)
    want = torch.empty((M, n_out), dtype=torch.float64)
    R.gemv_bf16(x.cpu(), w.cpu(), want, epi, 7.0)
    close(out, want, 1e-4, "gemv_bf16, tall")


@pytest.mark.parametrize("M", [1, 5, 8, 12, 40, 64])
@pytest.mark.parametrize("epi", [1, 3])
@pytest.mark.parametrize("I,K", [(8, 16), (320, 96), (1000, 104)])
def test_gemv_bf16_gated(M, epi, I, K):
    x = rnd((M, K), torch.bfloat16, 20)
    w = rnd((2 * I, K), torch.bfloat16, 21, std=0.2)
    out = torch.empty((M, I), dtype=torch.bfloat16, device=dev())
    ops().gemv_bf16(x, w, out, epi)
    want = torch.empty((M, I), dtype=torch.float64)
    R.gemv_bf16(x.cpu(), w.cpu(), want, epi)
    close(out, want, BF16_TOL, "gemv gated")


@pytest.mark.parametrize("M,N,K,cap", [(1, 256, 64, 30.0), (7, 1000, 96, 2.0), (64, 50, 40, 0.0)])
def test_gemv_bf16_softcap(M, N, K, cap):
    x = rnd((M, K), torch.bfloat16, 22, std=2.0)
    w = rnd((N, K), torch.bfloat16, 23)
    out = torch.empty((M, N), dtype=torch.float32, device=dev())
    ops().gemv_bf16(x, w, out, 2, cap)
    want = torch.empty((M, N), dtype=torch.float64)
    R.gemv_bf16(x.cpu(), w.cpu(), want, 2, cap)
    close(out, want, 1e-4, "gemv softcap")


def test_softcap_and_library_product_with_float_output():
    x = rnd((70, 96), torch.bfloat16, 60, std=3.0)
    w = rnd((1000, 96), torch.bfloat16, 61)
    out = torch.empty((70, 1000), dtype=torch.float32, device=dev())
    ops().matmul_bf16_to_f32(x, w, out)
    close(out, x.double().cpu() @ w.double().cpu().T, 1e-4, "library product, float32 out")
    want = 15.0 * torch.tanh(out.double().cpu() / 15.0)
    ops().softcap(out, 15.0)
    close(out, want, F32_TOL, "softcap")


def test_gemv_refuses_what_it_cannot_do():
    o = ops()
    x = rnd((2, 12), torch.bfloat16, 24)
    w = rnd((16, 12), torch.bfloat16, 25)
    with pytest.raises(o.KernelError, match="multiple of 8"):
        o.gemv_bf16(x, w, torch.empty((2, 16), dtype=torch.bfloat16, device=dev()))
    x = rnd((65, 16), torch.bfloat16, 24)
    w = rnd((16, 16), torch.bfloat16, 25)
    with pytest.raises(o.KernelError, match="at most 64"):
        o.gemv_bf16(x, w, torch.empty((65, 16), dtype=torch.bfloat16, device=dev()))


ATTN_SHAPES = [(4, 2, 16), (6, 1, 32), (3, 3, 48), (2, 2, 64), (9, 1, 80), (8, 4, 128), (8, 4, 256), (20, 2, 64)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd", ATTN_SHAPES)
@pytest.mark.parametrize("window,cap", [(0, 0.0), (7, 20.0), (64, 50.0)])
def test_attn_prefill(dtype, nq, nkv, hd, window, cap):
    lens = [1, 9, 70, 23]
    T = sum(lens)
    first = torch.tensor([0, 1, 10, 80], dtype=torch.int32)
    tok_pos = torch.cat([torch.arange(n) for n in lens]).int()
    tok_seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).int()
    qkv = rnd((T, nq + 2 * nkv, hd), dtype, 26)
    # one far key stands out: the first key of the long sequence matches its last query
    qkv[10, nq] = qkv[79, 0] * 3.0
    out = torch.empty((T, nq * hd), dtype=dtype, device=dev())
    scale = 1.0 / math.sqrt(hd)
    d = dev()
    ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, scale, cap, window)
    want = torch.empty((T, nq * hd), dtype=torch.float64)
    R.attn_prefill(qkv.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, scale, cap, window)
    close(out, want, tol_of(dtype), "attn_prefill")


@pytest.fixture(params=[3, 2, 0], ids=["tcgen05_ctas_that_stay", "tcgen05_cta_per_tile", "mma_sync"])
def prefill_kernel(request):
    """The bfloat16 prompt kernels: tcgen05 in both its forms (CTAs that stay and take item after item; a CTA per
    tile of queries and head) and mma.sync (head sizes the tcgen05 kernel does not take run mma.sync either way)."""
    yield request.param
    for hd in list(ops()._attn):                # the libraries that are loaded: back to their default
        ops().attn_set_prefill_kernel(hd, 1)
        ops().attn_set_prefill_piece(hd, 0)


@pytest.mark.parametrize("nq,nkv,hd", ATTN_SHAPES + [(2, 1, 96), (2, 2, 112)])
@pytest.mark.parametrize("window,cap", [(0, 0.0), (7, 20.0), (64, 50.0), (100, 30.0)])
def test_attn_prefill_tensor_cores(nq, nkv, hd, window, cap, prefill_kernel):
    """The bfloat16 tensor-core kernels: tiles of 128 queries and 64 keys, so lengths around 64 and 128,
    a window that cuts inside and across tiles, and a far key that must win."""
    if prefill_kernel and (hd % 64 or hd > 256):
        pytest.skip("the tcgen05 kernel takes head sizes that are a multiple of 64 up to 256")
    ops().attn_set_prefill_kernel(hd, prefill_kernel)
    lens = [1, 63, 64, 65, 200, 129]
    T = sum(lens)
    first = torch.tensor([0] + list(np.cumsum(lens)[:-1]), dtype=torch.int32)
    tok_pos = torch.cat([torch.arange(n) for n in lens]).int()
    tok_seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).int()
    seq_len = torch.tensor(lens, dtype=torch.int32)
    qkv = rnd((T, nq + 2 * nkv, hd), torch.bfloat16, 40)
    r0 = int(first[4])
    qkv[r0, nq] = qkv[r0 + 199, 0] * 3.0          # position 0 of the 200-token sequence answers its last query
    out = torch.full((T, nq * hd), 9.0, dtype=torch.bfloat16, device=dev())
    scale = 1.0 / math.sqrt(hd)
    d = dev()
    ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, scale, cap, window,
                       seq_len=seq_len.to(d))
    want = torch.empty((T, nq * hd), dtype=torch.float64)
    R.attn_prefill(qkv.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, scale, cap, window)
    # P is rounded to bfloat16 before P V: one more rounding step than the CUDA-core kernel
    close(out, want, 2 * BF16_TOL, "attn_prefill on tensor cores")
    assert ops().attn_tc05_timeouts(hd) == 0


@pytest.mark.parametrize("nq,nkv,hd", [(8, 4, 256), (4, 2, 64), (2, 1, 128), (3, 1, 48)])
@pytest.mark.parametrize("lens", [[1], [5], [3, 2], [64], [127, 1]])
def test_attn_prefill_of_a_few_tokens(nq, nkv, hd, lens, prefill_kernel):
    """Steps much shorter than a tile of queries or keys (the TMA boxes reach past the end of the rows)."""
    if prefill_kernel and (hd % 64 or hd > 256):
        pytest.skip("the tcgen05 kernel takes head sizes that are a multiple of 64 up to 256")
    ops().attn_set_prefill_kernel(hd, prefill_kernel)
    T = sum(lens)
    first = torch.tensor([0] + list(np.cumsum(lens)[:-1]), dtype=torch.int32)
    tok_pos = torch.cat([torch.arange(n) for n in lens]).int()
    tok_seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).int()
    qkv = rnd((T, nq + 2 * nkv, hd), torch.bfloat16, 43)
    d = dev()
    out = torch.full((T, nq * hd), 9.0, dtype=torch.bfloat16, device=d)
    ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, 1.0 / math.sqrt(hd), 25.0, 0,
                       seq_len=torch.tensor(lens, dtype=torch.int32, device=d))
    want = torch.empty((T, nq * hd), dtype=torch.float64)
    R.attn_prefill(qkv.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, 1.0 / math.sqrt(hd), 25.0, 0)
    close(out, want, 2 * BF16_TOL, "attn_prefill of a few tokens")
    assert ops().attn_tc05_timeouts(hd) == 0


@pytest.mark.parametrize("nq,nkv,hd", [(8, 4, 256), (4, 2, 64), (3, 1, 80), (2, 2, 128)])
@pytest.mark.parametrize("window,cap", [(0, 0.0), (100, 30.0), (300, 50.0)])
@pytest.mark.parametrize("piece", [0, 1, 3, 4])
def test_attn_prefill_shared_tiles(nq, nkv, hd, window, cap, piece, prefill_kernel):
    """Few tiles of queries: the long ones are cut into pieces for two to four CTAs that meet through scratch.
    Sequences long enough for tiles with many key tiles (2 to 11 of them: with pieces of 1, 3 and 4 every number
    of pieces occurs, in equal and unequal cuts; 0 is the library's own choice), a window that leaves some tiles unshared, a far
    key that must win, the same call without scratch, and with the lengths given to the host as well."""
    if prefill_kernel and (hd % 64 or hd > 256):
        pytest.skip("the tcgen05 kernel takes head sizes that are a multiple of 64 up to 256")
    ops().attn_set_prefill_kernel(hd, prefill_kernel)
    ops().attn_set_prefill_piece(hd, piece)
    lens = [700, 129, 300, 1]
    T = sum(lens)
    first = torch.tensor([0] + list(np.cumsum(lens)[:-1]), dtype=torch.int32)
    tok_pos = torch.cat([torch.arange(n) for n in lens]).int()
    tok_seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).int()
    seq_len = torch.tensor(lens, dtype=torch.int32)
    qkv = rnd((T, nq + 2 * nkv, hd), torch.bfloat16, 41)
    qkv[0, nq] = qkv[699, 0] * 3.0                # position 0 of the long sequence answers its last query
    d = dev()
    n = ops().attn_prefill_scratch_floats(T, len(lens), nq, hd)
    assert n > 0
    scratch = torch.full((n,), float("nan"), dtype=torch.float32, device=d)
    outs = []
    for sc, known in ((scratch, None), (None, None), (scratch, lens)):
        out = torch.full((T, nq * hd), 9.0, dtype=torch.bfloat16, device=d)
        ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, 1.0 / math.sqrt(hd), cap,
                           window, seq_len=seq_len.to(d), scratch=sc, host_lens=known)
        outs.append(out)
    want = torch.empty((T, nq * hd), dtype=torch.float64)
    R.attn_prefill(qkv.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, 1.0 / math.sqrt(hd), cap, window)
    close(outs[0], want, 2 * BF16_TOL, "attn_prefill with shared tiles")
    close(outs[1], want, 2 * BF16_TOL, "attn_prefill without scratch")
    close(outs[2], want, 2 * BF16_TOL, "attn_prefill with the lengths known to the host (no places to spare)")
    assert ops().attn_tc05_timeouts(hd) == 0


def test_attn_prefill_pieces_follow_the_steps_size():
    """The library's choice of piece for shared tiles of queries, from its model of the step's time: short prompts
    are cut finely (few CTAs otherwise), one of 2,048 tokens into pieces of about one and a half times an SM's
    even share, and a step that fills the SMs unshared is not cut at all (a piece as long as its longest tile)."""
    o = ops()
    assert 4 <= o.attn_prefill_piece(256, 1024, 1, 8) <= 8
    assert 18 <= o.attn_prefill_piece(256, 2048, 1, 8) <= 26
    assert o.attn_prefill_piece(256, 4096, 1, 8) == 64
    assert o.attn_prefill_piece(256, 2100, 3, 8) >= 11                 # three of 700: 11 key tiles at most, none shared
    assert o.attn_prefill_piece(256, 4096, 1, 8, window=1024) <= 18    # a window bounds the keys of a tile
    for hd, tc05 in ((128, True), (80, False)):
        assert 4 <= o.attn_prefill_piece(hd, 1536, 1, 4, tc05=tc05) <= 24


@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 64), (2, 1, 128), (8, 4, 256), (3, 1, 48), (4, 2, 16)])
@pytest.mark.parametrize("window,cap", [(0, 30.0), (100, 0.0)])
@pytest.mark.parametrize("from_kv_src", [False, True])
def test_attn_prefill_ignores_rows_that_are_not_a_sequences_own(nq, nkv, hd, window, cap, from_kv_src):
    """Rows before, between and behind the sequences hold NaN and +Inf (queries, keys and values alike): no
    sequence's result may change.  A tile of keys or values that runs past a sequence's end is masked in the
    scores, but a product of a zero weight with NaN is NaN, so the kernels must not let such rows into P V.
    Lengths end inside, on and just past tile borders; the last sequence is followed by garbage up to the end
    of the buffer.  All three prompt kernels: CUDA cores in float32 and bfloat16, mma.sync, tcgen05."""
    lens = [5, 63, 64, 70, 129, 200, 1]
    gaps = [3, 70, 1, 64, 130, 7, 9, 150]            # rows before sequence i; the last: behind them all
    first, row = [], 0
    for n, g in zip(lens, gaps):
        row += g
        first.append(row)
        row += n
    T = row + gaps[-1]
    d = dev()
    own = torch.zeros(T, dtype=torch.bool)
    for f, n in zip(first, lens):
        own[f:f + n] = True
    scale = 1.0 / math.sqrt(hd)
    # for the per-token CUDA-core kernel the rows of a gap are a sequence of garbage of their own
    g_first, g_len, prev = [], [], 0
    for f, n in zip(first + [T], lens + [0]):
        g_first.append(prev)
        g_len.append(f - prev)
        prev = f + n
    all_first = torch.tensor(first + g_first, dtype=torch.int32)
    all_len = lens + g_len
    tok_pos = torch.zeros(T, dtype=torch.int32)
    tok_seq = torch.zeros(T, dtype=torch.int32)
    for i, (f, n) in enumerate(zip(all_first.tolist(), all_len)):
        tok_pos[f:f + n] = torch.arange(n, dtype=torch.int32)
        tok_seq[f:f + n] = i
    for dtype in DTYPES:
        heads = nq if from_kv_src else nq + 2 * nkv
        clean = rnd((T, nq + 2 * nkv, hd), dtype, 44)
        poison = torch.where(torch.arange(T, device=d) % 2 == 0, float("nan"), float("inf")).to(dtype)
        dirty = torch.where(own.to(d)[:, None, None], clean, poison[:, None, None].expand_as(clean)).contiguous()
        q = dirty[:, :nq].contiguous() if from_kv_src else dirty
        kw = dict(kv_src=dirty, kv_row_heads=nq + 2 * nkv, kv_k_head0=nq) if from_kv_src else {}
        want = torch.zeros((T, nq * hd), dtype=torch.float64)
        R.attn_prefill(clean.cpu(), tok_pos, tok_seq, all_first, want, nq, nkv, hd, scale, cap, window)
        runs = [("cuda cores", dict(tensor_cores=False), 1)]
        if dtype == torch.bfloat16:
            runs.append(("mma.sync", dict(seq_len=torch.tensor(lens, dtype=torch.int32, device=d)), 0))
            if hd % 64 == 0 and hd <= 256:
                runs.append(("tcgen05, CTAs that stay", dict(seq_len=torch.tensor(lens, dtype=torch.int32, device=d)), 3))
                runs.append(("tcgen05, a CTA per tile", dict(seq_len=torch.tensor(lens, dtype=torch.int32, device=d)), 2))
        try:
            for name, extra, which in runs:
                ops().attn_set_prefill_kernel(hd, which)
                tensor_cores = "seq_len" in extra
                out = torch.full((T, nq * hd), 9.0, dtype=dtype, device=d)
                ops().attn_prefill(q, tok_pos.to(d), tok_seq.to(d),
                                   (all_first[:len(lens)] if tensor_cores else all_first).to(d), out, nq, nkv, hd, scale,
                                   cap, window, **kw, **extra)
                got = out.cpu()[own]
                assert torch.isfinite(got).all(), f"{name} {dtype}: rows of other sequences reached a result"
                close(got, want[own], (2 * BF16_TOL if tensor_cores else tol_of(dtype)), f"{name} {dtype} beside garbage")
                if tensor_cores:                     # rows that are nobody's are not written
                    assert (out.cpu()[~own] == 9.0).all()
        finally:
            ops().attn_set_prefill_kernel(hd, 1)
    assert ops().attn_tc05_timeouts(hd) == 0


@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 16), (6, 1, 32), (2, 2, 64), (8, 4, 256), (3, 1, 80), (2, 1, 272)])
@pytest.mark.parametrize("window,ring,cap", [(0, 0, 30.0), (40, 64, 20.0), (128, 128, 0.0), (100, 128, 50.0)])
def test_attn_prefill_continues_from_the_cache(nq, nkv, hd, window, ring, cap):
    """Sequences that bring several tokens onto what earlier steps stored: the earlier positions come from the
    paged cache (a ring for windowed lines, as the steps before left it), this step's own from the step's
    buffer.  Starts inside, on and beyond a page and a ring, a sequence that starts at 0 beside them, a step
    longer than the window and than the ring, pages scattered, and a far cached key that must win where it is
    visible.  CUDA-core kernel in both dtypes, mma.sync in bfloat16 (the tcgen05 kernel is not for such steps);
    with and without shared tiles."""
    starts = [0, 5, 64, 200, 130, 63]
    news = [70, 9, 1, 150, 260, 129]
    slots = [2, 0, 5, 1, 3, 4]
    n_seq = len(starts)
    T = sum(news)
    pages_per_seq = (ring // R.PAGE) if ring else 8
    n_pages = 6 * pages_per_seq + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(5))[:6 * pages_per_seq].view(6, pages_per_seq).int()
    first = torch.tensor([0] + list(np.cumsum(news)[:-1]), dtype=torch.int32)
    tok_pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, news)]).int()
    tok_seq = torch.repeat_interleave(torch.arange(n_seq), torch.tensor(news)).int()
    seq_start, seq_slot = torch.tensor(starts, dtype=torch.int32), torch.tensor(slots, dtype=torch.int32)
    seq_end = torch.tensor([s + n for s, n in zip(starts, news)], dtype=torch.int32)
    scale = 1.0 / math.sqrt(hd)
    d = dev()
    for dtype in DTYPES:
        k, v = _paged(n_pages, nkv, hd, dtype, 60)
        qkv = rnd((T, nq + 2 * nkv, hd), dtype, 62)
        # position 3 of the sequence that starts at 200 (slot 1) answers head 0 of its last query, where it is seen
        far = 3 % ring if ring else 3
        k[perm[1, far // R.PAGE].item(), 0, far % R.PAGE] = (qkv[int(first[3]) + 149, 0] * 3.0).to(dtype)
        want = torch.empty((T, nq * hd), dtype=torch.float64)
        R.attn_prefill(qkv.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, scale, cap, window, seq_start=seq_start,
                       seq_slot=seq_slot, kpool=k.cpu(), vpool=v.cpu(), page_table=perm, ring_len=ring)
        cached = dict(seq_start=seq_start.to(d), seq_slot=seq_slot.to(d), kpool=k, vpool=v, page_table=perm.to(d), ring_len=ring)
        out = torch.full((T, nq * hd), 9.0, dtype=dtype, device=d)
        ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, scale, cap, window,
                           tensor_cores=False, **cached)
        close(out, want, tol_of(dtype), f"continued prompt, CUDA cores, {dtype}")
        if dtype == torch.bfloat16:
            n = ops().attn_prefill_scratch_floats(T, n_seq, nq, hd)
            for scratch in ([torch.full((n,), float("nan"), dtype=torch.float32, device=d)] if n else []) + [None]:
                out = torch.full((T, nq * hd), 9.0, dtype=dtype, device=d)
                ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, scale, cap, window,
                                   seq_len=seq_end.to(d), scratch=scratch, **cached)
                close(out, want, 2 * BF16_TOL, f"continued prompt, mma.sync, scratch {scratch is not None}")
        # and the store that follows such a step: the same places and ring rule as the fused encoding kernel
        k2, v2 = k.clone(), v.clone()
        ops().kv_store(qkv, tok_pos.to(d), tok_seq.to(d), seq_slot.to(d), seq_end.to(d), nq, nkv, hd, k2, v2, perm.to(d), ring)
        kr, vr = k.cpu().clone(), v.cpu().clone()
        R.kv_store(qkv.cpu(), tok_pos, tok_seq, seq_slot, seq_end, nq, nkv, hd, kr, vr, perm, ring)
        same(k2.cpu(), kr, "kv_store keys")
        same(v2.cpu(), vr, "kv_store values")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attn_prefill_reads_another_layers_keys(dtype):
    nq, nkv, hd = 4, 2, 32
    lens = [6, 17]
    T = sum(lens)
    first = torch.tensor([0, 6], dtype=torch.int32)
    tok_pos = torch.cat([torch.arange(n) for n in lens]).int()
    tok_seq = torch.repeat_interleave(torch.arange(2), torch.tensor(lens)).int()
    src = rnd((T, nq + 2 * nkv, hd), dtype, 27)
    q = rnd((T, nq, hd), dtype, 28)
    d = dev()
    out = torch.empty((T, nq * hd), dtype=dtype, device=d)
    ops().attn_prefill(q, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, 0.3, 0.0, 0, kv_src=src,
                       kv_row_heads=nq + 2 * nkv, kv_k_head0=nq,
                       seq_len=torch.tensor(lens, dtype=torch.int32, device=d))
    want = torch.empty((T, nq * hd), dtype=torch.float64)
    R.attn_prefill(q.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, 0.3, 0.0, 0, kv_src=src.cpu(),
                   kv_row_heads=nq + 2 * nkv, kv_k_head0=nq)
    close(out, want, tol_of(dtype) * (2 if dtype == torch.bfloat16 else 1), "attn_prefill with kv_src")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd", ATTN_SHAPES)
@pytest.mark.parametrize("window,ring,chunk", [(0, 0, 64), (0, 0, 256), (0, 0, 320), (16, 64, 64), (100, 128, 64), (128, 128, 128),
                                               (128, 128, 384)])
@pytest.mark.parametrize("kernel", [2, 1, 0])
def test_attn_decode(dtype, nq, nkv, hd, window, ring, chunk, kernel):
    # sequences of unequal lengths in scattered pages; one padding row; lengths at page and chunk edges
    lens = [1, 64, 65, 300, 7, 129]
    slots = [3, 0, 5, 1, -1, 4]
    n_seq = len(lens)
    pages_per_seq = 6
    n_pages = 40
    g = torch.Generator().manual_seed(29)
    perm = torch.randperm(n_pages, generator=g)[: 6 * pages_per_seq].view(6, pages_per_seq).int()
    k, v = _paged(n_pages, nkv, hd, dtype, 30)
    qkv = rnd((n_seq, nq + 2 * nkv, hd), dtype, 32)
    # a far key that matters: position 0 of the 300-token sequence answers head 0's query (when it is visible)
    k[perm[1, 0].item(), 0, 0] = (qkv[3, 0] * 4.0).to(dtype)
    d = dev()
    seq_slot = torch.tensor(slots, dtype=torch.int32)
    seq_len = torch.tensor(lens, dtype=torch.int32)
    max_chunks = max((n + chunk - 1) // chunk for n in lens)
    scratch = torch.empty(ops().attn_decode_scratch_floats(n_seq, nq, hd, max_chunks), dtype=torch.float32, device=d)
    out = torch.full((n_seq, nq * hd), 7.0, dtype=dtype, device=d)
    scale, cap = 1.0 / math.sqrt(hd), 30.0
    if kernel == 2 and dtype != torch.bfloat16:
        pytest.skip("the tensor-core decode kernel is bfloat16 only")
    want = torch.empty((n_seq, nq * hd), dtype=torch.float64)
    R.attn_decode(qkv.cpu(), k.cpu(), v.cpu(), perm, seq_slot, seq_len, None, want, nq, nkv, hd, scale, cap, window,
                  ring, chunk, max_chunks)
    ops().attn_set_decode_kernel(hd, kernel)
    try:
        # the tensor-core kernel with both depths of its pipeline, and (this launch has fewer CTAs than a GPU has SMs)
        # with stages of 64 keys and of 32 at head sizes above 128
        for stages, wide in (((2, True), (3, True), (2, False)) if kernel == 2 else ((0, True),)):
            ops().attn_set_decode_stages(hd, stages)
            ops().attn_set_decode_wide(hd, wide)
            out.fill_(7.0)
            ops().attn_decode(qkv, k, v, perm.to(d), seq_slot.to(d), seq_len.to(d), scratch, out, nq, nkv, hd, scale, cap,
                              window, ring, chunk, max_chunks)
            close(out, want, tol_of(dtype), f"attn_decode (stages {stages}, wide {wide})")
    finally:
        ops().attn_set_decode_kernel(hd, 2)
        ops().attn_set_decode_stages(hd, 0)
        ops().attn_set_decode_wide(hd, True)
    assert ops().attn_wait_timeouts(hd) == 0


@pytest.mark.parametrize("hd", [144, 272, 496])
def test_attention_at_head_sizes_between_the_usual_ones(hd):
    """Head sizes whose 16-byte pieces do not divide evenly over a warp's lanes (the staged decode kernel then
    takes fewer warps so that its stages fit shared memory) and sizes beyond 256 (tiles of 32 keys in the prompt
    kernel, no tensor-core decode kernel): every kernel that takes them, both dtypes."""
    nq, nkv = 4, 2
    lens, slots = [70, 1, 200], [1, 2, 0]
    n_seq, pages_per_seq = 3, 4
    perm = torch.randperm(14, generator=torch.Generator().manual_seed(9))[:12].view(3, 4).int()
    d = dev()
    scale, cap = 1.0 / math.sqrt(hd), 25.0
    seq_slot, seq_len = torch.tensor(slots, dtype=torch.int32), torch.tensor(lens, dtype=torch.int32)
    for dtype in DTYPES:
        k, v = _paged(14, nkv, hd, dtype, 70)
        q = rnd((n_seq, nq + 2 * nkv, hd), dtype, 72)
        want = torch.empty((n_seq, nq * hd), dtype=torch.float64)
        R.attn_decode(q.cpu(), k.cpu(), v.cpu(), perm, seq_slot, seq_len, None, want, nq, nkv, hd, scale, cap, 0, 0, 64, 4)
        scratch = torch.empty(ops().attn_decode_scratch_floats(n_seq, nq, hd, 4), dtype=torch.float32, device=d)
        try:
            for kernel in (2, 1, 0):
                ops().attn_set_decode_kernel(hd, kernel)
                out = torch.full((n_seq, nq * hd), 7.0, dtype=dtype, device=d)
                ops().attn_decode(q, k, v, perm.to(d), seq_slot.to(d), seq_len.to(d), scratch, out, nq, nkv, hd, scale, cap,
                                  0, 0, 64, 4)
                close(out, want, tol_of(dtype), f"attn_decode kernel {kernel} at head size {hd}, {dtype}")
        finally:
            ops().attn_set_decode_kernel(hd, 2)
        T = sum(lens)
        first = torch.tensor([0, 70, 71], dtype=torch.int32)
        tok_pos = torch.cat([torch.arange(n) for n in lens]).int()
        tok_seq = torch.repeat_interleave(torch.arange(n_seq), torch.tensor(lens)).int()
        qkv = rnd((T, nq + 2 * nkv, hd), dtype, 74)
        want = torch.empty((T, nq * hd), dtype=torch.float64)
        R.attn_prefill(qkv.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, scale, cap, 50)
        out = torch.full((T, nq * hd), 7.0, dtype=dtype, device=d)
        ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, scale, cap, 50, tensor_cores=False)
        close(out, want, tol_of(dtype), f"attn_prefill on CUDA cores at head size {hd}, {dtype}")
        if dtype == torch.bfloat16:
            out = torch.full((T, nq * hd), 7.0, dtype=dtype, device=d)
            ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, scale, cap, 50, seq_len=seq_len.to(d))
            close(out, want, 2 * BF16_TOL, f"attn_prefill on tensor cores at head size {hd}")
    assert ops().attn_wait_timeouts(hd) == 0


@pytest.mark.parametrize("window,ring", [(0, 0), (1024, 1024)])
@pytest.mark.parametrize("chunk", [704, 128, 64])
def test_attn_decode_over_thousands_of_keys(window, ring, chunk):
    """Long sequences: many tiles per chunk, many chunks (8, 40 and 79 of them: the merge kernel's three ways of
    forming its weights), pages far apart, a far key that must win."""
    nq, nkv, hd = 4, 2, 128
    lens = [5000, 3, 2049]
    slots = [1, 2, 0]
    pages_per_seq = 80 if ring == 0 else ring // R.PAGE
    n_pages = 3 * pages_per_seq + 5
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3))[:3 * pages_per_seq].view(3, pages_per_seq).int()
    k, v = _paged(n_pages, nkv, hd, torch.bfloat16, 50)
    qkv = rnd((3, nq + 2 * nkv, hd), torch.bfloat16, 52)
    far = 0 if window == 0 else 5000 - window          # the oldest key the first sequence still sees
    idx = far % ring if ring else far
    k[perm[1, idx // R.PAGE].item(), 0, idx % R.PAGE] = (qkv[0, 0] * 4.0).to(torch.bfloat16)
    d = dev()
    seq_slot, seq_len = torch.tensor(slots, dtype=torch.int32), torch.tensor(lens, dtype=torch.int32)
    max_chunks = (5000 if window == 0 else window) // chunk + 2
    scratch = torch.empty(ops().attn_decode_scratch_floats(3, nq, hd, max_chunks), dtype=torch.float32, device=d)
    out = torch.full((3, nq * hd), 7.0, dtype=torch.bfloat16, device=d)
    ops().attn_decode(qkv, k, v, perm.to(d), seq_slot.to(d), seq_len.to(d), scratch, out, nq, nkv, hd, 1.0 / math.sqrt(hd),
                      50.0, window, ring, chunk, max_chunks)
    want = torch.empty((3, nq * hd), dtype=torch.float64)
    R.attn_decode(qkv.cpu(), k.cpu(), v.cpu(), perm, seq_slot, seq_len, None, want, nq, nkv, hd, 1.0 / math.sqrt(hd), 50.0,
                  window, ring, chunk, max_chunks)
    close(out, want, BF16_TOL, "attn_decode over thousands of keys")
    assert ops().attn_wait_timeouts(hd) == 0


@pytest.mark.parametrize("slope", [1.0, -1.0])
@pytest.mark.parametrize("hd", [64, 256])
def test_attn_prefill_with_scores_that_climb(hd, slope, prefill_kernel):
    """Scores that grow (or fall) steadily along the keys, by far more than the step after which the tcgen05
    kernel moves the reference of its exponentials: the accumulator is rescaled many times, and each row's
    weight sits on its newest (or oldest) keys."""
    nq, nkv = 2, 1
    ops().attn_set_prefill_kernel(hd, prefill_kernel)
    T = 700
    g = torch.Generator().manual_seed(77)
    u = torch.randn(hd, generator=g)
    u = u / u.norm()
    qkv = (torch.randn(T, nq + 2 * nkv, hd, generator=g) * 0.05)
    qkv[:, :nq] += u * 8.0                                        # every query points along u
    ramp = torch.arange(T, dtype=torch.float32) / T * slope       # key j: u * 60 j / T / 8 * sqrt(hd) -> score 60 j / T
    qkv[:, nq] += u[None, :] * (ramp[:, None] * 60.0 / 8.0 * math.sqrt(hd))
    qkv = qkv.to(torch.bfloat16).to(dev())
    first = torch.tensor([0], dtype=torch.int32)
    tok_pos = torch.arange(T).int()
    tok_seq = torch.zeros(T, dtype=torch.int32)
    d = dev()
    out = torch.full((T, nq * hd), 9.0, dtype=torch.bfloat16, device=d)
    ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, 1.0 / math.sqrt(hd), 0.0, 0,
                       seq_len=torch.tensor([T], dtype=torch.int32, device=d))
    want = torch.empty((T, nq * hd), dtype=torch.float64)
    R.attn_prefill(qkv.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, 1.0 / math.sqrt(hd), 0.0, 0)
    close(out, want, 2 * BF16_TOL, "attn_prefill with climbing scores")
    assert ops().attn_tc05_timeouts(hd) == 0


@pytest.mark.parametrize("hd,window,cap", [(256, 0, 50.0), (64, 150, 0.0), (128, 70, 30.0)])
def test_attn_prefill_of_many_sequences(hd, window, cap, prefill_kernel):
    """Forty sequences of 1 to 400 tokens at 8 heads: several hundred tiles of queries, so the CTAs that stay take
    four or five items each, one after another through the same rings and score buffers (tiles of 1 to 7 key
    tiles, in any order of parity), and the search for a tile's sequence runs over more than 32 sequences."""
    nq, nkv = 8, 4
    ops().attn_set_prefill_kernel(hd, prefill_kernel)
    rng = np.random.default_rng(61)
    lens = [int(n) for n in rng.integers(1, 401, size=40)]
    lens[7], lens[33] = 128, 257                                  # a tile border, and one token over it
    T = sum(lens)
    first = torch.tensor([0] + list(np.cumsum(lens)[:-1]), dtype=torch.int32)
    tok_pos = torch.cat([torch.arange(n) for n in lens]).int()
    tok_seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).int()
    qkv = rnd((T, nq + 2 * nkv, hd), torch.bfloat16, 67)
    d = dev()
    scale = 1.0 / math.sqrt(hd)
    for known in (None, lens):
        out = torch.full((T, nq * hd), 9.0, dtype=torch.bfloat16, device=d)
        ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, scale, cap, window,
                           seq_len=torch.tensor(lens, dtype=torch.int32, device=d), host_lens=known)
        if known is None:
            want = torch.empty((T, nq * hd), dtype=torch.float64)
            R.attn_prefill(qkv.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, scale, cap, window)
        close(out, want, 2 * BF16_TOL, "attn_prefill of forty sequences")
    assert ops().attn_tc05_timeouts(hd) == 0


@pytest.mark.parametrize("window", [0, 1024])
def test_attn_prefill_forms_agree_on_a_large_step(window):
    """A step of more than nine thousand tokens at Gemma2-2B's head shape (too large for the plain statement in a
    test's time): the two forms of the tcgen05 kernel walk the same tiles in the same order and give the same
    bits, and the mma.sync kernel agrees with them within the tolerance of bfloat16 outputs."""
    nq, nkv, hd = 8, 4, 256
    lens = [4096, 1500, 3000, 777]
    T = sum(lens)
    d = dev()
    first = torch.tensor([0] + list(np.cumsum(lens)[:-1]), dtype=torch.int32, device=d)
    tok_pos = torch.cat([torch.arange(n) for n in lens]).int().to(d)
    tok_seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).int().to(d)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=d)
    qkv = rnd((T, nq + 2 * nkv, hd), torch.bfloat16, 83)
    outs = {}
    try:
        for which in (3, 2, 0):
            ops().attn_set_prefill_kernel(hd, which)
            out = torch.full((T, nq * hd), 9.0, dtype=torch.bfloat16, device=d)
            ops().attn_prefill(qkv, tok_pos, tok_seq, first, out, nq, nkv, hd, 1.0 / math.sqrt(hd), 50.0, window,
                               seq_len=seq_len, host_lens=lens)
            outs[which] = out
    finally:
        ops().attn_set_prefill_kernel(hd, 1)
    assert torch.isfinite(outs[3].float()).all()
    assert torch.equal(outs[3], outs[2])
    # (each kernel is held to 2 x BF16_TOL of the exact result elsewhere: to each other they may differ by twice that)
    close(outs[3], outs[0].double().cpu(), 4 * BF16_TOL, "tcgen05 against mma.sync on a large step")
    assert ops().attn_tc05_timeouts(hd) == 0


@pytest.mark.parametrize("window", [0, 600])
def test_attn_prefill_of_a_long_prompt(window, prefill_kernel):
    """A prompt of many tiles next to short ones (no tile is shared: the step has enough of them)."""
    nq, nkv, hd = 4, 2, 128
    ops().attn_set_prefill_kernel(hd, prefill_kernel)
    lens = [1500, 70, 900]
    T = sum(lens)
    first = torch.tensor([0] + list(np.cumsum(lens)[:-1]), dtype=torch.int32)
    tok_pos = torch.cat([torch.arange(n) for n in lens]).int()
    tok_seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).int()
    qkv = rnd((T, nq + 2 * nkv, hd), torch.bfloat16, 53)
    if window == 0:
        qkv[0, nq] = qkv[1499, 0] * 3.0            # position 0 of the long prompt answers its last query
    d = dev()
    n = ops().attn_prefill_scratch_floats(T, len(lens), nq, hd)
    scratch = torch.empty((n,), dtype=torch.float32, device=d) if n else None
    out = torch.full((T, nq * hd), 9.0, dtype=torch.bfloat16, device=d)
    ops().attn_prefill(qkv, tok_pos.to(d), tok_seq.to(d), first.to(d), out, nq, nkv, hd, 1.0 / math.sqrt(hd), 50.0, window,
                       seq_len=torch.tensor(lens, dtype=torch.int32, device=d), scratch=scratch)
    want = torch.empty((T, nq * hd), dtype=torch.float64)
    R.attn_prefill(qkv.cpu(), tok_pos, tok_seq, first, want, nq, nkv, hd, 1.0 / math.sqrt(hd), 50.0, window)
    close(out, want, 2 * BF16_TOL, "attn_prefill of a long prompt")
    assert ops().attn_tc05_timeouts(hd) == 0


def test_a_wait_that_nothing_ends_gives_up_and_returns():
    """The kernels' waits are bounded: a barrier nobody completes makes the wait return a status, the host
    reads it, and the device goes on working."""
    hd = 96                                    # a library whose counter no other test expects to be zero
    before = ops().attn_wait_timeouts(hd)
    assert ops().attn_wait_probe(hd, tries=32) == 1
    assert ops().attn_wait_timeouts(hd) == before + 1
    x = rnd((3, 64), torch.float32, 90)
    out = torch.empty_like(x)
    ops().rmsnorm(x, torch.ones(64, device=dev()), 1e-6, out)
    assert torch.isfinite(out).all()


def test_attn_decode_marks_an_undersized_launch():
    nq, nkv, hd = 2, 1, 32
    d = dev()
    k, v = _paged(8, nkv, hd, torch.float32, 33)
    qkv = rnd((1, nq + 2 * nkv, hd), torch.float32, 34)
    table = torch.arange(8, dtype=torch.int32).view(1, 8).to(d)
    scratch = torch.empty(ops().attn_decode_scratch_floats(1, nq, hd, 1), dtype=torch.float32, device=d)
    out = torch.zeros((1, nq * hd), dtype=torch.float32, device=d)
    ops().attn_decode(qkv, k, v, table, torch.tensor([0], dtype=torch.int32, device=d),
                      torch.tensor([200], dtype=torch.int32, device=d), scratch, out, nq, nkv, hd, 1.0, 0.0, 0, 0, 64, 1)
    assert torch.isnan(out).all()
    # the same through the kernel that writes its result itself when a launch has one chunk per sequence
    outb = torch.zeros((1, nq * hd), dtype=torch.bfloat16, device=d)
    ops().attn_decode(qkv.bfloat16(), k.bfloat16(), v.bfloat16(), table, torch.tensor([0], dtype=torch.int32, device=d),
                      torch.tensor([200], dtype=torch.int32, device=d), scratch, outb, nq, nkv, hd, 1.0, 0.0, 0, 0, 64, 1)
    assert torch.isnan(outb.float()).all()
    # and with chunks to merge: two chunks where four are needed, beside a sequence that fits; then a launch of the
    # right size over the same scratch
    lens = torch.tensor([200, 100], dtype=torch.int32, device=d)
    table2 = torch.arange(8, dtype=torch.int32).view(2, 4).to(d)
    q2 = rnd((2, nq + 2 * nkv, hd), torch.bfloat16, 36)
    kb, vb = k.bfloat16(), v.bfloat16()
    scratch2 = torch.empty(ops().attn_decode_scratch_floats(2, nq, hd, 4), dtype=torch.float32, device=d)
    out2 = torch.zeros((2, nq * hd), dtype=torch.bfloat16, device=d)
    slots2 = torch.tensor([0, 1], dtype=torch.int32, device=d)
    ops().attn_decode(q2, kb, vb, table2, slots2, lens, scratch2, out2, nq, nkv, hd, 1.0, 0.0, 0, 0, 64, 2)
    assert torch.isnan(out2[0].float()).all() and torch.isfinite(out2[1].float()).all()
    ops().attn_decode(q2, kb, vb, table2, slots2, lens, scratch2, out2, nq, nkv, hd, 1.0, 0.0, 0, 0, 64, 4)
    want = torch.empty((2, nq * hd), dtype=torch.float64)
    R.attn_decode(q2.cpu(), kb.cpu(), vb.cpu(), table2.cpu(), slots2.cpu(), lens.cpu(), None, want, nq, nkv, hd, 1.0, 0.0, 0, 0, 64, 4)
    close(out2, want, BF16_TOL, "attn_decode after an undersized launch")


@pytest.mark.parametrize("Rn,V", [(1, 7), (5, 384), (3, 256000), (64, 1000), (2, 50003), (8, 32001), (32, 16384), (33, 20000)])
def test_argmax_lowest_id_wins(Rn, V):
    logits = rnd((Rn, V), torch.float32, 35)
    logits[0, V // 2] = 50.0
    logits[0, V - 1] = 50.0
    if Rn > 1:
        logits[1, 0] = 50.0
        logits[1, 3] = 50.0
    out = torch.empty((Rn,), dtype=torch.int32, device=dev())
    ops().argmax(logits, out)
    want = torch.empty((Rn,), dtype=torch.int32)
    R.argmax(logits.cpu(), want)
    assert out.cpu().tolist() == want.tolist()
    assert out[0].item() == V // 2


@pytest.fixture(params=[1, 0], ids=["shared", "global"])
def sample_kernel(request):
    """Both sampling kernels: the row's weights in the shared memory of a cluster, and every pass over global memory."""
    ops().set_sample_kernel(request.param)
    yield request.param
    ops().set_sample_kernel(1)


# 50 to 5,000: one CTA a row; 46,081 and 70,001: clusters of 2 (an odd vocabulary: stretches that are not
# multiples of 4); 150,000: 4; 256,000: 8; 400,000: too large for a cluster's shared memory, the other kernel
@pytest.mark.parametrize("V", [50, 384, 5000, 46081, 70001, 150000, 256000, 400000])
@pytest.mark.parametrize("temp,top_p", [(1.0, 1.0), (0.6, 0.95), (0.3, 0.5), (1.0, 0.05)])
def test_sample_matches_the_host_sampler(V, temp, top_p, sample_kernel):
    Rn = 6 if V <= 256000 else 2
    spread = [0.5, 2.0, 8.0][V % 3]
    logits = rnd((Rn, V), torch.float32, 36, std=spread)
    d = dev()
    ids = torch.arange(100, 100 + Rn, dtype=torch.int32, device=d)
    idx = torch.arange(Rn, dtype=torch.int32, device=d) * 3
    out = torch.empty((Rn,), dtype=torch.int32, device=d)
    u = torch.empty((Rn,), dtype=torch.float32, device=d)
    ops().sample(logits, out, temp, top_p, 1234567, ids, idx, u)
    for r in range(Rn):
        u_ref = R.philox_uniform(1234567, 100 + r, 3 * r)
        assert abs(u[r].item() - u_ref) < 1e-7
        assert out[r].item() == R.sample_row(logits[r].cpu(), temp, top_p, u_ref), f"row {r}"


def test_sample_with_ties_at_the_nucleus_edge(sample_kernel):
    V = 40
    logits = torch.zeros((1, V), dtype=torch.float32, device=dev())     # all equal: the nucleus is the first ids
    d = dev()
    seen = set()
    for i in range(200):
        out = torch.empty((1,), dtype=torch.int32, device=d)
        ops().sample(logits, out, 1.0, 0.25, 99, torch.tensor([i], dtype=torch.int32, device=d),
                     torch.tensor([0], dtype=torch.int32, device=d))
        seen.add(out.item())
    assert seen == set(range(10))


def test_sample_with_ties_across_the_ctas_of_a_cluster():
    """All logits equal over a vocabulary that a cluster of 8 shares: the nucleus is the lowest tenth of the ids,
    whichever CTA holds them, and every one of them can be drawn."""
    V = 256000
    d = dev()
    logits = torch.zeros((64, V), dtype=torch.float32, device=d)
    out = torch.empty((64,), dtype=torch.int32, device=d)
    ops().sample(logits, out, 1.0, 0.1, 7, torch.arange(64, dtype=torch.int32, device=d),
                 torch.zeros(64, dtype=torch.int32, device=d))
    got = out.cpu()
    assert int(got.min()) >= 0 and int(got.max()) < 25601 and len(set(got.tolist())) > 50
    assert int(got.max()) > 12800                      # and from all over that tenth (64 draws: the upper half is met)
    # top_p = 0.5: the kept ids span four CTAs' stretches (32,000 ids each)
    ops().sample(logits, out, 1.0, 0.5, 8, torch.arange(64, dtype=torch.int32, device=d),
                 torch.zeros(64, dtype=torch.int32, device=d))
    got = out.cpu()
    assert int(got.max()) < 128001 and len({int(t) // 32000 for t in got.tolist()}) == 4


def test_sample_does_not_depend_on_the_batch(sample_kernel):
    V = 1000
    logits = rnd((4, V), torch.float32, 37, std=3.0)
    d = dev()
    ids = torch.tensor([5, 6, 7, 8], dtype=torch.int32, device=d)
    idx = torch.tensor([0, 1, 2, 3], dtype=torch.int32, device=d)
    out = torch.empty((4,), dtype=torch.int32, device=d)
    ops().sample(logits, out, 0.8, 0.9, 42, ids, idx)
    one = torch.empty((1,), dtype=torch.int32, device=d)
    ops().sample(logits[2:3].contiguous(), one, 0.8, 0.9, 42, ids[2:3].contiguous(), idx[2:3].contiguous())
    assert one.item() == out[2].item()


def test_repeat_penalty_and_mask():
    V = 100
    logits = rnd((2, V), torch.float32, 38)
    ref = logits.cpu().clone()
    recent = torch.tensor([[3, 3, 7, -1], [99, 0, 0, 5]], dtype=torch.int32)
    ops().repeat_penalty(logits, recent.to(dev()), 1.3)
    R.repeat_penalty(ref, recent, 1.3)
    close(logits, ref, 1e-6, "repeat penalty")
    ids = torch.tensor([1, 50], dtype=torch.int32)
    ops().mask_tokens(logits, ids.to(dev()))
    assert torch.isinf(logits[:, 1]).all() and torch.isinf(logits[:, 50]).all()
    assert torch.isfinite(logits[:, 2]).all()
