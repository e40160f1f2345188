"""The tcgen05 skinny product (TMA-fed, accumulator in tensor memory, K split over a cluster) against
the plain statement of the product, at sizes that are no multiples of its tiles."""
from __future__ import annotations

import pytest
import torch

from tests import kernel_refs as R

pytestmark = pytest.mark.gpu


def ops():
    from janis_b200.kernels import ops as o
    return o


def rnd(shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(torch.bfloat16).to("cuda:0")


def check(M, N, K, epi, split, out_dtype=torch.float32, cap=7.0):
    x = rnd((M, K), 70 + M)
    w = rnd((N, K), 71 + N, std=0.1)
    n_out = N // 2 if epi in (1, 3) else N
    out = torch.full((M, n_out), 5.0, dtype=out_dtype, device="cuda:0")
    ops().gemm_tc05(x, w, out, epi, cap, split)
    want = torch.empty((M, n_out), dtype=torch.float64)
    R.gemv_bf16(x.cpu(), w.cpu(), want, epi, cap)
    got = out.double().cpu()
    assert torch.isfinite(got).all()
    scale = want.abs().max().item()
    err = (got - want).abs().max().item()
    tol = 1e-4 if out_dtype == torch.float32 else 2.0 ** -8 + 1e-4
    assert err <= tol * scale, f"M={M} N={N} K={K} epi={epi} split={split}: {err:.3e} vs {scale:.3e}"
    assert ops().tc05_timeouts() == 0


@pytest.mark.parametrize("M", [1, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K", [(128, 64), (256, 128), (2304, 2048), (1000, 328), (40, 72)])
def test_product(M, N, K):
    check(M, N, K, 0, 1)


@pytest.mark.parametrize("split", [2, 4, 8, 0])
@pytest.mark.parametrize("M,N,K", [(64, 2304, 9216), (20, 384, 96), (48, 128, 1032), (33, 4096, 2304)])
def test_k_split_over_a_cluster(split, M, N, K):
    check(M, N, K, 0, split)


@pytest.mark.parametrize("epi", [1, 2, 3])
@pytest.mark.parametrize("M,N,K", [(64, 18432, 2304), (17, 640, 96), (40, 2000, 104)])
def test_epilogues(epi, M, N, K):
    if epi in (1, 3) and N % 16:
        pytest.skip("gated rows come in groups of 16")
    check(M, N, K, epi, 0)
    check(M, N, K, epi, 0, out_dtype=torch.bfloat16)


@pytest.mark.parametrize("stages", [3, 4, 9])
@pytest.mark.parametrize("M,N,K,epi", [(64, 2304, 2048, 0), (17, 1002, 328, 0), (33, 1002, 328, 2), (40, 2000, 1032, 1),
                                       (5, 18, 8, 0)])
def test_depth_of_the_ring_and_row_stores(stages, M, N, K, epi):
    """Every depth of the ring of stages (more stages than K has tiles too), outputs whose rows allow 16-byte
    stores and outputs whose rows do not (N = 1002, 18)."""
    ops().tc05_set_stages(stages)
    try:
        check(M, N, K, epi, 1)
        check(M, N, K, epi, 1, out_dtype=torch.bfloat16)
    finally:
        ops().tc05_set_stages(0)
