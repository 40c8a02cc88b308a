"""tcgen05 GEMM against an fp32 PyTorch reference (and its fused epilogues)."""
import pytest
import torch

from pie_b200 import ops
from pie_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(torch.bfloat16)


def check(y, want, k):
    err = (y.float() - want.float()).abs().max().item()
    # bf16 output rounding (2^-8 relative) + fp32 accumulation over k terms
    tol = 2e-2 * want.float().abs().max().item() + 1e-3 * k ** 0.5
    assert err <= tol, f"max err {err} > {tol}"
    ops.check_kernel_status()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 4096), (1, 6144, 4096),
                                   (77, 4096, 4096), (512, 6144, 4096), (300, 1000, 328), (2048, 14336, 4096),
                                   (130, 128256, 256)])
@pytest.mark.parametrize("bn", [0, 64, 128, 256])
def test_gemm_plain(m, n, k, bn):
    if bn and (m * n > 4096 * 4096) and bn != 256:
        pytest.skip("large shape only with the automatic tile choice")
    x, w = bf(m, k, seed=1), bf(n, k, scale=0.05, seed=2)
    y = ops.gemm(x, w, force_bn=bn)
    check(y, x.float() @ w.float().t(), k)


@pytest.mark.parametrize("m,n,k", [(512, 6144, 4096), (512, 4096, 14336), (512, 768, 4096), (64, 4096, 4096),
                                   (300, 2048, 8192), (512, 28672, 4096)])
@pytest.mark.parametrize("epi", ["store", "residual", "swiglu"])
def test_gemm_stream_k_matches_whole_tile_and_reference(m, n, k, epi):
    """Skinny shapes take the stream-K schedule (split tiles fixed up through the workspace);
    force_bn=-1 forces whole-tile scheduling of the same kernel."""
    x, w = bf(m, k, seed=11), bf(n, k, scale=0.03, seed=12)
    r = bf(m, n, seed=13) if epi == "residual" else None
    e = {"store": ops.EPI_STORE, "residual": ops.EPI_RESIDUAL, "swiglu": ops.EPI_SWIGLU}[epi]
    for rep in range(2):     # twice: the arrival counters must be back at zero
        y = ops.gemm(x, w, residual=r, epilogue=e)
    y_dp = ops.gemm(x, w, residual=r, epilogue=e, force_bn=-1)
    want = x.float() @ w.float().t()
    if epi == "residual":
        want = want + r.float()
    if epi == "swiglu":
        want = ref.swiglu_interleaved(want)
    check(y, want, k)
    check(y_dp, want, k)


def test_gemm_residual():
    m, n, k = 333, 4096, 1024
    x, w, r = bf(m, k, seed=3), bf(n, k, scale=0.05, seed=4), bf(m, n, seed=5)
    y = ops.gemm(x, w, residual=r, epilogue=ops.EPI_RESIDUAL)
    check(y, x.float() @ w.float().t() + r.float(), k)


def test_gemm_swiglu():
    m, n, k = 200, 2 * 1408, 512
    x, w = bf(m, k, seed=6), bf(n, k, scale=0.05, seed=7)
    y = ops.gemm(x, w, epilogue=ops.EPI_SWIGLU)
    want = ref.swiglu_interleaved((x.float() @ w.float().t()))
    assert y.shape == (m, n // 2)
    check(y, want, k)


def test_gemm_strided_operands():
    m, n, k = 96, 512, 256
    big = bf(m, 3 * k, seed=8)
    x = big[:, k:2 * k]                      # row stride 3k
    w = bf(n, k, scale=0.05, seed=9)
    out = torch.zeros(m, 2 * n, dtype=torch.bfloat16, device=DEV)
    ops.gemm(x, w, out=out[:, n:])
    check(out[:, n:], x.float() @ w.float().t(), k)
    assert float(out[:, :n].abs().max()) == 0.0


@pytest.mark.parametrize("bn", [16, 48, 80, 112, 176, 208, 240])
@pytest.mark.parametrize("epi", ["store", "residual", "swiglu"])
def test_gemm_odd_tile_widths(bn, epi):
    """Tile widths between the native 64/128/256 (chosen to fill the machine's waves): the last
    tile of a row is ragged and the SwiGLU epilogue halves the column index."""
    m, n, k = 200, 2000 if epi != "swiglu" else 2016, 1024
    x, w = bf(m, k, seed=21), bf(n, k, scale=0.04, seed=22)
    r = bf(m, n, seed=23) if epi == "residual" else None
    e = {"store": ops.EPI_STORE, "residual": ops.EPI_RESIDUAL, "swiglu": ops.EPI_SWIGLU}[epi]
    ops.set_gemm_pairs(False)
    try:
        y = ops.gemm(x, w, residual=r, epilogue=e, force_bn=-bn)
    finally:
        ops.set_gemm_pairs(True)
    want = x.float() @ w.float().t()
    if epi == "residual":
        want = want + r.float()
    if epi == "swiglu":
        want = ref.swiglu_interleaved(want)
    check(y, want, k)


@pytest.mark.parametrize("m", [1, 7, 64, 65, 100, 128])
@pytest.mark.parametrize("n,k", [(6144, 4096), (4096, 14336), (1000, 512), (28672, 4096)])
@pytest.mark.parametrize("epi", ["store", "residual", "swiglu"])
def test_gemm_swapped_operands_small_batch(m, n, k, epi):
    """Batches of at most 128 rows run C^T = W A^T (weights on the 128-row side, transposed epilogue):
    same result as the direct orientation and as the fp32 reference, ragged feature counts included."""
    if epi == "swiglu" and n % 32:
        n = 992
    x, w = bf(m, k, seed=31), bf(n, k, scale=0.03, seed=32)
    r = bf(m, n, seed=33) if epi == "residual" else None
    e = {"store": ops.EPI_STORE, "residual": ops.EPI_RESIDUAL, "swiglu": ops.EPI_SWIGLU}[epi]
    ops.set_gemm_swap(1000)      # every shape, not only those the selection rule picks
    try:
        y = ops.gemm(x, w, residual=r, epilogue=e)
        ops.set_gemm_swap(0)
        y0 = ops.gemm(x, w, residual=r, epilogue=e)
    finally:
        ops.set_gemm_swap(128)
    ref = x.float() @ w.float().t()
    if epi == "residual":
        ref = ref + r.float()
    if epi == "swiglu":
        ref = torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
    check(y, ref, k)
    check(y0, ref, k)
    ops.check_kernel_status()
