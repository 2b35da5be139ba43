"""tcgen05 GEMM against a PyTorch fp32 restatement, all operand layouts and edge shapes."""
import pytest
import torch

from maltos_b200.ops import _lib
from maltos_b200.ops.gemm import gemm, linear

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    return af @ bf


def _mk(M, N, K, a_mn, b_mn, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).to(torch.bfloat16)
    return a, b


def _rel_err(c, ref):
    return ((c.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (200, 328, 136), (4096, 1024, 512)])
@pytest.mark.parametrize("block_n", [128, 256, 512, 1024])   # 512 / 1024 = CTA-pair kernels (cta_group::2), 256x256 / 256x512 tiles
def test_gemm_layouts(a_mn, b_mn, shape, block_n):
    M, N, K = shape
    a, b = _mk(M, N, K, a_mn, b_mn)
    c = gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=block_n)
    _lib.fetch_status()
    ref = _ref(a, b, a_mn, b_mn)
    assert _rel_err(c, ref) < 1e-2


def test_gemm_pair_kernel_many_tiles_per_pair():
    """More 256x256 tiles than SM pairs, several trips round the stage ring, ragged M/N/K edges, fp32 accumulate."""
    M, N, K = 4000, 5000, 1096
    a, b = _mk(M, N, K, False, False, seed=3)
    ref = _ref(a, b, False, False)
    for block_n in (512, 1024):
        c = gemm(a, b, block_n=block_n)
        _lib.fetch_status()
        assert _rel_err(c, ref) < 1e-2
        out = torch.ones((M, N), device="cuda", dtype=torch.float32)
        gemm(a, b, out=out, accumulate=True, block_n=block_n)
        _lib.fetch_status()
        assert _rel_err(out, ref + 1.0) < 2e-3


@pytest.mark.parametrize("shape", [(512, 1024, 9216), (1000, 1496, 8768), (8192, 4096, 8704), (2560, 512, 16384)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, True)])
def test_gemm_split_tail_of_the_wide_kernel(shape, a_mn, b_mn):
    """Few tiles in the last wave and a long k range: the 256x512 kernel computes each tail tile on several CTA pairs
    over disjoint k ranges and the warp that finishes last sums the fp32 partials. Same results as without the split,
    for plain, ragged, accumulating, fp32 and biased outputs."""
    import ctypes

    M, N, K = shape
    a, b = _mk(M, N, K, a_mn, b_mn, seed=7)
    ref = _ref(a, b, a_mn, b_mn)
    lib = _lib.lib()
    for split in (1, 0):
        lib.mb_gemm_set_tail_split(ctypes.c_int(split))
        try:
            c = gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=1024)
            _lib.fetch_status()
            assert _rel_err(c, ref) < 1e-2, split
            bias = torch.randn(N, device="cuda").to(torch.bfloat16)
            out = torch.ones((M, N), device="cuda", dtype=torch.float32)
            gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=True, bias=bias, block_n=1024)
            _lib.fetch_status()
            assert _rel_err(out, ref + bias.float() + 1.0) < 2e-3, split
        finally:
            lib.mb_gemm_set_tail_split(ctypes.c_int(1))
    # twice in a row on the same stream: the counters are re-armed by every launch
    c2 = gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=1024)
    assert torch.equal(c2, gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=1024))


def test_gemm_fp32_accumulate_and_bias():
    M, N, K = 256, 384, 512
    a, b = _mk(M, N, K, False, False, seed=1)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    out = torch.ones((M, N), device="cuda", dtype=torch.float32)
    gemm(a, b, out=out, accumulate=True, bias=bias)
    _lib.fetch_status()
    ref = _ref(a, b, False, False) + bias.float() + 1.0
    assert _rel_err(out, ref) < 2e-3
    outb = torch.ones((M, N), device="cuda", dtype=torch.bfloat16)
    gemm(a, b, out=outb, accumulate=True)
    ref2 = _ref(a, b, False, False) + 1.0
    assert _rel_err(outb, ref2) < 1e-2


def test_gemm_strided_output_and_many_tiles():
    M, N, K = 1024, 2048, 320
    a, b = _mk(M, N, K, False, False, seed=2)
    big = torch.zeros((M, N + 64), device="cuda", dtype=torch.bfloat16)
    gemm(a, b, out=big[:, :N])
    _lib.fetch_status()
    assert _rel_err(big[:, :N], _ref(a, b, False, False)) < 1e-2
    assert big[:, N:].abs().max().item() == 0


def test_linear_autograd_matches_fp32():
    torch.manual_seed(0)
    x = torch.randn(2, 192, 256, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (torch.randn(384, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    y = linear(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = torch.nn.functional.linear(xf, wf)
    yf.backward(dy.float())
    assert _rel_err(y, yf.detach()) < 1e-2
    assert _rel_err(x.grad, xf.grad) < 1e-2
    assert _rel_err(w.grad, wf.grad) < 1e-2
    _lib.fetch_status()
