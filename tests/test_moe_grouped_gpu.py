"""Grouped expert GEMMs with device-side row counts (``csrc/grouped_gemm.cu``) against per-expert fp32 matmuls."""
import pytest
import torch

from maltos_b200.ops import _lib
from maltos_b200.ops.moe import grouped_gemm, grouped_swiglu_experts

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, ref, tol=2e-2):
    err = (got.float() - ref).abs().max().item()
    assert torch.isfinite(got.float()).all()
    assert err <= tol * max(ref.abs().max().item(), 1e-3), (err, ref.abs().max().item())


@pytest.mark.parametrize("G,cap,K,N,counts", [(4, 256, 128, 320, [256, 0, 130, 1]), (8, 128, 256, 256, [5, 128, 64, 0, 127, 128, 33, 90]),
                                              (3, 384, 512, 1000, [384, 200, 65])])
def test_grouped_gemm_three_modes(G, cap, K, N, counts):
    torch.manual_seed(0)
    cnt = torch.tensor(counts, dtype=torch.int32, device=DEV)
    a = torch.zeros(G * cap, K, device=DEV, dtype=torch.bfloat16)
    for g, n in enumerate(counts):
        a[g * cap:g * cap + n] = torch.randn(n, K, device=DEV).bfloat16()
    w_nk = [(torch.randn(N, K, device=DEV) * 0.1).bfloat16() for _ in range(G)]
    w_kn = [(torch.randn(K, N, device=DEV) * 0.1).bfloat16() for _ in range(G)]
    y0 = grouped_gemm(0, a, w_nk, cnt, cap)
    y1 = grouped_gemm(1, a, w_kn, cnt, cap)
    b = torch.zeros(G * cap, N, device=DEV, dtype=torch.bfloat16)
    for g, n in enumerate(counts):
        b[g * cap:g * cap + n] = torch.randn(n, N, device=DEV).bfloat16()
    y2 = grouped_gemm(2, a, [b], cnt, cap, out_dtype=torch.float32)
    for g, n in enumerate(counts):
        rows = slice(g * cap, g * cap + n)
        if n:
            _close(y0[rows], a[rows].float() @ w_nk[g].float().t())
            _close(y1[rows], a[rows].float() @ w_kn[g].float())
        assert float(y0[g * cap + (n + 127) // 128 * 128:(g + 1) * cap].abs().max() if (n + 127) // 128 * 128 < cap else 0.0) == 0.0
        _close(y2[g], a[rows].float().t() @ b[rows].float() if n else torch.zeros(K, N, device=DEV), tol=2e-2)
    _lib.fetch_status()


def test_grouped_swiglu_experts_match_per_expert_autograd():
    torch.manual_seed(1)
    G, cap, H, F = 4, 128, 256, 384
    counts = [100, 0, 128, 37]
    cnt = torch.tensor(counts, dtype=torch.int32, device=DEV)
    x = torch.zeros(G * cap, H, device=DEV, dtype=torch.bfloat16)
    for g, n in enumerate(counts):
        x[g * cap:g * cap + n] = torch.randn(n, H, device=DEV).bfloat16()
    x.requires_grad_(True)
    mk = lambda *s: torch.nn.Parameter((torch.randn(*s, device=DEV) * 0.05).bfloat16())   # noqa: E731
    gates, ups, downs = [mk(F, H) for _ in range(G)], [mk(F, H) for _ in range(G)], [mk(H, F) for _ in range(G)]
    before = _lib.launch_count()
    y = grouped_swiglu_experts(x, cnt, cap, gates, ups, downs)
    dy = torch.zeros_like(y)
    for g, n in enumerate(counts):
        dy[g * cap:g * cap + n] = torch.randn(n, H, device=DEV).bfloat16()
    y.backward(dy)
    assert _lib.launch_count() - before <= 13         # 3 + 7 grouped GEMMs and the SwiGLU kernels, whatever the expert count
    for g, n in enumerate(counts):
        rows = slice(g * cap, g * cap + n)
        xf = x.detach()[rows].float().requires_grad_(True)
        wg, wu, wd = (w.detach().float().requires_grad_(True) for w in (gates[g], ups[g], downs[g]))
        ref = (torch.nn.functional.silu(xf @ wg.t()) * (xf @ wu.t())) @ wd.t()
        ref.backward(dy[rows].float())
        if n:
            _close(y[rows], ref.detach(), 3e-2)
            _close(x.grad[rows], xf.grad, 3e-2)
        _close(gates[g].grad, wg.grad if n else torch.zeros_like(wg), 3e-2)
        _close(ups[g].grad, wu.grad if n else torch.zeros_like(wu), 3e-2)
        _close(downs[g].grad, wd.grad if n else torch.zeros_like(wd), 3e-2)
    _lib.fetch_status()


def test_single_device_capacity_path_is_static_and_matches_the_per_expert_loop():
    from maltos_b200.models.tiny_moe_transformer import TopKMoE
    from maltos_b200.ops import moe as moe_ops

    torch.manual_seed(2)
    layer = TopKMoE(128, 256, 8, top_k=2, capacity_factor=1.0).to(DEV).bfloat16()
    x = torch.randn(2, 96, 128, device=DEV).bfloat16()
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya, aux = layer(xa, return_aux_loss=True)                       # grouped path (capacity set, SwiGLU experts, CUDA bf16)
    ya.float().pow(2).mean().backward()
    ga = [p.grad.clone() for p in layer.parameters()]
    for p in layer.parameters():
        p.grad = None
    orig = moe_ops.swiglu_expert_weights
    moe_ops.swiglu_expert_weights = lambda *a, **k: None           # force the per-expert loop with host-read counts
    try:
        yb = layer(xb)
    finally:
        moe_ops.swiglu_expert_weights = orig
    yb.float().pow(2).mean().backward()
    _close(ya, yb.float(), 3e-2)
    _close(xa.grad, xb.grad.float(), 3e-2)
    for a, p in zip(ga, layer.parameters()):
        _close(a, p.grad.float(), 4e-2)
    _lib.fetch_status()
