"""sm_100a layer kernels against their PyTorch fp32 restatements."""
import pytest
import torch
import torch.nn.functional as F

from maltos_b200.ops import _lib
from maltos_b200.ops.cross_entropy import cross_entropy_mean, linear_cross_entropy
from maltos_b200.ops.grouped import fuse_parameters, grouped_linear
from maltos_b200.ops.norm import add_rms_norm, rms_norm, rms_norm_reference
from maltos_b200.ops.optim import adamw_multi_tensor, clip_coefficient, scale_tensors_, sum_of_squares
from maltos_b200.ops.rope import apply_rope, build_rope_cache, rope_qkv_split, rope_reference
from maltos_b200.ops.swiglu import swiglu, swiglu_packed

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item()
    assert err <= tol * max(ref, 1e-3), f"max err {err} vs ref scale {ref}"


@pytest.mark.parametrize("rows,H", [(7, 64), (300, 512), (1024, 4096), (5, 16384)])
def test_rmsnorm_fwd_bwd(rows, H):
    torch.manual_seed(0)
    x = torch.randn(rows, H, device=DEV).bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16().requires_grad_()
    y = rms_norm(x, w, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = rms_norm_reference(xf, wf, 1e-5)
    yf.backward(dy.float())
    _close(y, yf, 1e-2)
    _close(x.grad, xf.grad, 2e-2)
    _close(w.grad, wf.grad, 2e-2)
    _lib.fetch_status()


def test_add_rmsnorm_fused_residual():
    torch.manual_seed(1)
    rows, H = 257, 1024
    a = torch.randn(rows, H, device=DEV).bfloat16().requires_grad_()
    r = torch.randn(rows, H, device=DEV).bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16().requires_grad_()
    y, h = add_rms_norm(a, r, w, 1e-6)
    dy, dh = torch.randn_like(y), torch.randn_like(h)
    torch.autograd.backward([y, h], [dy, dh])
    af, rf, wf = (t.detach().float().requires_grad_() for t in (a, r, w))
    hf = (af + rf).bfloat16().float() + 0 * af  # the residual stream is rounded to bf16 in the kernel too
    hf2 = af + rf
    yf = rms_norm_reference(hf2, wf, 1e-6)
    torch.autograd.backward([yf, hf2], [dy.float(), dh.float()])
    _close(h, hf2, 1e-2)
    _close(y, yf, 2e-2)
    _close(a.grad, af.grad, 2e-2)
    _close(r.grad, rf.grad, 2e-2)
    _close(w.grad, wf.grad, 3e-2)


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_and_qkv_split(interleaved):
    torch.manual_seed(2)
    B, S, hq, hkv, D = 2, 48, 8, 2, 64
    cos, sin = build_rope_cache(128, D, 10000.0, device=DEV)
    pos = torch.randint(0, 128, (B, S), device=DEV)
    x = torch.randn(B, S, hq, D, device=DEV).bfloat16().requires_grad_()
    y = apply_rope(x, cos, sin, position_ids=pos, interleaved=interleaved)
    g = torch.randn_like(y)
    y.backward(g)
    _close(y, rope_reference(x.detach(), cos, sin, pos, interleaved), 1e-2)
    _close(x.grad, rope_reference(g, cos, sin, pos, interleaved, inverse=True), 1e-2)
    W = (hq + 2 * hkv) * D
    qkv = torch.randn(B, S, W, device=DEV).bfloat16().requires_grad_()
    q, k, v = rope_qkv_split(qkv, cos, sin, num_heads=hq, num_kv_heads=hkv, head_dim=D, position_ids=pos, interleaved=interleaved)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    qr = rope_reference(qkv.detach()[..., :hq * D].reshape(B, S, hq, D), cos, sin, pos, interleaved)
    kr = rope_reference(qkv.detach()[..., hq * D:(hq + hkv) * D].reshape(B, S, hkv, D), cos, sin, pos, interleaved)
    _close(q, qr, 1e-2)
    _close(k, kr, 1e-2)
    assert torch.equal(v, qkv.detach()[..., (hq + hkv) * D:].reshape(B, S, hkv, D))
    exp = torch.cat([rope_reference(gq, cos, sin, pos, interleaved, inverse=True).reshape(B, S, -1),
                     rope_reference(gk, cos, sin, pos, interleaved, inverse=True).reshape(B, S, -1), gv.reshape(B, S, -1)], -1)
    _close(qkv.grad, exp, 1e-2)
    _lib.fetch_status()


def test_swiglu_both_forms():
    torch.manual_seed(3)
    T, Fd = 333, 1408
    gu = torch.randn(T, 2 * Fd, device=DEV).bfloat16().requires_grad_()
    out = swiglu_packed(gu)
    d = torch.randn_like(out)
    out.backward(d)
    guf = gu.detach().float().requires_grad_()
    ref = F.silu(guf[:, :Fd]) * guf[:, Fd:]
    ref.backward(d.float())
    _close(out, ref, 1e-2)
    _close(gu.grad, guf.grad, 2e-2)
    g = torch.randn(T, Fd, device=DEV).bfloat16().requires_grad_()
    u = torch.randn(T, Fd, device=DEV).bfloat16().requires_grad_()
    o2 = swiglu(g, u)
    o2.backward(d)
    gf, uf = g.detach().float().requires_grad_(), u.detach().float().requires_grad_()
    (F.silu(gf) * uf).backward(d.float())
    _close(g.grad, gf.grad, 2e-2)
    _close(u.grad, uf.grad, 2e-2)


@pytest.mark.parametrize("V", [1000, 96, 31])       # fewer classes than threads of a block: whole warps see no element
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy(dtype, V):
    torch.manual_seed(4)
    N = 300
    logits = (torch.randn(N, V, device=DEV) * 3).to(dtype).requires_grad_()
    labels = torch.randint(0, V, (N,), device=DEV)
    labels[::7] = -100
    loss = cross_entropy_mean(logits, labels)
    loss.backward()
    lf = logits.detach().float().requires_grad_()
    ref = F.cross_entropy(lf, labels, ignore_index=-100, reduction="sum") / (labels != -100).sum()
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    _close(logits.grad, lf.grad, 3e-2)
    empty = cross_entropy_mean(logits, torch.full_like(labels, -100))
    assert empty.item() == 0.0
    _lib.fetch_status()


@pytest.mark.parametrize("N,H,V", [(700, 256, 2048), (128, 128, 96)])
def test_linear_cross_entropy_matches_unfused(N, H, V):
    torch.manual_seed(5)
    h = torch.randn(N, H, device=DEV).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device=DEV) * 0.05).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (N,), device=DEV)
    labels[:50] = -100
    loss = linear_cross_entropy(h, w, labels, chunk_tokens=256)
    (loss * 0.5).backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = F.cross_entropy(hf @ wf.t(), labels, ignore_index=-100, reduction="sum") / (labels != -100).sum()
    (ref * 0.5).backward()
    assert abs(loss.item() - ref.item()) < 5e-3 * abs(ref.item())
    _close(h.grad, hf.grad, 3e-2)
    _close(w.grad, wf.grad, 3e-2)
    _lib.fetch_status()


def test_grouped_linear_fused_and_unfused():
    torch.manual_seed(6)
    K = 256
    ws = [torch.nn.Parameter((torch.randn(n, K, device=DEV) * 0.05).bfloat16()) for n in (512, 128, 128)]
    x = torch.randn(3, 40, K, device=DEV).bfloat16().requires_grad_()
    for fused in (False, True):
        if fused:
            fuse_parameters(ws)
        for w in ws:
            w.grad = None
        x.grad = None
        out, offs = grouped_linear(x, ws)
        assert offs == [0, 512, 640]
        d = torch.randn_like(out)
        out.backward(d)
        xf = x.detach().float().requires_grad_()
        wf = [w.detach().float().requires_grad_() for w in ws]
        ref = torch.cat([xf @ w.t() for w in wf], -1)
        ref.backward(d.float())
        _close(out, ref, 1e-2)
        _close(x.grad, xf.grad, 2e-2)
        for w, r in zip(ws, wf):
            _close(w.grad, r.grad, 2e-2)
    _lib.fetch_status()


def test_adamw_and_norm_kernels():
    torch.manual_seed(7)
    shapes = [(1000,), (33, 77), (5000, 13)]
    ps = [torch.randn(s, device=DEV) for s in shapes]
    gs = [torch.randn(s, device=DEV).bfloat16() if i % 2 == 0 else torch.randn(s, device=DEV) for i, s in enumerate(shapes)]
    ms = [torch.zeros_like(p) for p in ps]
    vs = [torch.zeros_like(p) for p in ps]
    lows = [p.bfloat16() for p in ps]
    ref_p = [p.clone() for p in ps]
    ref_opt = torch.optim.AdamW([torch.nn.Parameter(p) for p in ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    scale = torch.tensor([0.5], device=DEV)
    for step in (1, 2, 3):
        for rp, g in zip(ref_opt.param_groups[0]["params"], gs):
            rp.grad = g.float() * 0.5
        ref_opt.step()
        adamw_multi_tensor([(p, g, m, v, lo, float(step)) for p, g, m, v, lo in zip(ps, gs, ms, vs, lows)], lr=1e-2, beta1=0.9,
                           beta2=0.95, eps=1e-8, weight_decay=0.1, grad_scale=scale)
    for p, rp, lo in zip(ps, ref_opt.param_groups[0]["params"], lows):
        assert (p - rp.detach()).abs().max().item() < 1e-5
        assert torch.equal(lo, p.bfloat16())
    ss = sum_of_squares(gs, [1.0, 0.5, 1.0])
    ref = sum(w * g.double().pow(2).sum() for g, w in zip(gs, [1.0, 0.5, 1.0]))
    assert abs(ss.item() - ref.item()) < 1e-3 * ref.item()
    coef, norm = clip_coefficient(ss, 1.0)
    assert abs(norm.item() - ref.sqrt().item()) < 1e-3 * ref.sqrt().item()
    assert abs(coef.item() - 1.0 / (ref.sqrt().item() + 1e-6)) < 1e-5
    before = [g.clone() for g in gs]
    scale_tensors_(gs, coef)
    for g, b in zip(gs, before):
        _close(g, b.float() * coef.item(), 1e-2)
    _lib.fetch_status()


def test_adamw_takes_non_contiguous_gradients_of_equal_size():
    """Two same-sized transposed gradients: their contiguous copies are temporaries whose addresses go into the launch
    table, so both must stay allocated until the launch (a freed block would be reused by the second copy)."""
    from maltos_b200.ops.optim import _adamw_reference

    torch.manual_seed(11)
    ps = [torch.randn(64, 48, device=DEV) for _ in range(3)]
    gs = [torch.randn(48, 64, device=DEV).t() for _ in range(3)]
    assert not gs[0].is_contiguous()
    ms, vs = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
    ref = [(p.clone(), torch.zeros_like(p), torch.zeros_like(p)) for p in ps]
    adamw_multi_tensor([(p, g, m, v, None, 1.0) for p, g, m, v in zip(ps, gs, ms, vs)], lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                       weight_decay=0.1)
    for (rp, rm, rv), g, p in zip(ref, gs, ps):
        _adamw_reference(rp, g.contiguous(), rm, rv, None, 1.0, 1e-2, 0.9, 0.95, 1e-8, 0.1, None)
        assert (p - rp).abs().max().item() < 1e-5
    _lib.fetch_status()


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 8, 2), (128, 4, 4)])
def test_causal_attention_matches_fp32_reference(D, Hq, Hkv):
    from maltos_b200.ops.attention import attention_reference, causal_attention

    torch.manual_seed(3)
    B, S = 2, 384
    q, k, v = (torch.randn(B, S, h, D, device=DEV).bfloat16().requires_grad_() for h in (Hq, Hkv, Hkv))
    out = causal_attention(q, k, v)
    do = torch.randn_like(out)
    out.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qf, kf, vf, causal=True)
    ref.backward(do.float())
    _close(out, ref, 2e-2)
    _close(q.grad, qf.grad, 3e-2)
    _close(k.grad, kf.grad, 3e-2)
    _close(v.grad, vf.grad, 3e-2)


def test_packed_document_attention_matches_fp32_reference():
    from maltos_b200.ops.attention import attention_reference, causal_attention
    from maltos_b200.utils.constants import PAD_SEQUENCE_ID

    torch.manual_seed(5)
    B, S, Hq, Hkv, D = 2, 256, 8, 2, 64
    q, k, v = (torch.randn(B, S, h, D, device=DEV).bfloat16().requires_grad_() for h in (Hq, Hkv, Hkv))
    seq = torch.full((B, S), PAD_SEQUENCE_ID, dtype=torch.long, device=DEV)
    seq[0, :100], seq[0, 100:230] = 0, 1
    seq[1, :17], seq[1, 17:256] = 0, 1
    out = causal_attention(q, k, v, sequence_ids=seq)
    keep = (seq != PAD_SEQUENCE_ID).unsqueeze(-1).unsqueeze(-1)
    do = torch.randn_like(out) * keep
    out.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    order = torch.arange(S, device=DEV).unsqueeze(0).expand(B, S)
    ref = attention_reference(qf, kf, vf, q_positions=order, k_positions=order, q_sequence_ids=seq, k_sequence_ids=seq) * keep
    ref.backward(do.float())
    _close(out * keep, ref, 2e-2)
    _close(q.grad, qf.grad, 3e-2)
    _close(k.grad, kf.grad, 3e-2)
    _close(v.grad, vf.grad, 3e-2)


@pytest.mark.parametrize("E,k,renorm,dtype", [(64, 1, True, torch.float32), (64, 2, True, torch.bfloat16), (8, 2, False, torch.float32),
                                              (200, 4, True, torch.float32)])
def test_moe_router_matches_reference(E, k, renorm, dtype):
    from maltos_b200.ops.moe_router import load_balance_loss_from_stats, route, route_reference

    torch.manual_seed(9)
    N = 1000
    if dtype == torch.bfloat16:
        # bf16 logits tie easily and tie order is unspecified: use distinct, exactly representable values per row
        logits = (torch.argsort(torch.rand(N, E, device=DEV), dim=1).float() * 0.125 - 2.0).to(dtype).requires_grad_()
    else:
        logits = (torch.randn(N, E, device=DEV) * 2).to(dtype).requires_grad_()
    idx, gate, mean_prob, counts = route(logits, k, renorm)
    ref_logits = logits.detach().float().requires_grad_()
    ridx, rgate, rmean, rcounts = route_reference(ref_logits, k, renorm)
    assert torch.equal(idx, ridx) and torch.equal(counts, rcounts)
    _close(gate, rgate, 1e-2 if dtype == torch.bfloat16 else 1e-5)
    _close(mean_prob, rmean, 1e-4)
    dg = torch.randn(N, k, device=DEV)
    (gate.float() * dg).sum().add(3.0 * load_balance_loss_from_stats(mean_prob, counts)).backward()
    (rgate.float() * dg).sum().add(3.0 * load_balance_loss_from_stats(rmean, rcounts)).backward()
    _close(logits.grad, ref_logits.grad, 2e-2 if dtype == torch.bfloat16 else 1e-4)
    _lib.fetch_status()
