"""tcgen05 flash-attention forward and backward against the fp32 restatement: mask modes, GQA, ragged lengths,
log-sum-exp, gradients through autograd of the restatement."""
import pytest
import torch

from maltos_b200.ops import _lib
from maltos_b200.ops.attention import attention_block_forward, attention_reference
from maltos_b200.ops.flash_attn import flash_attention, flash_backward, flash_forward
from maltos_b200.utils.constants import PAD_SEQUENCE_ID

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _qkv(B, Sq, Sk, Hq, Hkv, D, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    mk = lambda s, h: torch.randn(B, s, h, D, device=DEV, generator=g).bfloat16()   # noqa: E731
    return mk(Sq, Hq), mk(Sk, Hkv), mk(Sk, Hkv)


def _check(out, lse, ref, ref_lse, tol=2e-2):
    finite = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), finite)
    assert (lse[finite] - ref_lse[finite]).abs().max().item() < 2e-2
    err = (out.float() - ref.float()).abs().max().item()
    assert err <= tol * max(ref.float().abs().max().item(), 1e-3), err


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,D", [(1, 128, 128, 2, 2, 128), (2, 384, 384, 4, 2, 128), (1, 300, 300, 4, 1, 64),
                                              (1, 1024, 1024, 8, 2, 128), (2, 200, 456, 2, 2, 64)])
@pytest.mark.parametrize("causal", [True, False])
def test_dense_modes(B, Sq, Sk, Hq, Hkv, D, causal):
    q, k, v = _qkv(B, Sq, Sk, Hq, Hkv, D)
    out, lse = flash_forward(q, k, v, mode=1 if causal else 0)
    _lib.fetch_status()
    ref, ref_lse = attention_reference(q.float(), k.float(), v.float(), causal=causal, return_lse=True)
    _check(out, lse, ref, ref_lse)


def test_general_mask_zigzag_blocks_and_documents():
    B, S, Hq, Hkv, D = 2, 256, 4, 2, 128
    q, k, v = _qkv(B, S, S, Hq, Hkv, D, seed=3)
    # query block = zigzag chunks (1, 6) of an 8-chunk sequence, key block = chunks (2, 5): partly visible
    chunk = S // 2
    q_pos = torch.cat([torch.arange(1 * chunk, 2 * chunk), torch.arange(6 * chunk, 7 * chunk)]).to(DEV).unsqueeze(0).expand(B, S).contiguous()
    k_pos = torch.cat([torch.arange(2 * chunk, 3 * chunk), torch.arange(5 * chunk, 6 * chunk)]).to(DEV).unsqueeze(0).expand(B, S).contiguous()
    out, lse = flash_forward(q, k, v, mode=2, q_positions=q_pos, k_positions=k_pos)
    ref, ref_lse = attention_reference(q.float(), k.float(), v.float(), q_positions=q_pos, k_positions=k_pos, return_lse=True)
    _check(out, lse, ref, ref_lse)
    assert not torch.isfinite(lse[:, :, :chunk]).any() and float(out[:, :chunk].abs().max()) == 0.0   # first half sees nothing
    # packed documents with padding
    seq = torch.full((B, S), PAD_SEQUENCE_ID, dtype=torch.long, device=DEV)
    seq[0, :100], seq[0, 100:250] = 0, 1
    seq[1, :30], seq[1, 30:256] = 0, 1
    order = torch.arange(S, device=DEV).unsqueeze(0).expand(B, S).contiguous()
    out, lse = flash_forward(q, k, v, mode=2, q_positions=order, k_positions=order, q_sequence_ids=seq, k_sequence_ids=seq)
    ref, ref_lse = attention_reference(q.float(), k.float(), v.float(), q_positions=order, k_positions=order, q_sequence_ids=seq,
                                       k_sequence_ids=seq, return_lse=True)
    _check(out, lse, ref, ref_lse)
    _lib.fetch_status()


def test_block_primitive_uses_the_kernel_and_strided_inputs(monkeypatch):
    B, S, Hq, Hkv, D = 1, 512, 8, 2, 128
    packed = torch.randn(B, S, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    q = packed[..., :Hq * D].view(B, S, Hq, D)
    k = packed[..., Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
    v = packed[..., (Hq + Hkv) * D:].view(B, S, Hkv, D)
    pos = torch.arange(S, device=DEV).unsqueeze(0)
    monkeypatch.setenv("MALTOS_B200_FLASH_BLOCKS", "1")
    before = _lib.launch_count()
    out, lse = attention_block_forward(q, k, v, q_positions=pos, k_positions=pos)
    assert _lib.launch_count() == before + 1 and out.dtype == torch.bfloat16
    ref, ref_lse = attention_reference(q.float(), k.float(), v.float(), causal=True, return_lse=True)
    _check(out, lse, ref, ref_lse)
    _lib.fetch_status()


# ------------------------------------------------------------------------------------------------ backward
def _reference_grads(q, k, v, dout, causal=True, **mask):
    """fp32 gradients from the closed-form block backward of the restatement (rows without a visible key give zeros)."""
    from maltos_b200.ops.attention import attention_block_backward

    qf, kf, vf = q.float(), k.float(), v.float()
    B, Sq, Sk = q.shape[0], q.shape[1], k.shape[1]
    if "q_positions" not in mask:
        if causal:
            mask["q_positions"] = torch.arange(Sk - Sq, Sk, device=q.device).unsqueeze(0).expand(B, Sq)
            mask["k_positions"] = torch.arange(Sk, device=q.device).unsqueeze(0).expand(B, Sk)
        else:
            mask["q_positions"] = torch.zeros(B, Sq, dtype=torch.long, device=q.device)
            mask["k_positions"] = torch.zeros(B, Sk, dtype=torch.long, device=q.device)
    out, lse = attention_reference(qf, kf, vf, return_lse=True, **mask)
    return attention_block_backward(qf, kf, vf, out, lse, dout.float(), **mask)


def _close(got, ref, tol=2.5e-2):
    err = (got.float() - ref).abs().max().item()
    assert torch.isfinite(got.float()).all()
    assert err <= tol * max(ref.abs().max().item(), 1e-3), (err, ref.abs().max().item())


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,D", [(1, 128, 128, 2, 2, 128), (2, 384, 384, 4, 2, 128), (1, 300, 300, 4, 1, 64),
                                              (1, 1024, 1024, 8, 2, 128), (2, 200, 456, 2, 2, 64)])
@pytest.mark.parametrize("causal", [True, False])
def test_backward_dense_modes(B, Sq, Sk, Hq, Hkv, D, causal):
    q, k, v = _qkv(B, Sq, Sk, Hq, Hkv, D, seed=1)
    dout = torch.randn(B, Sq, Hq, D, device=DEV).bfloat16()
    out, lse = flash_forward(q, k, v, mode=1 if causal else 0)
    dq, dk, dv = flash_backward(q, k, v, out, lse, dout, mode=1 if causal else 0)
    _lib.fetch_status()
    rq, rk, rv = _reference_grads(q, k, v, dout, causal=causal)
    _close(dq, rq), _close(dk, rk), _close(dv, rv)


def test_backward_general_mask_packed_documents_and_accumulate():
    B, S, Hq, Hkv, D = 2, 320, 4, 2, 128
    q, k, v = _qkv(B, S, S, Hq, Hkv, D, seed=5)
    dout = torch.randn(B, S, Hq, D, device=DEV).bfloat16()
    seq = torch.full((B, S), PAD_SEQUENCE_ID, dtype=torch.long, device=DEV)
    seq[0, :100], seq[0, 100:250] = 0, 1
    seq[1, :30], seq[1, 30:320] = 0, 1
    order = torch.arange(S, device=DEV).unsqueeze(0).expand(B, S).contiguous()
    mask = dict(q_positions=order, k_positions=order, q_sequence_ids=seq, k_sequence_ids=seq)
    rq, rk, rv = _reference_grads(q, k, v, dout, **mask)
    for mode in (2, 3):
        out, lse = flash_forward(q, k, v, mode=mode, **mask)
        ref, ref_lse = attention_reference(q.float(), k.float(), v.float(), return_lse=True, **mask)
        _check(out, lse, ref, ref_lse)
        dq, dk, dv = flash_backward(q, k, v, out, lse, dout, mode=mode, **mask)
        _close(dq, rq), _close(dk, rk), _close(dv, rv)
        assert float(dq[0, 250:].abs().max()) == 0.0          # padding rows get exact zeros
    # fp32 outputs, accumulated on top of existing values (ring attention adds block gradients this way)
    acc = tuple(torch.ones_like(t, dtype=torch.float32) for t in (q, k, v))
    flash_backward(q, k, v, out, lse, dout, mode=2, accumulate_into=acc, **mask)
    _close(acc[0] - 1.0, rq), _close(acc[1] - 1.0, rk), _close(acc[2] - 1.0, rv)
    _lib.fetch_status()


def test_autograd_entry_point_strided_qkv_and_zigzag_positions():
    B, S, Hq, Hkv, D = 1, 512, 8, 2, 128
    packed = torch.randn(B, S, (Hq + 2 * Hkv) * D, device=DEV).bfloat16().requires_grad_(True)
    q = packed[..., :Hq * D].view(B, S, Hq, D)
    k = packed[..., Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
    v = packed[..., (Hq + Hkv) * D:].view(B, S, Hkv, D)
    dout = torch.randn(B, S, Hq, D, device=DEV).bfloat16()
    before = _lib.launch_count()
    out = flash_attention(q, k, v, causal=True)
    out.backward(dout)
    # forward, preprocessing, dK/dV (+ the pass that folds the per-head-group partial sums of a small grid), dQ
    assert _lib.launch_count() - before in (4, 5)
    rq, rk, rv = _reference_grads(q.detach(), k.detach(), v.detach(), dout, causal=True)
    g = packed.grad
    _close(g[..., :Hq * D].view(B, S, Hq, D), rq)
    _close(g[..., Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D), rk)
    _close(g[..., (Hq + Hkv) * D:].view(B, S, Hkv, D), rv)
    # zigzag block pair (query chunks 1 and 6, key chunks 2 and 5 of an 8-chunk sequence): partly visible
    chunk = S // 2
    q_pos = torch.cat([torch.arange(1 * chunk, 2 * chunk), torch.arange(6 * chunk, 7 * chunk)]).to(DEV).unsqueeze(0)
    k_pos = torch.cat([torch.arange(2 * chunk, 3 * chunk), torch.arange(5 * chunk, 6 * chunk)]).to(DEV).unsqueeze(0)
    q2, k2, v2 = (t.detach().contiguous() for t in (q, k, v))
    out, lse = flash_forward(q2, k2, v2, mode=2, q_positions=q_pos, k_positions=k_pos)
    dq, dk, dv = flash_backward(q2, k2, v2, out, lse, dout, mode=2, q_positions=q_pos, k_positions=k_pos, fp32_out=True)
    rq, rk, rv = _reference_grads(q2, k2, v2, dout, q_positions=q_pos, k_positions=k_pos)
    _close(dq, rq), _close(dk, rk), _close(dv, rv)
    assert float(dq[:, :chunk].abs().max()) == 0.0            # rows that see no key
    _lib.fetch_status()


def test_checkpointed_layer_replays_attention_instead_of_recomputing_it():
    """Under activation checkpointing the original forward keeps attention's output and log-sum-exp; the recompute pass
    then launches no attention forward, and the gradients equal those of the plain (non-checkpointed) run."""
    from torch.utils.checkpoint import checkpoint

    from maltos_b200.utils.activation_checkpoint import activation_checkpoint_context_fn

    B, S, Hq, Hkv, D = 1, 256, 4, 2, 128
    q0, k0, v0 = _qkv(B, S, S, Hq, Hkv, D, seed=9)
    w = torch.randn(D, D, device=DEV).bfloat16()

    def layer(q, k, v):
        return flash_attention(q @ w, k, v, causal=True).float().square().mean()

    def run(use_ckpt):
        q, k, v = (t.clone().requires_grad_(True) for t in (q0, k0, v0))
        before = _lib.launch_count()
        if use_ckpt:
            loss = checkpoint(layer, q, k, v, use_reentrant=False, preserve_rng_state=False, context_fn=activation_checkpoint_context_fn)
        else:
            loss = layer(q, k, v)
        loss.backward()
        return _lib.launch_count() - before, q.grad, k.grad, v.grad

    n_plain, *g_plain = run(False)
    n_ckpt, *g_ckpt = run(True)
    assert n_ckpt == n_plain                      # one forward + three backward launches in both runs
    for a, b in zip(g_plain, g_ckpt):
        assert torch.equal(a, b)
    _lib.fetch_status()
