"""Ring attention on gloo ranks against single-device attention over the whole sequence: contiguous, zigzag (the
half-block schedule) and packed-document layouts, forward and gradients; and the per-micro-batch plan: one host read for
all layers that share the position tensor."""
import pytest
import torch

from tests.dist_utils import run_distributed


def _layout(kind, S_total, rank, world):
    from maltos_b200.runtime.layers.ring_layout import zigzag_positions

    local = S_total // world
    if kind == "zigzag":
        return zigzag_positions(S_total, rank, world)
    return torch.arange(rank * local, (rank + 1) * local)


def _ring_case(rank, world, kind, use_core):
    import torch.distributed as dist

    from maltos_b200.ops.attention import attention_reference
    from maltos_b200.runtime.layers import ring_attention as ra

    B, S_total, hq, hkv, D = 2, 32 * world, 4, 2, 16
    g = torch.Generator().manual_seed(11)
    q_all = torch.randn(B, S_total, hq, D, generator=g)
    k_all = torch.randn(B, S_total, hkv, D, generator=g)
    v_all = torch.randn(B, S_total, hkv, D, generator=g)
    w_all = torch.randn(B, S_total, hq, D, generator=g)
    packed = kind == "packed"
    idx = _layout("zigzag" if kind == "zigzag" else "contiguous", S_total, rank, world)
    pos_all = torch.arange(S_total).unsqueeze(0).expand(B, -1).contiguous()
    seq_all = None
    if packed:                       # three documents per row with boundaries that fall inside ranks; positions restart
        bounds = [0, S_total // 3 + 1, 2 * S_total // 3 + 5, S_total]
        seq_all = torch.zeros(B, S_total, dtype=torch.long)
        pos_all = torch.zeros(B, S_total, dtype=torch.long)
        for d in range(3):
            seq_all[:, bounds[d]:bounds[d + 1]] = d
            pos_all[:, bounds[d]:bounds[d + 1]] = torch.arange(bounds[d + 1] - bounds[d])
    # oracle on the whole sequence: causality by global index is what position + sequence id express
    qa, ka, va = (t.clone().requires_grad_() for t in (q_all, k_all, v_all))
    if packed:
        ref = attention_reference(qa, ka, va, q_positions=pos_all, k_positions=pos_all, q_sequence_ids=seq_all, k_sequence_ids=seq_all)
    else:
        ref = attention_reference(qa, ka, va, q_positions=pos_all, k_positions=pos_all)
    (ref * w_all).sum().backward()

    q, k, v = (t[:, idx].clone().requires_grad_() for t in (q_all, k_all, v_all))
    pos = pos_all[:, idx].contiguous()
    seq = seq_all[:, idx].contiguous() if packed else None
    group = dist.new_group(list(range(world)))
    builds_before = ra.plan_builds
    if use_core:
        core = ra.RingAttentionCore(group)
        out = core(q, k, v, position_ids=pos, sequence_ids=seq)
        again = core(q.detach(), k.detach(), v.detach(), position_ids=pos, sequence_ids=seq)    # a second "layer"
        assert torch.equal(again, out.detach())
        assert ra.plan_builds - builds_before == 1, "the plan of a micro-batch must be computed once for all layers"
        pos2 = pos.clone()                                                                       # a new micro-batch
        core(q.detach(), k.detach(), v.detach(), position_ids=pos2, sequence_ids=seq)
        assert ra.plan_builds - builds_before == 2
        pos2.add_(0)                                                                             # in-place change: re-plan
        core(q.detach(), k.detach(), v.detach(), position_ids=pos2, sequence_ids=seq)
        assert ra.plan_builds - builds_before == 3
    else:
        out = ra.flash_ring_attention(q, k, v, group, q_positions=pos, q_sequence_ids=seq)
    (out * w_all[:, idx]).sum().backward()
    plan = ra.build_ring_plan(pos, seq, group)
    err = {
        "out": (out.detach() - ref.detach()[:, idx]).abs().max().item(),
        "dq": (q.grad - qa.grad[:, idx]).abs().max().item(),
        "dk": (k.grad - ka.grad[:, idx]).abs().max().item(),
        "dv": (v.grad - va.grad[:, idx]).abs().max().item(),
    }
    return err, plan.zigzag, plan.visible


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("kind", ["contiguous", "zigzag", "packed"])
def test_ring_attention_matches_whole_sequence_attention(world, kind):
    results = run_distributed(_ring_case, world, kind, kind != "packed")
    for rank, (err, zigzag, visible) in enumerate(results):
        for name, e in err.items():
            assert e < 2e-4, (rank, kind, name, e)
        assert zigzag == (kind == "zigzag")
        if kind == "contiguous":      # blocks of later ranks are never launched
            assert visible == tuple(o <= rank for o in range(world))
        if kind == "zigzag":
            assert all(visible)


def test_block_primitives_without_positions_see_every_key():
    from maltos_b200.ops.attention import attention_block_backward, attention_block_forward, attention_reference

    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 8, 4, 16, generator=g, requires_grad=True)
    k = torch.randn(1, 12, 2, 16, generator=g, requires_grad=True)
    v = torch.randn(1, 12, 2, 16, generator=g, requires_grad=True)
    w = torch.randn(1, 8, 4, 16, generator=g)
    ref, ref_lse = attention_reference(q, k, v, causal=False, return_lse=True)
    (ref * w).sum().backward()
    out, lse = attention_block_forward(q.detach(), k.detach(), v.detach(), q_positions=None, k_positions=None)
    assert torch.allclose(out, ref.detach(), atol=1e-5) and torch.allclose(lse, ref_lse.detach(), atol=1e-5)
    dq, dk, dv = attention_block_backward(q.detach(), k.detach(), v.detach(), out, lse, w, q_positions=None, k_positions=None)
    for a, b in ((dq, q.grad), (dk, k.grad), (dv, v.grad)):
        assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.parametrize("world", [2, 4])
def test_zigzag_schedule_call_sequence_for_every_rank_in_one_process(world, monkeypatch):
    """The schedule of every rank, without process groups: which (query rows, key rows, masked?) block calls a rank makes
    for the blocks of all owners (the reference checks its flash ring the same way with fake groups,
    ``tests/sequence_ids_attention_mask.py:189-365``), and that merging those calls reproduces whole-sequence attention."""
    from maltos_b200.ops import attention as A
    from maltos_b200.runtime.layers import ring_attention as ra
    from maltos_b200.runtime.layers.ring_layout import zigzag_positions

    B, S, hq, hkv, D = 1, 16, 2, 1, 8
    g = torch.Generator().manual_seed(9)
    q_all, k_all, v_all = (torch.randn(B, S * world, h, D, generator=g) for h in (hq, hkv, hkv))
    pos_all = torch.arange(S * world).unsqueeze(0)
    ref = A.attention_reference(q_all, k_all, v_all, q_positions=pos_all, k_positions=pos_all)
    idx = [zigzag_positions(S * world, r, world) for r in range(world)]
    calls = []
    real = ra.attention_block_forward

    def recording(q, k, v, *, q_positions, k_positions, **kw):
        calls.append((q.shape[1], k.shape[1], q_positions is not None))
        return real(q, k, v, q_positions=q_positions, k_positions=k_positions, **kw)

    monkeypatch.setattr(ra, "attention_block_forward", recording)
    plan = ra.RingPlan(True, (True,) * world)
    for me in range(world):
        calls.clear()
        q = q_all[:, idx[me]]
        out = torch.zeros(B, S, hq, D)
        lse = torch.full((B, hq, S), float("-inf"))
        for step in range(world):
            owner = (me - step) % world
            blk = [k_all[:, idx[owner]], v_all[:, idx[owner]], pos_all[:, idx[owner]], torch.zeros_like(pos_all[:, idx[owner]])]
            out, lse = ra._block_forward(plan, me, owner, q, blk, pos_all[:, idx[me]], None, None, out, lse)
        want = []
        for step in range(world):
            owner = (me - step) % world
            want.append((S, S, True) if owner == me else ((S, S // 2, False) if owner < me else (S // 2, S, False)))
        assert calls == want, (me, calls, want)
        assert (out - ref[:, idx[me]]).abs().max() < 1e-5
    # the unmasked half blocks do half the score work of a masked full block
    full, half = S * S, S * (S // 2)
    assert half * 2 == full
