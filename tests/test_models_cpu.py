"""Model-level CPU tests: activation checkpointing, rotary variants, visibility masks, MoE load-balance loss, checkpoint
retention, and a two-rank ZeRO-1 save -> resume run of the GPT-style model."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from maltos_b200.models.activation_checkpointing import ActivationCheckpointConfig
from maltos_b200.models.llama import LlamaConfig, LlamaForCausalLM
from maltos_b200.ops.attention import build_visibility_mask
from maltos_b200.ops.rope import apply_rope, build_rope_cache
from maltos_b200.train.trainer import _apply_checkpoint_retention
from maltos_b200.utils.constants import PAD_SEQUENCE_ID
from tests.dist_utils import free_port

ROOT = Path(__file__).resolve().parents[1]


def _llama(ckpt: ActivationCheckpointConfig):
    torch.manual_seed(3)
    return LlamaForCausalLM(LlamaConfig(vocab_size=101, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                                        num_key_value_heads=2, max_position_embeddings=64, attention_backend="eager",
                                        activation_checkpointing=ckpt))


@pytest.mark.parametrize("every", [1, 2])
def test_activation_checkpointing_does_not_change_loss_or_gradients(every):
    g = torch.Generator().manual_seed(0)
    batch = {"input_ids": torch.randint(0, 101, (2, 32), generator=g), "labels": torch.randint(0, 101, (2, 32), generator=g)}
    plain, ckpt = _llama(ActivationCheckpointConfig()), _llama(ActivationCheckpointConfig(enabled=True, every_n_layers=every))
    ckpt.load_state_dict(plain.state_dict())
    outs = []
    for m in (plain, ckpt):
        m.train()
        out = m(batch)
        loss = out.loss if hasattr(out, "loss") else out
        loss.backward()
        outs.append(float(loss.detach()))
    assert outs[0] == pytest.approx(outs[1], abs=1e-6)
    for (n, a), (_, b) in zip(plain.named_parameters(), ckpt.named_parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-6), n
    with pytest.raises(ValueError):
        ActivationCheckpointConfig(every_n_layers=0)
    assert [ActivationCheckpointConfig(True, "block", 2).should_checkpoint_layer(i) for i in range(4)] == [False, True, False, True]


def test_rotary_interleaved_and_rotate_half_conventions():
    torch.manual_seed(0)
    B, S, H, D = 2, 9, 3, 8
    x = torch.randn(B, S, H, D)
    cos, sin = build_rope_cache(32, D, 10000.0)
    pos = torch.arange(S)
    c, s = cos[pos][None, :, None, :], sin[pos][None, :, None, :]
    # LLaMA convention: pairs (2i, 2i+1)
    even, odd = x[..., 0::2], x[..., 1::2]
    want = torch.stack([even * c - odd * s, even * s + odd * c], dim=-1).flatten(-2)
    assert torch.allclose(apply_rope(x, cos, sin, interleaved=True), want, atol=1e-6)
    # OLMo / HF convention: pairs (i, i + D/2)
    lo, hi = x[..., :D // 2], x[..., D // 2:]
    want_half = torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1)
    assert torch.allclose(apply_rope(x, cos, sin, interleaved=False), want_half, atol=1e-6)
    # explicit positions (packed documents restart at 0) and an offset (pipeline / context shards)
    ids = torch.tensor([[0, 1, 2, 0, 1, 2, 3, 0, 1]]).expand(B, S)
    packed = apply_rope(x, cos, sin, position_ids=ids, interleaved=True)
    assert torch.allclose(packed[:, 3:7], apply_rope(x[:, 3:7], cos, sin, interleaved=True), atol=1e-6)
    shifted = apply_rope(x, cos, sin, position_offset=5, interleaved=True)
    assert torch.allclose(shifted, apply_rope(x, cos, sin, position_ids=torch.arange(5, 5 + S), interleaved=True), atol=1e-6)
    # a rotation preserves norms
    assert torch.allclose(shifted.norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_visibility_mask_documents_padding_and_blocks():
    pos = torch.tensor([[0, 1, 2, 0, 1, 0]])
    seq = torch.tensor([[0, 0, 0, 1, 1, PAD_SEQUENCE_ID]])
    order = torch.arange(6).unsqueeze(0)
    m = build_visibility_mask(order, order, seq, seq)[0]
    want = torch.zeros(6, 6, dtype=torch.bool)
    want[:3, :3] = torch.tril(torch.ones(3, 3, dtype=torch.bool))
    want[3:5, 3:5] = torch.tril(torch.ones(2, 2, dtype=torch.bool))
    assert torch.equal(m, want)                              # padding sees nothing and is seen by nobody
    # a block strictly in the past is fully visible, one in the future not at all
    past = build_visibility_mask(torch.arange(8, 12).unsqueeze(0), torch.arange(0, 4).unsqueeze(0))
    future = build_visibility_mask(torch.arange(0, 4).unsqueeze(0), torch.arange(8, 12).unsqueeze(0))
    assert past.all() and not future.any()
    del pos


def test_moe_load_balance_loss_value_and_router_reference():
    from maltos_b200.models.tiny_moe_transformer import load_balance_loss, route_and_balance
    from maltos_b200.ops.moe_router import load_balance_loss_from_stats, route_reference

    torch.manual_seed(1)
    logits = torch.randn(50, 4)
    uniform = torch.zeros(40, 4)
    idx = torch.arange(40) % 4
    assert float(load_balance_loss(uniform, idx)) == pytest.approx(1.0)      # perfectly balanced router -> 1
    collapsed = torch.zeros(40, 4)
    collapsed[:, 0] = 20.0
    assert float(load_balance_loss(collapsed, torch.zeros(40, dtype=torch.long))) == pytest.approx(4.0, rel=1e-3)
    i1, g1, aux = route_and_balance(logits, 2, need_aux=True)
    i2, g2, mean_prob, counts = route_reference(logits, 2, True)
    assert torch.equal(i1, i2) and torch.allclose(g1, g2) and torch.allclose(g1.sum(-1), torch.ones(50))
    assert float(aux) == pytest.approx(float(load_balance_loss_from_stats(mean_prob, counts)), rel=1e-6)


def test_checkpoint_retention_policy(tmp_path):
    for s in (2, 4, 6, 8, 10, 12):
        (tmp_path / f"step_{s:08d}").mkdir()
    (tmp_path / "notes").mkdir()
    _apply_checkpoint_retention(tmp_path, current_step=12, keep_last=2, keep_every_n_steps=6)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["notes", "step_00000006", "step_00000010", "step_00000012"]


def _train(args, nproc):
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), "-m", "maltos_b200.tools.train", *args]
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=420)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    return [l.split("loss ")[1].split(" ")[0] for l in out.stdout.splitlines() if l.startswith("[step")]


def test_two_rank_zero1_clip_accum_save_load_resume(tmp_path):
    """DP2 + ZeRO-1, fp32, gradient accumulation 2, clipping 1.0: 10 steps straight equal 6 steps + resume + 4 steps."""
    data = tmp_path / "tokens"
    data.mkdir()
    np.random.default_rng(0).integers(0, 256, size=20000, dtype=np.uint32).tofile(data / "tokens_00000.bin")
    flags = ["--data", str(data), "--model", "tiny", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "128", "--n-layers", "2",
             "--vocab-size", "256", "--seq-len", "32", "--micro-batch-size", "2", "--grad-accum-steps", "2", "--dp-size", "2", "--zero-stage", "1",
             "--grad-clip", "1.0", "--log-every", "1", "--checkpoint-every", "6", "--lr", "1e-3"]
    full = _train([*flags, "--max-steps", "10", "--checkpoint-dir", str(tmp_path / "a")], 2)
    assert len(full) == 10
    _train([*flags, "--max-steps", "6", "--checkpoint-dir", str(tmp_path / "b")], 2)
    tail = _train([*flags, "--max-steps", "10", "--checkpoint-dir", str(tmp_path / "b"), "--resume-from", str(tmp_path / "b" / "step_00000006")], 2)
    assert tail == full[6:]
