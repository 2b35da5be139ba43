"""ByteScale HDP: scheduler invariants, batch materialisation, and training equivalence with a single process."""
import random

import pytest
import torch

from maltos_b200.data.bytescale_hdp import ByteScaleHdpDataLoader, build_bytescale_local_batches, schedule_document_waves
from maltos_b200.parallel.hdp_helper import (BYTESCALE_HDP_SCHEDULE_KEY, BYTESCALE_HDP_WAVES_KEY, ByteScaleHdpBalancedConfig,
                                             ByteScaleHdpCostModel, DocumentIndices)
from maltos_b200.utils.constants import IGNORE_INDEX, PAD_SEQUENCE_ID
from tests.dist_utils import run_distributed

VOCAB, SEQ = 96, 48
CLIP = 0.05     # below the gradient norm, so that clipping acts in every step


def _packed_batch(seed=0, rows=3):
    """[rows, SEQ] packed rows: documents of random length, the tail of each row is padding."""
    rng = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(1, VOCAB, (rows, SEQ), generator=g)
    seq = torch.full((rows, SEQ), PAD_SEQUENCE_ID, dtype=torch.long)
    pos = torch.zeros((rows, SEQ), dtype=torch.long)
    labels = torch.full((rows, SEQ), IGNORE_INDEX, dtype=torch.long)
    for r in range(rows):
        at, doc = 0, 0
        while at < SEQ - 4:
            n = min(rng.choice([3, 5, 9, 14, 30]), SEQ - 2 - at)
            seq[r, at:at + n] = doc
            pos[r, at:at + n] = torch.arange(n)
            labels[r, at:at + n - 1] = ids[r, at + 1:at + n]
            at += n
            doc += 1
    ids[seq == PAD_SEQUENCE_ID] = 0
    return {"input_ids": ids, "labels": labels, "position_ids": pos, "sequence_ids": seq}


def test_cost_model_and_config_validation():
    cm = ByteScaleHdpCostModel(alpha=0.5, beta=2.0, gamma=3.0)
    assert cm.sequence_cost(4) == 8 + 8 + 3 and cm.participant_cost(4, 2) == 8 + 3
    with pytest.raises(ValueError):
        ByteScaleHdpCostModel(alpha=-1)
    with pytest.raises(ValueError):
        ByteScaleHdpBalancedConfig(partition_tokens=7)
    cfg = ByteScaleHdpBalancedConfig(partition_tokens=8)
    assert cfg.participant_count(8, world_size=4) == 1 and cfg.participant_count(9, world_size=4) == 2
    with pytest.raises(ValueError):
        cfg.participant_count(33, world_size=4)
    with pytest.raises(ValueError):
        cfg.validate_tp_sp_partition(tp_size=3, use_sp=True)


@pytest.mark.parametrize("world,partition", [(2, 16), (4, 16), (4, 10)])
def test_schedule_covers_every_token_once_within_capacity(world, partition):
    batch = _packed_batch(seed=world + partition)
    docs = DocumentIndices.from_batch(batch)
    cfg = ByteScaleHdpBalancedConfig(partition_tokens=partition, cost_model=ByteScaleHdpCostModel(1.0, 4.0, 16.0))
    per_rank = [schedule_document_waves(docs, rank=r, world_size=world, config=cfg, global_valid_targets=1) for r in range(world)]
    waves = {len(l) for l in per_rank}
    assert len(waves) == 1                                    # every rank runs the same number of waves
    seen: dict[tuple[int, int], int] = {}
    for layouts in per_rank:
        for lay in layouts:
            assert lay.placement_tokens <= partition and lay.packed_rows <= 1
            spans = sorted((d.local_start, d.local_end) for d in lay.documents)
            assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))      # no overlap inside the row
            for d in lay.documents:
                degree = len(d.participant_ranks)
                assert d.padded_length % (2 * degree) == 0 and d.local_length == d.padded_length // degree
                assert degree == cfg.participant_count(d.sequence_length, world_size=world)
                for p in d.document_positions:
                    if p is not None:
                        seen[(d.document_id, p)] = seen.get((d.document_id, p), 0) + 1
    expected = {(i, p) for i, doc in enumerate(docs) for p in range(len(doc.source_indices))}
    assert set(seen) == expected and set(seen.values()) == {1}


def test_materialised_waves_carry_the_right_tokens_and_weights():
    batch = _packed_batch(seed=5)
    cfg = ByteScaleHdpBalancedConfig(partition_tokens=16)
    world = 2
    total_targets = int((batch["labels"] != IGNORE_INDEX).sum())
    weight_sum, target_sum = 0.0, 0
    for rank in range(world):
        waves, layouts = build_bytescale_local_batches(batch, rank=rank, world_size=world, config=cfg)
        for wave, lay in zip(waves, layouts):
            assert wave[BYTESCALE_HDP_SCHEDULE_KEY] is lay
            n = int((wave["labels"] != IGNORE_INDEX).sum())
            target_sum += n
            weight_sum += wave["loss_weight"]
            for d in lay.documents:
                for off, (src, p) in enumerate(zip(d.source_indices, d.document_positions)):
                    col = d.local_start + off
                    if src is None:
                        assert wave["sequence_ids"][d.local_row, col] == PAD_SEQUENCE_ID
                    else:
                        assert wave["input_ids"][d.local_row, col] == batch["input_ids"][d.source_row, src]
                        assert wave["position_ids"][d.local_row, col] == p
    assert target_sum == total_targets and abs(weight_sum - world) < 1e-9


class _FixedLoader:
    consumed_tokens = 0

    def __init__(self, batches):
        self.batches, self.i = batches, 0

    def next_batch(self, cp_rank=None):
        b = self.batches[self.i % len(self.batches)]
        self.i += 1
        return b

    def state_dict(self):
        return {"i": self.i}

    def load_state_dict(self, s):
        self.i = s["i"]


def _model():
    import maltos_b200  # noqa: F401
    from maltos_b200 import models

    torch.manual_seed(77)
    return models.TinyTransformer(64, 4, 2, 128, 1e-5, 2, VOCAB, SEQ)


def _opt(params):
    return torch.optim.AdamW(params, lr=1e-2, weight_decay=0.0)


def _hdp_worker(rank, world, partition_tokens=16):
    import maltos_b200  # noqa: F401
    from maltos_b200.runtime import MeshConfig, RuntimeCore
    from maltos_b200.runtime.layers import hdp_attention
    from maltos_b200.runtime.plugins import ddp, grad_clip
    from maltos_b200.runtime.plugins.hdp import ByteScaleHdpPlugin

    plans = []
    make_plan = hdp_attention.document_ring_plan

    def recording(**kw):
        plan = make_plan(**kw)
        plans.append((kw["ring_size"], plan.zigzag))
        return plan

    hdp_attention.document_ring_plan = recording
    cfg = ByteScaleHdpBalancedConfig(partition_tokens=partition_tokens, cost_model=ByteScaleHdpCostModel(1.0, 8.0, 32.0))
    rt = RuntimeCore(model=_model(), mesh=MeshConfig(dp=world), plugins=[ddp.DataParallelPlugin(), ByteScaleHdpPlugin(config=cfg), grad_clip.GradClipPlugin(CLIP)],
                     optimizer_factory=_opt, grad_accum_steps=1)
    rt.setup()
    loader = ByteScaleHdpDataLoader(_FixedLoader([_packed_batch(seed=11), _packed_batch(seed=12)]), hdp_rank=rank, hdp_world_size=world, config=cfg)
    losses, norms = [], []
    for _ in range(2):
        env = loader.next_batch()
        assert len(env[BYTESCALE_HDP_WAVES_KEY]) >= 1
        loss, should = rt.run_step(env)
        assert should
        rt.step_optimizer()
        losses.append(float(loss))
        norms.append(float(rt.collect_metrics()["grad_clip/grad_norm"]))
    metrics = rt.collect_metrics()
    params = {n: p.detach().clone() for n, p in rt.model.named_parameters()}
    import torch.distributed as dist

    spread = 0.0                      # every rank holds a replica: they must stay bit-identical
    for p in rt.model.parameters():
        lo, hi = p.detach().clone(), p.detach().clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        spread = max(spread, float((hi - lo).abs().max()))
    assert spread == 0.0, spread
    rt.close()
    return losses, params, {k: v for k, v in metrics.items() if "wave" in k}, plans, norms


def test_document_ring_plan_allows_the_half_block_schedule_only_with_confined_padding():
    from maltos_b200.runtime.layers.cp_functional import document_ring_plan

    ok = document_ring_plan(sequence_length=30, padded_length=32, local_length=8, ring_size=4)        # chunk 4, padding 2
    assert ok.zigzag and ok.visible == (True,) * 4
    assert document_ring_plan(sequence_length=32, padded_length=32, local_length=16, ring_size=2).zigzag
    assert not document_ring_plan(sequence_length=26, padded_length=32, local_length=8, ring_size=4).zigzag    # padding spills into chunk 6
    assert not document_ring_plan(sequence_length=30, padded_length=30, local_length=15, ring_size=2).zigzag   # not a multiple of 2R
    assert not document_ring_plan(sequence_length=8, padded_length=8, local_length=8, ring_size=1).zigzag


@pytest.mark.parametrize("world,partition_tokens", [(2, 16), (4, 8)])
def test_hdp_training_matches_single_process(world, partition_tokens):
    model = _model()
    opt = _opt(model.parameters())
    ref_losses, ref_norms = [], []
    for seed in (11, 12):
        opt.zero_grad(set_to_none=True)
        out = model(_packed_batch(seed=seed))
        loss = out.loss if hasattr(out, "loss") else out
        loss.backward()
        ref_norms.append(float(torch.nn.utils.clip_grad_norm_(model.parameters(), CLIP)))
        opt.step()
        ref_losses.append(float(loss.detach()))
    ref_params = {n: p.detach().clone() for n, p in model.named_parameters()}
    results = run_distributed(_hdp_worker, world, partition_tokens)
    rings = [p for r in results for p in r[3]]
    assert any(z for _, z in rings), "no document ring used the half-block schedule"
    if world == 4:
        assert {n for n, _ in rings} >= {2, 4}, rings                       # rings of different sizes in one batch
    for step in range(2):   # each rank reports world x its share of the global mean
        total = sum(r[0][step] for r in results) / world
        assert abs(total - ref_losses[step]) < 2e-4, (total, ref_losses[step])
    for r in results:            # the clipped norm is the norm of the global gradient (AdamW hides a wrong scale from the loss)
        assert all(abs(a - b) < 1e-5 for a, b in zip(r[4], ref_norms)), (r[4], ref_norms)
    for _, params, wave_metrics, *_ in results:
        assert wave_metrics.get("hdp/real_wave_count", wave_metrics.get("real_wave_count", 1)) >= 1
        for name, ref in ref_params.items():
            assert torch.allclose(params[name], ref, atol=2e-4, rtol=1e-3), name


def _idle_rank_worker(rank, world, zero_stage):
    """One short row for four ranks: in every wave some ranks get no tokens, and must still make the same collective calls
    (ZeRO-3 gathers parameters inside module hooks; the kind of the reference's ``tests/hdp_idle_zero3.py``)."""
    import maltos_b200  # noqa: F401
    from maltos_b200.train import cli, flags as F

    argv = ["--model", "tiny", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "128", "--n-layers", "2", "--vocab-size", str(VOCAB),
            "--seq-len", str(SEQ), "--micro-batch-size", "1", "--lr", "1e-2", "--seed", "3", "--precision", "fp32", "--grad-clip", str(CLIP),
            "--dp-size", str(world), "--hdp-balanced", "--hdp-partition-tokens", "24", "--zero-stage", str(zero_stage)]
    a = F.parse_args_from(argv, require_data=False)
    cli.validate_args(a, world)
    torch.manual_seed(a.seed)
    core = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
    core.setup()
    core.model.train()
    cfg = cli._build_hdp_config(a)
    loader = ByteScaleHdpDataLoader(_FixedLoader([_packed_batch(seed=21, rows=1), _packed_batch(seed=22, rows=1)]), hdp_rank=rank, hdp_world_size=world,
                                    config=cfg)
    losses, idle = [], []
    for _ in range(2):
        env = loader.next_batch()
        idle.append(sum(float(w["loss_weight"]) == 0.0 for w in env[BYTESCALE_HDP_WAVES_KEY]))
        loss, _ = core.run_step(env)
        core.step_optimizer()
        losses.append(float(loss.detach()))
    core.close()
    return losses, idle


@pytest.mark.parametrize("zero_stage", [1, 3])
def test_idle_hdp_ranks_still_join_every_collective(zero_stage):
    from maltos_b200.train import cli, flags as F

    a = F.parse_args_from(["--model", "tiny", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "128", "--n-layers", "2",
                           "--vocab-size", str(VOCAB), "--seq-len", str(SEQ), "--seed", "3", "--precision", "fp32"], require_data=False)
    torch.manual_seed(a.seed)
    model = cli._build_model(a)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2, weight_decay=a.weight_decay, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_eps)
    ref = []
    for seed in (21, 22):
        opt.zero_grad(set_to_none=True)
        out = model(_packed_batch(seed=seed, rows=1))
        loss = out.loss if hasattr(out, "loss") else out
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), CLIP)
        opt.step()
        ref.append(float(loss.detach()))
    results = run_distributed(_idle_rank_worker, 4, zero_stage)
    assert all(min(idle) >= 1 for _, idle in results), "the case is meant to leave every rank without tokens in some wave"
    for step in range(2):
        total = sum(r[0][step] for r in results) / 4
        assert abs(total - ref[step]) < 2e-4, (step, total, ref[step])


def test_command_line_builds_the_cost_model_and_counts_the_global_batch():
    """The HDP flags reach the config, and a step's token count has no data-parallel factor under HDP: every rank cuts
    its piece out of ONE canonical batch (reference ``tests/hdp_cli_cost_model.py``)."""
    from maltos_b200.train import cli, flags as F

    base = ["--model", "tiny", "--seq-len", "64", "--micro-batch-size", "3", "--grad-accum-steps", "2", "--dp-size", "4"]
    a = F.parse_args_from(base + ["--hdp-balanced", "--hdp-partition-tokens", "16", "--hdp-cost-alpha", "1.25", "--hdp-cost-beta", "3.5",
                                  "--hdp-cost-gamma", "7.0", "--hdp-balance-delta", "9"], require_data=False)
    cfg = cli._build_hdp_config(a)
    assert cfg.partition_tokens == 16 and cfg.balance_delta == 9
    assert (cfg.cost_model.alpha, cfg.cost_model.beta, cfg.cost_model.gamma) == (1.25, 3.5, 7.0)
    assert cli._global_batch_tokens(a) == 3 * 64 * 2
    assert cli._global_batch_tokens(F.parse_args_from(base, require_data=False)) == 3 * 64 * 4 * 2
