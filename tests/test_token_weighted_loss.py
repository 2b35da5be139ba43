"""``--token-weighted-loss``: with rows that carry different numbers of supervised targets (fine-tuning data), every
parallel layout reproduces the loss and the global gradient norm of a single process on the union of the rows; without
the option data-parallel training averages the ranks' means (the reference's behaviour) and differs."""
import pytest
import torch

from tests.dist_utils import run_distributed

VOCAB, SEQ, ROWS, STEPS = 64, 32, 8, 2
MODEL = ["--model", "llama", "--dim", "32", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "64", "--n-layers", "2", "--vocab-size", str(VOCAB),
         "--seq-len", str(SEQ), "--lr", "1e-2", "--seed", "3", "--precision", "fp32", "--grad-clip", "0.05"]


def _batches():
    g = torch.Generator().manual_seed(17)
    out = []
    for _ in range(STEPS):
        ids = torch.randint(0, VOCAB, (ROWS, SEQ), generator=g)
        labels = ids.roll(-1, 1)
        for r in range(ROWS):                      # row r supervises only its last 2 + 3 r tokens: 2 ... 23 targets
            labels[r, :SEQ - (2 + 3 * r)] = -100
        out.append({"input_ids": ids, "labels": labels})
    return out


def _worker(rank, world, flags):
    from maltos_b200.runtime.mesh import MeshAxis
    from maltos_b200.train import cli, flags as F

    a = F.parse_args_from(MODEL + flags, require_data=False)
    cli.validate_args(a, world)
    torch.manual_seed(a.seed)
    core = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
    core.setup()
    core.model.train()
    import torch.distributed as dist

    group = core.get_group(MeshAxis.DP)
    dp_rank = dist.get_rank(group) if group is not None else 0
    per = ROWS // a.dp_size
    losses, norms = [], []
    for batch in _batches():
        core.run_step({k: v[dp_rank * per:(dp_rank + 1) * per].clone() for k, v in batch.items()})
        core.step_optimizer()
        metrics = core.collect_metrics()
        losses.append(float(metrics["loss"]))
        norms.append(next(float(v) for k, v in metrics.items() if k.endswith("/grad_norm")))
    core.close()
    return losses, norms


def _mean(results, step):
    return sum(r[0][step] for r in results) / len(results)


@pytest.fixture(scope="module")
def single():
    return run_distributed(_worker, 1, ["--micro-batch-size", str(ROWS)])[0]


@pytest.mark.parametrize("name,world,flags", [
    ("dp4", 4, ["--dp-size", "4"]),
    ("dp2_cp2_ring_zero1", 4, ["--dp-size", "2", "--cp-size", "2", "--cp-attn-core", "ring", "--zero-stage", "1"]),
    ("dp2_pp2_1f1b", 4, ["--dp-size", "2", "--pp-size", "2", "--pp-microbatches", "2", "--pp-schedule", "1f1b"]),
    ("dp2_tp2_sp_zero3", 4, ["--dp-size", "2", "--tp-size", "2", "--use-sp", "--zero-stage", "3"]),
])
def test_layouts_reproduce_the_single_process_loss_and_norm(name, world, flags, single):
    results = run_distributed(_worker, world, flags + ["--micro-batch-size", str(ROWS // int(flags[flags.index("--dp-size") + 1])),
                                                     "--token-weighted-loss"])
    for step in range(STEPS):
        assert abs(_mean(results, step) - single[0][step]) < 2e-5, (name, step, _mean(results, step), single[0][step])
        for r in results:
            assert abs(r[1][step] - single[1][step]) < 2e-5 * max(1.0, single[1][step]), (name, step, r[1][step], single[1][step])


def test_without_the_option_data_parallel_ranks_average_their_means(single):
    results = run_distributed(_worker, 4, ["--dp-size", "4", "--micro-batch-size", "2"])
    assert abs(_mean(results, 0) - single[0][0]) > 1e-3          # rows with few targets weigh more than in a single process


def test_the_option_is_rejected_with_hdp():
    from maltos_b200.train import cli, flags as F

    a = F.parse_args_from(MODEL + ["--dp-size", "2", "--hdp-balanced", "--hdp-partition-tokens", "16", "--token-weighted-loss"], require_data=False)
    with pytest.raises(ValueError, match="implied by --hdp-balanced"):
        cli.validate_args(a, 2)
