"""fp16 loss scaling when gradients are spread over ranks (ZeRO shards, tensor-parallel shards): an overflow seen by ONE
rank must skip the step and back the scale off on EVERY rank; clipping must act on unscaled norms. Two gloo ranks on CPU
(the plugin is switched on for CPU explicitly; on CUDA it is active whenever the dtype is fp16)."""
import pytest
import torch

from tests.dist_utils import run_distributed


def _train(rank, world, mode):
    import torch.distributed as dist

    import maltos_b200  # noqa: F401
    from maltos_b200.runtime.plugins.fp16 import Fp16Plugin
    from maltos_b200.train import cli, flags as F
    from maltos_b200.utils.amp import DistributedGradScaler

    extra = {"zero1": ["--dp-size", "2", "--zero-stage", "1"], "zero3": ["--dp-size", "2", "--zero-stage", "3"],
             "tp": ["--tp-size", "2"]}[mode]
    argv = ["--model", "llama", "--dim", "32", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "64", "--n-layers", "2", "--vocab-size", "64",
            "--seq-len", "16", "--micro-batch-size", "2", "--lr", "1e-2", "--seed", "3", "--precision", "fp16", "--grad-clip", "1.0",
            "--disable-metrics", *extra]
    a = F.parse_args_from(argv, require_data=False)
    cli.validate_args(a, world)
    torch.manual_seed(a.seed)
    core = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
    plugin = next(p for p in core.plugins if isinstance(p, Fp16Plugin))
    plugin.allow_cpu, plugin.init_scale = True, 2.0 ** 24            # far too large: the first steps overflow
    core.setup()
    assert isinstance(core.state.scaler, DistributedGradScaler)
    core.model.train()
    g = torch.Generator().manual_seed(7 + (rank if mode != "tp" else 0))   # data-parallel ranks see different rows
    history = []
    for step in range(14):
        ids = torch.randint(0, 64, (2, 16), generator=g)
        core.run_step({"input_ids": ids, "labels": ids.roll(-1, 1)})
        core.step_optimizer()
        scale = float(core.state.scaler.get_scale())
        both = torch.tensor([scale, -scale])
        dist.all_reduce(both, op=dist.ReduceOp.MAX)                      # max(scale), -min(scale)
        assert float(both[0]) == -float(both[1]) == scale, (step, scale, both)
        history.append((scale, bool(core.state.metadata["overflow"]), core.state.metadata.get("grad_norm")))
    spread = 0.0
    if mode in ("zero1", "tp"):                                          # replicas (whole model / unsharded weights) stay identical
        group = core.get_group(__import__("maltos_b200.runtime.mesh", fromlist=["MeshAxis"]).MeshAxis.DP if mode == "zero1" else
                               __import__("maltos_b200.runtime.mesh", fromlist=["MeshAxis"]).MeshAxis.TP)
        for name, e in core.state_manager.params.items():
            if mode == "tp" and e.meta.logical_shapes != [list(e.param.shape)]:
                continue                                                 # sharded over the tensor-parallel group
            lo, hi = e.param.detach().float().clone(), e.param.detach().float().clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
            spread = max(spread, float((hi - lo).abs().max()))
    finite = all(bool(torch.isfinite(p).all()) for p in core.model.parameters() if p.untyped_storage().size())
    core.close()
    return history, spread, finite


def _check(results):
    for history, spread, finite in results:
        scales = [s for s, _, _ in history]
        skipped = [o for _, o, _ in history]
        assert skipped[0] and any(not o for o in skipped), history          # overflowed first, trained later
        assert scales[0] == 2.0 ** 23 and min(scales) < 2.0 ** 22           # backed off step by step
        assert spread == 0.0 and finite
    assert [h[:2] for h in results[0][0]] == [h[:2] for h in results[1][0]]  # the same decisions on both ranks


def test_overflow_is_a_global_decision_under_zero1():
    results = run_distributed(_train, 2, "zero1")
    _check(results)
    # once steps are applied the clipped norm is the norm of the UNSCALED gradients (a few units, not millions)
    applied = [n for _, o, n in results[0][0] if not o and n is not None]
    assert applied and all(n < 100.0 for n in applied), applied


def test_overflow_is_a_global_decision_under_zero3():
    _check(run_distributed(_train, 2, "zero3"))


def test_overflow_on_one_tensor_parallel_shard_skips_the_step_everywhere():
    _check(run_distributed(_train, 2, "tp"))


def test_fp16_logs_the_unscaled_loss_and_refuses_to_run_without_a_scaler():
    """The loss metric is the model's loss, not loss x scale (the step runner used to overwrite the value the plugin had
    kept before scaling - as the reference does), and float16 on CPU without ``allow_cpu`` is refused at setup instead of
    training without loss scaling (reference ``tests/smoke_runtime_core.py:716-733``)."""
    import torch.nn as nn

    from maltos_b200.runtime import RuntimeCore
    from maltos_b200.runtime.plugins.fp16 import Fp16Plugin

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(4, 4)

        def forward(self, x):
            return self.lin(x.to(self.lin.weight.dtype)).float().pow(2).mean()

    torch.manual_seed(0)
    core = RuntimeCore(model=Model(), dtype=torch.float16, grad_accum_steps=2, optimizer_factory=lambda p: torch.optim.SGD(p, lr=0.01),
                       plugins=[Fp16Plugin(allow_cpu=True)])
    core.setup()
    x = torch.randn(8, 4)
    expected = float(core.model(x))
    core.run_step(x)
    core.run_step(x)
    core.step_optimizer()
    metrics = core.collect_metrics()
    assert abs(float(metrics["loss"]) - expected) < 1e-3 * max(1.0, expected), (metrics["loss"], expected)
    assert float(core.state.scaler.get_scale()) >= 2.0 ** 15
    core.close()
    refused = RuntimeCore(model=Model(), dtype=torch.float16, optimizer_factory=lambda p: torch.optim.SGD(p, lr=0.01), plugins=[Fp16Plugin()])
    with pytest.raises(ValueError, match="requires CUDA model parameters"):
        refused.setup()
