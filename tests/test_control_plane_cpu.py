"""Single-process control-plane checks of the runtime core and the trainer (the kinds of the reference's
``tests/smoke_runtime_core.py`` and ``tests/smoke_trainer_loop.py``): phase order seen by a plugin, ownership conflicts,
accumulation cadence and the unscaled loss metric, profiler span names, log / checkpoint / upload cadence, interval
aggregation, resume with the prefetching loader, checkpoint-rank policy computed from the mesh alone."""
import json

import pytest
import torch
import torch.nn as nn

import maltos_b200  # noqa: F401
from maltos_b200.models import TinyModel
from maltos_b200.runtime import RuntimeCore
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import RuntimePhase, SetupPhase


class _Recorder(RuntimePlugin):
    def __init__(self, log, plugin_id=PluginId.CHECKPOINT, **kw):
        super().__init__(id=plugin_id, **kw)
        self.log = log

    def on_setup_phase(self, phase, model):
        self.log.append(("setup", phase))
        return model

    def annotate_param_metadata(self):
        self.log.append(("annotate", None))

    def on_step_phase(self, phase):
        self.log.append(("step", phase))


def _runtime(plugins=(), accum=1, **kw):
    torch.manual_seed(0)
    return RuntimeCore(model=TinyModel(), optimizer_factory=lambda p: torch.optim.AdamW(p, lr=1e-2), plugins=list(plugins),
                       grad_accum_steps=accum, **kw)


def test_a_plugin_sees_the_phases_in_order():
    log = []
    rt = _runtime([_Recorder(log)], accum=2)
    rt.setup()
    assert [p for k, p in log if k == "setup"] == [SetupPhase.TRANSFORM, SetupPhase.MATERIALIZE, SetupPhase.FINALIZE]
    assert ("annotate", None) in log and log.index(("annotate", None)) > log.index(("setup", SetupPhase.TRANSFORM))
    log.clear()
    micro = [RuntimePhase.PRE_STEP_RUNNER, RuntimePhase.PRE_FORWARD, RuntimePhase.POST_FORWARD, RuntimePhase.PRE_BACKWARD,
             RuntimePhase.POST_BACKWARD]
    _, should = rt.run_step(torch.randn(4, 32))
    assert not should and [p for _, p in log] == micro
    _, should = rt.run_step(torch.randn(4, 32))
    assert should and [p for _, p in log] == micro * 2
    log.clear()
    rt.step_optimizer()
    assert [p for _, p in log] == [RuntimePhase.PRE_STEP, RuntimePhase.POST_STEP]
    rt.close()


def test_two_owners_of_the_same_resource_are_rejected():
    class Owner(_Recorder):
        def get_optimizer_and_scheduler(self):
            return None, None

        def optimizer_state_source_rank(self, rank_id):
            return rank_id

    with pytest.raises(ValueError, match="optimizer"):
        _runtime([Owner([], PluginId.ZERO1, owns_optimizer=True), Owner([], PluginId.ZERO2, owns_optimizer=True)])
    with pytest.raises(ValueError, match="must satisfy StepRunnerOwner|owns_step_runner"):
        class Bad(RuntimePlugin):
            build_step_runner = None      # does not satisfy the protocol

        Bad(id=PluginId.PP, owns_step_runner=True)


def test_accumulation_cadence_and_unscaled_loss_metric():
    x = [torch.randn(4, 32) for _ in range(3)]
    whole = _runtime(accum=1)
    whole.setup()
    losses = []
    for b in x:
        loss, _ = whole.run_step(b)
        losses.append(float(loss))
        whole.model.zero_grad(set_to_none=True)
    rt = _runtime(accum=3)
    rt.setup()
    flags = [rt.run_step(b)[1] for b in x]
    assert flags == [False, False, True]
    with pytest.raises(RuntimeError):
        _runtime(accum=3).step_optimizer()                      # not set up / not at a boundary
    rt.step_optimizer()
    m = rt.collect_metrics()
    assert m["step"] == 1
    assert abs(m["loss"] - sum(losses) / 3) < 1e-5              # the mean of the micro-step losses, not a 1/accum-scaled one
    rt.close()
    whole.close()


def test_profiler_trace_has_the_semantic_span_names():
    rt = _runtime()
    rt.setup()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU]) as prof:
        rt.run_step(torch.randn(4, 32))
        rt.step_optimizer()
        rt.collect_metrics()
    names = {e.name for e in prof.events()}
    for want in ("maltos::micro_step_runner", "maltos::forward", "maltos::backward", "maltos::metrics.collect"):
        assert want in names, (want, sorted(n for n in names if n.startswith("maltos::")))
    rt.close()


class _Loader:
    """Endless loader of fixed batches with the stateful protocol of the real loaders."""

    def __init__(self):
        self.i = 0
        self.closed = False

    def next_batch(self, cp_rank=None):
        g = torch.Generator().manual_seed(self.i)
        self.i += 1
        return torch.randn(4, 32, generator=g)

    def state_dict(self):
        return {"i": self.i}

    def load_state_dict(self, state):
        self.i = int(state["i"])

    def close(self):
        self.closed = True


class _ListLogger:
    def __init__(self):
        self.rows = []

    def log(self, metrics):
        self.rows.append(dict(metrics))


class _Uploader:
    def __init__(self):
        self.uploads, self.closed = [], False

    def upload_checkpoint(self, path, step):
        self.uploads.append((str(path), step))

    def close(self):
        self.closed = True


def _trainer(tmp_path, *, max_steps, resume=None, prefetch=0, log_every=2, accum=2, keep_last=None, uploader=None):
    from maltos_b200.train.trainer import Trainer, TrainerConfig

    rt = _runtime(accum=accum)
    logger = _ListLogger()
    loader = _Loader()
    cfg = TrainerConfig(max_steps=max_steps, log_every=log_every, checkpoint_every=2, checkpoint_dir=tmp_path, resume_from=resume,
                        checkpoint_keep_last=keep_last, data_prefetch_batches=prefetch)
    tr = Trainer(runtime=rt, dataloader=loader, config=cfg, logger=logger, checkpoint_uploader=uploader, runtime_spec={"version": 1})
    tr.setup()
    return tr, logger, loader


def test_trainer_cadence_interval_aggregation_retention_and_uploads(tmp_path):
    up = _Uploader()
    tr, logger, loader = _trainer(tmp_path, max_steps=6, keep_last=2, uploader=up)
    tr.fit()
    assert [r["step"] for r in logger.rows] == [2, 4, 6]                       # every log_every steps, last one flushed at the end
    assert loader.i == 12 and loader.closed                                     # 6 steps x 2 micro-batches
    assert sorted(p.name for p in tmp_path.iterdir() if p.is_dir()) == ["step_00000004", "step_00000006"]
    assert [s for _, s in up.uploads] == [2, 4, 6] and up.closed
    assert json.loads((tmp_path / "runtime_spec.json").read_text()) == {"version": 1}
    # the logged loss of an interval is the mean over its optimizer steps
    single, single_log, _ = _trainer(tmp_path / "b", max_steps=2, log_every=1)
    single.fit()
    per_step = [r["loss"] for r in single_log.rows]
    assert abs(logger.rows[0]["loss"] - sum(per_step) / 2) < 1e-5


@pytest.mark.parametrize("prefetch", [0, 1])
def test_resume_equals_continuous_also_with_the_prefetching_loader(tmp_path, prefetch):
    full, full_log, _ = _trainer(tmp_path / "full", max_steps=4, log_every=1, prefetch=prefetch)
    full.fit()
    first, _, _ = _trainer(tmp_path / "part", max_steps=2, log_every=1, prefetch=prefetch)
    first.fit()
    rest, rest_log, loader = _trainer(tmp_path / "part", max_steps=4, log_every=1, prefetch=prefetch,
                                      resume=tmp_path / "part" / "step_00000002")
    assert rest.runtime.state.step_context.step == 2
    rest.fit()
    assert [r["step"] for r in rest_log.rows] == [3, 4]
    want = [r["loss"] for r in full_log.rows][2:]
    got = [r["loss"] for r in rest_log.rows]
    assert all(abs(a - b) < 1e-6 for a, b in zip(got, want)), (got, want)


def test_trainer_config_validation():
    from maltos_b200.train.trainer import Trainer, TrainerConfig

    for bad, match in ((dict(max_steps=-1), "max_steps"), (dict(max_steps=1, log_every=0), "log_every"),
                       (dict(max_steps=1, checkpoint_every=1), "checkpoint_dir is required"),
                       (dict(max_steps=1, data_prefetch_batches=2), "0 or 1"), (dict(max_steps=1, checkpoint_keep_last=-1), "keep_last")):
        with pytest.raises(ValueError, match=match):
            Trainer(runtime=_runtime(), dataloader=_Loader(), config=TrainerConfig(**bad))


def test_checkpoint_rank_policy_follows_the_mesh_without_process_groups():
    """Which rank writes a replicated tensor is a pure function of the mesh coordinates (rank order dp, pp, cp, tp)."""
    from maltos_b200.parallel.plan import ParallelPlan
    from maltos_b200.runtime.mesh import MeshAxis, MeshConfig

    mesh, plan = MeshConfig(dp=2, tp=2, pp=2, cp=2), ParallelPlan()
    assert mesh.world_size == 16
    for rank in range(mesh.world_size):
        dp, pp, cp, tp = mesh.rank_coordinates(rank)
        assert mesh.rank_id(dp=dp, pp=pp, cp=cp, tp=tp) == rank
        # replicated over data and context parallel ranks, sharded over tp and pp: written by (dp 0, cp 0) of the same tp / pp
        assert mesh.infer_checkpoint_rank(rank, plan=plan, replicated_axes={MeshAxis.DCP}) == mesh.rank_id(dp=0, pp=pp, cp=0, tp=tp)
        # additionally replicated over tp (norm weights without sequence parallelism)
        assert mesh.infer_checkpoint_rank(rank, plan=plan, replicated_axes={MeshAxis.DCP, MeshAxis.TP}) == mesh.rank_id(dp=0, pp=pp, cp=0, tp=0)
        assert mesh.infer_checkpoint_rank(rank, plan=plan, replicated_axes=set()) == rank
    with pytest.raises(ValueError):
        mesh.rank_coordinates(16)
    with pytest.raises(ValueError):
        MeshConfig(dp=0)


def test_module_without_parameters_is_rejected_by_the_optimizer_factory_path():
    class Empty(nn.Module):
        def forward(self, x):
            return x.sum()

    rt = RuntimeCore(model=Empty(), optimizer_factory=lambda p: torch.optim.SGD(p, lr=0.1))
    with pytest.raises((ValueError, RuntimeError)):
        rt.setup()


def test_plugin_bind_validation_with_stand_in_runtimes():
    """``bind`` rejects impossible configurations before any process group exists (stand-in runtimes, as the reference's
    ``tests/hdp_plugin_contract.py:215-241`` does)."""
    from types import SimpleNamespace

    from maltos_b200.parallel.hdp_helper import ByteScaleHdpBalancedConfig
    from maltos_b200.runtime.mesh import MeshConfig
    from maltos_b200.runtime.plugins.cp import ContextParallelPlugin
    from maltos_b200.runtime.plugins.hdp import ByteScaleHdpPlugin

    def runtime(mesh, plugins=()):
        return SimpleNamespace(mesh=mesh, plugins=list(plugins), has_plugin=lambda pid: any(p.id == pid for p in plugins))

    hdp = ByteScaleHdpPlugin(config=ByteScaleHdpBalancedConfig(partition_tokens=64))
    with pytest.raises(ValueError, match="DCP world size > 1"):
        hdp.bind(runtime(MeshConfig()))
    with pytest.raises(ValueError, match="cp_size=1"):
        hdp.bind(runtime(MeshConfig(dp=2, cp=2)))
    with pytest.raises(ValueError, match="pp_size=1"):
        hdp.bind(runtime(MeshConfig(dp=2, pp=2)))
    cp = ContextParallelPlugin()
    with pytest.raises(ValueError, match="mutually exclusive"):
        hdp.bind(runtime(MeshConfig(dp=2), [cp, hdp]))
    hdp.bind(runtime(MeshConfig(dp=2), [hdp]))                                     # the valid one
    with pytest.raises(ValueError, match="mesh.cp > 1"):
        cp.bind(runtime(MeshConfig(dp=2), [cp]))
    with pytest.raises(ValueError, match="mutually exclusive"):
        cp.bind(runtime(MeshConfig(cp=2), [cp, hdp]))


def test_context_parallel_local_loading_equals_runtime_sharding(tmp_path):
    """A loader that shards for its context-parallel rank hands out exactly what the plugin would cut from the whole batch."""
    import numpy as np

    from maltos_b200.data import PretrainingDataLoader, TokenShardDataset
    from maltos_b200.parallel import ContextParallelBatchSharder, ContextTokenPlannerType, build_context_token_planner

    np.random.default_rng(0).integers(0, 1000, size=4000, dtype=np.uint32).tofile(tmp_path / "tokens_00000.bin")
    for kind in (ContextTokenPlannerType.FIXED_ZIGZAG, ContextTokenPlannerType.FIXED_CONTIGUOUS):
        sharder = ContextParallelBatchSharder(build_context_token_planner(kind), 4)
        make = lambda **kw: PretrainingDataLoader(TokenShardDataset([tmp_path / "tokens_00000.bin"]), seq_len=32, micro_batch_size=2, **kw)  # noqa: E731
        whole = make().next_batch()
        for cp_rank in range(4):
            local = make(cp_batch_sharder=sharder).next_batch(cp_rank)
            cut = sharder.shard(whole, rank=cp_rank)
            for key in ("input_ids", "labels", "position_ids"):
                assert torch.equal(local[key], cut[key]), (kind, cp_rank, key)
            assert local["loss_weight"] == cut["loss_weight"] and local["position_offset"] == cut["position_offset"]
        # the four shares cover every token once
        covered = torch.cat([sharder.shard(whole, rank=r)["position_ids"][0] for r in range(4)]).sort().values
        assert torch.equal(covered, torch.arange(32))
    with pytest.raises(RuntimeError, match="cp_batch_sharder"):
        make().next_batch(1)


def test_torch_profiler_plugin_follows_its_schedule_and_writes_one_trace_per_cycle(tmp_path):
    from maltos_b200.runtime.plugins.torch_profiler import TorchProfilerPlugin

    plugin = TorchProfilerPlugin(str(tmp_path / "traces"), wait=1, warmup=1, active=2, repeat=2)
    rt = _runtime([plugin])
    rt.setup()
    for _ in range(9):                                   # two full cycles of 4 steps, then one more
        rt.run_step(torch.randn(4, 32))
        rt.step_optimizer()
    rt.close()
    names = sorted(p.name for p in (tmp_path / "traces" / "rank_00000").iterdir())
    assert names == ["trace.json", "trace_1.json"]
    events = json.loads((tmp_path / "traces" / "rank_00000" / "trace.json").read_text())["traceEvents"]
    spans = {e.get("name") for e in events}
    assert "maltos::forward" in spans and "maltos::backward" in spans
    # the active window holds exactly two optimizer steps
    assert sum(1 for e in events if e.get("name") == "maltos::micro_step_runner") == 2


def test_compile_plugin_is_scope_bookkeeping_only():
    """It validates the scope against the model's ``compile_spec()``, reports the covered modules and groups their parameters
    for ZeRO-3 - and compiles nothing: the modules are the same objects afterwards."""
    import maltos_b200.models as models
    from maltos_b200.runtime.plugins.compile import CompilePlugin

    torch.manual_seed(0)
    model = models.TinyTransformer(32, 4, 2, 64, 1e-5, 2, 64, 16)
    before = {n: id(m) for n, m in model.named_modules()}
    plugin = CompilePlugin(scope="mlp")
    rt = RuntimeCore(model=model, optimizer_factory=lambda p: torch.optim.SGD(p, lr=0.1), plugins=[plugin])
    rt.setup()
    assert {n: id(m) for n, m in rt.model.named_modules()} == before
    assert len(plugin.covered_paths) == 2 and all(p.endswith("mlp") for p in plugin.covered_paths)
    groups = plugin.param_materialization_groups()
    assert len(groups) == 2 and all(len(params) == 3 for _, params in groups)
    assert rt.collect_metrics()["compile/fused_scopes"] == 2
    rt.close()
    with pytest.raises(ValueError, match="not offered"):
        RuntimeCore(model=models.TinyTransformer(32, 4, 2, 64, 1e-5, 2, 64, 16), optimizer_factory=lambda p: torch.optim.SGD(p, lr=0.1),
                    plugins=[CompilePlugin(scope="attention_block_that_does_not_exist")]).setup()
    with pytest.raises(ValueError, match="compile_spec"):
        RuntimeCore(model=TinyModel(), optimizer_factory=lambda p: torch.optim.SGD(p, lr=0.1), plugins=[CompilePlugin()]).setup()
