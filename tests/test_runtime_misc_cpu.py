"""SFT loader resume and DP interleave, ChainedWork re-firing, asynchronous metric reduction over two gloo ranks."""
import json

import numpy as np
import pytest
import torch

from maltos_b200.data.sft import PackedSFTDataset, SFTDataLoader
from maltos_b200.runtime.plugins.zero_common import ChainedWork
from maltos_b200.utils.sft_messages import EncodedSFTExample
from maltos_b200.utils.sft_packing import PackedSFTWriter, export_packing_metadata
from tests.dist_utils import run_distributed


def _sft_dataset(tmp_path, rows=11, seq_len=16):
    w = PackedSFTWriter(output_dir=tmp_path, seq_len=seq_len, sequences_per_shard=4, max_sequences=None, pad_token_id=0,
                        packing_algorithm="next_fit")
    for r in range(rows):
        w.add_example(EncodedSFTExample([1000 * (r + 1) + i for i in range(seq_len)], [0] * 4 + [1] * (seq_len - 4)))
    summary = w.finish()
    meta = {"format": "maltos_sft_packed", "format_version": 2,
            "packing": export_packing_metadata(summary=summary, seq_len=seq_len, sequences_per_shard=4, packing_algorithm="next_fit", packing_buffer_size=1)}
    (tmp_path / "meta.json").write_text(json.dumps(meta))
    return PackedSFTDataset(tmp_path)


def test_sft_loader_interleaves_ranks_wraps_and_resumes(tmp_path):
    ds = _sft_dataset(tmp_path)
    assert len(ds) == 11 and len(ds.shards) == 3
    world, mb = 2, 2
    loaders = [SFTDataLoader(ds, micro_batch_size=mb, dp_rank=r, dp_world_size=world) for r in range(world)]
    seen = []
    for step in range(5):                      # 20 rows drawn from 11: wraps around
        for r, ld in enumerate(loaders):
            b = ld.next_batch()
            assert set(b) == {"input_ids", "labels", "position_ids", "sequence_ids"} and b["input_ids"].dtype == torch.int64
            for i in range(mb):
                k = (step * mb + i) * world + r
                assert int(b["input_ids"][i, 0]) == 1000 * (k % 11 + 1)
                seen.append(k)
    assert sorted(seen) == list(range(20))
    state = loaders[1].state_dict().__dict__
    again = SFTDataLoader(ds, micro_batch_size=mb, dp_rank=1, dp_world_size=world)
    again.load_state_dict(json.loads(json.dumps(state)))
    for _ in range(3):
        assert torch.equal(loaders[1].next_batch()["input_ids"], again.next_batch()["input_ids"])
    assert again.consumed_sequences == loaders[1].consumed_sequences


class _Handle:
    def __init__(self, log, name):
        self.log, self.name = log, name

    def wait(self):
        self.log.append(f"wait:{self.name}")

    def block_current_stream(self):
        self.log.append(f"block:{self.name}")


def test_chained_work_replays_its_whole_chain_on_every_fire():
    log = []
    root = ChainedWork(None, lambda: (log.append("fire:a"), _Handle(log, "a"))[1])
    mid = ChainedWork(root, lambda: (log.append("fire:b"), _Handle(log, "b"))[1], blocks_by_stream=False)
    leaf = ChainedWork(mid, lambda: (log.append("fire:c"), _Handle(log, "c"))[1])
    leaf.wait()                                 # not fired yet: fires the chain, then waits on the leaf
    assert log == ["fire:a", "block:a", "fire:b", "wait:b", "fire:c", "wait:c"]
    log.clear()
    leaf.fire()                                 # persistent chain: a second round starts from the root again
    leaf.wait()
    assert log == ["fire:a", "block:a", "fire:b", "wait:b", "fire:c", "wait:c"]


def _metric_worker(rank, world):
    from maltos_b200.utils import metrics as M

    agg = M.MetricAggregator()
    agg.update({"loss": 1.0 + rank, "tokens": 10 * (rank + 1), "lr": 0.1 * (rank + 1), "fp16/overflow": rank == 1, "perf/step_sec": 2.0 + rank,
                "memory/max_allocated_gb": 3.0 + rank, "step": 5})
    pending = agg.flush_async(step_delta=1)
    # the reduction is in flight: more values can be recorded for the next interval meanwhile
    agg.update({"loss": 100.0})
    out = pending.wait()
    return out, agg.has_values()


def test_metric_reduction_rules_across_ranks():
    results = run_distributed(_metric_worker, 2)
    assert abs(results[0][0]["lr"] - 0.1) < 1e-12          # "rank0" values are not communicated: the logging rank keeps its own
    for out, has_more in results:
        assert has_more
        assert out["loss"] == 1.5                      # mean over ranks
        assert out["step"] == 5
        assert out["memory/max_allocated_gb"] == 4.0   # max over ranks
        assert bool(out["fp16/overflow"]) is True      # any
    assert results[0][0].keys() == results[1][0].keys()


def test_cuda_graph_plugin_refuses_communicating_plugins():
    """The recorded micro-step cannot contain collectives: the plugin must say so at bind time, not fail in a capture."""
    import maltos_b200  # noqa: F401
    from maltos_b200 import models
    from maltos_b200.runtime import RuntimeCore
    from maltos_b200.runtime.plugins.cuda_graph import CudaGraphPlugin
    from maltos_b200.runtime.plugins.grad_clip import GradClipPlugin
    from maltos_b200.runtime.plugins.zero1 import Zero1Plugin

    def model():
        return models.TinyTransformer(32, 2, 2, 64, 1e-5, 1, 64, 16)

    opt = lambda ps: torch.optim.AdamW(ps, lr=1e-3)   # noqa: E731
    rt = RuntimeCore(model=model(), plugins=[CudaGraphPlugin(), GradClipPlugin(1.0)], optimizer_factory=opt)
    rt.setup()                                        # local plugins are fine; on CPU batches simply run eagerly
    ids = torch.randint(0, 64, (2, 16))
    rt.run_step({"input_ids": ids, "labels": ids.roll(-1, 1)})
    rt.step_optimizer()
    assert rt.collect_metrics()["cuda_graph/replays"] == 0.0
    rt.close()
    with pytest.raises(ValueError, match="single-process"):
        RuntimeCore(model=model(), plugins=[CudaGraphPlugin(), Zero1Plugin()], optimizer_factory=opt).setup()


def test_fp16_master_weights_with_fused_adamw_keeps_master_gradients():
    """fp16 runs unscale and inf-check the optimizer's own gradients through a GradScaler, so with fp16 parameters the
    fused AdamW consumes fp32 master-gradient copies instead of taking the model gradients by reference."""
    from maltos_b200.runtime.optim import FusedAdamW, MasterWeightsOptimizer

    torch.manual_seed(0)
    for dtype, direct in ((torch.float16, False), (torch.bfloat16, True)):
        w = torch.nn.Parameter(torch.randn(8, 4).to(dtype))
        opt = MasterWeightsOptimizer([w], optimizer_factory=lambda ps: FusedAdamW(ps, lr=1e-2, weight_decay=0.0))
        assert opt._direct_grads is direct
        w.grad = torch.ones_like(w)
        opt.copy_master_params()
        master = opt.master_params[0]
        assert master.grad is not None and master.grad.dtype == torch.float32      # CPU: copies in both cases
        before = w.detach().clone()
        opt.step()
        assert not torch.equal(w.detach(), before) and w.dtype == dtype
        assert torch.allclose(w.detach().float(), master.detach(), atol=1e-2)


def _zero3_prefetch_worker(rank, world):
    import torch.nn as nn

    import maltos_b200  # noqa: F401
    from maltos_b200 import models
    from maltos_b200.models.tiny_transformer import RmsNorm
    from maltos_b200.runtime import MeshConfig, RuntimeCore
    from maltos_b200.runtime.plugins import zero3

    torch.manual_seed(1)
    model = models.TinyTransformer(32, 4, 2, 64, 1e-5, 2, 64, 16)
    plug = zero3.Zero3Plugin(wrap_cls={nn.Linear, nn.Embedding, RmsNorm})
    rt = RuntimeCore(model=model, mesh=MeshConfig(dp=world), plugins=[plug], grad_accum_steps=1,
                     optimizer_factory=lambda ps: torch.optim.SGD(ps, lr=0.1))
    rt.setup()
    claimed_ahead, claimed_total = [0], [0]
    inner = plug._gather

    def counting_gather(b):
        claimed_total[0] += 1
        claimed_ahead[0] += int(b.prefetched)
        return inner(b)

    plug._gather = counting_gather
    g = torch.Generator().manual_seed(5 + rank)
    stats = []
    for step in range(2):
        ids = torch.randint(0, 64, (2, 16), generator=g)
        rt.run_step({"input_ids": ids, "labels": ids.roll(-1, 1)})
        stats.append((claimed_ahead[0], claimed_total[0], plug._order_final, len(plug._reduces),
                      all(not b.materialized and b.full_tensor.untyped_storage().size() == 0 for b in plug.buckets)))
        claimed_ahead[0] = claimed_total[0] = 0
        rt.step_optimizer()
    rt.close()
    return stats, len(plug.buckets)


def test_zero3_prefetches_in_observed_order_and_releases_everything():
    """First pass: the bucket order is observed (the backward already prefetches). Second pass: every bucket but the
    first of each direction is claimed from a gather that was started ahead of its use; after each micro-step no bucket
    holds memory and no reduce-scatter is left in flight."""
    results = run_distributed(_zero3_prefetch_worker, 2)
    for stats, n_buckets in results:
        (ahead0, total0, final0, pending0, clean0), (ahead1, total1, final1, pending1, clean1) = stats
        assert final0 and final1 and pending0 == 0 and pending1 == 0 and clean0 and clean1
        assert total0 == total1 == 2 * n_buckets
        assert ahead0 >= n_buckets // 2            # backward of the first pass
        assert ahead1 >= 2 * n_buckets - 6         # both directions of the second pass


def test_exposed_communication_is_comm_time_not_covered_by_compute():
    from maltos_b200.utils.profiling import exposed_comm_us, is_comm_kernel

    assert is_comm_kernel("ncclDevKernel_ReduceScatter_Sum_bf16_RING_LL(...)") and is_comm_kernel("void mb::pull_all_gather_kernel<8>(...)")
    assert not is_comm_kernel("void mb::gemm_bf16_pair_kernel<true>(...)")
    kernels = [("gemm", 0, 100), ("nccl_ag", 50, 100),          # 50..150: 50 us hidden, 50 us exposed
               ("gemm", 200, 50), ("pull_reduce_scatter", 210, 20),   # fully hidden
               ("nccl_ar", 300, 40), ("nccl_ar2", 320, 40),     # overlapping comm kernels, nothing else: 60 us exposed
               ("flash", 355, 100)]                             # covers the last 5 us of the comm union
    exposed, total, busy = exposed_comm_us(kernels)
    assert total == 100 + 20 + 60 and exposed == 50 + 0 + 55
    assert busy == 150 + 50 + (455 - 300)


def test_nvtx_ranged_library_brackets_launchers_only(monkeypatch):
    """With ``MALTOS_B200_NVTX=1`` every launcher call runs inside a range named after its C entry point; queries and
    setters do not; ``restype`` assignments reach the real function."""
    from maltos_b200.ops import _lib

    events = []

    class Fn:
        def __init__(self, name):
            self.name, self.restype = name, None

        def __call__(self, *args):
            events.append(("call", self.name, args))
            return 0

    class Handle:
        def __init__(self):
            self.fns = {}

        def __getattr__(self, name):
            return self.fns.setdefault(name, Fn(name))

    monkeypatch.setattr(_lib, "_range_push", lambda name: events.append(("push", name)))
    monkeypatch.setattr(_lib, "_range_pop", lambda: events.append(("pop",)))
    handle = Handle()
    ranged = _lib._RangedLibrary(handle)
    assert ranged.mb_gemm_bf16(1, 2) == 0
    assert events == [("push", "mb_gemm_bf16"), ("call", "mb_gemm_bf16", (1, 2)), ("pop",)]
    events.clear()
    ranged.mb_launch_count()
    ranged.mb_set_wait_timeout_ms(5)
    ranged.mb_status_fetch_and_clear(None, None)
    assert [e[0] for e in events] == ["call", "call", "call"]
    ranged.mb_flash_attn_bwd.restype = "marker"
    assert handle.fns["mb_flash_attn_bwd"].restype == "marker"
    monkeypatch.setenv("MALTOS_B200_NVTX", "1")
    assert _lib.nvtx_enabled()


def test_poison_fill_is_opt_in_and_limited_to_transfer_buffers(monkeypatch):
    from maltos_b200.ops import symm

    monkeypatch.delenv("MALTOS_B200_POISON", raising=False)
    assert not symm.poison_wanted("sp_partial")
    monkeypatch.setenv("MALTOS_B200_POISON", "1")
    assert symm.poison_wanted("sp_partial") and symm.poison_wanted("ring_kv")
    for name in ("signal_pad", "ring_dkv", "moe_dispatch_0", "zero3.shard.0", "ddp.grad"):
        assert not symm.poison_wanted(name)


def test_gemm_wrapper_handles_empty_problems_without_a_launch(monkeypatch):
    """An expert without tokens reaches the GEMM wrapper with zero rows (forward, dgrad) or an empty contraction (wgrad):
    the kernel library rejects empty problems, so the wrapper must answer them itself."""
    from maltos_b200.ops import _lib, gemm as G

    monkeypatch.setattr(_lib, "use_kernels", lambda *t: True)
    monkeypatch.setattr(_lib, "lib", lambda: (_ for _ in ()).throw(AssertionError("no launch expected")))
    w = torch.randn(6, 8).bfloat16()
    y = G.gemm(torch.zeros(0, 8).bfloat16(), w)
    assert y.shape == (0, 6)
    dw = G.gemm(torch.zeros(0, 6).bfloat16(), torch.zeros(0, 8).bfloat16(), a_mn=True, b_mn=True)
    assert dw.shape == (6, 8) and float(dw.abs().sum()) == 0.0
    acc = torch.ones(6, 8)
    G.gemm(torch.zeros(0, 6).bfloat16(), torch.zeros(0, 8).bfloat16(), a_mn=True, b_mn=True, out=acc, accumulate=True)
    assert float(acc.sum()) == 48.0


def test_experts_without_tokens_are_entered_only_when_hooks_need_it():
    from maltos_b200.ops.moe import moe_experts_forward

    calls = []

    class E(torch.nn.Module):
        def __init__(self, i):
            super().__init__()
            self.i, self.lin = i, torch.nn.Linear(4, 4)

        def forward(self, x):
            calls.append((self.i, x.shape[0]))
            return self.lin(x)

    experts = [E(i) for i in range(3)]
    flat = torch.randn(5, 4)
    idx = torch.zeros(5, 1, dtype=torch.long)             # every token to expert 0
    gate = torch.ones(5, 1)
    moe_experts_forward(flat, idx, gate, None, experts)
    assert calls == [(0, 5)]
    calls.clear()
    experts[2].lin.register_forward_pre_hook(lambda m, a: None)      # what a parameter-sharding plugin installs
    moe_experts_forward(flat, idx, gate, None, experts)
    assert calls == [(0, 5), (2, 0)]


def test_wandb_that_cannot_start_degrades_to_the_other_sinks(monkeypatch, capsys):
    """Only rank 0 builds loggers; an exception there would leave the other ranks in their next collective until the
    process-group timeout. The run goes on with console / JSONL logging unless the environment makes W&B mandatory."""
    import argparse

    from maltos_b200.train import cli
    from maltos_b200.utils import metrics

    def broken(**kw):
        raise RuntimeError("No API key configured")

    monkeypatch.setattr(metrics, "WandbMetricLogger", broken)
    args = argparse.Namespace(metrics_jsonl=None, wandb_project="p", wandb_mode=None, wandb_run_name=None, wandb_entity=None, wandb_run_id=None,
                              wandb_tags=None, wandb_checkpoint_every=5)
    loggers, uploader = cli._build_logging(args, 0)
    assert len(loggers) == 1 and uploader is None
    assert "could not be" in capsys.readouterr().err
    assert cli._build_logging(args, 1) == (None, None)
    monkeypatch.setenv("MALTOS_B200_WANDB_REQUIRED", "1")
    with pytest.raises(RuntimeError):
        cli._build_logging(args, 0)


def test_head_counts_that_tensor_parallelism_cannot_split_are_rejected_up_front():
    from maltos_b200.train import cli, flags as F

    base = ["--model", "llama", "--dim", "64", "--hidden-size", "128", "--n-layers", "2", "--vocab-size", "256", "--seq-len", "32"]
    ok = F.parse_args_from(base + ["--n-heads", "8", "--n-kv-heads", "4", "--tp-size", "4"], require_data=False)
    cli.validate_args(ok, 4)
    for extra, world, needle in ((["--n-heads", "8", "--n-kv-heads", "2", "--tp-size", "4"], 4, "--n-kv-heads=2 must be divisible by --tp-size=4"),
                                 (["--n-heads", "6", "--n-kv-heads", "4"], 1, "multiple of --n-kv-heads"),
                                 (["--n-heads", "5", "--n-kv-heads", "5"], 1, "--dim=64 must be divisible")):
        with pytest.raises(ValueError, match=needle):
            cli.validate_args(F.parse_args_from(base + extra, require_data=False), world)


def test_sequence_parallel_split_refuses_lengths_it_would_truncate():
    from maltos_b200.train import cli, flags as F

    base = ["--model", "llama", "--dim", "64", "--n-heads", "4", "--hidden-size", "128", "--n-layers", "2", "--vocab-size", "256", "--tp-size", "4", "--use-sp"]
    cli.validate_args(F.parse_args_from(base + ["--seq-len", "32"], require_data=False), 4)
    with pytest.raises(ValueError, match="must be divisible by --tp-size=4"):
        cli.validate_args(F.parse_args_from(base + ["--seq-len", "30"], require_data=False), 4)
    with pytest.raises(ValueError, match="must be divisible by --tp-size=4"):      # 48 / cp 2 = 24 per context-parallel rank: fine; 40 / 2 = 20: fine; 36 / 2 = 18: not
        cli.validate_args(F.parse_args_from(base + ["--seq-len", "36", "--cp-size", "2"], require_data=False), 8)


def test_tensor_parallel_overlap_workspace_is_sized_and_prewarmed_at_setup(monkeypatch):
    """The kind of the reference's ``tests/tp_native_overlap_workspace.py``: size estimate, prewarm on / off, command-line
    wiring, prewarm at plugin finalisation."""
    from unittest import mock

    import torch.distributed as dist
    import torch.nn as nn

    from maltos_b200.ops import comm, fused_tp
    from maltos_b200.runtime.layers import functional as Fn
    from maltos_b200.runtime.plugins import tp_sp
    from maltos_b200.runtime.types import SetupPhase
    from maltos_b200.train import cli, flags as F

    one = Fn.native_comm_overlap_workspace_bytes(micro_batch_size=1, seq_len=4096, hidden_size=5120, tp_size=2, dtype=torch.bfloat16)
    two = Fn.native_comm_overlap_workspace_bytes(micro_batch_size=2, seq_len=4096, hidden_size=5120, tp_size=2, dtype=torch.bfloat16)
    assert one == 80 * 2**20 and two == 160 * 2**20          # two parities of the full-sequence hidden states
    with pytest.raises(ValueError, match="must be divisible"):
        Fn.native_comm_overlap_workspace_bytes(micro_batch_size=1, seq_len=4095, hidden_size=5120, tp_size=2, dtype=torch.bfloat16)
    assert fused_tp.workspace_plan(2, 1024) == {"sp_gather": 1024, "sp_publish": 512, "sp_scatter": 1024}
    assert fused_tp.workspace_plan(8, 1024) == {"sp_gather": 1024, "sp_publish": 128, "sp_partial": 1024}
    assert fused_tp.workspace_plan(1, 1024) == {}

    group, symm = object(), mock.Mock()
    symm.world = 4
    symm.ensure_buffer.side_effect = lambda name, nbytes: mock.Mock(nbytes=nbytes)
    with mock.patch.object(torch.cuda, "is_available", return_value=True), mock.patch.object(torch.cuda, "synchronize") as sync, \
            mock.patch.object(dist, "get_backend", return_value="nccl"), mock.patch.object(comm, "context_for", return_value=symm) as ctx_for:
        assert Fn.prewarm_native_comm_overlap_workspace(group, min_workspace_bytes=4096) is True
    ctx_for.assert_called_once_with(group)
    assert {c.args for c in symm.ensure_buffer.call_args_list} == {("sp_gather", 4096), ("sp_publish", 1024), ("sp_partial", 4096)}
    sync.assert_called_once_with()
    with mock.patch.object(torch.cuda, "is_available", return_value=True), mock.patch.object(dist, "get_backend", return_value="gloo"), \
            mock.patch.object(comm, "context_for") as ctx_for:
        assert Fn.prewarm_native_comm_overlap_workspace(group, min_workspace_bytes=1) is False
    ctx_for.assert_not_called()

    args = F.parse_args_from(["--model", "llama", "--dim", "384", "--n-heads", "6", "--hidden-size", "1536", "--n-layers", "2", "--vocab-size", "256",
                              "--seq-len", "512", "--micro-batch-size", "1", "--dp-size", "2", "--tp-size", "2", "--use-sp", "--zero-stage", "3",
                              "--precision", "bf16", "--tp-native-comm-overlap"], require_data=False)
    runtime = cli._build_runtime(args, nn.Linear(1, 1), torch.device("cpu"))
    plugin = next(p for p in runtime.plugins if isinstance(p, tp_sp.TpSpPlugin))
    assert plugin.native_comm_overlap is True and plugin.native_comm_overlap_workspace_bytes == 2 * 512 * 384 * 2

    plugin = tp_sp.TpSpPlugin(native_comm_overlap=True, native_comm_overlap_workspace_bytes=80 * 2**20)
    plugin.runtime = mock.Mock()
    plugin.runtime.get_group.return_value = group
    with mock.patch.object(tp_sp, "prewarm_native_comm_overlap_workspace", return_value=True) as prewarm, \
            mock.patch.object(tp_sp.TensorParallelTransformPlugin, "on_setup_phase", lambda self, phase, model: model), \
            mock.patch.object(tp_sp.TpSpPlugin, "_wire_sequence_rules"), mock.patch.object(tp_sp.TpSpPlugin, "_collect_partial_params"):
        plugin.on_setup_phase(SetupPhase.FINALIZE, nn.Linear(1, 1))
    prewarm.assert_called_once_with(group, min_workspace_bytes=80 * 2**20)
    assert plugin.native_comm_overlap_workspace_prewarmed is True


def test_pipeline_micro_batches_must_divide_the_micro_batch():
    from maltos_b200.train import cli, flags as F

    base = ["--model", "llama", "--dim", "64", "--n-heads", "4", "--hidden-size", "128", "--n-layers", "2", "--vocab-size", "256", "--seq-len", "32",
            "--pp-size", "2"]
    cli.validate_args(F.parse_args_from(base + ["--micro-batch-size", "4", "--pp-microbatches", "2"], require_data=False), 2)
    with pytest.raises(ValueError, match="divisible by --pp-microbatches=2"):
        cli.validate_args(F.parse_args_from(base + ["--micro-batch-size", "3", "--pp-microbatches", "2"], require_data=False), 2)


def test_tied_embeddings_are_refused_when_a_plugin_splits_the_model():
    from maltos_b200.models import LlamaConfig, LlamaForCausalLM
    from maltos_b200.runtime import MeshConfig, RuntimeCore
    from maltos_b200.runtime.plugins.tp import TensorParallelPlugin

    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
                      max_position_embeddings=16, tie_word_embeddings=True)
    plain = RuntimeCore(model=LlamaForCausalLM(cfg), optimizer_factory=lambda p: torch.optim.SGD(p, lr=0.1))
    plain.setup()                                          # one process, nothing split: tying is fine
    ids = torch.randint(0, 64, (2, 16))
    plain.run_step({"input_ids": ids, "labels": ids.roll(-1, 1)})
    assert plain.model.lm_head.weight is plain.model.embed_tokens.weight
    split = RuntimeCore(model=LlamaForCausalLM(cfg), mesh=MeshConfig(tp=2), optimizer_factory=lambda p: torch.optim.SGD(p, lr=0.1),
                        plugins=[TensorParallelPlugin()])
    with pytest.raises(ValueError, match="shared between modules"):
        split.setup()
