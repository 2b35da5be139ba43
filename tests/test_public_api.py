"""The import paths and signatures a user of the reference relies on (its ``runtime/__init__.py:5-64``,
``state/__init__.py:27-47``, ``runtime/core.py:39-52``, ``train/flags.py:60-212``): every name exists here under the same
path and the constructors take the same keywords with the same defaults."""
import importlib
import inspect

import pytest

SURFACE = {
    "maltos_b200.runtime": "RuntimeCore MeshConfig MeshAxis ProcessGroupManager RuntimePlugin PluginId RuntimePhase SetupPhase StepContext "
                           "RuntimeState ParamRole PpStatus MetricValue StepRunner DefaultStepRunner PipelineStepRunner PipelineScheduleKind BufferHandle "
                           "BufferPolicy acquire_buffer release_buffer clear_buffer_pool global_buffer_pool TpSpParallelizableModule "
                           "PipelineParallelizableModule ContextParallelizableModule ExpertParallelizableModule",
    "maltos_b200.runtime.types": "LossOutput PipelineOutput PpStatus",
    "maltos_b200.runtime.plugins.ddp": "DataParallelPlugin BucketDataParallelPlugin",
    "maltos_b200.runtime.plugins.tp": "TensorParallelPlugin",
    "maltos_b200.runtime.plugins.tp_sp": "TpSpPlugin",
    "maltos_b200.runtime.plugins.pp": "PipelineParallelPlugin",
    "maltos_b200.runtime.plugins.cp": "ContextParallelPlugin",
    "maltos_b200.runtime.plugins.hdp": "ByteScaleHdpPlugin",
    "maltos_b200.runtime.plugins.ep": "ExpertParallelPlugin",
    "maltos_b200.runtime.plugins.zero1": "Zero1Plugin",
    "maltos_b200.runtime.plugins.zero2": "Zero2Plugin",
    "maltos_b200.runtime.plugins.zero3": "Zero3Plugin",
    "maltos_b200.runtime.plugins.fp16": "Fp16Plugin",
    "maltos_b200.runtime.plugins.grad_clip": "GradClipPlugin",
    "maltos_b200.runtime.plugins.metrics": "MetricPlugin",
    "maltos_b200.runtime.plugins.torch_profiler": "TorchProfilerPlugin",
    "maltos_b200.runtime.plugins.compile": "CompilePlugin",
    "maltos_b200.parallel": "ParallelPlan PipelineScheduleConfig specs protocols ContextParallelAttentionCoreType ContextTokenPlannerType "
                            "FixedContiguousTokenPlanner FixedZigzagTokenPlanner build_context_token_planner ContextParallelBatchSharder",
    "maltos_b200.parallel.hdp_helper": "ByteScaleHdpBalancedConfig ByteScaleHdpCostModel DocumentIndices",
    "maltos_b200.state": "StateManager ModelStateMeta ParamEntry RuntimeParamAttrs RngState TrainerState OptimizerState CheckpointManifest "
                         "save_sharded_checkpoint load_sharded_checkpoint load_checkpoint_manifest save_runtime_spec load_runtime_spec "
                         "save_logical_checkpoint load_logical_checkpoint load_logical_tensor iter_logical_checkpoint_tensors "
                         "iter_logical_tensors_from_runtime_checkpoint",
    "maltos_b200.data": "TokenShardDataset PretrainingDataLoader PretrainingDataState PackedSFTDataset SFTDataLoader SFTDataState "
                        "SimpleTensorDataLoader SimpleDataLoaderState PrefetchDataLoader StatefulDataLoaderProtocol",
    "maltos_b200.data.bytescale_hdp": "ByteScaleHdpDataLoader",
    "maltos_b200.train": "Trainer TrainerConfig",
    "maltos_b200.train.flags": "build_arg_parser parse_args_from build_runtime_spec parse_runtime_spec_args",
    "maltos_b200.train.cli": "main _build_model _build_runtime _build_dataloader _build_optimizer_factory _build_hdp_config _global_batch_tokens",
    "maltos_b200.utils.constants": "", "maltos_b200.utils.distributed": "", "maltos_b200.utils.metrics": "", "maltos_b200.utils.attention_backend": "",
    "maltos_b200.utils.losses": "", "maltos_b200.utils.profiling": "", "maltos_b200.utils.activation_checkpoint": "",
}


@pytest.mark.parametrize("module", sorted(SURFACE))
def test_module_exports(module):
    mod = importlib.import_module(module)
    missing = [n for n in SURFACE[module].split() if not hasattr(mod, n)]
    assert not missing, (module, missing)


def _defaults(fn):
    return {n: p.default for n, p in inspect.signature(fn).parameters.items() if n != "self" and p.default is not inspect.Parameter.empty}


def test_constructor_keywords_and_defaults():
    from maltos_b200.data import PretrainingDataLoader, SimpleTensorDataLoader
    from maltos_b200.parallel import ParallelPlan
    from maltos_b200.parallel.hdp_helper import ByteScaleHdpBalancedConfig, ByteScaleHdpCostModel
    from maltos_b200.runtime import RuntimeCore
    from maltos_b200.runtime.plugins import compile as compile_plugin, ddp, ep, metrics, pp, torch_profiler, tp_sp, zero1, zero2
    from maltos_b200.runtime.types import LossOutput
    from maltos_b200.state import iter_logical_tensors_from_runtime_checkpoint, load_sharded_checkpoint, save_sharded_checkpoint
    from maltos_b200.train import TrainerConfig

    core = inspect.signature(RuntimeCore.__init__).parameters
    assert list(core)[1:] == ["model", "mesh", "plan", "device", "dtype", "grad_accum_steps", "grad_clip_max_norm", "optimizer_factory",
                              "scheduler_factory", "plugins", "state_manager", "state"]
    assert core["grad_accum_steps"].default == 1 and core["grad_clip_max_norm"].default is None
    for method in ("setup run_step step_optimizer collect_metrics close get_group get_optimizer_and_scheduler create_optimizer create_scheduler "
                   "set_param_role get_param_role mark_module_path_omitted is_module_path_omitted add_module_replacement get_module_replacements "
                   "grad_norm_replica_factor should_save_optimizer optimizer_checkpoint_rank model_state_checkpoint_rank").split():
        assert callable(getattr(RuntimeCore, method)), method
    assert _defaults(RuntimeCore.setup) == {"checkpoint_path": None, "load_weights_only": False}

    assert _defaults(ddp.DataParallelPlugin.__init__)["async_op"] is False
    assert _defaults(ddp.BucketDataParallelPlugin.__init__)["bucket_mb_size"] == 25
    assert _defaults(zero1.Zero1Plugin.__init__)["bucket_mb_size"] == 25 and _defaults(zero2.Zero2Plugin.__init__)["bucket_mb_size"] == 25
    assert _defaults(ep.ExpertParallelPlugin.__init__)["bucket_mb_size"] == 25
    assert _defaults(pp.PipelineParallelPlugin.__init__)["schedule"] == "afab"
    assert _defaults(tp_sp.TpSpPlugin.__init__) == {"native_comm_overlap": False, "native_comm_overlap_workspace_bytes": None}
    assert _defaults(compile_plugin.CompilePlugin.__init__) == {"scope": "mlp", "backend": "inductor", "mode": "default"}
    assert _defaults(metrics.MetricPlugin.__init__)["include_cuda_memory"] is True
    assert _defaults(torch_profiler.TorchProfilerPlugin.__init__) == {"wait": 1, "warmup": 1, "active": 2, "repeat": 1, "record_shapes": False,
                                                                        "profile_memory": False, "with_stack": False, "with_flops": False,
                                                                        "rank0_only": False}
    plan = _defaults(ParallelPlan)
    assert plan["batch_data_cp_aware"] is False and plan["cp_token_planner"] is None and plan["reuse_tp_for_ep"] is True and plan["reuse_cp_for_ep"] is True
    assert plan["cp_attn_core"].value == "all_gather_kv"
    assert set(inspect.signature(ByteScaleHdpBalancedConfig).parameters) >= {"partition_tokens", "balance_delta", "cost_model"}
    assert list(inspect.signature(ByteScaleHdpCostModel).parameters)[:3] == ["alpha", "beta", "gamma"]
    assert list(inspect.signature(LossOutput).parameters) == ["loss", "metrics", "auxiliary_loss"]

    trainer = inspect.signature(TrainerConfig).parameters
    assert list(trainer) == ["max_steps", "log_every", "checkpoint_every", "checkpoint_dir", "resume_from", "load_weights_only", "checkpoint_keep_last",
                             "checkpoint_keep_every_n_steps", "checkpoint_min_free_gb", "data_prefetch_batches"]
    assert _defaults(PretrainingDataLoader.__init__) == {"dp_rank": 0, "dp_world_size": 1, "seed": 1234, "start_state": None, "cp_batch_sharder": None}
    assert _defaults(SimpleTensorDataLoader.__init__) == {"drop_last": True, "cp_batch_sharder": None}
    assert _defaults(save_sharded_checkpoint) == {"min_free_gb": None} and _defaults(load_sharded_checkpoint) == {"weights_only": False}
    assert _defaults(iter_logical_tensors_from_runtime_checkpoint) == {"ep_size": 1, "dp_size": 1, "tp_size": 1, "pp_size": 1, "cp_size": 1}


def test_every_flag_of_the_reference_command_line_parses():
    from maltos_b200.train.flags import build_arg_parser

    flags = {opt for action in build_arg_parser()._actions for opt in action.option_strings}
    wanted = """--data --data-format --token-dtype --seq-len --micro-batch-size --data-prefetch-batches --max-steps --dry-run --grad-accum-steps --lr
        --weight-decay --adam-beta1 --adam-beta2 --adam-eps --fused-adamw --lr-schedule --warmup-steps --min-lr --seed --model --dim --n-heads --n-kv-heads
        --hidden-size --n-layers --num-experts --moe-aux-loss-coef --vocab-size --eps --attention-backend --activation-checkpointing
        --activation-checkpoint-every-n-layers --dp-size --pp-size --pp-microbatches --cp-size --tp-size --ep-size --use-sp --zero-stage --ddp-mode
        --tp-native-comm-overlap --cp-attn-core --batch-data-cp-aware --cp-token-planner --hdp-balanced --hdp-partition-tokens --hdp-cost-alpha
        --hdp-cost-beta --hdp-cost-gamma --hdp-balance-delta --precision --grad-clip --compile --compile-scope --compile-mode --disable-metrics
        --log-every --metrics-jsonl --run-manifest --wandb-project --wandb-entity --wandb-run-name --wandb-run-id --wandb-mode --wandb-tags
        --wandb-checkpoint-every --checkpoint-dir --checkpoint-every --checkpoint-keep-last --checkpoint-keep-every-n-steps --checkpoint-min-free-gb
        --resume-from --load-weights-only --backend --master-addr --master-port --config --pp-schedule --rope-theta --moe-top-k --moe-capacity-factor
        --init-std""".split()
    missing = [f for f in wanted if f not in flags]
    assert not missing, missing
    assert sum(f.startswith("--torch-profiler") for f in flags) >= 10
