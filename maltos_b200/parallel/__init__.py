"""Parallel declarations: plans, model-side specs, protocols and CP token planners (no process groups here)."""
from .context_batch import ContextParallelBatchSharder
from .context_interfaces import ContextParallelAttentionCore, ContextParallelAttentionCoreType
from .context_token_planner import (ContextTokenPlan, ContextTokenPlanner, ContextTokenPlannerType,
                                    FixedContiguousTokenPlanner, FixedZigzagTokenPlanner, build_context_token_planner)
from .expert_interfaces import ExpertParallelMoEModule
from .plan import ParallelPlan, PipelineScheduleConfig, PipelineScheduleType
from .protocols import (CompilableModule, ContextParallelizableModule, ExpertParallelizableModule,
                        FlopsEstimatableModule, PipelineParallelizableModule, TpSpParallelizableModule)
from .specs import (ContextParallelSpec, ExpertParallelSpec, PipelineParallelSpec, TpSpComm, TpSpParallelSpec,
                    TpSpShardAxis, TpSpShardRule)

__all__ = [
    "CompilableModule", "ContextParallelAttentionCore", "ContextParallelAttentionCoreType", "ContextParallelBatchSharder",
    "ContextParallelSpec", "ContextParallelizableModule", "ContextTokenPlan", "ContextTokenPlanner",
    "ContextTokenPlannerType", "ExpertParallelMoEModule", "ExpertParallelSpec", "ExpertParallelizableModule",
    "FixedContiguousTokenPlanner", "FixedZigzagTokenPlanner", "FlopsEstimatableModule", "ParallelPlan",
    "PipelineParallelSpec", "PipelineParallelizableModule", "PipelineScheduleConfig", "PipelineScheduleType",
    "TpSpComm", "TpSpParallelSpec", "TpSpParallelizableModule", "TpSpShardAxis", "TpSpShardRule",
    "build_context_token_planner",
]
