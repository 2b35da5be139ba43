"""Execution plan knobs that are not mesh sizes (reference ``parallel/plan.py:14-39``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from .context_interfaces import ContextParallelAttentionCoreType
from .context_token_planner import ContextTokenPlannerType


class PipelineScheduleType(str, Enum):
    ALL_FWD_ALL_BWD = "afab"
    ONE_FWD_ONE_BWD = "1f1b"


@dataclass(frozen=True)
class PipelineScheduleConfig:
    schedule: PipelineScheduleType | str = PipelineScheduleType.ONE_FWD_ONE_BWD
    microbatches: int = 1

    def __post_init__(self) -> None:
        object.__setattr__(self, "schedule", PipelineScheduleType(self.schedule))
        if self.microbatches < 1:
            raise ValueError(f"microbatches must be >= 1, got {self.microbatches}")


@dataclass(frozen=True)
class ParallelPlan:
    #: attention core installed by the context-parallel plugin
    cp_attn_core: ContextParallelAttentionCoreType = ContextParallelAttentionCoreType.ALL_GATHER_KV
    #: the data loader already emits this rank's CP slice, so the runtime does not slice after H2D
    batch_data_cp_aware: bool = False
    #: placement of canonical tokens on CP ranks (None = the default of the chosen core)
    cp_token_planner: ContextTokenPlannerType | None = None
    pp_schedule: PipelineScheduleConfig = field(default_factory=PipelineScheduleConfig)
    #: expert-parallel groups may borrow TP ranks (needs SP) / CP ranks before spilling into DP
    reuse_tp_for_ep: bool = True
    reuse_cp_for_ep: bool = True
