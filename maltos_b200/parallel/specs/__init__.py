"""Model-side parallel declarations: a model says *where* it can be cut; plugins do the cutting."""
from .context import ContextParallelSpec
from .expert import ExpertParallelSpec
from .pipeline import PipelineParallelSpec
from .tp_sp import TpSpComm, TpSpParallelSpec, TpSpShardAxis, TpSpShardRule

__all__ = ["ContextParallelSpec", "ExpertParallelSpec", "PipelineParallelSpec", "TpSpComm", "TpSpParallelSpec",
           "TpSpShardAxis", "TpSpShardRule"]
