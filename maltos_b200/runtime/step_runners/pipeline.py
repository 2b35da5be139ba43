"""Pipeline-parallel step runner: AFAB and 1F1B over NCCL/gloo point-to-point.

One ``run`` consumes a whole micro-step batch, cuts it into ``plan.pp_schedule.microbatches`` pieces along dim 0
and executes this stage's action list. Boundary activations / gradients travel with batched isend/irecv between
ranks that share (dp, cp, tp); receives land in persistent per-micro-batch buffers. ``pp_status`` is set per
action so that ZeRO/DDP plugins see the accumulation window of the *whole* micro-step
(reference ``runtime/step_runners/pipeline.py:67-332``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import TYPE_CHECKING, Any

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.runtime.buffer_allocator import BufferPolicy, acquire_buffer
from maltos_b200.runtime.types import LossOutput, PipelineOutput, PpStatus
from maltos_b200.utils.constants import (AUX_LOSS_WEIGHT_KEY, HIDDEN_STATES_KEY, INPUT_IDS_KEY, LABELS_KEY, LOSS_SCALE_KEY, LOSS_TARGET_COUNTS_KEY, LOSS_WEIGHT_KEY, POSITION_IDS_KEY,
                                         POSITION_OFFSET_KEY, SEQUENCE_IDS_KEY)
from maltos_b200.utils.distributed import all_reduce_tensor, irecv_tensor_async, isend_tensor_async
from maltos_b200.utils.profiling import span

from .base import DefaultStepRunner

if TYPE_CHECKING:
    from maltos_b200.runtime.plugins.pp import PipelineParallelPlugin


class PipelineScheduleKind(str, Enum):
    AFAB = "afab"
    ONE_FWD_ONE_BWD = "1f1b"


class PipelineActionKind(str, Enum):
    FORWARD = "forward"
    BACKWARD = "backward"


@dataclass(frozen=True)
class PipelineAction:
    kind: PipelineActionKind
    microbatch_idx: int
    backward_step_idx: int = 0


@dataclass
class PipelineMicroState:
    input_activation: torch.Tensor | None = None
    output_activation: torch.Tensor | None = None
    raw_loss: torch.Tensor | None = None
    auxiliary_loss: torch.Tensor | None = None
    pending_sends: list = field(default_factory=list)


def afab_actions(m: int) -> list[PipelineAction]:
    fwd = [PipelineAction(PipelineActionKind.FORWARD, i) for i in range(m)]
    bwd = [PipelineAction(PipelineActionKind.BACKWARD, mb, step) for step, mb in enumerate(reversed(range(m)))]
    return fwd + bwd


def one_f_one_b_actions(m: int, stage: int, stages: int) -> list[PipelineAction]:
    warm = min(stages - stage - 1, m)
    out = [PipelineAction(PipelineActionKind.FORWARD, i) for i in range(warm)]
    for b in range(m):
        f = warm + b
        if f < m:
            out.append(PipelineAction(PipelineActionKind.FORWARD, f))
        out.append(PipelineAction(PipelineActionKind.BACKWARD, b, b))
    return out


_PASS_THROUGH_KEYS = (POSITION_OFFSET_KEY, POSITION_IDS_KEY, SEQUENCE_IDS_KEY, AUX_LOSS_WEIGHT_KEY)


@dataclass(frozen=True)
class PipelineStepRunner:
    plugin: "PipelineParallelPlugin"

    # ------------------------------------------------------------------ schedule
    def build_schedule(self, num_microbatches: int) -> list[PipelineAction]:
        kind = PipelineScheduleKind(self.plugin.schedule)
        if kind is PipelineScheduleKind.AFAB:
            return afab_actions(num_microbatches)
        return one_f_one_b_actions(num_microbatches, self.plugin.stage_index, self.plugin.stage_count)

    @staticmethod
    def build_afab_schedule(num_microbatches: int) -> list[PipelineAction]:
        return afab_actions(num_microbatches)

    def build_1f1b_schedule(self, num_microbatches: int) -> list[PipelineAction]:
        return one_f_one_b_actions(num_microbatches, self.plugin.stage_index, self.plugin.stage_count)

    # ------------------------------------------------------------------ driver
    def run(self, runtime, batch) -> torch.Tensor:
        m = runtime.plan.pp_schedule.microbatches
        pieces = split_batch(batch, m)
        states = [PipelineMicroState() for _ in range(m)]
        totals: dict[str, torch.Tensor | None] = {"loss": None, "aux": None}
        for action in self.build_schedule(m):
            with span(f"maltos::pp.{action.kind.value}.microbatch_{action.microbatch_idx}"):
                if action.kind is PipelineActionKind.FORWARD:
                    self._forward(runtime, pieces[action.microbatch_idx], states[action.microbatch_idx], action, totals)
                else:
                    self._backward(runtime, states[action.microbatch_idx], action, m)
        for st in states:
            for work in st.pending_sends:
                work.wait()
            st.pending_sends.clear()
        loss = self.broadcast_loss(runtime=runtime, total_loss=totals["loss"], total_auxiliary_loss=totals["aux"], batch=pieces[0])
        runtime.state.loss = loss
        # the metric of this micro-step is the mean loss over its pipeline micro-batches, on every stage
        runtime.state.metadata["raw_loss_for_metrics"] = loss.detach().float()
        return loss

    @property
    def _first(self) -> bool:
        return self.plugin.prev_global_rank is None

    @property
    def _last(self) -> bool:
        return self.plugin.next_global_rank is None

    def _forward(self, runtime, piece, st: PipelineMicroState, action: PipelineAction, totals) -> None:
        runtime.state.step_context.set_pp_state(microbatch_idx=action.microbatch_idx, status=PpStatus.FORWARD)
        if self._first:
            model_input: Any = piece
        else:
            buf, work = self.recv_activation_async(runtime, piece)
            work.wait()
            buf.requires_grad_(True)
            st.input_activation = buf
            model_input = {HIDDEN_STATES_KEY: buf}
            if isinstance(piece, dict):
                for key in _PASS_THROUGH_KEYS:
                    if key in piece:
                        model_input[key] = piece[key]
            if self._last:
                model_input[LABELS_KEY] = extract_labels(piece)
                if isinstance(piece, dict) and LOSS_WEIGHT_KEY in piece:
                    model_input[LOSS_WEIGHT_KEY] = piece[LOSS_WEIGHT_KEY]
                if isinstance(piece, dict) and LOSS_SCALE_KEY in piece:
                    model_input[LOSS_SCALE_KEY] = piece[LOSS_SCALE_KEY]
        DefaultStepRunner.run_forward(runtime, model_input)
        out = runtime.state.outputs

        def _add(name: str, value: torch.Tensor) -> None:
            totals[name] = value.detach() if totals[name] is None else totals[name] + value.detach()

        if self._last:
            if not torch.is_tensor(runtime.state.loss):
                raise TypeError("last PP stage must return a Tensor loss")
            st.raw_loss = runtime.state.loss
            if isinstance(out, LossOutput) and out.auxiliary_loss is not None:
                st.auxiliary_loss = out.auxiliary_loss
                _add("aux", out.auxiliary_loss)
            _add("loss", runtime.state.loss)
            return
        if isinstance(out, PipelineOutput):
            act = cast_boundary_activation(out.activation, runtime)
            st.auxiliary_loss = out.auxiliary_loss
            _add("aux", out.auxiliary_loss)
        elif torch.is_tensor(out):
            act = cast_boundary_activation(out, runtime)
        else:
            raise TypeError("non-last PP stage must return Tensor or PipelineOutput activations")
        runtime.state.outputs = act
        st.output_activation = act
        st.pending_sends.append(self.send_activation_async(act.detach())[1])

    def _backward(self, runtime, st: PipelineMicroState, action: PipelineAction, m: int) -> None:
        ctx = runtime.state.step_context
        if action.backward_step_idx == 0:
            status = PpStatus.BACKWARD_START
        elif action.backward_step_idx == m - 1:
            status = PpStatus.BACKWARD_END
        else:
            status = PpStatus.BACKWARD_MIDDLE
        if m == 1:
            status = PpStatus.IDLE  # a single micro-batch both opens and closes the window
        ctx.set_pp_state(microbatch_idx=action.microbatch_idx, status=status)
        if self._last:
            runtime.state.loss = st.raw_loss / float(m)
            DefaultStepRunner.run_backward(runtime)
        else:
            runtime.state.outputs = st.output_activation
            grad, work = self.recv_grad_async(runtime, st.output_activation)
            work.wait()
            if st.auxiliary_loss is None:
                DefaultStepRunner.run_backward(runtime, grad_output=grad)
            else:
                aux_grad = torch.ones_like(st.auxiliary_loss) / (float(m) * ctx.loss_divisor)
                DefaultStepRunner.run_backward_many(runtime, [st.output_activation, st.auxiliary_loss], [grad, aux_grad])
        if not self._first:
            g = st.input_activation.grad
            if g is None:
                raise RuntimeError("pipeline stage input received no gradient")
            st.pending_sends.append(self.send_grad_async(g.detach())[1])
        st.output_activation = None
        st.raw_loss = None

    # ------------------------------------------------------------------ loss reporting
    def broadcast_loss(self, *, runtime, total_loss, total_auxiliary_loss, batch) -> torch.Tensor:
        with span("maltos::pp.broadcast_loss"):
            m = float(runtime.plan.pp_schedule.microbatches)
            device = model_device(runtime.model)
            group = self.plugin.pp_group if self.plugin.stage_count > 1 else None

            def _sum_over_stages(t: torch.Tensor) -> torch.Tensor:
                if group is not None:
                    all_reduce_tensor(t, op=dist.ReduceOp.SUM, group=group)
                return t

            zero = torch.zeros((), device=device, dtype=torch.float32)
            loss = _sum_over_stages(total_loss.float() / m if self._last else zero.clone())
            if total_auxiliary_loss is None:
                return loss
            stage_aux = total_auxiliary_loss.float() / m
            all_aux = _sum_over_stages(stage_aux.clone())
            tail_aux = _sum_over_stages(stage_aux.clone() if self._last else zero.clone())
            ce = loss - tail_aux
            total = ce + all_aux
            coef = getattr(runtime.model, "moe_aux_loss_coef", 0.0)
            runtime.state.metadata["model_metrics"] = {
                "loss/ce": float(ce.item()),
                "moe/load_balance_loss": float((all_aux / coef).item()) if coef > 0 else 0.0,
                "loss/total": float(total.item()),
            }
            return total

    # ------------------------------------------------------------------ p2p
    def recv_activation_async(self, runtime, batch):
        mb = runtime.state.step_context.pp_cur_microbatch_idx
        shape = activation_shape(batch, self.plugin.hidden_size, sequence_parallel_world_size=self.plugin.sequence_parallel_world_size,
                                 context_parallel_world_size=getattr(self.plugin, "context_parallel_world_size", 1))
        buf = acquire_buffer(shape=shape, dtype=activation_dtype(runtime), device=model_device(runtime.model),
                             policy=BufferPolicy.PINNED, key=f"pp.recv_activation.mb{mb}").tensor.detach()
        buf.grad = None
        buf.requires_grad_(False)
        return buf, irecv_tensor_async(buf, self.plugin.prev_global_rank, group=self.plugin.pp_group)

    def send_activation_async(self, tensor: torch.Tensor):
        buf = tensor.contiguous()
        return buf, isend_tensor_async(buf, self.plugin.next_global_rank, group=self.plugin.pp_group)

    def recv_grad_async(self, runtime, output_activation: torch.Tensor):
        mb = runtime.state.step_context.pp_cur_microbatch_idx
        buf = acquire_buffer(shape=tuple(output_activation.shape), dtype=output_activation.dtype, device=output_activation.device,
                             policy=BufferPolicy.PINNED, key=f"pp.recv_grad.mb{mb}").tensor
        return buf, irecv_tensor_async(buf, self.plugin.next_global_rank, group=self.plugin.pp_group)

    def send_grad_async(self, tensor: torch.Tensor):
        buf = tensor.contiguous()
        return buf, isend_tensor_async(buf, self.plugin.prev_global_rank, group=self.plugin.pp_group)


# ---------------------------------------------------------------------- batch helpers
def batch_size(batch) -> int:
    first = batch.get(INPUT_IDS_KEY) if isinstance(batch, dict) else (batch[0] if isinstance(batch, (tuple, list)) and batch else batch)
    if torch.is_tensor(first):
        return int(first.size(0))
    raise TypeError(f"unsupported PP batch type={type(batch).__name__}")


def slice_batch(batch, start: int, length: int):
    def cut(v):
        if torch.is_tensor(v) and v.dim() >= 1 and v.size(0) >= start + length:
            return v.narrow(0, start, length).contiguous()
        return v

    if isinstance(batch, dict):
        return {k: cut(v) for k, v in batch.items()}
    if isinstance(batch, tuple):
        return tuple(cut(v) for v in batch)
    if isinstance(batch, list):
        return [cut(v) for v in batch]
    if torch.is_tensor(batch):
        return cut(batch)
    raise TypeError(f"unsupported PP batch type={type(batch).__name__}")


def split_batch(batch, num_microbatches: int) -> list:
    if num_microbatches == 1:
        return [batch]
    n = batch_size(batch)
    if n % num_microbatches:
        raise ValueError(f"pipeline microbatch split requires batch size divisible by microbatches, got batch_size={n}, microbatches={num_microbatches}")
    per = n // num_microbatches
    pieces = [slice_batch(batch, i * per, per) for i in range(num_microbatches)]
    if isinstance(batch, dict) and torch.is_tensor(batch.get(LOSS_TARGET_COUNTS_KEY)):
        # context-parallel loss weight of each piece from ITS rows (the batch-wide fraction is only right on average)
        from maltos_b200.parallel.context_batch import target_fraction

        for piece in pieces:
            piece[LOSS_WEIGHT_KEY] = target_fraction(piece[LOSS_TARGET_COUNTS_KEY])
    if isinstance(batch, dict) and torch.is_tensor(batch.get(LOSS_SCALE_KEY)) and torch.is_tensor(batch.get("loss_row_targets")):
        # token-weighted loss: a piece weighs by ITS targets (the runner averages the pieces): batch scale x piece / mean piece
        whole = batch["loss_row_targets"].sum().clamp_min(1.0)
        for piece in pieces:
            piece[LOSS_SCALE_KEY] = batch[LOSS_SCALE_KEY] * piece["loss_row_targets"].sum() * float(num_microbatches) / whole
    return pieces


def unpack_batch(batch):
    if isinstance(batch, dict):
        return batch[INPUT_IDS_KEY], batch.get(LABELS_KEY)
    if isinstance(batch, (tuple, list)):
        if len(batch) != 2:
            raise ValueError(f"expected (input_ids, labels) batch tuple, got len={len(batch)}")
        return batch[0], batch[1]
    if torch.is_tensor(batch):
        return batch, None
    raise TypeError(f"unsupported PP batch type={type(batch).__name__}")


def extract_labels(batch):
    return unpack_batch(batch)[1]


def activation_shape(batch, hidden_size: int, *, sequence_parallel_world_size: int = 1, context_parallel_world_size: int = 1):
    ids, _ = unpack_batch(batch)
    seq = int(ids.size(1))
    if sequence_parallel_world_size > 1:
        if seq % sequence_parallel_world_size:
            raise ValueError(f"PP+SP activation shape requires sequence length divisible by tp world size, got seq_len={seq}, tp={sequence_parallel_world_size}")
        seq //= sequence_parallel_world_size
    return int(ids.size(0)), seq, hidden_size


def model_device(model: nn.Module) -> torch.device:
    p = next(model.parameters(), None)
    if p is None:
        raise ValueError("PP model must have parameters")
    return p.device


def activation_dtype(runtime) -> torch.dtype:
    if runtime.dtype is not None:
        return runtime.dtype
    return next(runtime.model.parameters()).dtype


def cast_boundary_activation(tensor: torch.Tensor, runtime) -> torch.Tensor:
    want = activation_dtype(runtime)
    return tensor if tensor.dtype == want else tensor.to(want)
