"""Optimizers of the runtime.

``FusedAdamW`` is ``torch.optim.AdamW`` (same constructor, same ``state_dict`` layout:
``state{idx:{step,exp_avg,exp_avg_sq}}, param_groups``) whose ``step`` is ONE launch of the multi-tensor sm_100a
kernel in ``csrc/optim.cu`` on CUDA, and the plain PyTorch math on CPU.

``MasterWeightsOptimizer`` keeps the model parameters in bf16/fp16 and fp32 master copies inside the inner
optimizer (interface of the reference's ``runtime/optim.py:10-104``: ``copy_master_params``, ``step``,
``sync_master_params_from_model``, ``state_dict = {inner_optimizer, master_params, master_dtype}``). When the
inner optimizer is a ``FusedAdamW`` on CUDA, low-precision grads are consumed directly by the fused kernel
(grad cast, optional clip coefficient read from device memory, AdamW on the fp32 master, bf16 write-back), so no
fp32 copy of the gradients is ever materialised.
"""
from __future__ import annotations

from typing import Any, Iterable

import torch
import torch.nn as nn


class FusedAdamW(torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, **kwargs) -> None:
        kwargs.pop("fused", None)
        kwargs.pop("foreach", None)
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, foreach=False, fused=False, **kwargs)
        #: optional device scalar multiplied into every gradient inside the kernel (global-norm clip coefficient)
        self.grad_scale: torch.Tensor | None = None
        #: optional {id(master_param): low-precision model param} written back by the kernel
        self.low_precision_params: dict[int, torch.Tensor] = {}
        #: optional {id(master_param): tensor} gradients to use instead of ``param.grad`` (e.g. bf16 model grads)
        self.external_grads: dict[int, torch.Tensor] = {}
        #: optional {id(master_param): callable -> device addresses}: the updated values of that parameter are stored as
        #: bf16 at every address (peers' flat parameter buffers over NVLink) by the same kernel that does the update
        self.push_destinations: dict[int, object] = {}

    def _state_for(self, p: torch.Tensor) -> dict:
        st = self.state[p]
        if len(st) == 0:
            st["step"] = torch.tensor(0.0, dtype=torch.float32)
            st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return st

    def load_state_dict(self, state_dict) -> None:
        super().load_state_dict(state_dict)
        # Checkpoints written with torch's fused AdamW keep `step` on the device; this class counts on the host.
        for st in self.state.values():
            if torch.is_tensor(st.get("step")):
                st["step"] = st["step"].detach().to(device="cpu", dtype=torch.float32)
        for group in self.param_groups:
            group["fused"] = False
            group["foreach"] = False

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        from maltos_b200.ops.optim import adamw_multi_tensor

        for group in self.param_groups:
            if group.get("amsgrad") or group.get("maximize"):
                raise NotImplementedError("FusedAdamW supports neither amsgrad nor maximize")
            beta1, beta2 = group["betas"]
            items, pushed = [], []
            for p in group["params"]:
                g = self.external_grads.get(id(p), p.grad)
                if g is None:
                    continue
                st = self._state_for(p)
                st["step"] += 1
                destinations = self.push_destinations.get(id(p)) if p.is_cuda else None
                if destinations is not None:
                    pushed.append((p, g, st, destinations))
                else:
                    items.append((p, g, st["exp_avg"], st["exp_avg_sq"], self.low_precision_params.get(id(p)), float(st["step"])))
            lr = group["lr"]
            lr = float(lr) if not torch.is_tensor(lr) else float(lr.item())
            if items:
                adamw_multi_tensor(items, lr=lr, beta1=beta1, beta2=beta2, eps=group["eps"],
                                   weight_decay=group["weight_decay"], grad_scale=self.grad_scale)
            if pushed:
                from maltos_b200.ops.zero_fused import adamw_push

                for p, g, st, destinations in pushed:
                    adamw_push(p.data, g.contiguous(), st["exp_avg"], st["exp_avg_sq"], destinations(), step=float(st["step"]), lr=lr,
                               beta1=beta1, beta2=beta2, eps=group["eps"], weight_decay=group["weight_decay"], grad_scale=self.grad_scale)
        return loss


class MasterWeightsOptimizer(torch.optim.Optimizer):
    def __init__(self, params: Iterable[nn.Parameter], *, optimizer_factory, master_dtype: torch.dtype = torch.float32) -> None:
        self.model_params = [p for p in params if p.requires_grad]
        if not self.model_params:
            raise ValueError("MasterWeightsOptimizer requires at least one trainable parameter")
        self.master_dtype = master_dtype
        self.master_params = [nn.Parameter(p.detach().to(master_dtype), requires_grad=True) for p in self.model_params]
        self._model_by_master = {id(m): p for p, m in zip(self.model_params, self.master_params)}
        super().__init__(self.master_params, defaults={})
        self._optimizer = optimizer_factory(self.master_params)
        self._adopt_inner()
        self._master_grads_copied = False
        self._fused = isinstance(self._optimizer, FusedAdamW)
        # fp16 runs go through a GradScaler, which unscales and inf-checks `.grad` of the optimizer's own (master)
        # parameters: there the fp32 master-gradient copies are kept and the fused kernel consumes those.
        self._direct_grads = self._fused and self.model_params[0].dtype == torch.bfloat16
        if self._direct_grads:
            self._optimizer.low_precision_params = {id(m): p for p, m in zip(self.model_params, self.master_params)}

    def _adopt_inner(self) -> None:
        self.param_groups = self._optimizer.param_groups
        self.defaults = self._optimizer.defaults
        self.state = self._optimizer.state

    @property
    def inner(self) -> torch.optim.Optimizer:
        return self._optimizer

    def model_param_for(self, param: nn.Parameter) -> nn.Parameter:
        return self._model_by_master.get(id(param), param)

    def _fused_on_device(self) -> bool:
        return self._direct_grads and self.model_params[0].is_cuda

    def copy_master_params(self) -> None:
        """Make the model gradients visible to the inner optimizer (fp32 copies, or by reference when fused)."""
        if self._master_grads_copied:
            return
        if self._fused_on_device():
            self._optimizer.external_grads = {id(m): p.grad for p, m in zip(self.model_params, self.master_params) if p.grad is not None}
        else:
            for p, m in zip(self.model_params, self.master_params):
                if p.grad is None:
                    m.grad = None
                elif m.grad is None:
                    m.grad = p.grad.detach().to(device=m.device, dtype=m.dtype)
                else:
                    m.grad.copy_(p.grad.detach())
        self._master_grads_copied = True

    def grads_for_clipping(self) -> list[tuple[nn.Parameter, torch.Tensor]]:
        """(model param, gradient tensor the optimizer will consume) pairs, for norm computation / scaling."""
        self.copy_master_params()
        out = []
        for p, m in zip(self.model_params, self.master_params):
            g = self._optimizer.external_grads.get(id(m)) if self._fused_on_device() else m.grad
            if g is not None:
                out.append((p, g))
        return out

    def sync_master_params_from_model(self) -> None:
        with torch.no_grad():
            for p, m in zip(self.model_params, self.master_params):
                m.copy_(p.detach())
        self._master_grads_copied = False

    def step(self, closure=None):
        self.copy_master_params()
        loss = self._optimizer.step(closure)
        if not self._fused_on_device():
            with torch.no_grad():
                for p, m in zip(self.model_params, self.master_params):
                    p.copy_(m)
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        self._optimizer.zero_grad(set_to_none=set_to_none)
        if self._fused:
            self._optimizer.external_grads = {}
        for p in self.model_params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()
        self._master_grads_copied = False

    def state_dict(self) -> dict[str, Any]:
        return {
            "inner_optimizer": self._optimizer.state_dict(),
            "master_params": [m.detach().cpu().clone() for m in self.master_params],
            "master_dtype": str(self.master_dtype),
        }

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self._optimizer.load_state_dict(state_dict.get("inner_optimizer", state_dict))
        self._adopt_inner()
        saved = state_dict.get("master_params")
        if isinstance(saved, list):
            if len(saved) != len(self.master_params):
                raise ValueError(f"master_params length mismatch: checkpoint={len(saved)}, optimizer={len(self.master_params)}")
            for m, s in zip(self.master_params, saved):
                if not torch.is_tensor(s):
                    raise TypeError("master_params entries must be tensors")
                m.data.copy_(s)
        with torch.no_grad():
            for p, m in zip(self.model_params, self.master_params):
                p.copy_(m)
        self._master_grads_copied = False
