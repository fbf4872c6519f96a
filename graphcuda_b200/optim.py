"""Single-launch optimizers for the training scripts' ``optimizer.step()``
(reference tests/gcn/graphcuda_impl.py:45,56).

``FusedAdam`` follows ``torch.optim.Adam`` (amsgrad / maximize off) and
``FusedSGD`` the momentum-free ``torch.optim.SGD`` the reference's script
builds; both update every parameter of the model with one kernel
(``gc_adam_step_f32`` / ``gc_sgd_step_f32``).  The Adam step count lives on the
device, so ``step()`` can be recorded in a CUDA graph and replayed
(graphed.GraphedTrainStep); ``lr`` is read on the host when the launch is
issued -- or recorded -- so change it between captures, not between replays.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .ops import _stream

_MAX = 32  # tensors per launch (kMaxTensors in csrc/optim.cu)


def _ptr_array(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _check_param(p: torch.Tensor) -> None:
    if not (p.is_cuda and p.dtype == torch.float32 and p.is_contiguous()):
        raise RuntimeError("fused optimizers need contiguous float32 CUDA parameters")


def _grads_of(params):
    out = []
    for p in params:
        g = p.grad
        if g.is_sparse or g.dtype != torch.float32 or g.device != p.device:
            raise RuntimeError("fused optimizers need dense float32 gradients on the parameter's device")
        out.append(g if g.is_contiguous() else g.contiguous())
    return out


class FusedAdam(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("FusedAdam: invalid hyper-parameter")
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay))

    def _group_state(self, group, device, chunk):
        key = f"_gc_state_{device.index}_{chunk}"
        if key not in group:
            # [steps taken, CTA arrival counter]; zero before the first step
            group[key] = torch.zeros(2, dtype=torch.int64, device=device)
        return group[key]

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        L = _lib.lib()
        for group in self.param_groups:
            by_device = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                _check_param(p)
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                by_device.setdefault(p.device, []).append(p)
            for dev, all_ps in by_device.items():
                # one launch per 32 tensors; every launch keeps its own step count
                for chunk, i in enumerate(range(0, len(all_ps), _MAX)):
                    ps = all_ps[i:i + _MAX]
                    grads = _grads_of(ps)
                    ms = [self.state[p]["exp_avg"] for p in ps]
                    vs = [self.state[p]["exp_avg_sq"] for p in ps]
                    sizes = (C.c_int64 * len(ps))(*[p.numel() for p in ps])
                    with torch.cuda.device(dev):
                        rc = L.gc_adam_step_f32(len(ps), _ptr_array(ps), _ptr_array(grads), _ptr_array(ms),
                                                _ptr_array(vs), sizes, group["lr"], group["betas"][0],
                                                group["betas"][1], group["eps"], group["weight_decay"],
                                                self._group_state(group, dev, chunk).data_ptr(), _stream(dev))
                    _lib.check(rc, "gc_adam_step_f32")
        return loss

    def steps_taken(self) -> int:
        """Reads the device step count of the first group back (synchronises)."""
        for group in self.param_groups:
            for k, v in group.items():
                if k.startswith("_gc_state_"):
                    return int(v[0].item())
        return 0


class FusedSGD(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, weight_decay: float = 0.0):
        if lr < 0 or weight_decay < 0:
            raise ValueError("FusedSGD: invalid hyper-parameter")
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        L = _lib.lib()
        for group in self.param_groups:
            by_device = {}
            for p in group["params"]:
                if p.grad is not None:
                    _check_param(p)
                    by_device.setdefault(p.device, []).append(p)
            for dev, ps in by_device.items():
                for i in range(0, len(ps), _MAX):
                    chunk = ps[i:i + _MAX]
                    grads = _grads_of(chunk)
                    sizes = (C.c_int64 * len(chunk))(*[p.numel() for p in chunk])
                    with torch.cuda.device(dev):
                        rc = L.gc_sgd_step_f32(len(chunk), _ptr_array(chunk), _ptr_array(grads), sizes, group["lr"],
                                               group["weight_decay"], _stream(dev))
                    _lib.check(rc, "gc_sgd_step_f32")
        return loss
