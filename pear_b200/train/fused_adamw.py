"""AdamW whose update is one kernel pass per parameter tensor (``ops/csrc/optim_collective.cu: adamw_local_kernel``).

State layout and hyper-parameters are those of ``torch.optim.AdamW`` (``step``, ``exp_avg``, ``exp_avg_sq`` per parameter;
decoupled weight decay), so optimizer state dicts move between the two. fp32 parameters on a GPU take the kernel; anything
else (CPU tensors, other dtypes, non-contiguous tensors) takes the same statements in torch. ``grad_scale`` lets the
caller fold the clip coefficient into the pass instead of rescaling the gradients first. (Upstream steps the FSDP shards
with ``_multi_tensor_adam``: pear/trainer/engine.py:236.)
"""

from __future__ import annotations

import ctypes

import torch


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            lr, eps, wd = float(group["lr"]), float(group["eps"]), float(group["weight_decay"])
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = torch.zeros((), dtype=torch.float32)
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["step"] += 1
                t = float(st["step"])
                bias1, bias2 = 1.0 - b1 ** t, 1.0 - b2 ** t
                g, m, v = p.grad, st["exp_avg"], st["exp_avg_sq"]
                if (p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and g.is_contiguous() and m.is_contiguous()
                        and v.is_contiguous() and g.dtype in (torch.float32, torch.bfloat16)):
                    from ..ops import lib as _lib

                    f = ctypes.c_float
                    _lib.check(_lib.lib().pear_adamw_local(_lib.ptr(p), _lib.ptr(g), 1 if g.dtype == torch.bfloat16 else 0, _lib.ptr(m),
                                                           _lib.ptr(v), ctypes.c_size_t(p.numel()), f(lr), f(b1), f(b2), f(eps), f(wd), f(bias1),
                                                           f(bias2), f(grad_scale), _lib.stream()), "adamw_local")
                    _lib.count_launch()
                else:
                    gf = g.to(m.dtype) * grad_scale
                    m.mul_(b1).add_(gf, alpha=1.0 - b1)
                    v.mul_(b2).addcmul_(gf, gf, value=1.0 - b2)
                    p.mul_(1.0 - lr * wd).addcdiv_(m, v.sqrt().div_(bias2 ** 0.5).add_(eps), value=-lr / bias1)
        return loss
