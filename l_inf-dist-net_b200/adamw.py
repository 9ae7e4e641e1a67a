"""AdamW whose weight decay follows the l_p norm of each weight ROW (semantics of adamw.py:6-86
of zbh2047/L_inf-dist-net): before the Adam update a row x of a distance layer shrinks along
the gradient of ||x||_p, i.e. x_i -= lr*wd * (|x_i| / ||x||_p)^(p-2) * x_i; at p = inf only the
entry of largest magnitude shrinks; parameters of modules without a p shrink uniformly."""
import math

import torch
from torch.optim import Optimizer

from . import _lib
from .norm_dist import get_p_norm


class AdamW(Optimizer):
    def __init__(self, model, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        if lr < 0 or eps < 0 or weight_decay < 0:
            raise ValueError("lr, eps and weight_decay must be non-negative")
        if not (0 <= betas[0] < 1 and 0 <= betas[1] < 1):
            raise ValueError("betas must lie in [0, 1)")
        groups = [{"params": p, "module": m} for m in model.modules() for p in m.parameters(False)]
        super().__init__(groups, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @staticmethod
    def _fused_ok(p):
        return (p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and p.grad.is_contiguous()
                and p.grad.dtype == torch.float32 and p.dim() >= 1 and p.numel() > 0
                and p.numel() // p.size(0) <= 51200)

    @staticmethod
    def _decay(p, p_norm, lr_wd, eps):
        if p_norm is None:
            p.mul_(1 - lr_wd)
            return
        rows = p.view(p.size(0), -1)
        if math.isinf(p_norm):
            idx = rows.abs().argmax(dim=1, keepdim=True)
            rows.scatter_add_(1, idx, -lr_wd * rows.gather(1, idx))
            return
        sq = rows * rows + eps
        sq = sq / sq.amax(dim=1, keepdim=True)
        pw = sq.pow(p_norm / 2 - 1)
        scale = (sq * pw).sum(dim=1, keepdim=True).pow(2 / p_norm - 1) * pw
        p.addcmul_(scale.view_as(p), p, value=-lr_wd)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    self._update(p, group)
        return loss

    @torch.no_grad()
    def step_params(self, params):
        """Updates only the given parameters (each at most once per call).  Lets a data-parallel
        driver run the optimiser for one gradient bucket as soon as that bucket is reduced, while
        the remaining buckets are still in flight."""
        if not hasattr(self, "_group_of"):
            self._group_of = {id(q): g for g in self.param_groups for q in g["params"]}
        for p in params:
            if p.grad is not None:
                self._update(p, self._group_of[id(p)])

    @torch.no_grad()
    def step_rows(self, p, row0, nrows, grad_rows):
        """Updates rows [row0, row0 + nrows) of the CUDA parameter `p` from `grad_rows` (their
        gradient, [nrows, cols], contiguous).  The moment estimates of these rows live in tensors of
        their own, so a data-parallel driver that shards the optimiser keeps only its share of the
        state.  The row-wise decay rule makes whole rows the natural shard."""
        if not hasattr(self, "_group_of"):
            self._group_of = {id(q): g for g in self.param_groups for q in g["params"]}
        group = self._group_of[id(p)]
        beta1, beta2 = group["betas"]
        state = self.state[p]
        key = ("rows", row0, nrows)
        if key not in state:
            state[key] = {"step": 0, "exp_avg": torch.zeros_like(grad_rows), "exp_avg_sq": torch.zeros_like(grad_rows)}
        st = state[key]
        st["step"] += 1
        p_norm = get_p_norm(group["module"])
        cols = p.numel() // p.size(0)
        if not (p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and grad_rows.is_contiguous()
                and grad_rows.dtype == torch.float32 and cols <= 51200):
            raise RuntimeError("step_rows needs a contiguous fp32 CUDA parameter with rows of at most 51200 entries")
        with torch.cuda.device(p.device):
            rc = _lib.load().linf_adamw_step(
                p.data_ptr() + row0 * cols * 4, grad_rows.data_ptr(), st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(),
                nrows, cols, -1.0 if p_norm is None else float(p_norm), group["lr"], beta1, beta2,
                group["eps"], group["weight_decay"], st["step"], torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "adamw_step")

    def _update(self, p, group):
        if p.grad.is_sparse:
            raise RuntimeError("AdamW does not support sparse gradients")
        beta1, beta2 = group["betas"]
        state = self.state[p]
        if not state:
            state["step"] = 0
            state["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        state["step"] += 1
        p_norm = get_p_norm(group["module"])
        if self._fused_ok(p):
            # CUDA tensors: one fused launch per tensor (csrc/adamw.cu)
            rows = p.size(0)
            with torch.cuda.device(p.device):
                rc = _lib.load().linf_adamw_step(
                    p.data_ptr(), p.grad.data_ptr(), state["exp_avg"].data_ptr(), state["exp_avg_sq"].data_ptr(),
                    rows, p.numel() // rows, -1.0 if p_norm is None else float(p_norm), group["lr"], beta1, beta2,
                    group["eps"], group["weight_decay"], state["step"], torch.cuda.current_stream().cuda_stream)
            _lib.check(rc, "adamw_step")
            return
        self._decay(p, p_norm, group["lr"] * group["weight_decay"], group["eps"])
        m, v = state["exp_avg"], state["exp_avg_sq"]
        m.mul_(beta1).add_(p.grad, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(p.grad, p.grad, value=1 - beta2)
        denom = (v.sqrt() / math.sqrt(1 - beta2 ** state["step"])).add_(group["eps"])
        p.addcdiv_(m, denom, value=-group["lr"] / (1 - beta1 ** state["step"]))
