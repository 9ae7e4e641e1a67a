"""Test-only stand-in for the CUDA distance operator: the CPU checker wrapped as an autograd
Function, so that the host-side modules (nets, bound modules, optimiser, DDP wiring) can be
exercised on a machine without a GPU.  Never imported by the package."""
import math

import numpy as np
import torch

import oracle


class OracleDistF(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, group, p, tag):
        xn, wn = x.detach().numpy(), weight.detach().numpy()
        if math.isinf(p):
            y, pos = oracle.inf_dist_forward(xn, wn, group)
            ctx.pos = pos
        else:
            y = oracle.norm_dist_forward(xn, wn, group, p)
        ctx.save_for_backward(x, weight, torch.from_numpy(y))
        ctx.group, ctx.p = group, p
        return torch.from_numpy(y)

    @staticmethod
    def backward(ctx, grad_output):
        x, weight, y = ctx.saved_tensors
        g = np.ascontiguousarray(grad_output.numpy())
        if math.isinf(ctx.p):
            gx, gw = oracle.inf_dist_backward(g, ctx.pos, x.size(1), ctx.group)
        else:
            gx, gw = oracle.norm_dist_backward(g, x.detach().numpy(), weight.detach().numpy(), y.numpy(), ctx.group, ctx.p)
        return torch.from_numpy(gx), torch.from_numpy(gw), None, None, None


def cpu_norm_dist(input, weight, group, p, use_custom_cuda_func=True, tag=None):
    return OracleDistF.apply(input.contiguous(), weight.contiguous(), group, p, tag)


def cpu_inf_dist_bound(lower, upper, weight, group, use_custom_cuda_func=True, tag=None):
    lo, up = oracle.inf_dist_bound(lower.detach().numpy(), upper.detach().numpy(), weight.detach().numpy(), group)
    return torch.from_numpy(lo), torch.from_numpy(up)


def patch(monkeypatch):
    """Routes the package's distance operator to the CPU checker for the duration of a test."""
    import importlib
    nd = importlib.import_module("linfdist_b200.norm_dist")
    monkeypatch.setattr(nd, "norm_dist", cpu_norm_dist)
    monkeypatch.setattr(nd, "inf_dist_bound", cpu_inf_dist_bound)
