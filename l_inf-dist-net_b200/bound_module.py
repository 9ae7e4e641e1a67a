"""Interval-bound modules that follow the distance layers: every module maps a triple
(value, lower, upper) and the final ones turn bounds into worst-case margins.

API mirror of model/bound_module.py of zbh2047/L_inf-dist-net (BoundReLU :5-12, BoundTanh
:14-21, BoundLinear :28-46, BoundFinalLinear :48-68, BoundMeanNorm :70-93, BoundFinalIdentity
:95-103, Predictor :105-116).  These are small dense GEMMs and elementwise maps; they run on
stock torch ops (cuBLAS), not on custom kernels.
"""
import math

import torch
import torch.nn as nn

from .norm_dist import MeanNorm


class _BoundMonotone(nn.Module):
    """A non-decreasing elementwise map applies to value, lower and upper alike."""
    fn = None

    def forward(self, x, lower=None, upper=None):
        f = type(self).fn
        if lower is None or upper is None:
            return f(x), None, None
        return f(x), f(lower), f(upper)


class BoundReLU(_BoundMonotone):
    fn = staticmethod(torch.relu)


class BoundTanh(_BoundMonotone):
    fn = staticmethod(torch.tanh)


def _affine(x, weight, bias, w_scale, b_scale):
    out = torch.mm(x, weight.t()) * w_scale
    return out if bias is None else out + bias * b_scale


class BoundLinear(nn.Linear):
    """y = (w_scale / sqrt(in)) * x W^T + b_scale * b, with centre/radius interval arithmetic."""

    def __init__(self, in_features, out_features, bias=True, w_scale=1.0, b_scale=1.0):
        super().__init__(in_features, out_features, bias=bias)
        nn.init.normal_(self.weight)
        if self.bias is not None:
            nn.init.zeros_(self.bias)
        self.w_scale = w_scale / math.sqrt(in_features)
        self.b_scale = b_scale

    def forward(self, x, lower=None, upper=None):
        y = _affine(x, self.weight, self.bias, self.w_scale, self.b_scale)
        if lower is None or upper is None:
            return y, None, None
        half = self.w_scale / 2
        centre = _affine(lower + upper, self.weight, self.bias, half, self.b_scale)
        radius = torch.mm(upper - lower, self.weight.abs().t()) * half
        return y, centre - radius, centre + radius


class BoundFinalLinear(nn.Linear):
    """Last affine layer.  With targets it also returns, per sample, the worst case of
    logit_j - logit_target over the input box (row j; the target row is 0)."""

    def __init__(self, in_features, out_features, bias=True, w_scale=1.0, b_scale=1.0):
        super().__init__(in_features, out_features, bias=bias)
        nn.init.normal_(self.weight)
        nn.init.zeros_(self.bias)
        self.w_scale = w_scale / math.sqrt(in_features)
        self.b_scale = b_scale

    def forward(self, x, lower=None, upper=None, targets=None):
        y = _affine(x, self.weight, self.bias, self.w_scale, self.b_scale)
        if lower is None or upper is None or targets is None:
            return y
        half = self.w_scale / 2
        dw = self.weight.unsqueeze(0) - self.weight[targets].unsqueeze(1)          # [B, CO, CI]
        worst = torch.bmm(dw, (lower + upper).unsqueeze(-1)) * half
        if self.bias is not None:
            worst = worst + ((self.bias.unsqueeze(0) - self.bias[targets].unsqueeze(1)) * self.b_scale).unsqueeze(-1)
        worst = worst + torch.bmm(dw.abs(), (upper - lower).unsqueeze(-1)) * half
        return y, worst.squeeze(-1)


class BoundMeanNorm(MeanNorm):
    """MeanNorm on a triple: statistics come from the interval centre when training."""

    def forward(self, x, lower=None, upper=None):
        z = super().forward(x)
        if lower is None or upper is None:
            return z, None, None
        if self.training:
            mid = (lower + upper) / 2
            flat = mid.reshape(mid.size(0), mid.size(1), -1)
            mean = flat.mean(dim=-1).mean(dim=0) if mid.dim() > 2 else mid.mean(dim=0)
            with torch.no_grad():
                self.running_mean.mul_(1 - self.momentum).add_(mean, alpha=self.momentum)
        else:
            mean = self.running_mean
        shape = [1, -1] + [1] * (lower.dim() - 2)
        return z, lower - mean.view(shape), upper - mean.view(shape)


class BoundFinalIdentity(nn.Module):
    """For nets whose last distance layer already produces the logits: the worst-case margin
    of class j against the target is upper_j - lower_target (0 in the target column)."""

    def forward(self, x, lower=None, upper=None, targets=None):
        if lower is None or upper is None or targets is None:
            return x
        col = targets.unsqueeze(-1)
        worst = (upper - lower.gather(1, col)).scatter(1, col, 0.0)
        return x, worst


class Predictor(nn.Module):
    """BoundLinear -> tanh -> BoundFinalLinear head used by the '++' nets."""

    def __init__(self, in_features, hidden, out_dim):
        super().__init__()
        self.fc1 = BoundLinear(in_features, hidden, bias=True)
        self.tanh = BoundTanh()
        self.fc2 = BoundFinalLinear(hidden, out_dim)

    def forward(self, x, lower=None, upper=None, targets=None):
        triple = self.tanh(*self.fc1(x, lower, upper))
        return self.fc2(*triple, targets=targets)
