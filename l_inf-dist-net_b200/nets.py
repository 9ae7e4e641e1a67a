"""The two MLP assemblies of distance layers and the feature/predictor wrapper that the
training and certification paths run (shapes of model/mlp.py:5-39 and model/model.py:3-27 of
zbh2047/L_inf-dist-net).  `width` counts units of 1024 neurons."""
import math

import torch.nn as nn

from .norm_dist import NormDist

UNIT = 1024


def _flat(t):
    return None if t is None else t.reshape(t.size(0), -1)


def _numel(dim):
    return int(math.prod(dim)) if hasattr(dim, "__iter__") else int(dim)


class MLPFeature(nn.Module):
    """`depth` mean-normalised distance layers of `width`*1024 neurons, no bias."""

    def __init__(self, depth, width, input_dim):
        super().__init__()
        dims = [_numel(input_dim)] + [UNIT * width] * depth
        self.fc = nn.ModuleList(NormDist(a, b, bias=False, mean_normalize=True) for a, b in zip(dims, dims[1:]))
        self.out_features = dims[-1]

    def forward(self, x, lower=None, upper=None):
        t = (_flat(x), _flat(lower), _flat(upper))
        for layer in self.fc:
            t = layer(*t)
        return t


class MLP(nn.Module):
    """depth-1 hidden distance layers and a biased distance layer onto the classes.  A small
    distance means "close to the class", so the output is negated (and the bounds swap)."""

    def __init__(self, depth, width, input_dim, num_classes=10):
        super().__init__()
        dims = [_numel(input_dim)] + [UNIT * width] * (depth - 1)
        self.fc = nn.ModuleList(NormDist(a, b, bias=False, mean_normalize=True) for a, b in zip(dims, dims[1:]))
        self.fc_last = NormDist(dims[-1], num_classes, bias=True, mean_normalize=False)

    def forward(self, x, lower=None, upper=None):
        t = (_flat(x), _flat(lower), _flat(upper))
        for layer in self.fc:
            t = layer(*t)
        # negated layer: the value changes sign, the bounds change sign and places (model/mlp.py:22)
        return list(self.fc_last(*t, negate=True))


class Model(nn.Module):
    """feature -> predictor.  Without propagated bounds (training) the feature output gets the
    box [x - eps, x + eps]: a distance net is 1-Lipschitz in the sup norm."""

    def __init__(self, feature, predictor, eps):
        super().__init__()
        self.feature, self.predictor, self.eps = feature, predictor, eps

    def forward(self, x, lower=None, upper=None, targets=None):
        if targets is None:
            lower = upper = None
        if self.feature is not None:
            x, lower, upper = self.feature(x, lower=lower, upper=upper)
        if targets is not None and (lower is None or upper is None):
            lower, upper = x - self.eps, x + self.eps
        return self.predictor(x, lower, upper, targets=targets)


def set_eps(model, eps):
    for m in model.modules():
        if isinstance(m, Model):
            m.eps = eps


def get_eps(model):
    for m in model.modules():
        if isinstance(m, Model):
            return m.eps
    return None
