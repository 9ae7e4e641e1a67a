"""L_p / L_inf-distance neuron for NVIDIA B200 (sm_100a).

Drop-in for the `norm_dist_cpp` path of zbh2047/L_inf-dist-net: the same Python surface
(`DistF`, `norm_dist`, `inf_dist_bound`, `MeanNorm`, `NormDistConv`, `NormDist`,
`set_p_norm`, `get_p_norm`, the `Bound*` interval modules) on top of a C-ABI CUDA library
(`liblinfdist.so`, header `include/linfdist.h`).  There is no CPU implementation and no
PyTorch fallback: without the built library every operator raises.
"""
from . import _lib
from .norm_dist import (DistF, MeanNorm, NormDist, NormDistConv, get_p_norm, inf_dist_bound,
                        norm_dist, set_backward_mode, get_backward_mode, set_p_norm,
                        inf_dist_post, set_fused_epilogue, get_fused_epilogue)
from .bound_module import (BoundFinalIdentity, BoundFinalLinear, BoundLinear, BoundMeanNorm,
                           BoundReLU, BoundTanh, Predictor)
from .nets import MLP, MLPFeature, Model, get_eps, set_eps
from .adamw import AdamW
from .certify import AttackPGD, certified_accuracy, certify

__all__ = [
    "DistF", "norm_dist", "inf_dist_bound", "MeanNorm", "NormDistConv", "NormDist",
    "set_p_norm", "get_p_norm", "set_backward_mode", "get_backward_mode",
    "inf_dist_post", "set_fused_epilogue", "get_fused_epilogue",
    "BoundReLU", "BoundTanh", "BoundLinear", "BoundFinalLinear", "BoundMeanNorm",
    "BoundFinalIdentity", "Predictor", "MLP", "MLPFeature", "Model", "set_eps", "get_eps",
    "AdamW", "certify", "certified_accuracy", "AttackPGD",
]
