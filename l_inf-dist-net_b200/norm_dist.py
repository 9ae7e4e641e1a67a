"""Host side of the distance neuron: the reference's Python surface on top of liblinfdist.so.

Mirrors model/norm_dist.py of zbh2047/L_inf-dist-net name for name:
    DistF (:7-47), norm_dist (:49-58), inf_dist_bound (:60-76), MeanNorm (:78-100),
    NormDistConv (:102-169), NormDist (:171-187), set_p_norm / get_p_norm (:189-198).
Differences a caller can observe:
  * `use_custom_cuda_func=False` (the reference's pure-PyTorch debugging branch) is refused:
    the CUDA library is the only implementation here;
  * p = inf gradients are produced in a fixed summation order by default ("ordered" mode, see
    set_backward_mode); the reference's atomicAdd order is undefined;
  * tensors are validated (CUDA, contiguous, float32) before the call, as the reference's
    binding does with TORCH_CHECK (model/norm_dist.cpp:3-5).
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib

_backward_mode = "ordered"
_workspaces = {}


def set_backward_mode(mode):
    """'ordered': deterministic scatter (ascending source order, bit-reproducible);
    'atomic': one fused pass with warp-aggregated fp32 atomics (order across warps undefined)."""
    global _backward_mode
    if mode not in ("ordered", "atomic"):
        raise ValueError("backward mode must be 'ordered' or 'atomic'")
    _backward_mode = mode


def get_backward_mode():
    return _backward_mode


def _require(t, name, dtype=torch.float32):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}")


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _workspace(device, nbytes):
    """Scratch buffer cached per (device, stream); grows, never shrinks."""
    key = (device.index, _stream())
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _shape5(x, weight, group):
    return x.size(0), weight.size(0), x.size(1), group, x.size(2)


def _rows_view(t):
    """[B, C, HW] -> contiguous [B*HW, C, 1]: every spatial position becomes a row of a dense layer."""
    B, C, HW = t.shape
    return t.permute(0, 2, 1).reshape(B * HW, C, 1).contiguous()


def _from_rows(t, B, HW):
    """Inverse of _rows_view for a [B*HW, C, 1] tensor."""
    return t.view(B, HW, t.size(1)).permute(0, 2, 1).contiguous()


def _dense_route(x, weight, group):
    """Conv-shaped calls (HW > 1) whose channel counts suit the tiled dense kernels are run as a
    dense layer over B*HW rows (two permuting copies around the kernels).  Results are the same:
    forward values, arg-max and bounds are per-row quantities, and the ordered weight gradient
    adds its contributions in ascending b*HW + hw order either way."""
    ci_g, co_g = weight.size(1), weight.size(0) // group
    return x.size(2) > 1 and ci_g % 4 == 0 and co_g >= 32


class DistF(torch.autograd.Function):
    """y[b,o,hw] = || x[b,g,:,hw] - weight[o,:] ||_p ; x [B,CI,HW], weight [CO,CI/group]."""

    @staticmethod
    def forward(ctx, x, weight, group, p, tag):
        lib = _lib.load()
        _require(x, "input"); _require(weight, "weight")
        if x.dim() != 3 or weight.dim() != 2:
            raise RuntimeError("input must be [B, CI, HW] and weight [CO, CI/group]")
        assert weight.size(1) * group == x.size(1)
        if not (math.isinf(p) or p > 1):
            raise NotImplementedError
        ctx.rows = _dense_route(x, weight, group)
        ctx.shape = (x.size(0), x.size(2))
        xk = _rows_view(x) if ctx.rows else x
        B, CO, CI, G, HW = _shape5(xk, weight, group)
        y = torch.empty(B, CO, HW, device=x.device, dtype=torch.float32)
        with torch.cuda.device(x.device):
            if math.isinf(p):
                pos = torch.empty(B, CO, HW, device=x.device, dtype=torch.int32)
                need = lib.linf_inf_dist_forward_workspace_bytes(B, CO, CI, G, HW)
                if need:
                    ws = _workspace(x.device, need)
                    rc = lib.linf_inf_dist_forward_ws(xk.data_ptr(), weight.data_ptr(), B, CO, CI, G, HW,
                                                      y.data_ptr(), pos.data_ptr(), ws.data_ptr(),
                                                      ws.numel(), _stream())
                else:
                    rc = lib.linf_inf_dist_forward(xk.data_ptr(), weight.data_ptr(), B, CO, CI, G, HW,
                                                   y.data_ptr(), pos.data_ptr(), _stream())
                _lib.check(rc, "inf_dist_forward")
                ctx.save_for_backward(xk, weight, y, pos)
            else:
                rc = lib.linf_norm_dist_forward(xk.data_ptr(), weight.data_ptr(), B, CO, CI, G, HW,
                                                y.data_ptr(), float(p), _stream())
                _lib.check(rc, "norm_dist_forward")
                ctx.save_for_backward(xk, weight, y)
        ctx.group, ctx.p, ctx.tag = group, p, tag
        return _from_rows(y, *ctx.shape) if ctx.rows else y

    @staticmethod
    def backward(ctx, grad_output):
        lib = _lib.load()
        grad_output = _rows_view(grad_output) if ctx.rows else grad_output.contiguous()
        _require(grad_output, "grad_output")
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gx = gw = None
        with torch.cuda.device(grad_output.device):
            if math.isinf(ctx.p):
                x, weight, y, pos = ctx.saved_tensors
                B, CO, CI, G, HW = _shape5(x, weight, ctx.group)
                if _backward_mode == "atomic":
                    if need_x:
                        gx = torch.zeros_like(x)
                    if need_w:
                        gw = torch.zeros_like(weight)
                    if need_x or need_w:
                        rc = lib.linf_inf_dist_backward_atomic(
                            grad_output.data_ptr(), pos.data_ptr(), B, CO, CI, G, HW,
                            gx.data_ptr() if need_x else None, gw.data_ptr() if need_w else None, _stream())
                        _lib.check(rc, "inf_dist_backward_atomic")
                elif need_x and need_w:
                    gx = torch.empty_like(x); gw = torch.empty_like(weight)
                    rc = lib.linf_inf_dist_backward(grad_output.data_ptr(), pos.data_ptr(), B, CO, CI, G, HW,
                                                    gx.data_ptr(), gw.data_ptr(), _stream())
                    _lib.check(rc, "inf_dist_backward")
                else:
                    if need_x:
                        gx = torch.empty_like(x)
                        rc = lib.linf_inf_dist_backward_input(grad_output.data_ptr(), pos.data_ptr(),
                                                              B, CO, CI, G, HW, gx.data_ptr(), _stream())
                        _lib.check(rc, "inf_dist_backward_input")
                    if need_w:
                        gw = torch.empty_like(weight)
                        rc = lib.linf_inf_dist_backward_weight(grad_output.data_ptr(), pos.data_ptr(),
                                                               B, CO, CI, G, HW, gw.data_ptr(), _stream())
                        _lib.check(rc, "inf_dist_backward_weight")
            else:
                x, weight, y = ctx.saved_tensors
                B, CO, CI, G, HW = _shape5(x, weight, ctx.group)
                if need_x:
                    gx = torch.empty_like(x)
                    rc = lib.linf_norm_dist_backward_input(
                        grad_output.data_ptr(), x.data_ptr(), weight.data_ptr(), y.data_ptr(),
                        B, CO, CI, G, HW, gx.data_ptr(), float(ctx.p), _stream())
                    _lib.check(rc, "norm_dist_backward_input")
                if need_w:
                    gw = torch.empty_like(weight)
                    rc = lib.linf_norm_dist_backward_weight(
                        grad_output.data_ptr(), x.data_ptr(), weight.data_ptr(), y.data_ptr(),
                        B, CO, CI, G, HW, gw.data_ptr(), float(ctx.p), _stream())
                    _lib.check(rc, "norm_dist_backward_weight")
        if ctx.rows and gx is not None:
            gx = _from_rows(gx, *ctx.shape)
        return gx, gw, None, None, None


def _no_torch_branch():
    raise RuntimeError("use_custom_cuda_func=False is not available: this package has no "
                       "PyTorch/CPU implementation of the distance neuron")


def norm_dist(input, weight, group, p, use_custom_cuda_func=True, tag=None):
    if not use_custom_cuda_func:
        _no_torch_branch()
    return DistF.apply(input, weight, group, p, tag)


def _post_args(post):
    """(sub, add, negate) -> the three C arguments; vectors must be contiguous fp32 CUDA tensors or None."""
    sub, add, negate = post if post is not None else (None, None, False)
    for v, name in ((sub, "sub"), (add, "add")):
        if v is not None:
            _require(v, name)
    return (sub.data_ptr() if sub is not None else None, add.data_ptr() if add is not None else None, 1 if negate else 0)


@torch.no_grad()
def inf_dist_post(input, weight, group, post, tag=None):
    """Value of an inf-dist layer with the per-channel epilogue (sub, add, negate) folded into the
    kernel's store: ((y - sub[c]) + add[c]), negated if asked.  No arg-max is kept, so there is no
    gradient: the inference / certification path.  input [B, CI, HW], weight [CO, CI/group]."""
    lib = _lib.load()
    _require(input, "input"); _require(weight, "weight")
    assert weight.size(1) * group == input.size(1)
    B, CO, CI, G, HW = _shape5(input, weight, group)
    y = torch.empty(B, CO, HW, device=input.device, dtype=torch.float32)
    sub, add, neg = _post_args(post)
    with torch.cuda.device(input.device):
        need = lib.linf_inf_dist_forward_workspace_bytes(B, CO, CI, G, HW)
        ws = _workspace(input.device, need) if need else None
        rc = lib.linf_inf_dist_forward_post(input.data_ptr(), weight.data_ptr(), B, CO, CI, G, HW, sub, add, neg,
                                            y.data_ptr(), ws.data_ptr() if need else None, ws.numel() if need else 0, _stream())
    _lib.check(rc, "inf_dist_forward_post")
    return y


def inf_dist_bound(input_lower, input_upper, weight, group, use_custom_cuda_func=True, tag=None, post=None):
    """Interval bounds of an inf-dist layer; returns (output_lower, output_upper), no gradient.
    post = (sub, add, negate) folds the per-channel epilogue into the kernel (see inf_dist_post); with
    negate the two outputs are also exchanged, so that lower <= upper still holds."""
    if not use_custom_cuda_func:
        _no_torch_branch()
    lib = _lib.load()
    _require(input_lower, "input_lower"); _require(input_upper, "input_upper"); _require(weight, "weight")
    assert weight.size(1) * group == input_lower.size(1) and input_upper.shape == input_lower.shape
    rows = _dense_route(input_lower, weight, group)
    if rows and post is not None:
        raise RuntimeError("the fused epilogue is available for dense layers (one spatial position) only")
    shape = (input_lower.size(0), input_lower.size(2))
    if rows:
        input_lower, input_upper = _rows_view(input_lower), _rows_view(input_upper)
    B, CO, CI, G, HW = _shape5(input_lower, weight, group)
    lo = torch.empty(B, CO, HW, device=input_lower.device, dtype=torch.float32)
    up = torch.empty_like(lo)
    with torch.cuda.device(input_lower.device):
        if post is None:
            rc = lib.linf_inf_dist_bound_forward(input_lower.data_ptr(), input_upper.data_ptr(), weight.data_ptr(),
                                                 B, CO, CI, G, HW, lo.data_ptr(), up.data_ptr(), _stream())
        else:
            sub, add, neg = _post_args(post)
            rc = lib.linf_inf_dist_bound_forward_post(input_lower.data_ptr(), input_upper.data_ptr(), weight.data_ptr(),
                                                      B, CO, CI, G, HW, sub, add, neg, lo.data_ptr(), up.data_ptr(), _stream())
    _lib.check(rc, "inf_dist_bound_forward")
    if rows:
        return _from_rows(lo, *shape), _from_rows(up, *shape)
    return lo, up


class MeanShiftF(torch.autograd.Function):
    """x[B, C] -> x - column mean(x), with the exponential running mean updated in the same launch
    (csrc/epilogue.cu).  The backward is the same map applied to the gradient."""

    @staticmethod
    def forward(ctx, x, running_mean, momentum):
        lib = _lib.load()
        _require(x, "input")
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            rc = lib.linf_mean_shift(x.data_ptr(), x.size(0), x.size(1),
                                     running_mean.data_ptr() if running_mean is not None else None,
                                     float(momentum), out.data_ptr(), None, _stream())
        _lib.check(rc, "mean_shift")
        return out

    @staticmethod
    def backward(ctx, grad_output):
        lib = _lib.load()
        g = grad_output.contiguous()
        out = torch.empty_like(g)
        with torch.cuda.device(g.device):
            rc = lib.linf_mean_shift(g.data_ptr(), g.size(0), g.size(1), None, 0.0, out.data_ptr(), None, _stream())
        _lib.check(rc, "mean_shift backward")
        return out, None, None


_fused_mean_shift = True
_bounds_only = False


class bounds_only:
    """Context manager: distance layers that are given lower / upper bounds in eval mode skip their value
    path and return the lower bound in its place.  For passes that use the bounds alone (certification:
    the worst-case margins never look at the value), saving one forward kernel per layer."""

    def __enter__(self):
        global _bounds_only
        self.saved, _bounds_only = _bounds_only, True

    def __exit__(self, *exc):
        global _bounds_only
        _bounds_only = self.saved


def set_fused_epilogue(flag):
    """True (default): on CUDA, dense layers run the training-mode mean shift as one launch and fold the
    eval-mode mean shift / bias / sign flip into the forward and bound kernels.  False: the same steps as
    separate torch operations (the reference's sequence)."""
    global _fused_mean_shift
    _fused_mean_shift = bool(flag)


def get_fused_epilogue():
    return _fused_mean_shift


class MeanNorm(nn.Module):
    """Subtracts the per-channel mean: the batch mean while training (tracking an exponential
    running mean), the running mean in eval mode."""

    def __init__(self, out_channels, momentum=0.1):
        super().__init__()
        self.out_channels = out_channels
        self.momentum = momentum
        self.register_buffer("running_mean", torch.zeros(out_channels))

    def forward(self, x):
        if (self.training and _fused_mean_shift and x.is_cuda and x.dtype == torch.float32
                and x.numel() == x.size(0) * x.size(1) and x.numel() > 0 and self.running_mean.is_contiguous()):
            # dense activation: mean, running mean and subtraction in one launch
            return MeanShiftF.apply(x.reshape(x.size(0), x.size(1)).contiguous(), self.running_mean, self.momentum).view_as(x)
        flat = x.reshape(x.size(0), x.size(1), -1)
        if self.training:
            mean = flat.mean(dim=-1).mean(dim=0) if x.dim() > 2 else x.mean(dim=0)
            with torch.no_grad():
                self.running_mean.mul_(1 - self.momentum).add_(mean, alpha=self.momentum)
        else:
            mean = self.running_mean
        return (flat - mean.unsqueeze(-1)).view_as(x)

    def extra_repr(self):
        return str(self.out_channels)


class NormDistConv(nn.Module):
    """Convolution-shaped distance layer: every output is the L_p distance between an input
    patch and a weight row.  state_dict keys match the reference: weight [CO, CI/group, k, k],
    optional bias [CO], optional normalize.running_mean [CO]."""

    tag_counter = 0

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, group=1, p=0,
                 bias=True, mean_normalize=False, identity_init=True):
        super().__init__()
        assert in_channels % group == 0 and out_channels % group == 0
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = kernel_size, stride, padding, dilation
        self.group, self.p = group, p
        per_group = in_channels // group
        w = torch.randn(out_channels, per_group, kernel_size, kernel_size)
        if identity_init and in_channels <= out_channels:
            rows = torch.arange(out_channels)
            c = kernel_size // 2
            w[rows, rows % per_group, c, c] = -10.0
        self.weight = nn.Parameter(w)
        self.normalize = MeanNorm(out_channels) if mean_normalize else None
        self.bias = nn.Parameter(torch.zeros(out_channels)) if bias else None
        NormDistConv.tag_counter += 1
        self.tag = NormDistConv.tag_counter

    def _patches(self, t):
        if self.kernel_size == 1 and self.stride == 1 and self.padding == 0:
            return t.reshape(t.size(0), t.size(1), -1)      # a dense layer needs no unfold copy
        return F.unfold(t, self.kernel_size, self.dilation, self.padding, self.stride)

    def _post(self, t):
        if self.normalize is not None:
            t = self.normalize(t)
        if self.bias is not None:
            t = t + self.bias.view(1, -1, 1, 1)
        return t

    def _fused_post(self, negate):
        """(sub, add, negate) of this layer in eval mode, or None when the fused epilogue does not apply."""
        if not _fused_mean_shift or self.training or not math.isinf(self.p) or not self.weight.is_cuda:
            return None
        sub = self.normalize.running_mean if self.normalize is not None else None
        add = self.bias.detach() if self.bias is not None else None
        if sub is None and add is None and not negate:
            return None
        return (sub, add, negate)

    def forward(self, x, lower=None, upper=None, negate=False):
        """negate=True returns the negated layer (value negated, bounds negated and exchanged): the
        classifier layer of the distance nets, where a small distance means "this class"."""
        h, w = x.size(2), x.size(3)
        ho = (h + 2 * self.padding - self.dilation * (self.kernel_size - 1) - 1) // self.stride + 1
        wo = (w + 2 * self.padding - self.dilation * (self.kernel_size - 1) - 1) // self.stride + 1
        weight = self.weight.view(self.weight.size(0), -1)
        cols = self._patches(x)
        post = self._fused_post(negate)
        if post is not None and _dense_route(cols, weight, self.group):
            post = None
        needs_grad = torch.is_grad_enabled() and (cols.requires_grad or weight.requires_grad)
        if _bounds_only and lower is not None and upper is not None and not self.training and not needs_grad:
            y = None                     # filled with the lower bound below: nobody reads the value in such a pass
        elif post is not None and not needs_grad:
            # inference: mean shift, bias and sign flip leave the forward kernel already applied
            y = inf_dist_post(cols.contiguous(), weight.detach(), self.group, post, tag=self.tag).view(x.size(0), -1, ho, wo)
        else:
            y = norm_dist(cols, weight, self.group, p=self.p, tag=self.tag).view(x.size(0), -1, ho, wo)
            y = self._post(y)
            if negate:
                y = -y
        if lower is None or upper is None:
            return y, None, None
        assert math.isinf(self.p) and not self.training
        shape = (x.size(0), -1, ho, wo)
        if post is not None:
            lo, up = inf_dist_bound(self._patches(lower).contiguous(), self._patches(upper).contiguous(), weight.detach(),
                                    self.group, tag=self.tag, post=post)
            lo, up = lo.view(shape), up.view(shape)
        else:
            lo, up = inf_dist_bound(self._patches(lower), self._patches(upper), weight, self.group, tag=self.tag)
            lo, up = self._post(lo.view(shape)), self._post(up.view(shape))
            if negate:
                lo, up = -up, -lo
        return (lo if y is None else y), lo, up

    def extra_repr(self):
        s = f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}"
        if self.padding != 0:
            s += f", padding={self.padding}"
        if self.dilation != 1:
            s += f", dilation={self.dilation}"
        if self.group != 1:
            s += f", group={self.group}"
        if self.bias is None:
            s += ", bias=False"
        return s


class NormDist(NormDistConv):
    """Dense distance layer: a NormDistConv with a 1 x 1 kernel on [B, C] activations."""

    def __init__(self, in_features, out_features, p=0, bias=True, mean_normalize=False, identity_init=True):
        super().__init__(in_features, out_features, 1, p=p, bias=bias, mean_normalize=mean_normalize,
                         identity_init=identity_init)

    def forward(self, x, lower=None, upper=None, negate=False):
        as4d = lambda t: None if t is None else t.reshape(t.size(0), t.size(1), 1, 1)
        y, lo, up = super().forward(as4d(x), as4d(lower), as4d(upper), negate=negate)
        flat = lambda t: None if t is None else t.reshape(t.size(0), t.size(1))
        return flat(y), flat(lo), flat(up)

    def extra_repr(self):
        return f"in_features={self.in_channels}, out_features={self.out_channels}, bias={self.bias is not None}"


def set_p_norm(model, p):
    for m in model.modules():
        if isinstance(m, NormDistConv):
            m.p = p


def get_p_norm(model):
    for m in model.modules():
        if isinstance(m, NormDistConv):
            return m.p
    return None
