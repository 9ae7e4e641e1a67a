"""Certification and attack drivers on top of the distance layers.

certify / certified_accuracy follow certified_test of zbh2047/L_inf-dist-net (main.py:166-194): the
net is put in eval mode with p = inf, the input box [x - eps, x + eps] is clamped to the data range and
propagated through every layer with the fused lower/upper kernel (NormDist.forward with lower/upper,
model/norm_dist.py:141-155), and a sample counts as certified when the worst-case margin of every
other class against its label stays below the label's own entry (0), i.e. when the arg-max of the
worst-case margins is the label (main.py:186).

AttackPGD follows attack.py:5-36: projected gradient ascent on the cross entropy with sign steps.
The parameters do not require gradients during the search, so every distance layer runs only its
grad_input kernel in the backward pass (DistF.backward honours needs_input_grad).
"""
import torch
import torch.nn.functional as F

from .nets import get_eps, set_eps
from .norm_dist import bounds_only, get_p_norm, set_p_norm


@torch.no_grad()
def certify(net, inputs, targets, eps, up, down, values=False):
    """Worst-case margins of one batch under an l_inf perturbation of radius eps.

    up / down: tensors broadcastable to `inputs` with the largest / smallest valid input value per
    element (the normalised data range).  Returns (certified [B] bool, margins [B, classes]); the p
    norm, eps and train/eval state of the net are restored.  The margins depend on the propagated bounds
    alone, so by default the distance layers skip their value path (values=True runs it as the
    reference's loop does: same margins, one more kernel per layer)."""
    save_p, save_eps, was_training = get_p_norm(net), get_eps(net), net.training
    set_eps(net, eps)
    set_p_norm(net, float("inf"))
    net.eval()
    try:
        lower = torch.max(inputs - eps, down)
        upper = torch.min(inputs + eps, up)
        if values:
            margins = net(inputs, lower=lower, upper=upper, targets=targets)[1]
        else:
            with bounds_only():
                margins = net(inputs, lower=lower, upper=upper, targets=targets)[1]
    finally:
        set_p_norm(net, save_p)
        set_eps(net, save_eps)
        net.train(was_training)
    return margins.max(dim=1)[1] == targets, margins


@torch.no_grad()
def certified_accuracy(net, batches, eps, up, down, values=False):
    """Fraction of samples certified over an iterable of (inputs, targets) batches already on the
    net's device (the reference moves each batch there itself, main.py:177-180)."""
    good = total = 0
    for inputs, targets in batches:
        ok, _ = certify(net, inputs, targets, eps, up, down, values=values)
        good += int(ok.sum().item())
        total += targets.numel()
    return good / max(total, 1)


class AttackPGD:
    """Projected gradient attack in the l_inf ball of radius eps around the inputs, clamped to the
    data range [down, up]; `find` returns the perturbed inputs."""

    def __init__(self, net, eps, step_size, num_steps, up, down, random_start=True):
        self.net, self.eps, self.step_size, self.num_steps = net, eps, step_size, num_steps
        self.up, self.down, self.rand = up, down, random_start

    def find(self, inputs, targets):
        saved = [q.requires_grad for q in self.net.parameters()]
        self.net.requires_grad_(False)
        try:
            x = inputs.detach()
            if self.rand:
                noise = torch.zeros_like(x).normal_(0, self.eps / 4)
                x = x + torch.clamp(noise, -self.eps / 2, self.eps / 2)
                x = torch.min(torch.max(x, self.down), self.up)
            for _ in range(self.num_steps):
                x.requires_grad_()
                loss = F.cross_entropy(self.net(x), targets, reduction="sum")
                loss.backward()
                x = torch.add(x.detach(), torch.sign(x.grad.detach()), alpha=self.step_size)
                x = torch.min(torch.max(x, inputs - self.eps), inputs + self.eps)
                x = torch.min(torch.max(x, self.down), self.up)
        finally:
            for q, r in zip(self.net.parameters(), saved):
                q.requires_grad_(r)
        return x
