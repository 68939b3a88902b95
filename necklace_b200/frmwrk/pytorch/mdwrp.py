"""Model wrappers used by the ZeRO trainers (reference: necklace/frmwrk/pytorch/mdwrp.py:29-155).

``MdWrpWithSelfBkwd``  a model part that can run its own backward from the gradient of
                       its output; with ``do_acts_ckpt`` the forward runs without
                       building a graph (unless it is the last part) and is recomputed
                       with gradients inside ``mp_backward``.
``MdWrpWithCkpt``      forward through ``mpnn.checkpointing.checkpoint``.
``MdWrpWholeNet``      all parts in sequence (evaluation, whole-model state_dict with
                       keys ``whole_md.<i>.net...``)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .mpnn.checkpointing import checkpoint
from .mputils import _as_list


class MdWrpWithCkpt(nn.Module):
    def __init__(self, net, *args, **kwargs):
        super().__init__()
        self.net = net

    def forward(self, *inputs):
        return checkpoint(self.net, *inputs)


class MdWrpWithSelfBkwd(nn.Module):
    def __init__(self, submodules, mp_order=0, is_last_part=False, do_acts_ckpt=True,
                 *args, **kwargs):
        super().__init__()
        mods = _as_list(submodules)
        self.net = mods[0] if len(mods) == 1 else nn.Sequential(*mods)
        self.mp_order, self.is_last_part, self.do_acts_ckpt = mp_order, is_last_part, do_acts_ckpt
        self.inputs, self.output = None, None

    def _graded(self, inputs):
        out = []
        for x in inputs:
            if isinstance(x, torch.Tensor) and x.is_floating_point() and self.mp_order > 0:
                x = x.detach()
                x.requires_grad_(True)
            out.append(x)
        return out

    def cache_graded_input(self, *args, **kwargs):
        """Detach the inputs from the upstream graph (every unit but the first) so that their
        gradients can be read after ``mp_backward``, keep them, and return them
        (reference: necklace/frmwrk/pytorch/mdwrp.py:68-83)."""
        self.inputs = self._graded(args)
        return self.inputs

    @property
    def inp_cache(self):
        return self.inputs

    @property
    def out_cache(self):
        return self.output

    def forward(self, *inputs):
        self.inputs = self._graded(inputs)
        if self.do_acts_ckpt and not self.is_last_part and torch.is_grad_enabled():
            with torch.no_grad():
                self.output = self.net(*self.inputs)
        else:
            self.output = self.net(*self.inputs)
        return self.output

    def get_input_grads(self):
        return [x.grad for x in (self.inputs or [])
                if isinstance(x, torch.Tensor) and x.requires_grad and x.grad is not None]

    def mp_backward(self, grads):
        if self.do_acts_ckpt and not self.is_last_part:
            with torch.enable_grad():
                self.output = self.net(*self.inputs)  # recompute with a graph
        outs = [o for o in _as_list(self.output) if isinstance(o, torch.Tensor)]
        pairs = [(o, g) for o, g in zip(outs, _as_list(grads)) if o.requires_grad]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        self.output = None


class MdWrpWholeNet(nn.Module):
    def __init__(self, parts):
        super().__init__()
        self.whole_md = nn.Sequential(*parts)

    def forward(self, *inputs):
        x = inputs
        for m in self.whole_md:
            x = m(*x) if isinstance(x, (tuple, list)) else m(x)
        return x
