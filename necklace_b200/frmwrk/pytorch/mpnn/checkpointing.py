"""Activation checkpointing with a model-parallel RNG tracker.

``checkpoint(fn, *args)`` runs ``fn`` without keeping its internal activations and
recomputes them in backward under the same random state.  Two extras follow the
reference (necklace/frmwrk/pytorch/mpnn/checkpointing.py:108-371):

* ``CudaRNGStatesTracker`` keeps named RNG states so that dropout inside
  tensor-parallel regions differs between mp ranks while everything else agrees;
  ``model_parallel_cuda_manual_seed(seed)`` installs seed ``seed + 2718 + mp_rank``
  under the name ``model-parallel-rng`` and ``seed`` as the default state.
* with ``partition_activations_in_checkpoint(True)`` each mp rank keeps only its
  ``1/mp`` slice of every saved input and the slices are all-gathered (on a side
  stream that the recompute waits for) right before the recomputation.

Works on CPU as well (the CPU generator takes the place of the CUDA one), which is
how the CPU test-suite exercises it.
"""
from __future__ import annotations

import contextlib

import torch

from ....comm import fns
from . import initialize as mpu

_MODEL_PARALLEL_RNG_TRACKER_NAME = "model-parallel-rng"
_PARTITION_ACTIVATIONS = False


def _cuda() -> bool:
    return torch.cuda.is_available()


def _get_rng_state():
    return torch.cuda.get_rng_state() if _cuda() else torch.get_rng_state()


def _set_rng_state(state):
    if _cuda():
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


def _manual_seed(seed):
    if _cuda():
        torch.cuda.manual_seed(seed)
    else:
        torch.manual_seed(seed)


def detach_variable(inputs, device=None):
    if not isinstance(inputs, tuple):
        raise RuntimeError(f"only tuples of tensors are supported, got {type(inputs).__name__}")
    out = []
    for inp in inputs:
        if not isinstance(inp, torch.Tensor):
            out.append(inp)
            continue
        x = inp.detach() if device is None else inp.to(device).detach()
        x.requires_grad = inp.requires_grad
        out.append(x)
    return tuple(out)


class CudaRNGStatesTracker:
    """Named RNG states; ``fork(name)`` runs a block under that state and stores the
    advanced state back."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.states_, self.seeds_ = {}, set()

    def get_states(self):
        return dict(self.states_)

    def set_states(self, states):
        self.states_ = states

    def add(self, name, seed):
        if seed in self.seeds_:
            raise Exception(f"seed {seed} already exists")
        if name in self.states_:
            raise Exception(f"rng state {name} already exists")
        self.seeds_.add(seed)
        orig = _get_rng_state()
        _manual_seed(seed)
        self.states_[name] = _get_rng_state()
        _set_rng_state(orig)

    @contextlib.contextmanager
    def fork(self, name=_MODEL_PARALLEL_RNG_TRACKER_NAME):
        if name not in self.states_:
            raise Exception(f"rng state {name} is not added")
        orig = _get_rng_state()
        _set_rng_state(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = _get_rng_state()
            _set_rng_state(orig)


_TRACKER = CudaRNGStatesTracker()


def get_cuda_rng_tracker():
    return _TRACKER


def model_parallel_cuda_manual_seed(seed):
    """Default state: ``seed`` (same on all mp ranks).  Tracked model-parallel state:
    ``seed + 2718 + mp_rank`` (different per mp rank, same across dp ranks)."""
    mp_seed = seed + 2718 + mpu.get_model_parallel_rank()
    _TRACKER.reset()
    _manual_seed(seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG_TRACKER_NAME, mp_seed)


def partition_activations_in_checkpoint(partition_activation: bool):
    global _PARTITION_ACTIVATIONS
    _PARTITION_ACTIVATIONS = bool(partition_activation)


def get_partition_size(item):
    return item.numel() // mpu.get_model_parallel_world_size()


def get_partition_start(item):
    return get_partition_size(item) * mpu.get_model_parallel_rank()


def _partition(t):
    """My 1/mp slice of a tensor's flat data (a copy, so the full tensor can be freed)."""
    n, s = get_partition_size(t), get_partition_start(t)
    return t.detach().contiguous().view(-1).narrow(0, s, n).clone()


def get_full_inputs(parts, shapes):
    """All-gather the saved slices back into full tensors."""
    ws = mpu.get_model_parallel_world_size()
    out = []
    for part, shape in zip(parts, shapes):
        if shape is None:
            out.append(part)
            continue
        full = torch.empty(ws * part.numel(), dtype=part.dtype, device=part.device)
        fns.all_gather(full, part, group=mpu.get_model_parallel_group())
        out.append(full.view(shape))
    return out


class CheckpointFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_function, *args):
        ctx.run_function = run_function
        ctx.fwd_cpu_rng = torch.get_rng_state()
        ctx.fwd_dev_rng = _get_rng_state()
        ctx.fwd_tracker = get_cuda_rng_tracker().get_states()
        with torch.no_grad():
            outputs = run_function(*args)
        ws = mpu.get_model_parallel_world_size()
        ctx.partitioned = _PARTITION_ACTIVATIONS and ws > 1
        ctx.requires = [isinstance(a, torch.Tensor) and a.requires_grad for a in args]
        if ctx.partitioned:
            saved, shapes = [], []
            for a in args:
                if isinstance(a, torch.Tensor) and a.is_floating_point() and a.numel() % ws == 0 \
                        and a.numel() > 0:
                    saved.append(_partition(a))
                    shapes.append(tuple(a.shape))
                else:
                    saved.append(a)
                    shapes.append(None)
            ctx.shapes = shapes
            ctx.save_for_backward(*[s for s in saved if isinstance(s, torch.Tensor)])
            ctx.non_tensors = [None if isinstance(s, torch.Tensor) else s for s in saved]
        else:
            ctx.save_for_backward(*[a for a in args if isinstance(a, torch.Tensor)])
            ctx.non_tensors = [None if isinstance(a, torch.Tensor) else a for a in args]
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        if not torch.autograd._is_checkpoint_valid():
            raise RuntimeError("checkpointing is not compatible with .grad(); use .backward()")
        tensors = list(ctx.saved_tensors)
        inputs, ti = [], 0
        for nt in ctx.non_tensors:
            if nt is None:
                inputs.append(tensors[ti])
                ti += 1
            else:
                inputs.append(nt)
        if ctx.partitioned:
            if _cuda() and any(isinstance(t, torch.Tensor) and t.is_cuda for t in inputs):
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    inputs = get_full_inputs(inputs, ctx.shapes)
                torch.cuda.current_stream().wait_stream(side)
            else:
                inputs = get_full_inputs(inputs, ctx.shapes)
        bwd_cpu_rng, bwd_dev_rng = torch.get_rng_state(), _get_rng_state()
        bwd_tracker = get_cuda_rng_tracker().get_states()
        torch.set_rng_state(ctx.fwd_cpu_rng)
        _set_rng_state(ctx.fwd_dev_rng)
        get_cuda_rng_tracker().set_states(ctx.fwd_tracker)
        detached = []
        for t, req in zip(inputs, ctx.requires):
            if isinstance(t, torch.Tensor):
                d = t.detach()
                d.requires_grad = req
                detached.append(d)
            else:
                detached.append(t)
        with torch.enable_grad():
            outputs = ctx.run_function(*detached)
        torch.set_rng_state(bwd_cpu_rng)
        _set_rng_state(bwd_dev_rng)
        get_cuda_rng_tracker().set_states(bwd_tracker)
        if isinstance(outputs, torch.Tensor):
            outputs = (outputs,)
        pairs = [(o, g) for o, g in zip(outputs, grads)
                 if isinstance(o, torch.Tensor) and o.requires_grad]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None,) + tuple(d.grad if isinstance(d, torch.Tensor) else None for d in detached)


def checkpoint(function, *args):
    """Checkpoint a model or part of a model (reference: checkpointing.py:368-371)."""
    return CheckpointFunction.apply(function, *args)
