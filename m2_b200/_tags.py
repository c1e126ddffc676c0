"""Host-side plumbing shared by the modules: the forward-only guard and the record through which a
LayerNorm hands the next mixer the copies of its output it has already written.
"""
from __future__ import annotations

import functools
import warnings

import torch

_warned = False


def forward_only(fn):
    """Decorator for a module's forward: the kernels implement the forward pass only.  Called with
    autograd enabled (as the reference's own benchmark does, bert/benchmark_fwd.py:70-75, with
    parameters that require grad) the forward runs under torch.no_grad() and its outputs do not
    require grad; a warning says so once per process."""

    @functools.wraps(fn)
    def wrapper(self, *args, **kwargs):
        if not torch.is_grad_enabled():
            return fn(self, *args, **kwargs)
        global _warned
        if not _warned:
            needs = any(isinstance(a, torch.Tensor) and a.requires_grad for a in args) or \
                any(p.requires_grad for p in self.parameters())
            if needs:
                _warned = True
                warnings.warn("m2_b200 modules are forward-only: outputs are computed under torch.no_grad() "
                              "and carry no autograd graph", RuntimeWarning, stacklevel=2)
        with torch.no_grad():
            return fn(self, *args, **kwargs)

    return wrapper


def _version_of(t):
    try:
        return t._version
    except RuntimeError:          # tensors made under torch.inference_mode() keep no version counter
        return None


class Copies:
    """What a LayerNorm of this package already wrote next to its output `t`:
    bf16     (B*L, D) row-major bf16 copy (what in_linear reads under autocast), or None
    tm       (D, B, L) fp16 time-major copy (the residual filter's operand), or None
    src_dtype  dtype the reference's tensor would have at this point (decides one rounding)
    The copies describe `t` as it was when they were attached: `valid_for` compares the tensor's
    storage pointer and version counter, so an in-place edit of the hidden state between two layers
    (a hook, `h.mul_(mask)`) makes the next mixer fall back to reading `t` itself."""

    __slots__ = ("bf16", "tm", "src_dtype", "ptr", "version")

    def __init__(self, t, bf16=None, tm=None, src_dtype=None):
        self.bf16, self.tm = bf16, tm
        self.src_dtype = src_dtype if src_dtype is not None else t.dtype
        self.ptr, self.version = t.data_ptr(), _version_of(t)

    def valid_for(self, t):
        return t.data_ptr() == self.ptr and _version_of(t) == self.version


def attach(t, bf16=None, tm=None, src_dtype=None):
    t._m2_copies = Copies(t, bf16, tm, src_dtype)
    return t


def copies_of(t):
    """The record attached to `t` if it still describes it, else None."""
    rec = getattr(t, "_m2_copies", None)
    if rec is not None and rec.valid_for(t):
        return rec
    return None


def src_dtype_of(t):
    rec = getattr(t, "_m2_copies", None)
    return rec.src_dtype if rec is not None else t.dtype
