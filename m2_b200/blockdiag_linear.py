"""BlockdiagLinear / StructuredLinear with the reference's constructor, attributes and
state_dict keys (reference: bert/src/mm/blockdiag_linear.py:12-48,
bert/src/mm/structured_linear.py:11-70, bert/src/mm/blockdiag_multiply.py:10-60); the
multiply runs in the m2_b200 block-diagonal GEMM kernels.
"""
from __future__ import annotations

import math
from functools import partial

import torch
import torch.nn as nn
from torch.nn import init

from . import ops
from ._tags import forward_only
from .hyena_filter import _autocast_bf16


def blockdiag_weight_to_dense_weight(weight):
    """(nblocks, q, p) -> dense (nblocks*q, nblocks*p) block-diagonal matrix."""
    return torch.block_diag(*torch.unbind(weight, dim=0))


class _Bf16Cache:
    """bf16 copy of a float32 parameter, refreshed when the parameter changes."""

    def __init__(self):
        self.key, self.value = None, None

    def get(self, t):
        key = (t.data_ptr(), t._version, t.device)
        if key != self.key:
            self.value = t.detach().to(torch.bfloat16).contiguous()
            self.key = key
        return self.value


def _compute_dtype(x):
    """bf16 under CUDA autocast (the reference's BlockdiagMultiply casts its inputs to
    bf16 there, blockdiag_multiply.py:50), else the input's own dtype."""
    if _autocast_bf16():
        return torch.bfloat16
    return x.dtype


def blockdiag_multiply(x, weight, _cache=None):
    """out[..., k*q:(k+1)*q] = x[..., k*p:(k+1)*p] @ weight[k].T ; weight (nblocks, q, p)."""
    nb, q, p = weight.shape
    if x.shape[-1] != nb * p:
        raise AssertionError(f"last dimension {x.shape[-1]} != nblocks*p = {nb * p}")
    dt = _compute_dtype(x)
    w = weight.detach()
    if w.dtype != dt:
        w = _cache.get(weight) if (_cache is not None and dt == torch.bfloat16) else w.to(dt)
    x2 = x.reshape(-1, nb * p)
    if x2.dtype != dt:
        x2 = x2.to(dt)
    out = ops.blockdiag_fwd(x2, w.contiguous(), None, nb * p, nb * q)
    return out.reshape(*x.shape[:-1], nb * q)


class StructuredLinear(nn.Module):
    """Base class of structured linear maps: optional bias, in/out feature counts that a
    subclass may extend to a multiple of its block count."""

    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        if not hasattr(self, "in_features_extended"):
            self.in_features_extended = in_features
        if not hasattr(self, "out_features_extended"):
            self.out_features_extended = out_features
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)

    def reset_parameters(self) -> None:
        self.set_weights_from_dense_init(dense_init_fn_=partial(init.kaiming_uniform_, a=math.sqrt(5)))
        self.reset_parameters_bias()

    def set_weights_from_dense_init(self, dense_init_fn_):
        raise NotImplementedError

    def reset_parameters_bias(self):
        if self.bias is not None:
            fan_in = self.bias.shape[-1]
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            init.uniform_(self.bias, -bound, bound)

    @property
    def saving(self):
        raise NotImplementedError

    def convert_to_dense_weight(self):
        eye = torch.eye(self.in_features, device=self.weight.device, dtype=self.weight.dtype)
        return self.forward_matmul(eye).T

    def preprocess(self, x):
        missing = self.in_features_extended - x.shape[-1]
        return nn.functional.pad(x, (0, missing)) if missing > 0 else x

    def postprocess(self, output):
        return output[..., :self.out_features] if output.shape[-1] > self.out_features else output

    def forward_matmul(self, x):
        raise NotImplementedError

    def forward(self, x):
        out = self.forward_matmul(x)
        return out + self.bias.to(dtype=out.dtype) if self.bias is not None else out


class BlockdiagLinear(StructuredLinear):
    """Linear layer whose weight is block diagonal: nblocks independent
    (in/nblocks -> out/nblocks) maps; weight (nblocks, ceil(out/nb), ceil(in/nb))."""

    def __init__(self, *args, nblocks=4, shuffle=False, **kwargs):
        super().__init__(*args, **kwargs)
        p = int(math.ceil(self.in_features / nblocks))
        q = int(math.ceil(self.out_features / nblocks))
        self.in_features_extended = p * nblocks
        self.out_features_extended = q * nblocks
        self.shuffle = shuffle
        self.weight = nn.Parameter(torch.empty(nblocks, q, p))
        self._w_cache = _Bf16Cache()
        self.reset_parameters()

    def set_weights_from_dense_init(self, dense_init_fn_):
        dense = torch.empty(self.out_features_extended, self.in_features_extended,
                            device=self.weight.device, dtype=self.weight.dtype)
        dense_init_fn_(dense)
        dense *= math.sqrt(dense.numel() / self.weight.numel())   # the weight is sparse
        nb, q, p = self.weight.shape
        with torch.no_grad():
            # block k takes the first q rows of the dense init, columns [k*p, (k+1)*p)
            self.weight.copy_(dense[:q].reshape(q, nb, p).permute(1, 0, 2))

    @property
    def saving(self):
        return self.weight.numel() / (self.in_features * self.out_features)

    def _weight_as(self, dt):
        w = self.weight.detach()
        if w.dtype == dt:
            return w.contiguous()
        return self._w_cache.get(self.weight) if dt == torch.bfloat16 else w.to(dt)

    @forward_only
    def forward_matmul(self, x):
        return self._run(x, None)

    def _run(self, x, bias):
        nb, q, p = self.weight.shape
        if self.shuffle:
            x = self.preprocess(x)
            x = x.reshape(*x.shape[:-1], nb, p).transpose(-1, -2).reshape(*x.shape[:-1], nb * p)
        dt = _compute_dtype(x)
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != dt:
            x2 = x2.to(dt)
        out = ops.blockdiag_fwd(x2, self._weight_as(dt), bias, x2.shape[-1], self.out_features)
        return out.reshape(*x.shape[:-1], self.out_features)

    @forward_only
    def forward(self, x):
        """Padding of the input, the block multiply, the crop and the bias add run as one
        kernel."""
        if x.shape[-1] > self.in_features_extended:
            raise RuntimeError(f"input has {x.shape[-1]} features, layer takes {self.in_features}")
        return self._run(x, self.bias)
