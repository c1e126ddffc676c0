"""MonarchMixerSequenceMixing with the reference's constructor, forward signature and
state_dict layout (reference: bert/src/mm/monarch_mixer_sequence_mixer.py:12-154); the part
between in_linear and out_linear is one fused CUDA kernel.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .hyena_filter import HyenaFilter, _autocast_bf16


def _check_forward_only(module, x):
    """The kernels implement the forward pass only; refuse to build an autograd graph
    silently."""
    if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in module.parameters())):
        raise RuntimeError("m2_b200 modules are forward-only: call them under torch.no_grad() "
                           "or torch.inference_mode()")


class MonarchMixerSequenceMixing(nn.Module):
    """Gated bidirectional long-convolution sequence mixer.

    forward(u): u (B, L, d_model) -> (y (B, L, d_model), None) where, per channel,
    x1, x2, v = split(short_conv(in_linear(u)));  y = out_linear(long_conv(v * x1) * x2
    [+ long_conv2(u)]).  Under torch.autocast(bfloat16) the kernels round to bf16 exactly
    where the reference's PyTorch ops would.
    """

    def __init__(self, d_model, l_max=128, dropout=0.0, hyena_kernel_lr=None, bidirectional=False,
                 hyena_lr_pos_emb=1e-5, hyena_w=10, hyena_w_mod=1, hyena_wd=0.1, hyena_emb_dim=3,
                 hyena_filter_dropout=0.0, hyena_filter_order=16, residual_long_conv=False,
                 hyena_training_additions=False, verbose=False):
        super().__init__()
        self.d_model = d_model
        self.l_max = l_max
        self.kernel_lr = hyena_kernel_lr
        self.channels = 1
        self.bidirectional = bidirectional
        self.residual_long_conv = residual_long_conv
        self.NUM_PROJECTIONS = 3
        if verbose:
            print(f"-- Bidirectional: {bidirectional}  residual long conv: {residual_long_conv}  "
                  f"w: {hyena_w}  w_mod: {hyena_w_mod}  order: {hyena_filter_order}  emb: {hyena_emb_dim}")

        def make_filter():
            return HyenaFilter(d_model, order=hyena_filter_order, seq_len=l_max,
                               dropout=hyena_filter_dropout, bidirectional=bidirectional,
                               lr=hyena_kernel_lr, lr_pos_emb=hyena_lr_pos_emb, w=hyena_w,
                               w_mod=hyena_w_mod, wd=hyena_wd, emb_dim=hyena_emb_dim)

        self.filter_fn = make_filter()
        if residual_long_conv:
            self.filter_fn2 = make_filter()
        self.in_linear = nn.Linear(d_model, 3 * d_model)
        self.out_linear = nn.Linear(d_model, d_model)
        self.hyena_training_additions = hyena_training_additions
        if hyena_training_additions:
            self.act = nn.Identity()
            self.drop = nn.Dropout(dropout)
            self.layernorm = nn.LayerNorm(d_model)
        width = d_model * self.NUM_PROJECTIONS
        self.short_filter = nn.Conv1d(width, width, kernel_size=3, groups=width, padding=2)

    def forward(self, u, **kwargs):
        _check_forward_only(self, u)
        if not u.is_cuda:
            raise RuntimeError("m2_b200.MonarchMixerSequenceMixing needs CUDA tensors; there is no CPU fallback")
        if self.hyena_training_additions:
            if self.training and self.drop.p > 0:
                raise RuntimeError("m2_b200: dropout inside the fused mixer is not implemented; use eval()")
            u = self.layernorm(u)
        L = u.size(-2)
        bf16 = _autocast_bf16()
        if not bf16 and u.dtype != torch.float32:
            raise RuntimeError("m2_b200 mixer runs float32 inputs, or any input under "
                               "torch.autocast('cuda', dtype=torch.bfloat16); got "
                               f"{u.dtype} without autocast")
        if u.dim() == 2:
            u = u.unsqueeze(0)
        u_orig = u
        xin = self.in_linear(u)                        # bf16 under autocast, float32 otherwise
        kind = ops.longconv_kind(L, xin.dtype, self.d_model)
        filters = [self.filter_fn] + ([self.filter_fn2] if self.residual_long_conv else [])
        specs = [f.spectrum(L, bf16, kind) for f in filters]
        biases = [f.conv_bias() for f in filters]
        ures = u_orig if self.residual_long_conv else None
        if kind == 2:
            # the long-row kernel reads and writes time-contiguous rows: (B, channels, L)
            xin = xin.transpose(1, 2).contiguous().transpose(1, 2)
            if ures is not None:
                ures = ures.transpose(1, 2).contiguous().transpose(1, 2)
            out = torch.empty((u.shape[0], self.d_model, L), dtype=xin.dtype, device=xin.device).transpose(1, 2)
        else:
            out = None
        y = ops.longconv_fwd(xin, ures, self.short_filter.weight, self.short_filter.bias, specs, biases,
                             kind=kind, bf16_rounding=bf16, out=out)
        y = self.out_linear(y)
        return y, None
