"""MonarchMixerSequenceMixing with the reference's constructor, forward signature and
state_dict layout (reference: bert/src/mm/monarch_mixer_sequence_mixer.py:12-154); the part
between in_linear and out_linear is one fused CUDA kernel.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from ._tags import copies_of, forward_only, src_dtype_of
from .hyena_filter import HyenaFilter, _autocast_bf16


_PAD = 64   # extra contraction columns that carry the bias through the GEMM


class _AugmentedLinear:
    """bf16 copy of a Linear's weight with the bias as one more input column, refreshed when
    the parameters change.  Feeding an input whose extra column is 1 makes the GEMM add the
    (bf16-rounded, as under autocast) bias inside its float32 accumulator, so the result is
    rounded to bf16 exactly once -- like F.linear -- whatever layout the GEMM writes."""

    def __init__(self):
        self.key, self.w, self.b = None, None, None

    def get(self, lin):
        key = (lin.weight.data_ptr(), lin.weight._version, lin.bias._version, lin.weight.device)
        if key != self.key:
            out_f, in_f = lin.weight.shape
            w = torch.zeros((out_f, in_f + _PAD), dtype=torch.bfloat16, device=lin.weight.device)
            w[:, :in_f] = lin.weight.detach()
            w[:, in_f] = lin.bias.detach()
            self.key, self.w = key, w
            self.b = w[:, in_f].contiguous()          # the bf16-rounded bias on its own, for addmm
        return self.w


def make_augmented(m_rows, d, device):
    """(m_rows, d + _PAD) bf16 buffer whose extra columns are [1, 0, 0, ...]; the first d
    columns are left for the caller to fill."""
    buf = torch.empty((m_rows, d + _PAD), dtype=torch.bfloat16, device=device)
    buf[:, d] = 1.0
    buf[:, d + 1:] = 0.0
    return buf


def augmented_input(u):
    """bf16 copy of u with the bias column appended: reuses the copy a preceding m2_b200
    LayerNorm wrote (if u has not been edited since), else casts u."""
    B, L, D = u.shape
    rec = copies_of(u)
    aug = rec.bf16 if rec is not None else None
    if aug is not None and aug.shape == (B * L, D + _PAD) and aug.device == u.device:
        return aug.view(B, L, D + _PAD)
    aug = make_augmented(B * L, D, u.device).view(B, L, D + _PAD)
    aug[..., :D] = u
    return aug


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

    def _forward_long_rows(self, u, ures, specs, biases):
        """bf16 path for long sequences: the convolution kernel works on time-contiguous
        rows, so in_linear writes (B, 3D, L) and out_linear reads (B, D, L) -- both as
        library GEMMs on transposed operands, no transposed copy of an activation."""
        B, L, D = u.shape
        if not hasattr(self, "_aug_in"):
            self._aug_in, self._aug_out = _AugmentedLinear(), _AugmentedLinear()
        w_in, w_out = self._aug_in.get(self.in_linear), self._aug_out.get(self.out_linear)
        x_aug = augmented_input(u)
        with torch.autocast("cuda", enabled=False):
            xin_t = torch.matmul(w_in, x_aug.transpose(1, 2))                    # (B, 3D, L)
            u_view, yu_bf16 = None, False
            if ures is not None:
                rec = copies_of(ures)
                tm = rec.tm if rec is not None else None                         # (D, B, L) fp16 from the LayerNorm
                if tm is not None and tm.shape == (D, B, L) and tm.device == u.device:
                    u_view = tm.permute(1, 2, 0)                                 # (B, L, D) view, time-contiguous
                    yu_bf16 = src_dtype_of(ures) == torch.bfloat16
                else:
                    u_view = ures.transpose(1, 2).contiguous().transpose(1, 2)
            # allocated per call: inside a CUDA-graph capture the buffer then belongs to the graph's own pool
            y_t = torch.empty((B, D + _PAD, L), dtype=torch.bfloat16, device=u.device)
            y_t[:, D] = 1.0
            y_t[:, D + 1:] = 0.0
            ops.longconv_fwd(xin_t.transpose(1, 2), u_view,
                             self.short_filter.weight, self.short_filter.bias, specs, biases,
                             kind=2, bf16_rounding=True, out=y_t[:, :D].transpose(1, 2), yu_bf16=yu_bf16)
            return torch.matmul(y_t.transpose(1, 2), w_out.t())                  # (B, L, D)

    def _forward_toeplitz(self, u, ures, specs):
        """bf16 path for short sequences and large batches: the convolution kernel runs one
        Toeplitz GEMM per channel with the batch as its M dimension, on channel-major
        time-contiguous tensors -- in_linear writes (3D, B*L) and out_linear reads (D, B*L),
        both single library GEMMs on transposed operands."""
        B, L, D = u.shape
        if not hasattr(self, "_aug_in"):
            self._aug_in, self._aug_out = _AugmentedLinear(), _AugmentedLinear()
        w_in, w_out = self._aug_in.get(self.in_linear), self._aug_out.get(self.out_linear)
        x_aug = augmented_input(u).reshape(B * L, D + _PAD)
        with torch.autocast("cuda", enabled=False):
            xin_t = torch.matmul(w_in, x_aug.t())                                # (3D, B*L)
            u_t = None
            if ures is not None:
                rec = copies_of(ures)
                u_t = rec.tm if rec is not None else None
                if u_t is None or u_t.shape != (D, B, L) or u_t.device != u.device:
                    u_t = ops.time_major_f16(ures)
            # allocated per call: inside a CUDA-graph capture the buffer then belongs to the graph's own pool
            buf = torch.empty((D, B * L), dtype=torch.bfloat16, device=u.device)
            ops.longconv_fwd(xin_t.view(3 * D, B, L).permute(1, 2, 0),
                             u_t.permute(1, 2, 0) if u_t is not None else None,
                             self.short_filter.weight, self.short_filter.bias, specs, None,
                             kind=3, bf16_rounding=True, out=buf.view(D, B, L).permute(1, 2, 0),
                             yu_bf16=ures is not None and src_dtype_of(ures) == torch.bfloat16)
            # the output is row-major (B*L, D), so the library GEMM's own bias epilogue applies (bias added
            # in the float32 accumulator, one rounding, as F.linear) and K stays 768 instead of 768 + 64
            return torch.addmm(self._aug_out.b, buf.t(), w_out[:, :D].t()).view(B, L, D)

    @forward_only
    def forward(self, u, **kwargs):
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
        filters = [self.filter_fn] + ([self.filter_fn2] if self.residual_long_conv else [])
        biases = [f.conv_bias() for f in filters]
        act_dtype = torch.bfloat16 if bf16 else u.dtype
        kind = ops.longconv_kind_batch(u.size(0), L, act_dtype, self.d_model)
        specs = [f.spectrum(L, bf16, kind) for f in filters]
        ures = u_orig if self.residual_long_conv else None
        if kind == 3:
            return self._forward_toeplitz(u, ures, specs), None
        if kind == 2:
            return self._forward_long_rows(u, ures, specs, biases), None
        if bf16:
            # in_linear on the bf16 input with the bias carried as one more input column: the
            # same single rounding as F.linear under autocast, without per-call weight casts
            if not hasattr(self, "_aug_in"):
                self._aug_in, self._aug_out = _AugmentedLinear(), _AugmentedLinear()
            with torch.autocast("cuda", enabled=False):
                xin = torch.matmul(augmented_input(u), self._aug_in.get(self.in_linear).t())
        else:
            xin = self.in_linear(u)
        y = ops.longconv_fwd(xin, ures, self.short_filter.weight, self.short_filter.bias, specs, biases,
                             kind=kind, bf16_rounding=bf16)
        y = self.out_linear(y)
        return y, None
