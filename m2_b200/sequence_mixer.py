"""MonarchMixerSequenceMixing with the reference's constructor, forward signature and
state_dict layout (reference: bert/src/mm/monarch_mixer_sequence_mixer.py:12-154); the part
between in_linear and out_linear is one fused CUDA kernel.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops
from ._tags import copies_of, forward_only, src_dtype_of
from .hyena_filter import HyenaFilter, _autocast_bf16


class _Bf16Linear:
    """bf16 copy of a Linear's weight (what autocast would cast per call), refreshed when the parameter changes;
    the bias stays float32 -- the GEMM kernel rounds it to bf16 itself, as autocast's cast does."""

    def __init__(self):
        self.key, self.w = None, None

    def get(self, lin):
        key = (lin.weight.data_ptr(), lin.weight._version, lin.weight.device)
        if key != self.key:
            self.key, self.w = key, lin.weight.detach().to(torch.bfloat16).contiguous()
        return self.w


def bf16_input(u):
    """(B, L, D) bf16 tensor in_linear reads: the copy a preceding m2_b200 LayerNorm wrote (if u has not
    been edited since), else u cast to bf16."""
    B, L, D = u.shape
    rec = copies_of(u)
    c = rec.bf16 if rec is not None else None
    if c is not None and c.shape == (B * L, D) and c.device == u.device:
        return c.view(B, L, D)
    if u.dtype == torch.bfloat16 and u.stride(-1) == 1:
        return u
    return u.to(torch.bfloat16)


def _round_up(n, m):
    return (n + m - 1) // m * m


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

    def _weights(self):
        if not hasattr(self, "_w_in"):
            self._w_in, self._w_out = _Bf16Linear(), _Bf16Linear()
        return self._w_in.get(self.in_linear), self._w_out.get(self.out_linear)

    def _forward_long_rows(self, u, ures, specs, biases):
        """bf16 path for long sequences: the convolution kernel works on time-contiguous rows, so in_linear
        writes (B, 3D, L) and out_linear reads (B, D, L) -- both through the operand arrangements of
        m2_linear_fwd, no transposed copy of an activation.  Rows are padded to a multiple of 16 steps so
        that every row start is 32-byte aligned."""
        B, L, D = u.shape
        w_in, w_out = self._weights()
        Lp = _round_up(L, 16)
        # allocated per call: inside a CUDA-graph capture the buffers then belong to the graph's own pool
        xin_t = torch.empty((B, 3 * D, Lp), dtype=torch.bfloat16, device=u.device)[:, :, :L]
        ops.linear_fwd(bf16_input(u), w_in, self.in_linear.bias, out=xin_t.permute(0, 2, 1))
        u_view, yu_bf16 = None, False
        if ures is not None:
            rec = copies_of(ures)
            tm = rec.tm if rec is not None else None                         # (D, B, L) fp16 from the LayerNorm
            if tm is not None and tm.shape == (D, B, L) and tm.device == u.device:
                u_view = tm.permute(1, 2, 0)                                 # (B, L, D) view, time-contiguous
                yu_bf16 = src_dtype_of(ures) == torch.bfloat16
            else:
                u_view = ures.transpose(1, 2).contiguous().transpose(1, 2)
        y_t = torch.empty((B, D, Lp), dtype=torch.bfloat16, device=u.device)[:, :, :L]
        ops.longconv_fwd(xin_t.permute(0, 2, 1), u_view, self.short_filter.weight, self.short_filter.bias, specs,
                         biases, kind=2, bf16_rounding=True, out=y_t.permute(0, 2, 1), yu_bf16=yu_bf16)
        return ops.linear_fwd(y_t.permute(0, 2, 1), w_out, self.out_linear.bias)                      # (B, L, D)

    def _forward_toeplitz(self, u, ures, specs):
        """bf16 path for short sequences and large batches: the convolution kernel runs one Toeplitz GEMM
        per channel with the batch as its M dimension, on channel-major time-contiguous tensors -- in_linear
        writes (3D, B*L) and out_linear reads (D, B*L), each one launch of m2_linear_fwd."""
        B, L, D = u.shape
        w_in, w_out = self._weights()
        xin_t = torch.empty((3 * D, B, L), dtype=torch.bfloat16, device=u.device)
        ops.linear_fwd(bf16_input(u), w_in, self.in_linear.bias, out=xin_t.permute(1, 2, 0))
        u_t = None
        if ures is not None:
            rec = copies_of(ures)
            u_t = rec.tm if rec is not None else None
            if u_t is None or u_t.shape != (D, B, L) or u_t.device != u.device:
                u_t = ops.time_major_f16(ures)
        buf = torch.empty((D, B, L), dtype=torch.bfloat16, device=u.device)
        ops.longconv_fwd(xin_t.permute(1, 2, 0), u_t.permute(1, 2, 0) if u_t is not None else None,
                         self.short_filter.weight, self.short_filter.bias, specs, None,
                         kind=3, bf16_rounding=True, out=buf.permute(1, 2, 0),
                         yu_bf16=ures is not None and src_dtype_of(ures) == torch.bfloat16)
        return ops.linear_fwd(buf.permute(1, 2, 0), w_out, self.out_linear.bias)                     # (B, L, D)

    @forward_only
    def forward_channels(self, u, lo, hi):
        """Channels [lo, hi) of the tensor out_linear consumes, (B, L, hi - lo) bf16, computed from the full
        input u (B, L, d_model) under bf16 autocast -- the unit of work when the mixer is sharded by d_model
        channel over several GPUs: short convolution, gates and long convolutions are independent per
        channel, in_linear contributes its rows c, D + c, 2D + c, and only out_linear mixes channels (it is
        not part of a shard).  Shards computed on different GPUs and concatenated along the last axis equal
        forward_channels(u, 0, d_model) bit for bit.  The reference has no counterpart (its parallelism is
        data parallel only); this follows bert/src/mm/monarch_mixer_sequence_mixer.py:108-149 per channel."""
        if not (u.is_cuda and _autocast_bf16()):
            raise RuntimeError("forward_channels runs on CUDA tensors under torch.autocast('cuda', dtype=torch.bfloat16)")
        B, L, D = u.shape
        if not (0 <= lo < hi <= D):
            raise ValueError(f"channel range [{lo}, {hi}) outside d_model {D}")
        C = hi - lo
        filters = [self.filter_fn] + ([self.filter_fn2] if self.residual_long_conv else [])
        kind = ops.longconv_kind(L, torch.bfloat16, C)
        if kind == 1:
            kind = 0                         # the small-batch FFT family wants 128-channel tiles; a shard need not have them
        key = (lo, hi, L, kind, tuple(f._version_key() for f in filters),
               self.in_linear.weight._version, self.in_linear.bias._version,
               self.short_filter.weight._version, self.short_filter.bias._version,
               tuple(f.bias._version for f in filters))
        cache = getattr(self, "_shard_cache", None)
        if cache is None or cache[0] != key:
            rows = torch.cat([torch.arange(g * D + lo, g * D + hi, device=u.device) for g in range(3)])
            w_in, _ = self._weights()
            shard = dict(
                w=w_in[rows].contiguous(), b=self.in_linear.bias.detach()[rows].contiguous(),
                sw=self.short_filter.weight.detach()[rows].contiguous(), sb=self.short_filter.bias.detach()[rows].contiguous(),
                specs=[ops.filter_spectrum(f.time_filter(L, True)[lo:hi].contiguous(), L, kind) for f in filters],
                biases=[f.conv_bias().detach()[lo:hi].contiguous() for f in filters])
            self._shard_cache = cache = (key, shard)
        sh = cache[1]
        ures = u if self.residual_long_conv else None
        if kind == 2:
            Lp = _round_up(L, 16)
            xin_t = torch.empty((B, 3 * C, Lp), dtype=torch.bfloat16, device=u.device)[:, :, :L]
            ops.linear_fwd(bf16_input(u), sh["w"], sh["b"], out=xin_t.permute(0, 2, 1))
            u_view, yu_bf16 = None, False
            if ures is not None:
                rec = copies_of(ures)
                tm = rec.tm if rec is not None else None
                if tm is not None and tm.shape == (D, B, L):
                    u_view, yu_bf16 = tm[lo:hi].permute(1, 2, 0), src_dtype_of(ures) == torch.bfloat16
                else:
                    u_view = ures[..., lo:hi].transpose(1, 2).contiguous().transpose(1, 2)
            y_t = torch.empty((B, C, Lp), dtype=torch.bfloat16, device=u.device)[:, :, :L]
            ops.longconv_fwd(xin_t.permute(0, 2, 1), u_view, sh["sw"], sh["sb"], sh["specs"], sh["biases"],
                             kind=2, bf16_rounding=True, out=y_t.permute(0, 2, 1), yu_bf16=yu_bf16)
            return y_t.permute(0, 2, 1)
        xin = ops.linear_fwd(bf16_input(u), sh["w"], sh["b"])
        return ops.longconv_fwd(xin, ures[..., lo:hi] if ures is not None else None, sh["sw"], sh["sb"], sh["specs"],
                                sh["biases"], kind=kind, bf16_rounding=True)

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
            w_in, w_out = self._weights()
            xin = ops.linear_fwd(bf16_input(u), w_in, self.in_linear.bias)
        else:
            w_in, w_out = self.in_linear.weight.detach(), self.out_linear.weight.detach()
            xin = ops.linear_fwd(u, w_in, self.in_linear.bias)
        y = ops.longconv_fwd(xin, ures, self.short_filter.weight, self.short_filter.bias, specs, biases,
                             kind=kind, bf16_rounding=bf16)
        return ops.linear_fwd(y, w_out, self.out_linear.bias), None
