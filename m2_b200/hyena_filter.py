"""HyenaFilter and its parts with the reference's constructor arguments, attribute names
and state_dict keys (reference: bert/src/mm/hyena_utils.py:50-248 and
bert/src/utils/train.py:4-18), evaluated by the m2_b200 CUDA kernels.

The filter depends only on the parameters and the sequence length, so the time-domain
filter and the spectrum table the convolution kernel consumes are cached per
(sequence length, numeric mode) and recomputed when any parameter changes (in-place
updates and load_state_dict bump the tensors' version counters).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from . import ops
from ._tags import forward_only


class OptimModule(nn.Module):
    """nn.Module whose tensors can carry per-tensor optimizer settings.

    ``register(name, tensor, lr=0.0)`` stores a buffer; any other lr stores a Parameter
    with an ``_optim`` dict (``lr``, ``weight_decay``) that trainers may read.
    Same contract as the reference's OptimModule (bert/src/utils/train.py:4-18).
    """

    def register(self, name, tensor, lr=None, wd=0.0):
        if lr == 0.0:
            self.register_buffer(name, tensor)
            return
        self.register_parameter(name, nn.Parameter(tensor))
        hp = {}
        if lr is not None:
            hp["lr"] = lr
        if wd is not None:
            hp["weight_decay"] = wd
        getattr(self, name)._optim = hp


class Sin(nn.Module):
    """x -> sin(w_mod * freq * x) with a per-feature frequency (hyena_utils.py:50-63)."""

    def __init__(self, dim, w=10, w_mod=1, train_freq=True):
        super().__init__()
        f = w * torch.ones(1, dim)
        self.freq = nn.Parameter(f) if train_freq else f
        self.w_mod = w_mod

    def forward(self, x):
        return torch.sin(self.w_mod * self.freq * x)


class PositionalEmbedding(OptimModule):
    """Time feature t in [0,1] plus (emb_dim-1)/2 complex-exponential bands
    (hyena_utils.py:66-88): z = [t, Re e^{-i f w}, Im e^{-i f w}]."""

    def __init__(self, emb_dim: int, seq_len: int, lr_pos_emb: float = 1e-5, **kwargs):
        super().__init__()
        self.seq_len = seq_len
        t = torch.linspace(0, 1, seq_len)[None, :, None]
        bands = (emb_dim - 1) // 2 if emb_dim > 1 else 0
        pos = torch.linspace(0, seq_len - 1, seq_len)[None, :, None]
        w = 2 * math.pi * pos / seq_len
        f = torch.linspace(1e-4, bands - 1, bands)[None, None]
        phase = torch.exp(-1j * f * w)
        z = torch.cat([t, phase.real, phase.imag], dim=-1)
        self.register("z", z, lr=lr_pos_emb)
        self.register("t", t, lr=0.0)

    def forward(self, L):
        return self.z[:, :L], self.t[:, :L]


class ExponentialModulation(OptimModule):
    """h -> h * (exp(-t |delta_c|) + shift) with per-channel decay rates spread between a
    slow and a fast rate (hyena_utils.py:91-112)."""

    def __init__(self, d_model, fast_decay_pct=0.3, slow_decay_pct=1.5, target=1e-2,
                 modulation_lr=0.0, shift: float = 0.0, **kwargs):
        super().__init__()
        self.shift = shift
        fastest = math.log(target) / fast_decay_pct
        slowest = math.log(target) / slow_decay_pct
        self.register("deltas", torch.linspace(slowest, fastest, d_model)[None, None], lr=modulation_lr)

    def forward(self, t, x):
        return x * (torch.exp(-t * self.deltas.abs()) + self.shift)


def _autocast_bf16(device_type="cuda") -> bool:
    return torch.is_autocast_enabled(device_type) and torch.get_autocast_dtype(device_type) == torch.bfloat16


class HyenaFilter(OptimModule):
    """Implicit long-convolution filter: a small sine-activated MLP of the positional
    embedding, exponentially modulated; optionally a second MLP for the reversed direction.

    Constructor arguments, attributes and state_dict keys follow the reference
    (hyena_utils.py:115-199).  ``filter`` / ``filter_rev`` return (1, L, d_model) like the
    reference; ``forward`` runs the long convolution ``y = conv(x, k) + bias * x`` on
    (B, d_model, L) input (hyena_utils.py:219-248).
    """

    def __init__(self, d_model, emb_dim=3, order=16, seq_len=1024, lr=1e-3, lr_pos_emb=1e-5,
                 dropout=0.0, w=1, w_mod=1, wd=0, bias=True, num_inner_mlps=2,
                 linear_mixer=False, modulate: bool = True, normalized=False,
                 bidirectional=False, **kwargs):
        super().__init__()
        if emb_dim % 2 == 0 or emb_dim < 3:
            raise AssertionError("emb_dim must be odd and greater or equal to 3 (time, sine and cosine)")
        if linear_mixer or num_inner_mlps != 2 or not modulate or normalized:
            raise NotImplementedError(
                "m2_b200.HyenaFilter covers the M2-BERT configuration: num_inner_mlps=2, "
                "linear_mixer=False, modulate=True, normalized=False")
        self.d_model = d_model
        self.emb_dim = emb_dim
        self.seq_len = seq_len
        self.modulate = modulate
        self.use_bias = bias
        self.bidirectional = bidirectional
        self.normalized = normalized

        self.bias = nn.Parameter(torch.randn(d_model))
        self.dropout = nn.Dropout(dropout)
        act = Sin(dim=order, w=w, w_mod=w_mod)          # one instance shared by every slot
        self.pos_emb = PositionalEmbedding(emb_dim, seq_len, lr_pos_emb)

        def mlp():
            layers = [nn.Linear(emb_dim, order), act]
            for _ in range(num_inner_mlps):
                layers += [nn.Linear(order, order), act]
            layers.append(nn.Linear(order, d_model, bias=False))
            return nn.Sequential(*layers)

        self.implicit_filter = mlp()
        if bidirectional:
            self.implicit_filter_rev = mlp()
        self.modulation = ExponentialModulation(d_model, **kwargs)
        for child in self.implicit_filter.children():
            for name in child.state_dict():
                getattr(child, name)._optim = {"weight_decay": wd, "lr": lr}
        # the reference's encoder sets these when its FlashFFTConv route is on (bert_layers.py:616-626);
        # they are accepted and ignored: the kernels of this package are the only route
        self.flashfft = None
        self.use_flash_fft = False
        self._cache = {}

    # ---- cached kernel products -------------------------------------------------------
    def _net(self, rev):
        seq = self.implicit_filter_rev if rev else self.implicit_filter
        return [seq[i].weight for i in (0, 2, 4, 6)], [seq[i].bias for i in (0, 2, 4)]

    def _version_key(self):
        ts = [self.pos_emb.z, self.pos_emb.t, self.modulation.deltas, self.implicit_filter[1].freq]
        for rev in ([False, True] if self.bidirectional else [False]):
            w, b = self._net(rev)
            ts += w + b
        return tuple((t.data_ptr(), t._version) for t in ts)

    def time_filter(self, L, bf16_rounding):
        """Merged time-domain filter (d_model, R): [k_fwd | zeros | reversed k_rev]."""
        key = ("k", int(L), bool(bf16_rounding))
        ver = self._version_key()
        hit = self._cache.get(key)
        if hit is not None and hit[0] == ver:
            return hit[1]
        if L > self.pos_emb.z.shape[1]:
            raise RuntimeError(f"sequence length {L} exceeds the filter's seq_len {self.pos_emb.z.shape[1]}")
        w, b = self._net(False)
        wr, br = self._net(True) if self.bidirectional else (None, None)
        act = self.implicit_filter[1]
        k = ops.hyena_filter(self.pos_emb.z, self.pos_emb.t, w, b, wr, br, act.freq,
                             self.modulation.deltas, L, bidirectional=self.bidirectional,
                             bf16_rounding=bf16_rounding, w_mod=act.w_mod,
                             shift=self.modulation.shift)
        self._cache[key] = (ver, k)
        return k

    def spectrum(self, L, bf16_rounding, kind):
        key = ("s", int(L), bool(bf16_rounding), int(kind))
        ver = self._version_key()
        if kind == 3:   # this table holds the bias too
            ver = ver + ((self.bias.data_ptr(), self.bias._version, bool(self.use_bias)),)
        hit = self._cache.get(key)
        if hit is not None and hit[0] == ver:
            return hit[1]
        spec = ops.filter_spectrum(self.time_filter(L, bf16_rounding), L, kind,
                                   bias=self.conv_bias() if kind == 3 else None)
        self._cache[key] = (ver, spec)
        return spec

    def conv_bias(self, bias=None):
        b = self.bias if bias is None else bias.reshape(-1)
        return b if self.use_bias else torch.zeros_like(b)

    # ---- reference API ----------------------------------------------------------------
    def filter(self, L, *args, **kwargs):
        k = self.time_filter(L, _autocast_bf16())
        return k[:, :L].t().unsqueeze(0)

    def filter_rev(self, L, *args, **kwargs):
        if not self.bidirectional:
            raise AttributeError("filter_rev needs bidirectional=True")
        k = self.time_filter(L, _autocast_bf16())
        return k[:, -L:].flip(-1).t().unsqueeze(0)

    @forward_only
    def forward(self, x, L, k_fwd=None, k_rev=None, bias=None, *args, **kwargs):
        """y = long_conv(x) + bias * x for x (B, d_model, L).  Without k_fwd the filters are the
        module's own (cached).  Caller-supplied filters are used as the reference uses them
        (hyena_utils.py:219-234): k_fwd (d_model, L) and, for a bidirectional module, k_rev
        (d_model, L), merged as pad(k_fwd) + pad(flip(k_rev)); a tuple stands for its first entry."""
        if x.dim() != 3 or x.shape[1] != self.d_model:
            raise RuntimeError(f"HyenaFilter.forward expects (B, {self.d_model}, L), got {tuple(x.shape)}")
        rounding = x.dtype == torch.bfloat16 or _autocast_bf16()
        if k_fwd is None:
            return ops.plain_longconv(x, self, L, rounding, bias)
        k_fwd = k_fwd[0] if type(k_fwd) is tuple else k_fwd
        R = ops.filter_row_len(L)
        k = torch.zeros((self.d_model, R), dtype=torch.float32, device=x.device)
        k[:, :L] = k_fwd.detach().reshape(self.d_model, -1)[:, :L]
        if self.bidirectional:
            if k_rev is None:
                raise RuntimeError("HyenaFilter.forward: a bidirectional filter given k_fwd needs k_rev too")
            k_rev = k_rev[0] if type(k_rev) is tuple else k_rev
            k[:, R - L:] += k_rev.detach().reshape(self.d_model, -1)[:, :L].flip(-1)
        return ops.plain_longconv(x, self, L, rounding, bias, spec=ops.filter_spectrum(k, L, 0))
