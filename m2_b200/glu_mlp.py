"""The GLU feed-forward block of an M2-BERT layer on BlockdiagLinear weights, with the
reference's constructor, forward signature and state_dict keys (reference:
bert/src/bert_layers.py:457-508): gated_layers, wo, layernorm.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops
from ._tags import attach, forward_only
from .blockdiag_linear import BlockdiagLinear, _compute_dtype


class BertGatedLinearUnitMLP(nn.Module):
    """LayerNorm(wo(gelu(G[..., :I]) * G[..., I:]) + x),  G = gated_layers(x).

    `config` needs hidden_size, intermediate_size, monarch_mlp_nblocks, layer_norm_eps,
    hidden_dropout_prob (and use_monarch_mlp=True: dense nn.Linear layers are the
    reference's other option and are not what this package accelerates).  G is never
    materialised: the gated GEMM applies GELU and the product in its epilogue.
    """

    def __init__(self, config):
        super().__init__()
        self.config = config
        if not getattr(config, "use_monarch_mlp", True):
            raise NotImplementedError("m2_b200.BertGatedLinearUnitMLP needs use_monarch_mlp=True")
        self.is_padded = getattr(config, "monarch_mixer_sequence_mixing", True)
        nb = config.monarch_mlp_nblocks
        self.gated_layers = BlockdiagLinear(config.hidden_size, config.intermediate_size * 2,
                                            bias=False, nblocks=nb)
        self.act = nn.GELU(approximate="none")
        self.wo = BlockdiagLinear(config.intermediate_size, config.hidden_size, nblocks=nb)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)
        self.layernorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)

    @forward_only
    def forward(self, hidden_states: torch.Tensor, copies_only: bool = False) -> torch.Tensor:
        """copies_only (used by M2BertEncoder between layers): when the next mixer of this shape
        reads nothing but the bf16 and time-major fp16 copies of the output, skip the float32
        tensor and return the bf16 copy as the hidden state (tagged with the dtype the
        reference's tensor would have, which decides one rounding point in the mixer)."""
        if self.training and self.dropout.p > 0:
            raise RuntimeError("m2_b200: dropout inside the fused MLP is not implemented; use eval()")
        cfg = self.config
        x = hidden_states
        dt = _compute_dtype(x)
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != dt:
            x2 = x2.to(dt)
        h = ops.blockdiag_glu_fwd(x2, self.gated_layers._weight_as(dt), cfg.intermediate_size)
        o = ops.blockdiag_fwd(h, self.wo._weight_as(dt), self.wo.bias, cfg.intermediate_size,
                              cfg.hidden_size)
        # under autocast LayerNorm runs in float32 and returns float32
        out_dtype = torch.float32 if dt == torch.bfloat16 else dt
        aug = None
        if dt == torch.bfloat16 and x.dim() == 3 and x.shape[-1] % 256 == 0 and x.shape[-1] <= 2048:
            # the next layer's in_linear reads this output cast to bf16: write that copy here
            # instead of leaving it to a separate cast pass
            aug = torch.empty((x2.shape[0], x.shape[-1]), dtype=torch.bfloat16, device=x.device)
        tm = None
        if (aug is not None and x.shape[1] % 8 == 0
                and ops.longconv_kind_batch(x.shape[0], x.shape[1], torch.bfloat16, x.shape[2]) in (2, 3)):
            # a following mixer of this shape runs a time-contiguous convolution kernel, which reads the
            # layer input as a time-major fp16 tensor: written here too
            tm = torch.empty((x.shape[2], x.shape[0], x.shape[1]), dtype=torch.float16, device=x.device)
        skip = copies_only and tm is not None
        y = ops.add_layernorm_fwd(o, x2, self.layernorm.weight, self.layernorm.bias,
                                  self.layernorm.eps, None if skip else out_dtype, bf16_copy=aug, tm_copy=tm,
                                  fill_pad=False)
        if skip:
            y = aug[:, :x.shape[-1]].view(x.shape[0], x.shape[1], x.shape[2])
        else:
            y = y.reshape(x.shape)
        if aug is not None or tm is not None:
            attach(y, bf16=aug, tm=tm, src_dtype=out_dtype)
        return y
