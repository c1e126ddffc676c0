"""Host-side M2-BERT encoder around the accelerated mixer and MLP: embeddings, the layer
loop and (optionally) the MLM-free encoder output.  Parameter names follow the reference's
BertModel (bert/src/bert_layers.py:131-252 embeddings, :511-599 layer, :602-813 encoder,
:880-1021 model) so a reference state_dict loads unchanged:

    embeddings.{word,position,token_type}_embeddings.weight, embeddings.LayerNorm.*,
    encoder.layer.<i>.attention.* (mixer), encoder.layer.<i>.mlp.* (GLU MLP)

Unlike the reference's BertLayer this loop has no per-layer ``isnan().any()``
device-to-host synchronisation; ``check_finite=True`` restores an equivalent check once,
on the final output.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ._tags import attach
from .glu_mlp import BertGatedLinearUnitMLP
from .hyena_filter import _autocast_bf16
from .sequence_mixer import MonarchMixerSequenceMixing


@dataclass
class M2BertConfig:
    """The fields of the reference's BertConfig (bert/src/configuration_bert.py) that the
    Monarch-Mixer branch reads; defaults are the 80M pretraining yaml's."""
    vocab_size: int = 30528
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    max_position_embeddings: int = 128
    type_vocab_size: int = 2
    pad_token_id: int = 0
    layer_norm_eps: float = 1e-12
    hidden_dropout_prob: float = 0.1
    use_positional_encodings: bool = True
    monarch_mixer_sequence_mixing: bool = True
    use_glu_mlp: bool = True
    use_monarch_mlp: bool = True
    monarch_mlp_nblocks: int = 4
    long_conv_l_max: int = 128
    long_conv_kernel_learning_rate: float = 1e-3
    bidirectional: bool = True
    residual_long_conv: bool = True
    hyena_lr_pos_emb: float = 1e-5
    hyena_w: int = 10
    hyena_w_mod: int = 1
    hyena_wd: float = 0.1
    hyena_emb_dim: int = 5
    hyena_filter_dropout: float = 0.0
    hyena_filter_order: int = 128
    hyena_training_additions: bool = False
    pool_all: bool = False           # pooler: mean over unmasked positions instead of the first token
    use_cls_token: bool = True
    sequence_token_planting: bool = False


class M2BertEmbeddings(nn.Module):
    """word + token-type (+ learned position) embeddings, LayerNorm, dropout."""

    def __init__(self, config):
        super().__init__()
        self.word_embeddings = nn.Embedding(config.vocab_size, config.hidden_size,
                                            padding_idx=config.pad_token_id)
        self.use_positional_encodings = config.use_positional_encodings
        if config.use_positional_encodings:
            self.position_embeddings = nn.Embedding(config.max_position_embeddings, config.hidden_size)
            self.register_buffer("position_ids",
                                 torch.arange(config.max_position_embeddings).expand((1, -1)))
        self.token_type_embeddings = nn.Embedding(config.type_vocab_size, config.hidden_size)
        self.LayerNorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, input_ids, token_type_ids=None, position_ids=None):
        L = input_ids.shape[1]
        D = self.word_embeddings.weight.shape[1]
        if (input_ids.is_cuda and input_ids.dim() == 2 and not torch.is_grad_enabled() and _autocast_bf16()
                and not (self.training and self.dropout.p > 0) and D % 256 == 0 and D <= 2048
                and self.word_embeddings.weight.dtype == torch.float32):
            # gathers, adds, LayerNorm and the first mixer's copies in one launch
            return self._fused_embeddings(input_ids, token_type_ids, position_ids)
        e = self.word_embeddings(input_ids)
        if token_type_ids is None:
            e = e + self.token_type_embeddings.weight[0]
        else:
            e = e + self.token_type_embeddings(token_type_ids)
        if self.use_positional_encodings:
            if position_ids is None:
                position_ids = self.position_ids[:, :L]
            e = e + self.position_embeddings(position_ids)
        if (e.is_cuda and e.dim() == 3 and e.dtype == torch.float32 and not torch.is_grad_enabled()
                and _autocast_bf16()
                and not (self.training and self.dropout.p > 0) and e.shape[-1] % 256 == 0 and e.shape[-1] <= 2048):
            # the first mixer reads bf16 / time-major fp16 copies of this output: have the LayerNorm
            # kernel write them instead of separate cast, fill and transpose passes
            return self._layernorm_with_copies(e)
        return self.dropout(self.LayerNorm(e))

    def _fused_embeddings(self, input_ids, token_type_ids, position_ids):
        from . import ops
        B, L = input_ids.shape
        D = self.word_embeddings.weight.shape[1]
        aug = torch.empty((B * L, D), dtype=torch.bfloat16, device=input_ids.device)
        tm = None
        if L % 8 == 0 and ops.longconv_kind_batch(B, L, torch.bfloat16, D) in (2, 3):
            tm = torch.empty((D, B, L), dtype=torch.float16, device=input_ids.device)
        pos = self.position_embeddings.weight if self.use_positional_encodings else None
        if pos is not None and position_ids is None and L > pos.shape[0]:
            raise RuntimeError(f"sequence length {L} exceeds max_position_embeddings {pos.shape[0]}")
        y = ops.embed_layernorm_fwd(input_ids, self.word_embeddings.weight, self.token_type_embeddings.weight, pos,
                                    self.LayerNorm.weight, self.LayerNorm.bias, self.LayerNorm.eps,
                                    token_type_ids=token_type_ids, position_ids=position_ids,
                                    bf16_copy=aug, tm_copy=tm, fill_pad=False)
        return attach(y, bf16=aug, tm=tm)

    def _layernorm_with_copies(self, e):
        from . import ops
        B, L, D = e.shape
        aug = torch.empty((B * L, D), dtype=torch.bfloat16, device=e.device)
        tm = None
        if L % 8 == 0 and ops.longconv_kind_batch(B, L, torch.bfloat16, D) in (2, 3):
            tm = torch.empty((D, B, L), dtype=torch.float16, device=e.device)
        y = ops.add_layernorm_fwd(e.reshape(B * L, D), None, self.LayerNorm.weight, self.LayerNorm.bias,
                                  self.LayerNorm.eps, torch.float32, bf16_copy=aug, tm_copy=tm, fill_pad=False)
        y = y.view(B, L, D)
        return attach(y, bf16=aug, tm=tm)


class M2BertLayer(nn.Module):
    """Sequence mixing then state mixing; no residual or LayerNorm around the mixer."""

    def __init__(self, config):
        super().__init__()
        self.attention = MonarchMixerSequenceMixing(
            config.hidden_size, l_max=config.long_conv_l_max,
            hyena_kernel_lr=config.long_conv_kernel_learning_rate,
            bidirectional=config.bidirectional, hyena_lr_pos_emb=config.hyena_lr_pos_emb,
            hyena_w=config.hyena_w, hyena_w_mod=config.hyena_w_mod, hyena_wd=config.hyena_wd,
            hyena_emb_dim=config.hyena_emb_dim, hyena_filter_dropout=config.hyena_filter_dropout,
            hyena_filter_order=config.hyena_filter_order,
            residual_long_conv=config.residual_long_conv,
            hyena_training_additions=config.hyena_training_additions)
        self.mlp = BertGatedLinearUnitMLP(config)

    def forward(self, hidden_states, copies_only=False):
        mixed, _ = self.attention(hidden_states)
        return self.mlp(mixed, copies_only=copies_only)


class M2BertEncoder(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layer = nn.ModuleList([M2BertLayer(config) for _ in range(config.num_hidden_layers)])

    def forward(self, hidden_states, attention_mask=None, output_all_encoded_layers=False):
        # the mask does not enter the Monarch-Mixer layers (the reference passes it to the
        # layer, which ignores it on this branch); padded positions are mixed like any other
        outs = []
        for i, layer in enumerate(self.layer):
            # between two of these layers only the next mixer reads the hidden state, through the
            # copies the MLP's LayerNorm writes for it; the float32 tensor is materialised when
            # somebody else will see it (last layer, or every layer on request)
            inner = (i + 1 < len(self.layer) and not output_all_encoded_layers
                     and not self.layer[i + 1].attention.hyena_training_additions)
            hidden_states = layer(hidden_states, copies_only=inner)
            if output_all_encoded_layers:
                outs.append(hidden_states)
        if not output_all_encoded_layers:
            outs.append(hidden_states)
        return outs


class M2BertPooler(nn.Module):
    """dense + tanh on the first token, on the mean of the unmasked positions (config.pool_all), or on
    the "planted" token average (config.sequence_token_planting) -- every branch of the reference's
    BertPooler (bert/src/bert_layers.py:816-859).  State-dict keys `dense.weight`, `dense.bias`.

    The planting branch follows the reference to the letter: ONE vector -- the sum, over every example
    and every position 128, 256, ... whose mask is 1, of that position's hidden state -- is added to the
    first-token row of every example, in place in `hidden_states` as the reference does, and the result is
    divided by the number of positions summed (over all examples) before the dense layer."""

    def __init__(self, config):
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.hidden_size)
        self.activation = nn.Tanh()
        self.pool_all = getattr(config, "pool_all", False)
        self.use_cls_token = getattr(config, "use_cls_token", True)
        self.sequence_token_planting = getattr(config, "sequence_token_planting", False)

    def forward(self, hidden_states, pool=True, mask=None):
        if not self.pool_all:
            if self.sequence_token_planting:
                if mask is None:
                    raise ValueError("sequence_token_planting needs the attention mask")
                first = hidden_states[:, 0]
                n_slots = int(hidden_states.shape[1] / 128)
                if n_slots > 1:
                    planted = hidden_states[:, 128:128 * n_slots:128]                # positions 128, 256, ...
                    keep = (mask[:, 128:128 * n_slots:128] == 1)
                    count = keep.sum()
                    first += (planted * keep.unsqueeze(-1).to(planted.dtype)).sum(dim=(0, 1))
                else:
                    count = torch.zeros((), dtype=torch.long, device=hidden_states.device)
                first = first / count
            else:
                first = hidden_states[:, 0] if pool else hidden_states
            return self.activation(self.dense(first))
        if mask is None:
            raise ValueError("pool_all needs the attention mask")
        denom = torch.sum(mask, dim=1, keepdim=True)
        mean = torch.sum(hidden_states * mask.unsqueeze(-1), dim=1) / denom
        return self.activation(self.dense(mean))


class M2BertModel(nn.Module):
    """Embeddings + encoder (+ pooler); forward(input_ids, ...) -> (sequence_output, pooled_output or None),
    the reference BertModel's pair (bert/src/bert_layers.py:899-919)."""

    def __init__(self, config, check_finite=False, add_pooling_layer=False):
        super().__init__()
        self.config = config
        self.embeddings = M2BertEmbeddings(config)
        self.encoder = M2BertEncoder(config)
        self.pooler = M2BertPooler(config) if add_pooling_layer else None
        self.check_finite = check_finite

    def forward(self, input_ids, token_type_ids=None, attention_mask=None, position_ids=None,
                output_all_encoded_layers=False):
        h = self.embeddings(input_ids, token_type_ids, position_ids)
        outs = self.encoder(h, attention_mask, output_all_encoded_layers)
        if self.check_finite and not torch.isfinite(outs[-1]).all():
            raise ValueError("non-finite values in the encoder output")
        pooled = None
        if self.pooler is not None:
            pooled = self.pooler(outs[-1], mask=attention_mask)
        return (outs if output_all_encoded_layers else outs[-1]), pooled
