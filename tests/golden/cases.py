"""Seeded parity cases shared by the fixture generator and the tests.

Weights and inputs are *not* stored in the fixtures: they are regenerated from a numpy
PCG64 stream keyed on (seed, tensor name), which is stable across numpy versions and
machines.  The fixtures hold only what the reference produced for them.

Distributions follow the reference's constructors (nn.Linear / Conv1d: U(+-1/sqrt(fan_in));
HyenaFilter.bias: N(0,1), bert/src/mm/hyena_utils.py:157; Sin.freq: w, :50-60;
BlockdiagLinear: Kaiming-uniform scaled by sqrt(nblocks), bert/src/mm/blockdiag_linear.py:26-36).
"""
from __future__ import annotations

import math
import zlib

import numpy as np

from oracle import m2_oracle as O


def _rng(seed, name):
    return np.random.default_rng([seed, zlib.crc32(name.encode())])


def _uniform(seed, name, shape, bound):
    return _rng(seed, name).uniform(-bound, bound, size=shape).astype(np.float32)


def _normal(seed, name, shape, std=1.0):
    return (_rng(seed, name).standard_normal(size=shape) * std).astype(np.float32)


def filter_state(seed, prefix, d_model, l_max, emb_dim, order, w, bidirectional):
    sd = {}
    sd[prefix + "bias"] = _normal(seed, prefix + "bias", (d_model,))
    z, t = O.positional_embedding(emb_dim, l_max)
    sd[prefix + "pos_emb.z"] = z[None]
    sd[prefix + "pos_emb.t"] = t[None, :, None]
    freq = np.full((1, order), float(w), np.float32)
    for net in ["implicit_filter."] + (["implicit_filter_rev."] if bidirectional else []):
        p = prefix + net
        dims = [(order, emb_dim), (order, order), (order, order)]
        for li, (o, i) in zip((0, 2, 4), dims):
            sd[p + f"{li}.weight"] = _uniform(seed, p + f"{li}.weight", (o, i), 1 / math.sqrt(i))
            sd[p + f"{li}.bias"] = _uniform(seed, p + f"{li}.bias", (o,), 1 / math.sqrt(i))
            sd[p + f"{li + 1}.freq"] = freq
        sd[p + "6.weight"] = _uniform(seed, p + "6.weight", (d_model, order), 1 / math.sqrt(order))
    sd[prefix + "modulation.deltas"] = O.modulation_deltas(d_model)[None, None]
    return sd


def mixer_state(seed, d_model, l_max, emb_dim=5, order=128, w=10, bidirectional=True,
                residual_long_conv=True, prefix=""):
    D = d_model
    sd = {}
    for f in ["filter_fn."] + (["filter_fn2."] if residual_long_conv else []):
        sd.update(filter_state(seed, prefix + f, D, l_max, emb_dim, order, w, bidirectional))
    sd[prefix + "in_linear.weight"] = _uniform(seed, prefix + "in_linear.weight", (3 * D, D), 1 / math.sqrt(D))
    sd[prefix + "in_linear.bias"] = _uniform(seed, prefix + "in_linear.bias", (3 * D,), 1 / math.sqrt(D))
    sd[prefix + "out_linear.weight"] = _uniform(seed, prefix + "out_linear.weight", (D, D), 1 / math.sqrt(D))
    sd[prefix + "out_linear.bias"] = _uniform(seed, prefix + "out_linear.bias", (D,), 1 / math.sqrt(D))
    sd[prefix + "short_filter.weight"] = _uniform(seed, prefix + "short_filter.weight", (3 * D, 1, 3), 1 / math.sqrt(3))
    sd[prefix + "short_filter.bias"] = _uniform(seed, prefix + "short_filter.bias", (3 * D,), 1 / math.sqrt(3))
    return sd


def blockdiag_weight(seed, name, in_features, out_features, nblocks):
    p = int(math.ceil(in_features / nblocks))
    q = int(math.ceil(out_features / nblocks))
    # Kaiming-uniform(a=sqrt(5)) on the dense (out_ext, in_ext) matrix, scaled by sqrt(nblocks)
    bound = math.sqrt(nblocks) / math.sqrt(p * nblocks)
    return _uniform(seed, name, (nblocks, q, p), bound)


def mlp_state(seed, d_model, inter, nblocks=4, prefix=""):
    sd = {}
    sd[prefix + "gated_layers.weight"] = blockdiag_weight(seed, prefix + "gated_layers.weight", d_model, 2 * inter, nblocks)
    sd[prefix + "wo.weight"] = blockdiag_weight(seed, prefix + "wo.weight", inter, d_model, nblocks)
    sd[prefix + "wo.bias"] = _uniform(seed, prefix + "wo.bias", (d_model,), 1 / math.sqrt(d_model))
    sd[prefix + "layernorm.weight"] = (1.0 + 0.1 * _normal(seed, prefix + "layernorm.weight", (d_model,))).astype(np.float32)
    sd[prefix + "layernorm.bias"] = 0.1 * _normal(seed, prefix + "layernorm.bias", (d_model,))
    return sd


def encoder_state(seed, n_layers, d_model, inter, l_max, vocab=30528, emb_dim=5, order=128,
                  w=10, nblocks=4, with_embeddings=True):
    """State dict with the reference BertModel's key names (embeddings.*, encoder.layer.i.*)."""
    sd = {}
    if with_embeddings:
        e = "embeddings."
        we = _normal(seed, e + "word_embeddings.weight", (vocab, d_model), 0.02)
        we[0] = 0.0  # padding_idx row
        sd[e + "word_embeddings.weight"] = we
        sd[e + "position_embeddings.weight"] = _normal(seed, e + "position_embeddings.weight", (l_max, d_model), 0.02)
        sd[e + "token_type_embeddings.weight"] = _normal(seed, e + "token_type_embeddings.weight", (2, d_model), 0.02)
        sd[e + "LayerNorm.weight"] = (1.0 + 0.1 * _normal(seed, e + "LayerNorm.weight", (d_model,))).astype(np.float32)
        sd[e + "LayerNorm.bias"] = 0.1 * _normal(seed, e + "LayerNorm.bias", (d_model,))
    for i in range(n_layers):
        p = f"encoder.layer.{i}."
        sd.update(mixer_state(seed + 1000 + i, d_model, l_max, emb_dim, order, w, True, True,
                              prefix=p + "attention."))
        sd.update(mlp_state(seed + 1000 + i, d_model, inter, nblocks, prefix=p + "mlp."))
    return sd


def randn(seed, name, shape):
    return _normal(seed, name, shape)


def subsample(a, limit=8192):
    """Deterministic strided subsample of a flattened array (all of it if small)."""
    flat = np.asarray(a).reshape(-1)
    if flat.size <= limit:
        return flat
    stride = max(1, flat.size // limit) | 1   # odd stride: no aliasing with power-of-two dims
    return flat[::stride]


# name -> config.  "kind" selects what the reference is asked to compute.
CASES = {
    # mixer: MonarchMixerSequenceMixing.forward
    "mixer_small": dict(kind="mixer", seed=11, B=2, L=32, D=32, emb=5, order=16, w=10,
                        bidirectional=True, residual=True),
    "mixer_small_causal": dict(kind="mixer", seed=12, B=3, L=24, D=16, emb=3, order=16, w=1,
                               bidirectional=False, residual=False, l_max=32),
    "mixer_cfg1_res": dict(kind="mixer", seed=0, B=8, L=128, D=768, emb=5, order=128, w=10,
                           bidirectional=True, residual=True),
    "mixer_cfg1_nores": dict(kind="mixer", seed=0, B=8, L=128, D=768, emb=5, order=128, w=10,
                             bidirectional=True, residual=False),
    "mixer_L2048": dict(kind="mixer", seed=13, B=1, L=2048, D=64, emb=5, order=128, w=10,
                        bidirectional=True, residual=True),
    # BlockdiagLinear.forward
    "blockdiag_small": dict(kind="blockdiag", seed=21, M=10, inf=64, outf=96, nb=4, bias=True),
    "blockdiag_ragged": dict(kind="blockdiag", seed=22, M=7, inf=30, outf=50, nb=4, bias=True),
    "blockdiag_80m_gated": dict(kind="blockdiag", seed=23, M=64, inf=768, outf=6144, nb=4, bias=False),
    "blockdiag_80m_wo": dict(kind="blockdiag", seed=24, M=64, inf=3072, outf=768, nb=4, bias=True),
    # BertGatedLinearUnitMLP.forward
    "glu_small": dict(kind="glu", seed=31, B=2, L=8, D=64, I=128, nb=4),
    "glu_80m": dict(kind="glu", seed=32, B=1, L=64, D=768, I=3072, nb=4),
    # BertModel: embeddings + encoder, 2 layers
    "encoder_small": dict(kind="encoder", seed=41, B=2, L=32, D=64, I=256, layers=2, vocab=512,
                          order=32),
}


# Pooler branches of the reference's BertPooler (first token / masked mean / token planting): stored whole,
# they are a few hundred numbers.  Generated by make_golden.py into pooler.npz.
POOLER = dict(seed=51, B=3, L=384, D=32, valid=[384, 130, 300])


def pooler_inputs():
    """hidden states (B, L, D), mask (B, L) with `valid[b]` leading ones, dense weight and bias."""
    c = POOLER
    h = randn(c["seed"], "h", (c["B"], c["L"], c["D"]))
    mask = np.zeros((c["B"], c["L"]), dtype=np.float32)
    for b, n in enumerate(c["valid"]):
        mask[b, :n] = 1.0
    w = randn(c["seed"], "w", (c["D"], c["D"])) * 0.2
    bias = randn(c["seed"], "b", (c["D"],)) * 0.1
    return h, mask, w.astype(np.float32), bias.astype(np.float32)


# Checkpoint of a short model as the reference's `BertForMaskedLM.from_composer` expects it (bert/src/bert_layers.py:
# 1087-1209) when `expand_positional_embeddings` is set: 12 layers, keys under `model.bert.`.  The function tiles the
# position table five times and stretches every `pos_emb.z` sixteen-fold, so the receiving model has 5 L0 positions
# and filters of 16 L0 steps.  Generated by make_golden.py into checkpoint_expand.npz.
CKPT = dict(seed=61, L0=16, D=8, emb=5, layers=12, pos_copies=5, z_factor=16)


def checkpoint_expand_inputs():
    """name -> array of the short model's entries the expansion touches."""
    c = CKPT
    sd = {"model.bert.embeddings.position_embeddings.weight": randn(c["seed"], "pe", (c["L0"], c["D"])),
          "model.bert.embeddings.position_ids": np.arange(c["L0"], dtype=np.int64)[None, :]}
    for i in range(c["layers"]):
        for fn in ("filter_fn", "filter_fn2"):
            p = f"model.bert.encoder.layer.{i}.attention.{fn}.pos_emb."
            sd[p + "z"] = randn(c["seed"], p + "z", (1, c["L0"], c["emb"]))
            sd[p + "t"] = np.linspace(0.0, 1.0, c["L0"], dtype=np.float32)[None, :, None]
    return sd
