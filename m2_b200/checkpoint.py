"""Checkpoint adapters for the drop-in modules: the key surgery the reference performs when it loads a
pretrained M2-BERT into a model with a longer maximum sequence length.

Reference: `from_composer` in bert/src/bert_layers.py:1087-1209 (prefix stripping, the
`expand_positional_embeddings` branch at :1119-1164) and `expand_8k_model_to_32k` in
bert/src/embeddings/training_functions.py:430-470.  Those functions are hard-wired to the published
checkpoints (12 layers, d_model 768, fixed tiling counts); the functions here take the target length
and reproduce the same three operations on any state dict of the m2_b200 / reference layout:

* `embeddings.position_embeddings.weight` (L0, D) is tiled along the position axis;
* every `attention.filter_fn{,2}.pos_emb.z` (1, L0, emb) becomes zeros of the new length with copies of
  the old tensor in consecutive slots of L0 positions starting at slot 1 (the reference's 8k -> 32k
  recipe fills slots 1, 2, 3 of 16 and leaves slot 0 zero);
* `pos_emb.t` and `embeddings.position_ids` are dropped, so the longer model keeps the time axis and ids
  its own constructor built (the reference deletes them and loads with strict=False).

As committed, `from_composer` stops at its own shape assertions for every checkpoint (it tiles the position table
five times and then asserts 32768 rows) and `expand_8k_model_to_32k` opens with a `breakpoint()`.  With `assert`
statements switched off (python -O) `from_composer` runs through: tests/golden/checkpoint_expand.npz holds what it
loads into a model from a fabricated short checkpoint -- five copies of the position table, `pos_emb.z` sixteen
times as long with copies in slots 1, 2, 3 -- and the adapters here are held to those tensors bit for bit.
"""
from __future__ import annotations

import re

import torch

_Z_KEY = re.compile(r"(^|\.)attention\.filter_fn2?\.pos_emb\.z$")
_T_KEY = re.compile(r"(^|\.)attention\.filter_fn2?\.pos_emb\.t$")


def strip_prefix(state_dict, prefixes=("model.bert.", "model.", "bert.")):
    """Keys without the wrapper prefixes a Composer / HuggingFace checkpoint carries
    (bert_layers.py:1186-1200 consumes `model.` and `bert.`).  The first matching prefix is removed."""
    out = {}
    for k, v in state_dict.items():
        for p in prefixes:
            if k.startswith(p):
                k = k[len(p):]
                break
        out[k] = v
    return out


def expand_sequence_length(state_dict, new_len, *, position_len=None, z_first_slot=1, z_copies=3):
    """A copy of `state_dict` stretched to sequences of `new_len` positions (see the module docstring).

    position_len: rows of the tiled position table when they differ from `new_len` (the reference tiles the table
    five times while it stretches the filters sixteen-fold); default `new_len`.

    z_first_slot / z_copies: which slots of the old length receive a copy of `pos_emb.z`; copies that
    would fall outside the new length are dropped.  Tensors that already have `new_len` positions are
    left alone; a `new_len` that is not a multiple of the old length raises ValueError.
    """
    new_len = int(new_len)
    position_len = new_len if position_len is None else int(position_len)
    out = {}
    for k, v in state_dict.items():
        if _T_KEY.search(k) or k.endswith("embeddings.position_ids"):
            continue                                           # rebuilt by the longer model's constructor
        if k.endswith("embeddings.position_embeddings.weight"):
            l0 = v.shape[0]
            if l0 != position_len:
                if position_len % l0:
                    raise ValueError(f"{k}: new length {position_len} is not a multiple of {l0}")
                v = v.repeat(position_len // l0, 1)
        elif _Z_KEY.search(k):
            l0 = v.shape[1]
            if l0 != new_len:
                if new_len % l0:
                    raise ValueError(f"{k}: new length {new_len} is not a multiple of {l0}")
                z = torch.zeros((v.shape[0], new_len, v.shape[2]), dtype=v.dtype, device=v.device)
                for slot in range(z_first_slot, z_first_slot + z_copies):
                    if (slot + 1) * l0 <= new_len:
                        z[:, slot * l0:(slot + 1) * l0] = v
                v = z
        out[k] = v
    return out


def load_expanded(model, state_dict):
    """model.load_state_dict(..., strict=False) that accepts only the keys `expand_sequence_length`
    drops as missing; anything else missing or unexpected raises, as a strict load would."""
    res = model.load_state_dict(state_dict, strict=False)
    bad = [k for k in res.missing_keys if not (_T_KEY.search(k) or k.endswith("position_ids"))]
    if bad or res.unexpected_keys:
        raise RuntimeError(f"load_expanded: missing keys {bad}, unexpected keys {list(res.unexpected_keys)}")
    return res
