"""Shared by the GPU parity tests: build the package's modules from the seeded state
dicts of tests/golden/cases.py."""
import numpy as np
import torch

import m2_b200
from tests.golden import cases as C


def to_torch(sd, device="cpu", dtype=torch.float32):
    return {k: torch.from_numpy(np.asarray(v)).to(device=device, dtype=dtype) for k, v in sd.items()}


def build_mixer(cfg, device):
    l_max = cfg.get("l_max", cfg["L"])
    m = m2_b200.MonarchMixerSequenceMixing(
        cfg["D"], l_max=l_max, bidirectional=cfg["bidirectional"], hyena_emb_dim=cfg["emb"],
        hyena_filter_order=cfg["order"], hyena_w=cfg["w"], residual_long_conv=cfg["residual"],
        hyena_kernel_lr=1e-3, hyena_lr_pos_emb=1e-5).eval()
    sd = C.mixer_state(cfg["seed"], cfg["D"], l_max, cfg["emb"], cfg["order"], cfg["w"],
                       cfg["bidirectional"], cfg["residual"])
    missing, unexpected = m.load_state_dict(to_torch(sd), strict=True)
    return m.to(device), sd


class Cfg:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def build_glu(cfg, device):
    conf = Cfg(hidden_size=cfg["D"], intermediate_size=cfg["I"], monarch_mlp_nblocks=cfg["nb"],
               layer_norm_eps=1e-12, hidden_dropout_prob=0.1, use_monarch_mlp=True,
               monarch_mixer_sequence_mixing=True)
    m = m2_b200.BertGatedLinearUnitMLP(conf).eval()
    sd = C.mlp_state(cfg["seed"], cfg["D"], cfg["I"], cfg["nb"])
    m.load_state_dict(to_torch(sd), strict=True)
    return m.to(device), sd
