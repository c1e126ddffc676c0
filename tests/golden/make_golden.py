"""Generate the parity fixtures in this directory by running the REFERENCE on CPU.

Usage (only where the reference checkout is mounted):

    python -m tests.golden.make_golden /path/to/reference

(the checkpoint-expansion fixture is made by a child interpreter this command starts, see
``run_checkpoint_expand``)

The reference's modules are imported in place with two shims (a stub ``opt_einsum``,
whose ``contract`` the path binds but never calls, and a bare ``src`` package so that
``bert/src/__init__.py`` -- which needs MosaicML Composer -- is skipped).  Weights and
inputs come from ``cases.py``; for every case the reference is run in float64, float32
and under ``torch.autocast("cpu", bfloat16)`` and a deterministic subsample of each
output is stored in ``<case>.npz``.  Nothing of the reference's source is copied.
"""
from __future__ import annotations

import contextlib
import io
import os
import sys
import types

import numpy as np
import torch

from tests.golden import cases as C


def import_reference(ref_root):
    bert = os.path.join(ref_root, "bert")
    if "opt_einsum" not in sys.modules:
        m = types.ModuleType("opt_einsum")
        m.contract = None
        sys.modules["opt_einsum"] = m
    pkg = types.ModuleType("src")
    pkg.__path__ = [os.path.join(bert, "src")]
    sys.modules["src"] = pkg
    for p in (bert, os.path.join(bert, "src")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from src.mm.monarch_mixer_sequence_mixer import MonarchMixerSequenceMixing
    from src.mm.blockdiag_linear import BlockdiagLinear
    import src.bert_layers as bert_layers
    from src.configuration_bert import BertConfig
    return MonarchMixerSequenceMixing, BlockdiagLinear, bert_layers, BertConfig


def _load(module, sd):
    t = {k: torch.from_numpy(np.asarray(v)) for k, v in sd.items()}
    missing, unexpected = module.load_state_dict(t, strict=False)
    missing = [m for m in missing if "position_ids" not in m and "pooler" not in m]
    assert not missing and not unexpected, (missing, unexpected)


class _LayerNormFp32(torch.nn.Module):
    """LayerNorm as CUDA autocast runs it: float32 arithmetic on the upcast input."""

    def __init__(self, ln):
        super().__init__()
        self.ln = ln.float()

    def forward(self, x):
        return self.ln(x.float())


def _modes(fn, module, *inputs, bf16="autocast"):
    """fn(module, *tensors) in float64, float32 and bfloat16.

    bf16="autocast": under torch.autocast("cpu", bfloat16) -- the same cast policy as the
    CUDA autocast the reference benchmarks under, for the ops the mixer uses.
    bf16="cast": module and inputs converted to bfloat16.  BlockdiagMultiply casts its
    inputs to bfloat16 only under *CUDA* autocast (torch.cuda.amp.custom_fwd,
    bert/src/mm/blockdiag_multiply.py:50), which cannot be entered without a GPU;
    converting the operands by hand runs the same reference code on the same dtypes.
    bf16=None: no bfloat16 run.
    """
    out = {}
    with torch.no_grad():
        m64 = module.double()
        out["fp64"] = fn(m64, *[i.double() if i.is_floating_point() else i for i in inputs])
        m32 = module.float()
        out["fp32"] = fn(m32, *inputs)
        if bf16 == "autocast":
            with torch.autocast("cpu", dtype=torch.bfloat16):
                out["bf16"] = fn(m32, *inputs)
        elif bf16 == "cast":
            mb = module.bfloat16()
            if hasattr(mb, "layernorm"):
                mb.layernorm = _LayerNormFp32(mb.layernorm)
            out["bf16"] = fn(mb, *[i.bfloat16() if i.is_floating_point() else i for i in inputs])
    return out


def run_case(name, cfg, ref):
    Mixer, Blockdiag, bert_layers, BertConfig = ref
    kind, seed = cfg["kind"], cfg["seed"]
    store = {}

    def put(key, tensor):
        a = tensor.detach().to(torch.float64).numpy()
        store[key] = C.subsample(a).astype(np.float32 if "fp64" not in key else np.float64)

    if kind == "mixer":
        l_max = cfg.get("l_max", cfg["L"])
        with contextlib.redirect_stdout(io.StringIO()):
            m = Mixer(cfg["D"], l_max=l_max, bidirectional=cfg["bidirectional"],
                      hyena_emb_dim=cfg["emb"], hyena_filter_order=cfg["order"],
                      hyena_w=cfg["w"], residual_long_conv=cfg["residual"],
                      hyena_kernel_lr=1e-3, hyena_lr_pos_emb=1e-5).eval()
        sd = C.mixer_state(seed, cfg["D"], l_max, cfg["emb"], cfg["order"], cfg["w"],
                           cfg["bidirectional"], cfg["residual"])
        _load(m, sd)
        u = torch.from_numpy(C.randn(seed, "u", (cfg["B"], cfg["L"], cfg["D"])))
        for mode, y in _modes(lambda mod, x: mod(x)[0], m, u).items():
            put(f"out_{mode}", y)
        L = cfg["L"]
        filt = _modes(lambda mod: torch.stack(
            [mod.filter_fn.filter(L)[0]] +
            ([mod.filter_fn.filter_rev(L)[0]] if cfg["bidirectional"] else [])), m)
        for mode, k in filt.items():
            put(f"filter_{mode}", k)
    elif kind == "blockdiag":
        m = Blockdiag(cfg["inf"], cfg["outf"], bias=cfg["bias"], nblocks=cfg["nb"]).eval()
        sd = {"weight": C.blockdiag_weight(seed, "weight", cfg["inf"], cfg["outf"], cfg["nb"])}
        if cfg["bias"]:
            sd["bias"] = C.randn(seed, "bias", (cfg["outf"],))
        _load(m, sd)
        x = torch.from_numpy(C.randn(seed, "x", (cfg["M"], cfg["inf"])))
        for mode, y in _modes(lambda mod, a: mod(a), m, x, bf16="cast").items():
            put(f"out_{mode}", y)
    elif kind == "glu":
        conf = BertConfig(hidden_size=cfg["D"], intermediate_size=cfg["I"], use_glu_mlp=True,
                          use_monarch_mlp=True, monarch_mlp_nblocks=cfg["nb"],
                          monarch_mixer_sequence_mixing=True, hidden_dropout_prob=0.1)
        m = bert_layers.BertGatedLinearUnitMLP(conf).eval()
        _load(m, C.mlp_state(seed, cfg["D"], cfg["I"], cfg["nb"]))
        x = torch.from_numpy(C.randn(seed, "x", (cfg["B"], cfg["L"], cfg["D"])))
        for mode, y in _modes(lambda mod, a: mod(a), m, x, bf16="cast").items():
            put(f"out_{mode}", y)
    elif kind == "encoder":
        conf = BertConfig(vocab_size=cfg["vocab"], hidden_size=cfg["D"],
                          intermediate_size=cfg["I"], num_hidden_layers=cfg["layers"],
                          num_attention_heads=4, max_position_embeddings=cfg["L"],
                          use_glu_mlp=True, use_monarch_mlp=True, monarch_mlp_nblocks=4,
                          monarch_mixer_sequence_mixing=True, residual_long_conv=True,
                          bidirectional=True, use_positional_encodings=True,
                          hyena_filter_order=cfg["order"], hyena_emb_dim=5, hyena_w=10,
                          hyena_wd=0.1, hyena_lr_pos_emb=1e-5, long_conv_l_max=cfg["L"],
                          long_conv_kernel_learning_rate=1e-3, hyena_filter_dropout=0.0,
                          hyena_training_additions=False)
        with contextlib.redirect_stdout(io.StringIO()):
            m = bert_layers.BertModel(conf, add_pooling_layer=False).eval()
        _load(m, C.encoder_state(seed, cfg["layers"], cfg["D"], cfg["I"], cfg["L"],
                                 vocab=cfg["vocab"], order=cfg["order"]))
        ids = np.random.default_rng(seed).integers(0, cfg["vocab"], size=(cfg["B"], cfg["L"]))
        ids_t = torch.from_numpy(ids)
        for mode, y in _modes(lambda mod, a: mod(a)[0], m, ids_t, bf16=None).items():
            put(f"out_{mode}", y)
    else:
        raise ValueError(kind)
    return store


def dump_layout(ref, path):
    """Names and shapes of the reference modules' state_dicts (drop-in contract)."""
    import json
    Mixer, Blockdiag, bert_layers, BertConfig = ref
    with contextlib.redirect_stdout(io.StringIO()):
        m = Mixer(768, l_max=128, bidirectional=True, hyena_emb_dim=5, hyena_filter_order=128,
                  residual_long_conv=True)
        conf = BertConfig(hidden_size=768, intermediate_size=3072, use_glu_mlp=True,
                          use_monarch_mlp=True, monarch_mlp_nblocks=4,
                          monarch_mixer_sequence_mixing=True)
        mlp = bert_layers.BertGatedLinearUnitMLP(conf)
        lin = Blockdiag(30, 50, nblocks=4)
    shapes = lambda mod: {k: list(v.shape) for k, v in mod.state_dict().items()}
    layout = {
        "mixer": shapes(m),
        "mixer_freq_params": [n for n, _ in m.named_parameters() if n.endswith("freq")],
        "mixer_buffers": [n for n, _ in m.named_buffers()],
        "glu": shapes(mlp),
        "blockdiag_30_50": shapes(lin),
    }
    with open(path, "w") as f:
        json.dump(layout, f, indent=1, sort_keys=True)


def run_pooler(ref):
    """The three branches of the reference's BertPooler on the inputs of cases.pooler_inputs()."""
    _, _, bert_layers, _ = ref
    h, mask, w, b = C.pooler_inputs()
    store = {}
    for name, kw in (("first", dict(pool_all=False, sequence_token_planting=False)),
                     ("mean", dict(pool_all=True, sequence_token_planting=False)),
                     ("planting", dict(pool_all=False, sequence_token_planting=True))):
        conf = types.SimpleNamespace(hidden_size=h.shape[-1], use_cls_token=True, **kw)
        m = bert_layers.BertPooler(conf).eval()
        with torch.no_grad():
            m.dense.weight.copy_(torch.from_numpy(w))
            m.dense.bias.copy_(torch.from_numpy(b))
            hs = torch.from_numpy(h).float().clone()
            out = m(hs, mask=torch.from_numpy(mask))
        store[name] = out.numpy()
        store[name + "_row0_after"] = hs[:, 0].numpy()      # the planting branch edits the hidden states in place
    return store


def run_checkpoint_expand(ref):
    """The reference's `BertForMaskedLM.from_composer` with `expand_positional_embeddings` on the fabricated short
    checkpoint of cases.checkpoint_expand_inputs().  As committed the function stops at its own shape assertions for
    every input (five copies of a position table never make the 32768 rows it asserts), so this runs in a child
    interpreter started with -O, which drops `assert` statements and leaves the rest of the reference untouched."""
    import tempfile
    _, _, bert_layers, BertConfig = ref
    c = C.CKPT
    sd = {k: torch.from_numpy(np.asarray(v)).clone() for k, v in C.checkpoint_expand_inputs().items()}
    conf = BertConfig(vocab_size=64, hidden_size=c["D"], intermediate_size=16, num_hidden_layers=c["layers"],
                      num_attention_heads=4, max_position_embeddings=c["pos_copies"] * c["L0"],
                      use_glu_mlp=True, use_monarch_mlp=True, monarch_mlp_nblocks=4,
                      monarch_mixer_sequence_mixing=True, residual_long_conv=True,
                      bidirectional=True, use_positional_encodings=True,
                      hyena_filter_order=16, hyena_emb_dim=c["emb"], hyena_w=10,
                      hyena_wd=0.1, hyena_lr_pos_emb=1e-5, long_conv_l_max=c["z_factor"] * c["L0"],
                      long_conv_kernel_learning_rate=1e-3, hyena_filter_dropout=0.0,
                      hyena_training_additions=False, expand_positional_embeddings=True)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "short_model.pt")
        torch.save({"state": {"model": sd}}, path)
        with contextlib.redirect_stdout(io.StringIO()):
            torch.manual_seed(0)
            fresh = bert_layers.BertForMaskedLM(conf).state_dict()
            model = bert_layers.BertForMaskedLM.from_composer(path, config=conf)
    loaded = model.state_dict()
    store = {}
    for k, v in loaded.items():
        if k.endswith("position_embeddings.weight") or k.endswith("pos_emb.z"):
            store[k] = v.numpy()
    # the time axis and the position ids stay the longer model's own: the same as a freshly built model has
    for k in ("bert.encoder.layer.0.attention.filter_fn.pos_emb.t", "bert.encoder.layer.11.attention.filter_fn2.pos_emb.t",
              "bert.embeddings.position_ids"):
        if not torch.equal(loaded[k], fresh[k]):               # (`assert` is off in this interpreter)
            raise RuntimeError(k + ": differs from the freshly built model's")
        store[k] = loaded[k].numpy()
    return store


def main():
    if len(sys.argv) >= 3 and sys.argv[1] == "--checkpoint-expand":
        if __debug__:
            sys.exit("--checkpoint-expand needs an interpreter started with -O")
        here = os.path.dirname(os.path.abspath(__file__))
        store = run_checkpoint_expand(import_reference(sys.argv[2]))
        np.savez_compressed(os.path.join(here, "checkpoint_expand.npz"), **store)
        print("checkpoint_expand", len(store), "arrays")
        return
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of HazyResearch/m2>")
    ref_root = sys.argv[1]
    ref = import_reference(ref_root)
    here = os.path.dirname(os.path.abspath(__file__))
    dump_layout(ref, os.path.join(here, "state_dict_layout.json"))
    torch.manual_seed(0)
    for name, cfg in C.CASES.items():
        store = run_case(name, cfg, ref)
        np.savez_compressed(os.path.join(here, name + ".npz"), **store)
        print(name, {k: v.shape for k, v in store.items()})
    store = run_pooler(ref)
    np.savez_compressed(os.path.join(here, "pooler.npz"), **store)
    print("pooler", {k: v.shape for k, v in store.items()})
    import subprocess
    subprocess.run([sys.executable, "-O", "-m", "tests.golden.make_golden", "--checkpoint-expand", ref_root], check=True)


if __name__ == "__main__":
    main()
