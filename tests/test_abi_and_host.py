"""CPU-side checks: the C-ABI library loads and exports what the header declares, the
modules keep the reference's state_dict layout, argument errors come back as status codes,
and the sharding helpers partition correctly (including a 2-rank gloo run)."""
import ctypes as C
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

import m2_b200
from m2_b200 import _lib, sharding
from m2_b200.encoder import M2BertConfig, M2BertModel
from tests.golden import cases as CS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "m2_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(m2_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    lib = _lib.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/m2_b200.h but not exported"
    assert declared == set(_lib.SYMBOLS), (declared ^ set(_lib.SYMBOLS))
    assert lib.m2_version() == _lib.ABI_VERSION


def test_argument_errors_are_status_codes():
    lib = _lib.lib()
    assert lib.m2_hyena_filter(None, None) == 1
    assert b"NULL" in lib.m2_last_error()
    a = _lib.LongconvArgs()
    a.batch, a.seq_len, a.d_model, a.n_filters = 1, 8, 4, 3
    assert lib.m2_longconv_fwd(C.byref(a), None) == 1
    assert b"n_filters" in lib.m2_last_error()
    g = _lib.GluArgs()
    g.m, g.d_model, g.inter, g.nblocks = 4, 12, 24, 3
    assert lib.m2_blockdiag_glu_fwd(C.byref(g), None) == 2
    assert lib.m2_filter_row_len(128) == 256 and lib.m2_filter_row_len(100) == 256
    assert lib.m2_filter_row_len(1) == 4


def test_state_dict_layout_matches_reference():
    layout = json.load(open(os.path.join(ROOT, "tests", "golden", "state_dict_layout.json")))
    m = m2_b200.MonarchMixerSequenceMixing(768, l_max=128, bidirectional=True, hyena_emb_dim=5,
                                           hyena_filter_order=128, residual_long_conv=True)
    got = {k: list(v.shape) for k, v in m.state_dict().items()}
    assert got == layout["mixer"]
    # the six Sin slots of both nets share one frequency tensor
    f = m.filter_fn
    assert f.implicit_filter[1] is f.implicit_filter[5] is f.implicit_filter_rev[3]
    assert [n for n, _ in m.named_parameters() if n.endswith("freq")] == layout["mixer_freq_params"]
    assert {n for n, _ in m.named_buffers()} == set(layout["mixer_buffers"])
    conf = M2BertConfig(num_hidden_layers=1)
    mlp = m2_b200.BertGatedLinearUnitMLP(conf)
    assert {k: list(v.shape) for k, v in mlp.state_dict().items()} == layout["glu"]
    lin = m2_b200.BlockdiagLinear(30, 50, nblocks=4)
    assert {k: list(v.shape) for k, v in lin.state_dict().items()} == layout["blockdiag_30_50"]
    assert (lin.in_features_extended, lin.out_features_extended) == (32, 52)
    assert hasattr(f.implicit_filter[0].weight, "_optim") and hasattr(f.pos_emb.z, "_optim")


def test_blockdiag_init_matches_reference_construction():
    """Kaiming-uniform on the dense matrix scaled by sqrt(nblocks): bound check."""
    lin = m2_b200.BlockdiagLinear(768, 6144, bias=False, nblocks=4)
    bound = (4 ** 0.5) / (768 ** 0.5)
    assert lin.weight.abs().max() <= bound * 1.0001
    assert lin.weight.abs().max() > 0.9 * bound


def test_encoder_accepts_reference_keys():
    conf = M2BertConfig(num_hidden_layers=2, vocab_size=512, hidden_size=64, intermediate_size=256,
                        max_position_embeddings=32, long_conv_l_max=32, hyena_filter_order=32)
    model = M2BertModel(conf)
    sd = CS.encoder_state(41, 2, 64, 256, 32, vocab=512, order=32)
    missing, unexpected = model.load_state_dict(
        {k: torch.from_numpy(np.asarray(v)) for k, v in sd.items()}, strict=False)
    assert not unexpected and all("position_ids" in k for k in missing)


def test_no_cpu_fallback():
    m = m2_b200.MonarchMixerSequenceMixing(16, l_max=8, bidirectional=True, hyena_emb_dim=3,
                                           hyena_filter_order=16).eval()
    with torch.no_grad(), pytest.raises(RuntimeError, match="CUDA"):
        m(torch.zeros(1, 8, 16))
    lin = m2_b200.BlockdiagLinear(16, 16)
    with torch.no_grad(), pytest.raises(RuntimeError, match="CUDA"):
        lin(torch.zeros(2, 16))


def test_shard_ranges_cover_exactly():
    for n in (0, 1, 7, 8, 256, 768):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def test_channel_shard_state_reassembles_the_oracle():
    """Running the un-mixed middle of the mixer per channel shard and concatenating equals
    running it whole (checked with the numpy oracle: pure host logic)."""
    from oracle import m2_oracle as O
    D, L, B = 24, 16, 2
    sd = CS.mixer_state(3, D, L, 5, 16, 10, True, True)
    u = CS.randn(3, "u", (B, L, D))
    xin = O._linear(u, sd["in_linear.weight"], sd["in_linear.bias"], "fp64")
    whole = O.mixer_core(xin, u, sd, bidirectional=True, residual_long_conv=True)
    parts = []
    for r in range(3):
        lo, hi = sharding.shard_range(D, r, 3)
        sub = sharding.mixer_channel_shard_state({k: torch.from_numpy(np.asarray(v)) for k, v in sd.items()}, D, lo, hi)
        sub = {k: v.numpy() for k, v in sub.items()}
        assert "out_linear.weight" not in sub
        xin_r = O._linear(u, sub["in_linear.weight"], sub["in_linear.bias"], "fp64")
        parts.append(O.mixer_core(xin_r, u[..., lo:hi], sub, bidirectional=True, residual_long_conv=True))
    assert np.max(np.abs(np.concatenate(parts, axis=-1) - whole)) < 1e-12


_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from m2_b200 import sharding
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}",
                        rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
full = torch.arange(6 * 4 * 8, dtype=torch.float32).reshape(6, 4, 8)
mine = sharding.shard_batch(full, rank, 2) * 2.0          # each rank works on its rows only
out = sharding.gather_batch(mine)
assert torch.equal(out, full * 2.0)
lo, hi = sharding.shard_range(8, rank, 2)
outc = sharding.gather_channels(full[..., lo:hi] + 1.0)
assert torch.equal(outc, full + 1.0)
dist.barrier(); dist.destroy_process_group()
print("ok", rank)
"""


def test_two_rank_gloo_shard_and_gather(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = str(29500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("ok" in o for o in outs)


# ---- checkpoint adapters (longer maximum sequence length) -----------------------------------
def test_expand_sequence_length_roundtrip_into_longer_model():
    import torch
    from m2_b200 import checkpoint
    from m2_b200.encoder import M2BertConfig, M2BertModel
    small = dict(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, hyena_filter_order=8,
                 hyena_emb_dim=5, monarch_mlp_nblocks=4)
    torch.manual_seed(0)
    src = M2BertModel(M2BertConfig(max_position_embeddings=16, long_conv_l_max=16, **small))
    dst = M2BertModel(M2BertConfig(max_position_embeddings=64, long_conv_l_max=64, **small))
    sd = {"model.bert." + k: v.clone() for k, v in src.state_dict().items()}
    sd = checkpoint.strip_prefix(sd)
    assert set(sd) == set(src.state_dict())
    big = checkpoint.expand_sequence_length(sd, 64)
    # position embeddings: the old table repeated four times
    pe = big["embeddings.position_embeddings.weight"]
    assert pe.shape == (64, 32) and all(torch.equal(pe[16 * i:16 * (i + 1)], sd["embeddings.position_embeddings.weight"]) for i in range(4))
    z0 = sd["encoder.layer.1.attention.filter_fn2.pos_emb.z"]
    z = big["encoder.layer.1.attention.filter_fn2.pos_emb.z"]
    assert z.shape == (1, 64, 5) and bool((z[:, :16] == 0).all())           # slot 0 stays zero
    assert all(torch.equal(z[:, 16 * s:16 * (s + 1)], z0) for s in (1, 2, 3))
    assert not any(k.endswith("pos_emb.t") or k.endswith("position_ids") for k in big)
    before = dst.encoder.layer[0].attention.filter_fn.pos_emb.t.clone()
    res = checkpoint.load_expanded(dst, big)
    assert all(k.endswith("pos_emb.t") or k.endswith("position_ids") for k in res.missing_keys)
    assert torch.equal(dst.encoder.layer[0].attention.filter_fn.pos_emb.t, before)   # the longer model's own time axis
    assert torch.equal(dst.encoder.layer[0].attention.in_linear.weight, src.encoder.layer[0].attention.in_linear.weight)
    # a copy that does not fit is dropped, other lengths are rejected, wrong keys are loud
    z2 = checkpoint.expand_sequence_length(sd, 32)["encoder.layer.0.attention.filter_fn.pos_emb.z"]
    assert z2.shape == (1, 32, 5) and torch.equal(z2[:, 16:], sd["encoder.layer.0.attention.filter_fn.pos_emb.z"])
    with pytest.raises(ValueError):
        checkpoint.expand_sequence_length(sd, 40)
    big["encoder.layer.0.attention.nonsense"] = torch.zeros(1)
    with pytest.raises(RuntimeError):
        checkpoint.load_expanded(dst, big)


def test_expand_sequence_length_matches_the_reference_loader():
    """Bit-for-bit against what the reference's `BertForMaskedLM.from_composer` (bert/src/bert_layers.py:1087-1209,
    `expand_positional_embeddings`) loaded from the same fabricated short checkpoint
    (tests/golden/checkpoint_expand.npz, made by tests/golden/make_golden.py)."""
    import torch
    from m2_b200 import checkpoint
    from m2_b200.encoder import M2BertConfig, M2BertModel
    from tests.golden import cases as C
    c = C.CKPT
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "checkpoint_expand.npz"))
    sd = {k: torch.from_numpy(np.asarray(v)).clone() for k, v in C.checkpoint_expand_inputs().items()}
    big = checkpoint.expand_sequence_length(checkpoint.strip_prefix(sd, prefixes=("model.",)),
                                            c["z_factor"] * c["L0"], position_len=c["pos_copies"] * c["L0"])
    touched = [k for k in gold.files if k.endswith("position_embeddings.weight") or k.endswith("pos_emb.z")]
    assert len(touched) == 1 + 2 * c["layers"] and set(touched) == set(big)   # t and position_ids are dropped
    for k in touched:
        assert big[k].dtype == torch.float32 and big[k].shape == gold[k].shape, k
        assert np.array_equal(big[k].numpy(), gold[k]), k
    # loaded into the longer drop-in model, the untouched entries are the constructor's own, as in the reference
    torch.manual_seed(0)
    dst = M2BertModel(M2BertConfig(vocab_size=64, hidden_size=c["D"], intermediate_size=16, num_hidden_layers=c["layers"],
                                   hyena_filter_order=16, hyena_emb_dim=c["emb"], monarch_mlp_nblocks=4,
                                   max_position_embeddings=c["pos_copies"] * c["L0"],
                                   long_conv_l_max=c["z_factor"] * c["L0"]))
    part = {k[len("bert."):]: v for k, v in big.items()}
    res = dst.load_state_dict(part, strict=False)
    assert not res.unexpected_keys
    got = dst.state_dict()
    for k in gold.files:
        assert np.array_equal(got[k[len("bert."):]].numpy(), gold[k]), k


def test_flash_fft_attribute_protocol_is_accepted():
    """The reference's encoder pokes `flashfft` / `use_flash_fft` onto the filters
    (bert/src/bert_layers.py:616-626); the drop-in filters accept and ignore them."""
    from m2_b200 import HyenaFilter
    f = HyenaFilter(16, emb_dim=5, order=8, seq_len=32, bidirectional=True)
    assert f.flashfft is None and f.use_flash_fft is False
    f.flashfft, f.use_flash_fft = object(), True
    assert f.use_flash_fft is True


def test_pooler_and_embedder_staging():
    import torch
    from m2_b200.embed import M2BertEmbedder
    from m2_b200.encoder import M2BertConfig, M2BertModel, M2BertPooler
    cfg = M2BertConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, hyena_filter_order=8,
                       max_position_embeddings=16, long_conv_l_max=16, pool_all=True)
    pooler = M2BertPooler(cfg)
    h = torch.randn(3, 16, 32)
    m = torch.zeros(3, 16, dtype=torch.long)
    m[0, :5] = 1; m[1, :] = 1; m[2, :1] = 1
    ref = torch.tanh(pooler.dense(torch.stack([h[0, :5].mean(0), h[1].mean(0), h[2, :1].mean(0)])))
    assert torch.allclose(pooler(h, mask=m), ref, atol=1e-6)
    cfg.pool_all = False
    first = M2BertPooler(cfg)
    assert torch.allclose(first(h), torch.tanh(first.dense(h[:, 0])), atol=1e-6)
    model = M2BertModel(cfg, add_pooling_layer=True)
    assert {"pooler.dense.weight", "pooler.dense.bias"} <= set(model.state_dict())
    emb = M2BertEmbedder(model, max_len=16, batch_size=4)
    emb._fill([[5, 6, 7], list(range(1, 30))])                 # short text padded, long text cut
    assert emb._ids[0].tolist() == [5, 6, 7] + [cfg.pad_token_id] * 13 and emb._mask[0].tolist() == [1] * 3 + [0] * 13
    assert emb._ids[1].tolist() == list(range(1, 17)) and emb._mask[1].sum() == 16
    assert emb._mask[2].tolist() == [1] + [0] * 15             # empty rows keep a non-zero denominator
    with pytest.raises(ValueError):
        M2BertEmbedder(M2BertModel(cfg), max_len=16, batch_size=4)


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs the stock-op CPU path and prints one JSON line with the keys
    the measurement contract asks for (no GPU needed)."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=root)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "sequences/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["steps"] == 1 and line["n_gpus"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"]


def test_pooler_matches_reference_branches():
    """First token, masked mean and token planting against outputs of the reference's BertPooler
    (tests/golden/pooler.npz, written by make_golden.py), including the planting branch's in-place
    edit of the hidden states' first row."""
    from m2_b200.encoder import M2BertPooler
    gold = np.load(os.path.join(ROOT, "tests", "golden", "pooler.npz"))
    h, mask, w, b = CS.pooler_inputs()
    for name, kw in (("first", dict(pool_all=False, sequence_token_planting=False)),
                     ("mean", dict(pool_all=True, sequence_token_planting=False)),
                     ("planting", dict(pool_all=False, sequence_token_planting=True))):
        cfg = M2BertConfig(hidden_size=h.shape[-1], **kw)
        p = M2BertPooler(cfg).eval()
        with torch.no_grad():
            p.dense.weight.copy_(torch.from_numpy(w))
            p.dense.bias.copy_(torch.from_numpy(b))
            hs = torch.from_numpy(h).float().clone()
            out = p(hs, mask=torch.from_numpy(mask))
        assert np.allclose(out.numpy(), gold[name], atol=2e-6), name
        assert np.allclose(hs[:, 0].numpy(), gold[name + "_row0_after"], atol=2e-6), name


def test_forward_only_guard_runs_without_grad_and_warns_once():
    """With autograd on and parameters that require grad -- how the reference's own benchmark calls the
    modules -- the forward runs under no_grad instead of raising."""
    import warnings
    from m2_b200 import _tags

    class Probe(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.ones(2))

        @_tags.forward_only
        def forward(self, x):
            assert not torch.is_grad_enabled()
            return x * self.w

    _tags._warned = False
    m = Probe()
    with warnings.catch_warnings(record=True) as rec:
        warnings.simplefilter("always")
        y = m(torch.ones(2, requires_grad=True))
        m(torch.ones(2))
    assert not y.requires_grad
    assert len([r for r in rec if "forward-only" in str(r.message)]) == 1
    # the real modules reach the device check, not a forward-only error, when called with grad enabled
    mixer = m2_b200.MonarchMixerSequenceMixing(16, l_max=8, bidirectional=True, hyena_emb_dim=3, hyena_filter_order=16)
    with pytest.raises(RuntimeError, match="CUDA"):
        mixer(torch.zeros(1, 8, 16))


def test_copies_record_is_dropped_after_an_in_place_edit():
    from m2_b200 import _tags
    t = torch.zeros(2, 3)
    _tags.attach(t, bf16=torch.ones(2, 3, dtype=torch.bfloat16), src_dtype=torch.float32)
    assert _tags.copies_of(t) is not None
    t.add_(1.0)
    assert _tags.copies_of(t) is None and _tags.src_dtype_of(t) == torch.float32
    assert _tags.copies_of(torch.zeros(1)) is None
