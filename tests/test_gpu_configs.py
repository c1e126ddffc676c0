"""Parity at the shapes the benchmark configurations name (80M at L = 128 / 8192 / 32768, the large
shape at L = 128 / 2048), end to end: the package's own filter taps, GEMMs and convolution kernels
against the stock-op path (oracle/torch_oracle.py: cuBLAS, cuFFT and cuDNN under the same autocast),
whose taps are its own.  The path's tolerance (2e-2 on O.parity_error) is a statement per operator --
the mixer, the GLU MLP -- on the SAME input the stock-op path saw; a whole layer is the two in sequence
(the MLP re-mixes the mixer's legitimate bf16 rounding differences) and is held to twice that.  All tests
here need a B200."""
import numpy as np
import pytest
import torch

from m2_b200 import ops
from m2_b200.encoder import M2BertConfig, M2BertModel
from oracle import m2_oracle as O
from oracle import torch_oracle as T
from tests.golden import cases as C
from tests.helpers import to_torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_BF16 = 2e-2


@pytest.fixture(autouse=True)
def _no_grad_and_status():
    with torch.no_grad():
        yield
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    torch.cuda.empty_cache()


def err(got, ref):
    """O.parity_error on device tensors: max |got - ref| / (rms(ref) + |ref|)."""
    got, ref = got.float(), ref.float()
    rms = ref.pow(2).mean().sqrt()
    return float(((got - ref).abs() / (rms + ref.abs())).max())


def rel_rms(got, ref):
    got, ref = got.float(), ref.float()
    return float((got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())


def build(layers, D, I, L, seed, vocab=30528, order=128):
    conf = M2BertConfig(vocab_size=vocab, hidden_size=D, intermediate_size=I, num_hidden_layers=layers,
                        max_position_embeddings=L, long_conv_l_max=L, hyena_filter_order=order)
    model = M2BertModel(conf).eval()
    sd = C.encoder_state(seed, layers, D, I, L, vocab=vocab, order=order)
    missing, unexpected = model.load_state_dict(to_torch(sd), strict=False)
    assert not unexpected and all("position_ids" in k for k in missing)
    return model.to(DEV), to_torch(sd, DEV)


def check_layers(model, sdt, ids, want_kind, final_factor):
    """Per-layer parity on the stock-op path's own inputs, then the free-running model."""
    B, L = ids.shape
    D = model.config.hidden_size
    assert ops.longconv_kind_batch(B, L, torch.bfloat16, D) == want_kind
    worst = 0.0
    with torch.autocast("cuda", dtype=torch.bfloat16):
        h_ref = T.embeddings_forward(sdt, ids)
        assert err(model.embeddings(ids), h_ref) < 1e-5
        for i, layer in enumerate(model.encoder.layer):
            p = f"encoder.layer.{i}."
            a_ref = T.mixer_forward(sdt, h_ref, bidirectional=True, residual_long_conv=True, prefix=p + "attention.")
            nxt_ref = T.glu_mlp_forward(sdt, a_ref, prefix=p + "mlp.")
            a_own, _ = layer.attention(h_ref)
            e_mix, e_mlp, e_layer = err(a_own, a_ref), err(layer.mlp(a_ref), nxt_ref), err(layer(h_ref), nxt_ref)
            worst = max(worst, e_mix, e_mlp, e_layer)
            assert e_mix < TOL_BF16 and e_mlp < TOL_BF16 and e_layer < 2 * TOL_BF16, (i, e_mix, e_mlp, e_layer)
            del a_ref, a_own
            h_ref = nxt_ref
        y, _ = model(ids)
    # run free, each layer re-mixes the (legitimate) bf16 rounding differences of the layers before it
    assert err(y, h_ref) < final_factor * TOL_BF16 and rel_rms(y, h_ref) < TOL_BF16
    return worst


@pytest.mark.parametrize("L,B", [(8192, 2), (32768, 1)])
def test_80m_long_context_layers(L, B):
    """Configs 3 and 4 at their own d_model and length: two 80M-shaped layers through M2BertModel (the
    long-row host path: time-contiguous GEMM layouts, the LayerNorm's time-major hand-off, copies-only
    LayerNorm between layers) with ~10 % padding ids at the row ends, as the 8K config states."""
    model, sdt = build(2, 768, 3072, L, seed=61)
    rng = np.random.default_rng(L)
    ids = rng.integers(1, 30528, size=(B, L))
    for b in range(B):
        ids[b, L - int(0.1 * L * rng.uniform(0, 2)):] = 0          # pad_token_id
    check_layers(model, sdt, torch.from_numpy(ids).to(DEV), want_kind=2, final_factor=4)


@pytest.mark.parametrize("L,B,kind", [(128, 64, 3), (2048, 2, 2)])
def test_large_shape_layers(L, B, kind):
    """Config 5: d_model 1536, intermediate 6144 -- the Toeplitz family with half-filled batch tiles at
    L = 128, the long-row family at L = 2048, and the GLU / wo GEMMs at K = 384 / 1536 per block."""
    model, sdt = build(2, 1536, 6144, L, seed=62)
    ids = torch.from_numpy(np.random.default_rng(5).integers(0, 30528, size=(B, L))).to(DEV)
    check_layers(model, sdt, ids, want_kind=kind, final_factor=4)


def test_benchmark_graph_80m_b256_every_layer():
    """Config 2 exactly as bench.py runs it: 12 layers, batch 256, L = 128.  Every layer against the stock-op
    path on the same input; then the captured graph against the eager forward, bit for bit."""
    from m2_b200 import GraphedForward
    model, sdt = build(12, 768, 3072, 128, seed=63)
    ids = torch.from_numpy(np.random.default_rng(6).integers(0, 30528, size=(256, 128))).to(DEV)
    check_layers(model, sdt, ids, want_kind=3, final_factor=12)
    graphed = GraphedForward(model, ids)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        want, _ = model(ids)
    got, _ = graphed(ids)
    assert torch.equal(got, want)


def test_mixer_only_32k_batch8_rows_are_independent():
    """Config 4's mixer-only input, u ~ N(0, 1) at (8, 32768, 768): sequence 0 and 7 of the batched call
    equal the same sequences run alone (bit for bit), and sequence 0 matches the stock-op path."""
    model, sdt = build(1, 768, 3072, 32768, seed=64)
    mixer = model.encoder.layer[0].attention
    g = torch.Generator(device="cpu").manual_seed(9)
    u = torch.randn((8, 32768, 768), generator=g).to(DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y, _ = mixer(u)
        for b in (0, 7):
            yb, _ = mixer(u[b:b + 1])
            assert torch.equal(yb[0], y[b])
        ref = T.mixer_forward(sdt, u[:1], bidirectional=True, residual_long_conv=True,
                              prefix="encoder.layer.0.attention.")
    assert err(y[:1], ref) < TOL_BF16


def test_channel_shards_reassemble_the_mixer():
    """The d_model-channel sharding of config 4, on one GPU: shards of the un-mixed middle of the mixer,
    concatenated, equal the un-sharded tensor bit for bit; out_linear of it equals the mixer's forward."""
    from m2_b200 import sharding
    L, D = 8192, 768
    model, sdt = build(1, D, 3072, L, seed=65)
    mixer = model.encoder.layer[0].attention
    u = torch.randn((2, L, D), generator=torch.Generator(device="cpu").manual_seed(10)).to(DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        whole = mixer.forward_channels(u, 0, D).clone()
        parts = []
        for r in range(8):
            lo, hi = sharding.shard_range(D, r, 8)
            parts.append(mixer.forward_channels(u, lo, hi).clone())
        assert torch.equal(torch.cat(parts, dim=-1), whole)
        y, _ = mixer(u)
        w_out = mixer.out_linear.weight.detach().bfloat16().contiguous()
        assert torch.equal(ops.linear_fwd(whole.contiguous(), w_out, mixer.out_linear.bias), y)


_SHARD_WORKER = r"""
import os, sys, torch, torch.distributed as dist
root, port, rank, world = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4])
sys.path.insert(0, root)
os.environ["NCCL_NVLS_ENABLE"] = "0"
torch.cuda.set_device(rank)
dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                        device_id=torch.device("cuda", rank))
from m2_b200 import sharding
from tests.test_gpu_configs import build
import tests.test_gpu_configs as T
T.DEV = f"cuda:{rank}"
L, D = 4096, 768
model, _ = build(1, D, 3072, L, seed=66)
mixer = model.encoder.layer[0].attention
u = torch.randn((2, L, D), generator=torch.Generator(device="cpu").manual_seed(11)).to(T.DEV)
lo, hi = sharding.shard_range(D, rank, world)
with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
    mine = mixer.forward_channels(u, lo, hi).contiguous()
    gathered = sharding.gather_channels(mine)
    whole = mixer.forward_channels(u, 0, D)
assert torch.equal(gathered, whole), "gathered channel shards differ from the single-GPU tensor"
torch.cuda.synchronize()
dist.barrier(); dist.destroy_process_group()
print("ok", rank)
"""


def test_channel_shards_over_two_gpus_gathered_with_nccl(tmp_path):
    """Rank r computes channels [r D/2, (r+1) D/2) of the full batch on its own GPU; an NCCL all-gather (the
    only collective, for verification) reassembles them; equal to the single-GPU tensor."""
    import os
    import subprocess
    import sys
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "shard_worker.py"
    script.write_text(_SHARD_WORKER)
    port = str(29700 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), root, port, str(r), "2"],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
