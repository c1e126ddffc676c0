"""The modules as a caller of the reference would use them: with autograd left on, inside a
BertLayer-shaped wrapper, with hidden states edited in place between layers, with several captured
graphs alive, with ids outside the embedding tables -- and the failure path of the bounded device
waits.  All tests here need a B200; none faults, traps or hangs the GPU."""
import ctypes

import numpy as np
import pytest
import torch
import torch.nn as nn

import m2_b200
from m2_b200 import _lib, ops
from m2_b200.encoder import M2BertConfig, M2BertModel
from oracle import m2_oracle as O
from tests.golden import cases as C
from tests.helpers import build_mixer, to_torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def small_model(B_hint=64, L=128, D=256, I=1024, layers=2, seed=44, vocab=1000):
    conf = M2BertConfig(vocab_size=vocab, hidden_size=D, intermediate_size=I, num_hidden_layers=layers,
                        max_position_embeddings=L, long_conv_l_max=L, hyena_filter_order=32)
    model = M2BertModel(conf).eval()
    sd = C.encoder_state(seed, layers, D, I, L, vocab=vocab, order=32)
    model.load_state_dict(to_torch(sd), strict=False)
    return model.to(DEV)


class ReferenceShapedLayer(nn.Module):
    """The control flow of the reference's BertLayer.forward on the Monarch-Mixer branch
    (bert/src/bert_layers.py:552-599): anomaly-detection contexts, tuple unpacking, NaN checks."""

    def __init__(self, layer):
        super().__init__()
        self.attention, self.mlp = layer.attention, layer.mlp

    def forward(self, hidden_states, cu_seqlens=None, seqlen=None, subset_idx=None, indices=None, attn_mask=None, bias=None):
        with torch.autograd.set_detect_anomaly(True):
            attention_output = self.attention(hidden_states)
            if type(attention_output) == tuple:
                attention_output, _ = attention_output
        if torch.isnan(attention_output).any():
            raise ValueError()
        with torch.autograd.set_detect_anomaly(True):
            layer_output = self.mlp(attention_output)
        if torch.isnan(layer_output).any():
            raise ValueError()
        return layer_output


def test_reference_shaped_layer_with_autograd_enabled():
    """Called the way bert/benchmark_fwd.py:70-75 calls the encoder -- grad mode on, parameters requiring
    grad, under autocast -- the layer runs and returns what the no_grad call returns."""
    model = small_model()
    layer = ReferenceShapedLayer(model.encoder.layer[0])
    assert any(p.requires_grad for p in layer.parameters())
    u = torch.randn(64, 128, 256, device=DEV)
    mask = torch.ones(64, 128, dtype=torch.int64, device=DEV)
    m2_b200._tags._warned = False
    with pytest.warns(RuntimeWarning, match="forward-only"):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            assert torch.is_grad_enabled()
            out = layer(u, None, 128, None, None, mask)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        want = model.encoder.layer[0](u)
    assert not out.requires_grad and torch.equal(out, want)
    # float32 mode the same way
    out32 = layer(u[:2], attn_mask=mask[:2])
    with torch.no_grad():
        assert torch.equal(out32, model.encoder.layer[0](u[:2]))
    assert ops.device_status() == 0


@pytest.mark.parametrize("copies_only", [False, True])
@pytest.mark.parametrize("B", [4, 64])
def test_in_place_edit_between_layers_is_seen(B, copies_only):
    """A LayerNorm hands the next mixer copies of its output; after an in-place edit of the hidden state
    the copies no longer describe it and the mixer must read the edited tensor."""
    model = small_model()
    l0, l1 = model.encoder.layer
    u = torch.randn(B, 128, 256, device=DEV)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        h = l0(u, copies_only=copies_only)
        assert m2_b200._tags.copies_of(h) is not None
        untouched = l1(h).clone()
        h.mul_(0.5)
        assert m2_b200._tags.copies_of(h) is None
        edited = l1(h)
        # a tensor that never carried copies; it keeps only the note of which dtype the reference's hidden
        # state has at this point (float32: the bf16 tensor of the copies-only mode stands in for it)
        fresh = l1(m2_b200._tags.attach(h.clone(), src_dtype=m2_b200._tags.src_dtype_of(h)))
    assert torch.equal(edited, fresh)
    assert not torch.equal(edited, untouched)
    assert ops.device_status() == 0


def test_two_graphs_and_an_eager_call_do_not_share_buffers():
    """Capture at one batch size, run eagerly and capture again at another, then replay the first graph:
    its convolution output buffer must still be its own."""
    from m2_b200 import GraphedForward
    model = small_model()
    rng = np.random.default_rng(3)
    ids_a = torch.from_numpy(rng.integers(0, 1000, size=(64, 128))).to(DEV)
    ids_b = torch.from_numpy(rng.integers(0, 1000, size=(128, 128))).to(DEV)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        want_a = model(ids_a)[0].clone()
    g_a = GraphedForward(model, ids_a)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        want_b = model(ids_b)[0].clone()                    # eager call at another batch size
    g_b = GraphedForward(model, ids_b)
    filler = [torch.randn(64 * 128 * 256, device=DEV) for _ in range(4)]   # lands in whatever the allocator freed
    got_a = g_a(ids_a)[0].clone()
    got_b = g_b(ids_b)[0].clone()
    torch.cuda.synchronize()
    assert torch.equal(got_a, want_a) and torch.equal(got_b, want_b)
    del filler
    assert ops.device_status() == 0


def test_embedding_ids_outside_the_tables_are_reported_not_read():
    """Through the C ABI directly (never through a stock embedding op, which would assert on the device):
    ids outside a table are clamped and flagged in the device status word."""
    g = torch.Generator(device="cpu").manual_seed(4)
    V, TV, P, D, B, L = 1000, 2, 128, 256, 4, 128
    word, typ, pos = (torch.randn((r, D), generator=g).to(DEV) for r in (V, TV, P))
    w, b = torch.ones(D, device=DEV), torch.zeros(D, device=DEV)
    ids = torch.randint(0, V, (B, L), generator=g).to(DEV)

    def run(i, tt=None, pp=None):
        return ops.embed_layernorm_fwd(i, word, typ, pos, w, b, 1e-12, token_type_ids=tt, position_ids=pp)

    good = run(ids).clone()
    assert ops.device_status() == 0
    bad = ids.clone()
    bad[1, 5] = V + 7                 # past the vocabulary
    bad[2, 9] = -3
    out = run(bad)
    assert ops.device_status() == ops.DEV_BAD_INDEX
    assert ops.device_status() == 0                                   # reading clears it
    keep = torch.ones(B, L, dtype=torch.bool, device=DEV)
    keep[1, 5] = keep[2, 9] = False
    assert torch.equal(out[keep], good[keep]) and torch.isfinite(out).all()
    tt = torch.zeros_like(ids)
    tt[0, 0] = TV
    run(ids, tt=tt)
    assert ops.device_status() == ops.DEV_BAD_INDEX
    pp = torch.arange(L, device=DEV)[None].clone()
    pp[0, 3] = P
    run(ids, pp=pp)
    assert ops.device_status() == ops.DEV_BAD_INDEX
    # a sequence longer than the position table (positions implied by the row index) is refused on the host
    with pytest.raises(RuntimeError, match="position table"):
        ops.embed_layernorm_fwd(torch.zeros((1, P + 8), dtype=torch.long, device=DEV), word, typ, pos, w, b, 1e-12)
    assert torch.equal(run(ids), good)
    assert ops.device_status() == 0


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """A wait on a barrier nothing arrives at gives up after its limit, reports through the device status
    word and leaves the device usable -- the path every tensor-core kernel's waits share."""
    lib = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert ops.device_status() == 0
    assert lib.m2_selftest_wait_timeout(ctypes.c_ulonglong(0), stream) == 1          # rejected argument
    assert lib.m2_selftest_wait_timeout(ctypes.c_ulonglong(5 * 10 ** 9), stream) == 1
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.m2_selftest_wait_timeout(ctypes.c_ulonglong(20_000_000), stream) == 0  # 20 ms
    t1.record()
    torch.cuda.synchronize()
    assert 15.0 < t0.elapsed_time(t1) < 500.0
    assert ops.device_status() == ops.DEV_TIMEOUT_TMA
    assert ops.device_status() == 0
    # the next real launches run normally
    x = torch.randn(256, 256, device=DEV).bfloat16()
    w = (torch.randn(4, 64, 64, device=DEV) / 8).bfloat16()
    out = ops.blockdiag_fwd(x, w, None, 256, 256)
    ref = torch.einsum("mkp,kqp->mkq", x.float().view(256, 4, 64), w.float()).reshape(256, 256)
    assert O.parity_error(out.float().cpu().double().numpy(), ref.cpu().double().numpy()) < 2e-2
    assert ops.device_status() == 0


def test_hyena_filter_forward_uses_caller_filters():
    """HyenaFilter.forward with k_fwd / k_rev given convolves with THEM (reference hyena_utils.py:219-234)."""
    cfg = dict(C.CASES["mixer_small"], L=256, D=16, order=32)
    m, sd = build_mixer(cfg, DEV)
    f = m.filter_fn
    L, D = 256, 16
    x = torch.randn(2, D, L, device=DEV)
    with torch.no_grad():
        own = f(x, L)
        k_fwd = f.filter(L)[0].t().contiguous()              # (D, L), what the mixer passes in the reference
        k_rev = f.filter_rev(L)[0].t().contiguous()
        same = f(x, L, k_fwd=k_fwd, k_rev=k_rev)
        assert O.parity_error(same.cpu().double().numpy(), own.cpu().double().numpy()) < 1e-5
        other = f(x, L, k_fwd=(2.0 * k_fwd,), k_rev=0.5 * k_rev)
        ref = O.fftconv(x.cpu().double().numpy(),
                        O.merge_bidirectional(2.0 * k_fwd.cpu().double().numpy(), 0.5 * k_rev.cpu().double().numpy()),
                        np.asarray(sd["filter_fn.bias"], np.float64))
        assert O.parity_error(other.cpu().double().numpy(), ref) < 1e-4
        with pytest.raises(RuntimeError):
            f(x, L, k_fwd=k_fwd)
    assert ops.device_status() == 0
