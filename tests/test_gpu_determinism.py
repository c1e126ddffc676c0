"""Race and bounds checks without a sanitizer: every launching entry point is run twice on the same inputs into
output buffers that sit inside a larger allocation filled with a canary pattern; the two results must be equal bit
for bit (a data race or an uninitialised read shows up as a difference sooner or later) and the canaries before
and after the output must be untouched (an out-of-bounds write shows up there).  Needs a B200."""
import pytest
import torch

from m2_b200 import ops
from tests.golden import cases as C
from tests.helpers import build_mixer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GUARD = 4096          # elements of canary on each side


def guarded(shape, dtype):
    """A tensor of `shape` carved out of a larger canary-filled buffer; returns (view, check)."""
    n = 1
    for d in shape:
        n *= d
    raw = torch.empty(n + 2 * GUARD, dtype=torch.int16 if dtype in (torch.bfloat16, torch.float16) else torch.int32, device=DEV)
    raw.fill_(0x5A5A if raw.dtype == torch.int16 else 0x5A5A5A5A)
    view = raw[GUARD:GUARD + n].view(dtype).view(*shape)

    def check():
        pat = 0x5A5A if raw.dtype == torch.int16 else 0x5A5A5A5A
        assert bool((raw[:GUARD] == pat).all()) and bool((raw[GUARD + n:] == pat).all()), "canary overwritten"
    return view, check


def twice(run, shape, dtype):
    outs = []
    for _ in range(2):
        out, check = guarded(shape, dtype)
        run(out)
        torch.cuda.synchronize()
        check()
        outs.append(out.clone())
    assert torch.equal(outs[0].view(torch.int16 if dtype != torch.float32 else torch.int32),
                       outs[1].view(torch.int16 if dtype != torch.float32 else torch.int32))
    assert ops.device_status() == 0
    return outs[0]


@pytest.mark.parametrize("B,L,K,N,mode", [(64, 128, 256, 768, "rows"), (64, 128, 256, 768, "channels"), (3, 1000, 256, 256, "timein"),
                                          (5, 136, 64, 200, "rows")])
def test_linear_fwd_is_deterministic_and_stays_in_bounds(B, L, K, N, mode):
    g = torch.Generator(device="cpu").manual_seed(1)
    x = torch.randn((B, L, K), generator=g).to(DEV).bfloat16()
    w = (torch.randn((N, K), generator=g) / K ** 0.5).to(DEV).bfloat16()
    b = torch.randn((N,), generator=g).to(DEV)
    with torch.no_grad():
        if mode == "rows":
            twice(lambda out: ops.linear_fwd(x, w, b, out=out), (B, L, N), torch.bfloat16)
        elif mode == "channels":
            twice(lambda out: ops.linear_fwd(x, w, b, out=out.permute(1, 2, 0)), (N, B, L), torch.bfloat16)
        else:
            xt = x.permute(0, 2, 1).contiguous()
            twice(lambda out: ops.linear_fwd(xt.permute(0, 2, 1), w, b, out=out), (B, L, N), torch.bfloat16)


@pytest.mark.parametrize("L,D,B,kind", [(128, 16, 130, 3), (2048, 16, 2, 2), (8192, 8, 2, 2), (32768, 4, 1, 2), (300, 8, 3, 2), (128, 128, 3, 1)])
def test_longconv_is_deterministic_and_stays_in_bounds(L, D, B, kind):
    cfg = dict(C.CASES["mixer_small"], L=L, l_max=L, D=D, B=B, order=32, residual=True, seed=72)
    m, _ = build_mixer(cfg, DEV)
    g = torch.Generator(device="cpu").manual_seed(L)
    filters = [m.filter_fn, m.filter_fn2]
    with torch.no_grad():
        u = torch.randn((B, L, D), generator=g).to(DEV)
        if kind == 3:
            xin_t = (0.6 * torch.randn((3 * D, B, L), generator=g)).to(DEV).bfloat16()
            u_t = ops.time_major_f16(u)
            specs = [f.spectrum(L, True, 3) for f in filters]
            twice(lambda out: ops.longconv_fwd(xin_t.permute(1, 2, 0), u_t.permute(1, 2, 0), m.short_filter.weight, m.short_filter.bias,
                                               specs, None, kind=3, bf16_rounding=True, out=out.permute(1, 2, 0)), (D, B, L), torch.bfloat16)
        elif kind == 2:
            xin_t = (0.6 * torch.randn((B, 3 * D, L), generator=g)).to(DEV).bfloat16()
            u_t = u.transpose(1, 2).contiguous()
            specs = [f.spectrum(L, True, 2) for f in filters]
            twice(lambda out: ops.longconv_fwd(xin_t.transpose(1, 2), u_t.transpose(1, 2), m.short_filter.weight, m.short_filter.bias,
                                               specs, [f.conv_bias() for f in filters], kind=2, bf16_rounding=True,
                                               out=out.transpose(1, 2)), (B, D, L), torch.bfloat16)
        else:
            xin = (0.6 * torch.randn((B, L, 3 * D), generator=g)).to(DEV).bfloat16()
            specs = [f.spectrum(L, True, 1) for f in filters]
            twice(lambda out: ops.longconv_fwd(xin, u, m.short_filter.weight, m.short_filter.bias, specs,
                                               [f.conv_bias() for f in filters], kind=1, bf16_rounding=True, out=out), (B, L, D), torch.bfloat16)


def test_mlp_kernels_are_deterministic():
    g = torch.Generator(device="cpu").manual_seed(2)
    M, D, I = 1000, 768, 3072
    x = torch.randn((M, D), generator=g).to(DEV).bfloat16()
    wg = (torch.randn((4, 2 * I // 4, D // 4), generator=g) / (D // 4) ** 0.5).to(DEV).bfloat16()
    wo = (torch.randn((4, D // 4, I // 4), generator=g) / (I // 4) ** 0.5).to(DEV).bfloat16()
    bo = torch.randn((D,), generator=g).to(DEV)
    lw, lb = torch.ones(D, device=DEV), torch.zeros(D, device=DEV)
    with torch.no_grad():
        for variant in (0, 1, 3):
            a, b = (ops.blockdiag_glu_fwd(x, wg, I, variant=variant) for _ in range(2))
            assert torch.equal(a, b)
        h = ops.blockdiag_glu_fwd(x, wg, I)
        for variant in (0, 2):
            a, b = (ops.blockdiag_fwd(h, wo, bo, I, D, variant=variant) for _ in range(2))
            assert torch.equal(a, b)
        o = ops.blockdiag_fwd(h, wo, bo, I, D)
        a, b = (ops.add_layernorm_fwd(o, x, lw, lb, 1e-12, torch.float32) for _ in range(2))
        assert torch.equal(a, b)
    assert ops.device_status() == 0
