"""m2_linear_fwd (in_linear / out_linear of the mixer) through the C ABI against F.linear under autocast and
against the library's own CUDA-core kernel, in the three operand arrangements and at ragged sizes.  Needs a
B200."""
import pytest
import torch
import torch.nn.functional as F

from m2_b200 import ops
from oracle import m2_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# one bf16 step is 2^-8 relative; two correct float32 accumulations in different orders round a few outputs
# to neighbouring bf16 values, nothing more
TOL = 6e-3


@pytest.fixture(autouse=True)
def _status():
    with torch.no_grad():
        yield
    torch.cuda.synchronize()
    assert ops.device_status() == 0


def npy(t):
    return t.detach().float().cpu().double().numpy()


def make(B, L, K, N, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((B, L, K), generator=g).to(DEV).bfloat16()
    w = (torch.randn((N, K), generator=g) / K ** 0.5).to(DEV).bfloat16()
    b = torch.randn((N,), generator=g).to(DEV)
    return x, w, b


def ref_linear(x, w, b):
    return F.linear(x.float(), w.float(), b.bfloat16().float() if b is not None else None).bfloat16()


SHAPES = [(256, 128, 768, 2304), (256, 128, 768, 768), (2, 8192, 768, 2304), (3, 100, 64, 192), (1, 24, 16, 48),
          (5, 136, 256, 768), (64, 128, 1536, 4608), (1, 4100, 8, 24), (7, 72, 104, 40)]


@pytest.mark.parametrize("B,L,K,N", SHAPES)
@pytest.mark.parametrize("with_bias", [True, False])
def test_rows_in_rows_out(B, L, K, N, with_bias):
    x, w, b = make(B, L, K, N, 1)
    b = b if with_bias else None
    y = ops.linear_fwd(x, w, b)
    assert O.parity_error(npy(y), npy(ref_linear(x, w, b))) < TOL
    assert O.parity_error(npy(y), npy(ops.linear_fwd(x, w, b, force_simt=True))) < TOL


@pytest.mark.parametrize("B,L,K,N", SHAPES)
@pytest.mark.parametrize("layout", ["bnl", "channel_major"])
def test_rows_in_time_contiguous_out(B, L, K, N, layout):
    """in_linear writing (B, N, L) or channel-major (N, B*L): the transposed layouts of the convolution kernels."""
    x, w, b = make(B, L, K, N, 2)
    Lp = (L + 15) // 16 * 16 if layout == "bnl" else L
    if layout == "bnl":
        buf = torch.full((B, N, Lp), float("nan"), dtype=torch.bfloat16, device=DEV)
        view = buf[:, :, :L].permute(0, 2, 1)
    else:
        buf = torch.full((N, B, L), float("nan"), dtype=torch.bfloat16, device=DEV)
        view = buf.permute(1, 2, 0)
    ops.linear_fwd(x, w, b, out=view)
    assert torch.isfinite(view).all()
    assert O.parity_error(npy(view), npy(ref_linear(x, w, b))) < TOL
    if Lp > L:
        assert torch.isnan(buf[:, :, L:]).all()               # padding columns untouched


@pytest.mark.parametrize("B,L,K,N", SHAPES)
@pytest.mark.parametrize("layout", ["bkl", "channel_major"])
def test_time_contiguous_in_rows_out(B, L, K, N, layout):
    """out_linear reading (B, K, L) or channel-major (K, B*L) without a transposed copy."""
    x, w, b = make(B, L, K, N, 3)
    if layout == "bkl":
        Lp = (L + 7) // 8 * 8
        buf = torch.zeros((B, K, Lp), dtype=torch.bfloat16, device=DEV)
        buf[:, :, :L] = x.permute(0, 2, 1)
        buf[:, :, L:] = float("nan")                           # padding must never be read into a result
        view = buf[:, :, :L].permute(0, 2, 1)
    else:
        buf = x.permute(2, 0, 1).contiguous()                  # (K, B, L)
        view = buf.permute(1, 2, 0)
    y = ops.linear_fwd(view, w, b)
    assert torch.isfinite(y).all()
    assert O.parity_error(npy(y), npy(ref_linear(x, w, b))) < TOL


def test_rows_are_independent_of_the_batch():
    """The same token gives the same bits whatever else is in the batch (fixed accumulation order)."""
    x, w, b = make(16, 128, 768, 2304, 4)
    y = ops.linear_fwd(x, w, b)
    y1 = ops.linear_fwd(x[5:6], w, b)
    assert torch.equal(y[5:6], y1)


def test_float32_mode():
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn((3, 50, 96), generator=g).to(DEV)
    w = (torch.randn((40, 96), generator=g) / 10).to(DEV)
    b = torch.randn((40,), generator=g).to(DEV)
    y = ops.linear_fwd(x, w, b)
    ref = F.linear(x.double(), w.double(), b.double())
    assert O.parity_error(npy(y), ref.cpu().numpy()) < 1e-5
    yt = torch.empty((3, 40, 50), device=DEV)
    ops.linear_fwd(x, w, b, out=yt.permute(0, 2, 1))
    assert torch.equal(yt.permute(0, 2, 1), y)


@pytest.mark.parametrize("M,nb,p,q", [(32768, 4, 768, 192), (1000, 4, 768, 192), (257, 4, 1536, 384), (5000, 4, 64, 1536),
                                      (128, 2, 128, 48), (3000, 1, 256, 272), (20000, 4, 192, 1536)])
@pytest.mark.parametrize("with_bias", [True, False])
def test_blockdiag_pair_kernel_matches_single_cta_kernel(M, nb, p, q, with_bias):
    """BlockdiagLinear shapes on CTA-pair tiles (narrow blocks use a narrower pair tile, wide blocks several tiles
    with a ragged last one) against the single-CTA tensor-core kernel (bit for bit where that one applies) and
    against float32 arithmetic with the reference's two roundings."""
    g = torch.Generator(device="cpu").manual_seed(M + q)
    x = torch.randn((M, nb * p), generator=g).to(DEV).bfloat16()
    w = (torch.randn((nb, q, p), generator=g) / p ** 0.5).to(DEV).bfloat16()
    b = torch.randn((nb * q,), generator=g).to(DEV) if with_bias else None
    y = ops.blockdiag_fwd(x, w, b, nb * p, nb * q, variant=2)
    if q % 64 == 0:
        assert torch.equal(y, ops.blockdiag_fwd(x, w, b, nb * p, nb * q))
    rows = torch.tensor(sorted({0, 127, 128, 255, 256, M // 2, M - 1} & set(range(M))), device=DEV)
    ref = torch.einsum("mkp,kqp->mkq", x[rows].float().view(len(rows), nb, p), w.float()).reshape(len(rows), nb * q).bfloat16()
    if b is not None:
        ref = (ref + b.bfloat16()).float()
    assert O.parity_error(npy(y[rows]), npy(ref.float())) < TOL
