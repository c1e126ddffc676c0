"""Second oracle: the same forward path written with stock PyTorch ops, so that on a GPU it
runs the library kernels (cuBLAS, cuFFT, cuDNN) the reference itself would launch, under
the same ``torch.autocast`` policy.  TEST INFRASTRUCTURE ONLY -- nothing in the shipped
package imports it.

It restates bert/src/mm/monarch_mixer_sequence_mixer.py:100-154,
bert/src/mm/hyena_utils.py:16-42 and :201-248, bert/src/mm/blockdiag_multiply.py:49-60,
bert/src/mm/structured_linear.py:67-70 and bert/src/bert_layers.py:482-508 of the reference,
and is checked against the stored reference outputs in tests/test_oracle_golden.py.

State dicts map the reference's key names to torch tensors (float32 parameters).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _autocast_on(device_type):
    return torch.is_autocast_enabled(device_type)


def hyena_filter(sd, prefix, L, reverse=False, w_mod=1.0, shift=0.0):
    net = prefix + ("implicit_filter_rev." if reverse else "implicit_filter.")
    z = sd[prefix + "pos_emb.z"][:, :L]
    t = sd[prefix + "pos_emb.t"][:, :L]
    h = z
    for li in (0, 2, 4):
        h = F.linear(h, sd[net + f"{li}.weight"], sd[net + f"{li}.bias"])
        h = torch.sin(w_mod * sd[net + f"{li + 1}.freq"] * h)
    h = F.linear(h, sd[net + "6.weight"])
    decay = torch.exp(-t * sd[prefix + "modulation.deltas"].abs())
    return h * (decay + shift)                                   # (1, L, D)


def fftconv(u, k, bias):
    L = u.shape[-1]
    n = 2 * L
    k_f = torch.fft.rfft(k, n=n) / n
    u_f = torch.fft.rfft(u.to(dtype=k.dtype), n=n)
    y = torch.fft.irfft(u_f * k_f, n=n, norm="forward")[..., :L]
    return (y + u * bias).to(dtype=u.dtype)


def long_conv(sd, prefix, x, L, bidirectional):
    k = hyena_filter(sd, prefix, L).transpose(1, 2)[0]
    if bidirectional:
        kr = hyena_filter(sd, prefix, L, reverse=True).transpose(1, 2)[0]
        k = F.pad(k, (0, L)) + F.pad(kr.flip(-1), (L, 0))
    return fftconv(x, k, sd[prefix + "bias"][None, :, None]).to(dtype=x.dtype)


def mixer_forward(sd, u, *, bidirectional=True, residual_long_conv=False, prefix=""):
    D = u.shape[-1]
    L = u.shape[-2]
    g = lambda name: sd[prefix + name]
    x = F.linear(u, g("in_linear.weight"), g("in_linear.bias")).transpose(1, 2)
    uc = F.conv1d(x, g("short_filter.weight"), g("short_filter.bias"), padding=2, groups=3 * D)[..., :L]
    x1, x2, v = uc.split(D, dim=1)
    v = v * x1
    y = long_conv(sd, prefix + "filter_fn.", v, L, bidirectional)
    y = y * x2
    if residual_long_conv:
        y = y + long_conv(sd, prefix + "filter_fn2.", u.transpose(-1, -2), L, bidirectional)
    y = y.transpose(-1, -2)
    return F.linear(y, g("out_linear.weight"), g("out_linear.bias"))


def blockdiag_multiply(x, weight):
    """BlockdiagMultiply.forward: inputs cast to bf16 when CUDA autocast is on."""
    if x.is_cuda and _autocast_on("cuda"):
        x, weight = x.to(torch.bfloat16), weight.to(torch.bfloat16)
    with torch.autocast(x.device.type, enabled=False):
        nb, q, p = weight.shape
        xr = x.reshape(-1, nb, p).transpose(0, 1)
        out = torch.bmm(xr, weight.transpose(-1, -2)).transpose(0, 1)
        return out.reshape(*x.shape[:-1], nb * q)


def blockdiag_linear(x, weight, bias, out_features=None):
    nb, q, p = weight.shape
    if x.shape[-1] < nb * p:
        x = F.pad(x, (0, nb * p - x.shape[-1]))
    out = blockdiag_multiply(x, weight)
    if out_features is not None and out.shape[-1] > out_features:
        out = out[..., :out_features]
    return out + bias.to(dtype=out.dtype) if bias is not None else out


def glu_mlp_forward(sd, x, *, eps=1e-12, prefix=""):
    g = lambda name: sd[prefix + name]
    wg = g("gated_layers.weight")
    inter = wg.shape[0] * wg.shape[1] // 2
    h = blockdiag_linear(x, wg, None)
    h = F.gelu(h[..., :inter]) * h[..., inter:]
    h = blockdiag_linear(h, g("wo.weight"), g("wo.bias"), out_features=x.shape[-1])
    return F.layer_norm(h + x, (x.shape[-1],), g("layernorm.weight"), g("layernorm.bias"), eps)


def embeddings_forward(sd, input_ids, *, eps=1e-12, prefix="embeddings."):
    L = input_ids.shape[1]
    e = F.embedding(input_ids, sd[prefix + "word_embeddings.weight"])
    e = e + sd[prefix + "token_type_embeddings.weight"][0]
    if prefix + "position_embeddings.weight" in sd:
        e = e + sd[prefix + "position_embeddings.weight"][:L][None]
    return F.layer_norm(e, (e.shape[-1],), sd[prefix + "LayerNorm.weight"], sd[prefix + "LayerNorm.bias"], eps)


def encoder_forward(sd, h, n_layers, *, eps=1e-12, bidirectional=True, residual_long_conv=True,
                    prefix="encoder.layer."):
    for i in range(n_layers):
        p = f"{prefix}{i}."
        a = mixer_forward(sd, h, bidirectional=bidirectional, residual_long_conv=residual_long_conv,
                          prefix=p + "attention.")
        h = glu_mlp_forward(sd, a, eps=eps, prefix=p + "mlp.")
    return h
