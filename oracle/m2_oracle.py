"""CPU restatement (numpy) of the M2-BERT sequence-mixer / GLU-MLP forward path.

THIS FILE IS TEST INFRASTRUCTURE.  It is the checker that the CUDA path is compared
against; nothing in the shipped package imports it.  Only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may call it.

Every function restates one piece of the reference (HazyResearch/m2, paths relative to
the reference checkout) and cites the lines it follows.  Arithmetic is done in float64
unless a rounding point of the reference's bf16-autocast execution is being reproduced
(``mode="bf16"``), in which case values are rounded to bfloat16 (round-to-nearest-even)
exactly where torch autocast would round them.

Pinned against the reference itself: ``tests/golden/make_golden.py`` imports the
reference modules on CPU, runs them on seeded inputs, and stores inputs, weights and
outputs under ``tests/golden/``; ``tests/test_oracle_golden.py`` checks this file against
those stored outputs.  The reference ships no golden vectors of its own for this path.

State dicts use the reference's own key names (for example
``filter_fn.implicit_filter.0.weight``), values are numpy arrays.
"""
from __future__ import annotations

import math
from concurrent.futures import ThreadPoolExecutor

import numpy as np

try:  # scipy ships a vectorised erf; fall back to math.erf if absent
    from scipy.special import erf as _erf
except Exception:  # pragma: no cover
    _erf = np.vectorize(math.erf, otypes=[np.float64])


# --------------------------------------------------------------------------------------
# bfloat16 emulation
# --------------------------------------------------------------------------------------
def bf16_round(x):
    """Round to the nearest bfloat16 (ties to even); returns float64 holding bf16 values."""
    x32 = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    bits = x32.view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    rounded = (bits + np.uint32(0x7FFF) + lsb) & np.uint32(0xFFFF0000)
    out = rounded.view(np.float32).astype(np.float64)
    nan = np.isnan(x32)
    if nan.any():
        out = np.where(nan, np.nan, out)
    return out


def _r(x, mode):
    """Rounding point of a tensor that torch would hold in the autocast dtype."""
    return bf16_round(x) if mode == "bf16" else np.asarray(x, dtype=np.float64)


def _f32(x, mode):
    """Rounding point of a tensor torch holds in float32 while autocast is active."""
    if mode == "bf16":
        return np.asarray(x, dtype=np.float32).astype(np.float64)
    return np.asarray(x, dtype=np.float64)


# --------------------------------------------------------------------------------------
# HyenaFilter pieces
# --------------------------------------------------------------------------------------
def positional_embedding(emb_dim: int, seq_len: int):
    """z (seq_len, emb_dim) and t (seq_len,), bert/src/mm/hyena_utils.py:66-85.

    The reference builds these in float32 with torch.linspace and a complex exponential;
    the values stored in a checkpoint are what the filter consumes, so callers normally
    pass ``pos_emb.z`` / ``pos_emb.t`` from the state dict and use this only to build
    fresh state dicts.
    """
    assert emb_dim % 2 == 1 and emb_dim >= 3
    t = np.linspace(0.0, 1.0, seq_len, dtype=np.float32).astype(np.float64)
    bands = (emb_dim - 1) // 2
    t_rescaled = np.linspace(0.0, seq_len - 1, seq_len, dtype=np.float32).astype(np.float64)
    w = 2.0 * math.pi * t_rescaled / seq_len
    f = np.linspace(1e-4, bands - 1, bands, dtype=np.float32).astype(np.float64)
    ang = w[:, None] * f[None, :]
    z = np.concatenate([t[:, None], np.cos(ang), -np.sin(ang)], axis=1)
    return z.astype(np.float32), t.astype(np.float32)


def modulation_deltas(d_model, fast_decay_pct=0.3, slow_decay_pct=1.5, target=1e-2):
    """ExponentialModulation.deltas, bert/src/mm/hyena_utils.py:104-107."""
    max_decay = math.log(target) / fast_decay_pct
    min_decay = math.log(target) / slow_decay_pct
    return np.linspace(min_decay, max_decay, d_model, dtype=np.float32)


def _linear(x, w, b, mode):
    """nn.Linear.  Under autocast: bf16 inputs/weights/bias, fp32 accumulate, bf16 output."""
    if mode == "bf16":
        y = bf16_round(x) @ bf16_round(w).T
        if b is not None:
            y = y + bf16_round(b)
        return bf16_round(y)
    y = np.asarray(x, np.float64) @ np.asarray(w, np.float64).T
    if b is not None:
        y = y + np.asarray(b, np.float64)
    return y


def hyena_filter(sd, prefix, L, *, reverse=False, mode="fp64", w_mod=1.0, shift=0.0):
    """HyenaFilter.filter / filter_rev -> (L, D) float64 array.

    bert/src/mm/hyena_utils.py:201-217 (filter, filter_rev), :62-63 (Sin),
    :168-189 (MLP layout: Linear, Sin, [Linear, Sin] x2, Linear without bias),
    :109-112 (exponential modulation).  ``prefix`` is e.g. ``"filter_fn."``.

    mode="bf16" reproduces the autocast rounding points: each Linear is evaluated on
    bf16-rounded operands and rounded to bf16; Sin multiplies by the float32 ``freq``
    parameter so its argument and result are float32; the modulation multiplies the bf16
    MLP output by a float32 decay, so the filter itself is float32.
    """
    net = prefix + ("implicit_filter_rev." if reverse else "implicit_filter.")
    z = np.asarray(sd[prefix + "pos_emb.z"], np.float64)[0, :L]       # (L, emb)
    t = np.asarray(sd[prefix + "pos_emb.t"], np.float64)[0, :L, 0]    # (L,)
    h = z
    for li in (0, 2, 4):
        h = _linear(h, sd[net + f"{li}.weight"], sd[net + f"{li}.bias"], mode)
        freq = np.asarray(sd[net + f"{li + 1}.freq"], np.float64)[0]
        arg = _f32(_f32(w_mod * freq, mode) * h, mode)
        h = _f32(np.sin(arg), mode)
    h = _linear(h, sd[net + "6.weight"], None, mode)                   # (L, D)
    deltas = np.asarray(sd[prefix + "modulation.deltas"], np.float64).reshape(-1)
    decay = _f32(np.exp(_f32(-t[:, None] * np.abs(deltas)[None, :], mode)), mode)
    return _f32(h * _f32(decay + shift, mode), mode)


def merge_bidirectional(k_fwd, k_rev):
    """Length-2L kernel ``pad(k_fwd,(0,L)) + pad(flip(k_rev),(L,0))``; inputs (D, L).

    bert/src/mm/hyena_utils.py:231-234.
    """
    return np.concatenate([k_fwd, k_rev[:, ::-1]], axis=-1)


def fftconv(u, k, bias):
    """``irfft(rfft(u,n)*rfft(k,n)/n, norm="forward")[..., :L] + u*bias`` with n = 2L.

    bert/src/mm/hyena_utils.py:16-42 (gelu=False, dropout_mask=None, flashfft=None).
    u (..., D, L), k (D, L) or (D, 2L), bias (D,).  float64 throughout.
    """
    L = u.shape[-1]
    n = 2 * L
    k_f = np.fft.rfft(k, n=n, axis=-1) / n
    u_f = np.fft.rfft(u, n=n, axis=-1)
    y = np.fft.irfft(u_f * k_f, n=n, axis=-1) * n   # norm="forward": no 1/n on the inverse
    return y[..., :L] + u * np.asarray(bias, np.float64)[:, None]


def longconv_direct(u, k_fwd, k_rev, bias):
    """Closed form of the bidirectional long convolution by direct summation (O(L^2)).

    y[t] = sum_{s<=t} u[s] k_fwd[t-s] + sum_{s>t} u[s] k_rev[s-t-1] + bias*u[t]; this is
    what fftconv() yields for k = merge_bidirectional(k_fwd, k_rev) and is used as an
    FFT-free cross-check on small L.  k_rev may be None (causal only).
    """
    L = u.shape[-1]
    idx = np.arange(L)
    d = idx[:, None] - idx[None, :]                       # t - s
    T = np.where(d >= 0, k_fwd[:, np.clip(d, 0, L - 1)], 0.0)          # (D, t, s)
    if k_rev is not None:
        T = T + np.where(d < 0, k_rev[:, np.clip(-d - 1, 0, L - 1)], 0.0)
    return np.einsum("dts,...ds->...dt", T, u) + u * np.asarray(bias, np.float64)[:, None]


def short_conv(x, w, b):
    """Depthwise causal 3-tap FIR: Conv1d(k=3, padding=2, groups=C)(x)[..., :L].

    bert/src/mm/monarch_mixer_sequence_mixer.py:90-97 and :112.
    x (B, C, L), w (C, 1, K), b (C,):  y[t] = b + sum_j w[j] * x[t - (K-1) + j].
    """
    K = w.shape[-1]
    L = x.shape[-1]
    xp = np.concatenate([np.zeros(x.shape[:-1] + (K - 1,), x.dtype), x], axis=-1)
    y = np.zeros_like(x, dtype=np.float64)
    for j in range(K):
        y = y + np.asarray(w, np.float64)[None, :, 0, j, None] * xp[..., j:j + L]
    return y + np.asarray(b, np.float64)[None, :, None]


# --------------------------------------------------------------------------------------
# MonarchMixerSequenceMixing.forward
# --------------------------------------------------------------------------------------
def mixer_filters(sd, L, *, bidirectional=True, residual_long_conv=False, mode="fp64",
                  w_mod=1.0):
    """Time-domain filters the mixer uses: list of (k_fwd (D,L), k_rev (D,L)|None, bias)."""
    out = []
    for prefix in ["filter_fn."] + (["filter_fn2."] if residual_long_conv else []):
        kf = hyena_filter(sd, prefix, L, reverse=False, mode=mode, w_mod=w_mod).T
        kr = hyena_filter(sd, prefix, L, reverse=True, mode=mode, w_mod=w_mod).T \
            if bidirectional else None
        out.append((kf, kr, np.asarray(sd[prefix + "bias"], np.float64)))
    return out


def mixer_core(xin, u_orig, sd, *, bidirectional=True, residual_long_conv=False,
               mode="fp64", u_is_bf16=False, w_mod=1.0, filters=None):
    """Everything between in_linear and out_linear.

    bert/src/mm/monarch_mixer_sequence_mixer.py:109-149.  ``xin`` is the in_linear
    output (B, L, 3D) and ``u_orig`` the raw layer input (B, L, D); returns (B, L, D), the
    tensor out_linear consumes (already rounded to bf16 in mode="bf16").
    """
    B, L, D3 = xin.shape
    D = D3 // 3
    x = _r(np.transpose(xin, (0, 2, 1)), mode)                       # b d l
    w, b = sd["short_filter.weight"], sd["short_filter.bias"]
    uc = _r(short_conv(x, _r(w, mode), _r(b, mode)), mode)            # conv1d autocasts to bf16
    x1, x2, v = uc[:, :D], uc[:, D:2 * D], uc[:, 2 * D:]
    v = _r(v * x1, mode)
    if filters is None:
        filters = mixer_filters(sd, L, bidirectional=bidirectional,
                                residual_long_conv=residual_long_conv, mode=mode,
                                w_mod=w_mod)
    kf, kr, bias = filters[0]
    k = merge_bidirectional(kf, kr) if bidirectional else kf
    y = _r(fftconv(v, k, bias), mode)                                 # cast back to x.dtype
    y = _r(y * x2, mode)
    if residual_long_conv:
        kf2, kr2, bias2 = filters[1]
        k2 = merge_bidirectional(kf2, kr2) if bidirectional else kf2
        uo = np.transpose(np.asarray(u_orig, np.float64), (0, 2, 1))
        if mode == "bf16" and u_is_bf16:
            uo = bf16_round(uo)
            yu = bf16_round(fftconv(uo, k2, bias2))
            y = bf16_round(y + yu)
        else:
            # float32 layer input under autocast: yu and the sum stay float32 and are
            # rounded once, by out_linear's autocast cast of its input
            y = _r(y + fftconv(uo, k2, bias2), mode)
    return np.transpose(y, (0, 2, 1))


def mixer_forward(sd, u, *, bidirectional=True, residual_long_conv=False, mode="fp64",
                  u_is_bf16=False, w_mod=1.0):
    """MonarchMixerSequenceMixing.forward(u)[0] for hyena_training_additions=False.

    bert/src/mm/monarch_mixer_sequence_mixer.py:100-154.  u (B, L, D).
    """
    u = np.asarray(u, np.float64)
    if mode == "bf16" and u_is_bf16:
        u = bf16_round(u)
    xin = _linear(u, sd["in_linear.weight"], sd["in_linear.bias"], mode)
    y = mixer_core(xin, u, sd, bidirectional=bidirectional,
                   residual_long_conv=residual_long_conv, mode=mode, u_is_bf16=u_is_bf16,
                   w_mod=w_mod)
    return _linear(y, sd["out_linear.weight"], sd["out_linear.bias"], mode)


# --------------------------------------------------------------------------------------
# BlockdiagLinear and the GLU MLP
# --------------------------------------------------------------------------------------
def blockdiag_multiply(x, weight):
    """out[..., k*q:(k+1)*q] = x[..., k*p:(k+1)*p] @ weight[k].T

    bert/src/mm/blockdiag_multiply.py:19-34; weight (nblocks, q, p).
    """
    nb, q, p = weight.shape
    assert x.shape[-1] == nb * p
    xr = np.asarray(x, np.float64).reshape(x.shape[:-1] + (nb, p))
    out = np.einsum("...kp,kqp->...kq", xr, np.asarray(weight, np.float64))
    return out.reshape(x.shape[:-1] + (nb * q,))


def blockdiag_linear(x, weight, bias, out_features=None, mode="fp64"):
    """BlockdiagLinear.forward: pad input, block-diagonal multiply, crop, add bias.

    bert/src/mm/structured_linear.py:52-70, bert/src/mm/blockdiag_linear.py:42-48.
    Under autocast the multiply casts x and weight to bf16 and returns bf16
    (blockdiag_multiply.py:50); the bias is cast to the output dtype before the add.
    """
    nb, q, p = weight.shape
    pad = nb * p - x.shape[-1]
    if pad > 0:
        x = np.concatenate([x, np.zeros(x.shape[:-1] + (pad,), x.dtype)], axis=-1)
    out = _r(blockdiag_multiply(_r(x, mode), _r(weight, mode)), mode)
    if out_features is not None and out.shape[-1] > out_features:
        out = out[..., :out_features]
    if bias is not None:
        out = _r(out + _r(bias, mode), mode)
    return out


def gelu_exact(x):
    """nn.GELU(approximate='none'), bert/src/bert_layers.py:475."""
    x = np.asarray(x, np.float64)
    return 0.5 * x * (1.0 + _erf(x / math.sqrt(2.0)))


def layer_norm(x, w, b, eps):
    x = np.asarray(x, np.float64)
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * np.asarray(w, np.float64) + np.asarray(b, np.float64)


def glu_mlp_forward(sd, x, *, eps=1e-12, mode="fp64", prefix=""):
    """BertGatedLinearUnitMLP.forward with BlockdiagLinear layers, eval mode.

    bert/src/bert_layers.py:482-508.  Keys: gated_layers.weight, wo.weight, wo.bias,
    layernorm.weight, layernorm.bias.  In mode="bf16" the LayerNorm output is float32
    (autocast runs layer_norm in float32 on the bf16 sum).
    """
    x = _r(x, mode)
    wg = sd[prefix + "gated_layers.weight"]
    inter = wg.shape[0] * wg.shape[1] // 2
    h = blockdiag_linear(x, wg, None, mode=mode)
    gated, non_gated = h[..., :inter], h[..., inter:]
    h = _r(_r(gelu_exact(gated), mode) * non_gated, mode)
    h = blockdiag_linear(h, sd[prefix + "wo.weight"], sd[prefix + "wo.bias"],
                         out_features=x.shape[-1], mode=mode)
    h = _r(h + x, mode)
    return _f32(layer_norm(h, _f32(sd[prefix + "layernorm.weight"], mode),
                           _f32(sd[prefix + "layernorm.bias"], mode), eps), mode)


# --------------------------------------------------------------------------------------
# Encoder-level restatement (used by the benchmark's CPU leg and the end-to-end checks)
# --------------------------------------------------------------------------------------
def embeddings_forward(sd, input_ids, *, eps=1e-12, mode="fp64", prefix="embeddings."):
    """BertEmbeddings.forward with token_type_ids = 0, bert/src/bert_layers.py:185-252."""
    ids = np.asarray(input_ids)
    L = ids.shape[1]
    e = np.asarray(sd[prefix + "word_embeddings.weight"], np.float64)[ids]
    e = e + np.asarray(sd[prefix + "token_type_embeddings.weight"], np.float64)[0]
    if prefix + "position_embeddings.weight" in sd:
        e = e + np.asarray(sd[prefix + "position_embeddings.weight"], np.float64)[:L][None]
    e = _f32(e, mode)
    return _f32(layer_norm(e, sd[prefix + "LayerNorm.weight"], sd[prefix + "LayerNorm.bias"],
                           eps), mode)


def layer_forward(sd, h, prefix, *, eps=1e-12, mode="fp64", bidirectional=True,
                  residual_long_conv=True):
    """BertLayer.forward (mixer then GLU MLP), bert/src/bert_layers.py:575-599."""
    att = {k[len(prefix) + 10:]: v for k, v in sd.items() if k.startswith(prefix + "attention.")}
    mlp = {k[len(prefix) + 4:]: v for k, v in sd.items() if k.startswith(prefix + "mlp.")}
    a = mixer_forward(att, h, bidirectional=bidirectional,
                      residual_long_conv=residual_long_conv, mode=mode)
    return glu_mlp_forward(mlp, a, eps=eps, mode=mode)


def encoder_forward(sd, hidden, n_layers, *, eps=1e-12, mode="fp64", bidirectional=True,
                    residual_long_conv=True, prefix="encoder.layer."):
    """BertEncoder.forward for the Monarch-Mixer branch, bert/src/bert_layers.py:750-759."""
    h = hidden
    for i in range(n_layers):
        h = layer_forward(sd, h, f"{prefix}{i}.", eps=eps, mode=mode,
                          bidirectional=bidirectional, residual_long_conv=residual_long_conv)
    return h


def parallel_over_batch(fn, x, threads):
    """Run ``fn`` on slices of the leading (batch) axis with a thread pool (numpy's FFT
    and BLAS release the GIL); used only to time the CPU baseline on all host cores."""
    threads = max(1, min(threads, x.shape[0]))
    chunks = np.array_split(np.arange(x.shape[0]), threads)
    with ThreadPoolExecutor(threads) as ex:
        parts = list(ex.map(lambda idx: fn(x[idx[0]:idx[-1] + 1]), chunks))
    return np.concatenate(parts, axis=0)


# --------------------------------------------------------------------------------------
# Error measure shared by all parity tests
# --------------------------------------------------------------------------------------
def parity_error(got, ref):
    """max over elements of |got-ref| / (rms(ref) + |ref|).

    The tolerance of the path (1e-4 for float32, 2e-2 for bf16) is applied to this
    number: an allclose-style bound |got-ref| <= tol*rms(ref) + tol*|ref|.  A bare
    element-wise relative error is meaningless near zero crossings, and a bare absolute
    error ignores that the mixer output's scale grows with sqrt(L).
    """
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    rms = math.sqrt(float(np.mean(ref ** 2))) + 1e-300
    return float(np.max(np.abs(got - ref) / (rms + np.abs(ref))))
