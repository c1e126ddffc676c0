"""Tensor-level wrappers over the C ABI: validate, allocate outputs with torch, launch on
torch's current stream.  These are what the nn.Modules call."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import M2_BF16, M2_F16, M2_F32


LAUNCHES = 0          # kernels of this library launched since the counter was last reset
PROFILE = None        # a LaunchProfile while a benchmark wants per-kernel device times
NVTX = False          # True: every launch sits in an NVTX range named after its entry point (timeline tools)


class LaunchProfile:
    """CUDA-event pairs around individual C-ABI launches, on the launching stream."""

    def __init__(self):
        self.events = {}

    def names(self):
        return sorted(self.events)

    def count(self, name):
        return len(self.events.get(name, []))

    def mean_ms(self, name):
        ev = self.events.get(name, [])
        if not ev:
            return None
        torch.cuda.synchronize()
        return sum(s.elapsed_time(e) for s, e in ev) / len(ev)


def _launch(name, tensor, fn, *args):
    """Call one launching C-ABI entry point on torch's current stream of tensor's device."""
    global LAUNCHES
    with torch.cuda.device(tensor.device):
        st = torch.cuda.current_stream(tensor.device)
        prof = PROFILE
        if prof is not None:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(st)
        if NVTX:
            torch.cuda.nvtx.range_push(name)
        rc = fn(*args, C.c_void_p(st.cuda_stream))
        if NVTX:
            torch.cuda.nvtx.range_pop()
        if prof is not None:
            e.record(st)
            prof.events.setdefault(name, []).append((s, e))
    _lib.check(rc, name)
    LAUNCHES += 1


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return M2_F32
    if t.dtype == torch.bfloat16:
        return M2_BF16
    if t.dtype == torch.float16:
        return M2_F16
    raise TypeError(f"m2_b200 supports float32 and bfloat16 tensors, got {t.dtype}")


def _stream(t: torch.Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("m2_b200 kernels need CUDA tensors; there is no CPU fallback")


def _f32c(t: torch.Tensor) -> torch.Tensor:
    t = t.detach()
    if t.dtype != torch.float32:
        t = t.float()
    return t.contiguous()


def filter_row_len(seq_len: int) -> int:
    return _lib.lib().m2_filter_row_len(int(seq_len))


def hyena_filter(z, t, weights, biases, weights_rev, biases_rev, freq, deltas, seq_len, *,
                 bidirectional, bf16_rounding, w_mod=1.0, shift=0.0):
    """Merged time-domain filter (d_model, filter_row_len(seq_len)) float32.

    z (1, l_max, emb), t (1, l_max, 1): positional embedding buffers; weights = the four
    Linear weights of the filter MLP, biases = the first three biases (the *_rev lists are
    the reversed-direction net, ignored unless bidirectional).
    """
    _need_cuda(z)
    L = int(seq_len)
    d_model, order = weights[3].shape
    emb = weights[0].shape[1]
    keep = []

    def ptr(x):
        x = _f32c(x)
        keep.append(x)
        return x.data_ptr()

    a = _lib.FilterArgs()
    a.d_model, a.seq_len, a.order, a.emb_dim = d_model, L, order, emb
    a.bidirectional, a.bf16_rounding = int(bool(bidirectional)), int(bool(bf16_rounding))
    a.w_mod, a.shift = float(w_mod), float(shift)
    a.z = ptr(z[0, :L])
    a.t = ptr(t[0, :L, 0])
    for i in range(4):
        a.w[i] = ptr(weights[i])
    for i in range(3):
        a.b[i] = ptr(biases[i])
    if bidirectional:
        for i in range(4):
            a.w_rev[i] = ptr(weights_rev[i])
        for i in range(3):
            a.b_rev[i] = ptr(biases_rev[i])
    a.freq = ptr(freq.reshape(-1))
    a.deltas = ptr(deltas.reshape(-1))
    k = torch.empty((d_model, filter_row_len(L)), dtype=torch.float32, device=z.device)
    a.k_out = k.data_ptr()
    _launch("m2_hyena_filter", z, _lib.lib().m2_hyena_filter, C.byref(a))
    return k


def longconv_kind(seq_len: int, act_dtype: torch.dtype, d_model: int) -> int:
    return _lib.lib().m2_longconv_kind(int(seq_len), M2_BF16 if act_dtype == torch.bfloat16 else M2_F32,
                                       int(d_model))


def longconv_kind_batch(batch: int, seq_len: int, act_dtype: torch.dtype, d_model: int) -> int:
    return _lib.lib().m2_longconv_kind_batch(int(batch), int(seq_len),
                                             M2_BF16 if act_dtype == torch.bfloat16 else M2_F32, int(d_model))


def filter_spectrum(k: torch.Tensor, seq_len: int, kind: int, bias=None) -> torch.Tensor:
    """Spectrum table of one filter for kernel family `kind` (float32, opaque layout).
    Kind 3 folds the convolution's bias term into the table: pass it here."""
    _need_cuda(k)
    assert k.dtype == torch.float32 and k.is_contiguous()
    d_model = k.shape[0]
    n = _lib.lib().m2_filter_spectrum_floats(kind, d_model, int(seq_len))
    spec = torch.empty(n, dtype=torch.float32, device=k.device)
    if kind == 3:
        b = _f32c(bias) if bias is not None else None
        _launch("m2_filter_spectrum", k, _lib.lib().m2_filter_spectrum_bias, kind, d_model, int(seq_len),
                k.data_ptr(), b.data_ptr() if b is not None else None, spec.data_ptr())
    else:
        assert bias is None, "only kind 3 folds the bias into the spectrum"
        _launch("m2_filter_spectrum", k, _lib.lib().m2_filter_spectrum, kind, d_model, int(seq_len),
                k.data_ptr(), spec.data_ptr())
    return spec


def time_major_f16(u: torch.Tensor, out=None) -> torch.Tensor:
    """fp16 copy of u (B, L, D) laid out (D, B, L): the residual-filter operand of kind 3."""
    _need_cuda(u)
    B, L, D = u.shape
    if out is None:
        out = torch.empty((D, B, L), dtype=torch.float16, device=u.device)
    assert out.dtype == torch.float16 and out.shape == (D, B, L) and out.stride(2) == 1
    a = _lib.TimeMajorArgs()
    a.batch, a.seq_len, a.d_model, a.src_dtype = B, L, D, _dt(u)
    a.src, (a.src_sb, a.src_st, a.src_sc) = u.data_ptr(), u.stride()
    a.dst, a.dst_sc, a.dst_sb = out.data_ptr(), out.stride(0), out.stride(1)
    _launch("m2_time_major_f16", u, _lib.lib().m2_time_major_f16, C.byref(a))
    return out


def longconv_fwd(xin, u, short_w, short_b, specs, biases, *, kind, bf16_rounding, out=None, yu_bf16=False):
    """Fused short conv + gates + long convolution(s).

    xin (B, L, 3D) in_linear output (any strides with a unit stride along L or channels),
    u (B, L, D) raw layer input or None, specs/biases: one entry per filter (kind 3: biases
    None, they are inside its spectra, and u an fp16 view from time_major_f16).  Returns
    (B, L, D) in xin's dtype.
    """
    _need_cuda(xin)
    B, L, D3 = xin.shape
    D = D3 // 3
    nf = len(specs)
    if out is None:
        out = torch.empty((B, L, D), dtype=xin.dtype, device=xin.device)
    keep = [_f32c(short_w.reshape(D3, -1)), _f32c(short_b)] + [_f32c(b) for b in (biases or [])]
    if keep[0].shape[1] != 3:
        raise RuntimeError("m2_b200: short_filter must have kernel_size 3")
    a = _lib.LongconvArgs()
    a.batch, a.seq_len, a.d_model, a.n_filters, a.kind = B, L, D, nf, int(kind)
    a.act_dtype = _dt(xin)
    a.u_dtype = _dt(u) if u is not None else a.act_dtype
    a.bf16_rounding = int(bool(bf16_rounding))
    a.xin, (a.xin_sb, a.xin_st, a.xin_sc) = xin.data_ptr(), xin.stride()
    if u is not None:
        a.u, (a.u_sb, a.u_st, a.u_sc) = u.data_ptr(), u.stride()
    a.out, (a.out_sb, a.out_st, a.out_sc) = out.data_ptr(), out.stride()
    a.short_w, a.short_b = keep[0].data_ptr(), keep[1].data_ptr()
    a.yu_bf16 = int(bool(yu_bf16))
    for i in range(nf):
        a.spec[i] = specs[i].data_ptr()
        if biases:
            a.bias[i] = keep[2 + i].data_ptr()
    _launch("m2_longconv_fwd", xin, _lib.lib().m2_longconv_fwd, C.byref(a))
    return out


def linear_fwd(x, w, bias, out=None, *, force_simt=False):
    """nn.Linear on strided activations: y[b, t, n] = sum_k x[b, t, k] w[n, k] + bias[n].

    x (B, L, K) and out (B, L, N) are torch VIEWS with any strides that keep either the feature axis or the
    time axis contiguous (a permuted (B, K, L) or channel-major (K, B, L) buffer is passed as its (B, L, K)
    view); w (N, K) contiguous, dtype of x; bias float32-convertible (N) or None.  Returns `out` (allocated
    row-major when not given)."""
    _need_cuda(x, w)
    B, L, K = x.shape
    N = w.shape[0]
    assert w.shape == (N, K) and w.is_contiguous() and w.dtype == x.dtype
    if out is None:
        out = torch.empty((B, L, N), dtype=x.dtype, device=x.device)
    assert out.shape == (B, L, N) and out.dtype == x.dtype
    b = _f32c(bias) if bias is not None else None
    a = _lib.LinearArgs()
    a.batch, a.seq_len, a.in_features, a.out_features, a.dtype = B, L, K, N, _dt(x)
    a.x, (a.x_sb, a.x_st, a.x_sc) = x.data_ptr(), x.stride()
    a.w = w.data_ptr()
    a.bias = b.data_ptr() if b is not None else None
    a.out, (a.out_sb, a.out_st, a.out_sc) = out.data_ptr(), out.stride()
    a.force_simt = int(bool(force_simt))
    _launch("m2_linear_fwd", x, _lib.lib().m2_linear_fwd, C.byref(a))
    return out


def blockdiag_fwd(x2d, w, bias, in_features, out_features, variant=0):
    """x2d (m, in_features) @ blockdiag(w)^T (+ bias) -> (m, out_features), dtype of x2d.  variant=2 asks for
    the CTA-pair kernel (bit-identical results; for cross-checks)."""
    _need_cuda(x2d, w)
    nb, q, p = w.shape
    if x2d.stride(-1) != 1:
        x2d = x2d.contiguous()
    m = x2d.shape[0]
    out = torch.empty((m, out_features), dtype=x2d.dtype, device=x2d.device)
    b = _f32c(bias) if bias is not None else None
    a = _lib.BlockdiagArgs()
    a.m, a.nblocks, a.p, a.q = m, nb, p, q
    a.in_features, a.out_features, a.dtype = int(in_features), int(out_features), _dt(x2d)
    a.x, a.ldx, a.w = x2d.data_ptr(), x2d.stride(0) if m > 1 else max(x2d.stride(0), in_features), w.data_ptr()
    a.bias = b.data_ptr() if b is not None else None
    a.out, a.ldo, a.variant = out.data_ptr(), out.stride(0), int(variant)
    assert w.dtype == x2d.dtype and w.is_contiguous()
    _launch("m2_blockdiag_fwd", x2d, _lib.lib().m2_blockdiag_fwd, C.byref(a))
    return out


def blockdiag_glu_fwd(x2d, wg, inter, variant=0):
    """h = gelu(G[:, :inter]) * G[:, inter:], G = x2d @ blockdiag(wg)^T, without writing G.  variant=1 forces
    the general streaming kernel, variant=3 the CTA-pair kernel (bit-identical results; for cross-checks)."""
    _need_cuda(x2d, wg)
    nb, q, p = wg.shape
    if x2d.stride(-1) != 1:
        x2d = x2d.contiguous()
    m, d_model = x2d.shape
    assert nb * p == d_model and nb * q == 2 * inter and wg.dtype == x2d.dtype and wg.is_contiguous()
    h = torch.empty((m, inter), dtype=x2d.dtype, device=x2d.device)
    a = _lib.GluArgs()
    a.m, a.d_model, a.inter, a.nblocks, a.dtype = m, d_model, int(inter), nb, _dt(x2d)
    a.x, a.ldx, a.wg = x2d.data_ptr(), max(x2d.stride(0), d_model), wg.data_ptr()
    a.h, a.ldh, a.variant = h.data_ptr(), h.stride(0), int(variant)
    _launch("m2_blockdiag_glu_fwd", x2d, _lib.lib().m2_blockdiag_glu_fwd, C.byref(a))
    return h


def add_layernorm_fwd(a2d, b2d, weight, bias, eps, out_dtype, bf16_copy=None, tm_copy=None, fill_pad=False):
    """LayerNorm(a + b) over the last dimension; a, b (m, n) of the same dtype (b may be None).  bf16_copy:
    optional (m, >= n) bf16 tensor that receives the result rounded to bf16.  tm_copy: optional
    (n, B, L) fp16 tensor with B * L = m that receives the result time-major (see
    time_major_f16).  out_dtype=None writes only the copies and returns None."""
    _need_cuda(a2d, b2d)
    if a2d.stride(-1) != 1:
        a2d = a2d.contiguous()
    if b2d is not None and b2d.stride(-1) != 1:
        b2d = b2d.contiguous()
    m, n = a2d.shape
    assert b2d is None or (b2d.shape == a2d.shape and b2d.dtype == a2d.dtype)
    out = torch.empty((m, n), dtype=out_dtype, device=a2d.device) if out_dtype is not None else None
    w, bb = _f32c(weight), _f32c(bias)
    a = _lib.AddLayernormArgs()
    a.m, a.n, a.in_dtype = m, n, _dt(a2d)
    a.out_dtype = M2_BF16 if out_dtype == torch.bfloat16 else M2_F32
    a.a, a.lda = a2d.data_ptr(), max(a2d.stride(0), n)
    if b2d is not None:
        a.b, a.ldb = b2d.data_ptr(), max(b2d.stride(0), n)
    a.weight, a.bias, a.eps = w.data_ptr(), bb.data_ptr(), float(eps)
    if out is not None:
        a.out, a.ldo = out.data_ptr(), out.stride(0)
    else:
        assert bf16_copy is not None, "out_dtype=None (copies only) needs bf16_copy"
        a.ldo = n
    if bf16_copy is not None:
        assert bf16_copy.dtype == torch.bfloat16 and bf16_copy.stride(-1) == 1 and bf16_copy.shape[0] == m
        a.out_bf16, a.ld_bf16 = bf16_copy.data_ptr(), bf16_copy.stride(0)
        if fill_pad:     # columns n.. of the copy become [1, 0, 0, ...] (a constant-one input column for a following GEMM)
            a.bf16_pad_cols = bf16_copy.shape[1] - n
    if tm_copy is not None:
        assert tm_copy.dtype == torch.float16 and tm_copy.dim() == 3 and tm_copy.stride(2) == 1
        assert tm_copy.shape[0] == n and tm_copy.shape[1] * tm_copy.shape[2] == m
        a.out_tm_f16, a.tm_sc, a.tm_sb, a.seq_len = tm_copy.data_ptr(), tm_copy.stride(0), tm_copy.stride(1), tm_copy.shape[2]
    _launch("m2_add_layernorm_fwd", a2d, _lib.lib().m2_add_layernorm_fwd, C.byref(a))
    return out


def embed_layernorm_fwd(input_ids, word_table, type_table, pos_table, weight, bias, eps, *, token_type_ids=None,
                        position_ids=None, bf16_copy=None, tm_copy=None, fill_pad=False):
    """LayerNorm((word_table[input_ids] + type_table[token_type_ids]) + pos_table[position_ids]) in float32 for
    input_ids (B, L): the embeddings' gathers, adds and LayerNorm in one launch.  token_type_ids None = type 0,
    pos_table None = no position term, position_ids None = positions 0..L-1.  Returns (B, L, n) float32;
    bf16_copy / tm_copy / fill_pad as in add_layernorm_fwd."""
    _need_cuda(input_ids, word_table)
    B, L = input_ids.shape
    n = word_table.shape[1]
    m = B * L

    def ids64(t):
        return t.reshape(-1).to(torch.long).contiguous() if t is not None else None

    keep = [ids64(input_ids), ids64(token_type_ids),
            ids64(position_ids.expand(B, L)) if position_ids is not None else None,
            _f32c(word_table), _f32c(type_table), _f32c(pos_table) if pos_table is not None else None,
            _f32c(weight), _f32c(bias)]
    out = torch.empty((B, L, n), dtype=torch.float32, device=input_ids.device)
    a = _lib.EmbedLayernormArgs()
    a.m, a.n, a.eps, a.seq_len = m, n, float(eps), L
    a.vocab_rows, a.type_rows = word_table.shape[0], type_table.shape[0]
    a.pos_rows = pos_table.shape[0] if pos_table is not None else 0
    a.input_ids, a.word_table, a.type_table = keep[0].data_ptr(), keep[3].data_ptr(), keep[4].data_ptr()
    if keep[1] is not None:
        a.token_type_ids = keep[1].data_ptr()
    if keep[5] is not None:
        a.pos_table = keep[5].data_ptr()
        if keep[2] is not None:
            a.position_ids = keep[2].data_ptr()
    a.weight, a.bias = keep[6].data_ptr(), keep[7].data_ptr()
    a.out, a.ldo = out.data_ptr(), n
    if bf16_copy is not None:
        assert bf16_copy.dtype == torch.bfloat16 and bf16_copy.stride(-1) == 1 and bf16_copy.shape[0] == m
        a.out_bf16, a.ld_bf16 = bf16_copy.data_ptr(), bf16_copy.stride(0)
        if fill_pad:
            a.bf16_pad_cols = bf16_copy.shape[1] - n
    if tm_copy is not None:
        assert tm_copy.dtype == torch.float16 and tuple(tm_copy.shape) == (n, B, L) and tm_copy.stride(2) == 1
        a.out_tm_f16, a.tm_sc, a.tm_sb = tm_copy.data_ptr(), tm_copy.stride(0), tm_copy.stride(1)
    _launch("m2_embed_layernorm_fwd", input_ids, _lib.lib().m2_embed_layernorm_fwd, C.byref(a))
    return out


DEV_TIMEOUT_TMA, DEV_TIMEOUT_MMA, DEV_TIMEOUT_EPI, DEV_TIMEOUT_EMPTY, DEV_BAD_INDEX = 1, 2, 4, 8, 16


def device_status() -> int:
    """Reads and clears the device status word (synchronises): 0, or an OR of the DEV_* bits."""
    v = C.c_int(0)
    _lib.check(_lib.lib().m2_device_status(C.byref(v)), "m2_device_status")
    return v.value


def plain_longconv(x, filt, L, bf16_rounding, bias=None, spec=None):
    """HyenaFilter.forward alone: y = conv(x, k) + bias * x for x (B, d_model, L); `spec` (a kind-0
    table from filter_spectrum) replaces the module's own filter."""
    _need_cuda(x)
    B, D, Lx = x.shape
    assert Lx == L
    if spec is None:
        spec = filt.spectrum(L, bf16_rounding, 0)
    bvec = _f32c(filt.conv_bias(bias))
    out = torch.empty_like(x)
    a = _lib.LongconvArgs()
    a.batch, a.seq_len, a.d_model, a.n_filters, a.plain, a.kind = B, L, D, 1, 1, 0
    a.act_dtype = a.u_dtype = _dt(x)
    a.bf16_rounding = int(bool(bf16_rounding))
    a.xin, a.xin_sb, a.xin_sc, a.xin_st = x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)
    a.out, a.out_sb, a.out_sc, a.out_st = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    a.spec[0], a.bias[0] = spec.data_ptr(), bvec.data_ptr()
    _launch("m2_longconv_plain", x, _lib.lib().m2_longconv_fwd, C.byref(a))
    return out
