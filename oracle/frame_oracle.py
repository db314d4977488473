"""TEST INFRASTRUCTURE — CPU restatement (numpy) of the reference CPU backend's kernels
for the compiled-graph inference path.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this
module; it is the checker, never the thing measured or shipped.

Every function follows one reference kernel (paths inside the reference project) and keeps
its arithmetic ORDER: fp32 accumulators, sequential accumulation over the contraction index,
`acc += a*b` as a separate multiply and add (the reference is built with -ffp-contract=off),
one round-to-nearest-even conversion to the tensor dtype at the store
(src/backends/cpu/kernels/accum_cast.h:19-44).  Vectorisation is only ever over
*independent* outputs, so integer/indexing ops and fp32 ops without libm calls are
bit-identical to the reference; ops that call libm (exp, tanh) can differ in the last ulp.

Pinning: tests/test_oracle_pins.py checks these functions against (a) the hand-computed
known-answer vectors of the reference's own unit tests (tests/golden/reference_known_answers.json)
and (b) outputs of the unmodified reference CPU backend compiled from its sources
(tests/golden/ref_cpu_*.npz, made by tests/golden/make_golden.py).

Ops marked NEW (gelu, silu, softplus, exp, bias_add, mamba_scan) do not exist in the
reference: parity for them is UNPINNED by the reference; they are written in the reference's
kernel style and cross-checked against compositions of reference ops.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32

# DTypeCode numbering of the reference: include/frame/core/dtype.h:17-29
DT_F32, DT_F64, DT_F16, DT_BF16, DT_I8, DT_I16, DT_I32, DT_I64, DT_U8, DT_BOOL = range(10)


# --------------------------------------------------------------------------------------
# bf16 <-> f32, bit level.  include/frame/core/dtype.h:117-131
# --------------------------------------------------------------------------------------
def f32_to_bf16_bits(x) -> np.ndarray:
    """RTNE float32 -> bfloat16 bit pattern (uint16); NaN keeps its top payload bits and gets
    the quiet bit (dtype.h:117-126)."""
    x = np.ascontiguousarray(x, dtype=F32)
    bits = x.view(np.uint32)
    is_nan = (bits & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    bias = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    rounded = (bits.astype(np.uint64) + bias.astype(np.uint64)).astype(np.uint64) & np.uint64(0xFFFFFFFF)
    out = (rounded >> np.uint64(16)).astype(np.uint16)
    nan_out = ((bits >> np.uint32(16)) | np.uint32(0x0040)).astype(np.uint16)
    return np.where(is_nan, nan_out, out).astype(np.uint16)


def bf16_bits_to_f32(b) -> np.ndarray:
    """bfloat16 bit pattern -> float32, exact widening (dtype.h:128-131)."""
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << np.uint32(16)).view(F32)


def to_accum(x, dtype: int) -> np.ndarray:
    """Storage -> fp32 accumulator type (accum_cast.h:19-31)."""
    if dtype == DT_BF16:
        return bf16_bits_to_f32(x)
    if dtype == DT_F16:
        return np.asarray(x).view(np.float16).astype(F32)
    return np.asarray(x, dtype=F32)


def from_accum(x, dtype: int) -> np.ndarray:
    """fp32 -> storage with one RTNE rounding (accum_cast.h:33-44)."""
    if dtype == DT_BF16:
        return f32_to_bf16_bits(x)
    if dtype == DT_F16:
        return np.asarray(x, dtype=F32).astype(np.float16).view(np.uint16)
    return np.asarray(x, dtype=F32)


def round_through(x, dtype: int) -> np.ndarray:
    """Value after being stored in `dtype` and read back as fp32."""
    return to_accum(from_accum(x, dtype), dtype)


# --------------------------------------------------------------------------------------
# matmul.  src/backends/cpu/kernels/matmul.cpp:92-131
# --------------------------------------------------------------------------------------
def matmul(a, b, dtype: int = DT_F32) -> np.ndarray:
    """C[i,j] = sum_p A[i,p]*B[p,j], fp32 accumulator, p increasing, one rounding at the end."""
    a = to_accum(a, dtype)
    b = to_accum(b, dtype)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    acc = np.zeros((m, n), dtype=F32)
    for p in range(k):
        acc += a[:, p : p + 1] * b[p : p + 1, :]
    return from_accum(acc, dtype)


# --------------------------------------------------------------------------------------
# conv2d / conv1d.  src/backends/cpu/kernels/conv.cpp:225-257, 565-589
# --------------------------------------------------------------------------------------
def conv_out_size(size: int, k: int, stride: int, pad: int) -> int:
    """floor((in + 2p - k)/s) + 1  (src/ops/schemas/schema_math.h:43-47)."""
    return (size + 2 * pad - k) // stride + 1


def conv2d(x, w, bias=None, stride=(1, 1), padding=(0, 0), groups: int = 1, dtype: int = DT_F32):
    """NCHW cross-correlation; accumulation order ci -> kh -> kw; padded taps are skipped
    (not multiplied by zero); bias added last."""
    x = to_accum(x, dtype)
    w = to_accum(w, dtype)
    n, cin, h, wd = x.shape
    cout, cpg, kh, kw = w.shape
    sh, sw = stride
    ph, pw = padding
    oh = conv_out_size(h, kh, sh, ph)
    ow = conv_out_size(wd, kw, sw, pw)
    copg = cout // groups
    acc = np.zeros((n, cout, oh, ow), dtype=F32)
    for g in range(groups):
        co = slice(g * copg, (g + 1) * copg)
        for ci in range(cpg):
            cif = g * cpg + ci
            for i in range(kh):
                # valid output rows: 0 <= o*sh - ph + i < h
                o_lo = 0
                while o_lo < oh and o_lo * sh - ph + i < 0:
                    o_lo += 1
                o_hi = oh
                while o_hi > o_lo and (o_hi - 1) * sh - ph + i >= h:
                    o_hi -= 1
                if o_hi <= o_lo:
                    continue
                for j in range(kw):
                    q_lo = 0
                    while q_lo < ow and q_lo * sw - pw + j < 0:
                        q_lo += 1
                    q_hi = ow
                    while q_hi > q_lo and (q_hi - 1) * sw - pw + j >= wd:
                        q_hi -= 1
                    if q_hi <= q_lo:
                        continue
                    ih0 = o_lo * sh - ph + i
                    iw0 = q_lo * sw - pw + j
                    xs = x[:, cif, ih0 : ih0 + (o_hi - o_lo - 1) * sh + 1 : sh,
                           iw0 : iw0 + (q_hi - q_lo - 1) * sw + 1 : sw]
                    wv = w[co, ci, i, j]
                    acc[:, co, o_lo:o_hi, q_lo:q_hi] += xs[:, None, :, :] * wv[None, :, None, None]
    if bias is not None:
        acc += to_accum(bias, dtype)[None, :, None, None]
    return from_accum(acc, dtype)


def conv1d(x, w, bias=None, stride: int = 1, padding: int = 0, groups: int = 1, dtype: int = DT_F32):
    """NCL cross-correlation; accumulation order ci -> k; bias last (conv.cpp:565-589)."""
    x = to_accum(x, dtype)
    w = to_accum(w, dtype)
    n, cin, l = x.shape
    cout, cpg, k = w.shape
    ol = conv_out_size(l, k, stride, padding)
    copg = cout // groups
    acc = np.zeros((n, cout, ol), dtype=F32)
    for g in range(groups):
        co = slice(g * copg, (g + 1) * copg)
        for ci in range(cpg):
            cif = g * cpg + ci
            for i in range(k):
                lo = 0
                while lo < ol and lo * stride - padding + i < 0:
                    lo += 1
                hi = ol
                while hi > lo and (hi - 1) * stride - padding + i >= l:
                    hi -= 1
                if hi <= lo:
                    continue
                i0 = lo * stride - padding + i
                xs = x[:, cif, i0 : i0 + (hi - lo - 1) * stride + 1 : stride]
                acc[:, co, lo:hi] += xs[:, None, :] * w[co, ci, i][None, :, None]
    if bias is not None:
        acc += to_accum(bias, dtype)[None, :, None]
    return from_accum(acc, dtype)


# --------------------------------------------------------------------------------------
# max_pool2d.  src/backends/cpu/kernels/pool.cpp:187-233
# --------------------------------------------------------------------------------------
def max_pool2d(x, kernel=(2, 2), stride=(2, 2), padding=(0, 0), dtype: int = DT_F32):
    """Max over valid (non-padding) positions; the first valid tap seeds, later taps replace
    only on strict `>` (so ties keep the lowest linear index and a leading NaN sticks)."""
    xv = to_accum(x, dtype)
    n, c, h, wd = xv.shape
    kh, kw = kernel
    sh, sw = stride
    ph, pw = padding
    oh = conv_out_size(h, kh, sh, ph)
    ow = conv_out_size(wd, kw, sw, pw)
    best = np.zeros((n, c, oh, ow), dtype=F32)
    found = np.zeros((oh, ow), dtype=bool)
    for i in range(kh):
        for j in range(kw):
            ohs = np.arange(oh) * sh - ph + i
            ows = np.arange(ow) * sw - pw + j
            vo = (ohs >= 0) & (ohs < h)
            vq = (ows >= 0) & (ows < wd)
            if not vo.any() or not vq.any():
                continue
            oi = np.nonzero(vo)[0]
            qi = np.nonzero(vq)[0]
            vals = xv[:, :, ohs[oi]][:, :, :, ows[qi]]
            sub_found = found[np.ix_(oi, qi)]
            cur = best[:, :, oi[:, None], qi[None, :]]
            take = (~sub_found)[None, None] | (vals > cur)
            best[:, :, oi[:, None], qi[None, :]] = np.where(take, vals, cur)
            found[np.ix_(oi, qi)] = True
    assert found.all(), "max_pool2d window without a valid position"
    return from_accum(best, dtype)


def avg_pool2d(x, kernel=(2, 2), stride=(2, 2), padding=(0, 0), dtype: int = DT_F32):
    """Sum over the valid positions in (kh, kw) order, divided by KH*KW whatever the padding
    (src/backends/cpu/kernels/pool.cpp:280-303); fp32 accumulate, one rounding."""
    xv = to_accum(x, dtype)
    n, c, h, wd = xv.shape
    kh, kw = kernel
    sh, sw = stride
    ph, pw = padding
    oh = conv_out_size(h, kh, sh, ph)
    ow = conv_out_size(wd, kw, sw, pw)
    acc = np.zeros((n, c, oh, ow), dtype=F32)
    for i in range(kh):
        for j in range(kw):
            ohs = np.arange(oh) * sh - ph + i
            ows = np.arange(ow) * sw - pw + j
            oi = np.nonzero((ohs >= 0) & (ohs < h))[0]
            qi = np.nonzero((ows >= 0) & (ows < wd))[0]
            if oi.size == 0 or qi.size == 0:
                continue
            vals = xv[:, :, ohs[oi]][:, :, :, ows[qi]]
            acc[:, :, oi[:, None], qi[None, :]] = (acc[:, :, oi[:, None], qi[None, :]] + vals).astype(F32)
    return from_accum((acc / F32(kh * kw)).astype(F32), dtype)


def _pool_argmax(xv, kernel, stride, padding):
    """Flat index ih*W+iw of each window's first maximum (strict >), shape [n, c, oh, ow]
    (find_window_argmax, src/backends/cpu/kernels/pool.cpp:185-208)."""
    n, c, h, wd = xv.shape
    kh, kw = kernel
    sh, sw = stride
    ph, pw = padding
    oh = conv_out_size(h, kh, sh, ph)
    ow = conv_out_size(wd, kw, sw, pw)
    best = np.zeros((n, c, oh, ow), dtype=F32)
    arg = np.full((n, c, oh, ow), -1, dtype=np.int64)
    for i in range(kh):
        for j in range(kw):
            ohs = np.arange(oh) * sh - ph + i
            ows = np.arange(ow) * sw - pw + j
            oi = np.nonzero((ohs >= 0) & (ohs < h))[0]
            qi = np.nonzero((ows >= 0) & (ows < wd))[0]
            if oi.size == 0 or qi.size == 0:
                continue
            vals = xv[:, :, ohs[oi]][:, :, :, ows[qi]]
            cur = best[:, :, oi[:, None], qi[None, :]]
            cur_arg = arg[:, :, oi[:, None], qi[None, :]]
            take = (cur_arg < 0) | (vals > cur)
            flat = (ohs[oi][:, None] * wd + ows[qi][None, :])[None, None]
            best[:, :, oi[:, None], qi[None, :]] = np.where(take, vals, cur)
            arg[:, :, oi[:, None], qi[None, :]] = np.where(take, flat, cur_arg)
    assert (arg >= 0).all(), "max_pool2d window without a valid position"
    return arg


def max_pool2d_select(g, x, kernel, stride, padding, dtype: int = DT_F32):
    """out = g at each window's argmax of x (pool.cpp:459-483); pure data movement."""
    arg = _pool_argmax(to_accum(x, dtype), kernel, stride, padding)
    n, c, oh, ow = arg.shape
    flat = np.asarray(g).reshape(n * c, -1)
    return np.take_along_axis(flat, arg.reshape(n * c, -1), axis=1).reshape(n, c, oh, ow)


def max_pool2d_grad(dy, x, kernel, stride, padding, dtype: int = DT_F32):
    """dy added into each window's argmax of x, windows in (oh, ow) order, fp32 buffer rounded once
    (pool.cpp:356-389)."""
    xv = to_accum(x, dtype)
    dyv = to_accum(dy, dtype)
    n, c, h, wd = xv.shape
    arg = _pool_argmax(xv, kernel, stride, padding)
    oh, ow = arg.shape[2:]
    acc = np.zeros((n * c, h * wd), dtype=F32)
    rows = np.arange(n * c)
    arg2 = arg.reshape(n * c, oh, ow)
    dy2 = dyv.reshape(n * c, oh, ow)
    for o in range(oh):
        for q in range(ow):
            cols = arg2[:, o, q]
            acc[rows, cols] = (acc[rows, cols] + dy2[:, o, q]).astype(F32)
    return from_accum(acc.reshape(n, c, h, wd), dtype)


def _covering(size_in, k, s, p, size_out, tap):
    """Input positions i whose window through kernel tap `tap` is a valid output position o:
    i + p - tap == o * s, 0 <= o < size_out.  Returns (i, o) index arrays."""
    i = np.arange(size_in)
    num = i + p - tap
    ok = (num >= 0) & (num % s == 0) & (num // s < size_out)
    return i[ok], (num // s)[ok]


def avg_pool2d_grad(dy, input_shape, kernel, stride, padding, dtype: int = DT_F32):
    """dx = (sum of dy over the covering windows, kh then kw ascending) / (KH*KW) (pool.cpp:542-568)."""
    dyv = to_accum(dy, dtype)
    n, c, h, wd = input_shape
    kh, kw = kernel
    sh, sw = stride
    ph, pw = padding
    oh, ow = dyv.shape[2:]
    acc = np.zeros((n, c, h, wd), dtype=F32)
    for a in range(kh):
        ih, o = _covering(h, kh, sh, ph, oh, a)
        if ih.size == 0:
            continue
        for b in range(kw):
            iw, q = _covering(wd, kw, sw, pw, ow, b)
            if iw.size == 0:
                continue
            acc[:, :, ih[:, None], iw[None, :]] = (
                acc[:, :, ih[:, None], iw[None, :]] + dyv[:, :, o[:, None], q[None, :]]).astype(F32)
    return from_accum((acc / F32(kh * kw)).astype(F32), dtype)


def conv2d_grad_input(dy, w, input_shape, stride, padding, groups: int = 1, dtype: int = DT_F32):
    """BackwardData as a gather over dx, terms in (co, kh, kw) order, rounded products added in fp32
    (src/backends/cpu/kernels/conv.cpp:321-353)."""
    dyv = to_accum(dy, dtype)
    wv = to_accum(w, dtype)
    n, cin, h, wd = input_shape
    cout, cpg, kh, kw = wv.shape
    sh, sw = stride
    ph, pw = padding
    oh, ow = dyv.shape[2:]
    copg = cout // groups
    acc = np.zeros((n, cin, h, wd), dtype=F32)
    for g in range(groups):
        cis = slice(g * cpg, (g + 1) * cpg)
        for co in range(g * copg, (g + 1) * copg):
            for a in range(kh):
                ih, o = _covering(h, kh, sh, ph, oh, a)
                if ih.size == 0:
                    continue
                for b in range(kw):
                    iw, q = _covering(wd, kw, sw, pw, ow, b)
                    if iw.size == 0:
                        continue
                    d = dyv[:, co][:, o[:, None], q[None, :]]                      # [n, |ih|, |iw|]
                    prod = (d[:, None] * wv[co, :, a, b][None, :, None, None]).astype(F32)
                    sub = acc[:, cis][:, :, ih[:, None], iw[None, :]]
                    acc[:, cis, ih[:, None], iw[None, :]] = (sub + prod).astype(F32)
    return from_accum(acc, dtype)


def conv2d_grad_filter(x, dy, filter_shape, stride, padding, groups: int = 1, dtype: int = DT_F32):
    """BackwardFilter: one dot product per filter element, terms in (n, oh, ow) order
    (src/backends/cpu/kernels/conv.cpp:424-453)."""
    xv = to_accum(x, dtype)
    dyv = to_accum(dy, dtype)
    cout, cpg, kh, kw = filter_shape
    n, cin, h, wd = xv.shape
    sh, sw = stride
    ph, pw = padding
    oh, ow = dyv.shape[2:]
    copg = cout // groups
    acc = np.zeros((cout, cpg, kh, kw), dtype=F32)
    for g in range(groups):
        cos = slice(g * copg, (g + 1) * copg)
        cis = slice(g * cpg, (g + 1) * cpg)
        for b in range(n):
            for o in range(oh):
                ihs = o * sh - ph + np.arange(kh)
                av = np.nonzero((ihs >= 0) & (ihs < h))[0]
                if av.size == 0:
                    continue
                for q in range(ow):
                    iws = q * sw - pw + np.arange(kw)
                    bv = np.nonzero((iws >= 0) & (iws < wd))[0]
                    if bv.size == 0:
                        continue
                    xs = xv[b, cis][:, ihs[av][:, None], iws[bv][None, :]]          # [cpg, |a|, |b|]
                    prod = (xs[None] * dyv[b, cos, o, q][:, None, None, None]).astype(F32)
                    sub = acc[cos][:, :, av[:, None], bv[None, :]]
                    acc[cos, :, av[:, None], bv[None, :]] = (sub + prod).astype(F32)
    return from_accum(acc, dtype)


def matmul_grad_lhs(gy, b, dtype: int = DT_F32):
    """ga[i,p] = sum_j gy[i,j]*b[p,j], j increasing (src/backends/cpu/kernels/matmul.cpp:187-232)."""
    return matmul(gy, np.ascontiguousarray(np.asarray(b).T), dtype)


def matmul_grad_rhs(a, gy, dtype: int = DT_F32):
    """gb[p,j] = sum_i a[i,p]*gy[i,j], i increasing (matmul.cpp:289-330)."""
    return matmul(np.ascontiguousarray(np.asarray(a).T), gy, dtype)


def relu_grad(x, gy, dtype: int = DT_F32):
    """x > 0 ? gy : 0 (src/backends/cpu/kernels/elementwise.cpp:411-414)."""
    xv, gv = to_accum(x, dtype), to_accum(gy, dtype)
    return from_accum(np.where(xv > 0, gv, F32(0)).astype(F32), dtype)


def mse_loss(pred, target, dtype: int = DT_F32):
    """mean((pred-target)^2): squares added one after the other in fp32, then one division
    (src/backends/cpu/kernels/loss.cpp:108-150).  Result shape ()."""
    p, t = to_accum(pred, dtype).reshape(-1), to_accum(target, dtype).reshape(-1)
    diff = (p - t).astype(F32)
    sq = (diff * diff).astype(F32)
    acc = F32(0)
    for v in sq:
        acc = F32(acc + v)
    return np.asarray(from_accum(np.asarray(F32(acc / F32(p.size)), dtype=F32), dtype)).reshape(())


def mse_loss_grad(pred, target, gy, dtype: int = DT_F32):
    """(2*gy/numel) * (pred - target), the coefficient formed first (loss.cpp:225-255)."""
    p, t = to_accum(pred, dtype), to_accum(target, dtype)
    g = F32(to_accum(np.asarray(gy), dtype).reshape(-1)[0])
    coefficient = F32(F32(F32(2.0) * g) / F32(p.size))
    return from_accum((coefficient * (p - t).astype(F32)).astype(F32), dtype)


def rfft(x):
    """x[..., n] (float32) -> [..., n//2+1, 2], forward sign, unscaled (src/ops/schemas/fft.cpp:8).
    The reference CPU kernel calls pocketfft r2c in float32; this restatement evaluates the DFT sum
    itself in float64 and rounds once, pinned by the reference's known-answer tests
    (tests/cpp/ops/test_op_fft.cpp:287-395)."""
    xv = np.asarray(x, dtype=np.float64)
    n = xv.shape[-1]
    k = n // 2 + 1
    idx = (np.arange(n)[:, None] * np.arange(k)[None, :]) % n
    ang = -2.0 * np.pi * idx / n
    re = xv @ np.cos(ang)
    im = xv @ np.sin(ang)
    return np.stack([re, im], axis=-1).astype(F32)


def irfft(z, n: int):
    """z[..., n//2+1, 2] -> [..., n], scaled by 1/n; imaginary parts of the DC and (even n) Nyquist
    bins are ignored, as a c2r transform does (src/ops/schemas/fft.cpp:9; known answers
    tests/cpp/ops/test_op_fft.cpp:477-570)."""
    zv = np.asarray(z, dtype=np.float64)
    k = n // 2 + 1
    assert zv.shape[-1] == 2 and zv.shape[-2] == k
    re, im = zv[..., 0], zv[..., 1]
    weight = np.full(k, 2.0)
    weight[0] = 1.0
    im = im.copy()
    im[..., 0] = 0.0
    if n % 2 == 0:
        weight[k - 1] = 1.0
        im[..., k - 1] = 0.0
    idx = (np.arange(k)[:, None] * np.arange(n)[None, :]) % n
    ang = 2.0 * np.pi * idx / n
    out = (re * weight) @ np.cos(ang) - (im * weight) @ np.sin(ang)
    return (out / n).astype(F32)


def gather(x, indices):
    """out[k, :] = x[indices[k], :] along axis 0 (src/ops/schemas/gather.cpp:86-118); an index
    outside [0, N) is an error."""
    idx = np.asarray(indices).astype(np.int64)
    if idx.size and (idx.min() < 0 or idx.max() >= x.shape[0]):
        raise IndexError(f"gather: index out of range [0, {x.shape[0]})")
    return np.ascontiguousarray(np.asarray(x)[idx])


def scatter_add(updates, indices, output_shape, dtype: int = DT_F32):
    """out [V, F] = 0; out[indices[k], :] += updates[k, :] in increasing k, accumulated in fp32 and
    rounded once (scatter_add / gather_grad_internal of src/backends/cpu/kernels/gather.cpp)."""
    idx = np.asarray(indices).astype(np.int64)
    v, f = output_shape
    if idx.size and (idx.min() < 0 or idx.max() >= v):
        raise IndexError(f"scatter_add: index out of range [0, {v})")
    acc = np.zeros((v, f), dtype=F32)
    u = to_accum(updates, dtype)
    for k in range(idx.shape[0]):
        acc[idx[k]] = (acc[idx[k]] + u[k]).astype(F32)
    return from_accum(acc, dtype)


def heaviside_surrogate(x, dtype: int = DT_F32):
    """Forward of the surrogate step: x >= 0 ? 1 : 0 (alpha only shapes the backward graph)."""
    return _unary(lambda v: np.where(v >= 0, F32(1), F32(0)).astype(F32), x, dtype)


# --------------------------------------------------------------------------------------
# elementwise.  src/backends/cpu/kernels/elementwise.cpp:39-56,146-163,242-255,329-404
# --------------------------------------------------------------------------------------
def _unary(fn, x, dtype):
    return from_accum(fn(to_accum(x, dtype)), dtype)


def add(a, b, dtype: int = DT_F32):
    if dtype in (DT_I32, DT_I64):
        return (np.asarray(a) + np.asarray(b)).astype(np.asarray(a).dtype)
    return from_accum(to_accum(a, dtype) + to_accum(b, dtype), dtype)


def mul(a, b, dtype: int = DT_F32):
    return from_accum(to_accum(a, dtype) * to_accum(b, dtype), dtype)


def relu(x, dtype: int = DT_F32):
    # std::max(x, 0.0f) == (x < 0) ? 0 : x : NaN and -0.0 pass through (elementwise.cpp:323-331)
    return _unary(lambda v: np.where(v < F32(0), F32(0), v).astype(F32), x, dtype)


def square(x, dtype: int = DT_F32):
    return _unary(lambda v: v * v, x, dtype)


def _sigmoid_f32(v):
    v = np.asarray(v, dtype=F32)
    with np.errstate(over="ignore"):
        pos = F32(1) / (F32(1) + np.exp(-v, dtype=F32))
        ev = np.exp(v, dtype=F32)
        neg = ev / (F32(1) + ev)
    return np.where(v >= 0, pos, neg).astype(F32)


def sigmoid(x, dtype: int = DT_F32):
    """Two-branch stable form (elementwise.cpp:346-354)."""
    return _unary(_sigmoid_f32, x, dtype)


def tanh(x, dtype: int = DT_F32):
    return _unary(lambda v: np.tanh(v, dtype=F32), x, dtype)


def rsqrt(x, dtype: int = DT_F32):
    with np.errstate(divide="ignore", invalid="ignore"):
        return _unary(lambda v: (F32(1) / np.sqrt(v, dtype=F32)).astype(F32), x, dtype)


# NEW ops (no reference implementation; parity unpinned by the reference) ---------------
_GELU_C0 = F32(0.7978845608028654)  # sqrt(2/pi)
_GELU_C1 = F32(0.044715)


def _gelu_f32(v):
    v = np.asarray(v, dtype=F32)
    inner = _GELU_C0 * (v + _GELU_C1 * (v * v * v))
    return (F32(0.5) * v * (F32(1) + np.tanh(inner, dtype=F32))).astype(F32)


def gelu(x, dtype: int = DT_F32):
    """NEW: tanh-form GELU 0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715*x^3))), fp32 math."""
    return _unary(_gelu_f32, x, dtype)


def silu(x, dtype: int = DT_F32):
    """NEW: x*sigmoid(x) with the reference's two-branch sigmoid."""
    return _unary(lambda v: (v * _sigmoid_f32(v)).astype(F32), x, dtype)


def _softplus_f32(v):
    v = np.asarray(v, dtype=F32)
    with np.errstate(over="ignore"):
        small = np.log1p(np.exp(v, dtype=F32), dtype=F32)
    return np.where(v > F32(20), v, small).astype(F32)


def softplus(x, dtype: int = DT_F32):
    """NEW: log1p(exp(x)), identity above 20 (fp32)."""
    return _unary(_softplus_f32, x, dtype)


def exp(x, dtype: int = DT_F32):
    """NEW: expf."""
    with np.errstate(over="ignore"):
        return _unary(lambda v: np.exp(v, dtype=F32), x, dtype)


def bias_add(x, bias, dtype: int = DT_F32):
    """NEW: x[..., j] + bias[j] (row-broadcast over the last axis)."""
    return from_accum(to_accum(x, dtype) + to_accum(bias, dtype), dtype)


UNARY = {"relu": relu, "square": square, "sigmoid": sigmoid, "tanh": tanh, "rsqrt": rsqrt,
         "gelu": gelu, "silu": silu, "softplus": softplus, "exp": exp}
BINARY = {"add": add, "mul": mul}


def fused_elementwise(inputs, ops: str, arities, dtype: int = DT_F32):
    """fused_elementwise_internal: segment 0 takes its operands from the external list;
    segment i>0 takes the previous result as operand 0 and the next externals for the rest;
    every intermediate is rounded to the tensor dtype
    (src/ops/fused_elementwise_utils.cpp:88-101,122-206)."""
    names = ops.split(";")
    assert len(names) == len(arities)
    assert sum(arities) - (len(names) - 1) == len(inputs)
    nxt = 0
    cur = None
    for idx, (name, ar) in enumerate(zip(names, arities)):
        operands = []
        if idx > 0:
            operands.append(cur)
        while len(operands) < ar:
            operands.append(inputs[nxt])
            nxt += 1
        if ar == 1:
            cur = UNARY[name](operands[0], dtype)
        else:
            cur = BINARY[name](operands[0], operands[1], dtype)
    return cur


# --------------------------------------------------------------------------------------
# softmax / layer_norm.  src/backends/cpu/kernels/sequence.cpp:114-174, 182-279
# --------------------------------------------------------------------------------------
def softmax(x, dtype: int = DT_F32):
    """Rank-2, last axis: max (first element seeds, strict >), e = exp(x-max), sequential
    fp32 sum in increasing j, e/sum."""
    v = to_accum(x, dtype)
    n, d = v.shape
    row_max = v[:, 0].copy()
    for j in range(1, d):
        col = v[:, j]
        row_max = np.where(col > row_max, col, row_max)
    e = np.exp(v - row_max[:, None], dtype=F32)
    s = np.zeros(n, dtype=F32)
    for j in range(d):
        s += e[:, j]
    return from_accum(e / s[:, None], dtype)


def layer_norm(x, gamma, beta, eps: float = 1e-5, dtype: int = DT_F32):
    """mean = sum/D; var = sum((x-mean)^2)/D (second pass, biased); r = 1/sqrt(var+eps);
    out = g*((x-mean)*r) + b; sums sequential in increasing j."""
    v = to_accum(x, dtype)
    g = to_accum(gamma, dtype)
    b = to_accum(beta, dtype)
    n, d = v.shape
    s = np.zeros(n, dtype=F32)
    for j in range(d):
        s += v[:, j]
    mean = s / F32(d)
    vs = np.zeros(n, dtype=F32)
    for j in range(d):
        c = v[:, j] - mean
        vs += c * c
    var = vs / F32(d)
    r = F32(1) / np.sqrt(var + F32(eps), dtype=F32)
    xhat = (v - mean[:, None]) * r[:, None]
    return from_accum(g[None, :] * xhat + b[None, :], dtype)


# --------------------------------------------------------------------------------------
# selective_scan.  src/backends/cpu/kernels/sequence.cpp:95-106
# --------------------------------------------------------------------------------------
def selective_scan(x, a, b, c, d, dtype: int = DT_F32):
    """Per row (all leading axes), time on the last axis, fp32 state, state0 = 0:
        state = a*state + b*x ;  out = c*state + d*x."""
    xv, av, bv, cv, dv = (to_accum(t, dtype) for t in (x, a, b, c, d))
    shape = xv.shape
    steps = shape[-1]
    xv, av, bv, cv, dv = (t.reshape(-1, steps) for t in (xv, av, bv, cv, dv))
    out = np.empty_like(xv)
    state = np.zeros(xv.shape[0], dtype=F32)
    for t in range(steps):
        state = av[:, t] * state + bv[:, t] * xv[:, t]
        out[:, t] = cv[:, t] * state + dv[:, t] * xv[:, t]
    return from_accum(out.reshape(shape), dtype)


def mamba_scan(u, delta, A, B, C, D, z=None):
    """NEW fused op (no reference counterpart; parity unpinned by the reference), fp32 only.
    u, delta: [Bt, L, Dm] (time-major rows as the GEMMs produce them); A: [Dm, N];
    B, C: [Bt, L, N]; D: [Dm]; optional gate z: [Bt, L, Dm].
        h[n] = exp(delta*A[d,n]) * h[n] + (delta*B[n]) * u
        y    = sum_n C[n]*h[n]  (n increasing)  + D[d]*u ;  y *= silu(z) if z is given.
    Equals selective_scan on materialised [Bt,Dm,N,L] operands + sum over N + mul/add."""
    u = np.asarray(u, dtype=F32)
    delta = np.asarray(delta, dtype=F32)
    A = np.asarray(A, dtype=F32)
    B = np.asarray(B, dtype=F32)
    C = np.asarray(C, dtype=F32)
    D = np.asarray(D, dtype=F32)
    bt, L, dm = u.shape
    n = A.shape[1]
    h = np.zeros((bt, dm, n), dtype=F32)
    y = np.empty((bt, L, dm), dtype=F32)
    for t in range(L):
        dt = delta[:, t, :]
        da = np.exp(dt[:, :, None] * A[None], dtype=F32)
        db = dt[:, :, None] * B[:, t, None, :]
        h = da * h + db * u[:, t, :, None]
        acc = np.zeros((bt, dm), dtype=F32)
        for k in range(n):
            acc = acc + C[:, t, None, k] * h[:, :, k]
        y[:, t, :] = acc + D[None, :] * u[:, t, :]
    if z is not None:
        zz = np.asarray(z, dtype=F32)
        y = (y * (zz * _sigmoid_f32(zz))).astype(F32)
    return y


# --------------------------------------------------------------------------------------
# shape ops, sum, constant.  src/backends/cpu/kernels/shape.cpp:33,73,172,276;
# reduction.cpp:130; src/ops/constant_utils.h:46-55
# --------------------------------------------------------------------------------------
def reshape(x, target_shape):
    return np.ascontiguousarray(x).reshape(target_shape)


def transpose(x, perm):
    """out.dims[i] = x.dims[perm[i]] (src/ops/schemas/shape.cpp:424-429)."""
    return np.ascontiguousarray(np.transpose(np.asarray(x), perm))


def concat(xs, axis: int):
    return np.ascontiguousarray(np.concatenate([np.asarray(t) for t in xs], axis=axis))


def slice_(x, axis: int, start: int, stop: int):
    idx = [slice(None)] * np.asarray(x).ndim
    idx[axis] = slice(start, stop)
    return np.ascontiguousarray(np.asarray(x)[tuple(idx)])


def sum_axes(x, axes, keepdims: bool = False, dtype: int = DT_F32):
    """Sum over an axis subset: fp32 accumulator, reduced positions visited in row-major order
    of the reduced axes (src/backends/cpu/kernels/reduction.cpp:130)."""
    v = to_accum(x, dtype)
    axes = sorted(a % v.ndim for a in axes)
    keep = [a for a in range(v.ndim) if a not in axes]
    moved = np.transpose(v, keep + axes)
    kshape = moved.shape[: len(keep)]
    flat = moved.reshape(int(np.prod(kshape, dtype=np.int64)), -1)
    acc = np.zeros(flat.shape[0], dtype=F32)
    for j in range(flat.shape[1]):
        acc += flat[:, j]
    out = acc.reshape(kshape)
    if keepdims:
        full = list(v.shape)
        for a in axes:
            full[a] = 1
        out = out.reshape(full)
    return from_accum(out, dtype)


def constant(values, shape, dtype: int = DT_F32):
    """double array cast to the dtype (constant_utils.h:46-55); one value = splat."""
    vals = np.asarray(values, dtype=np.float64)
    numel = int(np.prod(shape, dtype=np.int64))
    if vals.size == 1 and numel != 1:
        vals = np.full(numel, vals.reshape(-1)[0])
    if dtype in (DT_I32,):
        return vals.astype(np.int32).reshape(shape)
    if dtype in (DT_I64,):
        return vals.astype(np.int64).reshape(shape)
    return from_accum(vals.astype(F32), dtype).reshape(shape)


# --------------------------------------------------------------------------------------
# tolerance.  tests/cpp/common/tolerance.h:41-98
# --------------------------------------------------------------------------------------
TOL = {DT_F32: (1e-5, 1e-6), DT_F16: (1e-2, 1e-3), DT_BF16: (2e-2, 2e-3)}
TOL_TF32 = (1e-3, 1e-4)


def attention_fan(q, k, v, dtype: int = DT_BF16):
    """One head of the attention fan as the three reference operators in a row, each rounding
    its result to the storage dtype: matmul(q, k^T) (src/backends/cpu/kernels/matmul.cpp:92-131),
    softmax over rows (src/backends/cpu/kernels/sequence.cpp:114-174), matmul(p, v).  q: [sq, d],
    k, v: [sk, d], all in storage form."""
    kt = np.ascontiguousarray(k.T)
    return matmul(softmax(matmul(q, kt, dtype), dtype), v, dtype)


def all_close(actual, expected, dtype: int = DT_F32, rtol=None, atol=None):
    """|a-e| <= atol + rtol*|e| elementwise; NaN/inf never compare equal unless bit-equal
    in class (the reference's helper rejects them; here inf==inf of the same sign passes)."""
    a = to_accum(actual, dtype).astype(np.float64)
    e = to_accum(expected, dtype).astype(np.float64)
    if dtype in (DT_I32, DT_I64):
        return bool(np.array_equal(actual, expected))
    r, t = TOL.get(dtype, (0.0, 0.0))
    rtol = r if rtol is None else rtol
    atol = t if atol is None else atol
    if a.shape != e.shape:
        return False
    same_inf = np.isinf(a) & np.isinf(e) & (np.sign(a) == np.sign(e))
    with np.errstate(invalid="ignore"):
        ok = (np.abs(a - e) <= atol + rtol * np.abs(e)) | same_inf
    return bool(np.all(ok))


def max_err(actual, expected, dtype: int = DT_F32):
    a = to_accum(actual, dtype).astype(np.float64)
    e = to_accum(expected, dtype).astype(np.float64)
    d = np.abs(a - e)
    return float(d.max(initial=0.0)), float((d / np.maximum(np.abs(e), 1e-30)).max(initial=0.0))
