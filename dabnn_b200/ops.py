"""Kernel-level host API over torch CUDA tensors - the Python mirror of the reference's free
functions (`pack_mat`, `pad`, `im2col`, `fused_binarize_im2col`, `bgemm`, `baseline_bconv` /
`bconv_3x3`, the float layers), with the same names and argument meaning.

torch is used for device memory and streams only; every function hands raw device pointers to the
C ABI (include/dabnn_b200.h) and enqueues on torch's current CUDA stream.  Bit tensors are
torch.int64 (a uint64 word per element; view as uint64 on the host).  All entry points accept a
leading batch dimension; 3-D inputs are treated as a batch of one like the reference.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi
from .capi import ENGINES, check


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _cuda(t, dtype):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == dtype and t.is_contiguous()):
        raise TypeError(f"expected a contiguous CUDA tensor of dtype {dtype}")
    return t


def _b4(t):
    return t if t.dim() == 4 else t.unsqueeze(0)


def _eng(engine):
    return ENGINES[engine] if isinstance(engine, str) else int(engine)


def out_dim(i, pad, dil, k, stride):
    return (i + 2 * pad - (dil * (k - 1) + 1)) // stride + 1


def pack_mat(x):
    """fp32 [..., H, W, C] -> int64 bits [..., H, W, C/64]   (reference dabnn/bitpack.h:277)."""
    x4 = _b4(_cuda(x, torch.float32))
    n, h, w, c = x4.shape
    out = torch.empty((*x.shape[:-1], max(c // 64, 0)), dtype=torch.int64, device=x.device)
    check(capi.load().dabnn_pack_mat(_ptr(x4), _ptr(out), n, h, w, c, _stream()))
    return out


def pad(x, pad_h, pad_w, val=0.0):
    """Spatial padding of a bit (int64) or float tensor   (reference dabnn/pad.h:7)."""
    x4 = _b4(x)
    n, h, w, c = x4.shape
    out = torch.empty((n, h + 2 * pad_h, w + 2 * pad_w, c), dtype=x.dtype, device=x.device)
    lib = capi.load()
    if x.dtype == torch.int64:
        if val != 0.0:
            raise ValueError("val cannot be set for DataType::Bit")  # pad.h:12
        check(lib.dabnn_pad_bits(_ptr(_cuda(x4, torch.int64)), _ptr(out), n, h, w, c, pad_h, pad_w, _stream()))
    else:
        check(lib.dabnn_pad_f32(_ptr(_cuda(x4, torch.float32)), _ptr(out), n, h, w, c, pad_h, pad_w, float(val), _stream()))
    return out if x.dim() == 4 else out[0]


def im2col(x, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h=1, dil_w=1):
    """[.., H, W, C] (float or bits) -> [.., OH*OW, kh*kw*C]   (reference dabnn/im2col.h:14)."""
    x4 = _b4(x)
    n, h, w, c = x4.shape
    oh, ow = out_dim(h, pad_h, dil_h, kh, stride_h), out_dim(w, pad_w, dil_w, kw, stride_w)
    out = torch.empty((n, max(oh * ow, 0), kh * kw * c), dtype=x.dtype, device=x.device)
    check(capi.load().dabnn_im2col(_ptr(x4.contiguous()), _ptr(out), x.element_size(), n, h, w, c, kh, kw, pad_h, pad_w,
                                   stride_h, stride_w, dil_h, dil_w, _stream()))
    return out if x.dim() == 4 else out[0]


def fused_binarize_im2col(x, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h=1, dil_w=1):
    """fp32 -> bit rows of ceil(kh*kw*C/128)*2 words   (reference dabnn/fused_binarize_im2col.h:6)."""
    x4 = _b4(_cuda(x, torch.float32))
    n, h, w, c = x4.shape
    oh, ow = out_dim(h, pad_h, dil_h, kh, stride_h), out_dim(w, pad_w, dil_w, kw, stride_w)
    out = torch.empty((n, max(oh * ow, 0), (kh * kw * c + 127) // 128 * 2), dtype=torch.int64, device=x.device)
    check(capi.load().dabnn_fused_binarize_im2col(_ptr(x4), _ptr(out), n, h, w, c, kh, kw, pad_h, pad_w, stride_h,
                                                  stride_w, dil_h, dil_w, _stream()))
    return out if x.dim() == 4 else out[0]


def bgemm(m, n, k, a, lda, b, ldb, c, ldc, engine="auto"):
    """C(i,j) += sum_h popcount(A(i,h) ^ B(h,j)) with the reference's operand layout
    (reference dabnn/bgemm.h:22-24,46): a[h*lda+i], b[j*ldb+h], c[j*ldc+i]; c is updated in place."""
    check(capi.load().dabnn_bgemm(m, n, k, _ptr(_cuda(a, torch.int64)), lda, _ptr(_cuda(b, torch.int64)), ldb,
                                  _ptr(_cuda(c, torch.float32)), ldc, _eng(engine), _stream()))
    return c


def bconv(x_bits, weight, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, engine="auto"):
    """Binary convolution on packed input: mismatch counts as fp32
    (reference common/baseline.h:77 baseline_bconv; dabnn/bconv.h:855 bconv_3x3 with pad 0)."""
    x4 = _b4(_cuda(x_bits, torch.int64))
    n, h, w, cw = x4.shape
    oh, ow = out_dim(h, pad_h, 1, kh, stride_h), out_dim(w, pad_w, 1, kw, stride_w)
    out = torch.empty((n, max(oh, 0), max(ow, 0), cout), dtype=torch.float32, device=x_bits.device)
    check(capi.load().dabnn_bconv(_ptr(x4), _ptr(_cuda(weight, torch.int64)), weight.numel(), _ptr(out), n, h, w, cw,
                                  cout, kh, kw, pad_h, pad_w, stride_h, stride_w, _eng(engine), _stream()))
    return out if x_bits.dim() == 4 else out[0]


def binconv_forward(x, weight, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, engine="auto"):
    """The BinConv operator: fp32 in, fp32 mismatch counts out
    (reference dabnn/layers/BinConv.cpp:144 forward_impl)."""
    x4 = _b4(_cuda(x, torch.float32))
    n, h, w, c = x4.shape
    lib = capi.load()
    oh, ow = out_dim(h, pad_h, 1, kh, stride_h), out_dim(w, pad_w, 1, kw, stride_w)
    out = torch.empty((n, max(oh, 0), max(ow, 0), cout), dtype=torch.float32, device=x.device)
    nbytes = lib.dabnn_binconv_workspace_bytes(n, h, w, c, kh, kw, pad_h, pad_w, stride_h, stride_w)
    ws = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=x.device)
    check(lib.dabnn_binconv_forward(_ptr(x4), _ptr(_cuda(weight, torch.int64)), weight.numel(), _ptr(out), n, h, w, c,
                                    cout, kh, kw, pad_h, pad_w, stride_h, stride_w, _ptr(ws), nbytes, _eng(engine),
                                    _stream()))
    return out if x.dim() == 4 else out[0]


def binconv_forward_static(x, weight, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, engine="auto"):
    """`binconv_forward` without any allocation inside the library: the packed intermediate lives
    in the library's built-in 16 MiB device buffer.  For hosts that own all device memory
    themselves or may not call cudaMalloc where they run inference.  `out` is still the caller's
    (here: a torch tensor allocated before the call).  Calls on one device must not overlap."""
    x4 = _b4(_cuda(x, torch.float32))
    n, h, w, c = x4.shape
    oh, ow = out_dim(h, pad_h, 1, kh, stride_h), out_dim(w, pad_w, 1, kw, stride_w)
    out = torch.empty((n, max(oh, 0), max(ow, 0), cout), dtype=torch.float32, device=x.device)
    check(capi.load().dabnn_binconv_forward_static(_ptr(x4), _ptr(_cuda(weight, torch.int64)), weight.numel(), _ptr(out),
                                                   n, h, w, c, cout, kh, kw, pad_h, pad_w, stride_h, stride_w,
                                                   _eng(engine), _stream()))
    return out if x.dim() == 4 else out[0]


def bconv_block(x_bits, weight, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, a=None, b=None, shortcut=None,
                want_f32=True, want_bits=False, engine="auto"):
    """Fused BinConv -> Affine -> Add -> sign bits (see dabnn_bconv_block).  Returns (f32, bits)."""
    x4 = _b4(_cuda(x_bits, torch.int64))
    n, h, w, cw = x4.shape
    oh, ow = out_dim(h, pad_h, 1, kh, stride_h), out_dim(w, pad_w, 1, kw, stride_w)
    dev = x_bits.device
    out = torch.empty((n, oh, ow, cout), dtype=torch.float32, device=dev) if want_f32 else None
    bits = torch.empty((n, oh, ow, cout // 64), dtype=torch.int64, device=dev) if want_bits else None
    check(capi.load().dabnn_bconv_block(_ptr(x4), _ptr(_cuda(weight, torch.int64)), weight.numel(), _ptr(a), _ptr(b),
                                        _ptr(shortcut), _ptr(out), _ptr(bits), n, h, w, cw, cout, kh, kw, pad_h, pad_w,
                                        stride_h, stride_w, _eng(engine), _stream()))
    return out, bits


def binarize_u8(x):
    """fp32 -> {0,1} bytes, byte = x > 0: the byte-activation engine's counterpart of pack_mat (bitpack.h:277)."""
    x = _cuda(x, torch.float32)
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    check(capi.load().dabnn_binarize_u8(_ptr(x), _ptr(out), x.numel(), _stream()))
    return out


def bconv_u8_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w):
    return bool(capi.load().dabnn_bconv_u8_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w))


def bconv_u8_expand_weights(weight, cout, kwords):
    """Packed filters (cout rows of kwords words) -> the byte-activation engine's weight buffer (a uint8 tensor)."""
    weight = _cuda(weight, torch.int64)
    buf = torch.empty(capi.load().dabnn_bconv_u8_weight_bytes(cout, kwords), dtype=torch.uint8, device=weight.device)
    check(capi.load().dabnn_bconv_u8_expand_weights(_ptr(weight), weight.numel(), cout, kwords, _ptr(buf), _stream()))
    return buf


def bconv_u8_block(x_u8, w_expanded, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, a=None, b=None, shortcut=None,
                   want_f32=True, want_u8=False, want_bits=False):
    """The fused block of bconv_block on {0,1}-byte activations (see dabnn_bconv_u8_block).  Returns (f32, u8, bits)."""
    x4 = _cuda(x_u8, torch.uint8)
    n, h, w, cin = x4.shape
    oh, ow = out_dim(h, pad_h, 1, kh, stride_h), out_dim(w, pad_w, 1, kw, stride_w)
    dev = x4.device
    out = torch.empty((n, oh, ow, cout), dtype=torch.float32, device=dev) if want_f32 else None
    o8 = torch.empty((n, oh, ow, cout), dtype=torch.uint8, device=dev) if want_u8 else None
    bits = torch.empty((n, oh, ow, cout // 64), dtype=torch.int64, device=dev) if want_bits else None
    check(capi.load().dabnn_bconv_u8_block(_ptr(x4), _ptr(w_expanded), _ptr(a), _ptr(b), _ptr(shortcut), _ptr(out), _ptr(o8),
                                           _ptr(bits), n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w,
                                           _stream()))
    return out, o8, bits


def bconv_u8_block_pooled_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w):
    return bool(capi.load().dabnn_bconv_u8_block_pooled_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w))


def bconv_u8_block_pooled(x_u8, w_expanded, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, a=None, b=None, shortcut=None,
                          want_u8=False):
    """bconv_u8_block that also returns the 2x2 stride-2 average pooling of its fp32 result (reference
    layers/AvePool.cpp:84 on the block's output).  Returns (f32, u8 or None, pooled f32)."""
    x4 = _cuda(x_u8, torch.uint8)
    n, h, w, cin = x4.shape
    oh, ow = out_dim(h, pad_h, 1, kh, stride_h), out_dim(w, pad_w, 1, kw, stride_w)
    dev = x4.device
    out = torch.empty((n, oh, ow, cout), dtype=torch.float32, device=dev)
    o8 = torch.empty((n, oh, ow, cout), dtype=torch.uint8, device=dev) if want_u8 else None
    pooled = torch.empty((n, oh // 2, ow // 2, cout), dtype=torch.float32, device=dev)
    check(capi.load().dabnn_bconv_u8_block_pooled(_ptr(x4), _ptr(w_expanded), _ptr(a), _ptr(b), _ptr(shortcut), _ptr(out), _ptr(o8), None,
                                                  _ptr(pooled), n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, _stream()))
    return out, o8, pooled


def affine_(x, a, b):
    """In place x = a[c]*x + b[c]   (reference dabnn/layers/Affine.cpp:10)."""
    c = x.shape[-1]
    check(capi.load().dabnn_affine(_ptr(_cuda(x, torch.float32)), _ptr(_cuda(a, torch.float32)),
                                   _ptr(_cuda(b, torch.float32)), x.numel() // c, c, _stream()))
    return x


def add_(x, y):
    """In place x += y   (reference dabnn/layers/Add.cpp:7)."""
    if x.shape != y.shape:
        raise ValueError("add: shapes differ")
    check(capi.load().dabnn_add(_ptr(_cuda(x, torch.float32)), _ptr(_cuda(y, torch.float32)), x.numel(), _stream()))
    return x


def relu_(x):
    """In place max(x, 0)   (reference dabnn/layers/Relu.cpp:21)."""
    check(capi.load().dabnn_relu(_ptr(_cuda(x, torch.float32)), x.numel(), _stream()))
    return x


def prelu_(x, slope):
    """In place x<0 ? x*slope : x   (reference dabnn/layers/PRelu.cpp:6)."""
    c = x.shape[-1]
    check(capi.load().dabnn_prelu(_ptr(_cuda(x, torch.float32)), _ptr(_cuda(slope, torch.float32)), slope.numel(),
                                  x.numel() // c, c, _stream()))
    return x


def _pool(fn, x, kh, kw, pad_h, pad_w, stride_h, stride_w):
    x4 = _b4(_cuda(x, torch.float32))
    n, h, w, c = x4.shape
    oh, ow = (h + 2 * pad_h - kh) // stride_h + 1, (w + 2 * pad_w - kw) // stride_w + 1
    out = torch.empty((n, max(oh, 0), max(ow, 0), c), dtype=torch.float32, device=x.device)
    check(fn(_ptr(x4), _ptr(out), n, h, w, c, kh, kw, pad_h, pad_w, stride_h, stride_w, _stream()))
    return out if x.dim() == 4 else out[0]


def maxpool(x, kh, kw, pad_h, pad_w, stride_h, stride_w):
    """reference dabnn/layers/MaxPool.cpp:209 max_pool_fallback."""
    return _pool(capi.load().dabnn_maxpool, x, kh, kw, pad_h, pad_w, stride_h, stride_w)


def avepool(x, kh, kw, pad_h, pad_w, stride_h, stride_w):
    """reference dabnn/layers/AvePool.cpp:84 ave_pool_fallback."""
    return _pool(capi.load().dabnn_avepool, x, kh, kw, pad_h, pad_w, stride_h, stride_w)


def concat(x1, x2):
    """Channel concatenation   (reference dabnn/layers/Concat.cpp:7)."""
    out = torch.empty((*x1.shape[:-1], x1.shape[-1] + x2.shape[-1]), dtype=torch.float32, device=x1.device)
    check(capi.load().dabnn_concat(_ptr(_cuda(x1, torch.float32)), x1.shape[-1], _ptr(_cuda(x2, torch.float32)),
                                   x2.shape[-1], _ptr(out), x1.numel() // x1.shape[-1], _stream()))
    return out


def fconv(x, weight, bias, pad_h, pad_w, stride_h, stride_w, dil_h=1, dil_w=1):
    """Float convolution, weight [Cout][kh][kw][Cin]   (reference dabnn/fconv.h:14,44)."""
    x4 = _b4(_cuda(x, torch.float32))
    n, h, w, c = x4.shape
    cout, kh, kw, _ = weight.shape
    oh, ow = out_dim(h, pad_h, dil_h, kh, stride_h), out_dim(w, pad_w, dil_w, kw, stride_w)
    out = torch.empty((n, max(oh, 0), max(ow, 0), cout), dtype=torch.float32, device=x.device)
    check(capi.load().dabnn_fconv(_ptr(x4), _ptr(_cuda(weight, torch.float32)), _ptr(bias), _ptr(out), n, h, w, c, cout,
                                  kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, _stream()))
    return out if x.dim() == 4 else out[0]


def fconv_maxpool_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w):
    return bool(capi.load().dabnn_fconv_maxpool_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w))


def fconv_maxpool(x, weight, bias, pad_h, pad_w, stride_h, stride_w, a=None, b=None, relu=False, want_u8=False):
    """Float convolution (+ bias, affine, relu) followed by a 3x3 stride-2 pad-1 max pooling, in one kernel (the stem of
    a ResNet: reference dabnn/fconv.h:14 -> Affine.cpp:10 -> Relu.cpp:21 -> MaxPool.cpp:209).  Returns (pooled fp32,
    sign bytes or None)."""
    x4 = _b4(_cuda(x, torch.float32))
    n, h, w, c = x4.shape
    cout, kh, kw, _ = weight.shape
    oh, ow = out_dim(h, pad_h, 1, kh, stride_h), out_dim(w, pad_w, 1, kw, stride_w)
    ph, pw = (oh - 1) // 2 + 1, (ow - 1) // 2 + 1
    out = torch.empty((n, ph, pw, cout), dtype=torch.float32, device=x.device)
    o8 = torch.empty((n, ph, pw, cout), dtype=torch.uint8, device=x.device) if want_u8 else None
    check(capi.load().dabnn_fconv_maxpool(_ptr(x4), _ptr(_cuda(weight, torch.float32)), _ptr(bias), _ptr(a), _ptr(b), int(relu), _ptr(out),
                                          _ptr(o8), n, h, w, c, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, _stream()))
    return out, o8


def measure_engine_peak(engine):
    """Register-resident peak of one contraction instruction in bit-op/s."""
    v = C.c_double()
    check(capi.load().dabnn_measure_engine_peak(_eng(engine), C.byref(v)))
    return v.value


def measure_tf32_peak():
    """Issue-bound rate of tcgen05.mma kind::tf32 in FLOP/s (the float convolution's denominator)."""
    v = C.c_double()
    check(capi.load().dabnn_measure_tf32_peak(C.byref(v)))
    return v.value


def engine_status():
    """0, or the code of the first bounded wait that gave up inside a tcgen05 kernel (synchronises)."""
    v = C.c_int()
    check(capi.load().dabnn_engine_status(C.byref(v)))
    return v.value


def last_engine():
    """Name of the engine the most recent bgemm / bconv / bconv_block / binconv_forward call of this thread launched
    (a "tcgen05" request falls back to "imma" for shapes the tensor-memory kernel does not take)."""
    code = capi.load().dabnn_last_engine()
    return next(k for k, v in ENGINES.items() if v == code)
