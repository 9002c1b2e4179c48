"""The three data transforms of the reference's offline converter (tools/onnx2bnn), in numpy.

Only the numeric transforms are restated - weight transposition, weight bit-packing and the
BatchNorm -> Affine fold with the binary-conv correction.  The ONNX graph passes that recognise
binary convolutions live in an un-vendored fork of onnx and are not part of this package.
"""
from __future__ import annotations

import numpy as np


def onnx_weight_to_bnn(w_oihw: np.ndarray) -> np.ndarray:
    """OIHW -> [O][kh][kw][I] (reference tools/onnx2bnn/OnnxConverter.h:130-152 OnnxToBnn)."""
    return np.ascontiguousarray(np.transpose(w_oihw, (0, 2, 3, 1)))


def sign_pack(x: np.ndarray) -> np.ndarray:
    """Last axis (multiple of 64) -> uint64 words, bit i = (x[..., 64*j + i] > 0), LSB first
    (reference common/common_bitpack.h:12-34)."""
    bits = (np.asarray(x) > 0).astype(np.uint8)
    packed = np.packbits(bits.reshape(*bits.shape[:-1], -1, 8), axis=-1, bitorder="little")
    return np.ascontiguousarray(packed.reshape(*bits.shape[:-1], -1)).view(np.uint64)


def bitpack_weight(w_ohwi: np.ndarray):
    """[O][kh][kw][I] float weights -> (flat uint64 words, align_hwc_to_128).

    Reference tools/onnx2bnn/OnnxConverter.cpp:121-156: when I == 64 the whole tensor is packed
    contiguously (kh*kw words per filter); otherwise each filter's kh*kw*I values are zero-extended
    to a multiple of 128 before packing, and the tensor is flagged align_hwc_to_128.
    """
    o, kh, kw, i = w_ohwi.shape
    hwc = kh * kw * i
    flat = np.asarray(w_ohwi, dtype=np.float32).reshape(o, hwc)
    if i == 64:
        return sign_pack(flat).reshape(-1), False
    padded = np.zeros((o, (hwc + 127) // 128 * 128), dtype=np.float32)
    padded[:, :hwc] = flat
    return sign_pack(padded).reshape(-1), True


def batchnorm_to_affine(scale, beta, mean, var, eps=1e-5, binary_k=0, conv_bias=None):
    """BatchNorm -> per-channel (a, b) of the Affine layer, in float32 like the converter.

    Reference tools/onnx2bnn/OnnxConverter.cpp:583-639 CalculateCoeff.  With `binary_k` =
    Cin*kh*kw > 0 (the BN follows a binary conv, whose runtime output is the XOR mismatch count m):
    b += K*a, optional conv bias folded as b += a*bias, then a *= -2, so that
    a*m + b == a0*(K - 2m) + b0.
    """
    f = np.float32
    scale, beta, mean, var = (np.asarray(v, dtype=f) for v in (scale, beta, mean, var))
    t = np.sqrt(var + f(eps), dtype=f)
    a = (scale / t).astype(f)
    b = (beta - (scale * mean).astype(f) / t).astype(f)
    if binary_k:
        b = (b + (f(binary_k) * a).astype(f)).astype(f)
        if conv_bias is not None:
            b = (b + (a * np.asarray(conv_bias, dtype=f)).astype(f)).astype(f)
        a = (a * f(-2)).astype(f)
    return a, b
