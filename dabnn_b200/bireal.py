"""Synthetic Bi-Real-Net-18-shaped model (random-init), expressed in dabnn layers.

The published Bi-Real-18 `.dab` files and ImageNet are not available offline, so throughput and
parity are measured on a network of the same shape with seeded random parameters:

  float stem   FpConv2D 7x7 s2 p3 (3 -> 64) + Affine(BN) + Relu + MaxPool 3x3 s2 p1
  16 blocks    BinConv2D 3x3 p1 (+ Affine = folded BN with the binary correction) + Add(shortcut),
               widths 64/128/256/512, 4 blocks per stage, first block of stages 2-4 has stride 2 and
               a real-valued downsample shortcut: AvePool 2x2 s2 -> FpConv2D 1x1 -> Affine(BN)
  head         AvePool (global, explicit kernel) -> FpConv2D 1x1 with bias (the 512 -> 1000 FC; the
               reference runtime has no FC handler, dabnn/net.cpp:263-266, so converters emit a conv)

Layer and parameter encodings follow the reference converter: weights [O][kh][kw][I], binary
weights bit-packed (`convert.bitpack_weight`), BN folded by `convert.batchnorm_to_affine`, pads in
ONNX order [top, left, bottom, right], strides [h, w].
"""
from __future__ import annotations

import zlib

import numpy as np

from .convert import batchnorm_to_affine, bitpack_weight
from .model_spec import LayerSpec, ModelSpec, TensorSpec


def _rng(seed, name):
    return np.random.Generator(np.random.PCG64([seed, zlib.crc32(name.encode())]))


def _bn(seed, name, c, binary_k=0):
    g = _rng(seed, name)
    gamma = g.uniform(0.5, 1.5, c).astype(np.float32)
    beta = g.normal(0.0, 0.1, c).astype(np.float32)
    mean = g.normal(0.0, 0.1, c).astype(np.float32)
    var = g.uniform(0.5, 1.5, c).astype(np.float32)
    return batchnorm_to_affine(gamma, beta, mean, var, 1e-5, binary_k)


def build_bireal18(image_hw=224, num_classes=1000, widths=(64, 128, 256, 512), blocks_per_stage=4,
                   in_channels=3, seed=2024) -> ModelSpec:
    """Return the ModelSpec of a Bi-Real-18-shaped network for square `image_hw` inputs."""
    tensors, layers = [], []

    def f32(name, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        tensors.append(TensorSpec(name, "f32", tuple(arr.shape), arr))
        return name

    def affine(x, c, tag, binary_k=0):
        a, b = _bn(seed, tag, c, binary_k)
        out = f"{tag}_out"
        layers.append(LayerSpec("Affine", tag, dict(input=x, a=f32(f"{tag}_a", a), b=f32(f"{tag}_b", b),
                                                    output=out)))
        return out

    def fconv(x, cin, cout, k, stride, pad, tag, bias=False):
        g = _rng(seed, tag)
        w = g.normal(0.0, np.sqrt(2.0 / (cin * k * k)), (cout, k, k, cin)).astype(np.float32)
        fields = dict(input=x, weight=f32(f"{tag}_w", w), pads=[pad] * 4, strides=[stride, stride],
                      dilations=[1, 1], output=f"{tag}_out")
        if bias:
            fields["bias"] = f32(f"{tag}_bias", g.normal(0.0, 0.01, cout).astype(np.float32))
        layers.append(LayerSpec("FpConv2D", tag, fields))
        return fields["output"]

    def bconv(x, cin, cout, stride, tag):
        g = _rng(seed, tag)
        w = np.where(g.random((cout, 3, 3, cin)) < 0.5, -1.0, 1.0).astype(np.float32)
        words, align = bitpack_weight(w)
        tensors.append(TensorSpec(f"{tag}_w", "bit", (cout, 3, 3, cin), words, align))
        layers.append(LayerSpec("BinConv2D", tag, dict(input=x, weight=f"{tag}_w", pads=[1] * 4,
                                                       strides=[stride, stride], dilations=[1, 1],
                                                       output=f"{tag}_out")))
        return f"{tag}_out"

    x = fconv("data", in_channels, widths[0], 7, 2, 3, "stem_conv")
    x = affine(x, widths[0], "stem_bn")
    layers.append(LayerSpec("Relu", "stem_relu", dict(input=x, output="stem_relu_out")))
    layers.append(LayerSpec("MaxPool", "stem_pool", dict(input="stem_relu_out", kernel_shape=[3, 3],
                                                         pads=[1] * 4, strides=[2, 2],
                                                         output="stem_pool_out")))
    x, cin = "stem_pool_out", widths[0]
    hw = ((image_hw + 6 - 7) // 2 + 1 + 2 - 3) // 2 + 1
    for s, cout in enumerate(widths):
        for blk in range(blocks_per_stage):
            tag = f"s{s + 1}b{blk + 1}"
            stride = 2 if (s > 0 and blk == 0) else 1
            y = bconv(x, cin, cout, stride, f"{tag}_bconv")
            y = affine(y, cout, f"{tag}_bn", binary_k=cin * 9)
            if stride == 2 or cin != cout:
                layers.append(LayerSpec("AvePool", f"{tag}_ds_pool",
                                        dict(input=x, kernel_shape=[2, 2], pads=[0] * 4, strides=[2, 2],
                                             output=f"{tag}_ds_pool_out")))
                sc = fconv(f"{tag}_ds_pool_out", cin, cout, 1, 1, 0, f"{tag}_ds_conv")
                sc = affine(sc, cout, f"{tag}_ds_bn")
                hw = (hw + 2 - 3) // 2 + 1
            else:
                sc = x
            layers.append(LayerSpec("Add", f"{tag}_add", dict(input1=y, input2=sc, output=f"{tag}_add_out")))
            x, cin = f"{tag}_add_out", cout
    layers.append(LayerSpec("AvePool", "head_pool", dict(input=x, kernel_shape=[hw, hw], pads=[0] * 4,
                                                         strides=[1, 1], output="head_pool_out")))
    fconv("head_pool_out", cin, num_classes, 1, 1, 0, "fc", bias=True)
    return ModelSpec("data", (1, image_hw, image_hw, in_channels), tensors, layers)


OUTPUT_BLOB = "fc_out"
