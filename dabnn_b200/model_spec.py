"""In-memory description of a dabnn model: the same information a `.dab` file carries.

Mirrors the reference's FlatBuffers schema (common/dab.fbs:1-153): a model is one input, a list of
initializer tensors (bit-packed uint64 or float32) and a list of layers whose parameters are blob /
tensor names plus small integer lists.  `dab_format` turns a ModelSpec into `.dab` bytes and back.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

# flatbnn::LayerType (reference common/dab.fbs:4-5)
LAYER_TYPES = ["FpConv2D", "AvePool", "MaxPool", "Relu", "Softmax", "FC", "Add", "Concat",
               "BinConv2D", "Affine", "Binarize", "Split", "Shuffle", "PRelu"]
MODEL_VERSION = 2  # reference common/macros.h:6 BNN_LATEST_MODEL_VERSION


@dataclass
class TensorSpec:
    name: str
    kind: str                 # "bit" (uint64 words) or "f32"
    shape: tuple              # bit / 4-D float: (O, kh, kw, I); 1-D float: (n,)
    data: np.ndarray
    align_hwc_to_128: bool = False   # reference dab.fbs:13, set by the converter iff I != 64


@dataclass
class LayerSpec:
    type: str                 # one of LAYER_TYPES
    name: str
    fields: dict = field(default_factory=dict)


@dataclass
class ModelSpec:
    input_name: str
    input_shape: tuple        # (1, H, W, C), NHWC
    tensors: list
    layers: list
    version: int = MODEL_VERSION
