"""TEST INFRASTRUCTURE ONLY: ctypes front-ends for the two CPU checkers.

* ``Port``  - oracle/port.c, the plain-C restatement of the reference's portable CPU path.
* ``Ref``   - oracle/_ref/libdabnn_ref.so, the reference's own sources compiled with two shim
  headers and a Net glue (oracle/ref_capi.cpp).  It can only be *built* where the reference
  checkout is present; the built library travels with the repository snapshot.

Only tests/, the smoke check and the CPU-baseline leg of bench.py import this module.  Nothing in
the product package does: the product path must fail loudly without its CUDA library instead of
falling back to anything here.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_SO = HERE / "_build" / "liboracle_port.so"
REF_SO = HERE / "_ref" / "libdabnn_ref.so"
REF_NATIVE_SO = HERE / "_ref" / "libdabnn_ref_native.so"
# where the reference checkout lies: only needed to (re)build oracle/_ref, never at test or bench time
REFERENCE_ROOT = Path(os.environ["DABNN_REFERENCE"]) if os.environ.get("DABNN_REFERENCE") else None

# numeric values of flatbnn::LayerType (reference common/dab.fbs:4-5)
LAYER_TYPE = {
    "FpConv2D": 0, "AvePool": 1, "MaxPool": 2, "Relu": 3, "Softmax": 4, "FC": 5, "Add": 6,
    "Concat": 7, "BinConv2D": 8, "Affine": 9, "Binarize": 10, "Split": 11, "Shuffle": 12, "PRelu": 13,
}


def build(port: bool = True, ref: bool = True) -> None:
    """Compile the checkers (the reference one only where the reference checkout exists)."""
    targets = []
    if port:
        targets.append("port")
    if ref and REFERENCE_ROOT is not None and (REFERENCE_ROOT / "dabnn" / "bgemm.h").exists():
        targets.append("ref")
    if targets:
        env = [f"DABNN_REFERENCE={REFERENCE_ROOT}"] if "ref" in targets else []
        subprocess.run(["make", "-s", "-C", str(HERE), *env, *targets], check=True)


def out_dim(i, pad, dil, k, stride):
    return (i + 2 * pad - (dil * (k - 1) + 1)) // stride + 1


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u64(a):
    return np.ascontiguousarray(a, dtype=np.uint64)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


class Port:
    """oracle/port.c through ctypes; numpy in, numpy out."""

    kind = "port"

    def __init__(self):
        if not PORT_SO.exists():
            build(port=True, ref=False)
        self.lib = C.CDLL(str(PORT_SO))
        self.lib.port_pack_weight.restype = C.c_size_t

    def pack_mat(self, x):
        x = _f32(x)
        *lead, c = x.shape
        out = np.empty((*lead, c // 64), dtype=np.uint64)
        n = int(np.prod(lead[:-2])) if len(lead) > 2 else 1
        rc = self.lib.port_pack_mat(_p(x), n, lead[-2], lead[-1], c, _p(out))
        if rc:
            raise RuntimeError("pack_mat: C % 64 != 0 or W*C % 64 != 0")
        return out

    def pack_64(self, x):
        x = _f32(x).ravel()
        out = np.empty(x.size // 64, dtype=np.uint64)
        self.lib.port_pack_64(_p(x), _p(out), C.c_size_t(x.size))
        return out

    def pack_weight(self, wf):
        """[O][kh][kw][I] floats -> packed uint64 words (offline weight rule)."""
        wf = _f32(wf)
        o, kh, kw, ic = wf.shape
        nw = self.lib.port_pack_weight(_p(wf), o, kh, kw, ic, None)
        out = np.empty(nw, dtype=np.uint64)
        self.lib.port_pack_weight(_p(wf), o, kh, kw, ic, _p(out))
        return out

    def pad_bits(self, x, pad_h, pad_w):
        x = _u64(x)
        h, w, cw = x.shape
        out = np.empty((h + 2 * pad_h, w + 2 * pad_w, cw), dtype=np.uint64)
        self.lib.port_pad_bits(_p(x), h, w, cw, pad_h, pad_w, _p(out))
        return out

    def pad_f32(self, x, pad_h, pad_w, val=0.0):
        x = _f32(x)
        h, w, c = x.shape
        out = np.empty((h + 2 * pad_h, w + 2 * pad_w, c), dtype=np.float32)
        self.lib.port_pad_f32(_p(x), h, w, c, pad_h, pad_w, C.c_float(val), _p(out))
        return out

    def im2col(self, x, kh, kw, ph, pw, sh, sw, dh=1, dw=1):
        x = np.ascontiguousarray(x)
        h, w, c = x.shape
        oh, ow = out_dim(h, ph, dh, kh, sh), out_dim(w, pw, dw, kw, sw)
        out = np.empty((oh * ow, kh * kw * c), dtype=x.dtype)
        self.lib.port_im2col(_p(x), h, w, C.c_size_t(c * x.itemsize), kh, kw, ph, pw, sh, sw, dh, dw,
                             _p(out))
        return out

    def fused_binarize_im2col(self, x, kh, kw, ph, pw, sh, sw, dh=1, dw=1):
        x = _f32(x)
        h, w, c = x.shape
        oh, ow = out_dim(h, ph, dh, kh, sh), out_dim(w, pw, dw, kw, sw)
        words = (kh * kw * c + 127) // 128 * 2
        out = np.empty((oh * ow, words), dtype=np.uint64)
        rc = self.lib.port_fused_binarize_im2col(_p(x), h, w, c, kh, kw, ph, pw, sh, sw, dh, dw, _p(out))
        if rc:
            raise RuntimeError(f"fused_binarize_im2col rc={rc}")
        return out

    def bgemm(self, m, n, k, a, lda, b, ldb, c, ldc):
        """In place: c (float32, flat) += popcount contraction; reference operand layout."""
        assert c.dtype == np.float32 and c.flags.c_contiguous
        a, b = _u64(a), _u64(b)
        self.lib.port_bgemm(m, n, k, _p(a), lda, _p(b), ldb, _p(c), ldc)
        return c

    def baseline_bconv(self, x, weight, out_c, kh, kw, ph, pw, sh, sw, dh=1, dw=1):
        x, weight = _u64(x), _u64(weight).ravel()
        h, w, cw = x.shape
        oh, ow = out_dim(h, ph, dh, kh, sh), out_dim(w, pw, dw, kw, sw)
        out = np.empty((oh, ow, out_c), dtype=np.float32)
        rc = self.lib.port_baseline_bconv(_p(x), h, w, cw, _p(weight), C.c_size_t(weight.size), kh, kw,
                                          ph, pw, sh, sw, dh, dw, out_c, _p(out))
        if rc:
            raise RuntimeError(f"baseline_bconv rc={rc}")
        return out

    def binconv_forward(self, x, weight, out_c, kh, kw, ph, pw, sh, sw):
        x, weight = _f32(x), _u64(weight).ravel()
        h, w, c = x.shape
        oh, ow = out_dim(h, ph, 1, kh, sh), out_dim(w, pw, 1, kw, sw)
        out = np.empty((oh, ow, out_c), dtype=np.float32)
        rc = self.lib.port_binconv_forward(_p(x), h, w, c, _p(weight), C.c_size_t(weight.size), out_c,
                                           kh, kw, ph, pw, sh, sw, _p(out))
        if rc:
            raise RuntimeError(f"binconv_forward rc={rc}")
        return out

    def affine(self, x, a, b):
        x = _f32(x).copy()
        c = x.shape[-1]
        self.lib.port_affine(_p(x), C.c_size_t(x.size // c), c, _p(_f32(a)), _p(_f32(b)))
        return x

    def add(self, x, y):
        x = _f32(x).copy()
        self.lib.port_add(_p(x), _p(_f32(y)), C.c_size_t(x.size))
        return x

    def relu(self, x):
        x = _f32(x).copy()
        self.lib.port_relu(_p(x), C.c_size_t(x.size))
        return x

    def prelu(self, x, slope):
        x, slope = _f32(x).copy(), _f32(slope).ravel()
        c = x.shape[-1]
        rc = self.lib.port_prelu(_p(x), C.c_size_t(x.size // c), c, _p(slope), slope.size)
        if rc:
            raise RuntimeError("slope must have size 1 or input.channels")
        return x

    def _pool(self, fn, x, kh, kw, ph, pw, sh, sw):
        x = _f32(x)
        h, w, c = x.shape
        oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
        out = np.empty((oh, ow, c), dtype=np.float32)
        fn(_p(x), h, w, c, kh, kw, ph, pw, sh, sw, _p(out))
        return out

    def maxpool(self, x, kh, kw, ph, pw, sh, sw):
        return self._pool(self.lib.port_maxpool, x, kh, kw, ph, pw, sh, sw)

    def avepool(self, x, kh, kw, ph, pw, sh, sw):
        return self._pool(self.lib.port_avepool, x, kh, kw, ph, pw, sh, sw)

    def concat(self, a, b):
        a, b = _f32(a), _f32(b)
        out = np.empty((*a.shape[:-1], a.shape[-1] + b.shape[-1]), dtype=np.float32)
        self.lib.port_concat(_p(a), a.shape[-1], _p(b), b.shape[-1],
                             C.c_size_t(a.size // a.shape[-1]), _p(out))
        return out

    def fconv(self, x, weight, bias, ph, pw, sh, sw, dh=1, dw=1):
        x, weight = _f32(x), _f32(weight)
        h, w, c = x.shape
        oc, kh, kw, _ = weight.shape
        oh, ow = out_dim(h, ph, dh, kh, sh), out_dim(w, pw, dw, kw, sw)
        out = np.empty((oh, ow, oc), dtype=np.float32)
        bp = _p(_f32(bias)) if bias is not None else None
        self.lib.port_fconv(_p(x), h, w, c, _p(weight), bp, kh, kw, ph, pw, sh, sw, dh, dw, oc, _p(out))
        return out

    def bn_to_affine(self, scale, beta, mean, var, eps, binary_k=0, conv_bias=None):
        scale, beta, mean, var = map(_f32, (scale, beta, mean, var))
        n = scale.size
        a, b = np.empty(n, np.float32), np.empty(n, np.float32)
        cb = _p(_f32(conv_bias)) if conv_bias is not None else None
        self.lib.port_bn_to_affine(_p(scale), _p(beta), _p(mean), _p(var), C.c_float(eps), n, binary_k,
                                   cb, _p(a), _p(b))
        return a, b

    # ---- whole-graph execution over a model description (one image) --------------------------
    def run_model(self, spec, image):
        """Run `spec` (dabnn_b200.model_spec.ModelSpec) on one HWC image, layer by layer, with the
        reference's in-place aliasing rules (Affine/Add/Relu/PRelu write into their first input,
        reference common/flatbuffers_helper.h:68-73).  Returns {blob name: ndarray}."""
        blobs = {spec.input_name: _f32(image)}
        t = {ts.name: ts for ts in spec.tensors}
        for l in spec.layers:
            f = l.fields
            if l.type == "BinConv2D":
                ws = t[f["weight"]]
                o, kh, kw, _ = ws.shape
                blobs[f["output"]] = self.binconv_forward(blobs[f["input"]], ws.data, o, kh, kw,
                                                          f["pads"][0], f["pads"][1], f["strides"][0],
                                                          f["strides"][1])
            elif l.type == "FpConv2D":
                ws = t[f["weight"]]
                bias = t[f["bias"]].data if f.get("bias") else None
                blobs[f["output"]] = self.fconv(blobs[f["input"]], ws.data.reshape(ws.shape), bias,
                                                f["pads"][0], f["pads"][1], f["strides"][0],
                                                f["strides"][1])
            elif l.type == "Affine":
                y = self.affine(blobs[f["input"]], t[f["a"]].data, t[f["b"]].data)
                blobs[f["input"]][...] = y
                blobs[f["output"]] = blobs[f["input"]]
            elif l.type == "Add":
                y = self.add(blobs[f["input1"]], blobs[f["input2"]])
                blobs[f["input1"]][...] = y
                blobs[f["output"]] = blobs[f["input1"]]
            elif l.type == "Relu":
                blobs[f["input"]][...] = self.relu(blobs[f["input"]])
                blobs[f["output"]] = blobs[f["input"]]
            elif l.type == "PRelu":
                blobs[f["input"]][...] = self.prelu(blobs[f["input"]], t[f["slope"]].data)
                blobs[f["output"]] = blobs[f["input"]]
            elif l.type in ("MaxPool", "AvePool"):
                fn = self.maxpool if l.type == "MaxPool" else self.avepool
                blobs[f["output"]] = fn(blobs[f["input"]], f["kernel_shape"][0], f["kernel_shape"][1],
                                        f["pads"][0], f["pads"][1], f["strides"][0], f["strides"][1])
            elif l.type == "Concat":
                blobs[f["output"]] = self.concat(blobs[f["inputs"][0]], blobs[f["inputs"][1]])
            elif l.type == "Binarize":
                # dabnn/layers/Binarize.cpp:9: pack_mat(input, output), the output a Bit mat of c / 64 words
                blobs[f["output"]] = self.pack_mat(blobs[f["input"]])
            elif l.type == "FC":
                # The reference runtime has no FC handler (dabnn/net.cpp:263-266); the converter emits the layer
                # for Gemm (tools/onnx2bnn/OnnxConverter.cpp:429-489) with weight [units][input_size] and a bias.
                # Over an NHWC blob that is dabnn/fconv.h:14-76 with a kernel as large as the input and no padding.
                x = blobs[f["input"]]
                ws = t[f["weight"]]
                bias = t[f["bias"]].data if f.get("bias") else None
                blobs[f["output"]] = self.fconv(x, ws.data.reshape(ws.shape[0], *x.shape), bias, 0, 0, 1, 1)
            else:
                raise RuntimeError(f"Not supported op {l.type}")
        return blobs


class Ref:
    """The compiled reference (oracle/_ref/libdabnn_ref.so) through ctypes."""

    kind = "reference"

    def __init__(self, native: bool = False):
        so = REF_NATIVE_SO if native else REF_SO
        if not so.exists():
            build(port=False, ref=True)
        if not so.exists():
            raise FileNotFoundError(f"{so} is not built and the reference checkout is not present")
        self.lib = C.CDLL(str(so))
        self.lib.ref_last_error.restype = C.c_char_p
        self.lib.ref_graph_new.restype = C.c_void_p
        self.lib.ref_net_build.restype = C.c_void_p

    def _ck(self, rc):
        if rc:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def pack_mat(self, x, baseline=False):
        x = _f32(x)
        h, w, c = x.shape
        out = np.empty((h, w, c // 64), dtype=np.uint64)
        fn = self.lib.ref_baseline_pack_mat if baseline else self.lib.ref_pack_mat
        self._ck(fn(_p(x), h, w, c, _p(out)))
        return out

    def pack_64(self, x):
        x = _f32(x).ravel()
        out = np.empty(x.size // 64, dtype=np.uint64)
        self._ck(self.lib.ref_pack_64(_p(x), _p(out), C.c_size_t(x.size)))
        return out

    def pack_64_bitset(self, x64, eff_bits=64):
        x = _f32(x64).ravel()
        out = np.empty(1, dtype=np.uint64)
        self._ck(self.lib.ref_pack_64_bitset(_p(x), _p(out), C.c_size_t(eff_bits)))
        return out[0]

    def pad_bits(self, x, pad_h, pad_w):
        x = _u64(x)
        h, w, cw = x.shape
        out = np.empty((h + 2 * pad_h, w + 2 * pad_w, cw), dtype=np.uint64)
        self._ck(self.lib.ref_pad_bits(_p(x), h, w, cw * 64, pad_h, pad_w, _p(out)))
        return out

    def pad_f32(self, x, pad_h, pad_w, val=0.0):
        x = _f32(x)
        h, w, c = x.shape
        out = np.empty((h + 2 * pad_h, w + 2 * pad_w, c), dtype=np.float32)
        self._ck(self.lib.ref_pad_f32(_p(x), h, w, c, pad_h, pad_w, C.c_float(val), _p(out)))
        return out

    def im2col(self, x, kh, kw, ph, pw, sh, sw, dh=1, dw=1):
        x = np.ascontiguousarray(x)
        h, w, c = x.shape
        is_bit = x.dtype == np.uint64
        oh, ow = out_dim(h, ph, dh, kh, sh), out_dim(w, pw, dw, kw, sw)
        out = np.empty((oh * ow, kh * kw * c), dtype=x.dtype)
        self._ck(self.lib.ref_im2col(_p(x), int(is_bit), h, w, c * 64 if is_bit else c, kh, kw, ph, pw,
                                     sh, sw, dh, dw, _p(out), C.c_size_t(out.size)))
        return out

    def fused_binarize_im2col(self, x, kh, kw, ph, pw, sh, sw, dh=1, dw=1):
        x = _f32(x)
        h, w, c = x.shape
        oh, ow = out_dim(h, ph, dh, kh, sh), out_dim(w, pw, dw, kw, sw)
        words = (kh * kw * c + 127) // 128 * 2
        out = np.empty((oh * ow, words), dtype=np.uint64)
        self._ck(self.lib.ref_fused_binarize_im2col(_p(x), h, w, c, kh, kw, ph, pw, sh, sw, dh, dw,
                                                    _p(out), C.c_size_t(out.size)))
        return out

    def bgemm(self, m, n, k, a, lda, b, ldb, c, ldc, naive=False):
        assert c.dtype == np.float32 and c.flags.c_contiguous
        a, b = _u64(a), _u64(b)
        fn = self.lib.ref_bgemm_naive if naive else self.lib.ref_bgemm
        self._ck(fn(m, n, k, _p(a), lda, _p(b), ldb, _p(c), ldc))
        return c

    def baseline_bconv(self, x, weight, out_c, kh, kw, ph, pw, sh, sw, dh=1, dw=1):
        x, weight = _u64(x), _u64(weight).ravel()
        h, w, cw = x.shape
        oh, ow = out_dim(h, ph, dh, kh, sh), out_dim(w, pw, dw, kw, sw)
        out = np.empty((oh, ow, out_c), dtype=np.float32)
        self._ck(self.lib.ref_baseline_bconv(_p(x), h, w, cw * 64, _p(weight), C.c_size_t(weight.size),
                                             kh, kw, ph, pw, sh, sw, dh, dw, out_c, _p(out)))
        return out

    def bconv_3x3(self, padded, weight, out_c, stride=1):
        padded, weight = _u64(padded), _u64(weight).ravel()
        hp, wp, cw = padded.shape
        oh, ow = (hp - 3) // stride + 1, (wp - 3) // stride + 1
        out = np.zeros((oh, ow, out_c), dtype=np.float32)
        self._ck(self.lib.ref_bconv_3x3(_p(padded), hp, wp, cw * 64, _p(weight),
                                        C.c_size_t(weight.size), out_c, stride, _p(out)))
        return out

    def fconv(self, x, weight, bias, ph, pw, sh, sw, dh=1, dw=1, baseline=False):
        x, weight = _f32(x), _f32(weight)
        h, w, c = x.shape
        oc, kh, kw, _ = weight.shape
        oh, ow = out_dim(h, ph, dh, kh, sh), out_dim(w, pw, dw, kw, sw)
        out = np.zeros((oh, ow, oc), dtype=np.float32)
        if baseline:
            assert bias is None
            self._ck(self.lib.ref_baseline_fconv(_p(x), h, w, c, _p(weight), kh, kw, ph, pw, sh, sw, dh,
                                                 dw, oc, _p(out)))
        else:
            bp = _p(_f32(bias)) if bias is not None else None
            self._ck(self.lib.ref_fconv(_p(x), h, w, c, _p(weight), bp, kh, kw, ph, pw, sh, sw, dh, dw,
                                        oc, _p(out)))
        return out

    # ---- Net level --------------------------------------------------------------------------
    def build_net(self, spec, optimize=True):
        return RefNet(self, spec, optimize)

    def run_model(self, spec, image, optimize=True):
        net = self.build_net(spec, optimize)
        try:
            return net.run(image)
        finally:
            net.close()

    def _single_layer(self, ltype, x, fields, tensors=()):
        from dabnn_b200.model_spec import LayerSpec, ModelSpec  # host-side description only
        spec = ModelSpec("x", (1, *x.shape), list(tensors),
                         [LayerSpec(ltype, "l", dict(fields))])
        return self.run_model(spec, x)

    def binconv_forward(self, x, weight, out_c, kh, kw, ph, pw, sh, sw, optimize=True):
        from dabnn_b200.model_spec import TensorSpec
        x = _f32(x)
        w = TensorSpec("w", "bit", (out_c, kh, kw, x.shape[-1]), _u64(weight).ravel())
        r = self._single_layer("BinConv2D", x, dict(input="x", weight="w", output="y", pads=[ph, pw, ph, pw],
                                                    strides=[sh, sw], dilations=[1, 1]), [w])
        return r["y"]


class RefNet:
    """A reference bnn::Net built from a ModelSpec through the glue in ref_capi.cpp."""

    def __init__(self, ref: Ref, spec, optimize=True):
        self.ref, self.spec = ref, spec
        lib = ref.lib
        _, h, w, c = spec.input_shape
        g = C.c_void_p(lib.ref_graph_new(spec.input_name.encode(), h, w, c))
        try:
            for t in spec.tensors:
                shape = np.asarray(t.shape, dtype=np.uint32)
                if t.kind == "bit":
                    data = _u64(t.data).ravel()
                    ref._ck(lib.ref_graph_add_bit_tensor(g, t.name.encode(), _p(shape), _p(data),
                                                         C.c_size_t(data.size)))
                else:
                    data = _f32(t.data).ravel()
                    ref._ck(lib.ref_graph_add_float_tensor(g, t.name.encode(), _p(shape), len(t.shape),
                                                           _p(data)))
            for l in spec.layers:
                f = l.fields
                pads, strides, kernel = f.get("pads", [0, 0]), f.get("strides", [1, 1]), \
                    f.get("kernel_shape", [0, 0])
                ints = (C.c_int * 6)(pads[0], pads[1], strides[0], strides[1], kernel[0], kernel[1])
                if l.type == "Concat":
                    in0, in1 = f["inputs"]
                elif l.type == "Add":
                    in0, in1 = f["input1"], f["input2"]
                else:
                    in0, in1 = f["input"], ""
                w = f.get("weight") or f.get("a") or f.get("slope") or ""
                b = f.get("bias") or f.get("b") or ""
                ref._ck(lib.ref_graph_add_layer(g, LAYER_TYPE[l.type], l.name.encode(), in0.encode(),
                                                in1.encode(), w.encode(), b.encode(),
                                                f["output"].encode(), ints))
            self.handle = C.c_void_p(lib.ref_net_build(g, int(optimize)))
            if not self.handle:
                raise RuntimeError(lib.ref_last_error().decode())
        finally:
            lib.ref_graph_free(g)

    def run(self, image, copy=True):
        # the reference adopts the caller's pointer and in-place layers write through it
        # (dabnn/net.cpp:276-277), so run on a private copy
        x = np.array(image, dtype=np.float32, order="C", copy=True)
        self._keep = x
        self.ref._ck(self.ref.lib.ref_net_run(self.handle, _p(x)))
        names = {self.spec.input_name}
        for l in self.spec.layers:
            names.add(l.fields["output"])
        return {n: self.get_blob(n, copy) for n in names}

    def get_blob(self, name, copy=True):
        data, dims, total = C.c_void_p(), (C.c_int * 5)(), C.c_size_t()
        self.ref._ck(self.ref.lib.ref_net_get_blob(self.handle, name.encode(), C.byref(data), dims,
                                                   C.byref(total)))
        n, h, w, c, is_bit = dims
        dt = np.uint64 if is_bit else np.float32
        cnt = n * h * w * c
        arr = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint64 if is_bit else C.c_float)),
                                    shape=(cnt,)).view(dt)
        # the glue mirrors the reference's Mat(H, W, C) call, which stores w=H, h=W (square only)
        arr = arr.reshape(w, h, c) if n == 1 else arr.reshape(n, w, h, c)
        return arr.copy() if copy else arr

    def close(self):
        if getattr(self, "handle", None):
            self.ref.lib.ref_net_free(self.handle)
            self.handle = None

    def __del__(self):
        self.close()
