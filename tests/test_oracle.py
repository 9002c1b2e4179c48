"""Pins the CPU oracle: the plain-C restatement (oracle/port.c) against
(1) fixtures generated from the reference's own compiled sources (tests/golden/make_golden.py),
(2) the reference's one literal golden vector (tests/im2col_test.cpp: a 4x4x2 ramp whose im2col
    equals the NHWC linear index of each tap, zero outside), and
(3) the compiled reference itself, live, on the shapes of the reference's own tests
    (tests/bgemm_test.cpp, tests/bconv_test.cpp, tests/bitpack_test.cpp) - skipped where the
    compiled reference is not available.
Integer / bit results must be identical; float layers must be bit-identical too except the float
convolution, whose summation order differs from Eigen's (tolerance 1e-5 absolute, the reference's
own Mat::operator== tolerance, dabnn/mat.h:314).
"""
from pathlib import Path

import numpy as np
import pytest

from dabnn_b200.bireal import build_bireal18
from dabnn_b200.convert import batchnorm_to_affine, bitpack_weight, sign_pack

G = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def k():
    return np.load(G / "kernels.npz")


def same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and a.tobytes() == b.tobytes()


# ------------------------------------------------------------------ (1) port vs golden fixtures
def test_pack_golden(port, k):
    assert same_bits(port.pack_mat(k["pack_edge_in"]), k["ref_pack_edge"])
    assert same_bits(port.pack_mat(k["pack_in"]), k["ref_pack"])
    # strict '>' : zeros, negative zero and NaN give bit 0
    x = np.zeros(64, np.float32)
    x[1], x[2], x[3], x[4] = -0.0, np.nan, 1e-45, np.inf
    assert int(port.pack_64(x)[0]) == (1 << 3) | (1 << 4)


def test_pad_im2col_golden(port, k):
    assert same_bits(port.pad_bits(k["pad_in"], 1, 2), k["ref_pad_1_2"])
    assert same_bits(port.im2col(k["pad_in"], 3, 3, 1, 1, 2, 2), k["ref_im2col_bits_3x3_p1_s2"])
    assert same_bits(port.fused_binarize_im2col(k["fbi_in64"], 3, 3, 1, 1, 1, 1), k["ref_fbi_64_3x3_p1_s1"])
    assert same_bits(port.fused_binarize_im2col(k["fbi_in128"], 3, 3, 1, 1, 2, 2), k["ref_fbi_128_3x3_p1_s2"])
    assert same_bits(port.fused_binarize_im2col(k["fbi_in32"], 5, 5, 2, 2, 1, 1), k["ref_fbi_32_5x5_p2_s1"])


def test_im2col_reference_ramp(port):
    x = np.arange(32, dtype=np.float32).reshape(4, 4, 2)
    col = port.im2col(x, 3, 3, 1, 1, 1, 1).reshape(4, 4, 3, 3, 2)
    for oy in range(4):
        for ox in range(4):
            for ky in range(3):
                for kx in range(3):
                    y, xx = oy - 1 + ky, ox - 1 + kx
                    exp = x[y, xx] if 0 <= y < 4 and 0 <= xx < 4 else np.zeros(2, np.float32)
                    assert np.array_equal(col[oy, ox, ky, kx], exp)
    # spot values of the reference's literal table: row 0 and row 5
    flat = col.reshape(16, 18)
    assert flat[0].tolist() == [0] * 8 + [0, 1, 2, 3, 0, 0, 8, 9, 10, 11]
    assert flat[5].tolist() == [0, 1, 2, 3, 4, 5, 8, 9, 10, 11, 12, 13, 16, 17, 18, 19, 20, 21]


def test_bgemm_golden(port, k):
    a, b, c0 = k["bgemm_a"], k["bgemm_b"], k["bgemm_c0"]
    kk, m = a.shape
    n = b.shape[0]
    c = port.bgemm(m, n, kk, a, m, b, kk, c0.copy().ravel(), m).reshape(n, m)
    assert same_bits(c, k["ref_bgemm"])


def test_bconv_golden(port, k):
    x, w = k["bconv_in"], k["bconv_w"]
    assert same_bits(port.baseline_bconv(x, w, 8, 3, 3, 1, 1, 1, 1), k["ref_bconv_c64_p1_s1"])
    assert same_bits(port.baseline_bconv(x, w, 8, 3, 3, 1, 1, 2, 2), k["ref_bconv_c64_p1_s2"])
    # bconv_3x3 on the padded input == baseline_bconv with pad 1 (reference tests/bconv_test.cpp)
    assert same_bits(k["ref_bconv3x3_padded"], k["ref_bconv_c64_p1_s1"])
    assert same_bits(port.baseline_bconv(port.pad_bits(x, 1, 1), w, 8, 3, 3, 0, 0, 1, 1), k["ref_bconv3x3_padded"])


@pytest.mark.parametrize("cin,cout,stride", [(64, 64, 1), (128, 64, 2), (192, 16, 1)])
def test_binconv_golden(port, k, cin, cout, stride):
    out = port.binconv_forward(k[f"binconv_in_{cin}"], k[f"binconv_w_{cin}"], cout, 3, 3, 1, 1, stride, stride)
    assert same_bits(out, k[f"ref_binconv_{cin}_{cout}_s{stride}"])


def test_float_layers_golden(port, k):
    x, a, b, other = k["fl_in"], k["fl_a"], k["fl_b"], k["fl_other"][0]
    assert same_bits(port.affine(x, a, b), k["ref_affine"])
    assert same_bits(port.add(x, other), k["ref_add"])
    assert same_bits(port.relu(x), k["ref_relu"])
    assert same_bits(port.prelu(x, a), k["ref_prelu_c"])
    assert same_bits(port.prelu(x, a[:1]), k["ref_prelu_1"])
    assert same_bits(port.maxpool(x, 3, 3, 1, 1, 2, 2), k["ref_maxpool_3_p1_s2"])
    assert same_bits(port.avepool(x, 3, 3, 1, 1, 2, 2), k["ref_avepool_3_p1_s2"])
    assert same_bits(port.avepool(x, 2, 2, 0, 0, 2, 2), k["ref_avepool_2_p0_s2"])
    assert same_bits(port.concat(x, other), k["ref_concat"])
    np.testing.assert_allclose(port.fconv(x, k["fconv_w"], k["fconv_bias"], 1, 1, 2, 2),
                               k["ref_fconv_p1_s2_bias"], rtol=0, atol=1e-5)
    np.testing.assert_allclose(port.fconv(x, k["fconv_w"], None, 0, 0, 1, 1), k["ref_fconv_p0_s1"],
                               rtol=0, atol=1e-5)


def test_bireal64_golden(port):
    g = np.load(G / "bireal64.npz")
    spec = build_bireal18(image_hw=64, num_classes=100)
    blobs = port.run_model(spec, g["image"])
    for name in ["stem_pool_out", "s1b1_bconv_out", "s1b1_add_out", "s2b1_add_out", "s3b1_add_out",
                 "s4b4_add_out", "head_pool_out", "fc_out"]:
        ref = g[f"ref_{name}"]
        np.testing.assert_allclose(blobs[name], ref, rtol=1e-4, atol=1e-4 * np.abs(ref).max(), err_msg=name)


# ------------------------------------------------------------------ host-side converter transforms
def test_converter_transforms(port):
    rng = np.random.default_rng(3)
    for shape in [(8, 3, 3, 64), (4, 3, 3, 128), (4, 3, 3, 192), (3, 1, 1, 256), (2, 5, 5, 32)]:
        w = rng.normal(size=shape).astype(np.float32)
        words, align = bitpack_weight(w)
        assert align == (shape[-1] != 64)
        assert same_bits(words, port.pack_weight(w))
    x = rng.normal(size=(5, 128)).astype(np.float32)
    assert same_bits(sign_pack(x), port.pack_64(x).reshape(5, 2))
    sc, be, mu, var = (rng.uniform(0.5, 1.5, 16).astype(np.float32) for _ in range(4))
    for kbin in (0, 576):
        a, b = batchnorm_to_affine(sc, be, mu, var, 1e-5, kbin)
        pa, pb = port.bn_to_affine(sc, be, mu, var, 1e-5, kbin)
        assert same_bits(a, pa) and same_bits(b, pb)


# ------------------------------------------------------------------ (3) port vs compiled reference
def test_live_pack_and_quirks(port, ref):
    rng = np.random.default_rng(0)
    x = (rng.normal(size=(64, 64, 256)) / 10).astype(np.float32)      # tests/bitpack_test.cpp:38-60
    assert same_bits(port.pack_mat(x), ref.pack_mat(x))
    assert same_bits(ref.pack_mat(x), ref.pack_mat(x, baseline=True))
    x64 = rng.normal(size=64).astype(np.float32)
    for eff in (64, 17, 0):
        exp = sum(1 << i for i in range(eff) if x64[i] > 0)
        assert int(ref.pack_64_bitset(x64, eff)) == exp


@pytest.mark.parametrize("m,n,kk", [(159, 253, 68), (128, 784, 18), (256, 196, 36), (512, 49, 72)])
def test_live_bgemm_reference_test_shapes(port, ref, m, n, kk):   # tests/bgemm_test.cpp
    rng = np.random.default_rng(m)
    a = rng.integers(0, 2**64, m * kk, dtype=np.uint64)
    b = rng.integers(0, 2**64, kk * n, dtype=np.uint64)
    c_ref = ref.bgemm(m, n, kk, a, m, b, kk, np.zeros(m * n, np.float32), m)
    c_naive = ref.bgemm(m, n, kk, a, m, b, kk, np.zeros(m * n, np.float32), m, naive=True)
    c_port = port.bgemm(m, n, kk, a, m, b, kk, np.zeros(m * n, np.float32), m)
    assert same_bits(c_ref, c_naive) and same_bits(c_ref, c_port)


@pytest.mark.parametrize("cin,cout,stride", [(64, 64, 1), (64, 64, 2), (128, 128, 1), (128, 256, 2),
                                             (256, 256, 1), (512, 256, 1)])
def test_live_bconv_reference_test_shapes(port, ref, cin, cout, stride):   # tests/bconv_test.cpp:164-431
    rng = np.random.default_rng(cin + cout)
    hw = 16                      # the reference uses 64x64; same code path, smaller to stay fast
    x = rng.integers(0, 2**64, (hw, hw, cin // 64), dtype=np.uint64)
    w = rng.integers(0, 2**64, cout * 9 * cin // 64, dtype=np.uint64)
    exp = ref.baseline_bconv(x, w, cout, 3, 3, 1, 1, stride, stride)
    assert same_bits(ref.bconv_3x3(ref.pad_bits(x, 1, 1), w, cout, stride), exp)
    assert same_bits(port.baseline_bconv(x, w, cout, 3, 3, 1, 1, stride, stride), exp)


def test_live_two_reference_paths_agree(port, ref):
    """pack_mat + baseline_bconv and fused_binarize_im2col + bgemm_naive give the same counts."""
    rng = np.random.default_rng(5)
    cin, cout, hw = 128, 32, 10
    x = rng.uniform(-1, 1, (hw, hw, cin)).astype(np.float32)
    w = rng.integers(0, 2**64, cout * 18, dtype=np.uint64)
    direct = ref.baseline_bconv(ref.pack_mat(x), w, cout, 3, 3, 1, 1, 1, 1)
    assert same_bits(ref.binconv_forward(x, w, cout, 3, 3, 1, 1, 1, 1), direct)
    assert same_bits(port.binconv_forward(x, w, cout, 3, 3, 1, 1, 1, 1), direct)


def test_live_net_optimize_flag(ref):
    """tests/net_test.cpp:29-50: optimize=false and optimize=true give equal outputs."""
    spec = build_bireal18(image_hw=32, num_classes=10)
    img = np.ones((32, 32, 3), np.float32)
    a = ref.run_model(spec, img, optimize=True)["fc_out"]
    b = ref.run_model(spec, img, optimize=False)["fc_out"]
    assert same_bits(a, b)


# ------------------------------------------------------------------ converter transforms and the layers beyond the reference runtime
@pytest.mark.parametrize("cin,cout,ks", [(64, 16, 3), (128, 8, 1), (32, 8, 3)])
def test_batchnorm_fold_is_batchnorm_of_the_signed_dot_product(port, cin, cout, ks):
    """tools/onnx2bnn/OnnxConverter.cpp:583-639 (b += K*a; a *= -2) is correct iff Affine(BinConv mismatch count)
    equals BatchNorm of the +-1 dot product (docs/onnx2bnn.md:9-13).  That identity pins the restated fold without
    the converter binary: dot product in float64, no padding (the reference pads with -1), 1e-5 of the largest output."""
    from dabnn_b200.convert import batchnorm_to_affine, bitpack_weight
    rng = np.random.default_rng(cin * 3 + cout)
    x = rng.normal(0, 1, (7, 7, cin)).astype(np.float32)
    wf = np.where(rng.random((cout, ks, ks, cin)) < 0.5, -1.0, 1.0).astype(np.float32)
    scale, beta = rng.uniform(0.5, 1.5, cout).astype(np.float32), rng.normal(0, 0.1, cout).astype(np.float32)
    mean, var = rng.normal(0, 3.0, cout).astype(np.float32), rng.uniform(0.5, 1.5, cout).astype(np.float32)
    K = ks * ks * cin
    a, b = batchnorm_to_affine(scale, beta, mean, var, 1e-5, binary_k=K)
    pa, pb = port.bn_to_affine(scale, beta, mean, var, 1e-5, binary_k=K)
    assert a.tobytes() == pa.tobytes() and b.tobytes() == pb.tobytes()
    wb, _ = bitpack_weight(wf)
    assert wb.tobytes() == port.pack_weight(wf).tobytes()
    cnt = port.binconv_forward(x, wb, cout, ks, ks, 0, 0, 1, 1)
    got = port.affine(cnt, a, b)
    xs = np.where(x > 0, 1.0, -1.0)
    oh = 7 - ks + 1
    dot = np.zeros((oh, oh, cout))
    for ky in range(ks):
        for kx in range(ks):
            dot += np.einsum("hwc,oc->hwo", xs[ky:ky + oh, kx:kx + oh, :], wf[:, ky, kx, :].astype(np.float64))
    assert np.array_equal(cnt, ((K - dot) / 2).astype(np.float32))            # Q3: the layer's output is the mismatch count
    bn = (dot - mean.astype(np.float64)) / np.sqrt(var.astype(np.float64) + 1e-5) * scale + beta
    np.testing.assert_allclose(got, bn, rtol=0, atol=1e-5 * np.abs(bn).max())
    # with a convolution bias folded in (OnnxConverter.cpp:617-623): BatchNorm sees dot + bias
    bias = rng.normal(0, 2.0, cout).astype(np.float32)
    a2, b2 = batchnorm_to_affine(scale, beta, mean, var, 1e-5, binary_k=K, conv_bias=bias)
    bn2 = (dot + bias - mean.astype(np.float64)) / np.sqrt(var.astype(np.float64) + 1e-5) * scale + beta
    np.testing.assert_allclose(port.affine(cnt, a2, b2), bn2, rtol=0, atol=1e-5 * np.abs(bn2).max())


def test_run_model_fc_and_binarize(port):
    """The checker's FC (a full-size valid fconv, dabnn/fconv.h:14-76) is a matrix product over the NHWC-flattened
    blob plus bias; its Binarize (dabnn/layers/Binarize.cpp:9) is pack_mat."""
    from dabnn_b200.model_spec import LayerSpec, ModelSpec, TensorSpec
    rng = np.random.default_rng(8)
    w = rng.normal(0, 0.1, (6, 4 * 4 * 64)).astype(np.float32)
    bias = rng.normal(0, 1, 6).astype(np.float32)
    spec = ModelSpec("data", (1, 4, 4, 64), [TensorSpec("w", "f32", w.shape, w), TensorSpec("b", "f32", (6,), bias)],
                     [LayerSpec("Binarize", "bin", dict(input="data", output="bits")),
                      LayerSpec("FC", "fc", dict(input="data", weight="w", bias="b", output="fc"))])
    x = rng.normal(0, 1, (4, 4, 64)).astype(np.float32)
    out = port.run_model(spec, x)
    np.testing.assert_allclose(out["fc"].ravel(), w.astype(np.float64) @ x.ravel().astype(np.float64) + bias, rtol=1e-5, atol=1e-5)
    assert out["bits"].shape == (4, 4, 1) and out["bits"].tobytes() == port.pack_mat(x).tobytes()
    word = int(out["bits"][1, 2, 0])
    assert [(word >> i) & 1 for i in range(64)] == [int(v > 0) for v in x[1, 2]]
