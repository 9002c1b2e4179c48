"""Regenerates tests/golden/*.npz from the reference's own code.

Every array named `ref_*` below is an output of the reference sources compiled into
oracle/_ref/libdabnn_ref.so (see oracle/Makefile), produced in a container that has the reference
checkout.  The fixtures pin the plain-C restatement (oracle/port.c) and the CUDA kernels where the
compiled reference is not available.  Run:  python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from dabnn_b200.bireal import build_bireal18  # noqa: E402
from oracle.oracle import Ref  # noqa: E402

OUT = Path(__file__).resolve().parent


def edge_floats():
    """Inputs on which `> 0` is delicate: zeros, denormals, infinities, NaNs (both signs)."""
    specials = np.array([0.0, -0.0, 1e-45, -1e-45, 1.17549435e-38, -1.17549435e-38, np.inf, -np.inf,
                         np.nan, -np.nan, 1.0, -1.0, 3.4028235e38, -3.4028235e38, 1e-20, -1e-20],
                        dtype=np.float32)
    rng = np.random.default_rng(7)
    x = rng.uniform(-1, 1, (4, 4, 128)).astype(np.float32)
    idx = rng.integers(0, specials.size, x.shape)
    mask = rng.random(x.shape) < 0.5
    x[mask] = specials[idx[mask]]
    return x


def main():
    ref = Ref()
    rng = np.random.default_rng(20240607)
    g = {}
    # --- bit packing -------------------------------------------------------------------------
    g["pack_edge_in"] = edge_floats()
    g["ref_pack_edge"] = ref.pack_mat(g["pack_edge_in"])
    x = rng.uniform(-1, 1, (6, 8, 192)).astype(np.float32)
    g["pack_in"], g["ref_pack"] = x, ref.pack_mat(x)
    # --- pad / im2col / fused binarize-im2col ----------------------------------------------------
    bits = rng.integers(0, 2**64, (5, 6, 2), dtype=np.uint64)
    g["pad_in"], g["ref_pad_1_2"] = bits, ref.pad_bits(bits, 1, 2)
    g["ref_im2col_bits_3x3_p1_s2"] = ref.im2col(bits, 3, 3, 1, 1, 2, 2)
    xf = rng.uniform(-1, 1, (7, 6, 64)).astype(np.float32)
    g["fbi_in64"] = xf
    g["ref_fbi_64_3x3_p1_s1"] = ref.fused_binarize_im2col(xf, 3, 3, 1, 1, 1, 1)
    xf = rng.uniform(-1, 1, (6, 6, 128)).astype(np.float32)
    g["fbi_in128"] = xf
    g["ref_fbi_128_3x3_p1_s2"] = ref.fused_binarize_im2col(xf, 3, 3, 1, 1, 2, 2)
    xf = rng.uniform(-1, 1, (5, 5, 32)).astype(np.float32)
    g["fbi_in32"] = xf
    g["ref_fbi_32_5x5_p2_s1"] = ref.fused_binarize_im2col(xf, 5, 5, 2, 2, 1, 1)
    # --- bgemm (reference operand layout, accumulating) ----------------------------------------------
    m, n, k = 37, 29, 5
    a = rng.integers(0, 2**64, (k, m), dtype=np.uint64)      # A(i,h) = a[h*lda + i]
    b = rng.integers(0, 2**64, (n, k), dtype=np.uint64)      # B(h,j) = b[j*ldb + h]
    c0 = rng.integers(0, 5, (n, m)).astype(np.float32)       # C(i,j) = c[j*ldc + i]
    g["bgemm_a"], g["bgemm_b"], g["bgemm_c0"] = a, b, c0
    g["ref_bgemm"] = ref.bgemm(m, n, k, a, m, b, k, c0.copy().ravel(), m).reshape(n, m)
    # --- baseline_bconv / bconv_3x3 -------------------------------------------------------------
    xb = rng.integers(0, 2**64, (5, 6, 1), dtype=np.uint64)
    wb = rng.integers(0, 2**64, 8 * 9, dtype=np.uint64)
    g["bconv_in"], g["bconv_w"] = xb, wb
    g["ref_bconv_c64_p1_s1"] = ref.baseline_bconv(xb, wb, 8, 3, 3, 1, 1, 1, 1)
    g["ref_bconv_c64_p1_s2"] = ref.baseline_bconv(xb, wb, 8, 3, 3, 1, 1, 2, 2)
    g["ref_bconv3x3_padded"] = ref.bconv_3x3(ref.pad_bits(xb, 1, 1), wb, 8, 1)
    # --- BinConv operator (float in, counts out) --------------------------------------------------
    for cin, cout, hw, stride in [(64, 64, 8, 1), (128, 64, 6, 2), (192, 16, 4, 1)]:
        xf = rng.uniform(-1, 1, (hw, hw, cin)).astype(np.float32)
        kw_ = 9 * cin // 64 if cin == 64 else (9 * cin + 127) // 128 * 2
        w = rng.integers(0, 2**64, cout * kw_, dtype=np.uint64)
        if cin != 64 and (9 * cin) % 128:
            w.reshape(cout, kw_)[:, -1] = 0            # converter zero-pads the 128-bit tail
        g[f"binconv_in_{cin}"], g[f"binconv_w_{cin}"] = xf, w
        g[f"ref_binconv_{cin}_{cout}_s{stride}"] = ref.binconv_forward(xf, w, cout, 3, 3, 1, 1, stride, stride)
    # --- float layers, through the reference Net glue ---------------------------------------------
    from dabnn_b200.model_spec import TensorSpec
    xf = rng.normal(0, 1, (6, 6, 8)).astype(np.float32)
    a_ = rng.uniform(0.5, 1.5, 8).astype(np.float32)
    b_ = rng.normal(0, 1, 8).astype(np.float32)
    other = rng.normal(0, 1, (1, 6, 6, 8)).astype(np.float32)
    g["fl_in"], g["fl_a"], g["fl_b"], g["fl_other"] = xf, a_, b_, other
    ta, tb = TensorSpec("a", "f32", (8,), a_), TensorSpec("b", "f32", (8,), b_)
    g["ref_affine"] = ref._single_layer("Affine", xf, dict(input="x", a="a", b="b", output="y"), [ta, tb])["y"]
    g["ref_add"] = ref._single_layer("Add", xf, dict(input1="x", input2="o", output="y"),
                                     [TensorSpec("o", "f32", other.shape, other)])["y"]
    g["ref_relu"] = ref._single_layer("Relu", xf, dict(input="x", output="y"))["y"]
    g["ref_prelu_c"] = ref._single_layer("PRelu", xf, dict(input="x", slope="a", output="y"), [ta])["y"]
    g["ref_prelu_1"] = ref._single_layer("PRelu", xf, dict(input="x", slope="s", output="y"),
                                         [TensorSpec("s", "f32", (1,), a_[:1])])["y"]
    pool = dict(input="x", kernel_shape=[3, 3], pads=[1] * 4, strides=[2, 2], output="y")
    g["ref_maxpool_3_p1_s2"] = ref._single_layer("MaxPool", xf, pool)["y"]
    g["ref_avepool_3_p1_s2"] = ref._single_layer("AvePool", xf, pool)["y"]
    g["ref_avepool_2_p0_s2"] = ref._single_layer("AvePool", xf, dict(pool, kernel_shape=[2, 2], pads=[0] * 4))["y"]
    g["ref_concat"] = ref._single_layer("Concat", xf, dict(inputs=["x", "o"], axis=3, output="y"),
                                        [TensorSpec("o", "f32", other.shape, other)])["y"]
    wf = rng.normal(0, 0.2, (5, 3, 3, 8)).astype(np.float32)
    bias = rng.normal(0, 1, 5).astype(np.float32)
    g["fconv_w"], g["fconv_bias"] = wf, bias
    g["ref_fconv_p1_s2_bias"] = ref.fconv(xf, wf, bias, 1, 1, 2, 2)
    g["ref_fconv_p0_s1"] = ref.fconv(xf, wf, None, 0, 0, 1, 1)
    np.savez_compressed(OUT / "kernels.npz", **g)
    # --- a whole (small) Bi-Real-18-shaped network ---------------------------------------------------
    spec = build_bireal18(image_hw=64, num_classes=100)
    img = np.random.default_rng(11).normal(0, 1, (64, 64, 3)).astype(np.float32)
    blobs = ref.run_model(spec, img)
    keep = ["stem_pool_out", "s1b1_bconv_out", "s1b1_add_out", "s2b1_add_out", "s3b1_add_out", "s4b4_add_out",
            "head_pool_out", "fc_out"]
    # s1b1_bconv_out is aliased by the in-place Affine/Add that follow it: it holds the block output
    np.savez_compressed(OUT / "bireal64.npz", image=img, **{f"ref_{k}": blobs[k] for k in keep})
    print("wrote", [p.name for p in OUT.glob("*.npz")])


if __name__ == "__main__":
    main()
