"""GPU parity tests, kernel level: every CUDA entry point (called through the C ABI) against the
CPU oracle on the same seeded inputs, and against the fixtures generated from the reference's own
compiled code.  Integer / bit results and the elementwise float layers must be bit-identical; the
float convolution is compared at 1e-4 relative (its summation order differs from Eigen's)."""
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from gpu_util import dev_bits, dev_f32, host, host_bits, rand_bits, same_bits  # noqa: E402

G = Path(__file__).resolve().parent / "golden"
ENGINES = ["popc", "b1", "imma", "tcgen05"]


@pytest.fixture(scope="module")
def ops():
    from dabnn_b200 import ops as o
    return o


@pytest.fixture(scope="module")
def k():
    return np.load(G / "kernels.npz")


# ------------------------------------------------------------------------------------ bit packing
def test_pack_golden_and_edges(ops, k):
    assert same_bits(host_bits(ops.pack_mat(dev_f32(k["pack_edge_in"]))), k["ref_pack_edge"])
    assert same_bits(host_bits(ops.pack_mat(dev_f32(k["pack_in"]))), k["ref_pack"])


@pytest.mark.parametrize("shape", [(1, 56, 56, 64), (3, 7, 8, 128), (2, 1, 1, 64), (1, 64, 64, 256), (5, 3, 2, 192)])
def test_pack_random(ops, port, shape):
    rng = np.random.default_rng(sum(shape))
    x = rng.uniform(-1, 1, shape).astype(np.float32)
    x[rng.random(shape) < 0.05] = 0.0
    assert same_bits(host_bits(ops.pack_mat(dev_f32(x))), port.pack_mat(x))


def test_pack_large_matches_torch_property(ops):
    """Full-size check at the batch-256 operand of the bgemm config: popcount of the packed words
    equals the number of positive inputs, and unpacking word 0 reproduces the signs."""
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.rand((802816, 576), device="cuda", generator=g) * 2 - 1
    bits = ops.pack_mat(x.view(1, 1, 802816, 576))
    b8 = bits.view(torch.uint8)
    lut = torch.tensor([bin(i).count("1") for i in range(256)], device="cuda", dtype=torch.int64)
    assert int(lut[b8.long()].sum()) == int((x > 0).sum())
    w0 = int(bits.view(-1)[0].item()) & (2**64 - 1)
    exp = sum(1 << i for i in range(64) if x[0, i] > 0)
    assert w0 == exp


# ------------------------------------------------------------------------------------ pad / im2col
def test_pad_im2col_golden(ops, k):
    assert same_bits(host_bits(ops.pad(dev_bits(k["pad_in"]), 1, 2)), k["ref_pad_1_2"])
    assert same_bits(host_bits(ops.im2col(dev_bits(k["pad_in"]), 3, 3, 1, 1, 2, 2)), k["ref_im2col_bits_3x3_p1_s2"])
    assert same_bits(host_bits(ops.fused_binarize_im2col(dev_f32(k["fbi_in64"]), 3, 3, 1, 1, 1, 1)), k["ref_fbi_64_3x3_p1_s1"])
    assert same_bits(host_bits(ops.fused_binarize_im2col(dev_f32(k["fbi_in128"]), 3, 3, 1, 1, 2, 2)), k["ref_fbi_128_3x3_p1_s2"])
    assert same_bits(host_bits(ops.fused_binarize_im2col(dev_f32(k["fbi_in32"]), 5, 5, 2, 2, 1, 1)), k["ref_fbi_32_5x5_p2_s1"])


def test_im2col_reference_ramp(ops):
    x = np.arange(32, dtype=np.float32).reshape(4, 4, 2)           # reference tests/im2col_test.cpp
    col = host(ops.im2col(dev_f32(x), 3, 3, 1, 1, 1, 1))
    assert col[0].tolist() == [0] * 8 + [0, 1, 2, 3, 0, 0, 8, 9, 10, 11]
    assert col[5].tolist() == [0, 1, 2, 3, 4, 5, 8, 9, 10, 11, 12, 13, 16, 17, 18, 19, 20, 21]


def test_pad_im2col_random_batched(ops, port):
    rng = np.random.default_rng(4)
    xb = rand_bits(rng, (3, 9, 7, 2))
    out = host_bits(ops.pad(dev_bits(xb), 2, 1))
    for i in range(3):
        assert same_bits(out[i], port.pad_bits(xb[i], 2, 1))
    xf = rng.normal(size=(2, 9, 7, 5)).astype(np.float32)
    out = host(ops.pad(dev_f32(xf), 1, 1, -3.5))
    for i in range(2):
        assert same_bits(out[i], port.pad_f32(xf[i], 1, 1, -3.5))
    col = host(ops.im2col(dev_f32(xf), 3, 2, 1, 0, 2, 1, 1, 2))
    for i in range(2):
        assert same_bits(col[i], port.im2col(xf[i], 3, 2, 1, 0, 2, 1, 1, 2))
    xf = rng.uniform(-1, 1, (2, 6, 5, 48)).astype(np.float32)
    col = host_bits(ops.fused_binarize_im2col(dev_f32(xf), 3, 3, 1, 1, 1, 2))
    for i in range(2):
        assert same_bits(col[i], port.fused_binarize_im2col(xf[i], 3, 3, 1, 1, 1, 2))


# ------------------------------------------------------------------------------------ bgemm
@pytest.mark.parametrize("engine", ENGINES)
def test_bgemm_golden(ops, k, engine):
    a, b, c0 = k["bgemm_a"], k["bgemm_b"], k["bgemm_c0"]
    kk, m = a.shape
    n = b.shape[0]
    c = dev_f32(c0)
    ops.bgemm(m, n, kk, dev_bits(a), m, dev_bits(b), kk, c, m, engine)
    assert same_bits(host(c), k["ref_bgemm"])


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("m,n,kk", [(159, 253, 68), (128, 784, 18), (256, 196, 36), (512, 49, 72),   # reference tests/bgemm_test.cpp
                                    (64, 3136, 9), (1, 1, 1), (65, 129, 17), (200, 300, 3)])
def test_bgemm_vs_oracle(ops, port, engine, m, n, kk):
    rng = np.random.default_rng(m * 7 + n)
    lda, ldb, ldc = m + 3, kk + 2, m + 5                         # padded leading dimensions
    a, b = rand_bits(rng, kk * lda), rand_bits(rng, n * ldb)
    c0 = rng.integers(0, 7, n * ldc).astype(np.float32)
    exp = port.bgemm(m, n, kk, a, lda, b, ldb, c0.copy(), ldc)
    c = dev_f32(c0)
    ops.bgemm(m, n, kk, dev_bits(a), lda, dev_bits(b), ldb, c, ldc, engine)
    assert same_bits(host(c), exp)


@pytest.mark.parametrize("M,N,K", [(3136, 64, 576), (784, 128, 1152), (196, 256, 2304), (49, 512, 4608)])
def test_bitpack_bgemm_config(ops, port, M, N, K):
    """Standalone bitpack + bgemm microbench shapes: fp32 operands sign-packed along K, then bgemm.
    Base size against the oracle, the x256 batch through engine agreement and the complement rule
    cnt(~x, w) = K - cnt(x, w)."""
    rng = np.random.default_rng(K)
    xf = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    wf = rng.uniform(-1, 1, (N, K)).astype(np.float32)
    xb = ops.pack_mat(dev_f32(xf).view(1, 1, M, K)).view(M, K // 64)
    wb = ops.pack_mat(dev_f32(wf).view(1, 1, N, K)).view(N, K // 64)
    assert same_bits(host_bits(xb), port.pack_64(xf).reshape(M, K // 64))
    kw = K // 64
    wt = wb.t().contiguous()                                     # reference layout of `a`: [k][m]
    exp = port.bgemm(N, M, kw, host_bits(wt), N, host_bits(xb), kw, np.zeros(M * N, np.float32), N)
    for eng in ENGINES:
        c = torch.zeros(M * N, device="cuda")
        ops.bgemm(N, M, kw, wt, N, xb, kw, c, N, eng)
        assert same_bits(host(c), exp), eng
    Mb = M * 256
    g = torch.Generator(device="cuda").manual_seed(K)
    xbig = torch.randint(-2**63, 2**63 - 1, (Mb, kw), device="cuda", dtype=torch.int64, generator=g)
    res = {}
    for eng in ("imma", "popc", "tcgen05", "auto"):   # the tensor-memory kernel with many pixel tiles per CTA
        c = torch.zeros(Mb * N, device="cuda")
        ops.bgemm(N, Mb, kw, wt, N, xbig, kw, c, N, eng)
        assert ops.last_engine() == ("tcgen05" if eng == "auto" else eng)
        res[eng] = c
    for eng in ("popc", "tcgen05", "auto"):
        assert torch.equal(res["imma"], res[eng]), eng
    assert ops.engine_status() == 0
    c = torch.zeros(Mb * N, device="cuda")
    ops.bgemm(N, Mb, kw, wt, N, ~xbig, kw, c, N, "tcgen05")
    assert torch.equal(c, K - res["tcgen05"])
    idx = [0, 127, 128, Mb // 2 + 1, min(148 * 128 * 4 + 5, Mb - 2), Mb - 129, Mb - 1]   # spot rows against the oracle, several per-CTA tile rounds apart
    sub = host_bits(xbig[idx].contiguous())
    exp = port.bgemm(N, len(idx), kw, host_bits(wt), N, sub, kw, np.zeros(len(idx) * N, np.float32), N)
    for eng in ("imma", "tcgen05"):
        assert same_bits(host(res[eng].view(Mb, N)[idx].contiguous()).ravel(), exp), eng


# ------------------------------------------------------------------------------------ bconv
CONV_SHAPES = [  # (H, Cin, Cout, k, stride, pad): the ResNet-18 stage shapes of the conv sweep
    (56, 64, 64, 3, 1, 1), (28, 128, 128, 3, 1, 1), (14, 256, 256, 3, 1, 1), (7, 512, 512, 3, 1, 1),
    (56, 64, 128, 3, 2, 1), (28, 128, 256, 3, 2, 1), (14, 256, 512, 3, 2, 1),
    (56, 64, 128, 1, 1, 0), (14, 256, 512, 1, 1, 0)]


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("H,cin,cout,ks,stride,pad", CONV_SHAPES)
def test_bconv_sweep_batch1(ops, port, engine, H, cin, cout, ks, stride, pad):
    rng = np.random.default_rng(H + cin + cout)
    x = rand_bits(rng, (H, H, cin // 64))
    w = rand_bits(rng, cout * ks * ks * cin // 64)
    exp = port.baseline_bconv(x, w, cout, ks, ks, pad, pad, stride, stride)
    out = ops.bconv(dev_bits(x), dev_bits(w), cout, ks, ks, pad, pad, stride, stride, engine)
    assert same_bits(host(out), exp)


@pytest.mark.parametrize("H,cin,cout,ks,stride,pad", CONV_SHAPES)
def test_bconv_sweep_batched(ops, port, H, cin, cout, ks, stride, pad):
    """Batch 16 against the oracle image by image; batch 256 by engine agreement + spot images."""
    rng = np.random.default_rng(H * 3 + cin)
    w = rand_bits(rng, cout * ks * ks * cin // 64)
    x = rand_bits(rng, (16, H, H, cin // 64))
    out = host(ops.bconv(dev_bits(x), dev_bits(w), cout, ks, ks, pad, pad, stride, stride, "imma"))
    for i in (0, 7, 15):
        assert same_bits(out[i], port.baseline_bconv(x[i], w, cout, ks, ks, pad, pad, stride, stride))
    g = torch.Generator(device="cuda").manual_seed(H)
    xb = torch.randint(-2**63, 2**63 - 1, (256, H, H, cin // 64), device="cuda", dtype=torch.int64, generator=g)
    wd = dev_bits(w)
    o_imma = ops.bconv(xb, wd, cout, ks, ks, pad, pad, stride, stride, "imma")
    o_popc = ops.bconv(xb, wd, cout, ks, ks, pad, pad, stride, stride, "popc")
    assert torch.equal(o_imma, o_popc)
    for eng in ("tcgen05", "auto"):   # what dabnn_bconv runs by default: the tensor-memory kernel, several tiles per CTA
        o = ops.bconv(xb, wd, cout, ks, ks, pad, pad, stride, stride, eng)
        assert ops.last_engine() == "tcgen05"
        assert torch.equal(o, o_imma), eng
    o16 = host(ops.bconv(dev_bits(x), dev_bits(w), cout, ks, ks, pad, pad, stride, stride, "tcgen05"))
    assert same_bits(o16, out)
    assert ops.engine_status() == 0
    for i in (0, 255):
        assert same_bits(host(o_imma[i]), port.baseline_bconv(host_bits(xb[i]), w, cout, ks, ks, pad, pad, stride, stride))


@pytest.mark.parametrize("cin,cout,stride", [(64, 64, 1), (64, 64, 2), (128, 128, 1), (128, 256, 2), (256, 256, 1),
                                             (512, 256, 1), (512, 1024, 2)])
def test_bconv_reference_test_shapes(ops, port, cin, cout, stride):       # reference tests/bconv_test.cpp:164-431
    rng = np.random.default_rng(cin * 2 + cout)
    x = rand_bits(rng, (64, 64, cin // 64))
    w = rand_bits(rng, cout * 9 * cin // 64)
    exp = port.baseline_bconv(x, w, cout, 3, 3, 1, 1, stride, stride)
    # pad + bconv_3x3 on the padded input, as the reference test does, and the direct form
    padded = ops.pad(dev_bits(x), 1, 1)
    assert same_bits(host(ops.bconv(padded, dev_bits(w), cout, 3, 3, 0, 0, stride, stride)), exp)
    assert same_bits(host(ops.bconv(dev_bits(x), dev_bits(w), cout, 3, 3, 1, 1, stride, stride)), exp)


@pytest.mark.parametrize("engine", ENGINES)
def test_bconv_odd_shapes(ops, port, engine):
    rng = np.random.default_rng(9)
    for (h, w_, cw, cout, kh, kw, ph, pw, sh, sw) in [(5, 6, 1, 8, 3, 3, 1, 1, 1, 1), (9, 4, 3, 24, 5, 3, 2, 1, 2, 1),
                                                      (3, 3, 2, 128, 3, 3, 0, 0, 2, 2), (1, 1, 1, 3, 1, 1, 0, 0, 1, 1),
                                                      (64, 64, 2, 128, 5, 5, 2, 2, 2, 2),
                                                      # channel counts that end in a clipped 32-channel box
                                                      (10, 10, 1, 48, 3, 3, 1, 1, 1, 1), (6, 6, 2, 80, 3, 3, 1, 1, 1, 1),
                                                      (12, 12, 1, 144, 3, 3, 1, 1, 1, 1)]:
        x = rand_bits(rng, (2, h, w_, cw))
        wt = rand_bits(rng, cout * kh * kw * cw)
        out = host(ops.bconv(dev_bits(x), dev_bits(wt), cout, kh, kw, ph, pw, sh, sw, engine))
        for i in range(2):
            assert same_bits(out[i], port.baseline_bconv(x[i], wt, cout, kh, kw, ph, pw, sh, sw))


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("cin,cout,stride", [(64, 64, 1), (128, 64, 2), (192, 16, 1)])
def test_binconv_operator_golden(ops, k, engine, cin, cout, stride):
    out = ops.binconv_forward(dev_f32(k[f"binconv_in_{cin}"]), dev_bits(k[f"binconv_w_{cin}"]), cout, 3, 3, 1, 1,
                              stride, stride, engine)
    assert same_bits(host(out), k[f"ref_binconv_{cin}_{cout}_s{stride}"])


def test_binconv_operator_non_multiple_of_64(ops, port):
    rng = np.random.default_rng(12)
    x = rng.uniform(-1, 1, (2, 6, 6, 32)).astype(np.float32)          # the im2col + packed-GEMM route
    wf = np.where(rng.random((16, 3, 3, 32)) < 0.5, -1.0, 1.0).astype(np.float32)
    w = port.pack_weight(wf)
    out = host(ops.binconv_forward(dev_f32(x), dev_bits(w), 16, 3, 3, 1, 1, 1, 1))
    for i in range(2):
        assert same_bits(out[i], port.binconv_forward(x[i], w, 16, 3, 3, 1, 1, 1, 1))


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("H,cin,cout,stride", [(14, 64, 64, 1), (8, 128, 128, 1), (8, 128, 256, 2), (7, 512, 512, 1)])
def test_bconv_block_fused_equals_layer_sequence(ops, port, engine, H, cin, cout, stride):
    rng = np.random.default_rng(H + cout)
    n = 3
    xf = rng.normal(0, 1, (n, H, H, cin)).astype(np.float32)
    wf = np.where(rng.random((cout, 3, 3, cin)) < 0.5, -1.0, 1.0).astype(np.float32)
    w = port.pack_weight(wf)
    a = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    b = rng.normal(0, 1, cout).astype(np.float32)
    oh = (H + 2 - 3) // stride + 1
    sc = rng.normal(0, 1, (n, oh, oh, cout)).astype(np.float32)
    xb = ops.pack_mat(dev_f32(xf))
    f32, bits = ops.bconv_block(xb, dev_bits(w), cout, 3, 3, 1, 1, stride, stride, dev_f32(a), dev_f32(b), dev_f32(sc),
                                want_f32=True, want_bits=True, engine=engine)
    for i in range(n):
        cnt = port.binconv_forward(xf[i], w, cout, 3, 3, 1, 1, stride, stride)
        exp = port.add(port.affine(cnt, a, b), sc[i])
        assert same_bits(host(f32[i]), exp)
        assert same_bits(host_bits(bits[i]), port.pack_mat(exp))
    # bits only / no shortcut / no affine variants agree with the full form
    f2, b2 = ops.bconv_block(xb, dev_bits(w), cout, 3, 3, 1, 1, stride, stride, dev_f32(a), dev_f32(b), None,
                             want_f32=True, want_bits=True, engine=engine)
    cnt0 = port.binconv_forward(xf[0], w, cout, 3, 3, 1, 1, stride, stride)
    assert same_bits(host(f2[0]), port.affine(cnt0, a, b))
    _, b3 = ops.bconv_block(xb, dev_bits(w), cout, 3, 3, 1, 1, stride, stride, dev_f32(a), dev_f32(b), None,
                            want_f32=False, want_bits=True, engine=engine)
    assert torch.equal(b2, b3)


# ------------------------------------------------------------------------------------ byte-activation engine
U8_SHAPES = [  # n, H, W, cin, cout, k, pad, stride
    (3, 14, 14, 64, 64, 3, 1, 1),      # whole images per tile would not fit: two tiles of 7 rows
    (5, 7, 7, 128, 128, 3, 1, 1),      # two images per tile, odd batch: the last tile is half empty
    (2, 56, 56, 64, 64, 3, 1, 1),      # resident weights, 2 rows per tile
    (2, 28, 28, 128, 256, 3, 1, 2),    # stride 2 (parity view), two channel blocks
    (2, 15, 13, 64, 48, 3, 1, 1),      # ragged rows per tile, 48 channels (a 16-column tail)
    (2, 20, 20, 128, 80, 1, 0, 1),     # 1x1, two boxes
    (1, 9, 9, 64, 192, 5, 2, 1),       # 5x5, channel blocks of 128 + 64
    (2, 12, 12, 64, 64, 3, 0, 1),      # no padding
    (2, 16, 16, 64, 64, 2, 0, 2),      # 2x2 stride 2
    (3, 14, 14, 256, 256, 3, 1, 1),    # the deep layers' shapes: four and eight boxes per tap
    (5, 7, 7, 512, 80, 3, 1, 1),       # with a 16-channel tail block
    (3, 14, 14, 256, 512, 3, 1, 2),    # and stride 2
    (148, 14, 14, 128, 128, 3, 1, 1),  # 296 tiles on 148 SMs: tiles handed out in pairs that share the weight stages
    (589, 7, 7, 128, 128, 3, 1, 1),    # 295 tiles: the last pair has one tile
    # 3x3 stride 1 runs on the kernel that loads a tile's halo once: more of its tilings
    (2, 28, 28, 128, 128, 3, 1, 1),    # four output rows per tile, two channel groups, streamed weights
    (1, 9, 126, 64, 64, 3, 1, 1),      # a 128-pixel halo pitch: one output row per tile
    (3, 10, 20, 64, 32, 3, 1, 1),      # not square, rows per tile do not divide the height
    (2, 56, 56, 64, 128, 3, 1, 1),     # 128 output channels on 64 inputs: weights too large to stay resident, one group
    (301, 14, 14, 256, 256, 3, 1, 1),  # 602 tiles in pairs over 74 CTAs per channel block: every ring wraps many times
    (1200, 7, 7, 512, 512, 3, 1, 1),   # four channel blocks, eight channel groups; two whole images per halo tile (pitch OW + 1)
    (7, 3, 3, 64, 64, 3, 1, 1),        # 3x3 images, two per tile, odd batch
    (1, 7, 7, 128, 128, 3, 1, 1),      # a single small image: the per-tap kernel
    (6, 7, 7, 64, 64, 3, 1, 1),        # two images per tile with resident weights
]


@pytest.mark.parametrize("n,H,W,cin,cout,k,pad,stride", U8_SHAPES)
def test_bconv_u8_block_equals_layer_sequence(ops, port, n, H, W, cin, cout, k, pad, stride):
    rng = np.random.default_rng(H * 131 + cout)
    xf = rng.normal(0, 1, (n, H, W, cin)).astype(np.float32)
    wf = np.where(rng.random((cout, k, k, cin)) < 0.5, -1.0, 1.0).astype(np.float32)
    w = port.pack_weight(wf)
    a = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    b = rng.normal(0, 1, cout).astype(np.float32)
    oh, ow = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    sc = rng.normal(0, 1, (n, oh, ow, cout)).astype(np.float32)
    assert ops.bconv_u8_supported(n, H, W, cin, cout, k, k, pad, pad, stride, stride)
    x8 = ops.binarize_u8(dev_f32(xf))
    assert np.array_equal(x8.cpu().numpy(), (xf > 0).astype(np.uint8))
    kwords = k * k * cin // 64
    we = ops.bconv_u8_expand_weights(dev_bits(w), cout, kwords)
    want_bits = cout % 64 == 0
    f32, o8, bits = ops.bconv_u8_block(x8, we, cout, k, k, pad, pad, stride, stride, dev_f32(a), dev_f32(b), dev_f32(sc),
                                       want_f32=True, want_u8=True, want_bits=want_bits)
    raw, _, _ = ops.bconv_u8_block(x8, we, cout, k, k, pad, pad, stride, stride)
    assert ops.engine_status() == 0
    for i in (range(n) if n <= 16 else sorted({0, 1, n // 3, n // 2, n - 2, n - 1})):
        cnt = port.binconv_forward(xf[i], w, cout, k, k, pad, pad, stride, stride)
        exp = port.add(port.affine(cnt, a, b), sc[i])
        assert same_bits(host(raw[i]), cnt)                     # BinConv.cpp:144: mismatch counts as fp32
        assert same_bits(host(f32[i]), exp)
        assert np.array_equal(o8[i].cpu().numpy(), (exp > 0).astype(np.uint8))
        if want_bits:
            assert same_bits(host_bits(bits[i]), port.pack_mat(exp))
    # the byte output alone equals the byte output of the full form
    _, o8b, _ = ops.bconv_u8_block(x8, we, cout, k, k, pad, pad, stride, stride, dev_f32(a), dev_f32(b), dev_f32(sc),
                                   want_f32=False, want_u8=True)
    assert torch.equal(o8, o8b)


def test_binarize_u8_edge_values(ops):
    vals = np.array([0.0, -0.0, 1e-45, -1e-45, np.inf, -np.inf, np.nan, 1.0, -1.0, 3e-39, -3e-39], dtype=np.float32)
    x = np.resize(vals, 16 * 5 + 7).astype(np.float32)          # a vector body and a scalar tail
    got = ops.binarize_u8(dev_f32(x)).cpu().numpy()
    with np.errstate(invalid="ignore"):
        assert np.array_equal(got, (x > 0).astype(np.uint8))    # strict >, NaN -> 0 (bitpack.h:29-37)


def test_bconv_u8_refuses_other_shapes(ops):
    assert not ops.bconv_u8_supported(1, 14, 14, 32, 64, 3, 3, 1, 1, 1, 1)      # cin % 64
    assert not ops.bconv_u8_supported(1, 14, 14, 64, 40, 3, 3, 1, 1, 1, 1)      # cout % 16
    assert not ops.bconv_u8_supported(1, 15, 15, 64, 64, 3, 3, 1, 1, 2, 2)      # stride 2 needs even h, w
    assert not ops.bconv_u8_supported(1, 14, 300, 64, 64, 3, 3, 1, 1, 1, 1)     # rows of more than 128 pixels
    assert not ops.bconv_u8_supported(1, 14, 14, 64, 64, 3, 3, 1, 1, 3, 3)      # stride 3
    x8 = torch.zeros((1, 14, 14, 32), dtype=torch.uint8, device="cuda")
    we = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    with pytest.raises(Exception):
        ops.bconv_u8_block(x8, we, 64, 3, 3, 1, 1, 1, 1)


# ------------------------------------------------------------------------------------ float layers
def test_float_layers_golden(ops, k):
    x, a, b, other = k["fl_in"], k["fl_a"], k["fl_b"], k["fl_other"][0]
    assert same_bits(host(ops.affine_(dev_f32(x), dev_f32(a), dev_f32(b))), k["ref_affine"])
    assert same_bits(host(ops.add_(dev_f32(x), dev_f32(other))), k["ref_add"])
    assert same_bits(host(ops.relu_(dev_f32(x))), k["ref_relu"])
    assert same_bits(host(ops.prelu_(dev_f32(x), dev_f32(a))), k["ref_prelu_c"])
    assert same_bits(host(ops.prelu_(dev_f32(x), dev_f32(a[:1]))), k["ref_prelu_1"])
    assert same_bits(host(ops.maxpool(dev_f32(x), 3, 3, 1, 1, 2, 2)), k["ref_maxpool_3_p1_s2"])
    assert same_bits(host(ops.avepool(dev_f32(x), 3, 3, 1, 1, 2, 2)), k["ref_avepool_3_p1_s2"])
    assert same_bits(host(ops.avepool(dev_f32(x), 2, 2, 0, 0, 2, 2)), k["ref_avepool_2_p0_s2"])
    assert same_bits(host(ops.concat(dev_f32(x), dev_f32(other))), k["ref_concat"])
    np.testing.assert_allclose(host(ops.fconv(dev_f32(x), dev_f32(k["fconv_w"]), dev_f32(k["fconv_bias"]), 1, 1, 2, 2)),
                               k["ref_fconv_p1_s2_bias"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(host(ops.fconv(dev_f32(x), dev_f32(k["fconv_w"]), None, 0, 0, 1, 1)),
                               k["ref_fconv_p0_s1"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("shape", [(2, 56, 56, 64), (3, 7, 7, 512), (2, 5, 3, 7), (1, 1, 1, 1000), (2, 9, 11, 64), (1, 18, 6, 128)])
def test_float_layers_random(ops, port, shape):
    rng = np.random.default_rng(sum(shape))
    x = rng.normal(0, 1, shape).astype(np.float32)
    x[rng.random(shape) < 0.05] = 0.0
    y = rng.normal(0, 1, shape).astype(np.float32)
    c = shape[-1]
    a, b = rng.normal(0, 1, c).astype(np.float32), rng.normal(0, 1, c).astype(np.float32)
    assert same_bits(host(ops.affine_(dev_f32(x), dev_f32(a), dev_f32(b))), port.affine(x, a, b))
    assert same_bits(host(ops.add_(dev_f32(x), dev_f32(y))), port.add(x, y))
    assert same_bits(host(ops.relu_(dev_f32(x))), port.relu(x))
    assert same_bits(host(ops.prelu_(dev_f32(x), dev_f32(a))), port.prelu(x, a))
    assert same_bits(host(ops.concat(dev_f32(x), dev_f32(y))), port.concat(x, y))
    if shape[1] >= 3:
        for (kk, p, s) in [(3, 1, 2), (2, 0, 2), (3, 1, 1)]:
            mp, ap = host(ops.maxpool(dev_f32(x), kk, kk, p, p, s, s)), host(ops.avepool(dev_f32(x), kk, kk, p, p, s, s))
            for i in range(shape[0]):
                assert same_bits(mp[i], port.maxpool(x[i], kk, kk, p, p, s, s))
                assert same_bits(ap[i], port.avepool(x[i], kk, kk, p, p, s, s))


@pytest.mark.parametrize("h,cin,cout,ks,stride,pad,bias", [(32, 3, 64, 7, 2, 3, False), (8, 64, 128, 1, 1, 0, False),
                                                           (1, 512, 1000, 1, 1, 0, True), (9, 5, 7, 3, 1, 1, True),
                                                           # tensor-memory path: more tiles than SMs, ragged channel blocks,
                                                           # padded K of 152 / 144 / 256, a partial last pixel tile
                                                           (224, 3, 64, 7, 2, 3, True), (14, 256, 48, 1, 1, 0, True),
                                                           (20, 16, 144, 3, 1, 1, False), (13, 28, 16, 3, 2, 1, True),
                                                           # staged rows: two segments per output row, with 16-byte copies at
                                                           # a non-zero alignment shift and with 4-byte copies
                                                           (136, 3, 16, 3, 1, 1, True), (150, 3, 16, 3, 1, 1, False),
                                                           (132, 4, 32, 5, 1, 2, True),
                                                           # K = 256: 32-channel weight blocks
                                                           (7, 256, 96, 1, 1, 0, True)])
def test_fconv_vs_oracle(ops, port, h, cin, cout, ks, stride, pad, bias):
    rng = np.random.default_rng(h + cin)
    x = rng.normal(0, 1, (2, h, h, cin)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (cin * ks * ks)), (cout, ks, ks, cin)).astype(np.float32)
    bv = rng.normal(0, 1, cout).astype(np.float32) if bias else None
    out = host(ops.fconv(dev_f32(x), dev_f32(w), dev_f32(bv) if bias else None, pad, pad, stride, stride))
    for i in range(2):
        exp = port.fconv(x[i], w, bv, pad, pad, stride, stride)
        np.testing.assert_allclose(out[i], exp, rtol=1e-4, atol=1e-4 * np.abs(exp).max())


def test_no_bounded_wait_gave_up(ops):
    assert ops.engine_status() == 0


def test_engine_peaks_are_measurable(ops):
    peaks = {e: ops.measure_engine_peak(e) for e in ["popc", "b1", "imma", "tcgen05"]}
    peaks["tf32"] = ops.measure_tf32_peak()
    assert all(v > 1e13 for v in peaks.values()), peaks


def test_last_engine_names_the_kernel_that_ran(ops, port):
    """A tcgen05 request is served by the mma.sync int8 kernel for channel counts and alignments the tensor-memory
    kernel does not take; dabnn_last_engine tells which one ran, so a test that names an engine cannot pass on another."""
    rng = np.random.default_rng(1)
    for (m, n, kk, pad_ld, expected) in [(128, 300, 9, 0, "tcgen05"), (64, 1000, 18, 4, "tcgen05"), (159, 253, 68, 0, "imma"),
                                         (128, 300, 9, 3, "imma"), (3, 50, 2, 0, "imma")]:
        lda, ldb, ldc = m + pad_ld, kk, m + pad_ld
        a, b = rand_bits(rng, kk * lda), rand_bits(rng, n * ldb)
        c0 = rng.integers(0, 5, n * ldc).astype(np.float32)
        exp = port.bgemm(m, n, kk, a, lda, b, ldb, c0.copy(), ldc)
        for req in ("tcgen05", "auto"):
            c = dev_f32(c0)
            ops.bgemm(m, n, kk, dev_bits(a), lda, dev_bits(b), ldb, c, ldc, req)
            assert ops.last_engine() == expected, (m, n, kk, pad_ld, req)
            assert same_bits(host(c), exp)
    for req in ("popc", "b1", "imma"):
        c = dev_f32(np.zeros(64 * 64, np.float32))
        ops.bgemm(64, 64, 1, dev_bits(rand_bits(rng, 64)), 64, dev_bits(rand_bits(rng, 64)), 1, c, 64, req)
        assert ops.last_engine() == req


@pytest.mark.parametrize("h,cin,cout,ks,stride,pad,dil", [(16, 5, 7, 3, 1, 2, 2), (20, 16, 32, 3, 1, 2, 2), (23, 3, 16, 3, 2, 2, 2),
                                                         (12, 64, 64, 1, 1, 0, 2)])
def test_fconv_dilation(ops, port, h, cin, cout, ks, stride, pad, dil):
    """Dilated windows (the reference's tests/fconv_test.cpp runs dilation 2) on every route: the mma.sync kernel
    (Cout % 16 != 0), staged rows, and a 1x1 kernel for which dilation must change nothing."""
    rng = np.random.default_rng(h * cin)
    x = rng.normal(0, 1, (2, h, h, cin)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (cin * ks * ks)), (cout, ks, ks, cin)).astype(np.float32)
    bv = rng.normal(0, 1, cout).astype(np.float32)
    out = host(ops.fconv(dev_f32(x), dev_f32(w), dev_f32(bv), pad, pad, stride, stride, dil, dil))
    for i in range(2):
        exp = port.fconv(x[i], w, bv, pad, pad, stride, stride, dil, dil)
        assert out[i].shape == exp.shape
        np.testing.assert_allclose(out[i], exp, rtol=1e-4, atol=1e-4 * np.abs(exp).max())
    assert ops.engine_status() == 0


@pytest.mark.parametrize("cin,cout,ks", [(64, 64, 3), (128, 32, 3), (64, 128, 1), (256, 64, 3)])
def test_batchnorm_fold_identity(ops, port, cin, cout, ks):
    """The converter's BatchNorm fold for a binary convolution (reference tools/onnx2bnn/OnnxConverter.cpp:583-639:
    b += K*a, then a *= -2) exists so that Affine(mismatch count) equals BatchNorm applied to the +-1 dot product
    (reference docs/onnx2bnn.md:9-13).  Checked against that product computed in float64, without padding (the
    reference pads with -1, a float convolution with 0).  Tolerance 1e-5 relative to the largest output."""
    from dabnn_b200.convert import batchnorm_to_affine, bitpack_weight
    rng = np.random.default_rng(cin + cout)
    x = rng.normal(0, 1, (2, 9, 9, cin)).astype(np.float32)
    wf = np.where(rng.random((cout, ks, ks, cin)) < 0.5, -1.0, 1.0).astype(np.float32)
    scale, beta = rng.uniform(0.5, 1.5, cout).astype(np.float32), rng.normal(0, 0.1, cout).astype(np.float32)
    mean, var = rng.normal(0, 3.0, cout).astype(np.float32), rng.uniform(0.5, 1.5, cout).astype(np.float32)
    K = ks * ks * cin
    a, b = batchnorm_to_affine(scale, beta, mean, var, 1e-5, binary_k=K)
    wb, _ = bitpack_weight(wf)
    cnt = ops.binconv_forward(dev_f32(x), dev_bits(wb), cout, ks, ks, 0, 0, 1, 1)
    got = host(ops.affine_(cnt.clone(), dev_f32(a), dev_f32(b)))       # Affine works in place
    xs = np.where(x > 0, 1.0, -1.0)
    oh = 9 - ks + 1
    dot = np.zeros((2, oh, oh, cout))
    for ky in range(ks):
        for kx in range(ks):
            dot += np.einsum("nhwc,oc->nhwo", xs[:, ky:ky + oh, kx:kx + oh, :], wf[:, ky, kx, :].astype(np.float64))
    bn = (dot - mean.astype(np.float64)) / np.sqrt(var.astype(np.float64) + 1e-5) * scale + beta
    np.testing.assert_allclose(got, bn, rtol=0, atol=1e-5 * np.abs(bn).max())
    assert same_bits(host(cnt)[0], ((K - dot[0]) / 2).astype(np.float32))   # count = (K - dot) / 2, exactly


@pytest.mark.parametrize("n,h,cin,cout,ks,pad,bias,spots", [
    (2, 224, 3, 64, 7, 3, True, None),        # the stem itself
    (37, 224, 3, 64, 7, 3, False, None),      # 4144 output rows on 148 CTAs: 28 per CTA, windows rolling through the slot ring, image changes inside a CTA
    (300, 130, 3, 32, 5, 2, True, (0, 1, 149, 298, 299)),   # 65-pixel output rows, one 32-channel box
    (3, 256, 3, 64, 3, 1, True, None),        # 128-pixel output rows, 256 converter threads busy, a one-instruction remainder contraction per window row
    (3, 256, 4, 64, 3, 1, True, None),        # four channels: not this kernel's (no spare entry per pixel), the staged-rows kernel takes it
    (2, 200, 1, 16, 7, 3, False, None),       # one channel, one 16-channel box (the three-instruction form)
    (2, 224, 3, 128, 7, 3, True, None),       # two channel blocks
    (5, 160, 2, 48, 4, 1, True, None),        # even kernel width (no dummy tap), 48 channels
])
def test_fconv_window_reading_kernel(ops, port, n, h, cin, cout, ks, pad, bias, spots):
    """Thin inputs with stride 2 (dabnn/fconv.h:14-76 on the shapes of a ResNet stem) run on the kernel whose tensor
    core reads the convolution windows straight out of the staged input rows; against the oracle at 1e-4."""
    rng = np.random.default_rng(n * h + cout)
    x = rng.normal(0, 1, (n, h, h, cin)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (cin * ks * ks)), (cout, ks, ks, cin)).astype(np.float32)
    bv = rng.normal(0, 1, cout).astype(np.float32) if bias else None
    out = host(ops.fconv(dev_f32(x), dev_f32(w), dev_f32(bv) if bias else None, pad, pad, 2, 2))
    assert ops.engine_status() == 0
    for i in (spots or range(n)):
        exp = port.fconv(x[i], w, bv, pad, pad, 2, 2)
        np.testing.assert_allclose(out[i], exp, rtol=1e-4, atol=1e-4 * np.abs(exp).max(), err_msg=f"image {i}")


@pytest.mark.parametrize("n,h,cin,cout,bias", [
    (2, 28, 64, 128, True),       # one channel block, two K chunks
    (70, 28, 64, 128, False),     # 429 pixel tiles on 148 CTAs: every ring wraps, a partial last tile
    (33, 14, 128, 256, True),     # two channel blocks per pixel tile
    (150, 7, 256, 512, True),     # four channel blocks, eight K chunks
    (3, 9, 32, 48, True),         # one K chunk, a 48-channel block (a 16-channel tail box)
    (2, 11, 96, 208, False),      # 208 = 128 + 80 channels
    (128, 1, 512, 1000, True),    # the classifier: one pixel tile, 32-channel work items, a last block of 8 channels
    (5, 3, 64, 20, True),         # a channel count that is no multiple of 16
    (1024, 1, 512, 1000, False),
])
def test_fconv_1x1_gemm_kernel(ops, port, n, h, cin, cout, bias):
    """1x1 float convolutions (the downsample branches: dabnn/fconv.h:14-76 with a 1x1 kernel) run on the TMA-fed GEMM
    kernel; against the oracle at 1e-4 on spot images."""
    rng = np.random.default_rng(n + cin + cout)
    x = rng.normal(0, 1, (n, h, h, cin)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / cin), (cout, 1, 1, cin)).astype(np.float32)
    bv = rng.normal(0, 1, cout).astype(np.float32) if bias else None
    out = host(ops.fconv(dev_f32(x), dev_f32(w), dev_f32(bv) if bias else None, 0, 0, 1, 1))
    assert ops.engine_status() == 0
    for i in sorted({0, 1, n // 2, n - 1}):
        exp = port.fconv(x[i], w, bv, 0, 0, 1, 1)
        np.testing.assert_allclose(out[i], exp, rtol=1e-4, atol=1e-4 * np.abs(exp).max(), err_msg=f"image {i}")


@pytest.mark.parametrize("n,h,cin,cout,ks,pad,relu", [
    (2, 224, 3, 64, 7, 3, True),        # the stem and its pool
    (37, 224, 3, 64, 7, 3, True),       # 2072 pooled rows on 148 CTAs: shares that start and end inside images
    (149, 130, 3, 32, 5, 2, False),     # 65-pixel rows (odd: the last column has a two-tap window), 33 pooled rows, no relu (negative maxima)
    (3, 255, 3, 64, 3, 1, True),        # 128 x 128 outputs from an odd-sized image
    (4, 180, 2, 32, 6, 2, True),        # two channels, six taps per window row (the remainder contraction pads them to eight)
    (5, 226, 1, 16, 7, 3, True),        # 113 output rows: an image's last pooled row ends on an even row
    (2, 224, 3, 128, 7, 3, True),       # two channel blocks
])
def test_fconv_maxpool_fused_is_bit_identical(ops, port, n, h, cin, cout, ks, pad, relu):
    """The fused stem kernel (convolution + bias + affine + relu + 3x3 / 2 max pooling, the convolution's output never
    written) against the same four steps run one after the other on the same kernels: bit for bit, sign bytes included;
    and against the oracle's FloatConv -> Affine -> Relu -> MaxPool at 1e-4 on spot images."""
    rng = np.random.default_rng(n * h + cout)
    x = rng.normal(0, 1, (n, h, h, cin)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (cin * ks * ks)), (cout, ks, ks, cin)).astype(np.float32)
    bv = rng.normal(0, 1, cout).astype(np.float32)
    a, b = rng.uniform(0.5, 1.5, cout).astype(np.float32), rng.normal(0, 0.5, cout).astype(np.float32)
    assert ops.fconv_maxpool_supported(n, h, h, cin, cout, ks, ks, pad, pad, 2, 2)
    xd, wd = dev_f32(x), dev_f32(w)
    fused, f8 = ops.fconv_maxpool(xd, wd, dev_f32(bv), pad, pad, 2, 2, dev_f32(a), dev_f32(b), relu, want_u8=True)
    y = ops.affine_(ops.fconv(xd, wd, dev_f32(bv), pad, pad, 2, 2), dev_f32(a), dev_f32(b))
    if relu:
        y = ops.relu_(y)
    steps = ops.maxpool(y, 3, 3, 1, 1, 2, 2)
    assert ops.engine_status() == 0
    assert torch.equal(fused, steps)
    assert torch.equal(f8, (steps > 0).to(torch.uint8))
    for i in sorted({0, n // 2, n - 1}):
        e = port.affine(port.fconv(x[i], w, bv, pad, pad, 2, 2), a, b)
        if relu:
            e = port.relu(e)
        e = port.maxpool(e, 3, 3, 1, 1, 2, 2)
        np.testing.assert_allclose(host(fused[i]), e, rtol=1e-4, atol=1e-4 * np.abs(e).max(), err_msg=f"image {i}")


def test_fconv_maxpool_refuses_other_shapes(ops):
    assert not ops.fconv_maxpool_supported(1, 64, 64, 3, 64, 7, 7, 3, 3, 2, 2)      # 32-pixel output rows: too short for the kernel
    assert not ops.fconv_maxpool_supported(1, 224, 224, 4, 64, 7, 7, 3, 3, 2, 2)    # more than three channels
    assert not ops.fconv_maxpool_supported(1, 224, 224, 3, 64, 7, 7, 3, 3, 1, 1)    # stride 1
    x, w = torch.zeros((1, 64, 64, 3), device="cuda"), torch.zeros((64, 7, 7, 3), device="cuda")
    with pytest.raises(Exception):
        ops.fconv_maxpool(x, w, None, 3, 3, 2, 2)


@pytest.mark.parametrize("n,H,cin,cout", [(3, 56, 64, 64), (5, 28, 128, 128), (4, 14, 256, 256), (2, 14, 256, 48), (150, 28, 128, 128)])
def test_bconv_u8_block_with_average_pooled_output(ops, port, n, H, cin, cout):
    """The fused block that also writes the 2x2 / 2 average pooling of its result (the next stage's downsample
    shortcut, reference layers/AvePool.cpp:84): the block's own outputs are unchanged and the pooled tensor is what
    dabnn_avepool gives on them, bit for bit; one image against the oracle's AvePool."""
    rng = np.random.default_rng(H + cout + n)
    xf = rng.normal(0, 1, (n, H, H, cin)).astype(np.float32)
    wf = np.where(rng.random((cout, 3, 3, cin)) < 0.5, -1.0, 1.0).astype(np.float32)
    w = port.pack_weight(wf)
    a = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    b = rng.normal(0, 1, cout).astype(np.float32)
    sc = rng.normal(0, 1, (n, H, H, cout)).astype(np.float32)
    assert ops.bconv_u8_block_pooled_supported(n, H, H, cin, cout, 3, 3, 1, 1, 1, 1)
    x8 = ops.binarize_u8(dev_f32(xf))
    we = ops.bconv_u8_expand_weights(dev_bits(w), cout, 9 * cin // 64)
    f32, o8, _ = ops.bconv_u8_block(x8, we, cout, 3, 3, 1, 1, 1, 1, dev_f32(a), dev_f32(b), dev_f32(sc), want_f32=True, want_u8=True)
    g32, g8, pooled = ops.bconv_u8_block_pooled(x8, we, cout, 3, 3, 1, 1, 1, 1, dev_f32(a), dev_f32(b), dev_f32(sc), want_u8=True)
    assert ops.engine_status() == 0
    assert torch.equal(f32, g32) and torch.equal(o8, g8)
    assert torch.equal(pooled, ops.avepool(f32, 2, 2, 0, 0, 2, 2))
    assert same_bits(host(pooled[n - 1]), port.avepool(host(f32[n - 1]), 2, 2, 0, 0, 2, 2))
    assert not ops.bconv_u8_block_pooled_supported(n, 15, 15, cin, cout, 3, 3, 1, 1, 1, 1)     # odd size
    assert not ops.bconv_u8_block_pooled_supported(n, H, H, cin, cout, 3, 3, 1, 1, 2, 2)       # stride 2


@pytest.mark.parametrize("n,H,cin,cout", [(9, 56, 64, 64), (33, 14, 256, 256), (150, 7, 512, 512)])
def test_block_kernels_and_their_tunings_agree(ops, n, H, cin, cout):
    """The two kernels a 3x3 stride-1 block can run on (one TMA box per tap / the tile's halo loaded once), every
    staging-tile setting of the halo kernel, and launches with and without programmatic overlap give the same bits
    (the reference has one result per layer: dabnn/layers/BinConv.cpp:144 + Affine.cpp:10 + Add.cpp:7)."""
    from dabnn_b200 import capi
    lib = capi.load()
    rng = np.random.default_rng(n + H)
    x8 = torch.from_numpy((rng.random((n, H, H, cin)) < 0.5).astype(np.uint8)).cuda()
    wbits = torch.from_numpy(rng.integers(-2**62, 2**62, cout * 9 * cin // 64, dtype=np.int64)).cuda()
    we = ops.bconv_u8_expand_weights(wbits, cout, 9 * cin // 64)
    a, b = dev_f32(rng.uniform(-0.1, 0.1, cout).astype(np.float32)), dev_f32(rng.normal(0, 1, cout).astype(np.float32))
    sc = dev_f32(rng.normal(0, 1, (n, H, H, cout)).astype(np.float32))
    run = lambda: ops.bconv_u8_block(x8, we, cout, 3, 3, 1, 1, 1, 1, a, b, sc, want_f32=True, want_u8=True, want_bits=True)
    try:
        lib.dabnn_debug_set_halo(0)
        base = run()
        for mode in (1, 1 | (2 << 4), 1 | (3 << 4), 1 | ((8 | 3) << 4), 1 | ((8 | 5) << 4)):
            lib.dabnn_debug_set_halo(mode)
            got = run()
            assert ops.engine_status() == 0
            assert all(torch.equal(g, e) for g, e in zip(got, base)), hex(mode)
        lib.dabnn_debug_set_halo(1)
        lib.dabnn_debug_set_launch_overlap(0)
        got = run()
        assert all(torch.equal(g, e) for g, e in zip(got, base))
    finally:
        lib.dabnn_debug_set_halo(1)
        lib.dabnn_debug_set_launch_overlap(1)
