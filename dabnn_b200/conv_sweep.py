"""Kernel-level timing of the binary convolution shapes of a Bi-Real-Net-18 (the reference's
benchmark/benchmark.cpp shapes: 3x3 stride 1 and 2 at 56/28/14/7 pixels, two 1x1 cases), at a chosen
batch, for one or more contraction engines.  Prints one JSON line per shape:

    python -m dabnn_b200.conv_sweep --batch 256 --engines tcgen05,imma

raw   = dabnn_bconv on packed bits (fp32 mismatch counts out),
block = dabnn_bconv_block (counts -> affine -> + shortcut -> fp32 and sign bits out).
Engine "u8" is the byte-activation engine (dabnn_bconv_u8_block: {0,1}-byte activations in and out,
weights expanded beforehand); shapes it does not take are reported as null.
Tbit-op/s counts 2*M*N*K with K the true bits; GB/s counts the block's algorithmic bytes
(bits in, shortcut in, fp32 + bits out).  Inputs are seeded random words; CUDA-event timing after
three warm-up calls.
"""
import argparse
import json

import torch

from . import ops

SHAPES = [(56, 64, 64, 3, 1, 1), (28, 128, 128, 3, 1, 1), (14, 256, 256, 3, 1, 1), (7, 512, 512, 3, 1, 1),
          (56, 64, 128, 3, 2, 1), (28, 128, 256, 3, 2, 1), (14, 256, 512, 3, 2, 1),
          (56, 64, 128, 1, 1, 0), (14, 256, 512, 1, 1, 0)]


def timeit(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--engines", default="tcgen05", help="comma list of popc, b1, imma, tcgen05, u8")
    ap.add_argument("--shapes", default="", help="comma list of shape indices (default: all)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--movers", action="store_true", help="also time bit-packing, im2col, elementwise and pooling kernels")
    args = ap.parse_args()
    B = args.batch
    g = torch.Generator(device="cuda").manual_seed(0)
    shapes = [SHAPES[int(i)] for i in args.shapes.split(",")] if args.shapes else SHAPES
    for (H, cin, cout, ks, s, p) in shapes:
        x = torch.randint(-2**63, 2**63 - 1, (B, H, H, cin // 64), device="cuda", dtype=torch.int64, generator=g)
        w = torch.randint(-2**63, 2**63 - 1, (cout * ks * ks * cin // 64,), device="cuda", dtype=torch.int64, generator=g)
        oh = (H + 2 * p - ks) // s + 1
        a, b = torch.rand(cout, device="cuda", generator=g), torch.rand(cout, device="cuda", generator=g)
        sc = torch.rand((B, oh, oh, cout), device="cuda", generator=g)
        bitops = 2.0 * B * oh * oh * cout * ks * ks * cin
        row = {"shape": f"{H}x{H}x{cin}->{cout} k{ks} s{s}", "batch": B}
        for e in args.engines.split(","):
            if e == "u8":
                if not ops.bconv_u8_supported(B, H, H, cin, cout, ks, ks, p, p, s, s):
                    row[e] = None
                    continue
                x8 = torch.randint(0, 2, (B, H, H, cin), device="cuda", dtype=torch.uint8, generator=g)
                we = ops.bconv_u8_expand_weights(w, cout, ks * ks * cin // 64)
                t_raw = timeit(lambda: ops.bconv_u8_block(x8, we, cout, ks, ks, p, p, s, s), args.iters)
                t_blk = timeit(lambda: ops.bconv_u8_block(x8, we, cout, ks, ks, p, p, s, s, a, b, sc, True, True, False), args.iters)
                row[e] = {"raw_ms": round(t_raw, 4), "raw_Tbitop_s": round(bitops / t_raw / 1e9, 1),
                          "block_ms": round(t_blk, 4), "block_Tbitop_s": round(bitops / t_blk / 1e9, 1),
                          "block_GB_s": round(B * (H * H * cin / 8 + oh * oh * cout * 8.125) / t_blk / 1e6, 1),
                          "block_moved_GB_s": round(B * (H * H * cin + oh * oh * cout * 9) / t_blk / 1e6, 1)}
                continue
            t_raw = timeit(lambda: ops.bconv(x, w, cout, ks, ks, p, p, s, s, e), args.iters)
            t_blk = timeit(lambda: ops.bconv_block(x, w, cout, ks, ks, p, p, s, s, a, b, sc, True, True, e), args.iters)
            row[e] = {"raw_ms": round(t_raw, 4), "raw_Tbitop_s": round(bitops / t_raw / 1e9, 1),
                      "block_ms": round(t_blk, 4), "block_Tbitop_s": round(bitops / t_blk / 1e9, 1),
                      "block_GB_s": round(B * (H * H * cin / 8 + oh * oh * cout * 8.125) / t_blk / 1e6, 1)}
        print(json.dumps(row), flush=True)
    if args.movers:
        movers(B, args.iters)


def movers(B, iters):
    """The data-movement functions of the path, in GB/s of algorithmic bytes (each tensor once)."""
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((B, 56, 56, 64), device="cuda", generator=g)
    y = torch.randn((B, 56, 56, 64), device="cuda", generator=g)
    a, b = torch.rand(64, device="cuda", generator=g), torch.rand(64, device="cuda", generator=g)
    x128 = torch.randn((B, 28, 28, 128), device="cuda", generator=g)
    stem = torch.randn((B, 112, 112, 64), device="cuda", generator=g)
    n = x.numel()
    cases = [
        ("pack_mat 56x56x64", lambda: ops.pack_mat(x), n * 4 + n / 8),
        ("fused_binarize_im2col 28x28x128 k3 p1", lambda: ops.fused_binarize_im2col(x128, 3, 3, 1, 1, 1, 1),
         x128.numel() * 4 + B * 28 * 28 * 18 * 8),
        ("affine 56x56x64 (in place)", lambda: ops.affine_(x, a, b), n * 8),
        ("add 56x56x64 (in place)", lambda: ops.add_(x, y), n * 12),
        ("maxpool 3x3 s2 p1 112x112x64", lambda: ops.maxpool(stem, 3, 3, 1, 1, 2, 2), stem.numel() * 4 * 1.25),
        ("avepool 2x2 s2 56x56x64", lambda: ops.avepool(x, 2, 2, 0, 0, 2, 2), n * 4 * 1.25),
    ]
    for name, fn, nbytes in cases:
        t = timeit(fn, iters)
        print(json.dumps({"kernel": name, "batch": B, "ms": round(t, 4), "GB_s": round(nbytes / t / 1e6, 1)}), flush=True)


if __name__ == "__main__":
    main()
