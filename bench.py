#!/usr/bin/env python
"""Throughput benchmark: Bi-Real-Net-18-shaped inference (images/s), the 1024-image batch sharded over N GPUs.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
           --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the reference's own CPU code on the host cores

One step = one pass of the network over the 1024-image batch of seeded synthetic images (fp32 N(0,1),
224x224x3, random-init weights).  With N GPUs rank r runs images shard_range(1024, r, N) on its own replica:
total work is fixed, so scaling is strong; no collective sits on the data path.  Rank 0 prints ONE JSON line.

  value     images/s with the inputs already resident in HBM, timed with CUDA events on the stream the
            kernels run on, barrier + synchronize on both sides, max over ranks.  The K timed steps are
            repeated until at least a second has been measured; the median repetition is reported.
  e2e       the same through the public Net API from pinned HOST memory: host->device copy of the
            batch and device->host read of the logits inside the timed region, every step.
  weak      the same two numbers with 1024 images on EVERY GPU (per-GPU work fixed).
  roofline  for the class of launches that takes most of the step (per-op CUDA events).
  cpu_baseline  the reference's CPU implementation timed on this box's host cores (N=1 only).
  conv_sweep / bgemm_micro / binconv_1x56x56x64 / small_batch (N=1 only): the per-shape kernel numbers of the
            other benchmark configurations, L2 flushed between timed calls.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

IMAGE_HW, CLASSES, GLOBAL_BATCH = 224, 1000, 1024
METRIC = "Bi-Real-18-shape images/s"
DTYPE = "b1 x b1 -> s32 (tcgen05 kind::i8 on bits held as {0,1} bytes) + fp32 (3xTF32)"


def measured_traffic():
    """DRAM bytes per image of each layer class from the committed ncu captures (profiles/traffic.json), or {}."""
    p = ROOT / "profiles" / "traffic.json"
    return json.loads(p.read_text()) if p.exists() else {}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock, max SM clock and throttle reasons of one GPU through NVML while running."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device_index):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(device_index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            pass

    def run(self):
        while self.ok and not self._halt.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.05)

    def stop(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def algorithmic_bytes(spec, batch):
    """Per layer class: bytes one step of the fused plan must move (each tensor read or written once), from the model
    description.  fp32 activations 4 B/element, packed bits 1/8 B/element, weights once.  A 3x3 / 2 max pooling
    behind a float convolution and a 2x2 / 2 average pooling behind a binary block happen in the producer's epilogue:
    the pooled tensor is written, the convolution's own output (max pooling) is not, and nothing is re-read."""
    shapes = {spec.input_name: spec.input_shape[1:]}
    made_by = {}   # blob name -> class of the convolution whose kernel writes it
    t = {x.name: x for x in spec.tensors}
    out = {}
    flops = {}   # multiply-adds * 2 per class (binary: per bit pair)

    def add(cls, n):
        out[cls] = out.get(cls, 0) + n

    for l in spec.layers:
        f = l.fields
        if l.type in ("FpConv2D", "BinConv2D"):
            h, w, c = shapes[f["input"]]
            o, kh, kw, _ = t[f["weight"]].shape
            oh = (h + 2 * f["pads"][0] - kh) // f["strides"][0] + 1
            ow = (w + 2 * f["pads"][1] - kw) // f["strides"][1] + 1
            shapes[f["output"]] = (oh, ow, o)
            cls = "Float Conv" if l.type == "FpConv2D" else "Bin Conv block"
            made_by[f["output"]] = cls
            flops[cls] = flops.get(cls, 0) + 2.0 * batch * oh * ow * o * kh * kw * c
            if l.type == "FpConv2D":
                add("Float Conv", batch * (h * w * c + oh * ow * o) * 4 + t[f["weight"]].data.size * 4)
            else:   # fused block: packed input, fp32 shortcut in, fp32 + packed out
                add("Bin Conv block", batch * (h * w * c / 8 + oh * ow * o * (4 + 4 + 1 / 8)) + t[f["weight"]].data.size * 8)
        elif l.type in ("MaxPool", "AvePool"):
            h, w, c = shapes[f["input"]]
            oh = (h + 2 * f["pads"][0] - f["kernel_shape"][0]) // f["strides"][0] + 1
            ow = (w + 2 * f["pads"][1] - f["kernel_shape"][1]) // f["strides"][1] + 1
            shapes[f["output"]] = (oh, ow, c)
            k, st, src = f["kernel_shape"][0], f["strides"][0], made_by.get(f["input"])
            if l.type == "MaxPool" and src == "Float Conv" and (k, st) == (3, 2):
                add(src, batch * (oh * ow * c - h * w * c) * 4)
            elif l.type == "AvePool" and src == "Bin Conv block" and (k, st) == (2, 2):
                add(src, batch * oh * ow * c * 4)
            else:
                add(l.type, batch * (h * w * c + oh * ow * c) * 4)
        elif l.type == "Add":
            shapes[f["output"]] = shapes[f["input1"]]
            made_by[f["output"]] = made_by.get(f["input1"])
        else:
            shapes[f["output"]] = shapes[f["input"]]
            made_by[f["output"]] = made_by.get(f["input"])
    return out, flops


# ---------------------------------------------------------------------------------------------------------
# Per-shape kernel numbers (the other benchmark configurations).  Every timed call starts with a cold L2: a
# 256 MB buffer is overwritten between calls, and the median of the per-call CUDA-event times is reported.
# ---------------------------------------------------------------------------------------------------------
CONV_SHAPES = [(56, 64, 64, 3, 1, 1), (28, 128, 128, 3, 1, 1), (14, 256, 256, 3, 1, 1), (7, 512, 512, 3, 1, 1),
               (56, 64, 128, 3, 2, 1), (28, 128, 256, 3, 2, 1), (14, 256, 512, 3, 2, 1),
               (56, 64, 128, 1, 1, 0), (14, 256, 512, 1, 1, 0)]
BGEMM_SHAPES = [(3136, 64, 576), (784, 128, 1152), (196, 256, 2304), (49, 512, 4608)]


class ColdTimer:
    def __init__(self, torch):
        self.torch = torch
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn, iters=10, warm=3):
        torch = self.torch
        for _ in range(warm):
            fn()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for e0, e1 in ev:
            self.flush.zero_()
            e0.record()
            fn()
            e1.record()
        torch.cuda.synchronize()
        return statistics.median(e0.elapsed_time(e1) for e0, e1 in ev)


def per_shape_numbers(torch, ops, hbm_gbs, peak_tbitops):
    """conv_sweep: the nine binary convolution shapes at batch 1 / 16 / 256 - `bconv` is dabnn_bconv on packed
    bits (counts out, default engine), `block_u8` the fused block on byte activations that the Net runs.
    bgemm_micro: sign-packing + bgemm at M and M x 256.  binconv_1x56x56x64: the BinConv operator on one image.
    Each entry: ms, Tbit-op/s (2*M*N*K, true K) and the fraction of its roofline, the slower of tensor time at the
    engine's measured peak and HBM time of the algorithmic bytes."""
    timer = ColdTimer(torch)
    g = torch.Generator(device="cuda").manual_seed(0)
    ri = lambda *shape: torch.randint(-2**63, 2**63 - 1, shape, device="cuda", dtype=torch.int64, generator=g)  # noqa: E731

    def entry(ms, bitops, nbytes):
        floor_ms = max(bitops / (peak_tbitops * 1e12), nbytes / (hbm_gbs * 1e9)) * 1e3
        return {"ms": round(ms, 4), "Tbit_op_per_s": round(bitops / ms / 1e9, 1), "GB_per_s": round(nbytes / ms / 1e6, 1),
                "roofline_frac": round(floor_ms / ms, 3), "bound": "tensor" if bitops / (peak_tbitops * 1e12) > nbytes / (hbm_gbs * 1e9) else "hbm"}

    sweep = []
    for (H, cin, cout, ks, s, p) in CONV_SHAPES:
        oh = (H + 2 * p - ks) // s + 1
        w = ri(cout * ks * ks * cin // 64)
        row = {"shape": f"{H}x{H}x{cin}->{cout} k{ks} s{s}"}
        for B in (1, 16, 256):
            x = ri(B, H, H, cin // 64)
            bitops = 2.0 * B * oh * oh * cout * ks * ks * cin
            raw_bytes = B * (H * H * cin / 8 + oh * oh * cout * 4) + cout * ks * ks * cin / 8
            r = {"bconv": entry(timer(lambda: ops.bconv(x, w, cout, ks, ks, p, p, s, s)), bitops, raw_bytes)}
            if ops.bconv_u8_supported(B, H, H, cin, cout, ks, ks, p, p, s, s):
                x8 = torch.randint(0, 2, (B, H, H, cin), device="cuda", dtype=torch.uint8, generator=g)
                we = ops.bconv_u8_expand_weights(w, cout, ks * ks * cin // 64)
                a, b = torch.rand(cout, device="cuda", generator=g), torch.rand(cout, device="cuda", generator=g)
                sc = torch.rand((B, oh, oh, cout), device="cuda", generator=g)
                blk_bytes = B * (H * H * cin / 8 + oh * oh * cout * 8.125) + cout * ks * ks * cin / 8
                r["block_u8"] = entry(timer(lambda: ops.bconv_u8_block(x8, we, cout, ks, ks, p, p, s, s, a, b, sc, True, True, False)),
                                      bitops, blk_bytes)
            row[f"batch{B}"] = r
        sweep.append(row)

    micro = []
    for (M, N, K) in BGEMM_SHAPES:
        row = {"M": M, "N": N, "K": K}
        for mult in (1, 256):
            Mb, kw = M * mult, K // 64
            xf = torch.rand((1, 1, Mb, K), device="cuda", generator=g) * 2 - 1
            wt = ri(kw, N)                                           # reference layout of `a`: [k][m]
            xb = ops.pack_mat(xf).view(Mb, kw)
            c = torch.zeros(Mb * N, device="cuda")
            t_pack = timer(lambda: ops.pack_mat(xf))
            t_gemm = timer(lambda: ops.bgemm(N, Mb, kw, wt, N, xb, kw, c, N))
            pack_bytes = Mb * K * 4 + Mb * K / 8
            bitops = 2.0 * Mb * N * K
            row[f"x{mult}"] = {"pack_ms": round(t_pack, 4), "pack_GB_per_s": round(pack_bytes / t_pack / 1e6, 1),
                               "pack_roofline_frac": round(pack_bytes / (hbm_gbs * 1e9) * 1e3 / t_pack, 3),
                               "bgemm": entry(t_gemm, bitops, Mb * K / 8 + N * K / 8 + 2 * Mb * N * 4)}   # C is read and written (+=)
            del xf, xb, c
        micro.append(row)

    x = torch.rand((1, 56, 56, 64), device="cuda", generator=g) * 2 - 1
    w = ri(64 * 9)
    t = timer(lambda: ops.binconv_forward(x, w, 64, 3, 3, 1, 1, 1, 1))
    one = entry(t, 2.0 * 3136 * 64 * 576, 3136 * 64 * 4 * 2 + 64 * 72)
    one["what"] = "BinConv operator on one 56x56x64 fp32 image: pack_mat + bconv (two launches), fp32 counts out"
    return sweep, micro, one


def small_batch_numbers(torch, Net, spec_bytes, batches=(1, 64), iters=30):
    """The network at batch 1 and 64 (device-resident inputs, CUDA-graph replay from the third run)."""
    out = {}
    for B in batches:
        net = Net.create()
        net.max_batch, net.engine, net.optimize = B, "auto", True
        net.read_buf(spec_bytes)
        x = torch.randn((B, IMAGE_HW, IMAGE_HW, 3), device="cuda")
        stream = torch.cuda.ExternalStream(net.cuda_stream)
        torch.cuda.synchronize()
        for _ in range(5):
            net.run_device_ptr(x.data_ptr(), B)
        net.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record()
            for _ in range(iters):
                net.run_device_ptr(x.data_ptr(), B)
            e1.record()
        net.sync()
        ms = e0.elapsed_time(e1) / iters
        out[f"batch{B}"] = {"ms_per_run": round(ms, 4), "images_per_s": round(B / ms * 1e3, 1)}
        net.close()
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    from dabnn_b200 import ops
    from dabnn_b200.bireal import OUTPUT_BLOB, build_bireal18
    from dabnn_b200.dab_format import write_dab
    from dabnn_b200.net import Net
    from dabnn_b200.replicas import bind_to_gpu_cpus, gather_logits, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    numa_bound = bind_to_gpu_cpus(local)   # before any pinned allocation
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    G = args.batch                                         # the global batch (1024)
    begin, end = shard_range(G, rank, world)
    Bs = end - begin                                       # this rank's shard
    spec = build_bireal18(image_hw=IMAGE_HW, num_classes=CLASSES)
    spec_bytes = write_dab(spec)
    net = Net.create()
    net.max_batch, net.engine, net.optimize = G, args.engine, True
    net.host_chunk = args.host_chunk
    net.read_buf(spec_bytes)
    stream = torch.cuda.ExternalStream(net.cuda_stream)

    # seeded synthetic inputs: the global batch in eight 128-image blocks, block j drawn from seed 1234 + j, so
    # that image i is the same image whatever the number of GPUs
    def images(lo, hi):
        parts = []
        for j in range(lo // 128, (hi + 127) // 128):
            gen = torch.Generator(device="cuda").manual_seed(1234 + j)
            blk = torch.randn((128, IMAGE_HW, IMAGE_HW, 3), device="cuda", generator=gen)
            parts.append(blk[max(lo - j * 128, 0):min(hi - j * 128, 128)])
        return torch.cat(parts).contiguous()

    x_full = images(0, G) if (world == 1 or args.weak) else None      # the weak leg runs all 1024 images on every GPU
    x_dev = x_full if world == 1 else images(begin, end)
    x_host = torch.empty((G if x_full is not None else Bs, IMAGE_HW, IMAGE_HW, 3), dtype=torch.float32, pin_memory=True)
    x_host[:Bs].copy_(x_dev)
    logits_ring = [torch.empty((G, CLASSES), dtype=torch.float32, pin_memory=True) for _ in range(2)]
    torch.cuda.synchronize()

    def make_steps(x_dev_t, x_host_t, B):
        dptr, hptr = x_dev_t.data_ptr(), x_host_t.data_ptr()
        e2e = {"k": 0, "pending": None}

        def step_device():
            net.run_device_ptr(dptr, B)

        # end to end: pipelined submissions, two in flight - the host copy of step k+1 overlaps the kernels of step k;
        # every step copies its input from pinned host memory and reads its logits back to the host
        def step_e2e():
            out = logits_ring[e2e["k"] & 1]          # the step two back, which used this buffer, has been waited for
            t = net.submit(hptr, B, OUTPUT_BLOB, out.data_ptr(), B * CLASSES)
            if e2e["pending"] is not None:
                net.wait(e2e["pending"])
            e2e["pending"], e2e["k"] = t, e2e["k"] + 1

        def drain():
            if e2e["pending"] is not None:
                net.wait(e2e["pending"])
                e2e["pending"] = None
        return step_device, step_e2e, drain

    def timed(fn, steps, on=None):
        on = on or stream
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(on):
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
        on.synchronize()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def repeated(fn, steps, after=None, on=None):
        """K steps, repeated until at least a second has been timed (every rank sees the same max-over-ranks time, so
        all agree on the count); returns (median ms of a repetition, repetitions)."""
        reps = [timed(fn, steps, on)]
        if after:
            after()
        for _ in range(min(args.max_reps - 1, int(args.min_seconds * 1e3 // max(reps[0], 1e-3)))):
            reps.append(timed(fn, steps, on))
            if after:
                after()
        return statistics.median(reps), len(reps)

    warm = max(args.warmup, 3)

    def measure(x_dev_t, x_host_t, B):
        step_device, step_e2e, drain = make_steps(x_dev_t, x_host_t, B)
        for _ in range(warm):
            step_device()
        net.sync()
        sampler = ClockSampler(local)
        sampler.start()
        ms_dev, reps_dev = repeated(step_device, args.steps)
        clocks = sampler.stop()
        for _ in range(2):
            step_e2e()
        drain()
        ms_e2e, reps_e2e = repeated(step_e2e, args.steps, after=drain)   # timed() synchronises the stream, so the last submission is inside
        return ms_dev, reps_dev, ms_e2e, reps_e2e, clocks

    ms_dev, reps_dev, ms_e2e, reps_e2e, clocks = measure(x_dev, x_host, Bs)

    # the bare copy: what the host side can deliver with no kernels at all (pinned -> device, every rank at once)
    # (on a stream torch owns: torch ties a pinned buffer to the streams that copied from it)
    h2d_stream = torch.cuda.Stream()

    def h2d_only():
        x_dev[:Bs].copy_(x_host[:Bs], non_blocking=True)
    with torch.cuda.stream(h2d_stream):
        h2d_only()
    ms_h2d, _ = repeated(h2d_only, args.steps, on=h2d_stream)

    weak = None
    if world > 1 and args.weak:
        x_host.copy_(x_full)
        w_dev, w_rd, w_e2e, w_re, _ = measure(x_full, x_host, G)
        weak = {"per_gpu_batch": G, "global_batch": G * world, "value": round(world * G * args.steps / (w_dev * 1e-3), 1),
                "ms_per_step": round(w_dev / args.steps, 4), "e2e_value": round(world * G * args.steps / (w_e2e * 1e-3), 1),
                "e2e_ms_per_step": round(w_e2e / args.steps, 4), "unit": "images/s"}

    # per-class device time of one step (CUDA events around every launch) -> roofline of the top class
    net.set_profiling(True)
    for _ in range(2):
        net.run_device_ptr(x_dev.data_ptr(), Bs)
        net.sync()
    classes = net.layer_times()
    net.set_profiling(False)
    stats = net.stats()

    # the final gather of logits (not on the data path): on rank 0, the logits rank 1 computed for its shard must be
    # bit-identical to rank 0's own run of the same images
    gathered_ok = None
    if world > 1:
        net.run_device_ptr(x_dev.data_ptr(), Bs)
        logits = torch.from_numpy(net.get_blob(OUTPUT_BLOB).reshape(Bs, CLASSES)).cuda()
        allv = gather_logits(logits, G)
        if rank == 0:
            b1, e1 = shard_range(G, 1, world)
            x1 = images(b1, e1)
            mine = torch.from_numpy(net.run(x1).get_blob(OUTPUT_BLOB).reshape(e1 - b1, CLASSES)).cuda()
            gathered_ok = bool(torch.equal(mine, allv[b1:e1])) and allv.shape == (G, CLASSES)

    result = None
    if rank == 0:
        hbm_gbs, peak_src = measured_peaks()
        total_ms = sum(classes.values())
        top = max(classes, key=classes.get)
        alg, flops = algorithmic_bytes(spec, Bs)
        layers = {k: {"ms": round(v, 4), "share": round(v / total_ms, 4),
                      "GBps": round(alg[k] / (v * 1e-3) / 1e9, 1) if k in alg else None} for k, v in classes.items()}
        peaks = {e: ops.measure_engine_peak(e) / 1e12 for e in ("tcgen05", "imma", "b1", "popc")}
        tf32_peak = ops.measure_tf32_peak() / 1e12
        eng = "tcgen05" if args.engine == "auto" else args.engine
        traffic = measured_traffic()
        conv_ms = classes.get("Bin Conv block", 0.0)
        conv_tops = flops["Bin Conv block"] / (conv_ms * 1e-3) / 1e12 if conv_ms else None
        if top == "Float Conv":
            # three tf32 products are issued per fp32 product; both sides of the fraction count issued products
            tf = 3.0 * flops[top] / (classes[top] * 1e-3) / 1e12
            roof = {"bound": "tensor", "kernel": "float convolutions (3xTF32 on tcgen05 kind::tf32)",
                    "achieved": round(tf, 1), "peak": round(tf32_peak, 1), "unit": "TFLOP/s", "frac": round(tf / tf32_peak, 4),
                    "peak_source": "tcgen05.mma kind::tf32 issue loop (128x128x8), measured in this run; "
                                   "achieved counts the 3 tf32 products issued per fp32 product",
                    "traffic": traffic.get(top, {}).get("bytes_per_image", 0) * Bs or None}
        else:
            gbps = alg[top] / (classes[top] * 1e-3) / 1e9
            blk = ("bconv_halo_kernel (13 launches: the 3x3 stride-1 blocks, halo tile read through shifted descriptors) + "
                   "bconv_u8_kernel (3 launches: the stride-2 blocks, one TMA box per tap); {0,1}-byte activations "
                   "loaded by TMA into tcgen05.mma kind::i8, affine + shortcut + signs (+ 2x2 average pooling) in the epilogue"
                   if eng == "tcgen05" else f"bcontract_kernel<{eng}> (16 fused binary conv blocks)")
            names = {"Bin Conv block": blk}
            roof = {"bound": "hbm", "kernel": names.get(top, top), "achieved": round(gbps, 1), "peak": hbm_gbs, "unit": "GB/s",
                    "frac": round(gbps / hbm_gbs, 4), "peak_source": peak_src,
                    "traffic": traffic.get(top, {}).get("bytes_per_image", 0) * Bs or None}
        whole = sum(alg.values()) / (ms_dev / args.steps * 1e-3) / 1e9
        h2d_bytes = Bs * IMAGE_HW * IMAGE_HW * 3 * 4
        h2d_gbps = world * h2d_bytes * args.steps / (ms_h2d * 1e-3) / 1e9     # ranks hold equal shards of 1024
        e2e_gbps = world * h2d_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
        result = {
            "metric": METRIC, "value": round(G * args.steps / (ms_dev * 1e-3), 1),
            "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": round(ms_dev / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": f"Bi-Real-Net-18-shaped BNN, 224x224x3 fp32 N(0,1) inputs, random-init, the {G}-image batch "
                                   f"sharded over {world} GPU(s) as independent replicas ({Bs} images per GPU), logits gathered at the end",
                       "global_batch": G, "per_gpu_batch": Bs, "engine": eng, "cpu_affinity": "gpu-local" if numa_bound else "default",
                       "timed_region": f"{args.steps} steps x {reps_dev} repetitions (median repetition reported)",
                       "l2": f"a step's activations ({stats['device_bytes'] * Bs // G >> 20} MB per GPU) exceed the 126 MB L2, so no tensor "
                             "survives in L2 from one step to the next; no flush needed"},
            "e2e": {"value": round(G * args.steps / (ms_e2e * 1e-3), 1), "unit": "images/s",
                    "h2d_bytes_per_step": h2d_bytes * world, "d2h_bytes_per_step": G * CLASSES * 4,
                    "ms_per_step": round(ms_e2e / args.steps, 4), "repetitions": reps_e2e,
                    "h2d_GBps": round(e2e_gbps, 1), "h2d_ceiling_GBps": round(h2d_gbps, 1),
                    "frac_of_h2d_ceiling": round(e2e_gbps / h2d_gbps, 3),
                    "note": "h2d_ceiling = the same pinned host->device copies with no kernels, all ranks at once"},
            "gpu_launches": stats["kernels_per_run"] * args.steps * world,
            "clocks": clocks, "roofline": roof,
            "whole_step": {"algorithmic_GB": round(sum(alg.values()) / 1e9, 3), "GBps": round(whole, 1), "frac_of_hbm": round(whole / hbm_gbs, 4)},
            "bconv_total": {"Tbit_op_per_s": round(conv_tops, 1) if conv_tops else None,
                            "engine_peaks_Tbit_op_per_s": {k: round(v, 1) for k, v in peaks.items()},
                            "tf32_peak_TFLOP_per_s": round(tf32_peak, 1)},
            "layers": layers, "device_bytes": stats["device_bytes"], "replica_check": gathered_ok, "weak": weak,
        }
        if world == 1 and not args.no_extras:
            sweep, micro, one = per_shape_numbers(torch, ops, hbm_gbs, peaks["tcgen05"])
            result["conv_sweep"], result["bgemm_micro"], result["binconv_1x56x56x64"] = sweep, micro, one
            result["small_batch"] = small_batch_numbers(torch, Net, spec_bytes)
            result["extras_note"] = ("per-shape numbers: L2 flushed (256 MB overwritten) before every timed call, median of 10; "
                                     "roofline_frac = max(2*M*N*K / measured tcgen05 int8 peak, algorithmic bytes / measured HBM copy rate) / time")
    net.sync()
    net.close()
    return result, world, rank


def run_reference(args, rounds, warmup):
    """The reference's CPU implementation, all host cores (P single-threaded processes)."""
    from oracle.cpu_baseline import ReferencePool
    pool = ReferencePool(IMAGE_HW, CLASSES, images_per_proc=args.cpu_images, rounds=rounds + warmup, native=True)
    try:
        for _ in range(warmup):
            pool.run_round()
        secs, imgs = 0.0, 0
        for _ in range(rounds):
            dt, n = pool.run_round()
            secs += dt
            imgs += n
    finally:
        pool.close()
    return {"value": round(imgs / secs, 2), "unit": "images/s", "cores": pool.procs_n, "kind": pool.kind,
            "sample": f"{pool.procs_n} single-threaded processes x {args.cpu_images} images x {rounds} rounds of the same "
                      f"network, reference sources built -O3 -march=native"}, secs / rounds


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="images per step over all GPUs")
    ap.add_argument("--engine", default="auto", choices=["auto", "tcgen05", "imma", "b1", "popc"])
    ap.add_argument("--host-chunk", type=int, default=512, help="images per staging buffer on the end-to-end path")
    ap.add_argument("--cpu-images", type=int, default=4, help="images per host process in the CPU baseline")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="the timed steps are repeated until this much has been measured")
    ap.add_argument("--max-reps", type=int, default=40)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-shape kernel numbers (N=1)")
    ap.add_argument("--no-weak", dest="weak", action="store_false", help="skip the 1024-images-per-GPU leg (N>1)")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    # stdout carries the one JSON line and nothing else: libraries that write to file descriptor 1 on their own (NCCL
    # prints its version banner there) are pointed at stderr, and the line goes out through a copy of the real stdout
    sys.stdout.flush()
    out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        if rank != 0:
            return
        base, sec_per_round = run_reference(args, rounds=max(1, args.steps), warmup=max(1, args.warmup))
        line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "images/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec_per_round * 1e3, 2),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64 xor-popcount + fp32 (CPU)",
                "data": "synthetic",
                "config": {"workload": "Bi-Real-Net-18-shaped BNN, 224x224x3 fp32 N(0,1) inputs, random-init; one step = a bounded "
                                       "sample of the 1024-image batch on the host cores", "global_batch": GLOBAL_BATCH},
                "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), file=out, flush=True)
        return

    if args.gpus > 1 and world == 1:   # convenience: launch the ranks ourselves
        import subprocess
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29517", str(Path(__file__).resolve()), *sys.argv[1:]]
        raise SystemExit(subprocess.call(cmd, stdout=out))

    result, world, rank = run_ours(args)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            try:
                result["cpu_baseline"], _ = run_reference(args, rounds=2, warmup=1)
            except Exception as e:  # the GPU numbers stand on their own
                result["cpu_baseline"] = {"unavailable": str(e)}
        print(json.dumps(result), file=out, flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
