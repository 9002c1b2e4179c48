"""TEST / MEASUREMENT INFRASTRUCTURE ONLY: times the reference's own CPU implementation of the
Bi-Real-18-shaped network on the host cores.

The reference is single-threaded and not re-entrant (function-local static scratch buffers, e.g.
dabnn/fused_binarize_im2col.h:23, dabnn/bgemm.h:79-81), so "all host cores" means P independent
single-threaded *processes*, each running the compiled reference (oracle/_ref/libdabnn_ref.so, or
the plain-C restatement when that library is absent) on its own images.  The parent releases all
workers at once and measures wall-clock time until the last one finishes.

Used by bench.py (`cpu_baseline` object and `--impl reference`).  Worker protocol on stdin/stdout:
the worker prints READY after building its net, waits for a line, runs, prints `DONE <seconds>`.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _worker(image_hw: int, classes: int, images: int, rounds: int, seed: int, native: int):
    import numpy as np
    sys.path.insert(0, str(ROOT))
    from dabnn_b200.bireal import build_bireal18
    from oracle.oracle import REF_NATIVE_SO, REF_SO, Port, Ref
    spec = build_bireal18(image_hw=image_hw, num_classes=classes)
    rng = np.random.default_rng(seed)
    imgs = rng.normal(0, 1, (images, image_hw, image_hw, 3)).astype(np.float32)
    so = REF_NATIVE_SO if native else REF_SO
    if so.exists():
        net = Ref(native=bool(native)).build_net(spec, optimize=True)

        def run(img):
            net.ref._ck(net.ref.lib.ref_net_run(net.handle, img.ctypes.data_as(ctypes.c_void_p)))
        kind = "reference"
    else:
        port = Port()

        def run(img):
            port.run_model(spec, img)
        kind = "port"
    run(imgs[0].copy())                                   # warm-up (also sizes the scratch mats)
    print("READY", kind, flush=True)
    for _ in range(rounds):
        if not sys.stdin.readline():
            return
        t0 = time.perf_counter()
        for i in range(images):
            run(imgs[i].copy())                           # in-place layers write through the input
        print("DONE", time.perf_counter() - t0, flush=True)


class ReferencePool:
    """P single-threaded reference processes, released together for each timed round."""

    def __init__(self, image_hw=224, classes=1000, images_per_proc=2, procs=None, rounds=1, native=False):
        self.procs_n = procs or len(os.sched_getaffinity(0))
        self.images_per_proc = images_per_proc
        self.rounds = rounds
        env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
        self.procs = [subprocess.Popen(
            [sys.executable, str(Path(__file__).resolve()), "worker", str(image_hw), str(classes),
             str(images_per_proc), str(rounds), str(1000 + i), str(int(native))],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env) for i in range(self.procs_n)]
        self.kind = None
        for p in self.procs:
            line = p.stdout.readline().split()
            if not line or line[0] != "READY":
                self.close()
                raise RuntimeError("reference worker failed to start")
            self.kind = line[1]

    def run_round(self):
        """One timed round: returns (wall seconds, images processed)."""
        t0 = time.perf_counter()
        for p in self.procs:
            p.stdin.write("go\n")
            p.stdin.flush()
        for p in self.procs:
            line = p.stdout.readline().split()
            if not line or line[0] != "DONE":
                raise RuntimeError("reference worker died")
        return time.perf_counter() - t0, self.procs_n * self.images_per_proc

    def close(self):
        for p in self.procs:
            try:
                p.stdin.close()
            except Exception:
                pass
        for p in self.procs:
            try:
                p.wait(timeout=10)
            except Exception:
                p.kill()


if __name__ == "__main__" and len(sys.argv) > 1 and sys.argv[1] == "worker":
    _worker(*map(int, sys.argv[2:8]))
