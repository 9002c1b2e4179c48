"""Python mirror of the reference's `bnn::Net` (dabnn/net.h:22-66) over the C ABI.

    net = Net.create()
    net.optimize = True            # public flags of the reference: optimize / run_fconv / strict
    net.read("model.dab")          # or net.read_buf(bytes)
    net.run(images)                # fp32 NHWC: numpy (host) array or torch CUDA tensor
    logits = net.get_blob("fc_out")

Differences from the reference, all additive: `run` accepts a batch of images (leading dimension)
and device-resident inputs; `get_blob` returns a numpy array copied from the device (or a torch
view of device memory with device=True).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .capi import DabnnError, check


class Net:
    def __init__(self):
        self._h = C.c_void_p()
        check(capi.load().dabnn_net_create(C.byref(self._h)))
        self.optimize, self.run_fconv, self.strict = True, True, True
        self.max_batch, self.engine = 1, "auto"
        self.host_chunk = 256   # images per staging buffer for host inputs (see dabnn_net_set_host_chunk)
        self._loaded = False
        self._keep = None

    @staticmethod
    def create():
        return Net()

    # ---- loading -------------------------------------------------------------------------------
    def _configure(self):
        lib = capi.load()
        check(lib.dabnn_net_set_flags(self._h, int(self.optimize), int(self.run_fconv), int(self.strict)))
        eng = capi.ENGINES[self.engine] if isinstance(self.engine, str) else int(self.engine)
        check(lib.dabnn_net_configure(self._h, int(self.max_batch), eng))
        check(lib.dabnn_net_set_host_chunk(self._h, int(self.host_chunk)))

    def read(self, path: str):
        self._configure()
        rc = capi.load().dabnn_net_read_file(self._h, str(path).encode())
        if rc == 3:
            raise ValueError(capi.load().dabnn_last_error().decode())   # std::invalid_argument, net.cpp:35
        check(rc)
        self._loaded = True

    def read_buf(self, buf: bytes):
        self._configure()
        check(capi.load().dabnn_net_read_buf(self._h, buf, len(buf)))
        self._loaded = True

    # ---- running -------------------------------------------------------------------------------
    def run(self, images):
        """images: fp32 NHWC, [H,W,C] or [B,H,W,C]; numpy array (host) or torch CUDA tensor."""
        lib = capi.load()
        if isinstance(images, np.ndarray):
            x = np.ascontiguousarray(images, dtype=np.float32)
            batch = x.shape[0] if x.ndim == 4 else 1
            self._keep = x
            check(lib.dabnn_net_run(self._h, x.ctypes.data_as(C.c_void_p), batch, 0))
        else:
            import torch
            if not (images.is_cuda and images.dtype == torch.float32 and images.is_contiguous()):
                raise TypeError("run: expected a contiguous fp32 CUDA tensor or a numpy array")
            batch = images.shape[0] if images.dim() == 4 else 1
            # the net enqueues on its own stream: order it after the producer of `images`
            torch.cuda.current_stream().synchronize()
            self._keep = images
            check(lib.dabnn_net_run(self._h, C.c_void_p(images.data_ptr()), batch, 1))
        return self

    def run_device_ptr(self, ptr: int, batch: int):
        """run() on a raw device pointer; the caller orders it after whatever produced the data."""
        check(capi.load().dabnn_net_run(self._h, C.c_void_p(ptr), batch, 1))

    def run_host_ptr(self, ptr: int, batch: int):
        """run() on a raw host pointer (e.g. pinned memory), no Python-side copies."""
        check(capi.load().dabnn_net_run(self._h, C.c_void_p(ptr), batch, 0))

    def submit(self, host_ptr: int, batch: int, blob: str, out_ptr: int, out_floats: int) -> int:
        """Enqueue run() on a (pinned) host input plus the copy of `blob` into the host buffer at
        `out_ptr`; returns a ticket for wait().  Keep two submissions in flight to overlap the host
        copy of one with the kernels of the other."""
        t = C.c_int()
        check(capi.load().dabnn_net_submit(self._h, C.c_void_p(host_ptr), batch, blob.encode(), C.c_void_p(out_ptr),
                                           out_floats, C.byref(t)))
        return t.value

    def wait(self, ticket: int):
        check(capi.load().dabnn_net_wait(self._h, ticket))

    def sync(self):
        check(capi.load().dabnn_net_sync(self._h))

    def blob_shape(self, name: str):
        dims = (C.c_int * 4)()
        rc = capi.load().dabnn_net_get_blob(self._h, name.encode(), dims, None, None, 0)
        if rc == 6:
            raise KeyError(capi.load().dabnn_last_error().decode())       # std::out_of_range, StrKeyMap.h:59
        check(rc)
        return tuple(dims)

    def get_blob(self, name: str, out: np.ndarray | None = None) -> np.ndarray:
        shape = self.blob_shape(name)
        if out is None:
            out = np.empty(shape, dtype=np.float32)
        check(capi.load().dabnn_net_get_blob(self._h, name.encode(), None, None, out.ctypes.data_as(C.c_void_p),
                                             out.size))
        return out

    def get_blob_bits(self, name: str) -> np.ndarray:
        """Packed sign bits written by a Binarize layer (reference dabnn/layers/Binarize.cpp:9): uint64 words
        [batch][h][w][c / 64]."""
        dims = (C.c_int * 4)()
        lib = capi.load()
        rc = lib.dabnn_net_get_blob_bits(self._h, name.encode(), dims, None, None, 0)
        if rc == 6:
            raise KeyError(lib.dabnn_last_error().decode())
        check(rc)
        out = np.empty(tuple(dims), dtype=np.uint64)
        check(lib.dabnn_net_get_blob_bits(self._h, name.encode(), None, None, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def get_blob_to_ptr(self, name: str, ptr: int, floats: int):
        check(capi.load().dabnn_net_get_blob(self._h, name.encode(), None, None, C.c_void_p(ptr), floats))

    def blob_device_ptr(self, name: str) -> int:
        p = C.c_void_p()
        check(capi.load().dabnn_net_get_blob(self._h, name.encode(), None, C.byref(p), None, 0))
        return p.value

    @property
    def output_names(self):
        lib, out, i = capi.load(), [], 0
        while True:
            s = lib.dabnn_net_output_name(self._h, i)
            if s is None:
                return out
            out.append(s.decode())
            i += 1

    @property
    def cuda_stream(self) -> int:
        return capi.load().dabnn_net_stream(self._h)

    def stats(self):
        k, b = C.c_int(), C.c_size_t()
        check(capi.load().dabnn_net_stats(self._h, C.byref(k), C.byref(b)))
        return {"kernels_per_run": k.value, "device_bytes": b.value}

    def set_profiling(self, on=True):
        check(capi.load().dabnn_net_set_profiling(self._h, int(on)))

    def layer_times(self):
        """Device milliseconds per layer class for the last run (reference Net::print_time)."""
        names, ms, n = (C.c_char_p * 32)(), (C.c_float * 32)(), C.c_int()
        check(capi.load().dabnn_net_layer_times(self._h, names, ms, 32, C.byref(n)))
        return {names[i].decode(): ms[i] for i in range(min(n.value, 32))}

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            capi.load().dabnn_net_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


__all__ = ["Net", "DabnnError"]
