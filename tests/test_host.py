"""CPU-only tests of the host logic: the .dab writer/reader pair, the synthetic model builder, the
C ABI surface (library loads and exports every declared symbol; argument checks that fail before
any CUDA work), and the multi-process logits gather over gloo."""
import ctypes as C
import os
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from dabnn_b200.bireal import build_bireal18
from dabnn_b200.dab_format import read_dab, write_dab
from dabnn_b200.model_spec import LayerSpec, ModelSpec

ROOT = Path(__file__).resolve().parent.parent


def test_dab_roundtrip():
    spec = build_bireal18(image_hw=64, num_classes=17)
    buf = write_dab(spec)
    back = read_dab(buf)
    assert back.version == 2 and back.input_name == "data" and tuple(back.input_shape) == (1, 64, 64, 3)
    assert len(back.layers) == len(spec.layers) and len(back.tensors) == len(spec.tensors)
    for a, b in zip(spec.tensors, back.tensors):
        assert (a.name, a.kind, tuple(a.shape), a.align_hwc_to_128) == (b.name, b.kind, tuple(b.shape), b.align_hwc_to_128)
        assert np.array_equal(np.asarray(a.data).ravel(), b.data.ravel())
    for a, b in zip(spec.layers, back.layers):
        assert (a.type, a.name, a.fields) == (b.type, b.name, b.fields)
    # wire-format invariants a FlatBuffers verifier would check: root offset in range, uint64
    # vectors 8-byte aligned
    assert int.from_bytes(buf[:4], "little") < len(buf)
    with pytest.raises(ValueError):
        read_dab(buf[:6])


def test_bireal18_shape():
    spec = build_bireal18()
    kinds = [l.type for l in spec.layers]
    assert kinds.count("BinConv2D") == 16 and kinds.count("Add") == 16
    assert kinds.count("FpConv2D") == 1 + 3 + 1 and kinds.count("AvePool") == 3 + 1
    t = {x.name: x for x in spec.tensors}
    assert t["s1b1_bconv_w"].data.size == 64 * 9 and not t["s1b1_bconv_w"].align_hwc_to_128
    assert t["s4b4_bconv_w"].data.size == 512 * 72 and t["s4b4_bconv_w"].align_hwc_to_128
    bitops = 0
    hw, cin = 56, 64
    for s, cout in enumerate((64, 128, 256, 512)):
        for blk in range(4):
            if s > 0 and blk == 0:
                hw //= 2
            bitops += 2 * hw * hw * cout * 9 * cin
            cin = cout
    assert abs(bitops - 3.353e9) < 2e6            # 16 binary convs = 3.353 Gbit-op per image


def test_library_exports_every_declared_symbol():
    from dabnn_b200 import capi
    from dabnn_b200.build import build_library
    build_library()
    lib = capi.load()
    header = (ROOT / "include" / "dabnn_b200.h").read_text()
    declared = set(re.findall(r"\b(dabnn_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(capi.declared_symbols()), declared ^ set(capi.declared_symbols())
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.dabnn_version().startswith(b"dabnn_b200")
    assert lib.dabnn_device_count() >= 0


def test_argument_checks_need_no_gpu():
    """The reference's BNN_ASSERT conditions are checked before any CUDA call."""
    from dabnn_b200 import capi
    lib = capi.load()
    x = np.zeros(128, np.float32)
    o = np.zeros(8, np.uint64)
    px, po = x.ctypes.data_as(C.c_void_p), o.ctypes.data_as(C.c_void_p)
    assert lib.dabnn_pack_mat(px, po, 1, 1, 2, 50, None) == 2                      # c % 64 != 0
    assert b"float_mat.c % 64 == 0" in lib.dabnn_last_error()
    assert lib.dabnn_pack_64(px, po, 100, None) == 2
    assert lib.dabnn_bgemm(-1, 1, 1, po, 1, po, 1, px, 1, 0, None) == 1
    assert lib.dabnn_bgemm(4, 4, 1, po, 2, po, 1, px, 4, 0, None) == 2             # lda < m
    assert lib.dabnn_bconv(po, po, 10, px, 1, 4, 4, 1, 3, 3, 3, 1, 1, 1, 1, 0, None) == 2   # 10 % 3 != 0
    assert lib.dabnn_prelu(px, px, 3, 4, 8, None) == 2
    assert b"slope must have size 1 or input.channels" in lib.dabnn_last_error()
    assert lib.dabnn_fused_binarize_im2col(px, po, 1, 4, 4, 7000, 3, 3, 1, 1, 1, 1, 1, 1, None) == 2
    assert lib.dabnn_net_run(None, px, 1, 0) == 1
    assert lib.dabnn_binconv_workspace_bytes(2, 8, 8, 64, 3, 3, 1, 1, 1, 1) == 2 * 8 * 8 * 8
    assert lib.dabnn_binconv_workspace_bytes(1, 8, 8, 32, 3, 3, 1, 1, 1, 1) == 64 * 6 * 8


def test_cpp_net_shim_compiles_and_fails_loudly_without_gpu(tmp_path):
    from dabnn_b200 import capi
    exe = tmp_path / "shim_check"
    lib_dir = capi.LIB_PATH.parent
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", f"-I{ROOT / 'include'}", str(ROOT / "tests" / "cpp_shim_check.cpp"),
                    "-o", str(exe), f"-L{lib_dir}", "-ldabnn_b200", f"-Wl,-rpath,{lib_dir}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    if capi.load().dabnn_device_count() == 0:
        assert r.returncode == 3 and "runtime_error" in r.stdout      # no device: loud failure, no fallback
    else:
        assert r.returncode == 0 and "created" in r.stdout


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from dabnn_b200 import capi
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(FileNotFoundError):
        capi.load()


def test_product_never_imports_the_oracle():
    for p in (ROOT / "dabnn_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".h", ".cpp") and p.is_file():
            text = p.read_text()
            assert "oracle" not in text.lower(), f"{p} mentions the oracle"


def test_shard_range():
    from dabnn_b200.replicas import shard_range
    for total, world in [(1024, 8), (10, 4), (3, 8), (0, 2)]:
        spans = [shard_range(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1


_WORKER = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
from dabnn_b200.replicas import shard_range, gather_logits
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
total, classes = 7, 5
full = torch.arange(total * classes, dtype=torch.float32).reshape(total, classes)
b, e = shard_range(total, rank, world)
out = gather_logits(full[b:e].clone(), total)
assert torch.equal(out, full), (rank, out)
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
"""


def test_two_rank_gather_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29531", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT)], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
