"""The allocation-free BinConv entry point (dabnn_binconv_forward_static).

It exists for hosts that cannot allocate device memory where they call the library - they own the
whole device heap themselves, or run inside a callback where cudaMalloc is forbidden - so its
scratch is a fixed buffer inside the library.  The test calls it twice in a row through the C ABI
(second call on a different, larger problem, so that stale contents of the shared buffer would show)
and requires bit-identical output to the workspace-taking entry point; it also checks the refusal of
shapes beyond the buffer.  Collected last on purpose: a run that stops at the first failure has
then already executed every other test."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_workspace_entry_twice():
    from dabnn_b200 import capi, ops
    lib = capi.load()
    cap = capi.BINCONV_STATIC_BYTES
    g = torch.Generator(device="cuda").manual_seed(77)
    cases = [(2, 14, 64, 64, 1), (5, 28, 128, 64, 2), (3, 6, 32, 16, 1), (2, 14, 64, 64, 1)]
    for n, hw, cin, cout, stride in cases:
        x = torch.rand((n, hw, hw, cin), device="cuda", generator=g) * 2 - 1
        kwords = 9 * cin // 64 if cin == 64 else (9 * cin + 127) // 128 * 2
        w = torch.randint(-2**63, 2**63 - 1, (cout * kwords,), device="cuda", dtype=torch.int64, generator=g)
        if (9 * cin) % 128 and cin != 64:
            w.view(cout, kwords)[:, -1] = 0       # the converter zero-fills the 128-bit tail
        expected = ops.binconv_forward(x, w, cout, 3, 3, 1, 1, stride, stride)
        first = ops.binconv_forward_static(x, w, cout, 3, 3, 1, 1, stride, stride)
        second = ops.binconv_forward_static(x, w, cout, 3, 3, 1, 1, stride, stride)
        assert torch.equal(first, expected)
        assert torch.equal(second, expected)
        if cin % 64 == 0 and n <= 3:   # and against the CPU checker, not only against the library's other entry
            from oracle.oracle import Port
            cnt = Port().binconv_forward(x[0].cpu().numpy(), w.cpu().numpy().view(np.uint64), cout, 3, 3, 1, 1, stride, stride)
            assert first[0].cpu().numpy().tobytes() == cnt.tobytes()
    # after the first call on the device (which loads the array's module and looks its address up) a call neither
    # takes nor returns device memory: the free-byte count of the device does not move
    n, hw, cin, cout, stride = cases[0]
    x = torch.rand((n, hw, hw, cin), device="cuda", generator=g) * 2 - 1
    w = torch.randint(-2**63, 2**63 - 1, (cout * 9,), device="cuda", dtype=torch.int64, generator=g)
    out = torch.empty((n, hw, hw, cout), device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        capi.check(lib.dabnn_binconv_forward_static(C.c_void_p(x.data_ptr()), C.c_void_p(w.data_ptr()), w.numel(),
                                                    C.c_void_p(out.data_ptr()), n, hw, hw, cin, cout, 3, 3, 1, 1, stride, stride, 0,
                                                    C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    # a problem whose packed input exceeds the built-in buffer is refused, nothing is launched
    n_big = cap // (56 * 56 * 8) + 1
    dummy = torch.empty(8, device="cuda")
    rc = lib.dabnn_binconv_forward_static(C.c_void_p(dummy.data_ptr()), C.c_void_p(dummy.data_ptr()), 64 * 9,
                                          C.c_void_p(dummy.data_ptr()), n_big, 56, 56, 64, 64, 3, 3, 1, 1, 1, 1, 0, None)
    assert rc == 2 and b"built-in buffer" in lib.dabnn_last_error()
    torch.cuda.synchronize()
