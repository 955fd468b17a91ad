"""tb200_gemv_w8_noalloc, the entry point for callers that may not allocate device memory
(hosts whose own allocator already owns the HBM; loops that cannot take an allocation's
device-wide synchronisation). Its split-K partial sums live in a fixed array inside the
library instead of the executable's arena. The test calls it through the C ABI twice in a
row, with different inputs, and wants the same bits as the executable path (tb200_dispatch
of a one-op graph) gives for those inputs: the second call also shows that what the first
call left in the shared scratch does not leak into the result. Runs last (file name), and
also on its own in a fresh process."""
import ctypes as C

import numpy as np
import pytest

from gpu_exec import run_graph_gpu
from torq_b200.bf16 import to_bf16
from torq_b200.oplist import Graph

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,K,N,splits,f32", [(1, 6912, 1152, 0, False), (4, 2048, 320, 4, True)])
def test_noalloc_gemv_matches_executable_path(device, B, K, N, splits, f32):
    lib = device._lib
    rng = np.random.default_rng(1234)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    scale = to_bf16((rng.uniform(0.5, 1.5, N) / (73.0 * np.sqrt(K))).astype(np.float32))
    g = Graph()
    g.output(g.gemv_w8(g.input((B, K), "bf16"), w, scale, splits=splits, out_dtype="f32" if f32 else "bf16"))
    d_x, d_w, d_s = device.alloc(B * K * 2), device.alloc(N * K), device.alloc(N * 2)
    out_dtype = np.float32 if f32 else np.uint16
    d_y = device.alloc(B * N * np.dtype(out_dtype).itemsize)
    d_w.upload(w), d_s.upload(scale)
    for call in range(2):  # two calls in a row share the library's scratch array
        x = to_bf16(rng.normal(0, 1 + call, (B, K)).astype(np.float32))
        want = run_graph_gpu(device, g, [x])[0]
        d_x.upload(x)
        st = lib.tb200_gemv_w8_noalloc(device.ordinal, C.c_void_p(device.stream), C.c_void_p(d_x.pointer),
                                       C.c_void_p(d_w.pointer), C.c_void_p(d_s.pointer), C.c_void_p(d_y.pointer),
                                       int(f32), B, N, K, splits)
        assert st == 0
        got = d_y.download((B, N), out_dtype)
        assert (got == want).all(), f"call {call}: {(got != want).sum()} of {got.size} differ"
        assert len(np.unique(got)) > 8
    for b in (d_x, d_w, d_s, d_y):
        b.free()


def test_noalloc_gemv_rejects_what_does_not_fit(device):
    lib = device._lib
    d = device.alloc(4096)
    p = C.c_void_p(d.pointer)
    # 16 slices x 32 rows x 4096 columns = 2,097,152 partial sums > 1,048,576
    assert lib.tb200_gemv_w8_noalloc(device.ordinal, None, p, p, p, p, 0, 32, 4096, 8192, 16) == 11  # OUT_OF_RANGE
    assert lib.tb200_gemv_w8_noalloc(device.ordinal, None, p, p, p, p, 0, 1, 64, 24, 1) == 3           # K % 16 != 0
    assert lib.tb200_gemv_w8_noalloc(device.ordinal, None, None, p, p, p, 0, 1, 64, 32, 1) == 3        # NULL input
    # pointers the kernels' 16-byte loads cannot take are refused on the host, nothing is launched
    off = C.c_void_p(d.pointer + 8)
    assert lib.tb200_gemv_w8_noalloc(device.ordinal, None, off, p, p, p, 0, 1, 64, 32, 1) == 3         # x misaligned
    assert lib.tb200_gemv_w8_noalloc(device.ordinal, None, p, off, p, p, 0, 1, 64, 32, 1) == 3         # W misaligned
    assert lib.tb200_gemv_w8_noalloc(device.ordinal, None, p, p, C.c_void_p(d.pointer + 1), p, 0, 1, 64, 32, 1) == 3
    assert lib.tb200_gemv_w8_noalloc(device.ordinal, None, p, p, p, C.c_void_p(d.pointer + 2), 1, 1, 64, 32, 1) == 3  # fp32 y
    # one slice of K = 4096 at batch 32 is more than the tensor-core kernel can stage in shared memory
    assert lib.tb200_gemv_w8_noalloc(device.ordinal, None, p, p, p, p, 0, 32, 8, 4096, 1) == 11
    d.free()


def test_noalloc_gemv_on_a_second_device_and_current_device_kept():
    """The scratch array's address and the kernels' attributes are per device; the caller's current device
    is left as it was."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from torq_b200.runtime import Device
    B, K, N = 32, 1152, 256   # batch 32: the tensor-core kernel with more than 48 KB of shared memory
    rng = np.random.default_rng(7)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    scale = to_bf16((rng.uniform(0.5, 1.5, N) / (73.0 * np.sqrt(K))).astype(np.float32))
    x = to_bf16(rng.normal(0, 1, (B, K)).astype(np.float32))
    results = []
    for ordinal in (0, 1):
        dev = Device(ordinal)
        torch.cuda.set_device(0)
        d_x, d_w, d_s, d_y = dev.alloc(x.nbytes), dev.alloc(w.nbytes), dev.alloc(scale.nbytes), dev.alloc(B * N * 2)
        d_x.upload(x), d_w.upload(w), d_s.upload(scale)
        dev.wait()
        torch.cuda.set_device(0)
        st = dev._lib.tb200_gemv_w8_noalloc(ordinal, C.c_void_p(dev.stream), C.c_void_p(d_x.pointer), C.c_void_p(d_w.pointer),
                                            C.c_void_p(d_s.pointer), C.c_void_p(d_y.pointer), 0, B, N, K, 0)
        assert st == 0
        assert torch.cuda.current_device() == 0
        results.append(d_y.download((B, N), np.uint16))
        for b in (d_x, d_w, d_s, d_y):
            b.free()
        dev.close()
    assert (results[0] == results[1]).all() and len(np.unique(results[0])) > 8
