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
    d.free()
