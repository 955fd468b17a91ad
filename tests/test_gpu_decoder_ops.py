"""Each decoder kernel on its own against a plain torch fp32 computation of the same op
(bf16 rounding at the same points). bf16 results may differ by one unit in the last place
where the fp32 sums are added in another order; the tolerance is 2 ulp (2**-7 relative)."""
import numpy as np
import pytest
import torch

from gpu_exec import run_graph_gpu
from torq_b200.bf16 import from_bf16, to_bf16
from torq_b200.oplist import Graph

pytestmark = pytest.mark.gpu
ULP2 = 2.0 ** -7


def _bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


def _close(got_bits, want, tol=ULP2, floor=1e-3):
    got = from_bf16(got_bits)
    want = want.numpy() if isinstance(want, torch.Tensor) else want
    err = np.abs(got - want) / np.maximum(np.abs(want), floor)
    assert err.max() <= tol, (float(err.max()), got.ravel()[:6], want.ravel()[:6])


def test_embed_and_rmsnorm(device):
    rng = np.random.default_rng(1234)
    V, H, B = 300, 256, 5
    table = rng.integers(-127, 128, (V, H), dtype=np.int8)
    scale = to_bf16(rng.uniform(0.001, 0.01, V).astype(np.float32))
    tok = rng.integers(0, V, B).astype(np.int32)
    w = to_bf16(rng.normal(0, 0.1, H).astype(np.float32))
    g = Graph()
    t = g.input((B,), "i32")
    x = g.embed(t, table, scale, 16.0)
    y = g.rmsnorm(x, w, 1e-6)
    z = g.rmsnorm(y, w, 1e-6, residual=x)
    g.output(x), g.output(y), g.output(z)
    gx, gy, gz = run_graph_gpu(device, g, [tok])
    sc = torch.from_numpy(from_bf16(scale))
    rx = _bf(_bf(torch.from_numpy(table[tok].astype(np.float32)) * sc[tok][:, None]) * 16.0)
    wt = torch.from_numpy(from_bf16(w))
    norm = lambda v: _bf(v * torch.rsqrt((v * v).mean(-1, keepdim=True) + 1e-6) * (1 + wt))
    ry = norm(rx)
    rz = _bf(rx + norm(ry))
    _close(gx, rx, tol=0)
    _close(gy, ry)
    _close(gz, rz)


@pytest.mark.parametrize("B,K,N,splits", [(1, 1152, 1536, 0), (1, 6912, 1152, 0), (3, 512, 200, 1), (3, 1024, 77, 2),
                                          (8, 2048, 64, 4), (32, 1152, 256, 0), (1, 1152, 4096, 1),
                                          # batches above 8: the tensor-core kernel (K % 64 == 0), ragged N, K splits
                                          (9, 1152, 1536, 0), (32, 6912, 1152, 0), (17, 256, 200, 0), (32, 1152, 4100, 1),
                                          (12, 1024, 77, 2), (24, 2048, 130, 5),
                                          (16, 1040, 64, 0),   # K % 64 != 0: stays on the CUDA-core kernel
                                          (4, 2048, 320, 4)])  # the shape the allocation-free entry point is checked on
@pytest.mark.parametrize("f32", [False, True])
def test_gemv_w8(device, B, K, N, splits, f32):
    rng = np.random.default_rng(1234 + K + N)
    x = to_bf16(rng.normal(0, 1, (B, K)).astype(np.float32))
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    s = to_bf16(rng.uniform(0.5, 1.5, N).astype(np.float32) / (73.0 * np.sqrt(K)))
    g = Graph()
    y = g.gemv_w8(g.input((B, K), "bf16"), w, s, splits=splits, out_dtype="f32" if f32 else "bf16")
    g.output(y)
    got = run_graph_gpu(device, g, [x])[0]
    want = (torch.from_numpy(from_bf16(x)) @ torch.from_numpy(w.astype(np.float32)).T) * torch.from_numpy(from_bf16(s))
    if f32:  # fp32 results: relative to the largest magnitude, the summation order differs from torch's
        assert got.dtype == np.float32
        err = np.abs(got - want.numpy()).max() / np.abs(want.numpy()).max()
        assert err <= 1e-5, err
        return
    _close(got, _bf(want), floor=0.05)


def test_rope_kv_and_attention(device):
    rng = np.random.default_rng(1234)
    B, n_q, D, T, window = 2, 4, 256, 40, 16
    qw = to_bf16(rng.normal(0, 0.1, D).astype(np.float32))
    kw = to_bf16(rng.normal(0, 0.1, D).astype(np.float32))
    g = Graph()
    qkv_in = g.input((B, (n_q + 2) * D), "bf16")
    pos_in = g.input((1,), "i32")
    kc, vc = g.state((B, T, D), "bf16"), g.state((B, T, D), "bf16")
    q = g.rope_kv(qkv_in, pos_in, qw, kw, kc, vc, n_q=n_q, n_kv=1, head_dim=D, theta=10000.0, eps=1e-6)
    a_loc = g.attn_decode(q, pos_in, kc, vc, n_q=n_q, n_kv=1, head_dim=D, window=window, scale=D ** -0.5)
    a_glob = g.attn_decode(q, pos_in, kc, vc, n_q=n_q, n_kv=1, head_dim=D, window=0, scale=D ** -0.5)
    g.output(q), g.output(a_loc), g.output(a_glob)
    from torq_b200.runtime import Executable
    ex = Executable(device, g.serialize())
    d_in, d_pos = device.alloc(B * (n_q + 2) * D * 2), device.alloc(4)
    outs = [device.alloc(B * n_q * D * 2) for _ in range(3)]
    qwt, kwt = torch.from_numpy(from_bf16(qw)), torch.from_numpy(from_bf16(kw))
    Kc, Vc = torch.zeros(B, T, D), torch.zeros(B, T, D)
    half = D // 2
    inv = torch.pow(torch.tensor(10000.0), -torch.arange(half, dtype=torch.float32) / half)
    for pos in range(30):
        qkv = to_bf16(rng.normal(0, 1, (B, (n_q + 2) * D)).astype(np.float32))
        d_in.upload(qkv), d_pos.upload(np.array([pos], np.int32))
        ex.dispatch([d_in, d_pos], outs)
        got = [o.download((B, n_q * D), np.uint16) for o in outs]
        t = torch.from_numpy(from_bf16(qkv))
        qh, kh, vh = t[:, :n_q * D].reshape(B, n_q, D), t[:, n_q * D:(n_q + 1) * D].reshape(B, 1, D), t[:, (n_q + 1) * D:]
        norm = lambda v, w: _bf(v * torch.rsqrt((v * v).mean(-1, keepdim=True) + 1e-6) * (1 + w))
        cs, sn = torch.cos(pos * inv), torch.sin(pos * inv)
        rope = lambda v: _bf(torch.cat([v[..., :half] * cs - v[..., half:] * sn, v[..., half:] * cs + v[..., :half] * sn], -1))
        qr, kr = rope(norm(qh, qwt)), rope(norm(kh, kwt))
        Kc[:, pos], Vc[:, pos] = kr.reshape(B, D), vh
        _close(got[0], qr.reshape(B, -1), floor=0.02)
        for win, gout in ((window, got[1]), (0, got[2])):
            lo = max(0, pos - win + 1) if win else 0
            s = torch.einsum("bhd,btd->bht", qr * D ** -0.5, Kc[:, lo:pos + 1])
            a = _bf(torch.einsum("bht,btd->bhd", torch.softmax(s, -1), Vc[:, lo:pos + 1]))
            _close(gout, a.reshape(B, -1), tol=2 * ULP2, floor=0.05)
    ex.destroy()


def test_geglu_and_argmax(device):
    rng = np.random.default_rng(1234)
    B, I, V = 3, 640, 5000
    gu = to_bf16(rng.normal(0, 1.5, (B, 2 * I)).astype(np.float32))
    g = Graph()
    g.output(g.geglu(g.input((B, 2 * I), "bf16")))
    got = run_graph_gpu(device, g, [gu])[0]
    t = torch.from_numpy(from_bf16(gu))
    want = _bf(_bf(torch.nn.functional.gelu(t[:, :I], approximate="tanh")) * t[:, I:])
    _close(got, want, floor=0.02)
    logits = to_bf16(rng.normal(0, 1, (B, V)).astype(np.float32))
    logits[1, 4000] = logits[1, 17] = to_bf16(np.array([9.0], np.float32))[0]  # a tie: lowest index wins
    g = Graph()
    g.output(g.argmax(g.input((B, V), "bf16")))
    got = run_graph_gpu(device, g, [logits])[0]
    want = from_bf16(logits).argmax(-1)
    assert (got == want).all() and got[1] == 17


@pytest.mark.parametrize("fn", ["sigmoid", "gelu_tanh", "exp", "tanh", "silu"])
def test_act_bf16(device, fn):
    """bf16 activations (the reference's Sigmoid/Gelu/Exp/Trig patterns, host semantics: fp32 math, one
    rounding). Tolerance: one bf16 ulp (2^-8 relative) against torch's fp32 functions."""
    rng = np.random.default_rng(99)
    x = to_bf16(np.concatenate([rng.normal(0, 3, 5000), np.linspace(-12, 12, 3001), [0.0, -0.0, 30.0, -30.0]]).astype(np.float32))
    g = Graph()
    g.output(g.act_bf16(g.input(x.shape, "bf16"), fn))
    got = from_bf16(run_graph_gpu(device, g, [x])[0])
    t = torch.from_numpy(from_bf16(x))
    want = {"sigmoid": torch.sigmoid, "gelu_tanh": lambda v: torch.nn.functional.gelu(v, approximate="tanh"), "exp": torch.exp,
            "tanh": torch.tanh, "silu": torch.nn.functional.silu}[fn](t).numpy()
    err = np.abs(got - want)
    # 1 + tanh(.) cancels for negative arguments: tanh-GELU's tiny outputs carry fp32's absolute error (~|x| * 2^-24)
    floor = 2e-6 if fn == "gelu_tanh" else 1e-30
    assert (err <= np.abs(want) * 2.0 ** -7 + floor).all(), float((err / (np.abs(want) + floor)).max())
    assert len(np.unique(got)) > 100


@pytest.mark.parametrize("B,K,N,with_zp", [(1, 640, 256, True), (3, 1152, 200, True), (8, 2048, 96, False),
                                           # above 8 tokens: the tensor-core kernel (K in chunks of 1024, ragged N and B)
                                           (9, 640, 256, True), (16, 1152, 200, True), (32, 2048, 1000, True),
                                           (27, 6912, 136, False)])
def test_gemv_block_quantised(device, B, K, N, with_zp):
    """The reference's Gemma weight form (tests/testdata/torch_ops/matmul_dql_q8_0.mlir: x 1x640 bf16, W 640x256
    si8, scales and zero points 20x256, block 32): dequantised weights are rounded to bf16, the product
    accumulates in fp32. First case = that fixture's shapes."""
    rng = np.random.default_rng(640 + K)
    x = to_bf16(rng.normal(0, 1, (B, K)).astype(np.float32))
    w = rng.integers(-128, 128, (K, N), dtype=np.int8)
    sc = to_bf16((rng.uniform(0.5, 1.5, (K // 32, N)) / (73.0 * np.sqrt(K))).astype(np.float32))
    zp = rng.integers(-8, 9, (K // 32, N), dtype=np.int8) if with_zp else None
    g = Graph()
    g.output(g.gemv_q8b(g.input((B, K), "bf16"), w, sc, zp, 32))
    got = run_graph_gpu(device, g, [x])[0]
    wz = torch.from_numpy(w.astype(np.float32)) - (torch.from_numpy(np.repeat(zp, 32, 0).astype(np.float32)) if with_zp else 0.0)
    wd = _bf(wz * torch.from_numpy(np.repeat(from_bf16(sc), 32, 0)))
    want = _bf(torch.from_numpy(from_bf16(x)) @ wd)
    _close(got, want, floor=0.05)
