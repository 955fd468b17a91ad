"""Host logic of tensor-parallel decode: the weight shards add up to the unsharded projections,
the sharded graphs have the shape the fused step expects, and the handle exchange keeps rank
order (2 gloo ranks on the CPU; the device-side exchange itself is covered by the GPU test)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from torq_b200.bf16 import from_bf16
from torq_b200.workloads import gemma3

CFG = gemma3.GemmaConfig(layers=2, hidden=128, intermediate=64 * 11, vocab=512, window=8, local_per_global=1, max_seq=32)


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_shards_add_up_to_the_full_projections(tp):
    P = gemma3.random_weights(CFG, 5)
    shards = [gemma3.shard_weights(CFG, P, tp, r) for r in range(tp)]
    rng = np.random.default_rng(1)
    D, nq, I = CFG.head_dim, CFG.n_q, CFG.intermediate
    L = P["layers"][0]
    # q rows split by head, the KV head replicated
    for s in shards:
        lay = s["layout"]
        hq, h0 = lay["heads"], lay["head0"]
        assert (s["layers"][0]["qkv"][0][:hq * D] == L["qkv"][0][h0 * D:(h0 + hq) * D]).all()
        assert (s["layers"][0]["qkv"][0][hq * D:] == L["qkv"][0][nq * D:]).all()
        # the o slice starts o_k_offset columns into the local attention output (the GPU's heads)
        assert lay["o_cols"][0] == h0 * D + lay["o_k_offset"] and 0 <= lay["o_k_offset"] < hq * D
    # every query head is computed by someone, the o columns tile [0, n_q * D)
    assert sorted({h for s in shards for h in range(s["layout"]["head0"], s["layout"]["head0"] + s["layout"]["heads"])}) == list(range(nq))
    assert [s["layout"]["o_cols"] for s in shards] == [(r * nq * D // tp, (r + 1) * nq * D // tp) for r in range(tp)]
    # o and down: the sum over the ranks of the K-split products is the full product (exact in integers)
    a = rng.integers(-50, 50, nq * D).astype(np.int64)
    full = L["o"][0].astype(np.int64) @ a
    parts = sum(s["layers"][0]["o"][0].astype(np.int64) @ a[s["layout"]["o_cols"][0]:s["layout"]["o_cols"][1]] for s in shards)
    assert (full == parts).all()
    act = rng.integers(-50, 50, I).astype(np.int64)
    full = L["down"][0].astype(np.int64) @ act
    parts = sum(s["layers"][0]["down"][0].astype(np.int64) @ act[s["layout"]["mlp"][0]:s["layout"]["mlp"][1]] for s in shards)
    assert (full == parts).all()
    assert shards[0]["layout"]["mlp"][0] == 0 and shards[-1]["layout"]["mlp"][1] == I
    # gate/up: a shard holds the gate rows and the matching up rows of its slice, with their scales
    for s in shards:
        w, sc = s["layers"][0]["gate_up"]
        i0, i1 = s["layout"]["mlp"]
        Il = i1 - i0
        assert Il % 64 == 0 and (w[:Il] == L["gate_up"][0][i0:i1]).all() and (w[Il:] == L["gate_up"][0][I + i0:I + i1]).all()
        assert (from_bf16(sc[Il:]) == from_bf16(L["gate_up"][1][I + i0:I + i1])).all()
    # LM head: vocabulary rows in rank order
    assert (np.concatenate([s["lm_head"][0] for s in shards]) == P["embed"][0]).all()
    assert [s["vocab_offset"] for s in shards] == [r * CFG.vocab // tp for r in range(tp)]


def test_sharded_graph_shape():
    P = gemma3.random_weights(CFG, 5)
    g = gemma3.build_decode_step(CFG, 1, gemma3.shard_weights(CFG, P, 2, 1), tp=2, rank=1)
    kinds = [op.kind for op in g.ops]
    assert kinds[:14] == ["embed", "rmsnorm", "gemv_w8", "rope_kv", "attn_decode", "gemv_w8", "allreduce", "rmsnorm", "rmsnorm",
                          "gemv_w8", "geglu", "gemv_w8", "allreduce", "rmsnorm"]
    assert all(op.attrs["i0"] == 2 and op.attrs["i1"] == 1 for op in g.ops if op.kind == "allreduce")
    assert g.ops[-1].kind == "argmax" and g.ops[-1].attrs["i0"] == CFG.vocab // 2 and g.ops[-1].attrs["i1"] == 2
    with pytest.raises(ValueError):
        gemma3.shard_weights(CFG, P, 3, 0)


WORKER = '''
import os, sys
import torch.distributed as dist
sys.path.insert(0, os.path.join(r"{root}", "torq-compiler_b200"))
from torq_b200.runtime import Executable

class Fake(Executable):
    def __init__(self, rank, size):
        self.rank, self.size, self.got = rank, size, None
    comm_info = property(lambda self: (self.rank, self.size))
    def comm_handle(self):
        return bytes([self.rank]) * 96
    def connect_peers(self, handles):
        self.got = handles

dist.init_process_group("gloo")
f = Fake(dist.get_rank(), dist.get_world_size())
f.connect_group()
assert [h[0] for h in f.got] == list(range(f.size)) and all(len(h) == 96 for h in f.got)
wrong = Fake((dist.get_rank() + 1) % 2, 2)
try:
    wrong.connect_group()
    raise SystemExit("a shard connected to a group where it has another rank")
except ValueError:
    pass
dist.destroy_process_group()
print("ok")
'''


def test_handle_exchange_keeps_rank_order_gloo(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=root))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29677", str(script)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    assert out.stdout.count("ok") == 2
