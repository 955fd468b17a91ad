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

CFG = gemma3.GemmaConfig(layers=2, hidden=128, intermediate=256, vocab=512, window=8, local_per_global=1, max_seq=32)


@pytest.mark.parametrize("tp", [2, 4])
def test_shards_add_up_to_the_full_projections(tp):
    P = gemma3.random_weights(CFG, 5)
    shards = [gemma3.shard_weights(CFG, P, tp, r) for r in range(tp)]
    rng = np.random.default_rng(1)
    D, nq, I = CFG.head_dim, CFG.n_q, CFG.intermediate
    L = P["layers"][0]
    # q rows split by head, the KV head replicated
    q_rows = np.concatenate([s["layers"][0]["qkv"][0][:nq // tp * D] for s in shards])
    assert (q_rows == L["qkv"][0][:nq * D]).all()
    for s in shards:
        assert (s["layers"][0]["qkv"][0][nq // tp * D:] == L["qkv"][0][nq * D:]).all()
    # o and down: the sum over the ranks of the K-split products is the full product (exact in integers)
    a = rng.integers(-50, 50, nq * D).astype(np.int64)
    full = L["o"][0].astype(np.int64) @ a
    parts = sum(s["layers"][0]["o"][0].astype(np.int64) @ a[r * nq // tp * D:(r + 1) * nq // tp * D] for r, s in enumerate(shards))
    assert (full == parts).all()
    act = rng.integers(-50, 50, I).astype(np.int64)
    full = L["down"][0].astype(np.int64) @ act
    parts = sum(s["layers"][0]["down"][0].astype(np.int64) @ act[r * I // tp:(r + 1) * I // tp] for r, s in enumerate(shards))
    assert (full == parts).all()
    # gate/up: shard r holds gate rows and the matching up rows of its slice, with their scales
    for r, s in enumerate(shards):
        w, sc = s["layers"][0]["gate_up"]
        Il = I // tp
        assert (w[:Il] == L["gate_up"][0][r * Il:(r + 1) * Il]).all() and (w[Il:] == L["gate_up"][0][I + r * Il:I + (r + 1) * Il]).all()
        assert (from_bf16(sc[Il:]) == from_bf16(L["gate_up"][1][I + r * Il:I + (r + 1) * Il])).all()
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
