"""One rank of the tensor-parallel decode check (run under torch.distributed.run, one process
per GPU): every rank builds its shard of the decode step, the shards connect through each
other's memory, and the group decodes teacher-forced tokens. Rank 0 compares the greedy ids and
the gathered logits with the fp32 torch reference of the unsharded model and writes the outcome
as one JSON line."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(HERE, "..", "torq-compiler_b200"))

from ref_decoder import RefDecoder  # noqa: E402
from torq_b200.runtime import Device, Executable  # noqa: E402
from torq_b200.workloads import gemma3  # noqa: E402


def main():
    size_name, batch, steps, gain = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), float(sys.argv[4])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo")  # host transport for the handles only
    cfg = {"small": gemma3.GemmaConfig(layers=3, hidden=256, intermediate=1024, vocab=4096, window=24, local_per_global=2,
                                       max_seq=96),
           # 8 GPUs: every GPU needs at least as many rows of each projection as it has SMs
           "small8": gemma3.GemmaConfig(layers=3, hidden=256, intermediate=64 * 27, vocab=4096, window=24, local_per_global=2,
                                        max_seq=96),
           # one query head over two GPUs: the shared-head path (o-projection column slices) and an uneven
           # MLP split (7 blocks of 64) at a group size of 2
           "shared": gemma3.GemmaConfig(layers=3, hidden=256, n_q=1, intermediate=64 * 7, vocab=4096, window=24,
                                        local_per_global=2, max_seq=96),
           "full": gemma3.GemmaConfig()}[size_name]
    params = gemma3.random_weights(cfg, 1234, gain)
    dev = Device(local)
    shard = gemma3.shard_weights(cfg, params, world, rank)
    ex = Executable(dev, gemma3.build_decode_step(cfg, batch, shard, with_logits=True, tp=world, rank=rank).serialize())
    assert ex.comm_info == (rank, world)
    assert ex.launch_count == 1, "the shard must run as the fused decode step"
    ex.connect_group()
    vl = cfg.vocab // world
    d_tok, d_pos = dev.alloc(batch * 4), dev.alloc(4)
    d_next, d_logits = dev.alloc(batch * 4), dev.alloc(batch * vl * 4)
    ref = RefDecoder(cfg, params, batch, device="cpu" if size_name != "full" else None) if rank == 0 else None
    rng = np.random.default_rng(7)
    toks = rng.integers(0, cfg.vocab, (steps, batch)).astype(np.int32)
    worst, agree, total = 0.0, 0, 0
    for pos in range(steps):
        d_tok.upload(toks[pos])
        d_pos.upload(np.array([pos], np.int32))
        ex.dispatch([d_tok, d_pos], [d_next, d_logits])
        dev.wait(30.0)
        nxt = d_next.download((batch,), np.int32)
        logits = torch.from_numpy(d_logits.download((batch, vl), np.float32))
        gathered = [torch.empty_like(logits) for _ in range(world)] if rank == 0 else None
        dist.gather(logits, gathered, dst=0)
        ids = [torch.empty(batch, dtype=torch.int32) for _ in range(world)] if rank == 0 else None
        dist.gather(torch.from_numpy(nxt.copy()), ids, dst=0)
        if rank == 0:
            full = torch.cat(gathered, -1).numpy()
            assert all((i.numpy() == nxt).all() for i in ids), "the ranks disagree on the greedy ids"
            assert (nxt == full.argmax(-1)).all(), "ids are not the arg max of the gathered logits"
            r_next, r_logits = ref.step(toks[pos], pos)
            worst = max(worst, float(np.abs(full - r_logits).max() / np.abs(r_logits).max()))
            agree += int((nxt == r_next).sum())
            total += batch
    if rank == 0:
        print("TP_RESULT " + json.dumps({"world": world, "batch": batch, "steps": steps, "worst_rel": worst,
                                         "agree": agree, "total": total}), flush=True)
    dist.barrier()
    ex.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
