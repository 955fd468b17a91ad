"""One rank of the "a member misses a step" check (run under torch.distributed.run, 2 processes, one per
GPU, kernel wait limit 250 ms through TB200_WAIT_LIMIT_MS; the ranks meet at a host barrier before every step, so
their launches are a few milliseconds apart at most). Both ranks decode three steps; at the fourth
rank 1 launches nothing (it stays alive, its memory stays mapped, none of its kernels is in flight), so the
cross-GPU barrier of rank 0's kernel runs into its limit: the kernel returns, the host wait answers
ABORTED, the device stays usable. Both ranks then destroy the shard executables, create and connect them
again and repeat the first three steps: the results must equal the first run's bit for bit. Nothing here
faults, traps or hangs a GPU: the only failure is a bounded wait that gives up."""
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(HERE, ".."))
sys.path.insert(0, os.path.join(HERE, "..", "torq-compiler_b200"))

from gpu_exec import run_graph_gpu  # noqa: E402
from oracle_exec import run_graph  # noqa: E402
from torq_b200.oplist import Graph  # noqa: E402
from torq_b200.runtime import Device, Executable, TorqB200Error  # noqa: E402
from torq_b200.workloads import gemma3  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    assert world == 2 and os.environ.get("TB200_WAIT_LIMIT_MS") == "250"
    dist.init_process_group("gloo")
    cfg = gemma3.GemmaConfig(layers=3, hidden=256, intermediate=1024, vocab=4096, window=24, local_per_global=2, max_seq=96)
    params = gemma3.random_weights(cfg, 1234, 0.3)
    dev = Device(local)
    shard = gemma3.shard_weights(cfg, params, world, rank)
    blob = gemma3.build_decode_step(cfg, 2, shard, with_logits=True, tp=world, rank=rank).serialize()
    vl = cfg.vocab // world
    d_tok, d_pos = dev.alloc(8), dev.alloc(4)
    d_next, d_logits = dev.alloc(8), dev.alloc(2 * vl * 4)
    toks = np.random.default_rng(7).integers(0, cfg.vocab, (4, 2)).astype(np.int32)

    def connect():
        ex = Executable(dev, blob)
        ex.connect_group()
        return ex

    def step(ex, pos, launch=True):
        d_tok.upload(toks[pos])
        d_pos.upload(np.array([pos], np.int32))
        dev.wait(30.0)
        dist.barrier()
        if launch:
            ex.dispatch([d_tok, d_pos], [d_next, d_logits])
        dev.wait(30.0)
        return d_next.download((2,), np.int32).copy(), d_logits.download((2, vl), np.float32).copy()

    ex = connect()
    first = [step(ex, pos) for pos in range(3)]
    dist.barrier()
    # the fourth step: rank 1 launches nothing
    aborted, message, waited = False, "", 0.0
    t0 = time.monotonic()
    try:
        step(ex, 3, launch=rank == 0)
    except TorqB200Error as e:
        aborted, message = e.status_name == "ABORTED", str(e)
    waited = time.monotonic() - t0
    dist.barrier()  # rank 0's kernel has returned: only now may either side free what the other one maps
    ex.destroy()
    dist.barrier()
    # the device is still usable: a single-GPU case against the oracle
    rng = np.random.default_rng(rank)
    x = rng.integers(-128, 128, (64, 256)).astype(np.int8)
    g = Graph()
    g.output(g.fully_connected(g.input(x.shape), rng.integers(-127, 128, (128, 256)).astype(np.int8),
                               rng.integers(-1000, 1000, 128).astype(np.int32), np.full(128, 1342177280, np.int32),
                               np.full(128, 40, np.int8), input_zp=3, out_zp=-2))
    single_ok = bool((run_graph_gpu(dev, g, [x])[0] == run_graph(g, [x])[0]).all())
    # create, connect, and repeat from position 0
    ex = connect()
    second = [step(ex, pos) for pos in range(3)]
    same = all((a[0] == b[0]).all() and (a[1].view(np.uint32) == b[1].view(np.uint32)).all() for a, b in zip(first, second))
    flags = torch.tensor([int(aborted), int(single_ok), int(same)], dtype=torch.int32)
    gathered = [torch.empty_like(flags) for _ in range(world)] if rank == 0 else None
    dist.gather(flags, gathered, dst=0)
    if rank == 0:
        print("TP_ABORT " + json.dumps({"rank0_aborted": bool(gathered[0][0]), "rank1_aborted": bool(gathered[1][0]),
                                        "message": message, "waited_s": round(waited, 3),
                                        "single_gpu_ok": [bool(t[1]) for t in gathered],
                                        "bit_identical_after_recreate": [bool(t[2]) for t in gathered]}), flush=True)
    dist.barrier()
    ex.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
