"""World-size-2 (gloo, CPU) check of the batch-replica host logic: scatter a batch, run each
shard through an engine (the CPU oracle stands in for the per-GPU executable here), gather,
and compare with the unsharded result."""
import os
import socket
import sys

import numpy as np
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_items, q):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "torq-compiler_b200"), os.path.join(root, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    from oracle_exec import run_graph
    from torq_b200 import replicas
    from torq_b200.workloads.mobilenet_v2 import build_mobilenet_v2, synthetic_images
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    res = 32
    x_global = synthetic_images(n_items, resolution=res) if rank == 0 else None
    x_local = replicas.scatter_batch(x_global, n_items, (res, res, 3), np.int8)
    lo, hi = replicas.shard_bounds(n_items, world, rank)
    assert x_local.shape[0] == hi - lo
    g, _ = build_mobilenet_v2(hi - lo, resolution=res)
    y_local = run_graph(g, [x_local])[0]
    y = replicas.gather_batch(y_local, n_items)
    slow = replicas.max_over_ranks(1.0 + rank)
    assert slow == float(world)
    if rank == 0:
        g_all, _ = build_mobilenet_v2(n_items, resolution=res)
        want = run_graph(g_all, [x_global])[0]
        q.put(bool((y == want).all()) and y.shape == want.shape)
    dist.barrier()
    dist.destroy_process_group()


def test_shard_bounds_cover_every_item():
    from torq_b200.replicas import shard_bounds
    for n in (1, 5, 8, 256, 257):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_rank_replicas_match_single_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 5, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


def test_numa_cpus_of_gpu_reads_sysfs(tmp_path):
    """The NUMA lookup against a fake sysfs tree: node of the PCI device -> that node's CPU list; absent or -1 -> empty."""
    from torq_b200.replicas import _parse_cpulist, numa_cpus_of_gpu
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("16-31,48-63\n")
    assert numa_cpus_of_gpu(0, 0x1b, 0, str(tmp_path)) == set(range(16, 32)) | set(range(48, 64))
    (dev / "numa_node").write_text("-1\n")
    assert numa_cpus_of_gpu(0, 0x1b, 0, str(tmp_path)) == set()
    assert numa_cpus_of_gpu(0, 0x3c, 0, str(tmp_path)) == set()
    assert _parse_cpulist("0,2-3") == {0, 2, 3}
