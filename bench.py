"""Benchmark of the hot path: MobileNetV2-int8 (random-init, synthetic images) images/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

One "step" = one pass of the whole network over one batch of B images per GPU.
Under torchrun (N > 1) every rank runs an independent replica on its own GPU on
its own B images (no data-path collective); the barrier and the max-over-ranks
time come from torch.distributed. Rank 0 prints one JSON line.

`value`   : device-resident throughput (inputs already in HBM), all ranks.
`e2e`     : the same metric through the host-pointer C-ABI call (tb200_invoke_host_async, one
            call per step, one wait at the end) from pinned host memory, every step's H2D and
            D2H inside the timed region.
`roofline`: the dominant kernel class timed live with CUDA events on the library's stream.
`cpu_baseline`: the CPU oracle (a port of the reference's host arithmetic) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "torq-compiler_b200"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

METRIC = "mobilenet_v2_int8_images_per_s"
UNIT = "images/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler(threading.Thread):
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self._halt = index, [], threading.Event()

    def run(self):
        while not self._halt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 7:
                    self.samples.append(parts)
            except Exception:
                pass
            self._halt.wait(0.1)

    def stop(self):
        self._halt.set()
        self.join(timeout=6)
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


def cpu_oracle_throughput(batch_sample: int, repeats: int):
    """Times the CPU oracle over a bounded sample of the same workload (images/s)."""
    from oracle import oracle as oc
    from oracle_exec import run_graph
    from torq_b200.workloads.mobilenet_v2 import build_mobilenet_v2, synthetic_images
    oc.set_num_threads(len(os.sched_getaffinity(0)))  # torchrun pins OMP_NUM_THREADS=1; use every host core
    g, _ = build_mobilenet_v2(batch_sample)
    x = synthetic_images(batch_sample)
    run_graph(g, [x])  # warm-up
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        run_graph(g, [x])
        times.append(time.perf_counter() - t0)
    return batch_sample / float(np.median(times)), oc.num_threads(), times


_DECODER_PARAMS = {}


def _decoder_params(cfg, tp, rank):
    """Random-init weights of the 1B shape (generated once per process: 1 GB of seeded integers)."""
    from torq_b200.workloads import gemma3
    if "full" not in _DECODER_PARAMS:
        # embedding gain 6.0: peaked logits, as a trained model has, so that greedy ids are a meaningful check
        # (with the nearly flat logits of plain random-init weights a single bf16 rounding flips the arg max)
        _DECODER_PARAMS["full"] = gemma3.random_weights(cfg, 1234, 6.0)
    if tp == 1:
        return _DECODER_PARAMS["full"]
    return gemma3.shard_weights(cfg, _DECODER_PARAMS["full"], tp, rank)


class _OpTimer:
    """Cold-cache timing of one executable: before every timed dispatch a buffer larger than L2 is
    overwritten on the same stream, and only the dispatch sits between the two events."""

    def __init__(self, dev, stream):
        import torch
        self.torch, self.dev, self.stream = torch, dev, stream
        with torch.cuda.stream(stream):
            self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def time_ms(self, ex, ins, outs, iters=10, warmup=3, cold=True):
        torch = self.torch
        for _ in range(warmup):
            ex.dispatch(ins, outs)
        self.dev.wait(120.0)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for e0, e1 in ev:
            if cold:
                with torch.cuda.stream(self.stream):
                    self.flush.zero_()
            e0.record(self.stream)
            ex.dispatch(ins, outs)
            e1.record(self.stream)
        self.dev.wait(120.0)
        torch.cuda.synchronize()
        return float(np.median([a.elapsed_time(b) for a, b in ev]))


def _run_single_op(timer, g, inputs, iters=10, cold=True):
    from torq_b200.runtime import Executable
    dev = timer.dev
    ex = Executable(dev, g.serialize())
    ins = [dev.alloc(a.nbytes) for a in inputs]
    for b, a in zip(ins, inputs):
        b.upload(a)
    outs = [dev.alloc(o.nbytes) for o in ex.outputs_info]
    dev.wait()
    ms = timer.time_ms(ex, ins, outs, iters=iters, cold=cold)
    # the same dispatch back to back (operands that fit stay in L2): total time of `iters` dispatches / iters
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(timer.stream)
    for _ in range(iters):
        ex.dispatch(ins, outs)
    e1.record(timer.stream)
    dev.wait(120.0)
    torch.cuda.synchronize()
    timer.last_warm_ms = e0.elapsed_time(e1) / iters
    kernels = [k for k in ex.op_kernels() if k != "view"]
    ex.destroy()
    for b in ins + outs:
        b.free()
    return ms, kernels


def ops_bench(dev, stream, peaks, i8_peak_tops):
    """The single-op configurations of the benchmark set, one line each: the single 3x3 convolution
    (batch 1 latency and batch 256 throughput), the M x K x N int8 FullyConnected sweep with both
    input zero points, max / average pooling and the 256-entry table, and MobileNetV2 at batch 1.
    Every entry states its algorithmic bytes and ops, the cold-cache CUDA-event time of one
    dispatch (`ms`: L2 flushed before it; the fractions use this one), the time per dispatch when the
    same dispatch runs back to back (`ms_warm_back_to_back`), and the fraction of the roofline that bounds it (tensor pipe for the contractions
    with M >= 64, HBM for the rest)."""
    from torq_b200.oplist import Graph
    from torq_b200.quant import quantize_multiplier, quantize_multipliers
    timer = _OpTimer(dev, stream)
    hbm = peaks["hbm_gbs"]
    rng = np.random.default_rng(1234)
    out = []

    def entry(name, ms, nbytes, ops, kernels, bound):
        e = {"name": name, "ms": round(ms, 5), "ms_warm_back_to_back": round(timer.last_warm_ms, 5), "algorithmic_bytes": int(nbytes), "ops": int(ops), "kernels": sorted(set(kernels)),
             "gbs": nbytes / (ms * 1e-3) / 1e9, "hbm_frac": nbytes / (ms * 1e-3) / 1e9 / hbm, "bound": bound}
        if ops:
            e["tops"] = ops / (ms * 1e-3) / 1e12
            e["tensor_frac"] = e["tops"] / i8_peak_tops if i8_peak_tops else None
        out.append(e)

    # ---- the single 3x3 convolution: 56x56x64 -> 64 filters, stride 1, SAME
    for batch in (1, 256):
        x = rng.integers(-128, 128, (batch, 56, 56, 64), dtype=np.int8)
        w = rng.integers(-127, 128, (64, 3, 3, 64), dtype=np.int8)
        m, s = quantize_multipliers(0.02 * rng.uniform(0.001, 0.01, 64) / 0.05)
        g = Graph()
        g.output(g.conv2d(g.input(x.shape), w, np.round(rng.normal(0, 2000, 64)).astype(np.int32), m, s, pad=(1, 1, 1, 1),
                          input_zp=-3, out_zp=5))
        ms, k = _run_single_op(timer, g, [x], iters=20)
        macs = batch * 56 * 56 * 64 * 9 * 64
        entry(f"conv3x3 {batch}x56x56x64->64", ms, 2 * x.nbytes + w.nbytes + 64 * 9, 2 * macs, k, "tensor" if batch > 1 else "latency")

    # ---- FullyConnected sweep: M in {1,64,512,4096}, K = N in {512,1024,4096,8192}, input zero point 0 / -7
    for kn in (512, 1024, 4096, 8192):
        w = rng.integers(-127, 128, (kn, kn), dtype=np.int8)
        m, s = quantize_multipliers(rng.uniform(0.5, 1.5, kn) * 40.0 / (np.sqrt(kn) * 74 * 74))
        bias = np.round(rng.normal(0, 1000, kn)).astype(np.int32)
        for M in (1, 64, 512, 4096):
            x = rng.integers(-128, 128, (M, kn), dtype=np.int8)
            for azp in (0, -7):
                g = Graph()
                g.output(g.fully_connected(g.input(x.shape), w, bias, m, s, input_zp=azp, out_zp=3))
                ms, k = _run_single_op(timer, g, [x], iters=6)
                entry(f"fc M={M} K=N={kn} azp={azp}", ms, M * kn + kn * kn + M * kn + kn * 9, 2 * M * kn * kn, k,
                      "tensor" if M >= 64 else "hbm")
        del w
    # ---- pooling on 64x112x112x64, 3x3 stride 2 (SAME: pad bottom/right), and the table on 64x56x56x256
    x = rng.integers(-128, 128, (64, 112, 112, 64), dtype=np.int8)
    for kind in ("max", "avg"):
        g = Graph()
        xi = g.input(x.shape)
        y = g.maxpool2d(xi, (3, 3), (2, 2), pad=(0, 1, 0, 1)) if kind == "max" else \
            g.avg_pool2d(xi, (3, 3), (2, 2), pad=(0, 1, 0, 1), input_zp=-3, output_zp=2)
        g.output(y)
        ms, k = _run_single_op(timer, g, [x])
        entry(f"{kind}pool 64x112x112x64 3x3 s2", ms, x.nbytes + x.nbytes // 4, 0, k, "hbm")
    x = rng.integers(-128, 128, (64, 56, 56, 256), dtype=np.int8)
    zp_in, s_in, s_out, zp_out = -4, 0.05, 1.0 / 256, -128
    tbl = np.clip(np.round(1.0 / (1.0 + np.exp(-s_in * (np.arange(-128, 128) - zp_in))) / s_out) + zp_out, -128, 127).astype(np.int8)
    g = Graph()
    g.output(g.table(g.input(x.shape), tbl))
    ms, k = _run_single_op(timer, g, [x])
    entry("table 64x56x56x256 (sigmoid)", ms, 2 * x.nbytes + 256, 0, k, "hbm")
    # rescaled add on the same shape (three exact rescales per element)
    from torq_b200.quant import add_rescale_params
    m0, m1, mo = add_rescale_params(0.04, 0.07, 0.09)
    g = Graph()
    a_in, b_in = g.input(x.shape), g.input(x.shape)
    g.output(g.add(a_in, b_in, a_zp=3, a_ms=m0, b_zp=-5, b_ms=m1, out_ms=mo, out_zp=1))
    x2 = rng.integers(-128, 128, x.shape, dtype=np.int8)
    ms, k = _run_single_op(timer, g, [x, x2])
    entry("add 64x56x56x256 (rescaled)", ms, 3 * x.nbytes, 0, k, "hbm")
    # ---- MobileNetV2 at batch 1: latency of one inference (graph replay, warm caches as in serving)
    from torq_b200.workloads.mobilenet_v2 import build_mobilenet_v2, synthetic_images
    g, layers = build_mobilenet_v2(1)
    ms, k = _run_single_op(timer, g, [synthetic_images(1)], iters=30, cold=False)
    macs = sum(l["macs"] for l in layers)
    nbytes = sum(l["in_bytes"] + l["out_bytes"] + l["weight_bytes"] for l in layers)
    entry("MobileNetV2 batch 1 (latency, warm)", ms, nbytes, 2 * macs, k, "latency")
    out[-1]["images_per_s"] = 1e3 / ms
    return out


def yolo_bench(dev, stream, batch: int = 64, steps: int = 5, parity: bool = False):
    """YOLOv8n-style int8 detector at 640x640 (the detector configuration of the benchmark set): images/s, inputs resident."""
    import torch
    from torq_b200.runtime import Executable
    from torq_b200.workloads.yolov8n import build_yolov8n, synthetic_images
    g, macs = build_yolov8n(batch, 640)
    ex = Executable(dev, g.serialize())
    x = synthetic_images(batch, 640)
    d_in = dev.alloc(x.nbytes)
    d_in.upload(x)
    outs = [dev.alloc(o.nbytes) for o in ex.outputs_info]
    for _ in range(3):
        ex.dispatch([d_in], outs)
    dev.wait(120.0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        ex.dispatch([d_in], outs)
    e1.record(stream)
    dev.wait(120.0)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    kernels = sorted(set(ex.op_kernels()))
    launches = ex.launch_count
    ex.destroy()
    for b in [d_in] + outs:
        b.free()
    result = {"workload": f"YOLOv8n-style int8 detector 640x640, batch {batch}", "images_per_s": batch / (ms * 1e-3),
              "ms_per_step": ms, "gmac_per_image": macs / 1e9, "launches_per_step": launches, "kernels": kernels}
    if parity:
        # one image through the same network on the GPU and on the CPU oracle (outside the timed region): bit-exact
        # or not, and what the oracle's pass took (the CPU figure beside the GPU one)
        from oracle import oracle as oc
        from oracle_exec import run_graph
        oc.set_num_threads(len(os.sched_getaffinity(0)))
        g1, _ = build_yolov8n(1, 640)
        x1 = synthetic_images(1, 640)
        ex1 = Executable(dev, g1.serialize())
        b_in = dev.alloc(x1.nbytes)
        b_in.upload(x1)
        b_out = [dev.alloc(o.nbytes) for o in ex1.outputs_info]
        ex1.dispatch([b_in], b_out)
        dev.wait(120.0)
        got = [b.download(o.shape, o.np_dtype) for b, o in zip(b_out, ex1.outputs_info)]
        t0 = time.perf_counter()
        want = run_graph(g1, [x1])
        cpu_s = time.perf_counter() - t0
        result["parity"] = {"batch": 1, "bit_exact": bool(all((a == b).all() for a, b in zip(got, want))),
                            "outputs": len(want), "checker": "CPU oracle (port of the reference's host arithmetic)"}
        result["cpu_baseline"] = {"value": 1.0 / cpu_s, "unit": "images/s", "cores": oc.num_threads(), "kind": "port",
                                  "sample": "one 640x640 image, one pass"}
        ex1.destroy()
        for b in [b_in] + b_out:
            b.free()
    return result


def decoder_bench(dev, stream, batch: int, prompt_len: int = 1024, gen_len: int = 128, tp: int = 1, rank: int = 0):
    """Gemma-3-1B-architecture int8-weight greedy decode (second metric of the benchmark set):
    tokens/s over `gen_len` decode steps after a `prompt_len`-token seeded prompt. One GPU, or
    (tp > 1, every rank of the process group calls this) tensor-parallel over tp GPUs: each rank
    runs its shard, the shards exchange partial results through peer memory inside the step kernel.
    Every step is one dispatch; the next token and position move on the device."""
    import torch
    from torq_b200.runtime import MEMORY_HOST_PINNED, Executable
    from torq_b200.workloads import gemma3
    cfg = gemma3.GemmaConfig()
    params = _decoder_params(cfg, tp, rank)
    g = gemma3.build_decode_step(cfg, batch, params, tp=tp, rank=rank)
    ex = Executable(dev, g.serialize())
    del params, g
    if tp > 1:
        ex.connect_group()
    rng = np.random.default_rng(1234)
    prompt = rng.integers(0, cfg.vocab, (prompt_len, batch)).astype(np.int32)
    steps = prompt_len + gen_len
    h_tok = dev.alloc(prompt.nbytes, MEMORY_HOST_PINNED)
    h_tok.as_numpy(prompt.shape, np.int32)[...] = prompt
    h_pos = dev.alloc(steps * 4, MEMORY_HOST_PINNED)
    h_pos.as_numpy((steps,), np.int32)[...] = np.arange(steps, dtype=np.int32)
    d_tok, d_pos, d_next = dev.alloc(batch * 4), dev.alloc(4), dev.alloc(batch * 4)
    lib = dev._lib
    import ctypes as C

    h_ids = dev.alloc(gen_len * batch * 4, MEMORY_HOST_PINNED)  # every generated id comes back to the host
    h_ids.as_numpy((gen_len, batch), np.int32)[...] = -1

    def step(pos, from_prompt):
        src = h_tok.pointer + pos * batch * 4 if from_prompt else d_next.pointer
        dev._check(lib.tb200_buffer_upload(d_tok._h, 0, C.c_void_p(src), batch * 4))
        dev._check(lib.tb200_buffer_upload(d_pos._h, 0, C.c_void_p(h_pos.pointer + pos * 4), 4))
        ex.dispatch([d_tok, d_pos], [d_next])
        if not from_prompt:  # stream-ordered device-to-host read of the step's result
            dev._check(lib.tb200_buffer_download(d_next._h, 0, C.c_void_p(h_ids.pointer + (pos - prompt_len) * batch * 4), batch * 4))

    for pos in range(prompt_len):
        step(pos, True)
    dev.wait(300.0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for pos in range(prompt_len, steps):
        step(pos, False)
    e1.record(stream)
    dev.wait(300.0)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if tp > 1:  # the slowest rank's time counts
        import torch.distributed as dist
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    last = d_next.download((batch,), np.int32)
    ids = h_ids.as_numpy((gen_len, batch), np.int32).copy()
    import hashlib
    ids_sha = hashlib.sha256(ids.tobytes()).hexdigest()[:16]
    h_ids.free()
    wbytes = gemma3.weight_bytes_per_token(cfg)
    kv_bytes = sum(2 * min(steps, cfg.max_seq if cfg.is_global(l) else cfg.window) * cfg.head_dim * 2 for l in range(cfg.layers)) * batch
    launches = ex.launch_count
    ex.destroy()
    for b in (h_tok, h_pos, d_tok, d_pos, d_next):
        b.free()
    step_ms = ms / gen_len
    return {"batch": batch, "tp": tp, "tok_per_s": batch * gen_len / (ms * 1e-3), "ms_per_step": step_ms,
            "weight_bytes_per_step": wbytes, "kv_bytes_per_step": kv_bytes,
            "hbm_gbs": (wbytes + kv_bytes) / (step_ms * 1e-3) / 1e9, "launches_per_step": launches,
            "last_tokens": [int(t) for t in last[:4]], "ids_sha": ids_sha, "distinct_ids": int(len(np.unique(ids))),
            "d2h_bytes_per_step": batch * 4, "h2d_bytes_per_step": 0}


def decoder_parity(dev, batch: int, steps: int = 12, tp: int = 1, rank: int = 0):
    """Outside any timed region: the same weights, `steps` teacher-forced seeded tokens, logits of every
    step against the fp32 torch reference of the unsharded model (tests/ref_decoder.py): relative max-abs
    error of the logits and whether every greedy id agrees. With tp > 1 every rank calls this; the logits
    shards are gathered to rank 0, which alone holds the reference and returns the outcome."""
    import torch
    from torq_b200.runtime import Executable
    from torq_b200.workloads import gemma3
    cfg = gemma3.GemmaConfig()
    params = _decoder_params(cfg, tp, rank)
    ex = Executable(dev, gemma3.build_decode_step(cfg, batch, params, with_logits=True, tp=tp, rank=rank).serialize())
    if tp > 1:
        ex.connect_group()
    vl = cfg.vocab // tp
    d_tok, d_pos, d_next, d_logits = dev.alloc(batch * 4), dev.alloc(4), dev.alloc(batch * 4), dev.alloc(batch * vl * 4)
    ref = None
    if rank == 0:
        from ref_decoder import RefDecoder
        ref = RefDecoder(cfg, _decoder_params(cfg, 1, 0), batch)
    toks = np.random.default_rng(99).integers(0, cfg.vocab, (steps, batch)).astype(np.int32)
    worst, agree = 0.0, True
    for pos in range(steps):
        d_tok.upload(toks[pos])
        d_pos.upload(np.array([pos], np.int32))
        ex.dispatch([d_tok, d_pos], [d_next, d_logits])
        dev.wait(60.0)
        nxt = d_next.download((batch,), np.int32)
        logits = d_logits.download((batch, vl), np.float32)
        if tp > 1:
            import torch.distributed as dist
            mine = torch.from_numpy(logits).cuda()
            parts = [torch.empty_like(mine) for _ in range(tp)] if rank == 0 else None
            dist.gather(mine, parts, dst=0)
            if rank == 0:
                logits = torch.cat(parts, -1).cpu().numpy()
        if rank == 0:
            r_next, r_logits = ref.step(toks[pos], pos)
            worst = max(worst, float(np.abs(logits - r_logits).max() / np.abs(r_logits).max()))
            agree = agree and bool((nxt == r_next).all())
    ex.destroy()
    for b in (d_tok, d_pos, d_next, d_logits):
        b.free()
    del ref
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    return {"steps": steps, "batch": batch, "rel_max_abs": worst, "tolerance": 1e-2, "ids_match_reference": agree,
            "reference": "fp32 torch model of the same int8 weights, teacher-forced seeded tokens"}


def run_reference(args, rank, world):
    """--impl reference: the reference's host arithmetic (CPU oracle port; IREE's llvm-cpu
    path cannot be built here) on all host threads, same metric and config."""
    if rank != 0:
        return
    sample = min(args.batch, 32)
    per_step = []
    from oracle import oracle as oc
    from oracle_exec import run_graph
    from torq_b200.workloads.mobilenet_v2 import build_mobilenet_v2, synthetic_images
    oc.set_num_threads(len(os.sched_getaffinity(0)))  # torchrun pins OMP_NUM_THREADS=1; use every host core
    g, _ = build_mobilenet_v2(sample)
    x = synthetic_images(sample)
    for _ in range(args.warmup):
        run_graph(g, [x])
    for _ in range(args.steps):
        t0 = time.perf_counter()
        run_graph(g, [x])
        per_step.append(time.perf_counter() - t0)
    total = sum(per_step)
    value = sample * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": {"workload": f"MobileNetV2-1.0 int8 224x224, batch {args.batch} per GPU", "sample_images_per_step": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oc.num_threads(), "kind": "port",
                         "sample": f"{sample} images per step x {args.steps} steps (of the batch-{args.batch} workload)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=256, help="images per GPU per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layer-table", default=None, help="write per-layer kernel, ms and GB/s to this CSV")
    ap.add_argument("--decoder", default="1,32", help="comma list of decode batch sizes for the Gemma-3-1B-shape "
                    "second metric (rank 0 on one GPU; with several ranks also tensor-parallel, batches <= 8); "
                    "empty string skips it")
    ap.add_argument("--no-yolo", action="store_true", help="skip the YOLOv8n-style detector timing")
    ap.add_argument("--no-ops", action="store_true", help="skip the single-op configurations (conv, FC sweep, pools, table)")
    ap.add_argument("--decode-prompt", type=int, default=1024, help="prompt length of the decode metric")
    ap.add_argument("--decode-gen", type=int, default=128, help="generated tokens of the decode metric")
    ap.add_argument("--only", choices=["all", "cnn", "decoder", "yolo"], default="all",
                    help="profiling aid: 'cnn' runs just the timed MobileNetV2 steps, 'decoder' just the decode metric "
                         "(one GPU), 'yolo' just the detector timing; the JSON line then carries only that part")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from torq_b200.runtime import MEMORY_HOST_PINNED, Device, Executable
    from torq_b200.workloads.mobilenet_v2 import build_mobilenet_v2, synthetic_images

    torch.cuda.set_device(local_rank)
    numa_cpus = []
    if world > 1:
        # each rank next to its GPU: the pinned staging buffers allocated below are then node-local
        from torq_b200.replicas import pin_rank_to_gpu_numa_node
        numa_cpus = pin_rank_to_gpu_numa_node(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()

    B = args.batch
    dev = Device(local_rank)
    if args.only == "yolo":
        stream = torch.cuda.ExternalStream(dev.stream, device=torch.device("cuda", local_rank))
        print(json.dumps({"only": "yolo", **yolo_bench(dev, stream, steps=args.steps)}), flush=True)
        return
    if args.only == "decoder":
        stream = torch.cuda.ExternalStream(dev.stream, device=torch.device("cuda", local_rank))
        runs = [decoder_bench(dev, stream, int(t), args.decode_prompt, args.decode_gen) for t in args.decoder.split(",") if t]
        print(json.dumps({"metric": "gemma3_1b_w8_decode_tok_per_s", "unit": "tokens/s", "only": "decoder", "runs": runs}), flush=True)
        return
    g, layers = build_mobilenet_v2(B)
    ex = Executable(dev, g.serialize())
    in_info, out_info = ex.inputs_info[0], ex.outputs_info[0]

    # 4 distinct resident input batches (4 x 38.5 MB > 126 MB L2) rotated between steps;
    # the 3.4 GB of activations one step streams exceed L2 many times over anyway.
    n_rot = 4
    ins = [dev.alloc(in_info.nbytes) for _ in range(n_rot)]
    out = dev.alloc(out_info.nbytes)
    host_in = [dev.alloc(in_info.nbytes, MEMORY_HOST_PINNED) for _ in range(n_rot)]
    host_out = dev.alloc(out_info.nbytes, MEMORY_HOST_PINNED)
    for i in range(n_rot):
        img = synthetic_images(B, seed=1234 + 17 * i + 1000 * rank)
        host_in[i].as_numpy(in_info.shape, np.int8)[...] = img
        ins[i].upload(host_in[i].as_numpy(in_info.shape, np.int8))
    dev.wait()

    stream = torch.cuda.ExternalStream(dev.stream, device=torch.device("cuda", local_rank))

    def timed(step_fn, steps, warmup):
        for i in range(warmup):
            step_fn(i)
        dev.wait()
        torch.cuda.synchronize()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            step_fn(i)
        e1.record(stream)
        dev.wait()
        torch.cuda.synchronize()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()

    # ---- device-resident throughput ----
    ms_total = timed(lambda i: ex.dispatch([ins[i % n_rot]], [out]), args.steps, args.warmup)
    value = B * world * args.steps / (ms_total * 1e-3)

    if args.only == "cnn":
        if sampler:
            sampler.stop()
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "only": "cnn", "steps": args.steps,
                              "ms_per_step": ms_total / args.steps, "gpu_launches": ex.launch_count * args.steps}), flush=True)
        barrier()
        if world > 1:
            dist.destroy_process_group()
        return
    # ---- end to end through the host-pointer call (pinned host memory) ----
    hin = [h.as_numpy(in_info.shape, np.int8) for h in host_in]
    hout = host_out.as_numpy(out_info.shape, np.int8)
    e2e_steps = max(3, args.steps)
    # pipelined host call: upload of step i+1 overlaps the kernels of step i; every step's H2D and
    # D2H copies are inside the timed region (dev.wait() closes it)
    ms_e2e = timed(lambda i: ex.invoke_host_async([hin[i % n_rot]], [hout]), e2e_steps, 3)
    e2e_value = B * world * e2e_steps / (ms_e2e * 1e-3)
    clocks = sampler.stop() if sampler else None

    # ---- tensor-parallel decode over all ranks ----
    decoder_tp = None
    if world in (2, 4, 8) and args.decoder:
        decoder_tp = []
        # the tensor-parallel step kernel takes up to 8 sequences: larger requests are measured at 8
        tp_batches = sorted({min(int(t), 8) for t in args.decoder.split(",") if t})
        for bsz in tp_batches:
            try:
                r = decoder_bench(dev, stream, bsz, args.decode_prompt, args.decode_gen, tp=world, rank=rank)
                r["parity"] = decoder_parity(dev, bsz, tp=world, rank=rank)
                decoder_tp.append(r)
            except Exception as e:
                decoder_tp.append({"batch": bsz, "tp": world, "error": repr(e)[:200]})
                break

    if rank != 0:
        barrier()
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel class (live CUDA-event timing per op) ----
    cnn_launches = ex.launch_count
    op_ms = ex.profile_ops([ins[0]], [out], warmup=2, iters=5)
    kernels = ex.op_kernels()
    real_layers = [l for l in layers]
    # ops and layer table line up except for the reshape view
    per_kernel = {}
    li = 0
    table = ["layer,kernel,ms,algorithmic_MB,GBps,GMACps"]
    for k, ms in zip(kernels, op_ms):
        if k == "view":
            continue
        layer = real_layers[li]
        li += 1
        alg_bytes = (layer["in_bytes"] + layer["out_bytes"]) * B + layer["weight_bytes"]
        table.append(f"{layer['name']},{k},{ms:.4f},{alg_bytes / 1e6:.2f},{alg_bytes / (ms * 1e-3) / 1e9:.0f},"
                     f"{layer['macs'] * B / (ms * 1e-3) / 1e9:.0f}")
        d = per_kernel.setdefault(k, {"ms": 0.0, "bytes": 0, "macs": 0, "launches": 0})
        d["ms"] += float(ms)
        d["bytes"] += alg_bytes
        d["macs"] += layer["macs"] * B
        d["launches"] += 1
    if args.layer_table:
        with open(args.layer_table, "w") as f:
            f.write("\n".join(table) + "\n")
    dom = max(per_kernel, key=lambda k: per_kernel[k]["ms"])
    peaks, peak_kind = measured_peaks()
    d = per_kernel[dom]
    # Per-op times come from a run that brackets every op with events, which adds a gap per op; the graph
    # replay of the timed region has none. Both are stated: `achieved` uses the per-op time of the class
    # (conservative), `achieved_in_step` scales it by (timed step / sum of per-op times).
    step_ms = ms_total / args.steps
    op_sum_ms = sum(v["ms"] for v in per_kernel.values())
    in_step = step_ms / op_sum_ms if op_sum_ms > 0 else 1.0
    achieved = d["bytes"] / (d["ms"] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                "traffic_source": "not measured by this run (DRAM bytes need the profiler; the committed ncu launch list of this workload gives them)",
                "peak_source": f"of {peak_kind}", "launches_per_step": d["launches"], "avg_launch_ms": d["ms"] / d["launches"],
                "algorithmic_bytes_per_launch": d["bytes"] / d["launches"],
                "achieved_in_step": achieved / in_step, "frac_in_step": achieved / in_step / peaks["hbm_gbs"],
                "sum_of_per_op_ms": op_sum_ms, "timed_step_ms": step_ms,
                "per_kernel_ms": {k: round(v["ms"], 4) for k, v in per_kernel.items()},
                "whole_step": {"algorithmic_bytes": sum(v["bytes"] for v in per_kernel.values()),
                               "gbs": sum(v["bytes"] for v in per_kernel.values()) / (step_ms * 1e-3) / 1e9,
                               "hbm_frac": sum(v["bytes"] for v in per_kernel.values()) / (step_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}}
    # int8 tensor-pipe ceiling measured now, on this GPU: resident-operand tcgen05.mma kind::i8 loop on every SM
    i8_peak = None
    try:
        from torq_b200.runtime import measure_i8_mma_peak
        burst, burst_ms = measure_i8_mma_peak(local_rank, 1000)
        sustained, sustained_ms = measure_i8_mma_peak(local_rank, 6000)
        i8_peak = {"burst_tops": burst, "burst_ms": burst_ms, "sustained_tops": sustained, "sustained_ms": sustained_ms,
                   "nominal_dense_tops": 4500.0, "how": "tcgen05.mma kind::i8 M128 N256 K32 back to back, operands in shared memory, "
                   "accumulators in TMEM, all SMs, no memory traffic"}
    except Exception as e:
        i8_peak = {"error": repr(e)[:200]}
    roofline_tensor = None
    contraction = [k for k in per_kernel if "tcgen05" in k]
    if contraction and i8_peak and "sustained_tops" in i8_peak:
        macs = sum(per_kernel[k]["macs"] for k in contraction)
        t_ms = sum(per_kernel[k]["ms"] for k in contraction)
        tops = 2.0 * macs / (t_ms * 1e-3) / 1e12
        roofline_tensor = {"kernels": contraction, "achieved_tops": tops, "peak_tops": i8_peak["sustained_tops"],
                           "frac": tops / i8_peak["sustained_tops"], "frac_of_nominal": tops / 4500.0,
                           "peak_source": "measured in this run (sustained loop; these kernels run inside a long step)",
                           "note": "1x1 convolutions with K = 16..960: arithmetic intensity 2*K*N/(K+N) op/B is below the "
                                   "int8 ridge, so HBM and the epilogue bound them, not the tensor pipe"}

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:  # with several ranks the host cores are shared: no meaningful number
        v, cores, times = cpu_oracle_throughput(16, 5)
        cpu_baseline = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"16 images x 5 passes of the same network (median {np.median(times):.3f} s per pass)"}

    decoder = None
    if args.decoder:
        decoder = {"metric": "gemma3_1b_w8_decode_tok_per_s", "unit": "tokens/s", "dtype": "bf16 activations, int8 weights",
                   "workload": "Gemma-3-1B architecture, random-init (embedding gain 6.0: peaked logits), 1024-token seeded prompt + 128 greedy tokens",
                   "hbm_peak_gbs": peaks["hbm_gbs"], "runs": []}
        ex.destroy()  # free the CNN arena first
        one_gpu_batches = [int(t) for t in args.decoder.split(",") if t]
        if decoder_tp:  # one GPU's ids for every batch the tensor-parallel runs used
            one_gpu_batches += [r["batch"] for r in decoder_tp if r.get("batch") not in one_gpu_batches]
        for bsz in one_gpu_batches:
            try:
                r = decoder_bench(dev, stream, bsz, args.decode_prompt, args.decode_gen)
                r["hbm_frac"] = r["hbm_gbs"] / peaks["hbm_gbs"]
                r["parity"] = decoder_parity(dev, bsz)
                decoder["runs"].append(r)
            except Exception as e:  # the headline line must still print
                decoder["runs"].append({"batch": bsz, "error": repr(e)[:200]})
        if decoder_tp:
            for r in decoder_tp:
                if "hbm_gbs" in r:  # per-GPU share of the bytes against one GPU's bandwidth
                    r["hbm_frac_per_gpu"] = r["hbm_gbs"] / r["tp"] / peaks["hbm_gbs"]
                # the tensor-parallel group must generate the very ids one GPU generates for the same prompt
                one = [q for q in decoder["runs"] if q.get("batch") == r.get("batch") and "ids_sha" in q]
                if one and "ids_sha" in r:
                    r["ids_equal_tp1"] = one[0]["ids_sha"] == r["ids_sha"]
            decoder["tensor_parallel_runs"] = decoder_tp

    ops = None
    if not args.no_ops and world == 1:
        try:
            ops = ops_bench(dev, stream, peaks, (i8_peak or {}).get("burst_tops"))
        except Exception as e:
            ops = {"error": repr(e)[:300]}

    yolo = None
    if not args.no_yolo:
        try:
            yolo = yolo_bench(dev, stream, parity=(world == 1 and not args.no_cpu_baseline))
        except Exception as e:
            yolo = {"error": repr(e)[:200]}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "i8", "data": "synthetic",
        "config": {"workload": f"MobileNetV2-1.0 int8 224x224, batch {B} per GPU", "global_batch": B * world,
                   "parallelism": f"replicas x{world} (batch split, no collective)",
                   "rank0_cpu_affinity": (f"{len(numa_cpus)} CPUs of the GPU's NUMA node" if numa_cpus else "unchanged"),
                   "l2": f"inputs rotate over {n_rot} resident batches ({n_rot * in_info.nbytes / 1e6:.0f} MB > L2); "
                         "activations per step exceed L2"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": in_info.nbytes, "d2h_bytes_per_step": out_info.nbytes,
                "steps": e2e_steps, "ms_per_step": ms_e2e / e2e_steps},
        "gpu_launches": cnn_launches * args.steps,
        "clocks": clocks, "roofline": roofline, "roofline_tensor": roofline_tensor, "i8_tensor_peak": i8_peak,
        "cpu_baseline": cpu_baseline, "ops": ops, "decoder": decoder, "yolo": yolo,
    }
    print(json.dumps(line), flush=True)
    barrier()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
