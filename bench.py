"""Benchmark of the BF16 lossless codec hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): BASELINE configuration 2 - an 8192 x 8192 BF16 weight-like tensor, i.i.d.
Laplace(0, 0.02) from a fixed seed with 1e-4 of the entries multiplied by 100,
``Distribution(LAPLACE, param=0.02)``, CLEAN layout, overflow tails in a shared ``TensorBuffer``.
One step = one ``compress`` + one ``decompress`` of such a tensor.  With N > 1 every rank runs
the same step on its own tensors (independent tensors partitioned across GPUs: weak scaling, no
data-path collective), and the value is the aggregate over ranks against the slowest rank's time.

Reported value: GB/s of BF16 data through the codec = (2N bytes encoded + 2N bytes decoded) /
(encode time + decode time), device time from CUDA events with the inputs already in HBM and the
L2 flushed (512 MiB written) before each timed phase.  Cycling three tensors instead of flushing
(inputs larger than L2) was measured too: the kernels take the same time and the event spans
then expose the host's launch latency, so the flush stayed.  ``e2e`` is the same figure
through the public API with host buffers: pinned-host -> device copy of the input, compress,
decompress, device -> pinned-host copy of the decoded tensor, all inside the timed region;
``e2e_copies_only`` is the same loop with the copies alone.

``triton_reference`` (N = 1, when a copy of the reference checkout is present) times the
reference's own Triton kernels, compiled for this GPU, on the same tensors in a process of its
own: the bar the kernels here are measured against.

``--impl reference`` times the CPU implementation of the same path: the C restatement of the
reference's kernels (the oracle), on all host threads, on the same tensor.  The reference itself
is a Python/Triton project with no CPU build; its interpreter mode needs minutes per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _path in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    if _path not in sys.path:
        sys.path.insert(0, _path)

import numpy as np  # noqa: E402
import torch  # noqa: E402

ROWS = COLS = 8192
METRIC = "codec_bf16_gbps_per_gpu"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
L2_FLUSH_BYTES = 512 << 20
WORKLOAD = ("config2: 8192x8192 BF16 Laplace(0,0.02)+1e-4 outliers x100, LAPLACE/CLEAN, "
            "shared arena; step = compress + decompress")
L2_NOTE = f"flushed ({L2_FLUSH_BYTES >> 20} MiB write) before each timed phase"


def bench_config(world: int) -> dict:
    """The ``config`` object of the JSON line, the same for both arms."""
    return {"workload": WORKLOAD, "l2": L2_NOTE,
            "parallelism": f"{world} independent tensor(s) per step, one per GPU"}


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of one ncu capture of the
# two kernels on this workload.  Reads equal the algorithmic reads; part of the written bytes is
# still in the 126 MB write-back L2 when the kernel ends, so the sum is below the algorithmic
# 227.6 MB.
NCU_TRAFFIC_BYTES = {"lct_encode": 184_880_896, "lct_decode": 169_537_792}


class LaunchTrace:
    """Counts the library's launches while active and, for the entry points named in ``timed``,
    brackets each launch with CUDA events on the launching stream (the roofline's durations)."""

    def __init__(self, timed=()):
        self.timed = set(timed)
        self.count = 0
        self.events: dict[str, list] = {name: [] for name in self.timed}

    def __enter__(self):
        from losslessly_compressed_tensors_b200.kernels import dispatch

        self._dispatch, self._call = dispatch, dispatch._call

        def traced(name, device, *args, launches=1):
            self.count += launches
            if name not in self.timed:
                return self._call(name, device, *args, launches=launches)
            stream = torch.cuda.current_stream(device)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            self._call(name, device, *args, launches=launches)
            end.record(stream)
            self.events[name].append((start, end))

        dispatch._call = traced
        return self

    def __exit__(self, *exc):
        self._dispatch._call = self._call

    def milliseconds(self, name: str) -> list[float]:
        """Durations of the timed launches of ``name`` (call after synchronising)."""
        return [start.elapsed_time(end) for start, end in self.events[name]]


def make_workload(seed: int) -> torch.Tensor:
    """Configuration-2 tensor, generated on the CPU so every machine sees the same bits."""
    n = ROWS * COLS
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(n, generator=g) - 0.5
    values = -0.02 * torch.sign(u) * torch.log1p(-2.0 * u.abs())
    del u
    outliers = torch.rand(n, generator=g) < 1e-4
    values[outliers] *= 100.0
    return values.to(torch.bfloat16).reshape(ROWS, COLS)


def peak_hbm_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.process = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def finish(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        out, _ = self.process.communicate(timeout=10)
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None,
                "samples": len(clocks), "reasons": sorted(reasons)}


def distributed_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        import datetime

        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=180))
    elif n_gpus > 1:
        raise SystemExit("launch N > 1 with torch.distributed.run (one process per GPU)")
    else:
        torch.cuda.set_device(0)
    return rank, world, local


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def cpu_leg(bits: np.ndarray, threads: int, budget_s: float, max_steps: int):
    """Time the CPU restatement on the whole workload; returns (GB/s, steps, threads used)."""
    from helpers import oracle_compress
    from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType
    from oracle import lct_oracle as oracle

    oracle.build()
    used = oracle.set_threads(threads)
    dist = Distribution(DistType.LAPLACE, param=0.02)
    arena = oracle.new_arena(64 << 20)
    elapsed, steps = 0.0, 0
    while steps < max_steps and (steps == 0 or elapsed < budget_s):
        t0 = time.perf_counter()
        c = oracle_compress(oracle, bits, dist, arena)
        y = oracle.decompress(c)
        elapsed += time.perf_counter() - t0
        oracle.buf_free(arena, c["descriptor"])
        steps += 1
    assert np.array_equal(y, bits)
    return 2 * bits.nbytes * steps / elapsed / 1e9, steps, used, elapsed / steps * 1e3


def run_reference(args, rank: int):
    """CPU arm: rank 0 alone works; one JSON line."""
    if rank != 0:
        return
    bits = make_workload(1).view(torch.int16).numpy().reshape(-1)
    cores = os.cpu_count() or 1
    for _ in range(args.warmup):
        cpu_leg(bits, cores, 0.0, 1)
    value, steps, used, ms = cpu_leg(bits, cores, 1e9, args.steps)
    sample = f"full workload ({ROWS}x{COLS} BF16), {steps} step(s) of compress+decompress"
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": bench_config(args.gpus), "where": "host cores, one rank",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": used, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


def triton_reference_leg(timeout_s: int = 420) -> dict:
    """The reference's own kernels, compiled by Triton for this GPU, timed on configurations 2
    and 4 in a process of its own (``tests/reference_runner.py``; CUDA events, L2 flushed before
    every timed call, the reference's single-configuration launch lists)."""
    import reference_runner

    if not reference_runner.available():
        return {"unavailable": "no copy of the reference checkout under baseline/_ref"}
    with tempfile.TemporaryDirectory() as scratch:
        out = os.path.join(scratch, "reference.json")
        command = [sys.executable, os.path.join(ROOT, "tests", "reference_runner.py"), "bench",
                   "--out", out, "--iters", "20"]
        try:
            done = subprocess.run(command, capture_output=True, text=True, timeout=timeout_s)
        except subprocess.TimeoutExpired:
            return {"unavailable": f"the reference did not finish within {timeout_s} s"}
        if done.returncode != 0 or not os.path.exists(out):
            return {"unavailable": "the reference failed: " + done.stderr.strip()[-300:]}
        with open(out) as handle:
            result = json.load(handle)
    result["note"] = ("reference kernels (Triton, compiled without Triton's warp-specialisation "
                      "pass, which aborts on its decoder for sm_100); L2 flushed before every call")
    return result


def sharded_leg(rank: int, world: int, steps: int = 5, warmup: int = 2, with_peer: bool = False) -> dict:
    """BASELINE configuration 5: a GPT-2-small-shaped BF16 weight set (148 tensors, 124 475 904
    parameters, N(0, 0.02), LayerNorm weights 1, biases 0), EMPIRICAL codebook, row-shards of at
    most 4 Mi elements spread over the ranks; every rank encodes its shards into its wire
    buffer, ONE all-gather moves the compressed bytes, every rank decodes the whole set."""
    from losslessly_compressed_tensors_b200 import sharded
    from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType

    shapes = sharded.gpt2_small_shapes()
    g = torch.Generator().manual_seed(3)
    tensors = []
    for name, shape in shapes:
        if name.endswith("bias"):
            w = torch.zeros(shape)
        elif "ln_" in name:
            w = torch.ones(shape)
        else:
            w = torch.randn(shape, generator=g) * 0.02
        tensors.append(w.to(torch.bfloat16).cuda())
    dist_cfg = Distribution(DistType.EMPIRICAL)
    plan = sharded.make_plan(shapes, world, dist_cfg, row_shard_elements=4 << 20)
    dense_bytes = 2 * sum(t.numel() for t in tensors)
    wire = torch.zeros(plan.wire_bytes, dtype=torch.uint8, device="cuda")
    times = {"encode": [], "gather": [], "decode": [], "serial": []}
    gathered = torch.empty(world * plan.wire_bytes, dtype=torch.uint8, device="cuda")
    restored = [torch.empty(s, dtype=torch.bfloat16, device="cuda") for _, s in shapes]
    # (1) the three phases one after the other: encode, ONE all-gather, decode everything
    for it in range(warmup + steps):
        barrier(world)
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        e[0].record()
        sharded.encode_rank(plan, rank, tensors, wire=wire)
        e[1].record()
        sharded.all_gather_wire(wire, plan, out=gathered)
        e[2].record()
        sharded.decode_all(plan, gathered, [s for _, s in shapes], outputs=restored)
        e[3].record()
        torch.cuda.synchronize()
        if it >= warmup:
            for key, a, b in (("encode", 0, 1), ("gather", 1, 2), ("decode", 2, 3), ("serial", 0, 3)):
                times[key].append(e[a].elapsed_time(e[b]))
    exact = all(torch.equal(a.view(torch.int16), b.view(torch.int16)) for a, b in zip(tensors, restored))
    ms = {k: max_over_ranks(statistics.mean(v), world) for k, v in times.items()}
    # (2) the overlapped step: encode (one CUDA graph), one fence, then source-by-source copies
    #     out of the peers' memory on a side stream while the main stream decodes what has landed
    overlapped = {}
    try:
        for t in restored:
            t.zero_()
        exchange = sharded.WeightSetExchange(plan, rank, tensors, [s for _, s in shapes],
                                             outputs=restored)
        spans, encode_spans = [], []
        overlap_warmup, overlap_steps = max(warmup, 5), max(2 * steps, 30)
        for it in range(overlap_warmup + overlap_steps):
            barrier(world)
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            exchange.encode()
            e[1].record()
            exchange.exchange_and_decode()
            e[2].record()
            torch.cuda.synchronize()
            if it >= overlap_warmup:
                spans.append(e[0].elapsed_time(e[2]))
                encode_spans.append(e[0].elapsed_time(e[1]))
        # Every step is timed on its own (events on the launching stream, a barrier in front);
        # the figure is the median step of the slowest rank - one late peer in one of thirty
        # sub-millisecond steps would otherwise decide it - with the mean beside it.
        overlapped = {
            "step_ms": max_over_ranks(statistics.median(spans), world),
            "step_ms_mean": max_over_ranks(statistics.mean(spans), world),
            "step_ms_max": max_over_ranks(max(spans), world),
            "steps": overlap_steps,
            "encode_ms": max_over_ranks(statistics.median(encode_spans), world),
            "bit_exact": bool(all(torch.equal(a.view(torch.int16), b.view(torch.int16))
                                  for a, b in zip(tensors, restored))),
            "multicast_bound": bool(exchange.wires[0].multicast),
        }
        del exchange
    except Exception as error:   # symmetric memory not available on this box / build
        overlapped = {"unavailable": f"{type(error).__name__}: {error}"[:200]}
    peer = (peer_decode_leg(plan, rank, world, tensors, shapes, steps, warmup)
            if world > 1 and with_peer else None)
    step_ms = overlapped.get("step_ms", ms["serial"])
    return {
        "workload": "config5: GPT-2-small-shaped weight set, 148 tensors, EMPIRICAL/CLEAN, "
                    "row-shards <= 4 Mi elements; step = encode own shards + exchange + decode all",
        "shards": sum(len(r) for r in plan.shards), "dense_bytes": dense_bytes,
        "wire_bytes_per_rank": plan.wire_bytes, "bit_exact": bool(exact),
        "encode_ms": ms["encode"], "all_gather_ms": ms["gather"], "decode_all_ms": ms["decode"],
        "serial_step_ms": ms["serial"],
        "encode_gbps_aggregate": dense_bytes / ms["encode"] / 1e6,
        "all_gather_gbps": world * plan.wire_bytes / ms["gather"] / 1e6,
        "decode_gbps_aggregate": world * dense_bytes / ms["decode"] / 1e6,
        "peer_decode": peer, "overlapped": overlapped,
        "step_ms": step_ms, "step_gbps_aggregate": world * dense_bytes / step_ms / 1e6,
    }


def peer_decode_leg(plan, rank, world, tensors, shapes, steps, warmup) -> dict:
    """The same weight set without the collective: wire buffers in symmetric memory, every rank
    decodes all shards by loading the other ranks' bytes straight over NVLink inside the decode
    launch (jobs interleaved over the sources, each rank starting at its right neighbour)."""
    from losslessly_compressed_tensors_b200 import sharded

    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    try:
        peer = sharded.PeerWire(plan, rank)
    except Exception as error:  # symmetric memory not available on this box / build
        return {"unavailable": f"{type(error).__name__}: {error}"[:200]}
    restored = [torch.empty(s, dtype=torch.bfloat16, device="cuda") for _, s in shapes]
    dense_bytes = 2 * sum(t.numel() for t in tensors)
    result = {"multicast_bound": peer.multicast, "note": "replaces all_gather_ms + decode_all_ms above"}
    # Direct: the decoder's own loads cross NVLink.  Staged: every CTA first copies its block's
    # side bytes into local scratch with 16-byte requests and decodes from the copy.
    for name, stage_for in (("direct", None), ("staged", rank)):
        encode, decode = [], []
        for it in range(warmup + steps):
            barrier(world)
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            sharded.encode_rank(plan, rank, tensors, wire=peer.local)
            e[1].record()
            peer.fence()                       # every rank's wire is complete
            sharded.decode_all(plan, peer.buffers, [s for _, s in shapes], outputs=restored,
                               interleave_from=rank + 1, stage_remote_for=stage_for)
            e[2].record()
            peer.fence()                       # nobody still reads what the next step overwrites
            torch.cuda.synchronize()
            if it >= warmup:
                encode.append(e[0].elapsed_time(e[1]))
                decode.append(e[1].elapsed_time(e[2]))
        exact = all(torch.equal(a.view(torch.int16), b.view(torch.int16))
                    for a, b in zip(tensors, restored))
        decode_ms = max_over_ranks(statistics.mean(decode), world)
        leg = {"bit_exact": bool(exact), "encode_ms": max_over_ranks(statistics.mean(encode), world),
               "fence_and_decode_all_ms": decode_ms,
               "decode_gbps_aggregate": world * dense_bytes / decode_ms / 1e6}
        if name == "direct":
            result.update(leg)
        else:
            result["side_bytes_staged"] = leg
        for t in restored:
            t.zero_()
    return result


def arena_leg(batches: int = 3) -> dict:
    """BASELINE configuration 3: ReLU activations 16384 x 4096 BF16 (about half exact zeros),
    LAPLACE zero_prob 0.5 / SPARSE layout, ONE 64 MiB arena; batches of 16 live compressed
    tensors: compress all, decode all, free all.  Four distinct inputs are cycled (the compressed
    results all stay live).  Reports device time per tensor and the arena's high-water mark."""
    from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
    from losslessly_compressed_tensors_b200.operations import compress, decompress
    from losslessly_compressed_tensors_b200.tensor_buffer import (
        TensorBuffer, _free_regions_snapshot, verify_buffer)

    dist_cfg = Distribution(DistType.LAPLACE, param=1.0, zero_prob=0.5, noise_level=NoiseLevel.SPARSE)
    capacity = 64 << 20
    buffer = TensorBuffer(capacity)
    inputs = []
    for seed in range(4):
        g = torch.Generator().manual_seed(2 + seed)
        inputs.append(torch.randn(16384, 4096, generator=g).relu_().to(torch.bfloat16).cuda())
    live_count, n = 16, inputs[0].numel()
    enc, dec, exact, high_water, ratio = [], [], True, 0, 0.0
    for batch in range(batches + 1):   # first batch is the warm-up
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        e[0].record()
        live = [compress(inputs[i % 4], dist_cfg, buffer) for i in range(live_count)]
        e[1].record()
        free_bytes = sum(size for _, size in _free_regions_snapshot(buffer))   # host sync
        high_water = max(high_water, capacity - free_bytes)
        e[2].record()
        outs = [decompress(c) for c in live]
        e[3].record()
        torch.cuda.synchronize()
        for i in (0, 5, 10, 15):
            exact &= torch.equal(outs[i].view(torch.int16), inputs[i % 4].view(torch.int16))
        ratio = 2 * n / live[0].memory_size()
        del outs
        for c in live:
            c.free()
        verify_buffer(buffer)
        if batch:
            enc.append(e[0].elapsed_time(e[1]) / live_count)
            dec.append(e[2].elapsed_time(e[3]) / live_count)
    assert _free_regions_snapshot(buffer) == [(0, capacity)]
    return {
        "workload": "config3: 16 live 16384x4096 BF16 ReLU activations, LAPLACE zp 0.5 / SPARSE, "
                    "one 64 MiB arena; back-to-back launches, L2 not flushed between tensors "
                    "(each tensor is 128 MiB, larger than L2)",
        "encode_ms_per_tensor": statistics.mean(enc), "decode_ms_per_tensor": statistics.mean(dec),
        "encode_gbps": 2 * n / statistics.mean(enc) / 1e6, "decode_gbps": 2 * n / statistics.mean(dec) / 1e6,
        "compression_ratio": ratio, "arena_high_water_bytes": high_water, "bit_exact": bool(exact),
    }


def update_leg(steps: int = 10, warmup: int = 3) -> dict:
    """BASELINE configuration 4: momentum tensors of 4096 x 4096 BF16 ~ N(0, 1e-3), GAUSSIAN /
    MEDIUM layout, shared arena; step = m <- 0.95 m + g on the compressed state (decode, fma,
    re-encode in one launch), fresh g every step.  Timed per tensor-step with CUDA events."""
    from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
    from losslessly_compressed_tensors_b200.codec import pointwise as pointwise_module
    from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
    from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer, verify_buffer

    dist_cfg = Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.MEDIUM)
    buffer = TensorBuffer(64 << 20)
    n_tensors, shape = 12, (4096, 4096)
    gen = torch.Generator(device="cuda").manual_seed(10)
    states = [LCTTensor((torch.randn(shape, device="cuda", generator=gen) * 1e-3).to(torch.bfloat16),
                        buffer, dist_cfg) for _ in range(n_tensors)]
    grads = [(torch.randn(shape, device="cuda", generator=gen) * 1e-3).to(torch.bfloat16)
             for _ in range(4)]
    alpha = torch.tensor([0.95], dtype=torch.float32, device="cuda")
    c = states[0].x
    per_tensor = 2 * (c.sign_mantissa.numel() + (c.data.numel() - 4) * 4) + 2 * c.logical_numel
    out = {}
    for label, fused in (("fused", True), ("two_stage", False)):
        pointwise_module.FUSED_UPDATE = fused
        times, walls = [], []
        for it in range(warmup + steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            a.record()
            for k, state in enumerate(states):
                state.mul_add_(alpha, grads[(it + k) % len(grads)])
            b.record()
            walls.append((time.perf_counter() - t0) / n_tensors)
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(a.elapsed_time(b) / n_tensors)
        out[label + "_ms_per_tensor_step"] = statistics.mean(times)
        out[label + "_host_ms_per_tensor_step"] = statistics.mean(walls[warmup:]) * 1e3
        out[label + "_algorithmic_gbps"] = per_tensor / statistics.mean(times) / 1e6
    pointwise_module.FUSED_UPDATE = True
    # The twelve states through the many-tensor call: five launches per group of tensors
    # (groups of 4: the host prepares the next group while the GPU works; one group of 12).
    for label, group in (("many", 4), ("many_one_call", None)):
        times = []
        for it in range(warmup + steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            updates = [grads[(it + k) % len(grads)] for k in range(n_tensors)]
            a.record()
            LCTTensor.mul_add_many_(states, alpha, updates, group=group)
            b.record()
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(a.elapsed_time(b) / n_tensors)
        out[label + "_ms_per_tensor_step"] = statistics.mean(times)
        out[label + "_algorithmic_gbps"] = per_tensor / statistics.mean(times) / 1e6
    # The same with everything but the launches prepared once (two alternating value sets, job
    # tables, work buffers): six launches per step for all twelve states.
    from losslessly_compressed_tensors_b200.update_plan import UpdatePlan

    plan = UpdatePlan(states, alpha)
    times, walls = [], []
    for it in range(warmup + steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        updates = [grads[(it + k) % len(grads)] for k in range(n_tensors)]
        t0 = time.perf_counter()
        a.record()
        plan.step(updates)
        b.record()
        walls.append((time.perf_counter() - t0) / n_tensors)
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(a.elapsed_time(b) / n_tensors)
    out["plan_ms_per_tensor_step"] = statistics.mean(times)
    out["plan_algorithmic_gbps"] = per_tensor / statistics.mean(times) / 1e6
    out["plan_host_ms_per_tensor_step"] = statistics.mean(walls[warmup:]) * 1e3
    # the compressed state still decodes to what the dense recurrence gives
    check = LCTTensor(torch.zeros(shape, dtype=torch.bfloat16, device="cuda"), buffer, dist_cfg)
    dense = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    for k, g in enumerate(grads):
        if k % 2:
            LCTTensor.mul_add_many_([check], alpha, [g])
        else:
            check.mul_add_(alpha, g)
        dense = torch.addcmul(g.float(), dense.float(), alpha).to(torch.bfloat16)
    out["bit_exact_vs_dense_fma"] = bool(torch.equal(check.decompress().view(torch.int16),
                                                     dense.view(torch.int16)))
    for state in states + [check]:
        state.free()
    verify_buffer(buffer)
    out["workload"] = ("config4: 12 x 4096x4096 BF16 momentum, GAUSSIAN/MEDIUM, m = 0.95 m + g; "
                       "wall of the whole update incl. host launches")
    out["algorithmic_bytes_per_tensor_step"] = per_tensor
    return out


def momentum_leg(steps: int = 10, warmup: int = 3) -> dict:
    """Muon's momentum step (reference: LCT/components/sparse_utils.py:88-90,133-146) on twelve
    4096 x 4096 BF16 momentum tensors in the optimizer's default codebook and one arena:
    momentum <- lerp(momentum, grad, 1 - mu), grad <- lerp(grad, momentum, mu).  `fused`: one
    launch chain per tensor on the compressed momentum that also writes the direction over the
    gradient; `plan`: the same for all twelve tensors as one prepared call (what SparseMuon.step
    does); `sequence`: the reference's decompress_free / lerp_ / lerp_ / compress.  CUDA events around
    all twelve, per tensor-step."""
    from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
    from losslessly_compressed_tensors_b200.components.dist_configs import momentum_dist
    from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer, verify_buffer

    mu, n_tensors, shape = 0.95, 12, (4096, 4096)
    buffer = TensorBuffer(64 << 20)
    gen = torch.Generator(device="cuda").manual_seed(20)
    start = [(torch.randn(shape, device="cuda", generator=gen) * 1e-3).to(torch.bfloat16)
             for _ in range(n_tensors)]
    grads = [(torch.randn(shape, device="cuda", generator=gen) * 1e-3).to(torch.bfloat16)
             for _ in range(4)]
    work = [torch.empty(shape, dtype=torch.bfloat16, device="cuda") for _ in range(n_tensors)]
    w_m = torch.tensor([1 - mu], dtype=torch.float32, device="cuda")
    w_d = torch.tensor([mu], dtype=torch.float32, device="cuda")
    out, final = {}, {}
    from losslessly_compressed_tensors_b200.codec import pointwise
    from losslessly_compressed_tensors_b200.kernels import dispatch
    from losslessly_compressed_tensors_b200.update_plan import UpdatePlan

    for label in ("fused", "plan", "sequence"):
        states = [LCTTensor(m, buffer, momentum_dist) for m in start]
        plan = (UpdatePlan(states, w_m, w_d, operation=pointwise.LERP, emit=dispatch.EMIT_NESTEROV)
                if label == "plan" else None)
        times, walls = [], []
        for it in range(warmup + steps):
            for k in range(n_tensors):        # the step's gradients (overwritten by the direction)
                work[k].copy_(grads[(it + k) % len(grads)])
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            a.record()
            if plan is not None:
                plan.step(work, dense_outs=work)
            for k, state in enumerate(states):
                if plan is not None:
                    break
                if label == "fused":
                    assert state.lerp_(work[k], w_m, nesterov_out=work[k], nesterov_weight=w_d)
                else:
                    dense = state.decompress_free()
                    dense.lerp_(work[k], 1 - mu)
                    work[k].lerp_(dense, mu)
                    states[k] = LCTTensor(dense, buffer, momentum_dist)
            b.record()
            walls.append((time.perf_counter() - t0) / n_tensors)
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(a.elapsed_time(b) / n_tensors)
        out[label + "_ms_per_tensor_step"] = statistics.mean(times)
        out[label + "_host_ms_per_tensor_step"] = statistics.mean(walls[warmup:]) * 1e3
        final[label] = ([s.decompress() for s in states], [w.clone() for w in work])
        if label == "fused":
            c = states[0].x
            out["algorithmic_bytes_per_tensor_step"] = (
                2 * (c.sign_mantissa.numel() + (c.data.numel() - 4) * 4) + 4 * c.logical_numel)
        for state in states:
            state.free()
    verify_buffer(buffer)
    out["fused_algorithmic_gbps"] = (out["algorithmic_bytes_per_tensor_step"]
                                     / out["fused_ms_per_tensor_step"] / 1e6)
    out["plan_algorithmic_gbps"] = (out["algorithmic_bytes_per_tensor_step"]
                                    / out["plan_ms_per_tensor_step"] / 1e6)
    out["speedup"] = out["sequence_ms_per_tensor_step"] / out["fused_ms_per_tensor_step"]
    out["plan_speedup"] = out["sequence_ms_per_tensor_step"] / out["plan_ms_per_tensor_step"]
    out["bit_exact_vs_torch_lerp"] = all(
        torch.equal(x.view(torch.int16), y.view(torch.int16))
        for label in ("fused", "plan")
        for part in (0, 1) for x, y in zip(final[label][part], final["sequence"][part]))
    out["workload"] = ("12 x 4096x4096 BF16 Muon momentum, EMPIRICAL/CLEAN zero_prob 0.02, mu 0.95, "
                       f"{warmup + steps} steps; bytes = compressed in + out, gradient in, direction out")
    return out


def activations_leg(steps: int = 10, warmup: int = 3) -> dict:
    """The activations one GPT-2-small block saves for backward (8 x 1024 tokens, d_model 768:
    block input, two layer-norm outputs, QKV, attention output, MLP pre-activation and GELU
    output; seeded N(0, 1) values through the real nonlinearities), kept compressed between
    forward and backward in one arena (reference pattern: LCT/components/layers.py:57,116,166,
    211,237 - compress at save, decompress + free in backward).  A step = store all, load all.
    `per_tensor`: one compress / decompress / free per tensor; `batched`: the group calls of
    ActivationCache(batch=0).  CUDA events around the step; launches counted on the host."""
    from losslessly_compressed_tensors_b200.components.activations import ActivationCache
    from losslessly_compressed_tensors_b200.components.dist_configs import act_dist
    from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer, verify_buffer

    tokens, d = 8 * 1024, 768
    gen = torch.Generator(device="cuda").manual_seed(30)

    def normal(cols):
        return torch.randn(tokens, cols, device="cuda", generator=gen)

    x = normal(d)
    ln1 = torch.nn.functional.layer_norm(x, (d,))
    qkv = normal(3 * d)
    attn = normal(d) * 0.5
    x2 = x + attn
    ln2 = torch.nn.functional.layer_norm(x2, (d,))
    fc = normal(4 * d)
    act = torch.nn.functional.gelu(fc)
    saved = [t.to(torch.bfloat16) for t in (x, ln1, qkv, attn, ln2, fc, act)]
    dense_bytes = sum(t.numel() * 2 for t in saved)
    buffer = TensorBuffer(64 << 20)
    out = {"tensors": len(saved), "dense_bytes_per_step": dense_bytes}
    for label, batch in (("per_tensor", None), ("batched", 0)):
        cache = ActivationCache(buffer, act_dist, min_elements=65536, batch=batch)
        times, exact = [], True
        for it in range(warmup + steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with LaunchTrace() as trace:
                a.record()
                handles = [cache.store(t) for t in saved]
                cache.flush()
                loaded = [h.load() for h in reversed(handles)]
                b.record()
            launches = trace.count
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(a.elapsed_time(b))
            if it == warmup:
                exact = all(torch.equal(got.view(torch.int16), want.view(torch.int16))
                            for got, want in zip(loaded, reversed(saved)))
            del handles, loaded
        out[label + "_ms_per_step"] = statistics.mean(times)
        out[label + "_launches_per_step"] = launches
        out[label + "_gbps"] = 2 * dense_bytes / statistics.mean(times) / 1e6
        out[label + "_bit_exact"] = exact
    verify_buffer(buffer)
    out["speedup"] = out["per_tensor_ms_per_step"] / out["batched_ms_per_step"]
    out["workload"] = ("saved activations of one GPT-2-small block, 8192 tokens, LAPLACE/CLEAN, one "
                       "64 MiB arena; step = compress all + decompress all + free all; "
                       "gbps = BF16 bytes in + out per step")
    return out


def run_ours(args, rank: int, world: int, local: int):
    from losslessly_compressed_tensors_b200.codec import encode as encode_module
    from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType
    from losslessly_compressed_tensors_b200.operations import compress, decompress
    from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer, verify_buffer

    dist_cfg = Distribution(DistType.LAPLACE, param=0.02)
    host_x = make_workload(1 + rank).pin_memory()
    x = host_x.cuda(non_blocking=True)
    buffer = TensorBuffer(64 << 20)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
    n = x.numel()
    bf16_bytes = 2 * n

    # Correctness of what is about to be timed, and the byte counts for the roofline.
    c = compress(x, dist_cfg, buffer)
    y = decompress(c)
    assert torch.equal(y.view(torch.int16), x.view(torch.int16)), "round trip is not bit-exact"
    memory = c.memory_size()
    tails = int(c.fallback_used.item()) + 2 * int(c.fallback_count.item())
    algorithmic = bf16_bytes + c.sign_mantissa.numel() + (c.data.numel() - 4) * 4 + tails
    oracle_match = full_size_oracle_check(host_x, c, dist_cfg) if rank == 0 else None
    c.free()
    del y

    def event():
        return torch.cuda.Event(enable_timing=True)

    def one_step(timed):
        flush.zero_()
        e0, e1, e2, e3 = event(), event(), event(), event()
        e0.record()
        c = compress(x, dist_cfg, buffer)
        e1.record()
        flush.zero_()
        e2.record()
        y = decompress(c)
        e3.record()
        c.free()
        if timed is not None:
            timed.append((e0, e1, e2, e3))
        return y

    for _ in range(args.warmup):
        one_step(None)
    barrier(world)
    sampler = ClockSampler(local) if rank == 0 else None
    spans = []
    with LaunchTrace(timed=("lct_decode",)) as trace:
        wall0 = time.perf_counter()
        for _ in range(args.steps):
            one_step(spans)
        barrier(world)
        wall = time.perf_counter() - wall0
    enc_ms = [a.elapsed_time(b) for a, b, _, _ in spans]
    dec_ms = [c_.elapsed_time(d) for _, _, c_, d in spans]
    step_ms = (sum(enc_ms) + sum(dec_ms)) / args.steps
    step_ms = max_over_ranks(step_ms, world)
    value = world * 2 * bf16_bytes / (step_ms * 1e-3) / 1e9
    launches = trace.count
    kernel_ms = {name: statistics.mean(trace.milliseconds(name)) for name in trace.timed}
    # The encoder kernel on its own: compress() above is one call whose four launches overlap,
    # so the kernel is timed in a pass of its own through the stage-by-stage calls (same kernels).
    encode_module.SINGLE_CALL_PIPELINE = False
    try:
        with LaunchTrace(timed=("lct_encode",)) as encode_trace:
            for _ in range(max(3, min(args.steps, 20))):
                flush.zero_()
                compress(x, dist_cfg, buffer).free()
            torch.cuda.synchronize()
    finally:
        encode_module.SINGLE_CALL_PIPELINE = True
    kernel_ms["lct_encode"] = statistics.mean(encode_trace.milliseconds("lct_encode"))
    # The step as one captured CUDA graph (compress + decompress + free, seven launches):
    # what a caller with fixed shapes pays per step once the host is out of the loop.  Back to
    # back, no L2 flush in between (the 128 MiB input and output are each larger than L2).
    graph_ms = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            c = compress(x, dist_cfg, buffer)
            graph_out = decompress(c)
            c.free()
        del c
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        replays = max(10, min(args.steps, 50))
        a, b = event(), event()
        a.record()
        for _ in range(replays):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        if torch.equal(graph_out.view(torch.int16), x.view(torch.int16)):
            graph_ms = a.elapsed_time(b) / replays
        del graph, graph_out
    except RuntimeError as error:   # capture refused by this driver / PyTorch build
        print(f"graph replay leg skipped: {error}", file=sys.stderr)
    # Without a shared arena (the reference's other mode): exact-size private overflow tensors
    # need the two totals on the host, i.e. one synchronisation inside every compress.
    private_ms = []
    for _ in range(max(3, min(args.steps, 10))):
        flush.zero_()
        a, b = event(), event()
        a.record()
        c = compress(x, dist_cfg, None)
        b.record()
        torch.cuda.synchronize()
        private_ms.append(a.elapsed_time(b))
        del c

    # End to end: host buffers in, host buffers out, copies inside the timed region.  Every step
    # copies its input from pinned host memory and its decoded result back to pinned host memory;
    # the three stages of consecutive steps overlap on three streams (two copy engines and the
    # SMs), with two sets of buffers, as a streaming user of the codec would run it.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    host_out = [torch.empty_like(host_x).pin_memory() for _ in range(2)]
    dev_in = [torch.empty_like(x) for _ in range(2)]
    dev_out = [None, None]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    for k in range(2):
        in_free[k].record(main)
        out_done[k].record(s_out)

    def e2e_step(i):
        k = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[k])               # the step two back has consumed dev_in[k]
            dev_in[k].copy_(host_x, non_blocking=True)
            in_ready[k].record(s_in)
        main.wait_event(in_ready[k])
        main.wait_event(out_done[k])                  # dev_out[k] of the step two back is on the host
        c = compress(dev_in[k], dist_cfg, buffer)
        in_free[k].record(main)
        dev_out[k] = decompress(c)
        c.free()
        out_ready[k].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(out_ready[k])
            host_out[k].copy_(dev_out[k], non_blocking=True)
            dev_out[k].record_stream(s_out)
            out_done[k].record(s_out)

    for i in range(4):
        e2e_step(i)
    barrier(world)
    e2e_steps = max(4, min(args.steps, 20))
    s, t = event(), event()
    s.record(main)
    for i in range(e2e_steps):
        e2e_step(i)
    main.wait_event(out_done[0])
    main.wait_event(out_done[1])
    t.record(main)
    barrier(world)
    e2e_ms = max_over_ranks(s.elapsed_time(t) / e2e_steps, world)
    for k in range(2):
        assert torch.equal(host_out[k].view(torch.int16), host_x.view(torch.int16))
    verify_buffer(buffer)
    e2e_value = world * 2 * bf16_bytes / (e2e_ms * 1e-3) / 1e9
    # The same loop with the copies alone (no codec): what the host link allows.
    def copy_step(i):
        k = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[k])
            dev_in[k].copy_(host_x, non_blocking=True)
            in_ready[k].record(s_in)
        with torch.cuda.stream(s_out):
            s_out.wait_event(in_ready[k])
            host_out[k].copy_(dev_in[k], non_blocking=True)
            in_free[k].record(s_out)
            out_done[k].record(s_out)

    for i in range(2):
        copy_step(i)
    barrier(world)
    s, t = event(), event()
    s.record(main)
    for i in range(e2e_steps):
        copy_step(i)
    main.wait_event(out_done[0])
    main.wait_event(out_done[1])
    t.record(main)
    barrier(world)
    copy_ms = max_over_ranks(s.elapsed_time(t) / e2e_steps, world)
    # Each direction alone: with both directions perfectly overlapped a step cannot take less
    # than the slower of the two.
    one_way_ms = []
    for direction in ("h2d", "d2h"):
        stream = s_in if direction == "h2d" else s_out
        s, t = event(), event()
        with torch.cuda.stream(stream):
            stream.wait_stream(main)
            s.record(stream)
            for i in range(e2e_steps):
                if direction == "h2d":
                    dev_in[i & 1].copy_(host_x, non_blocking=True)
                else:
                    host_out[i & 1].copy_(dev_in[i & 1], non_blocking=True)
            t.record(stream)
        main.wait_stream(stream)
        barrier(world)
        one_way_ms.append(max_over_ranks(s.elapsed_time(t) / e2e_steps, world))
    clocks = sampler.finish() if sampler else None   # sampled across the timed regions

    del host_out, dev_in, dev_out, x, flush
    legs = set() if args.no_sharded else set(args.legs.split(","))
    if world > 1:
        legs.add("peer")      # the peer-memory decode is part of every multi-GPU run
    sharded = sharded_leg(rank, world, with_peer="peer" in legs) if "sharded" in legs else None
    update = update_leg() if (rank == 0 and "update" in legs) else None
    arena = arena_leg() if (rank == 0 and "arena" in legs) else None
    momentum = momentum_leg() if (rank == 0 and "momentum" in legs) else None
    activations = activations_leg() if (rank == 0 and "activations" in legs) else None
    if rank != 0:
        return
    triton_reference = (triton_reference_leg() if world == 1 and "triton" in legs else None)
    peak, peak_kind = peak_hbm_gbs()
    kernels = {}
    for name, ms in kernel_ms.items():
        achieved = algorithmic / (ms * 1e-3) / 1e9
        kernels[name] = {"ms": ms, "achieved": achieved, "frac": achieved / peak,
                         "bf16_gbps": bf16_bytes / (ms * 1e-3) / 1e9}
    dominant = max(kernel_ms, key=kernel_ms.get)
    roofline = {
        "kernel": dominant, "bound": "hbm", "achieved": kernels[dominant]["achieved"], "peak": peak,
        "peak_source": f"{peak_kind} copy bandwidth", "unit": "GB/s",
        "frac": kernels[dominant]["frac"], "traffic": NCU_TRAFFIC_BYTES[dominant],
        "algorithmic_bytes": algorithmic,
    }
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": bench_config(world),
        "encode_ms": statistics.mean(enc_ms), "decode_ms": statistics.mean(dec_ms),
        "encode_gbps": bf16_bytes / statistics.mean(enc_ms) / 1e6,
        "decode_gbps": bf16_bytes / statistics.mean(dec_ms) / 1e6,
        "compression_ratio": bf16_bytes / memory, "memory_size": memory,
        "bit_exact_vs_oracle_full_size": oracle_match,
        "wall_ms_per_step": wall / args.steps * 1e3,
        "roofline": roofline, "kernels": kernels,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": bf16_bytes, "d2h_bytes_per_step": bf16_bytes},
        "e2e_copies_only": {"value": world * 2 * bf16_bytes / (copy_ms * 1e-3) / 1e9, "unit": UNIT,
                            "ms_per_step": copy_ms,
                            "h2d_alone_gbps": world * bf16_bytes / (one_way_ms[0] * 1e-3) / 1e9,
                            "d2h_alone_gbps": world * bf16_bytes / (one_way_ms[1] * 1e-3) / 1e9,
                            "duplex_ceiling": world * 2 * bf16_bytes / (max(one_way_ms) * 1e-3) / 1e9,
                            "note": "value: the same pinned H2D + D2H copies per step with no "
                                    "codec between them (both directions started together, which "
                                    "on some hosts is slower than the staggered copies of the real "
                                    "loop); *_alone: each direction by itself; duplex_ceiling: "
                                    "2 x bytes / the slower direction, which no e2e step can beat"},
        "gpu_launches": launches, "clocks": clocks,
        "encode_ms_without_arena": statistics.mean(private_ms),
        "graph_replay_ms_per_step": graph_ms, "arena": arena, "update": update,
        "momentum": momentum, "activations": activations,
    }
    if world == 1 and not args.no_cpu:
        bits = host_x.view(torch.int16).numpy().reshape(-1)
        cpu_value, cpu_steps, used, _ = cpu_leg(bits, 1, 15.0, 8)
        line["cpu_baseline"] = {
            "value": cpu_value, "unit": UNIT, "cores": used, "kind": "port",
            "sample": f"full workload, {cpu_steps} step(s) of compress+decompress, "
                      f"single-threaded C restatement of the reference kernels"}
    # Last, so that a reader of the line's tail sees them: the reference's own kernels on this
    # GPU, and the multi-GPU weight-set step.
    line["triton_reference"] = triton_reference
    line["sharded"] = sharded
    emit(line)


def full_size_oracle_check(host_x: torch.Tensor, c, dist_cfg) -> bool:
    """Every stored component of the 64 Mi-element result against the CPU restatement."""
    from helpers import oracle_compress
    from oracle import lct_oracle as oracle

    oracle.build()
    oracle.set_threads(0)
    want = oracle_compress(oracle, host_x.view(torch.int16).numpy().reshape(-1), dist_cfg, None)
    same = (torch.equal(c.data.cpu(), torch.from_numpy(want["encoded"]))
            and torch.equal(c.sign_mantissa.cpu(), torch.from_numpy(want["side"]))
            and torch.equal(c.fallback_blocks.cpu(), torch.from_numpy(want["blocks"]))
            and int(c.center.item()) == int(want["center"])
            and int(c.fallback_count.item()) == int(want["count"])
            and int(c.fallback_used.item()) == int(want["tail_bytes"]))
    return bool(same)


_RESULT_FD = None


def _keep_stdout_for_the_result() -> None:
    """The contract is ONE JSON line on standard output.  Libraries print there too (NCCL its
    version line when asked to), so from here on file descriptor 1 is standard error's, and the
    result line goes to a private copy of the original."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    text = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text)


def main():
    _keep_stdout_for_the_result()
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--no-sharded", action="store_true",
                        help="skip the extra legs (configurations 3, 4 and 5)")
    parser.add_argument("--legs", default="sharded,update,momentum,activations,arena,triton",
                        help="extra legs to run after configuration 2: sharded (configuration 5), "
                             "update (configuration 4), momentum (Muon's momentum step), activations (a block's saved activations), "
                             "arena (configuration 3), triton (the "
                             "reference's own kernels on this GPU, N = 1); with N > 1 the sharded "
                             "leg always includes the peer-memory decode")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args, int(os.environ.get("RANK", "0")))
        return
    args.warmup = max(args.warmup, 3)
    rank, world, local = distributed_setup(args.gpus)
    try:
        run_ours(args, rank, world, local)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
