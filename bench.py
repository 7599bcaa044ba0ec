#!/usr/bin/env python3
"""Benchmark of the PI0.5 policy forward (FP8) on 1..8 B200, one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Metric: action chunks per second over all GPUs. A step is one batched policy forward of
`--batch` (default 64) independent observations per GPU in FP8 — two 224x224 views, 10 prompt
tokens, horizon 50, 10 flow steps — with a full weight replica per GPU and no collective on
the data path (weak scaling). The same JSON line also carries the B=1 graph-replay latency
(p50 over 30 replays, two views, 10 tokens, horizon 10) since the headline metric quotes
both. Inputs are seeded synthetic stand-ins (uniform u8 images, uniform token ids, N(0,1)
noise); weights are the reference's seeded synthetic generator.

  value      device-resident: inputs already in HBM, CUDA-graph replays timed with CUDA
             events on the engine stream, max over ranks.
  e2e        the user-facing call with pinned HOST buffers: host->device copy of the images,
             ids and noise + replay + device->host read of the action chunks, every step.
  roofline   the dominant kernel (language gate_up GEMM + fused GeGLU), timed live with CUDA
             events around each of its launches in one eager pass on the engine stream.
  cpu_baseline / --impl reference
             the CPU oracle (NumPy port of the reference arithmetic, all host threads) on a
             bounded sample: PI0.5 has no CPU implementation in the reference, and its Rust
             host cannot be built here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from dataclasses import replace
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "pi05_fp8_action_chunks_per_s"
UNIT = "action chunks/s"


GATE_UP_DRAM_BYTES_BATCH64 = 276.02e6 + 508.51e6


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"],
                "bf16_tflops_sustained": data.get("bf16_tflops_sustained", data["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.device_index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(np.max(sm_max)) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def pinned_like(array, torch):
    t = torch.from_numpy(np.ascontiguousarray(array)).pin_memory()
    return t


# ---------------------------------------------------------------------------
# CPU baseline (oracle port on a bounded sample)
# ---------------------------------------------------------------------------


class CpuSample:
    """The NumPy oracle on depth-2 towers and one flow step (full widths, FP8 arithmetic,
    B=1, H=50); `seconds()` times it and scales by layer / step counts to one full forward.
    Weight generation happens once in the constructor and is not part of the timing."""

    def __init__(self):
        from oracle import pi05_oracle as O
        self.O = O
        self.full = replace(O.Pi05Config(), num_views=2, action_horizon=50)
        self.depth = 2
        full, depth = self.full, self.depth
        self.cfg = replace(full, vision_depth=depth, num_flow_steps=1,
                           language=replace(full.language, depth=depth + 1),
                           action_expert=replace(full.action_expert, depth=depth + 1))
        weights = O.SyntheticWeights(self.cfg, 0)
        weights.cache_prefixes = ("",)  # keep every tensor
        self.inputs = O.synthetic_observation(self.cfg, 1234, 10)
        self.oracle = O.Pi05Oracle(self.cfg, weights, O.OracleOptions(dtype="fp8", act_scale=0.05))
        self.oracle._prepare_all = True
        self.oracle.infer(*self.inputs)  # generates and caches the weights
        self.threads = os.cpu_count() or 1
        self.sample = (
            f"NumPy oracle, FP8 arithmetic, B=1: {depth} of {full.vision_depth} SigLIP layers, "
            f"{depth} of {full.language.depth - 1} Gemma-2B layers, 1 of {full.num_flow_steps} "
            f"flow steps over {depth + 1} of {full.action_expert.depth} expert layers, full widths; "
            f"scaled by layer and step counts; weight generation excluded")

    def seconds(self) -> float:
        images, tokens, noise = self.inputs
        full, depth, oracle = self.full, self.depth, self.oracle
        t0 = time.perf_counter()
        vision = oracle.encode_vision(images)
        t1 = time.perf_counter()
        prefix = oracle.embed_prefix(vision, tokens)
        keys, values = oracle.prefix_forward(prefix)
        t2 = time.perf_counter()
        oracle.denoise(noise, keys, values, prefix.shape[0])
        t3 = time.perf_counter()
        vision_s = (t1 - t0) / depth * full.vision_depth
        # depth+1 language layers ran, the last without its tail: count `depth` full layers
        prefix_s = (t2 - t1) / depth * (full.language.depth - 1)
        action_s = (t3 - t2) / (depth + 1) * full.action_expert.depth * full.num_flow_steps
        return vision_s + prefix_s + action_s


def cpu_block_cfg1():
    """BASELINE configuration 1: one Gemma-style decoder block (522 tokens, hidden 2048, 8 query
    heads / 1 KV head, head_dim 256, GeGLU 16384, causal) on the reference's CPU operators
    (naive single-threaded f32 sgemm), restated in C under oracle/. Timed on 4 tokens and scaled
    to 522 (the GEMMs, >99% of the work, are linear in tokens)."""
    from oracle import cpu_block
    tokens = 4
    case = cpu_block.make_case(0, seq=tokens, hidden=2048, heads=8, kv_heads=1, head_dim=256, mlp=16384)
    _, seconds = cpu_block.run_c(case, 8, 1, 256)
    full = seconds / tokens * 522
    return {"seconds_per_block": full, "gflops": 117.0 / full, "cores": 1, "kind": "port",
            "sample": f"{tokens} of 522 tokens timed ({seconds:.2f} s), scaled linearly"}


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    cpu = CpuSample()
    sample, threads = cpu.sample, cpu.threads
    times = []
    for i in range(args.warmup + args.steps):
        seconds = cpu.seconds()
        if i >= args.warmup:
            times.append(seconds)
    per_forward = float(np.mean(times))
    value = 1.0 / per_forward
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_forward * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8",
        "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "PI0.5 has no CPU implementation in the reference and its Rust host cannot be "
                "built in this image; this arm times the CPU oracle port of its arithmetic",
    }
    print(json.dumps(line), flush=True)
    return 0


def workload_config(args):
    return {"workload": (f"cfg5: PI0.5 FP8 batched policy forward, {args.batch} observations/GPU, "
                         "2 views 224x224 u8 NHWC, 10 prompt tokens, H=50, 10 flow steps, "
                         "random weights (seeded LCG), uniform FP8 activation scale 0.05"),
            "global_batch": args.batch * args.gpus, "parallelism": f"dp{args.gpus}",
            "l2": "weights (3.9 GB) and activations exceed the 126 MB L2 every step"}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------


def run_ours(args):
    import torch
    from apxinf_b200.engine import Pi05Config, Pi05Runtime
    from apxinf_b200.fixtures import synthetic_batch

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the PI0.5 path has no CPU fallback")
    torch.cuda.set_device(local)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if distributed:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    def max_over_ranks(value):
        if not distributed:
            return value
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    token_count = 10
    cfg_tp = Pi05Config(num_views=2, action_horizon=50)
    rt = Pi05Runtime.random(cfg_tp, dtype="fp8", seed=0, device=local, fp8_act_scale=0.05)
    graph = rt.capture_infer_rgb_u8(token_count, "nhwc", args.batch)
    images, tokens, noise = synthetic_batch(cfg_tp, args.batch, token_count, 1000 + rank * args.batch)
    from apxinf_b200.engine import float_to_bf16_bits
    h_images = pinned_like(images, torch)
    h_tokens = pinned_like(tokens.astype(np.uint32).view(np.int32), torch)
    h_noise = pinned_like(float_to_bf16_bits(noise).view(np.int16), torch)
    out_host = np.empty(graph.output_shape, dtype=np.float32)

    # ---- device-resident: graph replays ----
    graph.update_raw_image_inputs(h_images, h_tokens, h_noise)
    graph.synchronize()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    graph.synchronize()
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    ms = graph.time_replays(args.steps)
    barrier()
    clocks = sampler.stop()
    device_seconds = max_over_ranks(float(ms.sum()) / 1e3)
    chunks = args.batch * world * args.steps
    value = chunks / device_seconds

    # ---- end to end: host buffers in, host action chunks out ----
    for _ in range(2):
        graph.update_raw_image_inputs(h_images, h_tokens, h_noise)
        graph.replay()
        graph.output(out_host)
    barrier()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        graph.update_raw_image_inputs(h_images, h_tokens, h_noise)
        graph.replay()
        graph.output(out_host)
    e2e_seconds = time.perf_counter() - t0
    barrier()
    e2e_seconds = max_over_ranks(e2e_seconds)
    finite = bool(np.isfinite(out_host).all())
    h2d = int(images.nbytes + tokens.size * 4 + noise.size * 2)
    d2h = int(out_host.size * 2)

    line = None
    if rank == 0:
        # ---- roofline of the dominant kernel, live ----
        peaks = measured_peaks()
        lg = cfg_tp.language
        rows = args.batch * (cfg_tp.num_views * cfg_tp.patches_per_view + token_count)
        avg_ms, count = graph.time_launches("language.gate_up")
        flops = 2.0 * rows * (2 * lg.mlp_dim) * lg.width
        achieved = flops / (avg_ms * 1e-3) / 1e12
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        roofline = {
            "kernel": "gemm_umma_persistent_kernel<e4m3, 128x256 tile> language.gate_up + GeGLU epilogue",
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the single-pass ncu
            # capture of this workload summarised under profiles/ (batch 64 only)
            "traffic": GATE_UP_DRAM_BYTES_BATCH64 if args.batch == 64 else None,
            "launch_ms": avg_ms, "launches_timed": count,
            "flops_per_launch": flops,
            "peak_source": (f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}); "
                            "no FP8 peak is measured on this pool, FP8 dense = 2 x BF16 nominally"),
        }
        # ---- B=1 latency, the other half of the headline ----
        latency = measure_latency(rt_dtype="fp8", device=local)
        # the other two precisions of the path, same protocol (p50 only)
        latency["other_precisions_p50_ms"] = {
            dtype: measure_latency(rt_dtype=dtype, device=local)["p50_ms"] for dtype in ("bf16", "int8")}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": device_seconds / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8",
            "data": "synthetic", "config": workload_config(args), "clocks": clocks,
            "e2e": {"value": chunks / e2e_seconds, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h},
            "gpu_launches": (graph.num_launches() - 1) * args.steps,
            "roofline": roofline, "latency_b1": latency, "outputs_finite": finite,
        }
    graph.close()
    rt.close()
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            cpu = CpuSample()
            seconds = min(cpu.seconds() for _ in range(2))
            line["cpu_baseline"] = {"value": 1.0 / seconds, "unit": UNIT, "cores": cpu.threads,
                                    "kind": "port", "sample": cpu.sample}
            line["cpu_block_cfg1"] = cpu_block_cfg1()
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier(device_ids=[local])
        dist.destroy_process_group()
    return 0


def measure_latency(rt_dtype, device):
    """B=1 two-view graph-replay latency (pi05_bench protocol: 10 warm-ups, 30 replays)."""
    from apxinf_b200.engine import Pi05Config, Pi05Runtime
    from apxinf_b200.fixtures import synthetic_observation
    cfg = Pi05Config()
    rt = Pi05Runtime.random(cfg, dtype=rt_dtype, seed=0, device=device, fp8_act_scale=0.05)
    graph = rt.capture_infer_rgb_u8(10, "nhwc", 1)
    images, tokens, noise = synthetic_observation(cfg, 1234, 10)
    graph.update_raw_image_inputs(images[None], tokens[None], noise[None])
    for _ in range(10):
        graph.replay()
    graph.synchronize()
    ms = np.sort(graph.time_replays(30))
    t0 = time.perf_counter()
    out = graph.infer_host(images[None], tokens[None], noise[None])
    update_plus_graph = (time.perf_counter() - t0) * 1e3
    stages = graph.stage_times()
    result = {"workload": f"cfg{dict(bf16=2, fp8=3, int8=3)[rt_dtype]}: {rt_dtype.upper()}, B=1, 2 views, 10 tokens, H=10, 10 flow steps",
              "p50_ms": float(ms[len(ms) // 2]), "p95_ms": float(ms[int(round(0.95 * (len(ms) - 1)))]),
              "min_ms": float(ms[0]), "max_ms": float(ms[-1]),
              "input_update_plus_graph_ms": update_plus_graph, "launches": graph.num_launches(),
              "stage_ms_eager": stages, "finite": bool(np.isfinite(out).all())}
    graph.close()
    rt.close()
    return result


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--batch", type=int, default=64, help="observations per GPU per step")
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()
    _, world, _ = dist_env()
    if args.impl == "ours" and world != args.gpus:
        if args.gpus != 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks "
                             f"(WORLD_SIZE={world})")
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
