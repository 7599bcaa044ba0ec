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
import sys


def _host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


if "reference" in sys.argv[1:] or any(a.startswith("--impl=reference") for a in sys.argv[1:]):
    # the CPU arm uses every host thread it may run on, whatever the launcher exported
    # (torchrun sets OMP_NUM_THREADS=1); must happen before NumPy loads its BLAS
    for _name in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_name] = str(_host_threads())

import hashlib
import subprocess
import threading
import time
from dataclasses import replace
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "pi05_fp8_action_chunks_per_s"
UNIT = "action chunks/s"


# dram__bytes_read.sum + dram__bytes_write.sum of one language.gate_up launch at batch 64, from
# the single-pass ncu capture summarised in
# profiles/gemm_umma_persistent_e4m3_gate_up_batch64_dram_traffic.md, together with a digest
# of the kernel and planner sources that were profiled: the bench line reports the traffic only while the
# kernel source is still that one (null otherwise: a stale figure says nothing).
GATE_UP_DRAM_BYTES_BATCH64 = 275.0e6 + 505.1e6
GATE_UP_PROFILED_KERNEL_BLOB = "a069f6ec41f8"  # kernel_source_blob() of the profiled build


def kernel_source_blob() -> str:
    """Digest of the sources that decide the profiled launch: the kernel and its planner."""
    h = hashlib.sha1()
    for name in ("gemm_umma.cuh", "gemm.cu"):
        h.update((ROOT / "apxinf_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()[:12]


def algorithmic_work(cfg, token_count: int, batch: int, weight_bytes: int):
    """FLOPs of one batched forward and the minimum HBM bytes of one B=1 forward (every weight
    read once per use, the KV cache once per flow step), from the GEMM table of the model:
    vision patch/qkv/o/fc1/fc2/projector, language qkv/o/gate_up/down (17 full layers + the
    last layer's K/V projection), action in/out/qkv/o/gate_up/down per flow step, and the
    three attention shapes."""
    V = cfg.num_views * cfg.patches_per_view
    P, H, S = V + token_count, cfg.action_horizon, cfg.num_flow_steps
    vw, lg, ac = cfg.vision_width, cfg.language, cfg.action_expert
    qw = lg.num_heads * lg.head_dim
    kvw = qw + 2 * lg.head_dim
    vision_w = (3 * cfg.patch_size ** 2 * vw + cfg.vision_depth * (4 * vw * vw + 2 * vw * cfg.vision_mlp_dim)
                + vw * lg.width)
    language_full = lg.width * kvw + qw * lg.width + 3 * lg.width * lg.mlp_dim
    language_w = (lg.depth - 1) * language_full + lg.width * kvw
    action_layer = ac.width * kvw + qw * ac.width + 3 * ac.width * ac.mlp_dim
    action_w = ac.depth * action_layer + 2 * cfg.action_dim * ac.width
    gemm_flops = 2.0 * (V * vision_w + P * language_w + S * H * action_w)
    attn_flops = (4.0 * cfg.vision_depth * cfg.num_views * cfg.vision_heads * cfg.patches_per_view ** 2
                  * cfg.vision_head_dim
                  + 4.0 * (lg.depth - 1) * lg.num_heads * P * P * lg.head_dim
                  + 4.0 * S * ac.depth * ac.num_heads * H * (P + H) * ac.head_dim)
    kv_bytes = 2 * lg.depth * (P + H) * lg.head_dim * 2
    b1_bytes = weight_bytes * (vision_w + language_w + S * action_w) + (S + 1) * kv_bytes
    return {"flops_per_step": batch * (gemm_flops + attn_flops), "b1_hbm_bytes": b1_bytes}


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
        self.threads = _host_threads()
        self.sampled = {"siglip_layers": [depth, full.vision_depth],
                        "gemma_2b_layers": [depth, full.language.depth - 1],
                        "expert_layers": [depth + 1, full.action_expert.depth],
                        "flow_steps": [1, full.num_flow_steps]}
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


def complete_cpu_forward(budget_s: float, estimate_generation_s: float):
    """One complete oracle forward (every layer, every flow step) next to the scaled sample,
    when generating the full 2.6 G synthetic weights fits the time budget and host memory."""
    if estimate_generation_s > budget_s:
        return {"skipped": f"generating the full weights would take about {estimate_generation_s:.0f} s "
                           f"(budget {budget_s:.0f} s)"}
    try:
        available_gb = os.sysconf("SC_AVPHYS_PAGES") * os.sysconf("SC_PAGE_SIZE") / 2 ** 30
    except (ValueError, OSError):
        available_gb = 0.0
    if available_gb < 48:
        return {"skipped": f"{available_gb:.0f} GB of host memory free, 48 GB wanted for cached weights"}
    from oracle import pi05_oracle as O
    cfg = replace(O.Pi05Config(), num_views=2, action_horizon=50)
    weights = O.SyntheticWeights(cfg, 0)
    weights.cache_prefixes = ("",)
    oracle = O.Pi05Oracle(cfg, weights, O.OracleOptions(dtype="fp8", act_scale=0.05))
    oracle._prepare_all = True
    inputs = O.synthetic_observation(cfg, 1234, 10)
    t0 = time.perf_counter()
    oracle.infer(*inputs)  # generates, quantises and caches every weight
    first = time.perf_counter() - t0
    t0 = time.perf_counter()
    oracle.infer(*inputs)
    return {"seconds": time.perf_counter() - t0, "first_pass_with_weight_generation_s": first}


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=_host_threads())
    except Exception:
        pass
    t0 = time.perf_counter()
    cpu = CpuSample()
    construct_s = time.perf_counter() - t0
    sample, threads = cpu.sample, cpu.threads
    times = []
    for i in range(args.warmup + args.steps):
        seconds = cpu.seconds()
        if i >= args.warmup:
            times.append(seconds)
    per_forward = float(np.mean(times))
    value = 1.0 / per_forward
    sampled_seconds = float(np.sum(times))
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
        # the figure is an estimate: a few layers and one flow step are timed and scaled
        "extrapolated": True, "sampled": cpu.sampled, "timed_seconds_per_step": sampled_seconds / len(times),
        "note": "PI0.5 has no CPU implementation in the reference and its Rust host cannot be "
                "built in this image; this arm times the CPU oracle port of its arithmetic. "
                "ms_per_step is the scaled estimate of one complete forward, not a run of one",
    }
    if world == 1 and not args.no_complete_forward:
        # weight generation of the sample covered ~2/27 + 3/18 + 3/18 of the tensors
        line["complete_forward"] = complete_cpu_forward(args.complete_forward_budget, construct_s * 6.0)
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
    # this rank's contiguous shard of the global batch (observation i has seed 1000 + i)
    from apxinf_b200.parallel import shard_bounds
    shard = shard_bounds(args.batch * world, world)[rank]
    images, tokens, noise = synthetic_batch(cfg_tp, shard.size, token_count, 1000 + shard.start)
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
            "traffic": (GATE_UP_DRAM_BYTES_BATCH64
                        if args.batch == 64 and kernel_source_blob() == GATE_UP_PROFILED_KERNEL_BLOB else None),
            "traffic_profiled_kernel_blob": GATE_UP_PROFILED_KERNEL_BLOB,
            "kernel_blob_now": kernel_source_blob(),
            "launch_ms": avg_ms, "launches_timed": count,
            "flops_per_launch": flops,
            "peak_source": (f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}); "
                            "no FP8 peak is measured on this pool, FP8 dense = 2 x BF16 nominally"),
        }
        # ---- whole step against the same tensor peak ----
        work = algorithmic_work(cfg_tp, token_count, args.batch, 1)
        step_ms = device_seconds / args.steps * 1e3
        step_achieved = work["flops_per_step"] / (step_ms * 1e-3) / 1e12
        roofline_step = {"bound": "tensor", "flops_per_step": work["flops_per_step"],
                         "achieved": step_achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": step_achieved / peak, "peak_source": roofline["peak_source"]}
        # ---- B=1 latency, the other half of the headline ----
        latency = measure_latency(rt_dtype="fp8", device=local, per_op=True)
        b1 = algorithmic_work(Pi05Config(), token_count, 1, 1)
        latency["hbm_bytes"] = b1["b1_hbm_bytes"]
        latency["hbm_gbs"] = b1["b1_hbm_bytes"] / (latency["p50_ms"] * 1e-3) / 1e9
        latency["hbm_frac"] = latency["hbm_gbs"] / peaks["hbm_gbs"]
        latency["hbm_peak_gbs"] = peaks["hbm_gbs"]
        # the other two precisions of the path, same protocol (p50 only)
        bf16_latency = measure_latency(rt_dtype="bf16", device=local, per_op=True)
        latency["other_precisions_p50_ms"] = {
            "bf16": bf16_latency["p50_ms"], "int8": measure_latency(rt_dtype="int8", device=local)["p50_ms"]}
        ref_cuda = None
        if not args.no_ref_cuda and world == 1:
            ref_cuda = reference_cuda_leg(latency.pop("op_us", {}), bf16_latency.pop("op_us", {}),
                                          bf16_latency["stage_ms_eager"])
        latency.pop("op_us", None)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": device_seconds / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8",
            "data": "synthetic", "config": workload_config(args), "clocks": clocks,
            "e2e": {"value": chunks / e2e_seconds, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h},
            "gpu_launches": (graph.num_launches() - 1) * args.steps,
            "roofline": roofline, "roofline_step": roofline_step, "latency_b1": latency,
            "ref_cuda": ref_cuda, "outputs_finite": finite,
        }
    graph.close()
    rt.close()
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            cpu = CpuSample()
            seconds = min(cpu.seconds() for _ in range(2))
            line["cpu_baseline"] = {"value": 1.0 / seconds, "unit": UNIT, "cores": cpu.threads,
                                    "kind": "port", "sample": cpu.sample, "extrapolated": True,
                                    "sampled": cpu.sampled}
            line["cpu_block_cfg1"] = cpu_block_cfg1()
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier(device_ids=[local])
        dist.destroy_process_group()
    return 0


MODEL_GEMMS = {  # (M, N, K) of every GEMM of the replayed B=1 graph (2 views, 10 tokens, H=10)
    "vision.patch_embed": (512, 1152, 588), "vision.qkv": (512, 3456, 1152), "vision.o": (512, 1152, 1152),
    "vision.fc1": (512, 4304, 1152), "vision.fc2": (512, 1152, 4304), "vision.projector": (512, 2048, 1152),
    "language.qkv": (522, 2560, 2048), "language.o": (522, 2048, 2048),
    "language.gate_up": (522, 32768, 2048), "language.down": (522, 2048, 16384),
    "action.in": (10, 1024, 32), "action.qkv": (10, 2560, 1024), "action.o": (10, 1024, 2048),
    "action.gate_up": (10, 8192, 1024), "action.down": (10, 1024, 4096), "action.out": (10, 32, 1024),
}
MODEL_ATTENTION = {  # (query tokens, keys, heads, head_dim); SigLIP is per view
    "language.attn": (522, 522, 8, 256), "action.attn": (10, 532, 8, 256),
}


def reference_cuda_leg(ours_fp8_us, ours_bf16_us, ours_bf16_stage_ms):
    """The reference's own CUDA build on this GPU, beside ours (outside every timed region of
    the headline numbers): its B=1 BF16 forward replayed eagerly op by op over its compiled
    adapters (stage times), and single-op times of its cuBLASLt FP8 / BF16 linear layers and
    its three-launch cuBLAS MQA at the model's shapes. Ours: the same ops inside the B=1
    graphs' launch lists, each timed with a CUDA-event pair in one eager pass (ours carry
    their fused epilogues: bias, GELU, residual, GeGLU, quantisation). Needs oracle/_ref."""
    try:
        from oracle import ref_forward as R
        from oracle import pi05_oracle as O
        if not R.available():
            return {"unavailable": "oracle/_ref not built (make -C oracle with the reference tree present)"}
        cfg = O.Pi05Config()
        ref = R.RefBf16Forward(cfg, 0)
        inputs = O.synthetic_observation(cfg, 1234, 10)
        ref.infer(*inputs)  # warm-up: weight generation, cuBLAS heuristics
        runs = [ref.infer(*inputs, timed=True)[1] for _ in range(3)]
        ref.close()
        del ref
        import torch
        torch.cuda.empty_cache()
        stage = {k: float(np.median([r[k] for r in runs])) for k in ("vision", "prefix", "denoise")}
        gemms = R.time_gemms(MODEL_GEMMS)
        mqa = R.time_mqa(MODEL_ATTENTION)
        ours = ours_standalone_us(R.graph_time_us, R.weight_copies)
        table = {}
        for name, shape in MODEL_GEMMS.items():
            table[name] = {"mnk": list(shape), "ref_cublaslt_fp8_us": gemms[name].get("fp8_us"),
                           "ref_cublaslt_bf16_us": gemms[name].get("bf16_us"),
                           "ours_fp8_us": ours[name]["fp8_us"], "ours_bf16_us": ours[name]["bf16_us"],
                           "ours_fp8_in_graph_us": ours_fp8_us.get(name),
                           "ours_bf16_in_graph_us": ours_bf16_us.get(name)}
        for name, shape in MODEL_ATTENTION.items():
            table[name] = {"q_keys_heads_hd": list(shape), "ref_cublas_mqa_bf16_us": mqa[name]["us"],
                           "ours_bf16_us": ours[name]["bf16_us"],
                           "ours_fp8_in_graph_us": ours_fp8_us.get(name),
                           "ours_bf16_in_graph_us": ours_bf16_us.get(name)}
        return {"what": "reference CUDA kernels + cuBLAS(Lt) compiled for sm_100a from the reference tree, B=1",
                "bf16_b1_eager_stage_ms": {**stage, "total": sum(stage.values()), "launches": runs[0]["launches"]},
                "ours_bf16_b1_eager_stage_ms": ours_bf16_stage_ms,
                "per_op_us": table,
                "per_op_method": "ref_* and ours_*_us: 20 launches of the bare op captured into one CUDA graph, "
                                 "weights rotating through > L2 of copies, best of 5 replays / 20; "
                                 "ours_*_in_graph_us: the op inside the model's launch list with its fused "
                                 "epilogue, one CUDA-event pair per launch in an eager pass",
                "left_out": "CUTLASS sm100 FP8 GEMM / dual GeGLU / FMHA translation units: closed on this pool "
                            "(their tactics launch TMA multicast clusters)"}
    except Exception as error:  # the checker is optional equipment of the bench
        return {"unavailable": f"{type(error).__name__}: {error}"}


def ours_standalone_us(graph_time_us, weight_copies):
    """This library's kernels on the same bare problems and through the same timing harness as
    the reference's library calls: pi05_gemm (store epilogue, e4m3 -> bf16 and bf16 -> bf16)
    and pi05_attention (multi-query heads packed, key-split for the 10-token shape)."""
    import ctypes as C
    import torch
    from apxinf_b200 import _lib as L, kernels as K, lib
    results = {}
    partials = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")
    counters = torch.zeros(4096, dtype=torch.int32, device="cuda")
    status = K.new_status()
    for name, (m, n, k) in MODEL_GEMMS.items():
        entry = {}
        k_pad = (k + 15) // 16 * 16
        for label, dtype, op, elem in (("fp8", torch.float8_e4m3fn, L.OP_E4M3, 1), ("bf16", torch.bfloat16, L.OP_BF16, 2)):
            copies = weight_copies(n * k * elem)
            a = torch.zeros(m, k_pad, device="cuda").to(dtype)
            a[:, :k] = torch.randn(m, k, device="cuda").to(dtype)
            ws = []
            for _ in range(copies):
                w = torch.zeros(n, k_pad, device="cuda").to(dtype)
                w[:, :k] = torch.randn(n, k, device="cuda").to(dtype)
                ws.append(w)
            out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")

            def launch(i, a=a, ws=ws, out=out, op=op):
                K.gemm(a, ws[i % len(ws)], out, op=op, alpha=0.01, partials=partials, tile_counters=counters,
                       status=status)
            entry[label + "_us"] = graph_time_us(launch)
            del a, ws, out
        results[name] = entry
    handle = lib()

    class AttentionArgs(C.Structure):
        _fields_ = [("q", C.c_void_p), ("q_ld", C.c_int64), ("q_sb0", C.c_int64), ("q_sb1", C.c_int64),
                    ("k", C.c_void_p), ("k_ld", C.c_int64), ("k_sb0", C.c_int64), ("k_sb1", C.c_int64),
                    ("v", C.c_void_p), ("v_ld", C.c_int64), ("v_sb0", C.c_int64), ("v_sb1", C.c_int64),
                    ("out", C.c_void_p), ("out_ld", C.c_int64), ("out_sb0", C.c_int64), ("out_sb1", C.c_int64),
                    ("q_rows", C.c_int32), ("keys", C.c_int32), ("head_dim", C.c_int32),
                    ("nb0", C.c_int32), ("nb1", C.c_int32), ("scale", C.c_float),
                    ("out_e4m3", C.c_int32), ("out_inv_scale", C.c_float), ("status", C.c_void_p),
                    ("key_split", C.c_int32), ("split_scratch", C.c_void_p), ("split_scratch_bytes", C.c_int64)]
    handle.pi05_attention.argtypes = [C.POINTER(AttentionArgs), C.c_void_p]
    handle.pi05_attention.restype = C.c_int
    for name, (qt, kt, heads, hd) in MODEL_ATTENTION.items():
        q = torch.randn(qt, heads * hd, device="cuda").to(torch.bfloat16)
        kk = torch.randn(kt, hd, device="cuda").to(torch.bfloat16)
        vv = torch.randn(kt, hd, device="cuda").to(torch.bfloat16)
        out = torch.empty(qt, heads * hd, dtype=torch.bfloat16, device="cuda")
        args = AttentionArgs(q=q.data_ptr(), q_ld=heads * hd, q_sb0=hd, q_sb1=0, k=kk.data_ptr(), k_ld=hd,
                             v=vv.data_ptr(), v_ld=hd, out=out.data_ptr(), out_ld=heads * hd, out_sb0=hd,
                             q_rows=qt, keys=kt, head_dim=hd, nb0=heads, nb1=1, scale=1.0 / 16.0,
                             out_inv_scale=1.0, status=status.data_ptr(), key_split=int(qt * heads <= 128 * 31),
                             split_scratch=partials.data_ptr(), split_scratch_bytes=partials.numel())
        if qt * heads > 1024:
            args.key_split = 0

        def launch(i):
            rc = handle.pi05_attention(C.byref(args), C.c_void_p(torch.cuda.current_stream().cuda_stream))
            if rc != 0:
                raise RuntimeError(f"pi05_attention status {rc}")
        results[name] = {"bf16_us": graph_time_us(launch)}
    return results


def measure_latency(rt_dtype, device, per_op=False):
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
    op_us = {}
    if per_op:
        for name in list(MODEL_GEMMS) + ["vision.attn"] + list(MODEL_ATTENTION):
            mean_ms, count = graph.time_launches(name)
            if count > 0:
                op_us[name] = mean_ms * 1e3
    result = {"workload": f"cfg{dict(bf16=2, fp8=3, int8=3)[rt_dtype]}: {rt_dtype.upper()}, B=1, 2 views, 10 tokens, H=10, 10 flow steps",
              "p50_ms": float(ms[len(ms) // 2]), "p95_ms": float(ms[int(round(0.95 * (len(ms) - 1)))]),
              "min_ms": float(ms[0]), "max_ms": float(ms[-1]),
              "input_update_plus_graph_ms": update_plus_graph, "launches": graph.num_launches(),
              "stage_ms_eager": stages, "finite": bool(np.isfinite(out).all())}
    if per_op:
        result["op_us"] = op_us
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
    parser.add_argument("--no-ref-cuda", action="store_true",
                        help="skip the reference-CUDA comparison leg (needs oracle/_ref)")
    parser.add_argument("--no-complete-forward", action="store_true",
                        help="reference arm: skip the one complete CPU forward")
    parser.add_argument("--complete-forward-budget", type=float, default=150.0,
                        help="reference arm: seconds of weight generation allowed for the complete forward")
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
