"""pi05_bench CLI: flag validation mirrors the reference (crates/apxinf-model/examples/
pi05_bench.rs:804-862); on a GPU it prints the reference's JSON report keys."""
import json
import subprocess
from pathlib import Path

import pytest

EXE = Path(__file__).resolve().parent.parent / "apxinf_b200" / "pi05_bench"


def _run(*args):
    return subprocess.run([str(EXE), *args], capture_output=True, text=True, timeout=600)


def test_flag_validation_messages():
    assert EXE.exists(), "run `python -m apxinf_b200.build`"
    r = _run("random", "--dtype", "fp4")
    assert r.returncode == 1 and "--dtype must be bf16, fp8, or int8; got fp4" in r.stderr
    r = _run("model.safetensors", "--dtype", "bf16", "--views", "3")
    assert r.returncode == 1 and "only valid with the `random` source" in r.stderr
    r = _run("random", "--dtype", "bf16", "--calibration", "uniform:0.05")
    assert "--calibration only applies to --dtype fp8" in r.stderr
    r = _run("random", "--dtype", "int8", "--tactics", "t.json")
    assert "--tactics only applies to --dtype bf16 or fp8" in r.stderr
    r = _run("random", "--dtype", "fp8", "--reference", "ref.json")
    assert "--reference is not valid with the `random` source" in r.stderr
    r = _run("random", "--dtype", "fp8", "--image-input", "hwc")
    assert "image input must be patches, nhwc, or nchw; got hwc" in r.stderr
    r = _run("random", "--dtype", "fp8", "--token-count", "500")
    assert "token count must be in 1..=200, got 500" in r.stderr
    r = _run("random", "--dtype", "fp8", "--images-u8", "x.raw")
    assert "--images-u8 requires --image-input nhwc" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bf16", "fp8", "w8a8"])
def test_report_has_the_reference_keys(dtype):
    extra = ["--calibration", "uniform:0.05"] if dtype == "fp8" else []
    r = _run("random", "--dtype", dtype, "--views", "1", "--token-count", "8", "--iterations", "3",
             "--image-input", "nhwc", "--num-flow-steps", "2", *extra)
    assert r.returncode == 0, r.stderr[-2000:]
    report = json.loads(r.stdout)
    assert report["profile"] == "pi05_1view_h10_steps2"
    assert report["precision"] == {"bf16": "bf16", "fp8": "fp8", "w8a8": "int8_w8a8"}[dtype]
    assert report["weights"] == "synthetic" and report["token_count"] == 8 and report["iterations"] == 3
    assert set(report["latency_ms"]) == {"min", "p50", "p95", "max", "mean", "standard_deviation"}
    assert set(report["image_input"]) == {"kind", "graph_includes_cuda_preprocess",
                                          "graph_latency_includes_h2d",
                                          "input_update_plus_graph_latency_ms"}
    assert report["image_input"]["input_update_plus_graph_latency_ms"]["p50"] > 0
    assert report["workspace"]["used_bytes"] <= report["workspace"]["capacity_bytes"]
    assert report["integrity"]["passed"] and report["integrity"]["eager_vs_graph"]["bitwise_equal"]
    assert report["output_abs_checksum"] > 0
