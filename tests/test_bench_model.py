"""The byte and flop counts that bench.py's roofline fractions rest on, against figures worked out
by hand for the Qwen2.5-0.5B layer sizes, and the command line's refusals."""
import json
import subprocess
import sys

import bench
from helpers import ROOT


def test_decode_bytes_and_prefill_flops_of_the_headline_shape():
    cfg = bench.QWEN25_05B
    # weights: 24 layers x 14.91 M parameters + the 136.1 M of the head, two bytes each = 988.1 MB;
    # cache: 12,288 bytes per token of context and request.
    assert abs(bench.decode_bytes(cfg, 24, 1, 0) - 988.1e6) < 0.1e6
    for batch, want in ((1, 996e6), (8, 1051e6), (64, 1491e6)):
        assert abs(bench.decode_bytes(cfg, 24, batch, 640) - want) < 1e6
    assert bench.decode_bytes(cfg, 24, 8, 641) - bench.decode_bytes(cfg, 24, 8, 640) == 8 * 12288
    # 1.466 TFLOP in the products and 0.181 in attention (causal: every query meets the keys up to its own)
    assert abs(bench.prefill_flops(cfg, 24, 2048) - 1.646e12) < 0.002e12


def test_more_than_one_gpu_is_refused_and_the_reference_arm_says_why():
    many = subprocess.run([sys.executable, "bench.py", "--gpus", "2"], cwd=ROOT, capture_output=True, text=True)
    assert many.returncode == 2 and json.loads(many.stdout.strip().splitlines()[-1])["n_gpus"] == 2
    ref = subprocess.run([sys.executable, "bench.py", "--impl", "reference"], cwd=ROOT, capture_output=True, text=True)
    line = json.loads(ref.stdout.strip().splitlines()[-1])
    assert ref.returncode == 0 and line["impl"] == "reference" and "unavailable" in line
