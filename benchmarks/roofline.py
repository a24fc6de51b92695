#!/usr/bin/env python
"""Runs the single-kernel workloads of ``kernel_bench.py`` that matter for the flagship decode step and prints, per kernel,
the CUDA-event time and the achieved fraction of the measured peaks (``MEASURED_PEAKS.json``: HBM copy bandwidth and
cuBLAS bf16 throughput).  One GPU.

    python benchmarks/roofline.py            # table on stdout, JSON lines in benchmarks/roofline_last.jsonl
"""
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [
    ("MLA decode, 512 rows x 2048 ctx", ["mla_decode", "--bq", "512", "--ctx", "2048"]),
    ("q_b proj fp8 512x24576x1536", ["gemm", "--kind", "fp8", "--t", "512", "--n", "24576", "--k", "1536"]),
    ("o_proj fp8 512x7168x16384", ["gemm", "--kind", "fp8", "--t", "512", "--n", "7168", "--k", "16384"]),
    ("experts gate/up fp8 32x128 tok, SwiGLU+quant", ["grouped", "--kind", "fp8", "--epi", "swiglu_quant", "--n", "2048", "--k", "7168",
                                                      "--tokens-per-expert", "128"]),
    ("experts down fp8 32x128 tok", ["grouped", "--kind", "fp8", "--epi", "store", "--n", "7168", "--k", "2048", "--tokens-per-expert", "128"]),
    ("W_UK per-head bf16 512x128x(128->512)", ["bmm", "--t", "512", "--n", "512", "--k", "128"]),
    ("lm_head bf16 512x129280x7168", ["gemm", "--kind", "bf16", "--t", "512", "--n", "129280", "--k", "7168"]),
    ("MLA prefill FMHA 4096 tokens", ["fmha", "--ctx", "4096"]),
]


def main():
    rows = []
    for name, argv in CASES:
        r = subprocess.run([sys.executable, os.path.join(HERE, "kernel_bench.py")] + argv, capture_output=True, text=True)
        line = [l for l in r.stdout.splitlines() if l.startswith("{")]
        if r.returncode != 0 or not line:
            rows.append((name, None))
            continue
        rows.append((name, json.loads(line[-1])))
    with open(os.path.join(HERE, "roofline_last.jsonl"), "w") as f:
        for name, d in rows:
            f.write(json.dumps({"case": name, **(d or {"failed": True})}) + "\n")
    print(f"{'kernel / shape':52s} {'us':>9s} {'TB/s':>7s} {'of HBM':>7s} {'TFLOP/s':>9s} {'of bf16':>8s}")
    for name, d in rows:
        if d is None:
            print(f"{name:52s} failed")
            continue
        print(f"{name:52s} {d['us']:9.1f} {d['GB/s'] / 1e3:7.2f} {d['frac_hbm_of_measured']:7.2f} {d['TFLOP/s']:9.1f} "
              f"{d['frac_bf16_peak_of_measured']:8.2f}")


if __name__ == "__main__":
    main()
