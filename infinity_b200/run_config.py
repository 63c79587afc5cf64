"""Runs one of the five named configurations at full size on the GPU(s) and prints one JSON line
with tokens/s, step times and the per-kernel-class breakdown:

    python -m infinity_b200.run_config c3 --steps 3 [--devices 0,1] [--seqs N] [--layers L]
    python -m infinity_b200.run_config c2 --cuts 32        # batch latency: count cut vs token-budget cut

The line carries the git commit of the checkout (when git is present) and the SM clock sampled
with nvidia-smi while the timed forwards ran. ``--cuts SIZE`` splits the configuration's batch the
way a batcher would, once every SIZE sequences of the length-sorted list (the reference's cut,
infinity_emb/inference/queue.py:57-76) and once at the token budget that gives the same number of
batches, runs every batch as its own forward and reports the spread of the batch latencies.

Weights are seeded random-init (block formats are produced from the bf16 file by the CUDA
quantisers), inputs are the configuration's seeded synthetic batch. This is a measurement
helper; correctness is covered by the tests.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import tempfile
import time
from dataclasses import replace

import numpy as np
import torch

from . import batching as bt
from . import configs as cf
from . import weights as wt
from .clocks import ClockSampler
from .engine import B200Model


def git_commit() -> str:
    """The commit the loaded library was built from (recorded by the build), else the checkout's."""
    from . import build as b
    stamp = b.LIB_DIR / "commit.txt"
    if stamp.exists() and b.is_current():
        return stamp.read_text().strip()
    return b.source_commit()


def cut_latencies(model: B200Model, batch, size: int, repeats: int = 3) -> dict:
    """Per-batch latency (host clock around the forward call, host buffers) of the two cuts of one batch."""
    seqs = batch.sequences()
    lengths = [len(x) for x in seqs]
    by_count = bt.count_batches(lengths, size, sort=True)
    budget = int(np.ceil(sum(lengths) / len(by_count)))
    by_tokens = bt.token_budget_batches(lengths, budget)
    out = {"sequences_per_count_batch": size, "token_budget": budget}
    for name, cuts in (("count", by_count), ("tokens", by_tokens)):
        packed = [cf.pack([seqs[i] for i in idx]) for idx in cuts]
        for b in packed[:: max(1, len(packed) // 8)]:
            model.forward(b)  # warm-up over the range of sizes
        ms = []
        for _ in range(repeats):
            for b in packed:
                t0 = time.perf_counter()
                model.forward(b)
                ms.append((time.perf_counter() - t0) * 1e3)
        ms_sorted = np.sort(np.array(ms))
        out[name] = {"batches": len(cuts), "tokens_per_batch_min_max": [min(b.n_tokens for b in packed), max(b.n_tokens for b in packed)],
                     "latency_ms_p50": float(np.percentile(ms_sorted, 50)), "latency_ms_p99": float(np.percentile(ms_sorted, 99)),
                     "latency_ms_max": float(ms_sorted[-1]), "total_ms_per_pass": float(sum(ms) / repeats)}
    return out


def gemm_flops_per_token(spec) -> float:
    H, F = spec.hidden, spec.ffn
    qkv = (spec.n_heads + 2 * spec.n_kv_heads) * spec.head_dim
    total = 0.0
    for l in range(spec.n_layers):
        total += 2.0 * H * qkv + 2.0 * H * spec.n_heads * spec.head_dim
        if spec.arch == "decoder":
            total += 6.0 * H * F
        elif cf.is_moe_layer(spec, l):
            total += spec.top_k * 4.0 * H * F + 2.0 * H * spec.n_experts
        else:
            total += 4.0 * H * F
    return total


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", choices=sorted(cf.SPECS))
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--devices", default="0")
    ap.add_argument("--seqs", type=int, default=None, help="number of sequences (default: the configuration's)")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (for quick runs)")
    ap.add_argument("--keep", default=None, help="directory for the weight files (default: a temporary one)")
    ap.add_argument("--cuts", type=int, default=0, help="compare count-cut and token-cut batches of this many sequences")
    a = ap.parse_args()
    spec = cf.SPECS[a.config]
    if a.layers:
        spec = replace(spec, n_layers=a.layers)
    devices = tuple(int(x) for x in a.devices.split(","))
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    workdir = a.keep or tempfile.mkdtemp(prefix="b200emb_cfg_")
    path = os.path.join(workdir, f"{a.config}.b2ew")
    master = cf.init_weights(spec, cf.SEEDS[a.config][2])
    tensors = cf.runtime_tensors(master)
    del master
    wt.save_weights(path, tensors)
    n_params = sum(v.numel() for v in tensors.values())
    del tensors
    if spec.weight_format != "bf16":
        qpath = os.path.join(workdir, f"{a.config}.{spec.weight_format}.b2ew")
        wt.quantize_weight_file(path, qpath, spec.weight_format, devices[0])
        os.remove(path)
        path = qpath
    t_weights = time.perf_counter() - t0
    batch = cf.synth_batch(a.config, a.seqs)
    model = B200Model(spec, path, devices, max_tokens=batch.n_tokens if len(devices) == 1 else 0)
    if a.cuts > 0:
        line = {"config": a.config, "model": spec.name, "commit": git_commit(), "sequences": batch.n_seqs,
                "tokens": batch.n_tokens, "batch_cuts": cut_latencies(model, batch, a.cuts)}
        print(json.dumps(line), flush=True)
        model.close()
        if not a.keep:
            os.remove(path)
        return
    for _ in range(a.warmup):
        model.forward(batch)
    times, kern = [], []
    sampler = ClockSampler(devices[0])
    sampler.start()
    for _ in range(a.steps):
        t1 = time.perf_counter()
        out = model.forward(batch)
        times.append((time.perf_counter() - t1) * 1e3)
        kern.append(model.last_timing["kernels_ms"])
    clocks = sampler.stop()
    model.forward(batch, per_kernel=True)
    prof = model.last_timing
    att = float((batch.lengths.astype(np.float64) ** 2).sum()) * spec.hidden * spec.n_layers * (2.0 if spec.arch == "decoder" else 4.0)
    gemm = gemm_flops_per_token(spec) * batch.n_tokens
    ms = statistics.median(times)
    line = {
        "config": a.config, "commit": git_commit(), "clocks": clocks, "model": spec.name, "weight_format": spec.weight_format, "n_devices": len(devices),
        "layers": spec.n_layers, "parameters": n_params, "sequences": batch.n_seqs, "tokens": batch.n_tokens,
        "ms_per_forward_p50": ms, "kernels_ms_p50": statistics.median(kern), "tokens_per_s": batch.n_tokens / ms * 1e3,
        "algorithmic_tflop": (gemm + att) / 1e12, "tflops_achieved": (gemm + att) / ms / 1e9,
        "kernel_class_ms": prof["kclass_ms"], "kernel_launches": prof["launches"],
        "output_shape": list(out.shape), "finite": bool(np.isfinite(out).all()),
        "weights_prepared_s": round(t_weights, 1), "file_bytes": os.path.getsize(path),
    }
    print(json.dumps(line), flush=True)
    model.close()
    if not a.keep:
        os.remove(path)


if __name__ == "__main__":
    main()
