#!/usr/bin/env python
"""Benchmark of the DF11 -> BF16 decompression path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One *step* decompresses every compressed unit of a model once, in forward order, into one
reused BF16 buffer -- what one forward pass of the model triggers.  The default workload is
the Qwen3-8B-shaped model of the baseline configuration (36 transformer blocks of
192 937 984 elements plus two 622 329 856-element vocabulary matrices; weights N(0, 0.02),
embeddings N(0, 1), seeded, synthetic).  Rank r of N uses seed 1 + r and decodes its own
full copy (weak scaling, no data-path collective).

The JSON line printed by rank 0 reports
  value      algorithmic GB/s over all GPUs, inputs resident in HBM, CUDA-event timed;
             algorithmic bytes = compressed bytes read + 2 bytes written per element
  e2e        the same metric with the two large compressed tensors of every unit coming
             from pinned host memory each step (the `cpu_offload` path: host->device copies
             on a side stream overlapped with the previous unit's decode) and a small
             device->host read of the result at the end of the step
  roofline   the decode kernel against the measured HBM copy bandwidth
  cpu_baseline / --impl reference
             the CPU restatement of the reference's decode rule (oracle/) on the host cores
             (the reference has no CPU decoder of its own), on a bounded sample
  reference_gpu_kernel
             the reference's own CUDA kernel (its shipped PTX, loaded unmodified) timed on
             one transformer-block unit on the same GPU
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(name="qwen3-8b-shape", layers=36, hidden=4096, kv=1024, inter=12288, vocab=151936)
LLAMA_8B = dict(name="llama3.1-8b-shape", layers=32, hidden=4096, kv=1024, inter=14336, vocab=128256)
SMALL = dict(name="small-smoke", layers=2, hidden=1024, kv=256, inter=3072, vocab=8192)
ONE_BLOCK = dict(name="one-llama-block", layers=1, hidden=4096, kv=1024, inter=14336, vocab=0)
ONE_QWEN_BLOCK = dict(name="one-qwen3-block", layers=1, hidden=4096, kv=1024, inter=12288, vocab=0)
# Llama-3.1-405B shapes, tensor-parallel over the ranks of the job: every rank holds 1/T of each
# block's seven matrices as one unit and decodes only that; two activation all-reduces per layer.
LLAMA_405B_TP = dict(name="llama3.1-405b-shape-tp", layers=126, hidden=16384, kv=1024, inter=53248, vocab=0, tp=True)
# FLUX.1-dev-shaped diffusion transformer (hidden 3072, MLP ratio 4): 19 double-stream units of 14
# matrices (339.7 M weights) and 38 single-stream units of 6 matrices (141.6 M); one pass over all
# 57 units is the weight decode of one denoising step.
FLUX_DIT = dict(name="flux1-dev-shape", layers=57, hidden=3072, kv=3072, inter=12288, vocab=0,
                unit_sizes=[2 * 3072 * 18432 + 8 * 3072 * 3072 + 4 * 3072 * 12288] * 19
                + [3072 * 9216 + 3072 * 12288 + 15360 * 3072 + 3 * 3072 * 3072] * 38)
WORKLOADS = {"flux-dit": FLUX_DIT, "qwen3-8b": QWEN3_8B, "llama-8b": LLAMA_8B, "small": SMALL, "block": ONE_BLOCK, "qwen3-block": ONE_QWEN_BLOCK,
             "llama-405b-tp": LLAMA_405B_TP}


# DRAM bytes per element of one df11_fast_kernel launch on a 192.9 M-element Qwen3-8B block unit,
# from the ncu capture summarised in profiles/df11_fast_kernel_one_qwen3_block.md, by seek interval.
DRAM_BYTES_PER_ELEMENT = {16: 3.190, 32: 3.144}


def block_shapes(cfg):
    h, kv, it = cfg["hidden"], cfg["kv"], cfg["inter"]
    return [(h, h), (kv, h), (kv, h), (h, h), (it, h), (it, h), (h, it)]


def unit_plan(cfg):
    """(name, n_elements, std) of every compressed unit in forward order."""
    if cfg.get("unit_sizes"):
        return [(f"layers.{i}", n, 0.02) for i, n in enumerate(cfg["unit_sizes"])]
    n_block = sum(a * b for a, b in block_shapes(cfg))
    plan = [(f"layers.{i}", n_block, 0.02) for i in range(cfg["layers"])]
    if cfg["vocab"]:
        plan = [("embed_tokens", cfg["vocab"] * cfg["hidden"], 1.0)] + plan
        plan.append(("lm_head", cfg["vocab"] * cfg["hidden"], 0.02))
    return plan


def algorithmic_bytes(unit) -> int:
    """Compressed bytes read + BF16 bytes written for one decode of `unit`."""
    return (unit["n_bytes"] + unit["n_elements"] + unit["gaps"].numel() + unit["pos"].numel()
            + unit["luts"].numel() + 2 * unit["n_elements"])


def make_unit(n_elements, std, seed, device, keep_host=False, n_threads=None, keep_weights=False):
    """Synthesise one unit on the GPU, compress it (native host packer), put it in HBM."""
    from dfloat11_b200 import codec
    g = torch.Generator(device=device).manual_seed(seed)
    w = torch.empty(n_elements, dtype=torch.bfloat16, device=device)
    chunk = 1 << 26
    for s in range(0, n_elements, chunk):      # float32 staging in slices keeps peak memory low
        e = min(n_elements, s + chunk)
        w[s:e] = (torch.randn(e - s, generator=g, device=device) * std).to(torch.bfloat16)
    exponent, sign_mantissa = codec.split_bf16(w)
    hist = codec.exponent_histogram(exponent)
    lens = codec.code_lengths(hist)
    vals = codec.canonical_codes(lens)
    luts = codec.build_luts(lens, vals)
    enc_d, gaps_d, pos_d = codec.pack_exponents_gpu(exponent, lens, vals)      # the package's GPU bit packer
    del exponent
    positions = pos_d.cpu().numpy().view(np.uint32)
    unit = dict(
        luts=torch.from_numpy(luts).to(device), enc=enc_d, sm=sign_mantissa, pos=pos_d.view(torch.uint8),
        gaps=gaps_d, n_elements=n_elements, n_bytes=int(enc_d.numel()),
        widest=int(np.diff(positions.astype(np.int64)).max()),
        checksum=int(w.view(torch.int16).to(torch.int64).sum().item()),
    )
    if keep_host:
        unit["host"] = dict(luts=luts, enc=enc_d.cpu().numpy(), sm=sign_mantissa.cpu().numpy(), pos=positions,
                            gaps=gaps_d.cpu().numpy())
    if keep_weights:
        unit["weights"] = w
    return unit


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001 - clocks are advisory
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])), mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:  # noqa: BLE001
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons),
                       samples=len(sm))
        return out


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, stream copy)"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback (no MEASURED_PEAKS.json beside bench.py)"


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def all_max(value, world, device):
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_sum(value, world, device):
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def barrier(world, device):
    if world > 1:
        import torch.distributed as dist
        dist.barrier(device_ids=[device.index])
    torch.cuda.synchronize(device)


def time_reference_gpu_kernel(unit, scratch, iters=100, warmup=20):
    """The reference's shipped PTX on one unit: ms per launch, bit-compared with the new kernel."""
    from oracle import ref_kernel
    from dfloat11_b200 import ops
    if not ref_kernel.available("shipped_ptx"):
        return {"unavailable": "oracle/_ref/decode_shipped.ptx not built"}
    if unit["n_elements"] >= 2 ** 31:
        return {"unavailable": "unit exceeds the reference kernel's 32-bit sizes"}
    out = {}
    n = unit["n_elements"]
    mine = ops.decode(unit["luts"], unit["enc"], unit["sm"], unit["pos"], unit["gaps"],
                      max_block_elems=unit["widest"]).clone()
    smem = 512 * 4 + 4 + 2 * unit["widest"]
    for variant in ("shipped_ptx", "recompiled_sm100a"):
        if not ref_kernel.available(variant):
            continue
        buf = scratch[:n]
        for _ in range(warmup):
            ref_kernel.decode(unit["luts"], unit["enc"], unit["sm"], unit["pos"], unit["gaps"], buf, smem, variant)
        torch.cuda.synchronize()
        same = bool(torch.equal(buf.view(torch.int16), mine.view(torch.int16)))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            ref_kernel.decode(unit["luts"], unit["enc"], unit["sm"], unit["pos"], unit["gaps"], buf, smem, variant)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / iters
        out[variant] = {"ms_per_launch": round(ms, 4), "GBps": round(algorithmic_bytes(unit) / ms / 1e6, 1),
                        "bit_identical_to_ours": same, "warmup": warmup, "launches": iters}
    out["unit"] = f"{n} elements"
    return out


def cpu_decode_sample(host, n_threads, repeats, warmup=0):
    """Times the oracle's C decoder on host tensors; returns (mean seconds per decode over
    `repeats` runs after `warmup` untimed ones, out checksum)."""
    from oracle import df11_oracle as oracle
    out = host.get("_out")
    if out is None:                       # one output buffer, touched once: no page faults in the timings
        out = host["_out"] = np.ones(host["sm"].size, dtype=np.uint16)
    times = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        oracle.decode_c(host["luts"], host["enc"], host["sm"], host["pos"], host["gaps"],
                        n_threads=n_threads, strict=False, out=out)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return sum(times) / len(times), int(out.view(np.int16).astype(np.int64).sum())


_HOST_UNIT_SCRIPT = r"""
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
from dfloat11_b200 import codec
n, seed, threads, out = int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
g = torch.Generator().manual_seed(seed)
w = torch.empty(n, dtype=torch.bfloat16)
for s in range(0, n, 1 << 24):
    e = min(n, s + (1 << 24))
    w[s:e] = (torch.randn(e - s, generator=g) * 0.02).to(torch.bfloat16)
t = codec.encode_weights([w], n_threads=threads)
np.savez(out, luts=t["luts"].numpy(), enc=t["encoded_exponent"].numpy(), sm=t["sign_mantissa"].numpy(),
         pos=t["output_positions"].numpy().view(np.uint32), gaps=t["gaps"].numpy(),
         checksum=np.int64(w.view(torch.int16).numpy().astype(np.int64).sum()))
"""


def host_unit_from_subprocess(n, seed, threads):
    """One compressed unit as host arrays, made by a child process: the process that times the CPU
    decoder then never loads the package's native library, only the oracle's."""
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "unit.npz")
        subprocess.run([sys.executable, "-c", _HOST_UNIT_SCRIPT, ROOT, str(n), str(seed), str(threads), path],
                       check=True, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
        with np.load(path) as z:
            return {k: z[k].copy() for k in z.files}


def cpu_compress_sample(n=1 << 24, seed=5):
    """The reference's CPU compression rate (its per-symbol Python bit packer,
    dfloat11_utils.py:118-170,173-187, restated in oracle/): elements per second on one core,
    on `n` exponents of N(0, 0.02) weights, with the package's packers beside it."""
    from oracle import df11_oracle as oracle
    from dfloat11_b200 import codec
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16)
    exponent, _ = codec.split_bf16(w)
    lens = codec.code_lengths(codec.exponent_histogram(exponent))
    vals = codec.canonical_codes(lens)
    symbols = exponent.numpy().tolist()                 # as the reference does (`exponent_8bits.tolist()`)
    t0 = time.perf_counter()
    enc, gaps, pos = oracle.encode_stream_py(symbols, lens, vals, 0, 0)
    t_py = time.perf_counter() - t0
    t0 = time.perf_counter()
    enc_h, gaps_h, pos_h = codec.pack_exponents(exponent.numpy(), lens, vals)
    t_host = time.perf_counter() - t0
    out = {"value": round(n / t_py / 1e6, 3), "unit": "M elements/s", "cores": 1, "kind": "port",
           "sample": f"{n} exponents of N(0, 0.02) BF16 weights, per-symbol Python bit packer (one pass)",
           "host_packer_M_elements_per_s": round(n / t_host / 1e6, 1),
           "byte_identical": bool(np.array_equal(enc, np.asarray(enc_h)) and np.array_equal(gaps, np.asarray(gaps_h))
                                  and np.array_equal(pos, np.asarray(pos_h).view(np.uint32)))}
    if torch.cuda.is_available():
        dev_e = exponent.to("cuda")
        codec.pack_exponents_gpu(dev_e, lens, vals)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        codec.pack_exponents_gpu(dev_e, lens, vals)
        torch.cuda.synchronize()
        out["gpu_packer_M_elements_per_s"] = round(n / (time.perf_counter() - t0) / 1e6, 1)
    return out


def run_reference_arm(args, cfg):
    """--impl reference: the CPU decode (oracle port; the reference ships no CPU decoder) on all
    host threads.  The unit it decodes is made by a child process, so this process loads the
    oracle's library only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import df11_oracle as oracle
    oracle.build()
    cores = oracle.max_threads()
    n = sum(a * b for a, b in block_shapes(cfg))
    host = host_unit_from_subprocess(n, 1, cores)
    torch.set_num_threads(1)              # torch's worker threads must not compete with the decoder's
    nbytes = (host["enc"].size + n + host["gaps"].size + host["pos"].size * 4 + host["luts"].size + 2 * n)
    dt, checksum = cpu_decode_sample(host, cores, repeats=args.steps, warmup=args.warmup)   # the decode alone is timed
    assert checksum == int(host["checksum"]), "CPU decode is not bit-exact"
    gbps = nbytes / dt / 1e9
    sample = f"one transformer-block unit of {cfg['name']} ({n} elements) per step, {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": "df11_bf16_decompress_GBps", "value": round(gbps, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8/u16 integer",
        "data": "synthetic", "config": {"workload": cfg["name"], "sample": sample},
        "cpu_baseline": {"value": round(gbps, 3), "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample,
                         "statistic": f"mean of {args.steps} decodes after {args.warmup} untimed"},
        "e2e": {"value": round(gbps, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen3-8b", choices=sorted(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--batch", type=int, default=1, help="activation rows all-reduced per layer (TP workload)")
    ap.add_argument("--skip-extras", action="store_true", help="no CPU baseline / reference-kernel / e2e legs")
    ap.add_argument("--generation", action="store_true",
                    help="only: batch-1 greedy generation, DF11 vs uncompressed BF16, on the workload's model shape")
    ap.add_argument("--fused-gemv", action="store_true",
                    help="only: the matrix-vector products of one block at batch 1, fused with the decode "
                         "(df11_gemv_prepared) against decode-then-torch GEMV")
    ap.add_argument("--kernel-times", action="store_true",
                    help="with --generation: also sum the GPU kernel time per token with the torch profiler; run it "
                         "separately, the profiler leaves a per-launch cost behind that slows the eager legs after it")
    ap.add_argument("--cpu-offload", action="store_true",
                    help="with --generation: DF11 with cpu_offload=True at --batch sequences against resident BF16")
    ap.add_argument("--dit-step", action="store_true",
                    help="only: one denoising step of the FLUX.1-dev-shaped transformer, DF11 against BF16")
    ap.add_argument("--loader", action="store_true",
                    help="only: seconds to load a saved DF11 model (--layers blocks of the workload's shape) with this "
                         "package's loader and the reference's way")
    ap.add_argument("--slab-pipeline", action="store_true",
                    help="only: one block's batch-1 products with the weights decompressed slab by slab right "
                         "before each product (L2-resident) against decode-the-whole-block")
    ap.add_argument("--eager", action="store_true",
                    help="with --slab-pipeline: one untimed pass of each variant without CUDA graphs, for a profiler")
    ap.add_argument("--layers", type=int, default=0,
                    help="with --generation on the partitioned workload: transformer layers to build (0 = as many as fit)")
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--prompt-tokens", type=int, default=64)
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference_arm(args, cfg)
        return
    if args.generation and cfg.get("tp"):
        run_tp_generation(args, cfg)
        return
    if args.generation:
        run_generation(args, cfg)
        return
    if args.fused_gemv:
        run_fused_gemv(args, cfg)
        return
    if args.dit_step:
        run_dit_step(args)
        return
    if args.loader:
        run_loader(args, cfg)
        return
    if args.slab_pipeline:
        run_slab_pipeline(args, cfg)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    from dfloat11_b200 import ops

    rank, world, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)

    # ---- build the workload in HBM --------------------------------------------------------
    t_setup = time.time()
    plan = unit_plan(cfg)
    units = []
    activations = None
    if cfg.get("tp"):
        # One block-shard per rank (1/world of the block's elements; shards of i.i.d. weights are
        # i.i.d.), compressed once and cloned for the other layers: same traffic, distinct
        # allocations, far larger than L2.  As many of the 126 layers as fit in 150 GB.
        n_shard = plan[0][1] // world
        first = make_unit(n_shard, 0.02, seed=1000 * (1 + rank), device=device, keep_host=(rank == 0))
        per_layer = first["n_bytes"] + first["n_elements"] + first["n_elements"] // 7
        layers = int(min(cfg["layers"], (150e9 - 2 * n_shard) // per_layer))
        units = [first] + [dict(first, enc=first["enc"].clone(), sm=first["sm"].clone(),
                                pos=first["pos"].clone(), gaps=first["gaps"].clone()) for _ in range(layers - 1)]
        plan = [(f"layers.{i}", n_shard, 0.02) for i in range(layers)]
        activations = torch.zeros(args.batch, cfg["hidden"], dtype=torch.bfloat16, device=device)
    else:
        for i, (name, n, std) in enumerate(plan):
            keep = (name == "layers.0" and rank == 0)   # the first transformer block also feeds the CPU baseline
            units.append(make_unit(n, std, seed=1000 * (1 + rank) + i, device=device, keep_host=keep))
    scratch = torch.empty(max(u["n_elements"] for u in units), dtype=torch.bfloat16, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    for u in units:   # once per unit, at load time
        u["aux"] = ops.prepare(u["luts"], u["enc"], u["pos"], u["gaps"], u["n_elements"], status=status)
    torch.cuda.synchronize()
    setup_s = time.time() - t_setup

    def step(prepared=True):
        for u in units:
            out = scratch[:u["n_elements"]]
            if prepared:
                ops.decode_prepared(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], u["aux"], out=out,
                                    max_block_elems=u["widest"], status=status)
            else:
                ops.decode(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], out=out,
                           max_block_elems=u["widest"], status=status)
            if activations is not None and world > 1:
                import torch.distributed as dist
                dist.all_reduce(activations)       # after o_proj
                dist.all_reduce(activations)       # after down_proj

    # parity inside the bench: every unit's decode must reproduce its original checksum
    for u in units:
        for prepared in (True, False):
            out = scratch[:u["n_elements"]]
            out.zero_()
            if prepared:
                ops.decode_prepared(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], u["aux"], out=out,
                                    max_block_elems=u["widest"], status=status)
            else:
                ops.decode(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], out=out,
                           max_block_elems=u["widest"], status=status)
            got = int(out.view(torch.int16).to(torch.int64).sum().item())
            if got != u["checksum"] or status.item() != 0:
                raise SystemExit(f"decode mismatch on rank {rank} (prepared={prepared}, status={status.item()})")

    step_bytes = sum(algorithmic_bytes(u) for u in units)
    step_elems = sum(u["n_elements"] for u in units)

    step_spread = {}

    def timed(fn, steps, warmup, spread_key=None):
        for _ in range(warmup):
            fn()
        barrier(world, device)
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        marks[0].record()
        for i in range(steps):
            fn()
            marks[i + 1].record()
        barrier(world, device)
        if spread_key:                                  # per-step times on this rank, for median and min
            per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
            step_spread[spread_key] = {"min": round(per_step[0], 4), "median": round(per_step[len(per_step) // 2], 4),
                                       "max": round(per_step[-1], 4)}
        return all_max(marks[0].elapsed_time(marks[-1]) / steps, world, device)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(lambda: step(True), args.steps, args.warmup, spread_key="prepared")
    clocks = sampler.stop() if rank == 0 else None
    ms_two_pass = timed(lambda: step(False), max(1, args.steps // 2), max(3, args.warmup))
    total_bytes = all_sum(step_bytes, world, device)
    value = total_bytes / ms / 1e6                      # GB/s over all ranks

    # ---- e2e: compressed tensors come from pinned host memory every step --------------------
    e2e = None
    if not args.skip_extras:
        e2e = run_e2e(units, scratch, status, device, world, args)

    result = {
        "metric": "df11_bf16_decompress_GBps", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "ms_per_step_spread": step_spread.get("prepared"),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8/u16 integer",
        "data": "synthetic",
        "config": {
            "workload": cfg["name"], "units_per_step": len(units), "elements_per_step": step_elems,
            "algorithmic_bytes_per_step": step_bytes, "bytes_per_element": round(step_bytes / step_elems, 4),
            "path": "df11_decode_prepared", "l2": f"inputs larger than L2 (every unit >= {min(algorithmic_bytes(u) for u in units) // 10**6} MB of traffic)",
            "per_gpu_GBps": round(value / world, 1), "setup_s": round(setup_s, 1),
            **({"parallelism": f"tp{world}", "layers_resident": len(units), "all_reduces_per_step": 2 * len(units),
                "all_reduce_shape": [args.batch, cfg["hidden"]],
                "note": "one block-shard per rank compressed once and cloned per layer"} if cfg.get("tp") else {}),
        },
        "gpu_launches": len(units) * args.steps,
        "two_pass": {"path": "df11_decode", "ms_per_step": round(ms_two_pass, 4),
                     "GBps": round(total_bytes / ms_two_pass / 1e6, 1)},
    }
    tp_result = None
    if world > 1 and not args.skip_extras and not cfg.get("tp"):
        try:
            tp_result = tp_block(args, rank, world, device)
        except Exception as exc:                            # report, do not lose the line
            tp_result = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    if rank == 0:
        peak, how = measured_hbm_peak()
        per_gpu = step_bytes / ms / 1e6
        result["roofline"] = {
            "bound": "hbm", "achieved": round(per_gpu, 1), "peak": peak, "unit": "GB/s",
            "frac": round(per_gpu / peak, 4),
            # what the kernel really asks of memory per launch: stream + sign/mantissa + seek points in,
            # BF16 out (it never reads gaps / output_positions, which `algorithmic` counts)
            "actual_bytes_per_launch": int(sum(u["n_bytes"] + 3 * u["n_elements"] + u["aux"].numel() - (8 << 12)
                                               for u in units) / len(units)),
            "actual_GBps": round(sum(u["n_bytes"] + 3 * u["n_elements"] + u["aux"].numel() - (8 << 12)
                                     for u in units) / ms / 1e6, 1),
            # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of one launch on one
            # transformer-block unit of this workload under ncu, per element, scaled to the average unit
            "traffic": (int(DRAM_BYTES_PER_ELEMENT[ops.seek_interval()] * step_elems / len(units))
                        if DRAM_BYTES_PER_ELEMENT.get(ops.seek_interval()) else None),
            "algorithmic_bytes_per_launch": step_bytes // len(units),
            "peak_source": how,
            "kernel": f"df11_fast_kernel<12,{ops.seek_interval()}>", "frac_of_nominal_8000": round(per_gpu / 8000.0, 4),
            "avg_launch_ms": round(ms / len(units), 4),
        }
        result["clocks"] = clocks
        if tp_result is not None:
            result["tp"] = tp_result
        if e2e is not None:
            result["e2e"] = e2e
        if not args.skip_extras:
            def extra(key, fn):                             # an extra leg that fails is reported, the line still prints
                try:
                    result[key] = fn()
                except Exception as exc:  # noqa: BLE001
                    result[key] = {"error": f"{type(exc).__name__}: {exc}"[:300]}

            block = next(u for u, (name, _, _) in zip(units, plan) if name == "layers.0")
            extra("reference_gpu_kernel", lambda: time_reference_gpu_kernel(block, scratch))

            def cpu_legs():
                from oracle import df11_oracle as oracle
                oracle.build()
                cores = oracle.max_threads()
                mean, checksum = cpu_decode_sample(block["host"], cores, repeats=5, warmup=1)
                one, _ = cpu_decode_sample(block["host"], 1, repeats=1)
                return {
                    "value": round(algorithmic_bytes(block) / mean / 1e9, 3), "unit": "GB/s", "cores": cores,
                    "kind": "port", "single_core_GBps": round(algorithmic_bytes(block) / one / 1e9, 3),
                    "bit_exact": checksum == block["checksum"],
                    "sample": f"one transformer-block unit ({block['n_elements']} elements), mean of 5 decodes after "
                              f"1 untimed, {cores} threads; CPU restatement of the reference decode rule "
                              "(the reference has no CPU decoder)",
                    "compress": cpu_compress_sample(),
                }

            extra("cpu_baseline", cpu_legs)
            if world == 1 and cfg.get("vocab"):
                del units, u, block, out                    # `out` is a view of the scratch: it would keep it alive
                scratch = None
                extra("generation", lambda: generation_block(cfg, device))
        print(json.dumps(result))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


GEN_PATTERNS = {
    r"model\.embed_tokens": [],
    r"model\.layers\.\d+": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                             "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"],
    r"lm_head": [],
}


def run_fused_gemv(args, cfg):
    """One block of the workload's shape, one activation vector: the block's products as the
    package runs them with DF11_FUSED_GEMV=1 (q/k/v stacked, o, gate/up stacked, down: four
    fused launches) against decode-then-GEMV (one decode, seven torch products).  CUDA events,
    L2 flushed before every timed pass."""
    import torch.nn.functional as F
    from dfloat11_b200 import ops
    dev = torch.device("cuda", 0)
    shapes = block_shapes(cfg)
    n = sum(a * b for a, b in shapes)
    unit = make_unit(n, 0.02, 7, dev)
    aux = ops.prepare(unit["luts"], unit["enc"], unit["pos"], unit["gaps"], n)
    out = torch.empty(n, dtype=torch.bfloat16, device=dev)
    starts = [0]
    for a, b in shapes:
        starts.append(starts[-1] + a * b)
    g = torch.Generator(device=dev).manual_seed(3)
    x_h = torch.randn(1, cfg["hidden"], generator=g, device=dev).to(torch.bfloat16)
    x_i = torch.randn(1, cfg["inter"], generator=g, device=dev).to(torch.bfloat16)
    h, kv, it = cfg["hidden"], cfg["kv"], cfg["inter"]
    stacked = [(starts[0], h + 2 * kv, h, x_h), (starts[3], h, h, x_h), (starts[4], 2 * it, h, x_h), (starts[6], h, it, x_i)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def decode():
        ops.decode_prepared(unit["luts"], unit["enc"], unit["sm"], unit["pos"], unit["gaps"], aux, out=out)

    def products():
        for i, (a, b) in enumerate(shapes):
            F.linear(x_i if b == it else x_h, out[starts[i]:starts[i + 1]].view(a, b))

    def fused():
        return [ops.gemv_prepared(unit["luts"], unit["enc"], unit["sm"], aux, x, first, rows, cols)
                for first, rows, cols, x in stacked]

    def timed(fn):
        for _ in range(max(args.warmup, 1)):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(args.steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / args.steps

    decode()
    ys = fused()
    torch.cuda.synchronize()
    worst = 0.0
    for (first, rows, cols, x), y in zip(stacked, ys):
        want = x.float() @ out[first:first + rows * cols].view(rows, cols).float().T
        worst = max(worst, float(((y.float() - want).abs() / (want.abs() + 1e-3)).max()))
    t_decode, t_products, t_fused = timed(decode), timed(products), timed(fused)
    t_both = timed(lambda: (decode(), products()))
    compressed = unit["n_bytes"] + n + aux.numel()
    print(json.dumps({
        "metric": "batch1_block_products_ms", "unit": "ms", "workload": cfg["name"], "elements": n,
        "decode_then_gemv_ms": round(t_both, 4), "decode_ms": round(t_decode, 4), "bf16_gemv_ms": round(t_products, 4),
        "fused_ms": round(t_fused, 4), "fused_launches": 4, "speedup_vs_decode_then_gemv": round(t_both / t_fused, 3),
        "fused_vs_bf16_gemv": round(t_fused / t_products, 3),
        "fused_GBps_of_compressed_bytes_read": round(compressed / t_fused / 1e6, 1),
        "max_relative_difference_to_fp32_product": round(worst, 5), "steps": args.steps, "data": "synthetic",
    }))


def run_generation(args, cfg):
    """Batch-1 greedy generation with Hugging Face `generate` (the protocol of the reference's
    inference.py:45-95: warm-up forward, synchronize, wall clock, tokens / latency), on a
    random-init model of the workload's architecture: uncompressed BF16 first, then the same
    model object with its weights compressed in place.  Same harness, same attention
    implementation, same inputs; the generated ids must be identical."""
    import dfloat11_b200 as df11
    dev = torch.device("cuda", 0)
    # built inside a helper: a loop variable left over from initialising the weights would keep the
    # last parameter (the vocabulary-sized head) alive after the model has been compressed
    model, vocab_size = _random_init_model(cfg, dev)
    common = {"vocab_size": vocab_size}
    ids = torch.randint(0, common["vocab_size"], (args.batch if args.cpu_offload else 1, args.prompt_tokens), device=dev,
                        generator=torch.Generator(device=dev).manual_seed(2))

    def timed_generate():
        with torch.no_grad():
            model(input_ids=ids, use_cache=False)            # warm-up forward, as inference.py:45-52
            model.generate(ids, max_new_tokens=8, min_new_tokens=8, do_sample=False)   # and of generate itself
            best = None
            for _ in range(1 if args.cpu_offload else 2):    # best of two: the first pass still warms the allocator
                torch.cuda.synchronize()
                t0 = time.time()
                out = model.generate(ids, max_new_tokens=args.new_tokens, min_new_tokens=args.new_tokens,
                                     do_sample=False)
                torch.cuda.synchronize()
                dt = time.time() - t0
                best = dt if best is None else min(best, dt)
            return out, best

    def gpu_ms_per_token():
        """Sum of kernel time of one single-token forward with a KV cache (torch profiler): what
        the GPU is busy for, whatever the Python harness adds on the host.  Only with
        --kernel-times: once the profiler has run, every later launch of the process costs more
        host time, which would be charged to whichever model is timed after it."""
        if not args.kernel_times:
            return None
        from torch.profiler import ProfilerActivity, profile
        with torch.no_grad():
            pkv = model(input_ids=ids, use_cache=True).past_key_values
            tok = ids[:, -1:]
            for _ in range(2):
                model(input_ids=tok, past_key_values=pkv, use_cache=True)
            torch.cuda.synchronize()
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(4):
                    model(input_ids=tok, past_key_values=pkv, use_cache=True)
                torch.cuda.synchronize()
        total_us = sum(e.self_device_time_total for e in prof.key_averages())
        return total_us / 4 / 1e3

    def graph_generate():
        """The same greedy generation through the package's GraphedGreedyDecoder: a static KV
        cache and one CUDA graph per single-token step (the decode hooks run at capture time).
        Wall clock of prefill + `new_tokens` - 1 replays, and the ids produced."""
        n_prompt, n_new = ids.shape[1], args.new_tokens
        try:
            decoder = df11.GraphedGreedyDecoder(model, max_cache_len=n_prompt + n_new + 16)
            decoder.generate(ids, 8)                            # warm-up steps and the capture
            torch.cuda.synchronize()
            t0 = time.time()
            out = decoder.generate(ids, n_new)
            torch.cuda.synchronize()
            dt = time.time() - t0
            return dict(tok_s=n_new / dt, ids=out[0, n_prompt:].cpu(), steps=n_new)
        except Exception as exc:                                # report, do not hide
            return dict(tok_s=None, ids=None, error=f"{type(exc).__name__}: {exc}"[:300])

    if args.cpu_offload:
        # Compressed tensors in pinned host memory, one block's worth in HBM at a time (the
        # reference's cpu_offload=True): every generated token moves the whole compressed model
        # over PCIe, overlapped with decode by the hook's side stream.
        # The DF11 run comes first, in a process that has held nothing but the model before it, so
        # that its peak is its own; the BF16 weights wait in host memory for the reference run.
        from dfloat11_b200.dfloat11 import _OffloadStager
        bf16_state = {k: v.detach().cpu() for k, v in model.state_dict().items()}
        df11.compress_in_place(model, GEN_PATTERNS, cpu_offload=True)
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        out_df11, t_df11 = timed_generate()
        mem_df11 = torch.cuda.max_memory_allocated() / 1e9
        stager = _OffloadStager.get(dev)
        stats = stager.stats
        held = {"staging_slots": sum(b.numel() for slot in stager.slots for b in slot["buf"].values()),
                "scratch": sum(t.numel() * 2 for t in df11.TensorManager._tensors.values()),
                "seek_points_and_tables": sum(m.__dict__["df11_aux"].numel() for m in model.modules()
                                              if m.__dict__.get("df11_aux") is not None),
                "gaps_positions_luts": sum(getattr(m, k).numel() for m in model.modules() if hasattr(m, "luts")
                                           for k in ("gaps", "output_positions", "luts") if getattr(m, k).is_cuda)}
        held["everything_else"] = torch.cuda.memory_allocated() - sum(held.values())
        largest = sorted((b["size"] for seg in torch.cuda.memory_snapshot() for b in seg["blocks"]
                          if b["state"] == "active_allocated" and b["size"] >= 64 << 20), reverse=True)
        stats = dict(stats)
        del model, stager                                       # nothing of the DF11 run stays on the device
        df11.TensorManager.release()
        _OffloadStager._by_device.clear()
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        left_behind = torch.cuda.memory_allocated() / 1e9
        model, _ = _random_init_model(cfg, dev)
        model.load_state_dict(bf16_state)
        del bf16_state
        torch.cuda.reset_peak_memory_stats()
        out_bf16, t_bf16 = timed_generate()
        mem_bf16 = torch.cuda.max_memory_allocated() / 1e9
        tokens = args.batch * args.new_tokens
        print(json.dumps({
            "metric": "offload_generation_tok_per_s", "unit": "tok/s", "workload": cfg["name"], "batch": args.batch,
            "prompt_tokens": args.prompt_tokens, "new_tokens": args.new_tokens,
            "harness": "transformers generate, greedy, eager; DF11 with cpu_offload (compressed tensors in pinned host memory)",
            "bf16_resident_tok_s": round(tokens / t_bf16, 2), "df11_offload_tok_s": round(tokens / t_df11, 2),
            "df11_offload_s_per_step": round(t_df11 / args.new_tokens, 4),
            "identical_tokens": bool(torch.equal(out_bf16, out_df11)),
            "peak_mem_GB": {"bf16_resident": round(mem_bf16, 2), "df11_offload": round(mem_df11, 2)},
            "df11_device_memory_after_GB": {k: round(v / 1e9, 3) for k, v in held.items()},
            "allocator_blocks_over_64MB_after": [round(x / 2 ** 20) for x in largest[:8]],
            "device_memory_left_before_bf16_GB": round(left_behind, 3),
            "h2d_GB": round(stats["h2d_bytes"] / 1e9, 2), "prefetch_hits": stats["prefetch_hits"], "data": "synthetic",
        }))
        return

    out_bf16, t_bf16 = timed_generate()
    gpu_bf16 = gpu_ms_per_token()
    graph_bf16 = graph_generate()
    mem_bf16 = torch.cuda.max_memory_allocated() / 1e9
    t0 = time.time()
    df11.compress_in_place(model, GEN_PATTERNS)
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    t_compress = time.time() - t0
    out_df11, t_df11 = timed_generate()
    gpu_df11 = gpu_ms_per_token()
    graph_df11 = graph_generate()
    mem_df11 = torch.cuda.max_memory_allocated() / 1e9
    # the same model with single-token steps multiplied straight from the compressed weights
    os.environ["DF11_FUSED_GEMV"] = "1"
    try:
        gpu_fused = gpu_ms_per_token()
        graph_fused = graph_generate()
    finally:
        os.environ.pop("DF11_FUSED_GEMV", None)
    if graph_bf16["tok_s"] and graph_fused.get("tok_s"):
        same = (graph_fused["ids"] == graph_bf16["ids"])
        fused = {"df11_tok_s": round(graph_fused["tok_s"], 2),
                 "slowdown_vs_bf16": round(graph_bf16["tok_s"] / graph_fused["tok_s"], 3),
                 "gpu_kernel_ms_per_token": round(gpu_fused, 2) if gpu_fused else None,
                 "tokens_equal_to_bf16": int(same.sum()), "tokens": int(same.numel()),
                 "note": "products exact, fp32 sums in another order than the library GEMV: not bit-identical by design"}
    else:
        fused = {"unavailable": graph_fused.get("error")}
    if graph_bf16["tok_s"] and graph_df11["tok_s"]:
        graphed = {"bf16_tok_s": round(graph_bf16["tok_s"], 2), "df11_tok_s": round(graph_df11["tok_s"], 2),
                   "slowdown_vs_bf16": round(graph_bf16["tok_s"] / graph_df11["tok_s"], 3),
                   "identical_tokens": bool(torch.equal(graph_bf16["ids"], graph_df11["ids"])),
                   "timed_steps": graph_df11["steps"]}
    else:
        graphed = {"unavailable": graph_bf16.get("error") or graph_df11.get("error")}
    n = args.new_tokens
    print(json.dumps({
        "metric": "batch1_generation_tok_per_s", "unit": "tok/s", "workload": cfg["name"],
        "prompt_tokens": args.prompt_tokens, "new_tokens": n, "harness": "transformers generate, greedy, eager",
        "bf16_tok_s": round(n / t_bf16, 2), "df11_tok_s": round(n / t_df11, 2),
        "slowdown_vs_bf16": round(t_df11 / t_bf16, 3),
        "gpu_kernel_ms_per_token": ({"bf16": round(gpu_bf16, 2), "df11": round(gpu_df11, 2),
                                     "ratio": round(gpu_df11 / gpu_bf16, 3)} if gpu_bf16 else None),
        "identical_tokens": bool(torch.equal(out_bf16, out_df11)),
        "cuda_graph_static_cache": graphed,
        "cuda_graph_fused_gemv": fused,
        "peak_mem_GB": {"bf16": round(mem_bf16, 2), "df11": round(mem_df11, 2)},
        "compress_s": round(t_compress, 1), "data": "synthetic",
    }))


def _random_init_model(cfg, dev, layers=None):
    from transformers import Qwen3Config, Qwen3ForCausalLM, LlamaConfig, LlamaForCausalLM
    common = dict(hidden_size=cfg["hidden"], intermediate_size=cfg["inter"],
                  num_hidden_layers=layers or cfg["layers"],
                  num_attention_heads=cfg["hidden"] // 128, num_key_value_heads=cfg["kv"] // 128,
                  vocab_size=max(cfg["vocab"], 1024), tie_word_embeddings=False, max_position_embeddings=4096)
    torch.manual_seed(1)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with dev:
            if "qwen" in cfg["name"]:
                model = Qwen3ForCausalLM(Qwen3Config(head_dim=128, **common))
            else:
                model = LlamaForCausalLM(LlamaConfig(**common))
    finally:
        torch.set_default_dtype(old)
    model.eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.normal_(0.0, 1.0 if "embed_tokens" in name else 0.02)
    return model, common["vocab_size"]


def _graph_generate(model, ids, n_new):
    """Greedy generation through GraphedGreedyDecoder (static KV cache, one CUDA graph per
    single-token step): the reference's protocol (warm-up, synchronize, wall clock, tokens /
    latency, inference.py:45-95) with the host taken out of the per-token loop."""
    import dfloat11_b200 as df11
    n_prompt = ids.shape[1]
    torch.cuda.reset_peak_memory_stats()
    decoder = df11.GraphedGreedyDecoder(model, max_cache_len=n_prompt + n_new + 16)
    decoder.generate(ids, 8)                            # warm-up steps and the capture
    torch.cuda.synchronize()
    t0 = time.time()
    out = decoder.generate(ids, n_new)
    torch.cuda.synchronize()
    dt = time.time() - t0
    return dict(tok_s=n_new / dt, ids=out[0, n_prompt:].cpu(), peak=torch.cuda.max_memory_allocated() / 1e9)


def generation_block(cfg, dev, new_tokens=128, prompt_tokens=64):
    """Batch-1 greedy generation on the workload's architecture (random init): uncompressed BF16,
    then the same model object compressed in place (the default, bit-identical path), then the
    opt-in fused products.  tok/s, ratio to BF16, whether the ids are BF16's, peak device memory."""
    import dfloat11_b200 as df11
    from dfloat11_b200.dfloat11 import TensorManager, _OffloadStager
    TensorManager.release()                 # nothing of the decode legs above may count in the peaks below
    _OffloadStager._by_device.clear()
    torch.cuda.empty_cache()
    model, vocab = _random_init_model(cfg, dev)
    ids = torch.randint(0, vocab, (1, prompt_tokens), device=dev, generator=torch.Generator(device=dev).manual_seed(2))
    out = {"workload": cfg["name"], "prompt_tokens": prompt_tokens, "new_tokens": new_tokens,
           "harness": "greedy, static KV cache, one CUDA graph per single-token step (GraphedGreedyDecoder); "
                      "wall clock of prefill + steps"}
    with torch.no_grad():
        bf16 = _graph_generate(model, ids, new_tokens)
        out["bf16"] = {"tok_s": round(bf16["tok_s"], 2), "peak_mem_GB": round(bf16["peak"], 2)}
        t0 = time.time()
        df11.compress_in_place(model, GEN_PATTERNS)
        torch.cuda.empty_cache()
        out["compress_s"] = round(time.time() - t0, 1)
        legs = [("df11", {}), ("df11_fused_gemv", {"DF11_FUSED_GEMV": "1"})]
        for name, env in legs:
            os.environ.update(env)
            try:
                r = _graph_generate(model, ids, new_tokens)
                same = r["ids"] == bf16["ids"]
                out[name] = {"tok_s": round(r["tok_s"], 2), "slowdown_vs_bf16": round(bf16["tok_s"] / r["tok_s"], 3),
                             "ids_identical": bool(same.all()), "ids_equal": int(same.sum()),
                             "peak_mem_GB": round(r["peak"], 2),
                             "peak_mem_vs_bf16": round(r["peak"] / bf16["peak"], 3)}
            except Exception as exc:                        # report, do not hide
                out[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            finally:
                for k in env:
                    os.environ.pop(k, None)
        held = {"compressed": 0, "seek_points_and_tables": 0, "gaps_positions_luts": 0}
        for m in model.modules():
            if hasattr(m, "sign_mantissa") and isinstance(getattr(m, "sign_mantissa"), torch.Tensor):
                held["compressed"] += m.encoded_exponent.numel() + m.sign_mantissa.numel()
                held["gaps_positions_luts"] += sum(getattr(m, k).numel() for k in ("gaps", "output_positions", "luts")
                                                   if getattr(m, k).is_cuda)
                aux = m.__dict__.get("df11_aux")
                held["seek_points_and_tables"] += aux.numel() if aux is not None else 0
        held["scratch"] = sum(t.numel() * 2 for t in TensorManager._tensors.values())
        held["everything_else"] = torch.cuda.memory_allocated() - sum(held.values())
        out["df11_memory_GB"] = {k: round(v / 1e9, 3) for k, v in held.items()}
        out["df11_stats"] = {k: v for k, v in df11.stats().items() if k in ("decodes", "prepares", "sparse_lookups",
                                                                            "fused_products", "slab_products")}
    del model
    TensorManager.release()
    torch.cuda.empty_cache()
    return out


TOY_TP = dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=3, num_attention_heads=8,
              num_key_value_heads=8, vocab_size=8192, max_position_embeddings=256, tie_word_embeddings=False)


def tp_block(args, rank, world, device):
    """The partitioned mode on the job's own ranks (N > 1): (1) a small Llama, sharded then
    compressed by rank 0 into one directory per rank, loaded by every rank through
    DFloat11Model.from_pretrained(tp_size=N): logits of the DF11 shards against BF16 shards of the
    same model, bit for bit; (2) per-rank decode of Llama-3.1-405B block shards (one shard per
    rank compressed once and cloned for the layers) with the two activation all-reduces per
    layer, per-GPU GB/s, and the cost of one such all-reduce; (3) whole units placed on two
    devices by device_map="auto" (rank 0 only, devices 0 and 1) against the one-GPU BF16 model."""
    import torch.distributed as dist
    import dfloat11_b200 as df11
    from dfloat11_b200 import ops, tp
    from dfloat11_b200.dfloat11 import TensorManager
    from transformers import LlamaConfig, LlamaForCausalLM
    out = {}

    def toy(seed):
        # built in BF16 from the start, as from_pretrained builds its skeleton: the rotary tables then
        # stay fp32 in both (a model cast to BF16 afterwards has them rounded, and other logits)
        from transformers import AutoModelForCausalLM
        torch.manual_seed(seed)
        m = AutoModelForCausalLM.from_config(LlamaConfig(**TOY_TP), dtype=torch.bfloat16).eval()
        with torch.no_grad():
            for name, p in m.named_parameters():
                if p.dim() == 2:
                    p.copy_((torch.randn(p.shape) * (1.0 if "embed" in name else 0.02)).to(torch.bfloat16))
        return m

    # (1) parity of the partitioned mode
    shared = [None]
    if rank == 0:
        shared[0] = tempfile.mkdtemp(prefix="df11_tp_")
        tp.compress_model_tp(toy(0), GEN_PATTERNS, shared[0], tp_size=world)
    dist.broadcast_object_list(shared, src=0)
    bf16 = toy(0).to(device)
    tp.apply_tensor_parallel(bf16, GEN_PATTERNS, world, rank)
    model = df11.DFloat11Model.from_pretrained(shared[0], device=str(device), tp_size=world, tp_rank=rank)
    ids = torch.randint(0, TOY_TP["vocab_size"], (2, 40), generator=torch.Generator().manual_seed(4)).to(device)
    with torch.no_grad():
        same = bool(torch.equal(model(input_ids=ids).logits, bf16(input_ids=ids).logits))
        tok = bool(torch.equal(model.generate(ids[:1, :8], max_new_tokens=16, do_sample=False),
                               bf16.generate(ids[:1, :8], max_new_tokens=16, do_sample=False)))
    flag = torch.tensor([int(same), int(tok)], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    out["parity"] = {"model": "3-layer Llama, hidden 1024, vocabulary 8192, sharded before compression",
                     "logits_identical_to_bf16_shards": bool(flag[0].item()),
                     "generated_ids_identical": bool(flag[1].item()),
                     "vocabulary_parallel": model.lm_head.out_features == TOY_TP["vocab_size"] // world,
                     "all_reduces": ("own kernel over NVLink peer memory (NCCL where its buffers cannot be set up)"
                                     if os.environ.get("DF11_PEER_ALLREDUCE", "1") != "0" else "NCCL")}
    del model, bf16
    TensorManager.release()
    torch.cuda.empty_cache()
    dist.barrier(device_ids=[device.index])
    if rank == 0:
        import shutil
        shutil.rmtree(shared[0], ignore_errors=True)

    # (2) 405B block shards: decode + all-reduces
    cfg = LLAMA_405B_TP
    n_shard = sum(a * b for a, b in block_shapes(cfg)) // world
    layers = 16
    first = make_unit(n_shard, 0.02, seed=7000 + rank, device=device)
    units = [first] + [dict(first, enc=first["enc"].clone(), sm=first["sm"].clone()) for _ in range(layers - 1)]
    status = torch.zeros(1, dtype=torch.int32, device=device)
    for u in units:
        u["aux"] = ops.prepare(u["luts"], u["enc"], u["pos"], u["gaps"], u["n_elements"], status=status)
    scratch = torch.empty(n_shard, dtype=torch.bfloat16, device=device)
    act = torch.zeros(args.batch, cfg["hidden"], dtype=torch.bfloat16, device=device)

    def step(reduce):
        for u in units:
            ops.decode_prepared(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], u["aux"], out=scratch, status=status)
            if reduce:
                dist.all_reduce(act)
                dist.all_reduce(act)

    def timed(fn, steps=10, warmup=3):
        for _ in range(warmup):
            fn()
        barrier(world, device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier(world, device)
        return all_max(a.elapsed_time(b) / steps, world, device)

    def graphed(fn):
        """fn captured into one CUDA graph after a run on a side stream; returns the replay."""
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream(device).wait_stream(side)
        barrier(world, device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        return graph.replay

    ms_with = timed(lambda: step(True))
    ms_without = timed(lambda: step(False))
    ms_reduce = timed(lambda: [dist.all_reduce(act) for _ in range(2 * layers)])
    # the same step as one CUDA graph (what a generation loop replays): no host time between the launches
    ms_graph, ms_reduce_graph, graph_error = None, None, None
    try:
        ms_graph = timed(graphed(lambda: step(True)))
        # the all-reduces alone as one graph: their cost on the device, no host time and no decode between them
        ms_reduce_graph = timed(graphed(lambda: [dist.all_reduce(act) for _ in range(2 * layers)]), steps=50)
    except Exception as exc:                                # report, do not hide
        graph_error = f"{type(exc).__name__}: {exc}"[:200]
    # the same step with this library's one-kernel all-reduce over NVLink peer memory
    peer_result = None
    try:
        from dfloat11_b200.comm import PeerAllReduce
        peer = PeerAllReduce.get(None, device)
        agreed = torch.tensor([int(peer is not None)], device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)       # every rank takes the same branch below
        if int(agreed.item()):
            # one call first: a rank whose peers do not answer gives up after two seconds, and then
            # the timed loops (hundreds of calls) are not run at all
            probe = torch.ones(args.batch * cfg["hidden"], dtype=torch.bfloat16, device=device)
            fine = peer.all_reduce_(probe)
            torch.cuda.synchronize(device)
            fine = fine and int(peer.status.item()) == 0 and bool((probe == float(world)).all())
            agreed = torch.tensor([int(fine)], device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            peer.status.zero_()
        if not int(agreed.item()):
            peer_result = {"unavailable": "symmetric memory could not be set up on every rank, or the first call failed"}
        else:
            def step_peer():
                for u in units:
                    ops.decode_prepared(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], u["aux"], out=scratch,
                                        status=status)
                    peer.all_reduce_(act)
                    peer.all_reduce_(act)

            ms_peer = timed(step_peer)
            ms_peer_alone = timed(lambda: [peer.all_reduce_(act) for _ in range(2 * layers)])
            ms_peer_graph = timed(graphed(step_peer))
            ms_peer_alone_graph = timed(graphed(lambda: [peer.all_reduce_(act) for _ in range(2 * layers)]), steps=50)
            peer.check()
            total_p = all_sum(sum(algorithmic_bytes(u) for u in units), world, device)
            peak_p, _ = measured_hbm_peak()
            peer_result = {
                "ms_per_step": round(ms_peer, 3), "per_gpu_GBps": round(total_p / ms_peer / 1e6 / world, 1),
                "per_gpu_frac_of_measured_peak": round(total_p / ms_peer / 1e6 / world / peak_p, 4),
                "us_per_all_reduce_back_to_back": round(ms_peer_alone * 1e3 / (2 * layers), 2),
                "us_per_all_reduce_in_a_graph_of_all_reduces": round(ms_peer_alone_graph * 1e3 / (2 * layers), 2),
                "buffers_bound_to_a_multicast_object": peer.multicast_bound,
                "cuda_graph": {"ms_per_step": round(ms_peer_graph, 3),
                               "per_gpu_GBps": round(total_p / ms_peer_graph / 1e6 / world, 1),
                               "per_gpu_frac_of_measured_peak": round(total_p / ms_peer_graph / 1e6 / world / peak_p, 4),
                               "us_per_all_reduce_in_step": round((ms_peer_graph - ms_without) * 1e3 / (2 * layers), 2)}}
    except Exception as exc:                                # report, do not hide
        peer_result = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    ok = int(scratch.view(torch.int16).to(torch.int64).sum().item()) == first["checksum"] and status.item() == 0
    total = all_sum(sum(algorithmic_bytes(u) for u in units), world, device)
    peak, _ = measured_hbm_peak()
    out["llama_405b_shards"] = {
        "parallelism": f"tp{world}", "layers": layers, "elements_per_rank_and_layer": n_shard,
        "all_reduces_per_step": 2 * layers, "all_reduce_shape": [args.batch, cfg["hidden"]],
        "ms_per_step": round(ms_with, 3), "aggregate_GBps": round(total / ms_with / 1e6, 1),
        "per_gpu_GBps": round(total / ms_with / 1e6 / world, 1),
        "per_gpu_frac_of_measured_peak": round(total / ms_with / 1e6 / world / peak, 4),
        "cuda_graph": ({"ms_per_step": round(ms_graph, 3), "per_gpu_GBps": round(total / ms_graph / 1e6 / world, 1),
                        "per_gpu_frac_of_measured_peak": round(total / ms_graph / 1e6 / world / peak, 4),
                        "us_per_all_reduce_in_step": round((ms_graph - ms_without) * 1e3 / (2 * layers), 2)}
                       if ms_graph else {"error": graph_error}),
        "decode_only_ms_per_step": round(ms_without, 3),
        "us_per_all_reduce_back_to_back": round(ms_reduce * 1e3 / (2 * layers), 2),
        "us_per_all_reduce_in_a_graph_of_all_reduces": (round(ms_reduce_graph * 1e3 / (2 * layers), 2)
                                                        if ms_reduce_graph else None),
        "us_per_all_reduce_in_step": round((ms_with - ms_without) * 1e3 / (2 * layers), 2),
        "bit_exact": bool(ok),
        "peer_all_reduce": peer_result,
        "note": "one block-shard per rank compressed once and cloned per layer; the figures outside "
                "`peer_all_reduce` use NCCL's all-reduce, those inside the library's own kernel (the default "
                "of the partitioned mode)"}
    del units, first, scratch
    torch.cuda.empty_cache()

    # (3) layer placement over two devices, one process (what the reference does with accelerate).
    # Rank 0 borrows rank 1's GPU for it, so the other ranks wait on the host (the job's key-value
    # store), not inside a collective: no kernel of theirs sits on a GPU that rank 0 is using.
    barrier(world, device)
    store = dist.distributed_c10d._get_default_store()
    if rank != 0:
        store.wait(["df11_bench_placement_done"])
    if rank == 0 and torch.cuda.device_count() >= 2:
        try:
            with tempfile.TemporaryDirectory() as tmp:
                ref = toy(3)
                import copy
                df11.compress_model(copy.deepcopy(ref), GEN_PATTERNS, tmp, save_single_file=False, check_correctness=False)
                placed = df11.DFloat11Model.from_pretrained(tmp, device=None, device_map="auto")
                ref = ref.to(device)
                with torch.no_grad():
                    a = placed(input_ids=ids.to(device)).logits
                    b = ref(input_ids=ids.to(device)).logits
                devices = sorted({str(t.device) for t in placed.state_dict().values() if t.is_cuda})
                out["device_map_auto"] = {"devices_used": devices, "logits_identical_to_one_gpu_bf16": bool(torch.equal(a.to(b.device), b))}
                del placed, ref
        except Exception as exc:                            # report, do not hide
            out["device_map_auto"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        TensorManager.release()
        torch.cuda.empty_cache()
        for d in range(torch.cuda.device_count()):
            torch.cuda.synchronize(d)
    if rank == 0:
        store.set("df11_bench_placement_done", "1")
    barrier(world, device)
    return out


def run_tp_generation(args, cfg):
    """Greedy generation in the partitioned mode on the job's ranks: a Llama-3.1-405B-shaped
    model (hidden 16384, 128 / 8 heads, intermediate 53248, vocabulary 128256; as many of the 126
    layers as `--layers` or the memory allow) whose every rank holds only its tensor-parallel
    shards, random init.  First the BF16 shards, then the same modules compressed in place; both
    through GraphedGreedyDecoder with the activation all-reduces, the embedding all-reduce and
    the logits all-gather inside the captured step.  Ids must be identical."""
    import torch.distributed as dist
    import dfloat11_b200 as df11
    from dfloat11_b200 import tp
    from dfloat11_b200.dfloat11 import TensorManager
    from transformers import LlamaConfig, LlamaForCausalLM
    rank, world, local = dist_setup(args.gpus)
    if world < 2:
        raise SystemExit("the partitioned generation leg needs 2, 4 or 8 ranks (torchrun)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    per_layer = 2 * sum(a * b for a, b in block_shapes(cfg)) // world
    vocab = 128256
    fixed = 2 * 2 * vocab * cfg["hidden"] // world
    layers = args.layers or int(min(cfg["layers"], (140e9 - fixed) // per_layer))
    config = LlamaConfig(hidden_size=cfg["hidden"], intermediate_size=cfg["inter"], num_hidden_layers=layers,
                         num_attention_heads=cfg["hidden"] // 128, num_key_value_heads=cfg["kv"] // 128,
                         vocab_size=vocab, tie_word_embeddings=False, max_position_embeddings=4096)
    with torch.device("meta"):
        model = LlamaForCausalLM(config).to(torch.bfloat16).eval()
    tp.apply_tensor_parallel(model, GEN_PATTERNS, world, rank)           # shapes and collectives; no data yet
    rotary = type(model.model.rotary_emb)
    model.to_empty(device=dev)
    model.model.rotary_emb = rotary(config=config, device=dev)           # its tables are computed, not loaded
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.normal_(0.0, 1.0 if "embed_tokens" in name else 0.02, generator=g)
            else:
                p.fill_(1.0)
        del name, p                                          # or the last parameter (the head) outlives its compression
    ids = torch.randint(0, vocab, (args.batch, args.prompt_tokens), device=dev,
                        generator=torch.Generator(device=dev).manual_seed(2))   # the same prompts on every rank

    def generate():
        torch.cuda.reset_peak_memory_stats()
        decoder = df11.GraphedGreedyDecoder(model, max_cache_len=args.prompt_tokens + args.new_tokens + 16)
        decoder.generate(ids, 8)
        barrier(world, dev)
        t0 = time.time()
        out = decoder.generate(ids, args.new_tokens)
        barrier(world, dev)
        return out[:, args.prompt_tokens:], time.time() - t0, torch.cuda.max_memory_allocated() / 1e9

    with torch.no_grad():
        out_bf16, t_bf16, mem_bf16 = generate()
        t0 = time.time()
        df11.compress_in_place(model, GEN_PATTERNS)
        torch.cuda.empty_cache()
        t_compress = time.time() - t0
        out_df11, t_df11, mem_df11 = generate()
    same = torch.tensor([int(torch.equal(out_bf16, out_df11))], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    t_bf16, t_df11 = all_max(t_bf16, world, dev), all_max(t_df11, world, dev)
    tokens = args.batch * args.new_tokens
    if rank == 0:
        print(json.dumps({
            "metric": "tp_generation_tok_per_s", "unit": "tok/s", "workload": cfg["name"], "parallelism": f"tp{world}",
            "layers": layers, "layers_of_the_full_model": cfg["layers"], "batch": args.batch,
            "prompt_tokens": args.prompt_tokens, "new_tokens": args.new_tokens,
            "harness": "greedy, static KV cache, one CUDA graph per step with the collectives inside",
            "activation_all_reduce": ("own kernel over NVLink peer memory"
                                     if os.environ.get("DF11_PEER_ALLREDUCE", "1") != "0" else "NCCL (DF11_PEER_ALLREDUCE=0)"),
            "fused_gemv": os.environ.get("DF11_FUSED_GEMV", "0") == "1",
            "bf16_shards_tok_s": round(tokens / t_bf16, 2), "df11_shards_tok_s": round(tokens / t_df11, 2),
            "slowdown_vs_bf16_shards": round(t_df11 / t_bf16, 3), "ids_identical": bool(same.item()),
            "peak_mem_GB_per_rank": {"bf16": round(mem_bf16, 1), "df11": round(mem_df11, 1)},
            "compress_s": round(t_compress, 1), "vocabulary_parallel": True, "data": "synthetic",
        }))
    TensorManager.release()
    dist.destroy_process_group()


def run_loader(args, cfg):
    """Load time of a DF11 model directory: this package's loader (files memory-mapped, every large
    tensor copied once -- through pinned staging and a copy stream to the GPU, or straight into
    pinned memory of its own under cpu_offload) against the reference's way (dfloat11.py:215-219,
    256-263: `safetensors.torch.load_file` of every file, then `pin_memory()` or a pageable
    host -> device copy per tensor).  The model has the workload's shapes with `--layers` blocks
    (default 8) plus embedding and head; files come from the page cache in both cases (each way is
    run twice, the second run counts)."""
    import copy
    import dfloat11_b200 as df11
    from safetensors.torch import load_file
    dev = torch.device("cuda", 0)
    layers = args.layers or 8
    model, vocab = _random_init_model(cfg, dev, layers=layers)
    tmp = tempfile.mkdtemp(prefix="df11_load_")
    try:
        t0 = time.time()
        df11.compress_model(model, GEN_PATTERNS, tmp, save_single_file=False, check_correctness=False)
        t_save = time.time() - t0
        del model
        torch.cuda.empty_cache()
        files = sorted(f for f in os.listdir(tmp) if f.endswith(".safetensors"))
        total = sum(os.path.getsize(os.path.join(tmp, f)) for f in files)

        def ours(offload):
            torch.cuda.synchronize()
            t0 = time.time()
            m = df11.DFloat11Model.from_pretrained(tmp, device="cuda:0", cpu_offload=offload)
            torch.cuda.synchronize()
            dt = time.time() - t0
            del m
            df11.TensorManager.release()
            torch.cuda.empty_cache()
            return dt

        def ours_tensors_only(offload):
            # the loader proper, on a skeleton built beforehand (what from_pretrained does first)
            from transformers import AutoConfig, AutoModelForCausalLM
            try:
                from transformers.initialization import no_init_weights
            except ImportError:
                from transformers.modeling_utils import no_init_weights
            config = AutoConfig.from_pretrained(tmp)
            with no_init_weights():
                skeleton = AutoModelForCausalLM.from_config(config, dtype=torch.bfloat16).eval()
            torch.cuda.synchronize()
            t0 = time.time()
            df11.load_and_replace_tensors(skeleton, tmp, config.dfloat11_config, cpu_offload=offload, device="cuda:0")
            skeleton.to("cuda:0")
            torch.cuda.synchronize()
            dt = time.time() - t0
            del skeleton
            df11.TensorManager.release()
            torch.cuda.empty_cache()
            return dt

        def reference_way(offload):
            torch.cuda.synchronize()
            t0 = time.time()
            kept = []
            for f in files:
                for name, value in load_file(os.path.join(tmp, f)).items():
                    leaf = name.rsplit(".", 1)[-1]
                    if offload and leaf in ("encoded_exponent", "sign_mantissa"):
                        kept.append(value.pin_memory())
                    else:
                        kept.append(value.to(dev))
            torch.cuda.synchronize()
            dt = time.time() - t0
            del kept
            torch.cuda.empty_cache()
            return dt

        out = {"metric": "df11_model_load_s", "unit": "s", "workload": cfg["name"], "layers": layers,
               "files": len(files), "bytes": total, "save_s": round(t_save, 1), "data": "synthetic"}
        for offload in (False, True):
            ours(offload), reference_way(offload), ours_tensors_only(offload)
            a, b, c = ours(offload), reference_way(offload), ours_tensors_only(offload)
            key = "cpu_offload" if offload else "resident"
            out[key] = {"from_pretrained_s": round(a, 3),
                        "load_and_replace_tensors_s": round(c, 3), "load_and_replace_tensors_GBps": round(total / c / 1e9, 2),
                        "load_file_then_copy_s": round(b, 3), "load_file_then_copy_GBps": round(total / b / 1e9, 2),
                        "note": "from_pretrained also builds the skeleton; load_and_replace_tensors reads, copies, "
                                "validates and arms every unit; the last only reads and copies the tensors"}
        print(json.dumps(out))
    finally:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)


def run_dit_step(args):
    """One denoising step of a FLUX.1-dev-shaped diffusion transformer (19 double-stream + 38
    single-stream blocks, hidden 3072, 24 heads, MLP ratio 4; 4096 latent + 512 text tokens;
    random init N(0, 0.02)): the uncompressed BF16 model, then the same model object compressed in
    place.  Step time by CUDA events, outputs compared bit for bit."""
    import dfloat11_b200 as df11
    from dfloat11_b200.dfloat11 import TensorManager
    dev = torch.device("cuda", 0)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with dev:
            model = FluxShapedDiT().eval()
    finally:
        torch.set_default_dtype(old)
    with torch.no_grad():
        g = torch.Generator(device=dev).manual_seed(4)
        for p in model.parameters():
            p.normal_(0.0, 0.02, generator=g)
    x = torch.randn(1, 4096, 3072, device=dev, generator=g).to(torch.bfloat16)
    ctx = torch.randn(1, 512, 3072, device=dev, generator=g).to(torch.bfloat16)
    cond = torch.randn(1, 1, 3072, device=dev, generator=g).to(torch.bfloat16)
    n_weights = sum(p.numel() for p in model.parameters() if p.dim() == 2)

    def timed():
        with torch.no_grad():
            for _ in range(max(args.warmup, 1)):
                out = model(x, ctx, cond)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                out = model(x, ctx, cond)
            b.record()
            torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps, out

    torch.cuda.reset_peak_memory_stats()
    ms_bf16, out_bf16 = timed()
    mem_bf16 = torch.cuda.max_memory_allocated() / 1e9
    t0 = time.time()
    df11.compress_in_place(model, {k: list(v) for k, v in FLUX_PATTERNS.items()})
    torch.cuda.empty_cache()
    t_compress = time.time() - t0
    torch.cuda.reset_peak_memory_stats()
    ms_df11, out_df11 = timed()
    mem_df11 = torch.cuda.max_memory_allocated() / 1e9
    print(json.dumps({
        "metric": "dit_denoising_step_ms", "unit": "ms", "workload": FLUX_DIT["name"], "weights": n_weights,
        "tokens": {"latent": 4096, "text": 512}, "bf16_ms": round(ms_bf16, 3), "df11_ms": round(ms_df11, 3),
        "slowdown_vs_bf16": round(ms_df11 / ms_bf16, 4), "identical_output": bool(torch.equal(out_bf16, out_df11)),
        "peak_mem_GB": {"bf16": round(mem_bf16, 2), "df11": round(mem_df11, 2)}, "compress_s": round(t_compress, 1),
        "steps": args.steps, "warmup": args.warmup, "data": "synthetic",
        "df11_stats": {k: v for k, v in df11.stats().items() if isinstance(v, int)},
    }))
    TensorManager.release()


def run_slab_pipeline(args, cfg):
    """Decode-in-slabs against decode-the-whole-block, for one transformer block's seven batch-1
    products: each matrix (or slab of its rows, or run of neighbouring matrices) of at most B MB of
    BF16 is decompressed into the same scratch addresses right before the library product that
    reads it, so that the BF16 copy can stay in the L2 cache.  Four distinct blocks are cycled so
    that compressed data always comes from HBM; each variant is captured in a CUDA graph."""
    import torch.nn.functional as F
    from dfloat11_b200 import ops
    dev = torch.device("cuda", 0)
    shapes = block_shapes(cfg)
    n = sum(a * b for a, b in shapes)
    n_blocks = 4
    units = [make_unit(n, 0.02, 200 + i, dev, keep_weights=True) for i in range(n_blocks)]
    auxs = [ops.prepare(u["luts"], u["enc"], u["pos"], u["gaps"], n) for u in units]
    scratch = torch.empty(n, dtype=torch.bfloat16, device=dev)
    starts = [0]
    for a, b in shapes:
        starts.append(starts[-1] + a * b)
    xs = {b: torch.randn(1, b, device=dev).to(torch.bfloat16) for _, b in shapes}
    outs = [torch.empty(1, a, dtype=torch.bfloat16, device=dev) for a, _ in shapes]

    def bf16_block(i):
        w = units[i]["weights"]
        for k, (a, b) in enumerate(shapes):
            torch.mm(xs[b], w[starts[k]:starts[k + 1]].view(a, b).t(), out=outs[k])

    def whole(i):
        u = units[i]
        ops.decode_prepared(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], auxs[i], out=scratch)
        for k, (a, b) in enumerate(shapes):
            torch.mm(xs[b], scratch[starts[k]:starts[k + 1]].view(a, b).t(), out=outs[k])

    def decode_only(i):
        u = units[i]
        ops.decode_prepared(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], auxs[i], out=scratch)

    def slabbed(budget_mb):
        budget = (budget_mb << 20) // 2
        plan, k = [], 0
        while k < len(shapes):
            a, b = shapes[k]
            if a * b <= budget:                       # this matrix and the ones after it, while they fit
                first, total, parts = starts[k], 0, []
                while k < len(shapes) and total + shapes[k][0] * shapes[k][1] <= budget:
                    parts.append((k, 0, shapes[k][0], total))
                    total += shapes[k][0] * shapes[k][1]
                    k += 1
                plan.append((first, total, parts))
            else:                                     # slabs of rows
                n_slabs = -(-a // max(1, budget // b))
                rows = (-(-a // n_slabs) + 7) // 8 * 8
                for r0 in range(0, a, rows):
                    r1 = min(a, r0 + rows)
                    plan.append((starts[k] + r0 * b, (r1 - r0) * b, [(k, r0, r1, 0)]))
                k += 1
        slab = scratch[:max(p[1] for p in plan)]

        def run(i):
            u = units[i]
            for first, total, parts in plan:
                ops.decode_range_prepared(u["luts"], u["enc"], u["sm"], auxs[i], first, total, out=slab)
                for (k, r0, r1, off) in parts:
                    a, b = shapes[k]
                    torch.mm(xs[b], slab[off:off + (r1 - r0) * b].view(r1 - r0, b).t(), out=outs[k][:, r0:r1])
        return run, len(plan), sum(len(p[2]) for p in plan)

    def graph_ms(fn):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(n_blocks):
                fn(i)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n_blocks):
                fn(i)
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps / n_blocks

    if args.eager:
        # for a profiler: block 1's products once the plain way, once in 48 MB slabs, launched one by
        # one (no graph, no timing); blocks 2 and 3 in between push block 1's leftovers out of L2
        for fn in (whole, slabbed(48)[0]):
            fn(1)
            fn(2)
            fn(3)
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_push("measured")
            fn(1)
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()
        print(json.dumps({"eager": True, "order": ["decode whole + 7 products", "48 MB slabs: 8 decodes + 10 products"]}))
        return
    bf16_block(0)
    want = [o.clone() for o in outs]
    result = {"metric": "batch1_block_products_ms", "unit": "ms per block", "workload": cfg["name"],
              "elements_per_block": n, "bf16_products": round(graph_ms(bf16_block), 4),
              "decode_whole_then_products": round(graph_ms(whole), 4), "decode_whole_alone": round(graph_ms(decode_only), 4),
              "slabs": {}, "steps": args.steps, "data": "synthetic"}
    for mb in (16, 32, 48, 64, 101):
        run, n_dec, n_mm = slabbed(mb)
        for o in outs:
            o.zero_()
        run(0)
        same = all(bool(torch.equal(o, w)) for o, w in zip(outs, want))
        result["slabs"][f"{mb}MB"] = {"ms": round(graph_ms(run), 4), "decode_launches": n_dec, "products": n_mm,
                                      "bits_of_the_whole_products": same}
    print(json.dumps(result))


class FluxShapedDiT(torch.nn.Module):
    """A diffusion-transformer stack with the module names and Linear shapes of the reference's
    FLUX pattern dictionary (examples/compress_flux1/compress_flux.py:49-74): double-stream blocks
    with separate image / text projections and a joint attention, single-stream blocks with a
    fused MLP + attention output.  FLUX.1-dev has hidden 3072, 24 heads, 19 + 38 blocks; the tests
    build it at toy size.  Own minimal forward (diffusers is not a dependency): what matters for
    the decompression path are the units, their shapes and that every Linear runs."""

    class _Mod(torch.nn.Module):
        def __init__(self, h, n):
            super().__init__()
            self.linear = torch.nn.Linear(h, n * h)
            self.n = n

        def forward(self, cond):
            return self.linear(torch.nn.functional.silu(cond)).chunk(self.n, dim=-1)

    class _Attn(torch.nn.Module):
        def __init__(self, h, heads, joint):
            super().__init__()
            self.heads = heads
            self.to_q, self.to_k, self.to_v = torch.nn.Linear(h, h), torch.nn.Linear(h, h), torch.nn.Linear(h, h)
            if joint:
                self.add_q_proj, self.add_k_proj, self.add_v_proj = torch.nn.Linear(h, h), torch.nn.Linear(h, h), torch.nn.Linear(h, h)
                self.to_out = torch.nn.ModuleList([torch.nn.Linear(h, h)])
                self.to_add_out = torch.nn.Linear(h, h)

        def _split(self, t):
            b, n, h = t.shape
            return t.view(b, n, self.heads, h // self.heads).transpose(1, 2)

        def forward(self, x, ctx=None):
            q, k, v = self.to_q(x), self.to_k(x), self.to_v(x)
            if ctx is not None:
                q = torch.cat([self.add_q_proj(ctx), q], 1)
                k = torch.cat([self.add_k_proj(ctx), k], 1)
                v = torch.cat([self.add_v_proj(ctx), v], 1)
            o = torch.nn.functional.scaled_dot_product_attention(self._split(q), self._split(k), self._split(v))
            o = o.transpose(1, 2).reshape(q.shape)
            if ctx is None:
                return o
            n_ctx = ctx.shape[1]
            return self.to_out[0](o[:, n_ctx:]), self.to_add_out(o[:, :n_ctx])

    class _FF(torch.nn.Module):
        class _Proj(torch.nn.Module):
            def __init__(self, h, m):
                super().__init__()
                self.proj = torch.nn.Linear(h, m)

            def forward(self, x):
                return torch.nn.functional.gelu(self.proj(x), approximate="tanh")

        def __init__(self, h, m):
            super().__init__()
            self.net = torch.nn.ModuleList([self._Proj(h, m), torch.nn.Identity(), torch.nn.Linear(m, h)])

        def forward(self, x):
            return self.net[2](self.net[0](x))

    class _Double(torch.nn.Module):
        def __init__(self, h, heads):
            super().__init__()
            self.norm1, self.norm1_context = FluxShapedDiT._Mod(h, 6), FluxShapedDiT._Mod(h, 6)
            self.attn = FluxShapedDiT._Attn(h, heads, joint=True)
            self.ff, self.ff_context = FluxShapedDiT._FF(h, 4 * h), FluxShapedDiT._FF(h, 4 * h)
            self.ln = torch.nn.LayerNorm(h, elementwise_affine=False)

        def forward(self, x, ctx, cond):
            s1, c1, g1, s2, c2, g2 = self.norm1(cond)
            t1, d1, h1, t2, d2, h2 = self.norm1_context(cond)
            a, b = self.attn(self.ln(x) * (1 + c1) + s1, self.ln(ctx) * (1 + d1) + t1)
            x, ctx = x + g1 * a, ctx + h1 * b
            x = x + g2 * self.ff(self.ln(x) * (1 + c2) + s2)
            ctx = ctx + h2 * self.ff_context(self.ln(ctx) * (1 + d2) + t2)
            return x, ctx

    class _Single(torch.nn.Module):
        def __init__(self, h, heads):
            super().__init__()
            self.norm = FluxShapedDiT._Mod(h, 3)
            self.proj_mlp = torch.nn.Linear(h, 4 * h)
            self.proj_out = torch.nn.Linear(5 * h, h)
            self.attn = FluxShapedDiT._Attn(h, heads, joint=False)
            self.ln = torch.nn.LayerNorm(h, elementwise_affine=False)

        def forward(self, x, cond):
            s, c, g = self.norm(cond)
            y = self.ln(x) * (1 + c) + s
            m = torch.nn.functional.gelu(self.proj_mlp(y), approximate="tanh")
            return x + g * self.proj_out(torch.cat([self.attn(y), m], dim=-1))

    def __init__(self, h=3072, heads=24, n_double=19, n_single=38):
        super().__init__()
        self.transformer_blocks = torch.nn.ModuleList([self._Double(h, heads) for _ in range(n_double)])
        self.single_transformer_blocks = torch.nn.ModuleList([self._Single(h, heads) for _ in range(n_single)])
        self.proj_out = torch.nn.Linear(h, 16)

    def forward(self, x, ctx, cond):
        for blk in self.transformer_blocks:
            x, ctx = blk(x, ctx, cond)
        x = torch.cat([ctx, x], dim=1)
        for blk in self.single_transformer_blocks:
            x = blk(x, cond)
        return self.proj_out(x[:, ctx.shape[1]:])


FLUX_PATTERNS = {                                  # tuples, dotted paths: as the reference writes them
    r"transformer_blocks\.\d+": ("norm1.linear", "norm1_context.linear", "attn.to_q", "attn.to_k", "attn.to_v",
                                 "attn.add_k_proj", "attn.add_v_proj", "attn.add_q_proj", "attn.to_out.0",
                                 "attn.to_add_out", "ff.net.0.proj", "ff.net.2", "ff_context.net.0.proj",
                                 "ff_context.net.2"),
    r"single_transformer_blocks\.\d+": ("norm.linear", "proj_mlp", "proj_out", "attn.to_q", "attn.to_k", "attn.to_v"),
}


class _Unit(torch.nn.Module):
    """A compressed unit as the loader leaves it under ``cpu_offload``: small tensors as device
    buffers, the two large ones in pinned host memory, nothing to inject weights into."""

    def __init__(self, u, device):
        super().__init__()
        for name, key in (("luts", "luts"), ("output_positions", "pos"), ("gaps", "gaps")):
            self.register_buffer(name, u[key])
        self.offloaded_tensors = {"encoded_exponent": u["enc"].cpu().pin_memory(),
                                  "sign_mantissa": u["sm"].cpu().pin_memory()}
        self.split_positions, self.weight_injection_modules = [], []
        self.max_block_elems = u["widest"]
        self.df11_aux = u["aux"]

    def forward(self):
        return None


def run_e2e(units, scratch, status, device, world, args):
    """The user-facing path with host-resident compressed tensors: every unit's forward pre-hook
    (dfloat11_b200.get_hook, the hook `DFloat11Model.from_pretrained(..., cpu_offload=True)`
    installs) pulls its encoded_exponent / sign_mantissa from pinned host memory through the
    side-stream staging slots and decodes into the shared scratch; host->device copies are
    inside the timed region, and a slice of the result is read back every step."""
    import dfloat11_b200 as df11
    from dfloat11_b200.dfloat11 import TensorManager, _OffloadStager
    TensorManager._tensors[(device, 0)] = scratch     # same scratch as the resident runs
    hook = df11.get_hook((512,), 8)
    # pinned host memory is bounded (24 GB per rank, 64 GB per job): the workload's first units up to that size
    budget, kept = min(24e9, 64e9 / world), []
    for u in units:
        budget -= u["n_bytes"] + u["n_elements"]
        if budget < 0 and len(kept) >= 2:
            break
        kept.append(u)
    units = kept
    mods = [_Unit(u, device) for u in units]
    for a, b in zip(mods, mods[1:] + mods[:1]):
        a.__dict__["df11_next_offloaded"] = b
        a.register_forward_pre_hook(hook)
    h2d = sum(t.numel() for m in mods for t in m.offloaded_tensors.values())
    result_host = torch.empty(1024, dtype=torch.bfloat16).pin_memory()

    def step():
        for m in mods:
            m()                                        # pre-hook: fetch + decode; the forward itself is empty
        result_host.copy_(scratch[:1024], non_blocking=True)

    step()
    barrier(world, device)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.e2e_steps):
        step()
    b.record()
    barrier(world, device)
    ms = all_max(a.elapsed_time(b) / args.e2e_steps, world, device)
    total = all_sum(sum(algorithmic_bytes(u) for u in units), world, device)
    got = int(scratch[:units[-1]["n_elements"]].view(torch.int16).to(torch.int64).sum().item())
    if got != units[-1]["checksum"]:
        raise SystemExit("e2e decode mismatch")
    stats = _OffloadStager.get(device).stats
    # the ceiling of this leg: bare pinned-host -> HBM copies of the same tensors, all ranks at once
    # (they share the host's memory system and PCIe root ports), nothing decoded
    copy_stream = torch.cuda.Stream(device=device)
    sink = torch.empty(max(t.numel() for m in mods for t in m.offloaded_tensors.values()), dtype=torch.uint8,
                       device=device)
    barrier(world, device)
    with torch.cuda.stream(copy_stream):
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for m in mods:
            for t in m.offloaded_tensors.values():
                sink[:t.numel()].copy_(t, non_blocking=True)
        c1.record()
    copy_stream.synchronize()
    barrier(world, device)
    copy_ms = all_max(c0.elapsed_time(c1), world, device)
    return {"value": round(total / ms / 1e6, 1), "unit": "GB/s", "h2d_bytes_per_step": int(h2d),
            "bare_h2d_copy_ms_per_step": round(copy_ms, 3),
            "bare_h2d_copy_GBps_per_rank": round(h2d / copy_ms / 1e6, 1),
            "frac_of_bare_copy_ceiling": round(copy_ms / ms, 3),
            "d2h_bytes_per_step": int(result_host.numel() * 2), "ms_per_step": round(ms, 3),
            "steps": args.e2e_steps, "units": len(units), "prefetch_hits": stats["prefetch_hits"],
            "path": "forward pre-hook of the package with cpu_offload units: pinned host encoded_exponent + "
                    "sign_mantissa -> cudaMemcpyAsync on a side stream into two staging slots -> "
                    "df11_decode_prepared (C ABI)"}


if __name__ == "__main__":
    main()
