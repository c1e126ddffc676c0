"""Forward-throughput benchmark of the M2-BERT hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one forward of the 12-layer M2-BERT-80M-shaped encoder (embeddings + 12 x
[sequence mixer, GLU MLP]) under torch.autocast(bfloat16) on one synthetic batch; each rank
owns its own batch (weak scaling by batch, no collective on the data path).  Prints one
JSON line (rank 0).  Keys:
  value        sequences/s over all ranks, inputs resident in HBM
  e2e          the same through the public API with pinned host token ids copied to the
               device and the [CLS] rows copied back inside the timed region
  roofline     fused long-convolution kernel: algorithmic bytes / mean launch time (CUDA
               events on the launching stream, during the timed steps) / measured HBM peak
  cpu_baseline the stock-PyTorch-op restatement of the same forward (what the reference
               runs on a CPU) timed on this box's host cores on a bounded sample
`--impl reference` times that CPU path alone, on the same config and metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

WORKLOADS = {
    # name: (layers, d_model, inter, L, batch per GPU)
    "m2bert80m-L128": dict(layers=12, D=768, I=3072, L=128, B=256),
    "m2bert80m-L8192": dict(layers=12, D=768, I=3072, L=8192, B=4),
    "m2bert80m-L32768": dict(layers=12, D=768, I=3072, L=32768, B=1),
    "m2bert-large-L128": dict(layers=24, D=1536, I=6144, L=128, B=64),
    "m2bert-large-L2048": dict(layers=24, D=1536, I=6144, L=2048, B=8),
}
VOCAB = 30528
METRIC = "M2-BERT-80M fwd sequences/sec"
UNIT = "sequences/s"


def seeded_state(model, seed):
    """Random-init weights of the reference's constructor distributions, re-seeded per
    layer (the reference deep-copies one layer, which would make all layers identical)."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("freq") or "pos_emb" in name:
                continue
            if p.dim() >= 2:
                fan_in = p.shape[-1] * (p.shape[-2] if name.endswith("short_filter.weight") else 1)
                bound = 1.0 / max(1.0, float(fan_in)) ** 0.5
                if "embeddings" in name:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.02)
                elif "gated_layers.weight" in name or "wo.weight" in name:
                    p.copy_((torch.rand(p.shape, generator=g) * 2 - 1) * (p.shape[0] ** 0.5) / (p.shape[0] * p.shape[2]) ** 0.5)
                else:
                    p.copy_((torch.rand(p.shape, generator=g) * 2 - 1) * bound)
            elif name.endswith("filter_fn.bias") or name.endswith("filter_fn2.bias"):
                p.copy_(torch.randn(p.shape, generator=g))
            elif "LayerNorm" in name or "layernorm" in name:
                p.copy_(torch.ones_like(p) if name.endswith("weight") else torch.zeros_like(p))
            else:
                p.copy_((torch.rand(p.shape, generator=g) * 2 - 1) * 0.03)


def build_model(w, seed=0):
    from m2_b200.encoder import M2BertConfig, M2BertModel
    conf = M2BertConfig(vocab_size=VOCAB, hidden_size=w["D"], intermediate_size=w["I"],
                        num_hidden_layers=w["layers"], max_position_embeddings=w["L"],
                        long_conv_l_max=w["L"])
    model = M2BertModel(conf).eval()
    seeded_state(model, seed)
    return model


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.idx), "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = [s for s in sm if s > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def cpu_forward_fn(w, n_layers, sample_b, seed=0):
    """The stock-op CPU restatement on a state dict with our model's weights."""
    from oracle import torch_oracle as T
    model = build_model(w, seed)
    sd = {k: v.detach().float() for k, v in model.state_dict().items()}
    ids = torch.randint(0, VOCAB, (sample_b, w["L"]), generator=torch.Generator().manual_seed(1))

    def run():
        with torch.no_grad():
            h = T.embeddings_forward(sd, ids)
            return T.encoder_forward(sd, h, n_layers)
    return run


def time_cpu(w, sample_b, reps):
    torch.set_num_threads(os.cpu_count() or 1)
    run = cpu_forward_fn(w, w["layers"], sample_b)
    run()
    t0 = time.perf_counter()
    for _ in range(reps):
        run()
    dt = (time.perf_counter() - t0) / reps
    return sample_b / dt, dt


def config_of(name, w, n, graph=True):
    return {"workload": f"{name}: {w['layers']}-layer M2-BERT encoder fwd (embeddings + mixer + BlockdiagLinear GLU MLP), "
                        f"d_model {w['D']}, L={w['L']}, batch {w['B']} per GPU, token ids uniform in [0,{VOCAB}), "
                        "random-init weights, bf16 autocast",
            "batch_per_gpu": w["B"], "global_batch": w["B"] * n, "seq_len": w["L"],
            "parallelism": f"batch-sharded x{n}, no data-path collective",
            "launch": "one CUDA-graph replay per forward" if graph else "eager, one Python call per kernel",
            "l2": "explicit L2 flush (256 MiB write) between timed iterations"}


def run_reference(args, name, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # bounded sample: a batch small enough that steps+warmup end within minutes
    sample_b = max(1, min(w["B"], 32 if w["L"] <= 128 else 1))
    torch.set_num_threads(os.cpu_count() or 1)
    run = cpu_forward_fn(w, w["layers"], sample_b)
    for _ in range(args.warmup):
        run()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter(); run(); times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    val = sample_b / (ms / 1e3)
    sample = f"{sample_b} sequences per step of the same workload, float32, stock PyTorch ops on CPU"
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(name, w, args.gpus, graph=not args.no_graph),
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="m2bert80m-L128", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch per GPU")
    args = ap.parse_args()
    name, w = args.workload, dict(WORKLOADS[args.workload])
    if args.batch > 0:
        w["B"] = args.batch
    if args.impl == "reference":
        run_reference(args, name, w)
        return

    import torch.distributed as dist
    from m2_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus or world == 1 and args.gpus == 1, "launch with torchrun for --gpus > 1"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    model = build_model(w, seed=0).to(dev)
    B, L = w["B"], w["L"]
    g = torch.Generator().manual_seed(1234 + rank)
    ids_host = torch.randint(0, VOCAB, (B, L), generator=g).pin_memory()
    ids_dev = ids_host.to(dev)
    cls_host = torch.empty((B, w["D"]), dtype=torch.float32).pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)

    def step_eager():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            out, _ = model(ids_dev)
        return out

    if args.no_graph:
        step_resident = step_eager

        def step_e2e():
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                ids = ids_host.to(dev, non_blocking=True)
                out, _ = model(ids)
                cls_host.copy_(out[:, 0].float(), non_blocking=True)
            return out
    else:
        # the public fixed-shape entry point: one captured forward, replayed per batch
        from m2_b200.graph import GraphedForward
        graphed = GraphedForward(model, ids_dev, warmup=max(args.warmup, 3))

        def step_resident():
            return graphed(graphed.static_in[0])[0]

        def step_e2e():
            out, _ = graphed(ids_host)                      # pinned host ids -> static device buffer
            cls_host.copy_(out[:, 0], non_blocking=True)
            return out

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(step, steps):
        """Per-step CUDA events on the launching stream, L2 flushed between steps."""
        evs = []
        for _ in range(steps):
            flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream); step(); e.record(stream)
            evs.append((s, e))
        torch.cuda.synchronize(dev)
        return sum(s.elapsed_time(e) for s, e in evs)      # ms over exactly `steps` steps

    for _ in range(max(args.warmup, 3)):
        step_resident()
    step_e2e()
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ops.LAUNCHES = 0
    total_ms = timed(step_resident, args.steps)
    launches = ops.LAUNCHES
    barrier()
    e2e_ms = timed(step_e2e, args.steps)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    # per-kernel device times: a separate eager pass with an event pair around every launch of
    # this library (the events would perturb the timed steps)
    ops.PROFILE = ops.LaunchProfile()
    prof_steps = 3
    for _ in range(prof_steps):
        flush.fill_(1)
        step_eager()
    torch.cuda.synchronize(dev)
    prof, ops.PROFILE = ops.PROFILE, None

    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = t.tolist()

    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = world * B / (ms_per_step / 1e3)
        e2e_value = world * B / (e2e_ms / args.steps / 1e3)
        # roofline of the fused long-convolution kernel (one launch per layer per step)
        conv_ms = prof.mean_ms("m2_longconv_fwd")
        D = w["D"]
        alg_bytes = 10.0 * B * D * L + 16.0 * D * L          # bf16 activations, two filters
        peak, peak_src = measured_peaks()
        achieved = alg_bytes / (conv_ms * 1e-3) / 1e9 if conv_ms else None
        # DRAM bytes per launch of that kernel from the ncu captures summarised under profiles/
        # (dram__bytes_read.sum + dram__bytes_write.sum); None where no capture of the shape exists
        traffic = {"m2bert80m-L128": 247.2e6, "m2bert80m-L8192": 564e6}.get(name)
        roof = {"bound": "hbm", "kernel": "m2_longconv_fwd", "achieved": achieved, "peak": peak,
                "peak_source": peak_src, "unit": "GB/s", "frac": (achieved / peak) if achieved else None,
                "traffic": traffic, "launch_ms": conv_ms, "algorithmic_bytes_per_launch": alg_bytes,
                "kernel_ms_per_step": {k: prof.mean_ms(k) * prof.count(k) / prof_steps for k in prof.names()}}
        cpu = None
        if not args.no_cpu_baseline:
            sample_b = 32 if L <= 128 else 1
            reps = 3
            v, dt = time_cpu(w, sample_b, reps)
            cpu = {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                   "sample": f"{reps} forwards of {sample_b} sequences of the same workload "
                             f"({dt:.2f} s each), float32, stock PyTorch ops on the host CPU"}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": config_of(name, w, world, graph=not args.no_graph),
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": ids_host.numel() * 8,
                        "d2h_bytes_per_step": cls_host.numel() * 4},
                "gpu_launches": launches, "clocks": clocks, "roofline": roof, "cpu_baseline": cpu}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
