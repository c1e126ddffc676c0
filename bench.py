"""Forward-throughput benchmark of the M2-BERT hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one forward of the M2-BERT-shaped encoder (embeddings + layers x [sequence mixer, GLU MLP]) under
torch.autocast(bfloat16) on one synthetic batch.  Rank 0 prints ONE JSON line.

The headline (top-level keys) is the 12-layer 80M encoder at L = 128 with 256 sequences per GPU (weak scaling by
batch, no collective on the data path).  Without --workload the same run also measures, under `workloads`, the
other configurations at their stated GLOBAL batch sizes split over the ranks (strong scaling): 80M at L = 8192
(global batch 32) and L = 32768 (8), the large shape at L = 128 (512) and L = 2048 (64), and -- under
`channel_shard` -- the 32K mixer's un-mixed middle sharded by d_model channel (each rank computes its channels
of the full batch of 8; an NCCL all-gather outside the timed region checks the reassembled tensor).

Keys per measurement:
  value        sequences/s over all ranks, inputs resident in HBM
  e2e          the same through the public API with pinned host token ids copied to the device and the [CLS]
               rows (what a pooled-embedding caller reads) copied back inside the timed region
  roofline     fused long-convolution kernel: algorithmic bytes / mean launch time (CUDA events on the launching
               stream, in a separate eager pass) / measured HBM peak
  kernel_ms_per_step   device time of every launch of this library per step, by entry point
  cold_first_forward_ms  first forward after construction: filter MLPs and spectrum tables are generated
  cpu_baseline the stock-PyTorch-op restatement of the same forward (what the reference runs on a CPU) timed on
               this box's host cores on a bounded sample (N = 1, rank 0, headline only)
`--impl reference` times that CPU path alone, on the headline's config and metric.
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
    # name: layers, d_model, intermediate, L and either a batch per GPU (weak scaling) or a global batch split
    # over the ranks (strong scaling) -- the batch sizes of the benchmark configurations
    "m2bert80m-L128": dict(layers=12, D=768, I=3072, L=128, per_gpu=256),
    "m2bert80m-L8192": dict(layers=12, D=768, I=3072, L=8192, global_batch=32),
    "m2bert80m-L32768": dict(layers=12, D=768, I=3072, L=32768, global_batch=8),
    "m2bert-large-L128": dict(layers=24, D=1536, I=6144, L=128, global_batch=512),
    "m2bert-large-L2048": dict(layers=24, D=1536, I=6144, L=2048, global_batch=64),
}
HEADLINE = "m2bert80m-L128"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the long-convolution kernel, from the ncu captures
# summarised under profiles/ (file named beside each value); None where no capture of the current kernel exists
TRAFFIC = {
    "m2bert80m-L128": (247.2e6, "profiles/longconv_tz_m2bert80m-L128.md"),
    "m2bert80m-L8192": (1990e6, "profiles/longconv_tcl_m2bert80m-L8192.md (batch-8 capture scaled to batch 32)"),
    "m2bert80m-L32768": (2169e6, "profiles/longconv_tcl_m2bert80m-L32768.md (batch-2 capture scaled to batch 8)"),
    "m2bert-large-L2048": (1973e6, "profiles/longconv_tcl_m2bert-large-L2048.md (batch-16 capture scaled to batch 64)"),
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


def batch_per_gpu(w, world):
    if "per_gpu" in w:
        return w["per_gpu"], "weak"
    g = w["global_batch"]
    if g % world:
        raise SystemExit(f"global batch {g} does not split over {world} ranks")
    return g // world, "strong"


def config_of(name, w, B, n, scaling, graph=True):
    return {"workload": f"{name}: {w['layers']}-layer M2-BERT encoder fwd (embeddings + mixer + BlockdiagLinear GLU MLP), "
                        f"d_model {w['D']}, L={w['L']}, batch {B} per GPU, token ids uniform in [0,{VOCAB}), "
                        "random-init weights, bf16 autocast",
            "batch_per_gpu": B, "global_batch": B * n, "seq_len": w["L"], "scaling": scaling,
            "parallelism": f"batch-sharded x{n}, no data-path collective",
            "launch": "one CUDA-graph replay per forward" if graph else "eager, one Python call per kernel",
            "l2": "explicit L2 flush (256 MiB write) between timed iterations",
            "e2e_result": "[CLS] row of every sequence (the pooled-embedding caller's read), float32"}


def run_reference(args, name, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B, scaling = batch_per_gpu(w, max(args.gpus, 1))
    # bounded sample: a batch small enough that steps+warmup end within minutes
    sample_b = max(1, min(B, 32 if w["L"] <= 128 else 1))
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
            "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(name, w, B, args.gpus, scaling, graph=not args.no_graph),
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


class Ctx:
    """Process-wide state of one benchmark run."""

    def __init__(self, args):
        import torch.distributed as dist
        self.args, self.dist = args, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        assert self.world == args.gpus or self.world == 1 and args.gpus == 1, "launch with torchrun for --gpus > 1"
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
        self.stream = torch.cuda.current_stream(self.dev)

    def barrier(self):
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.dev)

    def timed(self, step, steps):
        """Per-step CUDA events on the launching stream, L2 flushed between steps; ms over exactly `steps`."""
        evs = []
        for _ in range(steps):
            self.flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(self.stream); step(); e.record(self.stream)
            evs.append((s, e))
        torch.cuda.synchronize(self.dev)
        return sum(s.elapsed_time(e) for s, e in evs)

    def max_over_ranks(self, values):
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()


def measure(ctx, name, w, steps, warmup, clocks=False):
    """One workload on every rank: resident and end-to-end throughput, per-kernel device times, roofline of the
    long-convolution kernel.  Returns the measurement dict on rank 0 (None elsewhere)."""
    from m2_b200 import ops
    args, dev, world, rank = ctx.args, ctx.dev, ctx.world, ctx.rank
    B, scaling = batch_per_gpu(w, world)
    L, D = w["L"], w["D"]
    model = build_model(w, seed=0).to(dev)
    g = torch.Generator().manual_seed(1234 + rank)
    ids_host = torch.randint(0, VOCAB, (B, L), generator=g).pin_memory()
    ids_dev = ids_host.to(dev)
    cls_host = torch.empty((B, D), dtype=torch.float32).pin_memory()

    def step_eager():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            out, _ = model(ids_dev)
        return out

    # cold: the first forward generates every layer's filters (MLP on CUDA cores) and spectrum tables
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    step_eager()
    torch.cuda.synchronize(dev)
    cold_ms = 1e3 * (time.perf_counter() - t0)

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
        graphed = GraphedForward(model, ids_dev, warmup=max(warmup, 3))

        def step_resident():
            return graphed(graphed.static_in[0])[0]

        def step_e2e():
            out, _ = graphed(ids_host)                      # pinned host ids -> static device buffer
            cls_host.copy_(out[:, 0], non_blocking=True)
            return out

    for _ in range(max(warmup, 3)):
        step_resident()
    step_e2e()
    ctx.barrier()
    sampler = ClockSampler(ctx.local) if (clocks and rank == 0) else None
    if sampler:
        sampler.start()
    ops.LAUNCHES = 0
    total_ms = ctx.timed(step_resident, steps)
    launches = ops.LAUNCHES
    ctx.barrier()
    e2e_ms = ctx.timed(step_e2e, steps)
    ctx.barrier()
    clock_rec = sampler.stop() if sampler else None
    # per-kernel device times: a separate eager pass with an event pair around every launch of this library
    # (the events would perturb the timed steps)
    ops.PROFILE = ops.LaunchProfile()
    prof_steps = 3
    for _ in range(prof_steps):
        ctx.flush.fill_(1)
        step_eager()
    torch.cuda.synchronize(dev)
    prof, ops.PROFILE = ops.PROFILE, None
    total_ms, e2e_ms = ctx.max_over_ranks([total_ms, e2e_ms])
    res = None
    if rank == 0:
        ms_per_step = total_ms / steps
        conv_ms = prof.mean_ms("m2_longconv_fwd")
        alg_bytes = 10.0 * B * D * L + 16.0 * D * L          # bf16 activations, two filters
        peak, peak_src = measured_peaks()
        achieved = alg_bytes / (conv_ms * 1e-3) / 1e9 if conv_ms else None
        full_batch = B == WORKLOADS[name].get("per_gpu", WORKLOADS[name].get("global_batch"))      # captures are of that batch
        traffic, traffic_src = TRAFFIC.get(name, (None, None)) if full_batch else (None, None)
        res = {"value": world * B / (ms_per_step / 1e3), "unit": UNIT, "ms_per_step": ms_per_step, "steps": steps,
               "scaling": scaling, "config": config_of(name, w, B, world, scaling, graph=not args.no_graph),
               "e2e": {"value": world * B / (e2e_ms / steps / 1e3), "unit": UNIT,
                       "h2d_bytes_per_step": ids_host.numel() * 8, "d2h_bytes_per_step": cls_host.numel() * 4},
               "tokens_per_ms": world * B * L / ms_per_step,
               "gpu_launches": launches, "cold_first_forward_ms": cold_ms, "clocks": clock_rec,
               "roofline": {"bound": "hbm", "kernel": "m2_longconv_fwd", "achieved": achieved, "peak": peak,
                            "peak_source": peak_src, "unit": "GB/s", "frac": (achieved / peak) if achieved else None,
                            "traffic": traffic, "traffic_source": traffic_src, "launch_ms": conv_ms,
                            "algorithmic_bytes_per_launch": alg_bytes},
               "kernel_ms_per_step": {k: prof.mean_ms(k) * prof.count(k) / prof_steps for k in prof.names()}}
    return res


def measure_channel_shard(ctx, steps, warmup):
    """The 32K mixer sharded by d_model channel: every rank holds the full batch of 8 and computes channels
    [r D/N, (r+1) D/N) of the tensor out_linear consumes (in_linear rows, short conv, gates, both long
    convolutions).  Timed region: that computation only (max over ranks); afterwards an NCCL all-gather
    reassembles the shards and rank 0 compares them with the tensor computed whole on its own GPU."""
    from m2_b200 import sharding
    w = dict(WORKLOADS["m2bert80m-L32768"], layers=1)
    B, L, D = w["global_batch"], w["L"], w["D"]
    dev, world, rank = ctx.dev, ctx.world, ctx.rank
    mixer = build_model(w, seed=0).to(dev).encoder.layer[0].attention
    u = torch.randn((B, L, D), generator=torch.Generator().manual_seed(4321)).to(dev)     # the same on every rank
    lo, hi = sharding.shard_range(D, rank, world)

    def step():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            return mixer.forward_channels(u, lo, hi)

    for _ in range(max(warmup, 3)):
        step()
    ctx.barrier()
    ms = ctx.timed(step, steps)
    ctx.barrier()
    (ms,) = ctx.max_over_ranks([ms])
    mine = step().contiguous()
    equal = None
    if world > 1:
        gathered = sharding.gather_channels(mine)
        if rank == 0:
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                equal = bool(torch.equal(gathered, mixer.forward_channels(u, 0, D)))
        del gathered
    res = None
    if rank == 0:
        res = {"workload": f"sequence mixer without out_linear, d_model {D}, L={L}, batch {B} on every rank, "
                           f"{D // world} channels per rank, u ~ N(0,1), bf16 autocast",
               "value": B / (ms / steps / 1e3), "unit": UNIT, "ms_per_step": ms / steps, "steps": steps,
               "scaling": "strong", "channels_per_gpu": hi - lo,
               "gathered_equals_single_gpu": equal, "collective": "NCCL all_gather after the timed region (verification only)"}
    del mixer, u, mine
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="measure only this workload (default: the L=128 headline plus all others under `workloads`)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--batch", type=int, default=0, help="override the headline workload's batch per GPU")
    args = ap.parse_args()
    name = args.workload or HEADLINE
    w = dict(WORKLOADS[name])
    if args.batch > 0:
        w.pop("global_batch", None)
        w["per_gpu"] = args.batch
    if args.impl == "reference":
        run_reference(args, name, w)
        return

    import gc
    ctx = Ctx(args)
    head = measure(ctx, name, w, args.steps, max(args.warmup, 3), clocks=True)
    gc.collect(); torch.cuda.empty_cache()
    others, shard = {}, None
    if args.workload is None:
        sub_steps = max(3, min(args.steps, 5))
        for other, ow in WORKLOADS.items():
            if other == name:
                continue
            try:
                r = measure(ctx, other, dict(ow), sub_steps, 3)
            except SystemExit as e:                      # a global batch that does not split over this many ranks
                r = {"skipped": str(e)} if ctx.rank == 0 else None
            if ctx.rank == 0:
                others[other] = r
            gc.collect(); torch.cuda.empty_cache()
        if WORKLOADS["m2bert80m-L32768"]["D"] % ctx.world == 0:
            shard = measure_channel_shard(ctx, sub_steps, 3)
            gc.collect(); torch.cuda.empty_cache()

    if ctx.rank == 0:
        cpu = None
        if not args.no_cpu_baseline and ctx.world == 1:
            sample_b = 32 if w["L"] <= 128 else 1
            reps = 3
            v, dt = time_cpu(w, sample_b, reps)
            cpu = {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                   "sample": f"{reps} forwards of {sample_b} sequences of the same workload "
                             f"({dt:.2f} s each), float32, stock PyTorch ops on the host CPU"}
        line = {"metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": ctx.world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True,
                "scaling": head["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": head["config"], "e2e": head["e2e"], "gpu_launches": head["gpu_launches"],
                "clocks": head["clocks"], "tokens_per_ms": head["tokens_per_ms"],
                "cold_first_forward_ms": head["cold_first_forward_ms"],
                "roofline": dict(head["roofline"], kernel_ms_per_step=head["kernel_ms_per_step"]),
                "cpu_baseline": cpu}
        if others:
            line["workloads"] = others
        if shard is not None:
            line["channel_shard"] = shard
        print(json.dumps(line))
    if ctx.world > 1:
        ctx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
