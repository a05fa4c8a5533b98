#!/usr/bin/env python
"""Headline benchmark: GPT-2-small training throughput (tokens/s over the whole job).

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Config (the reference's GPT-2-small line): 12 layers, d_model 768, 12 heads, MLP
3072, vocab 50304, sequence 2048, global batch 64, bf16, flash attention, Adam;
tensor parallel over the N GPUs (TP = N), so the total work is fixed ("strong").
Synthetic data: token ids uniform over the vocabulary, weights N(0, 0.02).

Prints ONE JSON line on rank 0.  `value` is device-timed (CUDA events around
exactly K steps, max over ranks) with the batch already on the device; `e2e` times
the same K steps through the public API (`Trainer.step`) including, per step, the
host->device copy of the batch from pinned memory and a device->host read of the loss.

`--impl reference` reports the reference arm.  The reference (a C11 CPU library
with no Python packaging and no runnable transformer path) cannot be installed, so
that arm prints its `unavailable` line.  `--impl torch` runs the same model with
PyTorch library kernels (cuBLAS + SDPA + NCCL), the comparison point named for the
configs the reference cannot run: tensor parallel over the N ranks as all-gather ->
GEMM and GEMM -> reduce-scatter with NCCL collectives, the reference's unfused design.

The default arm measures that baseline too, in the same process right after its own
timed regions (same N, same batch, same warm-up; `--baseline-steps` timed steps), and
reports `vs_baseline` = value / baseline value, with the baseline's own numbers under
`baseline`.  On one GPU the INT4 speculative-decoding configuration (Llama-7B shape, batch 16,
512-token prompts, 256 new tokens, gamma 4) then runs once in a child process and is reported under
`int4_spec_decode` (`--serving off` skips it; with several GPUs run `benchmarks/spec_decode.py` under
the launcher).  The headline figures are fixed before any of these extras start; an extra that does not
come back within its limit (ranks that lost each other inside it) ends the run with the line as it
stands and an `error` entry under the extra's key.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REF_UNAVAILABLE = ("pip install of the reference failed: \"Neither 'setup.py' nor 'pyproject.toml' found\" "
                   "(pure-C CMake project whose library target does not compile; no transformer training path)")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cogito", choices=["cogito", "reference", "torch"])
    ap.add_argument("--micro-batch", type=int, default=0,
                    help="sequences per micro-batch; 0 = the whole batch of the rank in one pass (no gradient "
                         "accumulation)")
    ap.add_argument("--global-batch", type=int, default=64)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--parallelism", default="tp", choices=["tp", "dp"])
    ap.add_argument("--no-alt", action="store_true", help="with several GPUs, skip the extra data-parallel measurement")
    ap.add_argument("--baseline-steps", type=int, default=-1,
                    help="timed steps of the PyTorch-library baseline measured in the same run (-1 = min(steps, 5), "
                         "0 = skip it and leave vs_baseline null)")
    ap.add_argument("--serving", default="auto", choices=["auto", "on", "off"],
                    help="on one GPU, also run the INT4 speculative-decoding configuration (Llama-7B shape, batch 16, "
                         "512-token prompts, 256 new tokens, gamma 4) as a child process after the training "
                         "measurements and report it under \"int4_spec_decode\" (auto = on)")
    ap.add_argument("--timeline", default="", help="after the timed regions, trace two more steps and write the device "
                    "time per kernel name (rank 0) to this JSON file; not part of any reported number")
    args = ap.parse_args()
    if args.micro_batch <= 0:
        dp = args.gpus if (args.parallelism == "dp" or args.impl != "cogito") else 1
        args.micro_batch = max(1, args.global_batch // dp)
    return args


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


class Reporter:
    """Holds the result line and prints it exactly once (rank 0): at the end of main(), or from a timer
    thread when one of the extra measurements that follow the headline (library baseline, data-parallel
    variant) does not come back, e.g. because one rank failed inside it and the others wait for it in a
    collective.  Every rank arms the same timer, so all of them leave together."""

    def __init__(self, rank: int):
        self.rank = rank
        self.out = None
        self._lock = threading.Lock()
        self._done = False

    def emit(self):
        with self._lock:
            if self._done:
                return
            self._done = True
            if self.rank == 0 and self.out is not None:
                print(json.dumps(self.out), flush=True)

    def guard(self, seconds: float, key: str) -> threading.Timer:
        def fire():
            if self.out is not None:
                self.out[key] = {"error": f"no result within {seconds:.0f} s; the run ended here"}
            self.emit()
            sys.stderr.write(f"bench.py: '{key}' did not finish within {seconds:.0f} s, leaving\n")
            sys.stderr.flush()
            os._exit(0)

        t = threading.Timer(seconds, fire)
        t.daemon = True
        t.start()
        return t


def kernel_timeline(step, path, rank, barrier, steps=2):
    """Device time per kernel name over `steps` steps (kineto trace; shares, not a benchmark)."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    barrier()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
    barrier()
    if rank != 0:
        return
    rows = []
    for ev in prof.key_averages():
        t = getattr(ev, "device_time_total", None)
        if t is None:
            t = getattr(ev, "cuda_time_total", 0.0)
        if getattr(ev, "device_type", None) is not None and "CUDA" in str(ev.device_type) and t > 0:
            rows.append({"kernel": ev.key[:120], "calls_per_step": ev.count / steps, "ms_per_step": t / 1e3 / steps})
    rows.sort(key=lambda r: -r["ms_per_step"])
    # the launches of the last traced step in launch order (name, microseconds): calls of one kernel
    # with different shapes can be told apart by their position in the step
    seq = []
    try:
        evs = [e for e in prof.events() if "CUDA" in str(getattr(e, "device_type", "")) and e.time_range is not None]
        evs.sort(key=lambda e: e.time_range.start)
        evs = evs[len(evs) - len(evs) // steps:]
        seq = [[e.name[:48], round(getattr(e, "device_time", 0.0) or (e.time_range.end - e.time_range.start), 1)] for e in evs]
    except Exception:
        seq = []
    with open(path, "w") as f:
        json.dump({"steps": steps, "total_ms_per_step": sum(r["ms_per_step"] for r in rows), "kernels": rows,
                   "last_step_launches": seq}, f, indent=1)


def main():
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return 0

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py: --gpus {args.gpus} needs torch.distributed.run with {args.gpus} ranks", file=sys.stderr)
            return 2
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from cogito_b200.bench_support import build_job

    job = build_job(args, rank, world, dev)
    flops_per_token = job.flops_per_token
    B, T = args.global_batch, args.seq_len
    tokens_per_step = B * T

    g = torch.Generator().manual_seed(1234)
    host_ids = torch.randint(0, job.vocab, (B, T), generator=g).pin_memory()
    host_tg = torch.randint(0, job.vocab, (B, T), generator=g).pin_memory()
    dev_ids, dev_tg = host_ids.to(dev), host_tg.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    loss_box = [None]

    def step_device():
        loss_box[0] = job.step(dev_ids, dev_tg)

    def step_e2e():
        loss_box[0] = float(job.step(host_ids, host_tg))      # H2D copy inside, D2H read of the loss

    for _ in range(max(args.warmup, 3)):
        step_device()
    job.reset_launch_count()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(step_device, args.steps)
    launches = job.launch_count()
    clocks = sampler.stop() if rank == 0 else None
    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    final_loss = float(loss_box[0])
    if args.timeline:
        kernel_timeline(step_device, args.timeline, rank, barrier)

    ms_per_step = ms / args.steps
    value = tokens_per_step / (ms_per_step * 1e-3)
    e2e_val = tokens_per_step / (ms_e2e / args.steps * 1e-3)
    rep = Reporter(rank)
    rep.out = out = {
        "metric": "train tok/s/box (GPT-2-small, whole job)", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (uniform token ids, N(0,0.02) weights)", "impl": args.impl,
        "config": {"model": "gpt2-small", "layers": args.layers, "d_model": 768, "heads": 12, "mlp": 3072,
                   "vocab": 50304, "global_batch": B, "seq_len": T, "micro_batch": args.micro_batch,
                   "parallelism": f"{args.parallelism}{world}", "optimizer": "adam",
                   "l2": "inputs larger than L2: each step streams >10 GB of activations and weights"},
        "clocks": clocks,
        "e2e": {"value": e2e_val, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                # every rank copies the whole global batch (ids and targets, int64): under tensor
                # parallelism each rank needs all tokens; the figure is per rank
                "h2d_bytes_per_step": host_ids.numel() * 8 + host_tg.numel() * 8, "d2h_bytes_per_step": 4},
        "gpu_launches": launches, "final_loss": final_loss,
        "model_tflops_per_gpu": flops_per_token * value / world / 1e12,
    }

    # The comparison point: the identical configuration on PyTorch library kernels (NCCL + cuBLAS +
    # SDPA + fused AdamW), measured here and now so that both numbers come from the same GPUs.
    baseline = None
    nb = min(args.steps, 5) if args.baseline_steps < 0 else args.baseline_steps
    if args.impl == "cogito" and nb > 0:
        watch = rep.guard(300, "baseline")
        try:
            import copy
            import gc
            job = None
            loss_box[0] = None
            gc.collect()
            torch.cuda.empty_cache()
            ab = copy.copy(args)
            ab.impl = "torch"
            if ab.parallelism == "dp":
                ab.micro_batch = max(1, B // world)
            jobb = build_job(ab, rank, world, dev)

            def step_base():
                loss_box[0] = jobb.step(dev_ids, dev_tg)

            for _ in range(3):
                step_base()
            msb = timed(step_base, nb) / nb
            baseline = {"impl": "torch: NCCL collectives + cuBLAS + SDPA + fused AdamW, " + f"{args.parallelism}{world}",
                        "value": tokens_per_step / (msb * 1e-3), "unit": "tokens/s", "ms_per_step": msb, "steps": nb,
                        "warmup": 3, "final_loss": float(loss_box[0])}
            jobb = None
            loss_box[0] = None
            gc.collect()
            torch.cuda.empty_cache()
        except Exception as e:
            baseline = {"error": repr(e)[:300]}
        watch.cancel()
        out["baseline"] = baseline
        if "value" in baseline:
            out["vs_baseline"] = value / baseline["value"]

    # The named configuration is tensor parallel; the same model and batch under data parallelism (the
    # fused all-reduce + Adam kernel) is measured as well and reported beside it under "alt".
    alt = None
    if world > 1 and args.impl == "cogito" and args.parallelism == "tp" and not args.no_alt:
        watch = rep.guard(240, "alt")
        try:
            import copy
            import gc
            job = None
            loss_box[0] = None
            gc.collect()
            torch.cuda.empty_cache()
            a2 = copy.copy(args)
            a2.parallelism, a2.micro_batch = "dp", max(1, B // world)
            job2 = build_job(a2, rank, world, dev)

            def step_alt():
                loss_box[0] = job2.step(dev_ids, dev_tg)

            for _ in range(3):
                step_alt()
            ms2 = timed(step_alt, args.steps) / args.steps
            alt = {"parallelism": f"dp{world}", "value": tokens_per_step / (ms2 * 1e-3), "ms_per_step": ms2,
                   "micro_batch": a2.micro_batch, "final_loss": float(loss_box[0])}
        except Exception as e:                          # the headline number above stands on its own
            alt = {"parallelism": f"dp{world}", "error": repr(e)[:300]}
        watch.cancel()
        out["alt"] = alt

    # The serving half of the reference's headline: INT4 speculative decoding at the named size.  It runs
    # as a child process with a time limit, after the training jobs have released their memory, so that
    # nothing that happens there can touch the numbers above; one GPU only (a child per rank would need
    # its own rendezvous - under the launcher use benchmarks/spec_decode.py directly).
    serving = None
    if args.impl == "cogito" and (args.serving == "on" or (args.serving == "auto" and world == 1)) and world == 1:
        try:
            import gc
            job = None
            loss_box[0] = None
            gc.collect()
            torch.cuda.empty_cache()
            here = os.path.dirname(os.path.abspath(__file__))
            env = dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", str(local)))
            for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
                env.pop(k, None)
            r = subprocess.run([sys.executable, os.path.join(here, "benchmarks", "spec_decode.py")], env=env, cwd=here,
                               capture_output=True, text=True, timeout=600)
            line = next((ln for ln in reversed(r.stdout.splitlines()) if ln.startswith("{")), None)
            if r.returncode == 0 and line:
                rec = json.loads(line)
                serving = {k: rec.get(k) for k in ("value", "unit", "ms_per_step", "steps", "acceptance_rate", "prefill_ms",
                                                   "cuda_graph", "launches_per_step", "config")}
            else:
                serving = {"error": f"exit code {r.returncode}: " + (r.stderr or r.stdout)[-300:]}
        except Exception as e:
            serving = {"error": repr(e)[:300]}
        out["int4_spec_decode"] = serving

    rep.emit()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
