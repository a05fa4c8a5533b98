"""Command line: ``python -m cogito_b200 <command> [config.yaml] [key=value ...]``.

    train     run a training job described by a YAML config (see ``DEFAULTS``): GPT-2, Llama, MLP or
              convolutional classifier; data / tensor / pipeline / 3-D parallel under a launcher
    generate  INT4 speculative decoding with a draft / target pair (tensor parallel under a launcher)
    info      versions, device, library status

A config is a nested mapping; ``section.key=value`` arguments override it (``train.steps=20``,
``train.schedule.kind=step``).  Sections: ``model``, ``parallel``, ``train``, ``data``, ``checkpoint``
(``dir``, ``every``, ``resume``, ``init_from``), ``failure`` (heartbeats), ``log``, ``profile``,
``generate``.  Under torchrun the job is multi-rank: ``parallel: {dp, tp, pp}`` must multiply to the
world size.

The reference has no configuration layer: its examples hard-code sizes and hyper-parameters
(examples/xor.c, examples/mnist.c) and the CMake options are the only switchboard.
"""
from __future__ import annotations

import argparse
import copy
import itertools
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import yaml

DEFAULTS = {
    "seed": 0,
    "device": "auto",                      # auto | cpu | cuda
    "model": {"family": "gpt2", "vocab_size": 50304, "n_layer": 12, "d_model": 768, "n_head": 12, "n_kv_head": None,
              "d_ff": 3072, "max_seq_len": 2048, "hidden": [512, 512], "in_features": 784, "classes": 10,
              "in_channels": 1, "image": 28, "channels": [16, 32]},
    "parallel": {"dp": 1, "tp": 1, "pp": 1, "microbatches": 1, "virtual_stages": 1},
    "train": {"steps": 10, "batch": 8, "micro_batch": None, "seq_len": 1024, "lr": 3e-4, "weight_decay": 0.0,
              "max_grad_norm": 1.0, "loss_scale": 65536.0, "optimizer": "adam",
              # learning-rate schedule of the reference's optimizers: "step" multiplies by gamma every step_size steps,
              # "exp" sets lr * gamma^step
              "schedule": {"kind": None, "step_size": 100, "gamma": 0.5}},
    "data": {"kind": "synthetic", "images": None, "labels": None},
    "checkpoint": {"dir": None, "every": 0, "resume": False, "init_from": None},   # init_from: COG1 file of the model (cg_save_model / save_model)
    # multi-rank jobs: heartbeats in the job's store, checked before every step; a rank that stopped answering ends
    # the run with exit code 3 (restart it with checkpoint.resume=true); device_check_every n reads the kernels'
    # status word every n steps (a bounded device-side wait that ran out)
    "failure": {"heartbeat": False, "interval_s": 0.5, "timeout_s": 10.0, "device_check_every": 0},
    "log": {"path": None, "every": 1},
    "profile": False,
}


def _merge(base, over):
    out = copy.deepcopy(base)
    for k, v in (over or {}).items():
        out[k] = _merge(out[k], v) if isinstance(v, dict) and isinstance(out.get(k), dict) else v
    return out


def _override(cfg, item):
    key, _, raw = item.partition("=")
    node = cfg
    parts = key.split(".")
    for p in parts[:-1]:
        node = node.setdefault(p, {})
    node[parts[-1]] = yaml.safe_load(raw)


def load_config(path, overrides=()):
    cfg = _merge(DEFAULTS, yaml.safe_load(open(path)) if path else {})
    for item in overrides:
        _override(cfg, item)
    return cfg


def _device(cfg):
    want = cfg["device"]
    if want == "auto":
        want = "cuda" if torch.cuda.is_available() else "cpu"
    if want == "cuda":
        local = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local)
        return torch.device("cuda", local)
    return torch.device("cpu")


def cmd_train(cfg):
    from .data.datasets import BatchIterator, SyntheticTokens, load_mnist
    from .io import checkpoint as ckpt
    from .optim.fused import FusedAdam, FusedSGD, GradScaler, exp_lr, step_lr
    from .train import Trainer
    from .utils import rng
    from .utils.profiler import Profiler, instrument

    dev = _device(cfg)
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if dev.type == "cuda" else "gloo", **({"device_id": dev} if dev.type == "cuda" else {}))
    rng.manual_seed(cfg["seed"])
    m, p, t = cfg["model"], cfg["parallel"], cfg["train"]
    dtype = torch.bfloat16 if dev.type == "cuda" else None
    if p["dp"] * p["tp"] * p["pp"] != world:
        raise SystemExit(f"parallel.dp*tp*pp = {p['dp'] * p['tp'] * p['pp']} but the job has {world} ranks")
    scaler_on = t["loss_scale"] is not None and dev.type == "cuda"
    family = m["family"]
    step_fn, model, opt = None, None, None
    logger = rank == 0
    if family == "llama" and world > 1:
        from .models.llama import LlamaConfig
        from .parallel.groups import init_parallel
        from .parallel.llama_parallel import Trainer3D
        lc = LlamaConfig(vocab_size=m["vocab_size"], n_layer=m["n_layer"], d_model=m["d_model"], n_head=m["n_head"],
                         n_kv_head=m["n_kv_head"] or m["n_head"], d_ff=m["d_ff"], max_seq_len=m["max_seq_len"])
        ctx = init_parallel(p["dp"], p["tp"], p["pp"])
        mb = t["micro_batch"] or 1
        t3 = Trainer3D(lc, ctx, dev, p["microbatches"], mb, t["seq_len"], lr=t["lr"], loss_scale=t["loss_scale"] if scaler_on else None,
                       max_grad_norm=t["max_grad_norm"], weight_decay=t["weight_decay"],
                       virtual_stages=p.get("virtual_stages", 1) or 1)
        model, opt = t3.stage, t3.opt
        batch_rows = p["microbatches"] * mb
        step_fn = t3.step
        # the loss exists on the last pipeline stage: its first rank of the first replica reports
        c = ctx.coords
        logger = c.pp_rank == c.pp - 1 and c.dp_rank == 0 and c.tp_rank == 0
    else:
        if family == "gpt2":
            from .models.gpt2 import GPT2, GPT2Config
            gc = GPT2Config(vocab_size=m["vocab_size"], n_layer=m["n_layer"], d_model=m["d_model"], n_head=m["n_head"], d_ff=m["d_ff"],
                            max_seq_len=m["max_seq_len"])
            if p["tp"] > 1:
                from .parallel.tensor_parallel import build_tp_gpt2
                model, sync = build_tp_gpt2(gc, rank, world, dev, micro_tokens=(t["micro_batch"] or t["batch"]) * t["seq_len"])
                params, parallel = model._ordered, sync
            else:
                model = GPT2(gc, device=dev, dtype=dtype)
                params, parallel = list(model.parameters()), None
        elif family == "llama":
            from .models.llama import Llama, LlamaConfig
            model = Llama(LlamaConfig(vocab_size=m["vocab_size"], n_layer=m["n_layer"], d_model=m["d_model"], n_head=m["n_head"],
                                      n_kv_head=m["n_kv_head"] or m["n_head"], d_ff=m["d_ff"], max_seq_len=m["max_seq_len"]), device=dev, dtype=dtype)
            params, parallel = list(model.parameters()), None
        elif family == "mlp":
            from .models.mlp import MLPClassifier
            model = MLPClassifier(m["in_features"], m["hidden"], m["classes"], device=dev, dtype=dtype)
            params, parallel = list(model.parameters()), None
        elif family == "cnn":
            from .models.cnn import ConvClassifier
            model = ConvClassifier(m["in_channels"], m["image"], m["channels"], m["classes"], device=dev, dtype=dtype)
            params, parallel = list(model.parameters()), None
        else:
            raise SystemExit(f"unknown model.family {family}")
        scaler = GradScaler(dev, enabled=scaler_on, init_scale=t["loss_scale"] or 1.0)
        kw = dict(lr=t["lr"], weight_decay=t["weight_decay"], scaler=scaler, max_grad_norm=t["max_grad_norm"])
        if p["dp"] > 1 and p["tp"] == 1:
            from .parallel.data_parallel import DPFusedAdam
            opt = DPFusedAdam(params, dist.group.WORLD, **kw)
        elif t["optimizer"] == "sgd":
            opt = FusedSGD(params, momentum=0.9, **kw)
        else:
            opt = FusedAdam(params, **kw)
        if p["tp"] > 1:
            parallel.attach(opt)
        trainer = Trainer(model, opt, micro_batch=t["micro_batch"], log_path=cfg["log"]["path"] if rank == 0 else None, parallel=parallel)
        batch_rows = t["batch"] // max(p["dp"], 1)
        step_fn = trainer.step

    # ---- data
    d = cfg["data"]
    if family == "mlp":
        if d["kind"] == "mnist":
            x, y = load_mnist(d["images"], d["labels"])
        else:
            g = torch.Generator().manual_seed(cfg["seed"] + 1 + rank)
            x, y = torch.rand(batch_rows * t["steps"], m["in_features"], generator=g), torch.randint(0, m["classes"], (batch_rows * t["steps"],), generator=g)
        batches = BatchIterator(x, y, batch_rows, shuffle=True, seed=cfg["seed"] + rank)
    elif family == "cnn":
        side, ch = m["image"], m["in_channels"]
        if d["kind"] == "mnist":
            x, y = load_mnist(d["images"], d["labels"])
            x = x.view(-1, ch, side, side)
        else:
            # one random prototype per class plus noise: separable, so the loss shows whether training works
            g = torch.Generator().manual_seed(cfg["seed"] + 1 + rank)
            n = batch_rows * t["steps"]
            proto = torch.randn(m["classes"], ch, side, side, generator=torch.Generator().manual_seed(cfg["seed"]))
            y = torch.randint(0, m["classes"], (n,), generator=g)
            x = 0.5 * proto[y] + 0.7 * torch.randn(n, ch, side, side, generator=g)
        batches = BatchIterator(x, y, batch_rows, shuffle=True, seed=cfg["seed"] + rank)
    else:
        batches = SyntheticTokens(m["vocab_size"], batch_rows, t["seq_len"], t["steps"], seed=cfg["seed"] + 17 * (rank // max(p["tp"] * p["pp"], 1)))

    # ---- resume
    ck = cfg["checkpoint"]
    start = 0
    base = None
    # Pure data-parallel jobs write one replicated model file and one optimizer shard per rank in a layout that a
    # job of ANOTHER size can read (the shards are re-cut for the new group): lose a GPU, restart with the rest.
    dp_job = world > 1 and p["dp"] == world and hasattr(opt, "shard_state")
    dp_base = os.path.join(ck["dir"], "dp") if ck["dir"] else None

    def save_state(at_step):
        if not dp_job:
            ckpt.save_training_state(base, model, opt, at_step)
            return
        import glob
        if rank == 0:
            for f in glob.glob(glob.escape(dp_base) + ".opt.dp*of*.state"):
                if not f.endswith(f"of{world:02d}.state"):
                    os.remove(f)                              # shards of an earlier group size
        dist.barrier()
        ckpt.save_dp_optimizer_shard(dp_base, opt)
        if rank == 0:
            ckpt.save_model(dp_base + ".cog", model)
            with open(dp_base + ".json", "w") as f:
                json.dump({"step": int(at_step), "lr": float(opt.lr), "ranks": world}, f)
        dist.barrier()                                        # the set is complete before anyone moves on

    if ck["init_from"]:
        if p["tp"] > 1 or p["pp"] > 1:
            raise SystemExit("checkpoint.init_from takes a whole-model file: shard it with parallel.tensor_parallel.shard_gpt2_state / "
                             "parallel.llama_parallel.shard_llama_state for tensor- or pipeline-parallel runs")
        ckpt.load_model(ck["init_from"], model)
        if hasattr(opt, "refresh_master"):
            opt.refresh_master()                              # fp32 master copies follow the loaded weights
    if ck["dir"]:
        os.makedirs(ck["dir"], exist_ok=True)
        base = os.path.join(ck["dir"], f"rank{rank:03d}")
        if ck["resume"] and dp_job and os.path.exists(dp_base + ".json"):
            with open(dp_base + ".json") as f:
                meta = json.load(f)
            ckpt.load_model(dp_base + ".cog", model)
            ckpt.load_dp_optimizer_resharded(dp_base, opt)    # whatever size the job that wrote them had
            opt.lr, start = meta["lr"], meta["step"]
        elif ck["resume"] and os.path.exists(base + ".state"):
            start = ckpt.load_training_state(base, model, opt)["step"]
    prof = Profiler(enabled=bool(cfg["profile"]))
    if cfg["profile"]:
        instrument(model, prof)
    log_f = open(cfg["log"]["path"], "a") if (cfg["log"]["path"] and logger) else None
    step, last = start, None
    sched = t["schedule"]
    if sched["kind"] == "exp" and start:
        exp_lr(opt, t["lr"], float(sched["gamma"]), start)
    fcfg, hb, failed = cfg["failure"], None, None
    if world > 1 and fcfg["heartbeat"]:
        from .utils.failure import Heartbeat, RankFailure, check_device
        hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world, interval=fcfg["interval_s"],
                       timeout=fcfg["timeout_s"]).start()
    t0 = time.time()
    t_mark, step_mark = None, start                                # the first interval (compilation, first-touch) is not a rate
    units_per_step = batch_rows * max(p["dp"], 1) * (1 if family in ("mlp", "cnn") else t["seq_len"])
    # a resumed run goes on with the batch after the last one it trained on, as an uninterrupted run would
    for x, y in itertools.islice(iter(batches), start, None):
        if step >= t["steps"]:
            break
        x, y = x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)
        if hb is None:
            loss = step_fn(x, y)
        else:
            try:
                hb.check()                                   # never enter a collective a dead peer cannot complete
                loss = hb.guard(step_fn, x, y)
                if fcfg["device_check_every"] and (step + 1) % fcfg["device_check_every"] == 0:
                    check_device()
            except RankFailure as e:
                failed = e
                break
        step += 1
        if sched["kind"] == "step":
            step_lr(opt, step, int(sched["step_size"]), float(sched["gamma"]))
        elif sched["kind"] == "exp":
            exp_lr(opt, t["lr"], float(sched["gamma"]), step)
        elif sched["kind"] is not None:
            raise SystemExit(f"unknown train.schedule.kind {sched['kind']}")
        prof.step_end()
        if loss is not None and step % cfg["log"]["every"] == 0:
            last = float(loss)                                   # waits for the step
            now = time.time()
            rec = {"step": step, "loss": last, "lr": float(opt.lr), "elapsed_s": round(now - t0, 3)}
            if t_mark is not None and now > t_mark:
                rec["per_s"] = round(units_per_step * (step - step_mark) / (now - t_mark), 1)      # tokens (samples for MLP / CNN) over the whole job
            t_mark, step_mark = now, step
            scaler = getattr(opt, "scaler", None)
            if scaler is not None and scaler.enabled:
                st = scaler.sync()
                rec["loss_scale"], rec["skipped"] = st["scale"], st["skipped"]
            if logger:
                print(json.dumps(rec), flush=True)
            if log_f:
                log_f.write(json.dumps(rec) + "\n")
                log_f.flush()
        if base and ck["every"] and step % ck["every"] == 0:
            save_state(step)
    if failed is not None:
        # the peers are gone: no collective, no barrier; the last periodic checkpoint is the restart point
        rec = {"event": "rank_failure", "rank": rank, "dead": failed.dead, "step": step, "detail": str(failed)}
        print(json.dumps(rec), flush=True)
        if log_f:
            log_f.write(json.dumps(rec) + "\n")
            log_f.close()
        hb.stop(announce=True)
        sys.stdout.flush()
        os._exit(3)
    if hb is not None:
        hb.stop(announce=True)
    if base:
        save_state(step)
    if cfg["profile"] and rank == 0:
        prof.report()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return last


def cmd_generate(cfg):
    from .models.llama import Llama, LlamaConfig
    from .serve.engine import LlamaInt4Engine, SpeculativeDecoder
    from .utils import rng
    dev = _device(cfg)
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    group = None
    if world > 1:                                                # under a launcher: tensor-parallel serving over all ranks
        if not dist.is_initialized():
            dist.init_process_group("nccl" if dev.type == "cuda" else "gloo", **({"device_id": dev} if dev.type == "cuda" else {}))
        group = dist.group.WORLD
    rng.manual_seed(cfg["seed"])
    m = cfg["model"]
    g = cfg.get("generate", {})
    dtype = torch.bfloat16 if dev.type == "cuda" else None
    tc = LlamaConfig(vocab_size=m["vocab_size"], n_layer=m["n_layer"], d_model=m["d_model"], n_head=m["n_head"],
                     n_kv_head=m["n_kv_head"] or m["n_head"], d_ff=m["d_ff"], max_seq_len=m["max_seq_len"])
    dc = LlamaConfig(vocab_size=m["vocab_size"], n_layer=g.get("draft_layers", 2), d_model=m["d_model"], n_head=m["n_head"],
                     n_kv_head=m["n_kv_head"] or m["n_head"], d_ff=m["d_ff"], max_seq_len=m["max_seq_len"])
    B, L, new = g.get("batch", 4), g.get("prompt_len", 16), g.get("new_tokens", 32)
    if g.get("prompts"):                                          # a JSON list of B token-id lists of equal length
        with open(g["prompts"]) as f:
            prompts = torch.tensor(json.load(f), dtype=torch.int64)
        if prompts.dim() != 2 or prompts.shape[0] != B:
            raise SystemExit(f"generate.prompts must hold {B} token lists of equal length")
        L = prompts.shape[1]
    else:
        prompts = torch.randint(0, m["vocab_size"], (B, L), generator=torch.Generator().manual_seed(cfg["seed"]))
    from .io import checkpoint as ckpt

    def engine(lc, weights, quantised):
        """generate.target_int4 / draft_int4: an engine file written by LlamaInt4Engine.save (one process only);
        generate.target_weights / draft_weights: a COG1 file of the full-precision model (save_model), quantised
        here; neither: random weights (a timing run)."""
        if quantised:
            if world > 1:
                raise SystemExit("an INT4 engine file holds one rank's unsplit engine: run one process, or give the full-precision weights")
            return LlamaInt4Engine.load(quantised, lc, B, device=dev, max_seq_len=L + new + 16)
        model = Llama(lc, device=dev, dtype=dtype)
        if weights:
            ckpt.load_model(weights, model)
        return LlamaInt4Engine(model, B, L + new + 16, tp_group=group)

    target = engine(tc, g.get("target_weights"), g.get("target_int4"))
    draft = engine(dc, g.get("draft_weights"), g.get("draft_int4"))
    if g.get("save_int4") and world == 1:                        # write the quantised engines for later runs
        target.save(g["save_int4"] + ".target.cog")
        draft.save(g["save_int4"] + ".draft.cog")
    dec = SpeculativeDecoder(draft, target, gamma=g.get("gamma", 4), temperature=g.get("temperature", 0.8), top_k=g.get("top_k", 50),
                             top_p=g.get("top_p", 0.9), seed=cfg["seed"])
    prompts = prompts.to(dev)
    t0 = time.time()
    seqs, stats = dec.generate(prompts, new)
    dt = time.time() - t0
    out = {"generated": stats.generated, "steps": stats.steps, "acceptance_rate": round(stats.acceptance_rate, 4),
           "tok_per_s": round(stats.generated / dt, 1), "tp": world}
    if rank == 0:
        if g.get("out"):                                         # the generated sequences (prompt + new tokens)
            with open(g["out"], "w") as f:
                json.dump([[int(v) for v in row] for row in (seqs.tolist() if torch.is_tensor(seqs) else seqs)], f)
        print(json.dumps(out))
    if world > 1:
        dec.close()
        dist.barrier()
        dist.destroy_process_group()
    return out


def cmd_info(_cfg):
    from . import __version__
    from .ops import _lib
    lib_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
    info = {"version": __version__, "torch": torch.__version__, "cuda": torch.cuda.is_available(),
            "kernel_library": _lib.available(), "host_library": os.path.exists(os.path.join(lib_dir, "libcogito.so")),
            "debug_kernel_library": os.path.exists(os.path.join(lib_dir, "libcogito_kernels_dbg.so"))}
    if torch.cuda.is_available():
        prop = torch.cuda.get_device_properties(0)
        info["device"] = prop.name
        info["devices"] = torch.cuda.device_count()
        info["sms"] = prop.multi_processor_count
        info["memory_gib"] = round(prop.total_memory / 2 ** 30, 1)
        info["compute_capability"] = f"{prop.major}.{prop.minor}"
        info["kernel_library_version"] = _lib.lib().cgk_version()
    print(json.dumps(info))
    return info


def main(argv=None):
    ap = argparse.ArgumentParser(prog="cogito_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command", choices=["train", "generate", "info"])
    ap.add_argument("--config", default=None)
    args, rest = ap.parse_known_args(argv)
    if args.config is None and rest and "=" not in rest[0] and not rest[0].startswith("-"):
        args.config, rest = rest[0], rest[1:]              # `train configs/x.yaml key=value ...`
    bad = [r for r in rest if "=" not in r or r.startswith("-")]
    if bad:
        ap.error(f"expected key.sub=value overrides, got {bad}")
    cfg = load_config(args.config, rest)
    return {"train": cmd_train, "generate": cmd_generate, "info": cmd_info}[args.command](cfg)


if __name__ == "__main__":
    main()
