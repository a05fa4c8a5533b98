"""INT4 speculative-decoding benchmark (serving configuration of the baseline list).

    python benchmarks/spec_decode.py [--layers 32] [--batch 16] [--prompt 512] [--new 256] [--gamma 4]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/spec_decode.py   # TP=8

Target: Llama-7B-shaped model (32 layers, d_model 4096, 32 query / 8 KV heads, d_ff 11008, vocabulary 32000) with
INT4 weights in groups of 128 and an INT4 KV cache; draft: 2 layers of the same width; random
weights (N(0, 0.02)) and uniform random prompts.  gamma drafted tokens per step, temperature 0.8,
top-k 50, top-p 0.9.  One JSON line from rank 0: decode tokens/s over all sequences (device time of
the decode loop, max over ranks), prefill time, acceptance rate, launches per step.  With random
weights the draft seldom agrees with the target, so the acceptance rate is that of unrelated
models; ``--self-draft`` uses the target's first layers as the draft to show the accepted-path cost.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run(layers=32, draft_layers=2, batch=16, prompt=512, new=256, gamma=4, kv_heads=8, self_draft=False,
        tp_graph=False, no_graph=False, group=None, dev=None):
    """Builds the engines, runs one prefill and the decode loop, returns the result record (the same
    on every rank).  ``group``: the tensor-parallel process group, None on one GPU."""
    from cogito_b200.models.llama import Llama, LlamaConfig
    from cogito_b200.ops import _lib
    from cogito_b200.serve.engine import LlamaInt4Engine, SpeculativeDecoder
    from cogito_b200.utils import rng

    world = dist.get_world_size(group) if group is not None else 1
    rng.manual_seed(0)
    shape = dict(vocab_size=32000, d_model=4096, n_head=32, n_kv_head=kv_heads, d_ff=11008, max_seq_len=prompt + new + 64)
    tcfg = LlamaConfig(n_layer=layers, **shape)
    dcfg = LlamaConfig(n_layer=draft_layers, **shape)
    cap = prompt + new + 32
    # build and quantise one model at a time: the bf16 copy is dropped once its INT4 engine exists
    model = Llama(tcfg, device=dev, dtype=torch.bfloat16)
    target = LlamaInt4Engine(model, batch, cap, tp_group=group)
    if self_draft:
        model.blocks = model.blocks[:draft_layers]
        draft = LlamaInt4Engine(model, batch, cap, tp_group=group)
    else:
        del model
        draft = LlamaInt4Engine(Llama(dcfg, device=dev, dtype=torch.bfloat16), batch, cap, tp_group=group)
    model = None
    torch.cuda.empty_cache()
    dec = SpeculativeDecoder(draft, target, gamma=gamma, temperature=0.8, top_k=50, top_p=0.9, seed=0,
                             use_graph=False if no_graph else (True if tp_graph else None))
    prompts = torch.randint(0, 32000, (batch, prompt), generator=torch.Generator().manual_seed(1)).to(dev)

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    dec.generate(prompts[:, :32], 8)                        # warm-up: tile reordering, workspaces
    dec.stats.__init__()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(group)
    _lib.reset_launches()
    ev[0].record()
    last = dec.prefill(prompts)
    ev[1].record()
    produced, steps, generated, accepted = 0, 0, 0, 0
    while produced < new:
        n_acc, out, nxt = dec.advance(last)
        n_host = n_acc.tolist()                              # the per-step host read a serving loop needs to emit tokens
        last = nxt.clone()
        produced += min(n_host) + 1
        generated += sum(n + 1 for n in n_host)
        accepted += sum(n_host)
        steps += 1
    ev[2].record()
    torch.cuda.synchronize()
    t = torch.tensor([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    prefill_ms, decode_ms = t.tolist()
    rec = {
        "metric": "int4_speculative_decode_tokens_per_s", "value": round(generated / decode_ms * 1e3, 1), "unit": "tokens/s",
        "n_gpus": world, "decode_ms": round(decode_ms, 2), "prefill_ms": round(prefill_ms, 2), "steps": steps,
        "ms_per_step": round(decode_ms / steps, 3), "acceptance_rate": round(accepted / (steps * batch * gamma), 4),
        "generated": generated, "cuda_graph": dec._graph is not None,
        "launches_per_step": getattr(dec, "graph_launches", None) if dec._graph is not None else round(_lib.launches() / max(1, steps), 1),
        "weight_bytes_per_gpu": target.weight_bytes() + draft.weight_bytes(),
        "config": {"layers": layers, "draft_layers": draft_layers, "batch": batch, "prompt": prompt, "new": new,
                   "gamma": gamma, "kv_heads": kv_heads, "tp": world, "self_draft": self_draft, "data": "synthetic"}}
    dec.close()                                           # drop the captured collectives before the process group goes
    del dec, target, draft
    torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--draft-layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--gamma", type=int, default=4)
    ap.add_argument("--kv-heads", type=int, default=8, help="KV heads of the target (grouped-query attention: 32 query heads share them)")
    ap.add_argument("--self-draft", action="store_true")
    ap.add_argument("--tp-graph", action="store_true", help="replay the step from a CUDA graph under tensor parallelism too")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    rec = run(args.layers, args.draft_layers, args.batch, args.prompt, args.new, args.gamma, args.kv_heads, args.self_draft,
              args.tp_graph, args.no_graph, group, dev)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
