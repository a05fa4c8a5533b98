"""Worker of the multi-GPU tests: run under torchrun, one rank per GPU.

    torchrun --nproc-per-node N tests/mgpu_worker.py <mode> [dp tp pp]

mode tp  : tensor-parallel GPT-2 (fused all-gather->GEMM / GEMM->reduce-scatter) against the
           single-device model trained on the same batch
mode dp  : fused all-reduce + Adam optimizer step against the single-device full-batch run
mode 3d  : DP x TP x PP Llama (1F1B; a fourth number > 1 = chunks per rank, interleaved 1F1B) against the
           single-device model
mode serve: tensor-parallel INT4 engine and speculative decoder against the unsplit engine
Every rank prints one line "RESULT <json>"; the test reads rank 0's.
"""
import json
import os
import sys

import torch
import torch.distributed as dist


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from cogito_b200.ops import _lib
    from cogito_b200.optim.fused import FusedAdam
    from cogito_b200.train import Trainer
    from cogito_b200.utils.rng import manual_seed
    manual_seed(0)
    out = {"mode": mode, "world": world}
    g = torch.Generator().manual_seed(1)
    if mode == "tp":
        from cogito_b200.models.gpt2 import GPT2, GPT2Config
        from cogito_b200.parallel.tensor_parallel import build_tp_gpt2, shard_gpt2_state
        heads = world + world // 2                 # head_dim 64; uneven on purpose (8 ranks: 12 heads, dealt 2,2,2,2,1,1,1,1)
        mb = max(2, world // 2)                    # every rank keeps at least 128 rows of a micro-batch
        cfg = GPT2Config(vocab_size=1024 * world, n_layer=2, d_model=64 * heads, n_head=heads, d_ff=256 * heads, max_seq_len=256)
        full = GPT2(cfg, device=dev, dtype=torch.bfloat16)
        tp, sync = build_tp_gpt2(cfg, rank, world, dev, dist.group.WORLD, micro_tokens=mb * 256)
        shard_gpt2_state(full, tp)
        ids = torch.randint(0, cfg.vocab_size, (2 * mb, 256), generator=g).to(dev)
        tg = torch.randint(0, cfg.vocab_size, (2 * mb, 256), generator=g).to(dev)
        of, ot = FusedAdam(full.parameters(), lr=1e-3), FusedAdam(tp._ordered, lr=1e-3)
        sync.attach(ot)
        tf, tt = Trainer(full, of, micro_batch=mb), Trainer(tp, ot, micro_batch=mb, parallel=sync)
        out["ref"] = [float(tf.step(ids, tg)) for _ in range(4)]
        out["got"] = [float(tt.step(ids, tg)) for _ in range(4)]
    elif mode == "dp":
        from cogito_b200.models.gpt2 import GPT2, GPT2Config
        from cogito_b200.parallel.data_parallel import DPFusedAdam
        cfg = GPT2Config(vocab_size=2048, n_layer=2, d_model=256, n_head=4, d_ff=1024, max_seq_len=128)
        full = GPT2(cfg, device=dev, dtype=torch.bfloat16)
        mine = GPT2(cfg, device=dev, dtype=torch.bfloat16)
        mine.load_state_dict(full.state_dict())
        ids = torch.randint(0, 2048, (2 * world, 128), generator=g).to(dev)
        tg = torch.randint(0, 2048, (2 * world, 128), generator=g).to(dev)
        tf = Trainer(full, FusedAdam(full.parameters(), lr=1e-3), micro_batch=2)
        # several buckets (the last one short), as a full-size model has: every bucket runs its own handshake
        td = Trainer(mine, DPFusedAdam(mine.parameters(), dist.group.WORLD, lr=1e-3, bucket_elems=300_000), micro_batch=2)
        out["ref"] = [float(tf.step(ids, tg)) for _ in range(4)]
        got = []
        for _ in range(4):
            loss = td.step(ids[2 * rank:2 * rank + 2], tg[2 * rank:2 * rank + 2]).detach().float()
            dist.all_reduce(loss)
            got.append(float(loss) / world)
        out["got"] = got
    elif mode == "3d":
        dp, tp, pp = (int(a) for a in sys.argv[2:5])
        virtual = int(sys.argv[5]) if len(sys.argv) > 5 else 1      # chunks per pipeline rank (interleaved 1F1B)
        scaled = len(sys.argv) > 6 and sys.argv[6] == "scaled"       # loss scaling and clipping on: replica-wide statistics
        recompute = sys.argv[7] if len(sys.argv) > 7 and sys.argv[7] in ("block", "stage") else None
        from cogito_b200.optim.fused import GradScaler
        from cogito_b200.models.llama import Llama, LlamaConfig
        from cogito_b200.parallel.groups import init_parallel
        from cogito_b200.parallel.llama_parallel import Trainer3D, shard_llama_state
        cfg = LlamaConfig(vocab_size=2048, n_layer=4, d_model=256, n_head=4, n_kv_head=2, d_ff=512, max_seq_len=256)
        full = Llama(cfg, device=dev, dtype=torch.bfloat16)
        ctx = init_parallel(dp, tp, pp)
        M, mb, T = 4, 1, 256
        t3 = Trainer3D(cfg, ctx, dev, num_microbatches=M, micro_batch=mb, seq_len=T, lr=1e-3, loss_scale=1024.0 if scaled else None,
                       max_grad_norm=1.0 if scaled else 0.0, virtual_stages=virtual, recompute=recompute)
        t3.load_from(full)
        ids = torch.randint(0, 2048, (dp * M * mb, T), generator=g).to(dev)
        tg = torch.randint(0, 2048, (dp * M * mb, T), generator=g).to(dev)
        ref_opt = FusedAdam(full.parameters(), lr=1e-3, scaler=GradScaler(dev, init_scale=1024.0), max_grad_norm=1.0) if scaled \
            else FusedAdam(full.parameters(), lr=1e-3)
        tf = Trainer(full, ref_opt, micro_batch=mb)
        out["ref"] = [float(tf.step(ids, tg)) for _ in range(3)]
        d = ctx.coords.dp_rank
        got = []
        for _ in range(3):
            loss = t3.step(ids[d * M * mb:(d + 1) * M * mb], tg[d * M * mb:(d + 1) * M * mb])
            v = torch.zeros(2, device=dev)
            if loss is not None and ctx.coords.tp_rank == 0:
                v[0], v[1] = loss.float(), 1.0
            dist.all_reduce(v)
            got.append(float(v[0] / v[1]))
        out["got"] = got
        out["p2p_bytes"] = t3.pipe.p2p_bytes
        out["peak_mem_mb"] = torch.cuda.max_memory_allocated(dev) / 2 ** 20
        out["fused_dp"] = type(t3.opt).__name__
    elif mode == "serve":
        # tensor-parallel INT4 engine (fused all-reduce + residual + RMSNorm over peer memory) against
        # the unsplit engine on the same GPU; head_dim 128 keeps every slice on a weight-group boundary
        from cogito_b200.models.llama import Llama, LlamaConfig
        from cogito_b200.serve.engine import LlamaInt4Engine, SpeculativeDecoder
        cfg = LlamaConfig(vocab_size=2048, n_layer=2, d_model=128 * world, n_head=world, n_kv_head=world, d_ff=256 * world, max_seq_len=256)
        dcfg = LlamaConfig(vocab_size=2048, n_layer=1, d_model=128 * world, n_head=world, n_kv_head=world, d_ff=128 * world, max_seq_len=256)
        target = Llama(cfg, device=dev, dtype=torch.bfloat16)
        draft = Llama(dcfg, device=dev, dtype=torch.bfloat16)
        one = LlamaInt4Engine(target, batch=4)
        tp = LlamaInt4Engine(target, batch=4, tp_group=dist.group.WORLD)
        prompt = torch.randint(0, 2048, (4, 40), generator=g).to(dev)
        a, b = one.forward(prompt, commit=True), tp.forward(prompt, commit=True)
        nxt = torch.randint(0, 2048, (4, 5), generator=g).to(dev)
        a2, b2 = one.forward(nxt), tp.forward(nxt)
        scale = float(a.abs().max())
        out["ref"] = [0.0, 0.0]
        out["got"] = [float((a - b).abs().max()) / scale, float((a2 - b2).abs().max()) / scale]
        dec = SpeculativeDecoder(LlamaInt4Engine(draft, batch=4, tp_group=dist.group.WORLD), tp, gamma=3, temperature=0.8, top_k=20, top_p=0.9, seed=5)
        seqs, stats = dec.generate(prompt, 16)
        flat = torch.tensor([t for s in seqs for t in s[:56]], device=dev, dtype=torch.int64)
        lo, hi = flat.clone(), flat.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        out["tokens_agree"] = bool((lo == hi).all())
        out["fused"] = bool(tp.ar.fused)
        out["acceptance"] = stats.acceptance_rate
        out["graph"] = dec._graph is not None
        dec.close()                               # the captured step holds collectives of the process group
    else:
        raise SystemExit(f"unknown mode {mode}")
    out["status"] = list(_lib.read_status())
    # guard regions around every symmetric buffer (COGITO_SYMM_CANARY=1): no peer stored out of range
    torch.cuda.synchronize()
    dist.barrier()
    from cogito_b200.parallel.symm import check_all_canaries
    out["canaries_ok"] = check_all_canaries()
    print("RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
