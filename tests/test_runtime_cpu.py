"""Runtime services on CPU: COG1 checkpoints (Python <-> C library), exact resume, the
elementwise JIT, profiler, datasets, config CLI, failure detection and restart."""
import ctypes
import json
import os
import socket
import struct
from ctypes import POINTER, byref, c_char_p, c_int

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from capi_defs import L, T, TensorP, borrowed
from cogito_b200 import jit
from cogito_b200.cli import load_config, main as cli_main
from cogito_b200.data.datasets import BatchIterator, PrefetchLoader, SyntheticTokens, accuracy, horizontal_flip_, load_mnist, onehot
from cogito_b200.io import checkpoint as ckpt
from cogito_b200.models.gpt2 import GPT2, GPT2Config
from cogito_b200.optim.fused import FusedAdam
from cogito_b200.train import Trainer
from cogito_b200.utils import rng
from cogito_b200.utils.failure import Heartbeat, RankFailure, run_with_restarts
from cogito_b200.utils.profiler import Profiler, instrument


def test_checkpoint_files_are_interchangeable_with_the_c_library(tmp_path):
    lib = L()
    # C writes, Python reads
    a, b = T(np.arange(12, dtype=np.float32).reshape(3, 4)), T(np.array([0.5, -1.5], np.float32))
    p1 = str(tmp_path / "c.cog")
    lib.cg_save_model(p1.encode(), (TensorP * 2)(a._ptr, b._ptr), (c_char_p * 2)(b"w", b"b"), 2)
    got = ckpt.load_tensors(p1)
    assert list(got) == ["w", "b"] and torch.equal(got["w"], torch.arange(12.0).view(3, 4)) and got["b"].tolist() == [0.5, -1.5]
    # Python writes (fp32 + bf16 + packed int4), C reads the fp32 / bf16 entries
    p2 = str(tmp_path / "py.cog")
    w16 = torch.randn(4, 4).bfloat16()
    n = ckpt.save_tensors(p2, {"layer.w": torch.ones(2, 3), "layer.w16": w16})
    assert n == os.path.getsize(p2) and struct.unpack_from("<IIIIQ", open(p2, "rb").read(24)) == (0x434F4731, 1, 2, 0, n)
    ts, ns, cnt = POINTER(TensorP)(), POINTER(c_char_p)(), c_int()
    lib.cg_load_model(p2.encode(), byref(ts), byref(ns), byref(cnt))
    assert cnt.value == 2 and ns[1] == b"layer.w16"
    assert np.array_equal(borrowed(ts[1]), w16.float().numpy()) and borrowed(ts[0]).sum() == 6
    packed = torch.randint(0, 256, (8,), dtype=torch.uint8)
    ckpt.save_tensors(p2, {"q": packed, "q.scales": torch.ones(1)}, int4_shapes={"q": (4, 4)})
    back = ckpt.load_tensors(p2)
    assert torch.equal(back["q"], packed) and back["q"].logical_shape == (4, 4)
    with pytest.raises(ValueError):
        (tmp_path / "bad.cog").write_bytes(b"\0" * 64)
        ckpt.load_tensors(str(tmp_path / "bad.cog"))


def _tiny_trainer(seed=0):
    rng.manual_seed(seed)
    model = GPT2(GPT2Config(vocab_size=64, n_layer=1, d_model=32, n_head=2, d_ff=64, max_seq_len=16))
    return model, Trainer(model, FusedAdam(model.parameters(), lr=1e-2), micro_batch=2)


def test_resume_continues_the_same_trajectory(tmp_path):
    data = list(SyntheticTokens(64, 4, 16, steps=6, seed=3))
    model, tr = _tiny_trainer()
    for x, y in data[:3]:
        tr.step(x, y)
    base = str(tmp_path / "run")
    ckpt.save_training_state(base, model, tr.opt, step=3)
    tail = [float(tr.step(x, y)) for x, y in data[3:]]
    model2, tr2 = _tiny_trainer(seed=99)                 # different init: everything must come from the files
    meta = ckpt.load_training_state(base, model2, tr2.opt)
    assert meta["step"] == 3
    tail2 = [float(tr2.step(x, y)) for x, y in data[3:]]
    assert tail == tail2


def test_jit_traces_fuses_and_compiles_for_sm100a():
    f = jit.fuse(lambda x, b: jit.gelu(x + b) * 0.5 + (x + b) / (jit.exp(-x) + 1.0))
    x, b = torch.randn(6, 8), torch.randn(8)
    ref = torch.nn.functional.gelu(x + b, approximate="tanh") * 0.5 + (x + b) / (torch.exp(-x) + 1.0)
    assert torch.allclose(f(x, b), ref, atol=1e-6)
    src = f.source(x.bfloat16(), b)
    assert src.count("__global__") == 1 and src.count("(v0 + v1)") == 1          # one kernel, x + b computed once
    assert "__bfloat162float(in0[i % mod0])" in src and "in1[i % mod1]" in src
    assert len(jit.cubin_for(src)) > 1000                                         # NVRTC accepts it for sm_100a
    with pytest.raises((ValueError, RuntimeError)):
        f(torch.randn(6, 8), torch.randn(6))                                      # not a trailing-dimension broadcast


def test_profiler_and_instrumentation():
    model, tr = _tiny_trainer()
    prof = Profiler(nvtx=False)
    instrument(model, prof, depth=2)
    x, y = next(iter(SyntheticTokens(64, 2, 16, steps=1)))
    with prof.range("step"):
        tr.step(x, y)
    prof.step_end()
    assert prof.count("step") == 1 and prof.count("blocks.0") == 1 and prof.total_ms("step") >= prof.total_ms("blocks.0") > 0
    assert "blocks.0" in prof.report(file=open(os.devnull, "w")) and prof.steps == 1
    prof.reset()
    assert prof.count("step") == 0


def test_datasets_and_loaders(tmp_path):
    imgs = np.random.default_rng(0).integers(0, 256, (10, 4, 4), dtype=np.uint8)
    labs = np.arange(10, dtype=np.uint8)
    (tmp_path / "i").write_bytes(struct.pack(">IIII", 2051, 10, 4, 4) + imgs.tobytes())
    (tmp_path / "l").write_bytes(struct.pack(">II", 2049, 10) + labs.tobytes())
    x, y = load_mnist(str(tmp_path / "i"), str(tmp_path / "l"))
    assert x.shape == (10, 16) and torch.allclose(x, torch.from_numpy(imgs.reshape(10, 16) / 255.0).float()) and y.tolist() == list(range(10))
    it = BatchIterator(x, y, 4, shuffle=True, seed=1)
    e1 = [b[1].tolist() for b in it]
    e2 = [b[1].tolist() for b in it]
    assert [len(b) for b in e1] == [4, 4, 2] and sorted(sum(e1, [])) == list(range(10)) and e1 != e2
    assert [b[0].shape[0] for b in PrefetchLoader(BatchIterator(x, y, 4, shuffle=False), "cpu")] == [4, 4, 2]
    oh = onehot(y, 10)
    assert accuracy(oh, y) == 1.0 and accuracy(oh.roll(1, 1), y) == 0.0
    flipped = horizontal_flip_(x.clone(), 1.0)
    assert torch.equal(flipped.view(10, 4, 4), x.view(10, 4, 4).flip(-1))
    with pytest.raises(ValueError):
        load_mnist(str(tmp_path / "l"), str(tmp_path / "i"))


def test_cli_config_merge_and_train(tmp_path, capsys):
    cfg_file = tmp_path / "c.yaml"
    cfg_file.write_text("device: cpu\nmodel: {family: gpt2, vocab_size: 64, n_layer: 1, d_model: 32, n_head: 2, d_ff: 64, max_seq_len: 16}\n"
                        "train: {steps: 3, batch: 2, seq_len: 16, loss_scale: null}\n")
    cfg = load_config(str(cfg_file), ["train.lr=0.01", f"checkpoint.dir={tmp_path}/ck", "log.path=" + str(tmp_path / "log.jsonl")])
    assert cfg["train"]["lr"] == 0.01 and cfg["model"]["n_layer"] == 1 and cfg["parallel"]["tp"] == 1
    cli_main(["train", "--config", str(cfg_file), f"checkpoint.dir={tmp_path}/ck", "log.path=" + str(tmp_path / "log.jsonl")])
    recs = [json.loads(l) for l in open(tmp_path / "log.jsonl")]
    assert [r["step"] for r in recs] == [1, 2, 3] and os.path.exists(tmp_path / "ck" / "rank000.state")
    # resume: starts at step 3, so two more steps of a 5-step run
    cli_main(["train", "--config", str(cfg_file), f"checkpoint.dir={tmp_path}/ck", "checkpoint.resume=true", "train.steps=5",
              "log.path=" + str(tmp_path / "log2.jsonl")])
    resumed = [json.loads(l) for l in open(tmp_path / "log2.jsonl")]
    assert [r["step"] for r in resumed] == [4, 5]
    # the resumed run continues the data stream: same losses as five steps in one go
    cli_main(["train", "--config", str(cfg_file), "train.steps=5", "log.path=" + str(tmp_path / "log3.jsonl")])
    whole = [json.loads(l) for l in open(tmp_path / "log3.jsonl")]
    assert [r["loss"] for r in whole[3:]] == pytest.approx([r["loss"] for r in resumed], rel=1e-6)


def test_convolutional_classifier_trains_from_the_command_line_and_matches_torch_gradients(tmp_path):
    from cogito_b200.models.cnn import ConvClassifier
    from cogito_b200.utils import rng
    # the shipped configuration, config path given positionally, a few steps
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cli_main(["train", os.path.join(root, "configs", "mnist_cnn_cpu.yaml"), "train.steps=25", "log.path=" + str(tmp_path / "cnn.jsonl")])
    losses = [json.loads(l)["loss"] for l in open(tmp_path / "cnn.jsonl")]
    assert len(losses) == 25 and sum(losses[-5:]) / 5 < 0.7 * sum(losses[:3]) / 3, losses
    # gradients of the whole stack against the same network written with torch.nn.functional
    rng.manual_seed(3)
    m = ConvClassifier(2, 8, (3, 5), 4)
    x, y = torch.randn(6, 2, 8, 8), torch.randint(0, 4, (6,))
    m(x, y).backward()
    ps = {k: v.detach().clone().requires_grad_(True) for k, v in m.named_parameters()}
    h = x
    for i, (ic, oc) in enumerate(((2, 3), (3, 5))):
        h = torch.nn.functional.conv2d(h, ps[f"convs.{i}.weight"].view(oc, ic, 3, 3), ps[f"convs.{i}.bias"], padding=1)
        h = torch.nn.functional.batch_norm(h, None, None, ps[f"norms.{i}.weight"], ps[f"norms.{i}.bias"], training=True, eps=1e-5)
        h = torch.nn.functional.max_pool2d(torch.relu(h), 2)
    logits = h.flatten(1) @ ps["head.weight"].T + ps["head.bias"]
    torch.nn.functional.cross_entropy(logits, y).backward()
    for k, v in m.named_parameters():
        assert torch.allclose(v.grad, ps[k].grad, atol=1e-5, rtol=1e-4), k


# ------------------------------------------------------------ failure detection
class DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d.get(k)


def test_heartbeat_detects_silent_and_exited_ranks():
    store, now = DictStore(), [100.0]
    hbs = [Heartbeat(store, r, 3, interval=0, timeout=5.0, clock=lambda: now[0]).start() for r in range(3)]
    hbs[0].check()
    now[0] = 103.0
    hbs[0].beat(); hbs[1].beat()                         # rank 2 goes silent
    now[0] = 107.0
    hbs[0].beat()
    assert hbs[0].dead_ranks() == [2]
    with pytest.raises(RankFailure) as e:
        hbs[0].check()
    assert e.value.dead == [2]
    hbs[1].stop()                                        # announced exit is seen at once
    assert hbs[0].dead_ranks() == [1, 2]


def test_guard_turns_a_transport_error_into_a_rank_failure_only_when_a_peer_is_dead():
    store = DictStore()
    hbs = [Heartbeat(store, r, 2, interval=0, timeout=0.2).start() for r in range(2)]

    def broken():
        raise RuntimeError("Connection reset by peer")

    assert hbs[0].guard(lambda a: a + 1, 1) == 2
    hbs[1].announce_exit()                               # the peer left while we were inside the collective
    with pytest.raises(RankFailure) as e:
        hbs[0].guard(broken)
    assert e.value.dead == [1]
    hbs[1].beat()                                        # alive again: the error is not a rank failure
    with pytest.raises(RuntimeError, match="Connection reset"):
        Heartbeat(store, 0, 1, interval=0, timeout=0.1).start().guard(broken)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _elastic_worker(rank, world, port, tmp, q):
    import torch.distributed as dist
    from datetime import timedelta
    torch.set_num_threads(1)
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=timedelta(seconds=60))
    state = {"ranks": list(range(world))}
    losses = []

    def make_group(attempt, dead):
        if dist.is_initialized():
            dist.destroy_process_group()
        state["ranks"] = [r for r in state["ranks"] if r not in dead]
        if rank not in state["ranks"]:
            return None
        sub = dist.PrefixStore(f"attempt{attempt}", store)
        dist.init_process_group("gloo", store=sub, rank=state["ranks"].index(rank), world_size=len(state["ranks"]),
                                timeout=timedelta(seconds=20))
        hb = Heartbeat(dist.PrefixStore(f"hb{attempt}", store), state["ranks"].index(rank), len(state["ranks"]), interval=0.1, timeout=4.0).start()
        return {"hb": hb, "attempt": attempt}

    def train(info):
        hb = info["hb"]
        model, tr = _tiny_trainer()
        base = os.path.join(tmp, f"r{rank}")
        start = ckpt.load_training_state(base, model, tr.opt)["step"] if os.path.exists(base + ".state") else 0
        data = list(SyntheticTokens(64, 2, 16, steps=8, seed=5))
        for step in range(start, 8):
            if rank == 1 and step == 4 and info["attempt"] == 0:
                hb.stop()                                # leaves between steps, nothing in flight
                os._exit(0)
            hb.check()                                   # host-side check before entering collectives
            loss = tr.step(*data[step])
            for p in model.parameters():                 # data-parallel gradient agreement check
                pass
            v = loss.detach().clone()
            hb.guard(dist.all_reduce, v)                  # a rank that left mid-collective surfaces as RankFailure too
            losses.append((info["attempt"], step, float(v) / dist.get_world_size()))
            ckpt.save_training_state(base, model, tr.opt, step + 1)
            import time
            time.sleep(0.05)
        hb.stop()
        return losses

    try:
        out = run_with_restarts(train, make_group, max_restarts=2)
        q.put((rank, out))
    except Exception as e:                               # pragma: no cover - reported to the parent
        q.put((rank, repr(e)))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_survivors_detect_a_lost_rank_and_resume_from_the_checkpoint(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_elastic_worker, args=(r, 3, port, str(tmp_path), q)) for r in range(3)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))     # rank 1 exits without reporting
    for p in procs:
        p.join(timeout=60)
    assert set(res) == {0, 2}
    for rank, out in res.items():
        assert isinstance(out, list), out
        steps0 = [s for a, s, _ in out if a == 0]
        steps1 = [s for a, s, _ in out if a == 1]
        assert steps0 and steps1 and max(steps0) >= 3 and steps1[-1] == 7
        assert steps1[0] == max(steps0) + 1 or steps1[0] == max(steps0)      # resumed where the checkpoint left off
        assert sorted(set(steps0 + steps1)) == list(range(8))


def test_python_examples_train_on_the_cpu():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "examples", "xor.py")], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "final loss 0.0000" in p.stdout, p.stdout[-500:] + p.stderr[-500:]
    p = subprocess.run([sys.executable, os.path.join(root, "examples", "mnist_mlp.py"), "--epochs", "2", "--samples", "512", "--batch", "64"],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "accuracy 1.000" in p.stdout.splitlines()[-1], p.stdout[-500:] + p.stderr[-500:]


def test_cli_trains_the_3d_parallel_llama_on_eight_cpu_ranks_and_reports_from_the_last_stage(tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    log = tmp_path / "3d.jsonl"
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "8", "--master-addr", "127.0.0.1",
                        "--master-port", str(_free_port()), "-m", "cogito_b200", "train", os.path.join(root, "configs", "llama_tiny_3d_cpu.yaml"),
                        "train.steps=3", f"log.path={log}"], capture_output=True, text=True, timeout=600, cwd=root)
    assert p.returncode == 0, p.stderr[-1500:]
    recs = [json.loads(l) for l in open(log)]
    assert [r["step"] for r in recs] == [1, 2, 3] and all(5.0 < r["loss"] < 7.5 for r in recs)       # ln(512) = 6.24 at the start
    assert len([l for l in p.stdout.splitlines() if l.startswith("{")]) == 3                         # one rank prints


def test_cli_generate_runs_alone_and_tensor_parallel_on_two_cpu_ranks():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    over = ["device=cpu", "model.vocab_size=512", "model.n_layer=2", "model.d_model=128", "model.n_head=4", "model.n_kv_head=2",
            "model.d_ff=256", "model.max_seq_len=128", "generate.batch=2", "generate.prompt_len=8", "generate.new_tokens=10",
            "generate.draft_layers=1"]
    cfg = os.path.join(root, "configs", "spec_decode_int4.yaml")
    one = cli_main(["generate", cfg] + over)
    assert one["generated"] >= 2 * 10 and one["tp"] == 1 and 0.0 <= one["acceptance_rate"] <= 1.0
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", str(_free_port()), "-m", "cogito_b200", "generate", cfg] + over, capture_output=True, text=True, timeout=600, cwd=root)
    assert p.returncode == 0, p.stderr[-1500:]
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1 and lines[0]["tp"] == 2 and lines[0]["generated"] >= 2 * 10


def _cli_failure_worker(rank, port, tmp):
    """Two data-parallel CLI ranks; rank 1 is told to train two steps only and leaves the job there
    (its closing barrier is replaced by an exit: a rank that is gone, not one that waits)."""
    import torch.distributed as dist
    os.environ.update(RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    sys_stdout = open(os.path.join(tmp, f"out{rank}.txt"), "w")
    os.dup2(sys_stdout.fileno(), 1)
    if rank == 1:
        dist.barrier = lambda *a, **k: os._exit(0)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cli_main(["train", os.path.join(root, "configs", "tiny_cpu.yaml"), "parallel.dp=2", f"train.steps={2 if rank == 1 else 40}",
              "failure.heartbeat=true", "failure.interval_s=0.1", "failure.timeout_s=3.0"])
    os._exit(0)


def test_cli_with_heartbeats_ends_with_code_3_and_an_event_when_a_rank_leaves(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_cli_failure_worker, args=(r, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    assert procs[1].exitcode == 0 and procs[0].exitcode == 3, [p.exitcode for p in procs]
    recs = [json.loads(l) for l in open(tmp_path / "out0.txt") if l.startswith("{")]
    assert [r["step"] for r in recs if "loss" in r][:2] == [1, 2]
    ev = [r for r in recs if r.get("event") == "rank_failure"]
    assert len(ev) == 1 and ev[0]["dead"] == [1] and 2 <= ev[0]["step"] < 40


def test_cli_data_parallel_checkpoints_resume_exactly_and_on_a_smaller_group(tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(ranks, steps, *extra):
        p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(ranks), "--master-addr",
                            "127.0.0.1", "--master-port", str(_free_port()), "-m", "cogito_b200", "train",
                            os.path.join(root, "configs", "tiny_cpu.yaml"), "train.batch=6", f"train.steps={steps}", f"parallel.dp={ranks}",
                            *extra], capture_output=True, text=True, timeout=600, cwd=root)
        assert p.returncode == 0, p.stderr[-1500:]
        return {r["step"]: r["loss"] for r in (json.loads(l) for l in p.stdout.splitlines() if l.startswith("{"))}

    whole = run(3, 4)
    ck = f"checkpoint.dir={tmp_path}/ck"
    first = run(3, 2, ck)
    assert first[2] == whole[2]
    same = run(3, 4, ck, "checkpoint.resume=true")
    assert sorted(same) == [3, 4] and same[3] == whole[3] and same[4] == whole[4]        # same group: the same run
    assert sorted(f for f in os.listdir(tmp_path / "ck") if "of" in f) == [f"dp.opt.dp0{r}of03.state" for r in range(3)]
    fewer = run(2, 6, ck, "checkpoint.resume=true")                                       # one rank fewer: shards re-cut
    assert sorted(fewer) == [5, 6] and all(4.5 < v < 6.5 for v in fewer.values())
    assert sorted(f for f in os.listdir(tmp_path / "ck") if "of" in f) == [f"dp.opt.dp0{r}of02.state" for r in range(2)]


def test_cli_generate_from_saved_weights_prompts_and_int4_engine_files(tmp_path):
    import cogito_b200 as cg
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = os.path.join(root, "configs", "spec_decode_int4.yaml")
    shape = dict(vocab_size=512, d_model=128, n_head=4, n_kv_head=2, d_ff=256, max_seq_len=128)
    over = ["device=cpu"] + [f"model.{k}={v}" for k, v in shape.items()] + ["model.n_layer=2", "generate.batch=2", "generate.new_tokens=8",
                                                                                  "generate.draft_layers=1"]
    cg.manual_seed(0)
    target, draft = cg.Llama(cg.LlamaConfig(n_layer=2, **shape)), cg.Llama(cg.LlamaConfig(n_layer=1, **shape))
    cg.save_model(str(tmp_path / "t.cog"), target)
    cg.save_model(str(tmp_path / "d.cog"), draft)
    (tmp_path / "p.json").write_text(json.dumps([[1, 2, 3, 4, 5], [6, 7, 8, 9, 10]]))
    common = [f"generate.prompts={tmp_path}/p.json"]
    a = cli_main(["generate", cfg] + over + common + [f"generate.target_weights={tmp_path}/t.cog", f"generate.draft_weights={tmp_path}/d.cog",
                                                       f"generate.out={tmp_path}/a.json", f"generate.save_int4={tmp_path}/eng"])
    b = cli_main(["generate", cfg] + over + common + [f"generate.target_int4={tmp_path}/eng.target.cog", f"generate.draft_int4={tmp_path}/eng.draft.cog",
                                                       f"generate.out={tmp_path}/b.json"])
    sa, sb = json.load(open(tmp_path / "a.json")), json.load(open(tmp_path / "b.json"))
    assert sa == sb and a["generated"] == b["generated"]                     # the engine files hold exactly what was quantised
    assert [s[:5] for s in sa] == [[1, 2, 3, 4, 5], [6, 7, 8, 9, 10]] and all(len(s) >= 5 + 8 for s in sa)


def test_cli_starts_training_from_a_model_file(tmp_path):
    import cogito_b200 as cg
    from cogito_b200.data.datasets import SyntheticTokens
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = os.path.join(root, "configs", "tiny_cpu.yaml")
    cli_main(["train", cfg, "train.steps=3", f"checkpoint.dir={tmp_path}/ck"])
    got = cli_main(["train", cfg, "train.steps=1", "train.lr=0.0", f"checkpoint.init_from={tmp_path}/ck/rank000.cog"])
    cg.manual_seed(0)
    model = cg.GPT2(cg.GPT2Config(vocab_size=256, n_layer=2, d_model=64, n_head=4, d_ff=128, max_seq_len=64))
    cg.load_model(str(tmp_path / "ck" / "rank000.cog"), model)
    x, y = next(iter(SyntheticTokens(256, 4, 32, 1, seed=0)))
    assert got == pytest.approx(float(model(x, y)), rel=1e-5)


def test_cli_learning_rate_schedules(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = os.path.join(root, "configs", "tiny_cpu.yaml")
    cli_main(["train", cfg, "train.steps=4", "train.lr=0.01", "train.schedule.kind=step", "train.schedule.step_size=2", "train.schedule.gamma=0.5",
              f"log.path={tmp_path}/a.jsonl"])
    assert [json.loads(l)["lr"] for l in open(tmp_path / "a.jsonl")] == pytest.approx([0.01, 0.005, 0.005, 0.0025])
    cli_main(["train", cfg, "train.steps=3", "train.lr=0.01", "train.schedule.kind=exp", "train.schedule.gamma=0.9", f"log.path={tmp_path}/b.jsonl"])
    assert [json.loads(l)["lr"] for l in open(tmp_path / "b.jsonl")] == pytest.approx([0.009, 0.0081, 0.00729])
