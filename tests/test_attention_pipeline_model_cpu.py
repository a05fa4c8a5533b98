"""Host models of the mbarrier pipelines inside the flash-attention kernels, checked without a GPU.

The kernels (csrc/kernels/flash_fwd.cu, flash_bwd_kernel.cuh) are sets of roles - a TMA producer,
several MMA-issuing threads, softmax / compute warpgroups, a dQ drain warpgroup - that meet only
at mbarriers.  Here every role is a sequential program of atomic steps, asynchronous work (TMA
loads, the MMAs a thread has issued, bulk reductions) completes at arbitrary later points, and the
explorer walks EVERY interleaving of a small instance (depth-first over the reachable states).
It reports

* a deadlock (no role can move and not all are finished),
* a lost phase: an mbarrier that completes two phases while a role still waits for the first
  (a parity wait cannot tell them apart),
* a data hazard: a buffer overwritten while an MMA or a copy in flight still reads it, a tile
  read before it was produced, an accumulator rewritten before its reader took it.

The programs below restate the waits, arrivals and commits of the kernels step by step; the
negative cases remove one of them and the explorer must find the resulting hazard.
"""
import pytest


class Model:
    """barriers: name -> arrival count.  roles: name -> list of steps.  Steps:
    ("wait", bar, k)               block until phase k of bar has completed
    ("arrive", bar)
    ("write", buf, version)        synchronous write (generic-proxy stores, tcgen05.st)
    ("read", buf, version)         synchronous read (tcgen05.ld); marks the buffer as taken
    ("tma", buf, version, bar)     asynchronous write; arrives on bar when it lands
    ("mma", queue, reads, writes)  asynchronous: reads = ((buf, version), ...), writes = ((buf, version), ...)
    ("commit", queue, bar)         arrives on bar once everything issued earlier on the queue is done
    ("copy_out", buf)              asynchronous read of buf (bulk store / reduction from shared memory)
    ("wait_copies", buf)           block until no copy_out of buf is in flight
    ("bulk_store", group_queue, buf)  asynchronous read of buf, one bulk async-group of its own on that queue
    ("wait_group", group_queue, n)    block until all but the n most recent groups of the queue have read their source
    """

    def __init__(self, barriers, roles, check_taken=()):
        self.bars = list(barriers)
        self.count = [barriers[b] for b in self.bars]
        self.bidx = {b: i for i, b in enumerate(self.bars)}
        self.roles = list(roles)
        self.prog = [roles[r] for r in self.roles]
        bufs, queues = set(), set()
        for p in self.prog:
            for st in p:
                if st[0] in ("write", "read", "tma", "copy_out", "wait_copies"):
                    bufs.add(st[1])
                if st[0] == "bulk_store":
                    bufs.add(st[2])
                if st[0] == "mma":
                    queues.add(st[1])
                    bufs.update(b for b, _ in st[2])
                    bufs.update(b for b, _ in st[3])
                if st[0] == "commit":
                    queues.add(st[1])
        self.bufs = sorted(bufs)
        self.fidx = {b: i for i, b in enumerate(self.bufs)}
        self.queues = sorted(queues)
        self.qidx = {q: i for i, q in enumerate(self.queues)}
        self.check_taken = {self.fidx[b] for b in check_taken if b in self.fidx}     # accumulators: must be read before they are rewritten
        self.groups = sorted({st[1] for p in self.prog for st in p if st[0] in ("bulk_store", "wait_group")})
        self.gidx = {g: i for i, g in enumerate(self.groups)}

    def explore(self, limit=2_000_000):
        nb, nf = len(self.bars), len(self.bufs)
        # state: pcs, (arrivals, completed) per barrier, per buffer (version, taken, readers, writers, copies), queues, tma in flight
        start = (tuple(0 for _ in self.prog),
                 tuple((0, 0) for _ in range(nb)),
                 tuple((None, True, 0, 0, 0) for _ in range(nf)),
                 tuple(() for _ in self.queues),
                 (),
                 (tuple(0 for _ in self.groups), ()))          # groups issued per queue, (queue, number, buffer) in flight
        seen, stack = {start}, [start]
        problems, finals = [], 0

        def arrive(bars, b):
            a, c = bars[b]
            a += 1
            if a == self.count[b]:
                a, c = 0, c + 1
            return bars[:b] + ((a, c),) + bars[b + 1:]

        while stack:
            if len(seen) > limit:
                raise AssertionError("state space larger than expected")
            pcs, bars, bufs, queues, tmas, (issued, stores) = stack.pop()
            moves = []
            # lost phases: a role parked at a wait whose barrier ran two phases ahead
            for r, pc in enumerate(pcs):
                if pc < len(self.prog[r]):
                    st = self.prog[r][pc]
                    if st[0] == "wait" and bars[self.bidx[st[1]]][1] >= st[2] + 2:
                        problems.append(("lost phase", self.roles[r], st))
            # role steps
            for r, pc in enumerate(pcs):
                if pc >= len(self.prog[r]):
                    continue
                st = self.prog[r][pc]
                kind = st[0]
                nbars, nbufs, nqueues, ntmas, ngroups = bars, bufs, queues, tmas, (issued, stores)
                if kind == "wait":
                    if bars[self.bidx[st[1]]][1] <= st[2]:
                        continue
                elif kind == "arrive":
                    nbars = arrive(bars, self.bidx[st[1]])
                elif kind == "write":
                    f = self.fidx[st[1]]
                    v, taken, rd, wr, cp = bufs[f]
                    if rd or wr or cp:
                        problems.append(("written while in use", self.roles[r], st))
                    if f in self.check_taken and not taken:
                        problems.append(("rewritten before it was read", self.roles[r], st))
                    nbufs = bufs[:f] + ((st[2], False, rd, wr, cp),) + bufs[f + 1:]
                elif kind == "read":
                    f = self.fidx[st[1]]
                    v, taken, rd, wr, cp = bufs[f]
                    if wr or v != st[2]:
                        problems.append(("read before it was produced", self.roles[r], st, v))
                    nbufs = bufs[:f] + ((v, True, rd, wr, cp),) + bufs[f + 1:]
                elif kind == "tma":
                    f = self.fidx[st[1]]
                    v, taken, rd, wr, cp = bufs[f]
                    if rd or wr or cp:
                        problems.append(("loaded over a buffer in use", self.roles[r], st))
                    nbufs = bufs[:f] + ((v, taken, rd, wr + 1, cp),) + bufs[f + 1:]
                    ntmas = tuple(sorted(tmas + ((f, st[2], self.bidx[st[3]]),)))
                elif kind == "mma":
                    q = self.qidx[st[1]]
                    lb = list(bufs)
                    for b, ver in st[2]:
                        f = self.fidx[b]
                        v, taken, rd, wr, cp = lb[f]
                        if wr or v != ver:
                            problems.append(("MMA operand not ready", self.roles[r], st, b, v))
                        lb[f] = (v, taken, rd + 1, wr, cp)
                    for b, ver in st[3]:
                        f = self.fidx[b]
                        v, taken, rd, wr, cp = lb[f]
                        if f in self.check_taken and not taken and v is not None and ver != v:
                            problems.append(("accumulator rewritten before it was read", self.roles[r], st, b))
                        lb[f] = (v, taken, rd, wr + 1, cp)
                    nbufs = tuple(lb)
                    nqueues = queues[:q] + (queues[q] + (("op", st[2], st[3]),),) + queues[q + 1:]
                elif kind == "commit":
                    q = self.qidx[st[1]]
                    if queues[q]:
                        nqueues = queues[:q] + (queues[q] + (("commit", self.bidx[st[2]]),),) + queues[q + 1:]
                    else:
                        nbars = arrive(bars, self.bidx[st[2]])
                elif kind == "copy_out":
                    f = self.fidx[st[1]]
                    v, taken, rd, wr, cp = bufs[f]
                    nbufs = bufs[:f] + ((v, taken, rd, wr, cp + 1),) + bufs[f + 1:]
                elif kind == "wait_copies":
                    if bufs[self.fidx[st[1]]][4]:
                        continue
                elif kind == "bulk_store":
                    gq, f = self.gidx[st[1]], self.fidx[st[2]]
                    v, taken, rd, wr, cp = bufs[f]
                    if wr:
                        problems.append(("stored while being written", self.roles[r], st))
                    nbufs = bufs[:f] + ((v, taken, rd, wr, cp + 1),) + bufs[f + 1:]
                    ngroups = (issued[:gq] + (issued[gq] + 1,) + issued[gq + 1:], tuple(sorted(stores + ((gq, issued[gq], f),))))
                elif kind == "wait_group":
                    gq = self.gidx[st[1]]
                    if any(q == gq and n < issued[gq] - st[2] for q, n, _ in stores):
                        continue
                moves.append((pcs[:r] + (pc + 1,) + pcs[r + 1:], nbars, nbufs, nqueues, ntmas, ngroups))
            # asynchronous completions: a TMA load lands, the oldest entry of an MMA queue finishes, a copy-out ends
            for i, (f, ver, b) in enumerate(tmas):
                v, taken, rd, wr, cp = bufs[f]
                nbufs = bufs[:f] + ((ver, False, rd, wr - 1, cp),) + bufs[f + 1:]
                moves.append((pcs, arrive(bars, b), nbufs, queues, tmas[:i] + tmas[i + 1:], (issued, stores)))
            for q, items in enumerate(queues):
                if not items:
                    continue
                head = items[0]
                nbars, lb = bars, list(bufs)
                if head[0] == "op":
                    for b, _ in head[1]:
                        f = self.fidx[b]
                        v, taken, rd, wr, cp = lb[f]
                        lb[f] = (v, taken, rd - 1, wr, cp)
                    for b, ver in head[2]:
                        f = self.fidx[b]
                        v, taken, rd, wr, cp = lb[f]
                        lb[f] = (ver, False if ver != v else taken, rd, wr - 1, cp)
                else:
                    nbars = arrive(bars, head[1])
                moves.append((pcs, nbars, tuple(lb), queues[:q] + (items[1:],) + queues[q + 1:], tmas, (issued, stores)))
            for f in range(nf):
                v, taken, rd, wr, cp = bufs[f]
                if cp > sum(1 for _, _, sf in stores if sf == f):          # a copy_out (the bulk stores end below)
                    moves.append((pcs, bars, bufs[:f] + ((v, taken, rd, wr, cp - 1),) + bufs[f + 1:], queues, tmas, (issued, stores)))
            for i, (gq, n, f) in enumerate(stores):                       # groups end in any order
                v, taken, rd, wr, cp = bufs[f]
                moves.append((pcs, bars, bufs[:f] + ((v, taken, rd, wr, cp - 1),) + bufs[f + 1:], queues, tmas,
                              (issued, stores[:i] + stores[i + 1:])))
            if not moves:
                if any(pc < len(self.prog[r]) for r, pc in enumerate(pcs)):
                    stuck = {self.roles[r]: self.prog[r][pc] for r, pc in enumerate(pcs) if pc < len(self.prog[r])}
                    problems.append(("deadlock", stuck))
                else:
                    finals += 1
            for m in moves:
                if m not in seen:
                    seen.add(m)
                    stack.append(m)
            if len(problems) > 20:
                break
        return problems, finals, len(seen)


# --------------------------------------------------------------------------------------------
# forward: producer, one MMA issuer and one softmax warpgroup per query tile
# --------------------------------------------------------------------------------------------
def forward_model(hi_t=(2, 3), ring=3, empty_count=2, wait_s_free=True, wait_o_done=True, take_turns=True):
    lo, hi = 0, max(hi_t)
    bars = {"q_full": 1}
    for s in range(ring):
        bars[f"full{s}"] = 1
        bars[f"empty{s}"] = empty_count
    for t in range(2):
        for b in ("s_full", "p_ready", "o_done", "s_free", "exp_done"):
            bars[f"{b}{t}"] = 1                      # one arrival per warpgroup (the kernel counts its four warps)
    # the ring order: K_lo, then (K_{j+1}, V_j) per key tile
    order = [("K", lo)]
    for j in range(lo, hi):
        if j + 1 < hi:
            order.append(("K", j + 1))
        order.append(("V", j))
    slot_of = {tile: n for n, tile in enumerate(order)}

    producer = [("tma", "Q", 0, "q_full")]
    for n, tile in enumerate(order):
        s, rnd = n % ring, n // ring
        if rnd > 0:
            producer.append(("wait", f"empty{s}", rnd - 1))
        producer.append(("tma", f"slot{s}", tile, f"full{s}"))

    roles = {"producer": producer}
    for t in range(2):
        my_hi = hi_t[t]
        q = f"mma{t}"
        prog = [("wait", "q_full", 0)]
        state = {"f": 0, "p": 0}

        def take(tile, prog=prog):
            n = slot_of[tile]
            prog.append(("wait", f"full{n % ring}", n // ring))
            return n % ring

        def release(s, used, prog=prog, q=q):
            prog.append(("commit", q, f"empty{s}") if used else ("arrive", f"empty{s}"))

        s = take(("K", lo))
        if lo < my_hi:
            prog.append(("mma", q, ((f"slot{s}", ("K", lo)),), ((f"S{t}", lo),)))
            prog.append(("commit", q, f"s_full{t}"))
        release(s, lo < my_hi)
        for j in range(lo, hi):
            if j + 1 < hi:
                s = take(("K", j + 1))
                use = j + 1 < my_hi
                if use:
                    if wait_s_free:
                        prog.append(("wait", f"s_free{t}", state["f"]))
                    state["f"] += 1
                    prog.append(("mma", q, ((f"slot{s}", ("K", j + 1)),), ((f"S{t}", j + 1),)))
                    prog.append(("commit", q, f"s_full{t}"))
                release(s, use)
            s = take(("V", j))
            use = j < my_hi
            if use:
                prog.append(("wait", f"p_ready{t}", state["p"]))
                state["p"] += 1
                prog.append(("mma", q, ((f"P{t}", j), (f"slot{s}", ("V", j))), ((f"O{t}", j),)))
                prog.append(("commit", q, f"o_done{t}"))
            release(s, use)
        roles[f"issuer{t}"] = prog

        n_other = hi_t[1 - t] - lo
        sm = []
        for it, j in enumerate(range(lo, my_hi)):
            sm.append(("wait", f"s_full{t}", it))
            sm.append(("read", f"S{t}", j))
            sm.append(("arrive", f"s_free{t}"))
            if it > 0 and wait_o_done:
                sm.append(("wait", f"o_done{t}", it - 1))
            if take_turns:
                if t == 0 and it > 0 and it - 1 < n_other:
                    sm.append(("wait", "exp_done1", it - 1))
                if t == 1 and it < n_other:
                    sm.append(("wait", "exp_done0", it))
            sm.append(("write", f"P{t}", j))
            sm.append(("arrive", f"exp_done{t}"))
            sm.append(("arrive", f"p_ready{t}"))
        if my_hi > lo:
            sm.append(("wait", f"o_done{t}", my_hi - lo - 1))
            sm.append(("read", f"O{t}", my_hi - 1))
        roles[f"softmax{t}"] = sm
    return Model(bars, roles, check_taken=("S0", "S1"))


@pytest.mark.parametrize("hi_t", [(2, 2), (2, 3), (1, 3)])
def test_forward_pipeline_has_no_deadlock_lost_phase_or_hazard(hi_t):
    problems, finals, states = forward_model(hi_t).explore()
    assert not problems, problems[:3]
    assert finals >= 1 and states > 100


def test_forward_model_finds_a_slot_released_by_one_issuer_only():
    # a K/V slot that a single release frees is refilled while the other tile's MMAs still read it
    problems, _, _ = forward_model((2, 2), empty_count=1).explore()
    assert any(p[0] in ("loaded over a buffer in use", "MMA operand not ready", "lost phase", "deadlock") for p in problems)


def test_forward_model_finds_the_missing_wait_for_the_scores():
    # Q K^T of the next key tile without waiting until the softmax warps hold the current scores
    problems, _, _ = forward_model((2, 2), wait_s_free=False).explore()
    assert any(p[0] in ("accumulator rewritten before it was read", "read before it was produced", "lost phase") for p in problems)


def test_forward_model_finds_the_missing_wait_for_pv():
    # P rewritten without waiting for the previous P V: the softmax warps run ahead of their issuer,
    # which then finds a newer P than the one it was told about (or misses a p_ready phase altogether)
    problems, _, _ = forward_model((2, 2), wait_o_done=False, take_turns=False).explore()
    assert any(p[0] in ("written while in use", "MMA operand not ready", "lost phase") for p in problems)


# --------------------------------------------------------------------------------------------
# backward: producer, three MMA issuers, two compute warpgroups, the dQ drain warpgroup
# --------------------------------------------------------------------------------------------
def backward_model(steps=3, stages=2, tiles_gate="pds_free", drained_wait=True):
    bars = {"kv_full": 1, "sdp_full": 1, "pds_ready": 2, "dq_full": 1, "dq_drained": 1, "sdp_consumed": 2, "pds_free": 2}
    for s in range(stages):
        bars[f"full{s}"] = 1
        bars[f"empty{s}"] = 1
    producer = [("tma", "KV", 0, "kv_full")]
    for n in range(steps):
        s = n % stages
        if n >= stages:
            producer.append(("wait", f"empty{s}", n // stages - 1))
        producer.append(("tma", f"qdo{s}", n, f"full{s}"))
    a = [("wait", "kv_full", 0)]
    b = [("wait", "kv_full", 0)]
    c = [("wait", "kv_full", 0)]
    for n in range(steps):
        s = n % stages
        a.append(("wait", f"full{s}", n // stages))
        if n > 0:
            a.append(("wait", "sdp_consumed", n - 1))
        a.append(("mma", "qa", ((f"qdo{s}", n), ("KV", 0)), (("SdP", n),)))
        a.append(("commit", "qa", "sdp_full"))
        b.append(("wait", f"full{s}", n // stages))
        b.append(("wait", "pds_ready", n))
        b.append(("mma", "qb", (("PdS0", n), ("PdS1", n), (f"qdo{s}", n)), (("dVdK", n),)))
        b.append(("commit", "qb", f"empty{s}"))
        b.append(("commit", "qb", "pds_free"))
        c.append(("wait", "pds_ready", n))
        if n > 0 and drained_wait:
            c.append(("wait", "dq_drained", n - 1))
        c.append(("mma", "qc", (("PdS0", n), ("PdS1", n), ("KV", 0)), (("dQ", n),)))
        c.append(("commit", "qc", "dq_full"))
        c.append(("commit", "qc", "pds_free"))
    roles = {"producer": producer, "issuer_sdp": a, "issuer_dvdk": b, "issuer_dq": c}
    for w in range(2):
        p = []
        for n in range(steps):
            p.append(("wait", "sdp_full", n))
            p.append(("read", "SdP", n))
            if n > 0:
                p.append(("wait", tiles_gate, n - 1))
            p.append(("write", f"PdS{w}", n))
            p.append(("arrive", "sdp_consumed"))
            p.append(("arrive", "pds_ready"))
        p.append(("wait", "pds_free", steps - 1))
        p.append(("read", "dVdK", steps - 1))
        roles[f"compute{w}"] = p
    d = []
    for n in range(steps):
        d.append(("wait", "dq_full", n))
        if n > 0:
            d.append(("wait_copies", "staging"))
        d.append(("read", "dQ", n))
        d.append(("write", "staging", n))
        d.append(("arrive", "dq_drained"))
        d.append(("copy_out", "staging"))
    roles["drain"] = d
    return Model(bars, roles, check_taken=("SdP", "dQ"))


@pytest.mark.parametrize("steps,stages", [(3, 2), (4, 3)])
def test_backward_pipeline_has_no_deadlock_lost_phase_or_hazard(steps, stages):
    problems, finals, states = backward_model(steps, stages).explore()
    assert not problems, problems[:3]
    assert finals >= 1 and states > 100


def test_backward_model_finds_tiles_gated_on_the_dq_product_only():
    # with three issuers, "dQ is done" no longer implies that dV and dK have read the P / dS tiles
    problems, _, _ = backward_model(3, 2, tiles_gate="dq_full").explore()
    assert any(p[0] == "written while in use" for p in problems)


def test_backward_model_finds_the_missing_wait_for_the_drain():
    problems, _, _ = backward_model(3, 2, drained_wait=False).explore()
    assert any(p[0] in ("accumulator rewritten before it was read", "read before it was produced") for p in problems)
