"""Host models of the cross-GPU handshakes of the fused tensor-parallel kernels
(csrc/comm/fused_tp.cu) and of the data-parallel optimizer step (csrc/comm/dp_adam.cu), checked
without a GPU.

Every rank runs its calls in stream order; inside a call the transfer role (copy / reduce CTAs)
and the GEMM role run side by side.  Each role is a sequence of atomic steps on words and
buffers in symmetric memory, and the explorer walks EVERY interleaving of all ranks' roles for a
few calls (depth-first over the reachable states), looking for a read that sees another call's
data and for states in which nobody can move.

* GEMM -> reduce-scatter: a rank writes its partial rows for every owner into its own buffer of
  the call's parity and counts them on the owner's flag of that parity; the owner waits for all P
  counts, reads the P partials and clears the flag.  Two parities are enough because a rank
  cannot be two calls ahead of a peer whose partial it needs; with one the explorer finds the
  overwritten partial (or the cleared count).
* all-gather -> GEMM over the switch's multicast: a rank announces that its kernel of this call
  is running, waits for every peer's announcement, then stores its shard into every rank's
  gathered buffer and sets the chunk flag there; the GEMM role waits for the flag of each source.
  Without the announcement round a fast rank's next call lands in a buffer that a slow rank
  still reads.
* data-parallel step: per bucket "my gradients are complete" to every peer, wait for the peers',
  sum the owned part over all ranks' gradient buffers; then Adam on the owned parts, the new
  weights stored into every rank's parameters, "my stores are done" to every peer and a wait for
  the peers' before the kernel ends.  The next step's forward pass then reads only new weights and
  its backward pass never overwrites a gradient a peer has yet to read; without the closing wait
  the explorer finds both.
"""
import pytest


def _explore(P, calls, make_roles, init_shared, step):
    """Generic explorer.  make_roles(rank, call) -> list of role programs (lists of steps) that run
    side by side inside the call.  State: per rank (call, tuple of pcs), and the shared state.
    step(shared, rank, call, st) -> (new shared | None when blocked, problem | None)."""
    start = (tuple((1, (0, 0)) for _ in range(P)), init_shared)
    seen, stack = {start}, [start]
    problems, finals = [], 0
    progs = {}

    def roles(r, e):
        if (r, e) not in progs:
            progs[(r, e)] = make_roles(r, e)
        return progs[(r, e)]

    while stack:
        ranks, shared = stack.pop()
        moved = False
        for r in range(P):
            e, pcs = ranks[r]
            if e > calls:
                continue
            rl = roles(r, e)
            for i, pc in enumerate(pcs):
                if pc >= len(rl[i]):
                    continue
                ns, prob = step(shared, r, e, rl[i][pc])
                if prob:
                    problems.append(prob)
                if ns is None:
                    continue
                npcs = pcs[:i] + (pc + 1,) + pcs[i + 1:]
                if all(npcs[k] >= len(rl[k]) for k in range(len(rl))):
                    nr = (e + 1, (0, 0))                 # both roles done: the kernel ends, the next call may start
                else:
                    nr = (e, npcs)
                nxt = (ranks[:r] + (nr,) + ranks[r + 1:], ns)
                moved = True
                if nxt not in seen:
                    seen.add(nxt)
                    stack.append(nxt)
        if not moved:
            if any(e <= calls for e, _ in ranks):
                problems.append(("deadlock", ranks))
            else:
                finals += 1
        if len(problems) > 10:
            break
    return problems, finals, len(seen)


# ------------------------------------------------------------------ GEMM -> reduce-scatter
def reduce_scatter(P, calls, parities):
    # shared: partial[rank][parity][owner] = call that wrote it; flag[owner][parity] = count
    init = (tuple(tuple((0,) * P for _ in range(parities)) for _ in range(P)),
            tuple((0,) * parities for _ in range(P)))

    def make_roles(r, e):
        par = e % parities
        gemm = []
        for o in range(P):
            gemm.append(("write", o, par))
            gemm.append(("count", o, par))
        red = [("wait", par)] + [("read", s, par) for s in range(P)] + [("clear", par)]
        return [gemm, red]

    def step(shared, r, e, st):
        partial, flag = shared
        kind = st[0]
        if kind == "write":
            _, o, par = st
            row = list(partial[r][par]); row[o] = e
            pr = list(partial[r]); pr[par] = tuple(row)
            return (partial[:r] + (tuple(pr),) + partial[r + 1:], flag), None
        if kind == "count":
            _, o, par = st
            f = list(flag[o]); f[par] += 1
            return (partial, flag[:o] + (tuple(f),) + flag[o + 1:]), None
        if kind == "wait":
            return ((partial, flag), None) if flag[r][st[1]] >= P else (None, None)
        if kind == "read":
            _, s, par = st
            got = partial[s][par][r]
            return (partial, flag), (None if got == e else ("partial of another call", r, s, e, got))
        # clear
        f = list(flag[r]); f[st[1]] = 0
        return (partial, flag[:r] + (tuple(f),) + flag[r + 1:]), None

    return _explore(P, calls, make_roles, init, step)


@pytest.mark.parametrize("P,calls", [(2, 4), (3, 2)])
def test_two_parities_keep_every_partial_until_its_owner_has_read_it(P, calls):
    problems, finals, states = reduce_scatter(P, calls, parities=2)
    assert not problems, problems[:3]
    assert finals >= 1 and states > 50


def test_one_parity_is_a_race_and_the_model_finds_it():
    problems, _, _ = reduce_scatter(2, 3, parities=1)
    assert problems


# ------------------------------------------------------------------ all-gather -> GEMM (multicast)
def all_gather_multicast(P, calls, handshake=True):
    # shared: sig[owner][from] = last call announced; gathered[rank][src] = call whose shard it holds;
    # cflag[rank][src] = last call whose shard is flagged complete there
    z = tuple((0,) * P for _ in range(P))
    init = (z, z, z)

    def make_roles(r, e):
        copy = []
        if handshake:
            copy += [("announce", p) for p in range(P) if p != r]
            copy += [("wait_announce", p) for p in range(P) if p != r]
        copy += [("multicast",), ("flag_all",)]
        gemm = []
        for d in range(P):                       # own shard first, then the others (the tile order of the kernel)
            src = (r + d) % P
            gemm += [("wait_flag", src), ("read", src)]
        return [copy, gemm]

    def step(shared, r, e, st):
        sig, gathered, cflag = shared
        kind = st[0]
        if kind == "announce":
            p = st[1]
            row = list(sig[p]); row[r] = e
            return (sig[:p] + (tuple(row),) + sig[p + 1:], gathered, cflag), None
        if kind == "wait_announce":
            return (shared, None) if sig[r][st[1]] >= e else (None, None)
        if kind == "multicast":                  # one store lands in every rank's gathered buffer
            ng = tuple(tuple(e if s == r else v for s, v in enumerate(gathered[q])) for q in range(P))
            return (sig, ng, cflag), None
        if kind == "flag_all":
            nf = tuple(tuple(e if s == r else v for s, v in enumerate(cflag[q])) for q in range(P))
            return (sig, gathered, nf), None
        if kind == "wait_flag":
            return (shared, None) if cflag[r][st[1]] >= e else (None, None)
        got = gathered[r][st[1]]                 # read
        return shared, (None if got == e else ("shard of another call", r, st[1], e, got))

    return _explore(P, calls, make_roles, init, step)


@pytest.mark.parametrize("P,calls", [(2, 3), (3, 2)])
def test_multicast_gather_never_lands_in_a_buffer_still_being_read(P, calls):
    problems, finals, states = all_gather_multicast(P, calls)
    assert not problems, problems[:3]
    assert finals >= 1 and states > 50


def test_without_the_announcement_round_the_model_finds_the_overwrite():
    problems, _, _ = all_gather_multicast(2, 2, handshake=False)
    assert any(p[0] == "shard of another call" for p in problems)


# ------------------------------------------------------------------ data-parallel step
def data_parallel_step(P, steps, buckets, closing_wait=True):
    # shared: grad[rank][bucket] = step whose gradients it holds; ready[owner][bucket][from] = step announced;
    # param[rank][part] = step whose update it holds (part p is written by rank p); done[owner][from] = step
    zb = tuple((0,) * buckets for _ in range(P))
    init = (zb, tuple(tuple((0,) * P for _ in range(buckets)) for _ in range(P)), tuple((0,) * P for _ in range(P)),
            tuple((0,) * P for _ in range(P)))

    def make_roles(r, e):
        main = [("forward", q) for q in range(P)]                       # reads every part of its own parameter copy
        for b in reversed(range(buckets)):                               # backward produces the last bucket first
            main.append(("backward", b))
        side = []
        for b in reversed(range(buckets)):
            side.append(("need_grad", b))                                # the bucket's hook has fired on the main stream
            side += [("announce", b, q) for q in range(P) if q != r]
            side += [("wait_ready", b, q) for q in range(P) if q != r]
            side += [("pull", b, q) for q in range(P)]
        side += [("store", q) for q in range(P)]
        side += [("done", q) for q in range(P) if q != r]
        if closing_wait:
            side += [("wait_done", q) for q in range(P) if q != r]
        return [main, side]

    def step(shared, r, e, st):
        grad, ready, param, done = shared
        kind = st[0]
        if kind == "forward":
            got = param[r][st[1]]
            return shared, (None if got == e - 1 else ("weights of another step", r, st[1], e, got))
        if kind == "backward":
            row = list(grad[r]); row[st[1]] = e
            return (grad[:r] + (tuple(row),) + grad[r + 1:], ready, param, done), None
        if kind == "need_grad":
            return (shared, None) if grad[r][st[1]] == e else (None, None)
        if kind == "announce":
            _, b, q = st
            rb = list(ready[q]); row = list(rb[b]); row[r] = e; rb[b] = tuple(row)
            return (grad, ready[:q] + (tuple(rb),) + ready[q + 1:], param, done), None
        if kind == "wait_ready":
            _, b, q = st
            return (shared, None) if ready[r][b][q] >= e else (None, None)
        if kind == "pull":
            _, b, q = st
            got = grad[q][b]
            return shared, (None if got == e else ("gradient of another step", r, q, b, e, got))
        if kind == "store":
            q = st[1]
            row = list(param[q]); row[r] = e
            return (grad, ready, param[:q] + (tuple(row),) + param[q + 1:], done), None
        if kind == "done":
            q = st[1]
            row = list(done[q]); row[r] = e
            return (grad, ready, param, done[:q] + (tuple(row),) + done[q + 1:]), None
        return (shared, None) if done[r][st[1]] >= e else (None, None)           # wait_done

    return _explore(P, steps, make_roles, init, step)


@pytest.mark.parametrize("P,steps,buckets", [(2, 3, 2), (3, 2, 1)])
def test_data_parallel_step_reads_only_its_own_steps_gradients_and_weights(P, steps, buckets):
    problems, finals, states = data_parallel_step(P, steps, buckets)
    assert not problems, problems[:3]
    assert finals >= 1 and states > 50


def test_without_the_closing_wait_the_next_step_races_with_slow_peers():
    problems, _, _ = data_parallel_step(2, 2, 1, closing_wait=False)
    assert any(p[0] in ("weights of another step", "gradient of another step") for p in problems)
