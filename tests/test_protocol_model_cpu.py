"""Host models of the flag protocols the peer-memory kernels use, checked without a GPU.

1. The one-shot all-reduce of the serving path (csrc/comm/serve_allreduce.cu): every rank writes
   its partial into its own symmetric slot, stores the epoch into each peer's flag array with
   release semantics, waits (bounded) until its own flags show the epoch for every peer, then
   loads every peer's slot.  Slots alternate between two buffers from call to call.  The model
   runs the ranks as sequential programs of atomic steps and explores EVERY interleaving (depth-
   first over the reachable states): with two buffers no rank ever reads a slot that a faster
   peer has already overwritten for a later call; with one buffer the explorer finds the race.
   A peer that never signals makes the wait run out: the rank records a status and finishes.
2. The last-arriver hand-off used by the split-K GEMMs and by the all-reduce's call counter: each
   worker adds its part, then bumps a counter; the one that sees the last count finishes and
   resets the counter, so the scratch is clean for the next launch.
3. The same all-reduce protocol once more with real threads and random delays."""
import random
import threading
import time

import pytest


def explore(ranks, epochs, buffers, dead=()):
    """Exhaustive interleaving search.  Returns (violations, finished_states, timeouts_seen)."""
    P = ranks
    live = [r for r in range(P) if r not in dead]
    # program counter: (epoch, phase, peer_index); phases: 0 write, 1 signal, 2 wait, 3 read peers, then next epoch
    start = (tuple((1, 0, 0) for _ in range(P)),                 # pcs
             tuple((0,) * buffers for _ in range(P)),            # slots[rank][buffer] = epoch whose partial it holds
             tuple((0,) * P for _ in range(P)),                  # sig[owner][from] = last epoch signalled
             tuple(0 for _ in range(P)))                         # status word per rank (0 ok, else 4000 + peer)
    seen, stack = {start}, [start]
    violations, finals, timeouts = [], 0, 0
    while stack:
        pcs, slots, sig, status = stack.pop()
        progressed = False
        for r in live:
            e, phase, k = pcs[r]
            if e > epochs:
                continue
            npcs, nslots, nsig, nstatus = list(pcs), slots, sig, status
            if phase == 0:                                       # the GEMM before the collective writes the partial
                row = list(slots[r]); row[e % buffers] = e
                nslots = slots[:r] + (tuple(row),) + slots[r + 1:]
                npcs[r] = (e, 1, 0)
            elif phase == 1:                                     # st.release.sys of the epoch into every peer's flags
                nsig = tuple(tuple(e if (f == r) else v for f, v in enumerate(sig[o])) for o in range(P))
                npcs[r] = (e, 2, 0)
            elif phase == 2:                                     # bounded wait on my own flag array
                missing = [p for p in range(P) if sig[r][p] < e]
                if not missing:
                    npcs[r] = (e, 3, 0)
                elif all(p in dead for p in missing):            # nothing will ever set it: the wait runs out
                    nstatus = status[:r] + (4000 + missing[0],) + status[r + 1:]
                    npcs[r] = (e + 1, 0, 0)                      # reduce skipped, kernel ends normally
                    timeouts += 1
                else:
                    continue                                     # blocked for now
            else:                                                # load peer k's slot
                got = slots[k][e % buffers]
                if got != e:
                    violations.append((r, k, e, got))
                npcs[r] = (e, 3, k + 1) if k + 1 < P else (e + 1, 0, 0)
            progressed = True
            nxt = (tuple(npcs), nslots, nsig, nstatus)
            if nxt not in seen:
                seen.add(nxt)
                stack.append(nxt)
        if not progressed:
            assert all(pcs[r][0] > epochs for r in live), ("deadlock", pcs, sig)
            finals += 1
    return violations, finals, timeouts


@pytest.mark.parametrize("ranks,epochs", [(2, 4), (3, 2)])
def test_double_buffered_slots_are_never_overwritten_before_they_are_read(ranks, epochs):
    violations, finals, _ = explore(ranks, epochs, buffers=2)
    assert not violations and finals >= 1


def test_a_single_buffer_is_a_race_and_the_model_finds_it():
    violations, _, _ = explore(2, 3, buffers=1)
    assert violations
    r, k, e, got = violations[0]
    assert got > e                                               # the peer had already written a later call's partial


def test_a_silent_peer_ends_the_wait_with_a_status_and_no_deadlock():
    violations, finals, timeouts = explore(3, 2, buffers=2, dead=(2,))
    assert not violations and finals >= 1 and timeouts > 0


def test_last_arriver_finishes_and_leaves_the_scratch_clean():
    """Split-K hand-off under every interleaving of 3 workers x (add part, bump counter)."""
    W = 3
    start = ((0,) * W, 0, 0, None)                               # pcs, acc, counter, result
    seen, stack, results = {start}, [start], set()
    while stack:
        pcs, acc, cnt, res = stack.pop()
        moved = False
        for w in range(W):
            if pcs[w] == 0:                                      # red.add of this worker's partial, then a fence
                nxt = (pcs[:w] + (1,) + pcs[w + 1:], acc + (w + 1), cnt, res)
            elif pcs[w] == 1:                                    # atomicAdd on the tile counter returns the old value
                if cnt == W - 1:                                 # last arriver: read the sum, zero scratch and counter
                    nxt = (pcs[:w] + (2,) + pcs[w + 1:], 0, 0, acc)
                else:
                    nxt = (pcs[:w] + (2,) + pcs[w + 1:], acc, cnt + 1, res)
            else:
                continue
            moved = True
            if nxt not in seen:
                seen.add(nxt)
                stack.append(nxt)
        if not moved:
            results.add((acc, cnt, res))
    assert results == {(0, 0, sum(range(1, W + 1)))}             # one finisher, complete sum, clean scratch


def test_symmetric_buffer_canaries_catch_a_store_outside_the_usable_range():
    import torch
    from cogito_b200.parallel.symm import GUARD_BYTES, SymmetricBuffer
    buf = SymmetricBuffer(1000, "cpu", canary=True)
    assert buf.nbytes == 1024 and buf.local.numel() == 1024 and buf.ptrs[0] == buf.local.data_ptr()
    v = buf.view(512, (64,), torch.float32)
    v.fill_(3.0)
    buf.view(0, (256,), torch.int32).fill_(-1)
    assert buf.check_canaries()
    buf._raw[GUARD_BYTES + 1024] = 0                             # one byte past the end, as a bad peer store would
    assert not buf.check_canaries()
    plain = SymmetricBuffer(1000, "cpu", canary=False)
    assert plain.guard == 0 and plain.check_canaries()


def test_all_reduce_protocol_with_real_threads_and_random_delays():
    P, E = 4, 25
    slots = [[None, None] for _ in range(P)]
    sig = [[0] * P for _ in range(P)]
    cond = threading.Condition()
    errors, sums = [], [[None] * E for _ in range(P)]
    rnd = random.Random(0)
    delays = [[rnd.random() * 0.002 for _ in range(E)] for _ in range(P)]

    def rank(r):
        for e in range(1, E + 1):
            slots[r][e % 2] = (e, r * 1000 + e)                  # partial of call e
            time.sleep(delays[r][e - 1])
            with cond:
                for p in range(P):
                    sig[p][r] = e
                cond.notify_all()
                ok = cond.wait_for(lambda: all(sig[r][p] >= e for p in range(P)), timeout=5.0)
            if not ok:
                errors.append(("timeout", r, e))
                return
            total = 0
            for p in range(P):
                tag, val = slots[p][e % 2]
                if tag != e:
                    errors.append(("stale or overwritten", r, p, e, tag))
                total += val
            sums[r][e - 1] = total

    threads = [threading.Thread(target=rank, args=(r,)) for r in range(P)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=30)
    assert not errors, errors[:3]
    for e in range(1, E + 1):
        want = sum(p * 1000 + e for p in range(P))
        assert all(sums[r][e - 1] == want for r in range(P))
