"""Host model of the persistent GEMM kernel's pipelines (csrc/kernels/gemm_tc_body.cuh,
gemm_tc_epilogue.inc), explored over every interleaving of a small instance without a GPU.

Roles: the TMA producer (operand ring, `full` / `empty` barriers), the MMA-issuing thread (two
accumulators in tensor memory, `tfull` / `tempty`), and epilogue warps.  An epilogue warp stages its
slice of the bias for the tile in a double-buffered shared array behind a barrier all epilogue warps
pass, reads its accumulator rows chunk by chunk, writes each chunk to its staging tile and sends it off
as one bulk tensor store per chunk (one bulk async-group each); the staging tile has two halves:

* plain output: successive chunks alternate between the halves and wait until all but the most recent
  store group have read their source;
* with an epilogue input fetched by bulk loads (activation-derivative operand or residual): the input
  of chunk c + 1 is requested into the second half once chunk c's input is in registers, the output
  always uses the first half and waits for every earlier store.

The explorer (tests/test_attention_pipeline_model_cpu.py) reports deadlocks, lost barrier phases,
buffers overwritten under an asynchronous reader and accumulators rewritten before they were read.
"""
import pytest

from test_attention_pipeline_model_cpu import Model


def gemm_model(tiles=3, kblocks=2, stages=2, warps=2, chunks=2, tma_in=False, groups_pending=None,
               tempty_count=None, wait_empty=True, bias_barrier=True):
    if groups_pending is None:
        groups_pending = 0 if tma_in else 1
    bars = {}
    for s in range(stages):
        bars[f"full{s}"] = 1
        bars[f"empty{s}"] = 1
    for a in range(2):
        bars[f"tfull{a}"] = 1
        bars[f"tempty{a}"] = warps if tempty_count is None else tempty_count
        bars[f"epi{a}"] = warps
    for w in range(warps):
        bars[f"in{w}"] = 1

    producer, mma = [], []
    for it in range(tiles):
        a = it & 1
        if it >= 2:
            mma.append(("wait", f"tempty{a}", (it >> 1) - 1))
        for kb in range(kblocks):
            n = it * kblocks + kb
            s = n % stages
            if n >= stages and wait_empty:
                producer.append(("wait", f"empty{s}", n // stages - 1))
            producer.append(("tma", f"slot{s}", n, f"full{s}"))
            mma.append(("wait", f"full{s}", n // stages))
            mma.append(("mma", "tc", ((f"slot{s}", n),), ((f"acc{a}", it),)))
            mma.append(("commit", "tc", f"empty{s}"))
        mma.append(("commit", "tc", f"tfull{a}"))
    roles = {"producer": producer, "mma": mma}

    for w in range(warps):
        prog, nst, nin = [], 0, 0
        for it in range(tiles):
            a = p = it & 1
            prog.append(("write", f"bias{p}_{w}", it))                     # this warp's slice of the tile's bias
            if bias_barrier:
                prog.append(("arrive", f"epi{p}"))
                prog.append(("wait", f"epi{p}", it >> 1))
            prog.append(("wait", f"tfull{a}", it >> 1))
            if tma_in:
                prog.append(("tma", f"stage{w}_1", (it, 0), f"in{w}"))       # post_input(first chunk)
            for c in range(chunks):
                prog.append(("read", f"acc{a}", it))                         # tcgen05.ld of the chunk
                half = 0 if tma_in else nst & 1
                prog.append(("wait_group", f"g{w}", groups_pending))
                if tma_in:
                    prog.append(("wait", f"in{w}", nin))
                    prog.append(("read", f"stage{w}_1", (it, c)))
                    nin += 1
                    if c + 1 < chunks:
                        prog.append(("tma", f"stage{w}_1", (it, c + 1), f"in{w}"))
                for other in range(warps):                                   # the bias of the chunk's columns: any warp's slice
                    prog.append(("read", f"bias{p}_{other}", it))
                prog.append(("write", f"stage{w}_{half}", (it, c)))
                prog.append(("bulk_store", f"g{w}", f"stage{w}_{half}"))
                nst += 1
            prog.append(("arrive", f"tempty{a}"))
        prog.append(("wait_group", f"g{w}", 0))
        roles[f"epilogue{w}"] = prog
    return Model(bars, roles, check_taken=("acc0", "acc1"))


@pytest.mark.parametrize("kw", [dict(), dict(tma_in=True), dict(stages=3, kblocks=3, tiles=2), dict(tiles=4, kblocks=1, chunks=1)])
def test_gemm_pipeline_has_no_deadlock_lost_phase_or_hazard(kw):
    problems, finals, states = gemm_model(**kw).explore(limit=6_000_000)
    assert not problems, problems[:3]
    assert finals >= 1 and states > 100


def test_two_pending_store_groups_would_overwrite_a_half_that_is_still_being_read():
    problems, _, _ = gemm_model(tiles=2, kblocks=1, warps=1, chunks=3, groups_pending=2).explore()
    assert any(p[0] == "written while in use" for p in problems)


def test_output_half_shared_with_pending_store_when_an_input_tile_uses_the_other_half():
    # with the input tile in the second half every output goes through the first: one pending group is one too many
    problems, _, _ = gemm_model(tiles=1, kblocks=1, warps=1, chunks=2, tma_in=True, groups_pending=1).explore()
    assert any(p[0] == "written while in use" for p in problems)


def test_accumulator_released_by_one_warp_only_is_rewritten_under_the_other():
    problems, _, _ = gemm_model(tiles=3, kblocks=1, chunks=1, tempty_count=1).explore()
    assert any(p[0] in ("accumulator rewritten before it was read", "read before it was produced", "lost phase") for p in problems)


def test_operand_slot_refilled_without_waiting_for_its_mma():
    problems, _, _ = gemm_model(tiles=2, kblocks=2, stages=2, warps=1, chunks=1, wait_empty=False).explore()
    assert any(p[0] in ("loaded over a buffer in use", "MMA operand not ready", "lost phase") for p in problems)


def test_bias_slices_without_the_epilogue_barrier_are_overwritten_under_a_slow_warp():
    problems, _, _ = gemm_model(tiles=3, kblocks=1, chunks=1, bias_barrier=False).explore()
    assert any(p[0] in ("read before it was produced",) for p in problems)
