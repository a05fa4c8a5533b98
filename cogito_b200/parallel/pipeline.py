"""Pipeline parallelism: the 1F1B schedule and its executor over point-to-point transfers.

``one_f_one_b`` generates one stage's program (S-1-stage warm-up forwards, steady
one-forward/one-backward, cool-down backwards), the same program as
``cg_pipeline_gen_1f1b_stage`` of the host library (reference: cg_schedule_op /
cg_schedule_step / cg_pipeline_gen_1f1b, include/cg_pipeline.h:121-142; the reference
generator only produces stage 0 and its executor ``cg_pipeline_forward_backward`` is declared
only, src/pipeline/pipeline.c).

Transfers are NCCL (or gloo) point-to-point calls on a side stream, overlapped with the
compute of the neighbouring micro-batch (see ``PipelineExecutor``).  With tensor parallelism
inside a stage the residual stream is sequence-sharded, so rank (tp=i) of one stage talks only
to rank (tp=i) of the next and moves 1/tp of the activation.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

# the numbering of cg_schedule_op (include/cogito_ext.h): WAIT and SYNC are the reference's, unused by these generators
FORWARD, BACKWARD, SEND_FWD, RECV_FWD, SEND_BWD, RECV_BWD, WAIT, SYNC, OPTIMIZER = range(9)


@dataclass(frozen=True)
class Step:
    action: int
    microbatch: int
    stage: int


def one_f_one_b(num_stages: int, num_microbatches: int, stage: int) -> list[Step]:
    S, M = num_stages, num_microbatches
    if not (S > 0 and M > 0 and 0 <= stage < S):
        raise ValueError("bad pipeline shape")
    out: list[Step] = []

    def fwd(m):
        if stage != 0:
            out.append(Step(RECV_FWD, m, stage))
        out.append(Step(FORWARD, m, stage))
        if stage != S - 1:
            out.append(Step(SEND_FWD, m, stage))

    def bwd(m):
        if stage != S - 1:
            out.append(Step(RECV_BWD, m, stage))
        out.append(Step(BACKWARD, m, stage))
        if stage != 0:
            out.append(Step(SEND_BWD, m, stage))

    warm = min(S - 1 - stage, M)
    f = b = 0
    while f < warm:
        fwd(f); f += 1
    while f < M:
        fwd(f); f += 1
        bwd(b); b += 1
    while b < M:
        bwd(b); b += 1
    out.append(Step(OPTIMIZER, -1, stage))
    return out


class PipelineExecutor:
    """Runs one training step of one pipeline stage.

    stage_fn(x_or_ids, microbatch) -> activation (or the loss on the last stage);
    first stage receives the micro-batch's token ids, later stages the received activation.

    Transfers never wait on the compute stream before their data is needed.  Every transfer is
    issued on a side stream (``comm_stream``) behind an event of the compute stream; a send keeps
    its tensor alive until the step ends; a receive is posted one compute step AHEAD of the
    forward / backward pass that consumes it (the receive for micro-batch i + 1 is in flight while
    micro-batch i is computed), at most two per direction at a time, and the compute stream waits
    on it only when that pass starts.  ``links`` names one process group per neighbour and
    direction (see ``ParallelContext.pipeline_links``): each carries the transfers of one
    direction between one pair of stages in micro-batch order, so a receive posted early never
    holds up a send to the other neighbour.  Without ``links`` (one shared group) a send that is
    directly followed by a receive in the program is posted together with it as one batch, which
    is what keeps two neighbouring stages from waiting on each other's queues.

    ``recompute=True`` keeps only the input of every in-flight micro-batch: the forward pass runs
    without autograd and is run again right before the backward pass (stage-level activation
    recomputation; per-block recomputation is the model's ``recompute`` option).

    Reference counterparts: comm_stream, the A/B buffers and send_event_a/b of cg_pipeline_stage
    (include/cg_pipeline.h:39-58), cg_pipeline_send/recv_activation (src/pipeline/pipeline.c:98-127),
    use_recompute (include/cg_pipeline.h:81-82).
    """

    def __init__(self, stage: int, num_stages: int, num_microbatches: int, prev_rank: int | None, next_rank: int | None,
                 act_shape, act_dtype, device, group=None, links: dict | None = None, recompute: bool = False):
        self.stage, self.S, self.M = stage, num_stages, num_microbatches
        self.prev, self.next = prev_rank, next_rank
        self.shape, self.dtype, self.device = tuple(act_shape), act_dtype, torch.device(device)
        self.group = group
        self.links = links or {}
        self.recompute = recompute
        self.program = one_f_one_b(num_stages, num_microbatches, stage)
        self.p2p_bytes = 0
        self.cuda = self.device.type == "cuda"
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.max_recvs_in_flight = 0

    # -------------------------------------------------------------- transfers
    def _group_for(self, kind):
        """kind: 'recv_fwd' | 'send_fwd' | 'recv_bwd' | 'send_bwd'."""
        return self.links.get(kind, self.group)

    def _issue(self, ops):
        """Start a batch of point-to-point operations on the side stream; returns their handles."""
        if not ops:
            return []
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self.comm_stream.wait_event(ev)           # tensors produced / buffers allocated on the compute stream
            with torch.cuda.stream(self.comm_stream):
                return dist.batch_isend_irecv(ops)
        return dist.batch_isend_irecv(ops)

    def _send_op(self, t, peer, kind):
        self.p2p_bytes += t.numel() * t.element_size()
        return dist.P2POp(dist.isend, t, peer, self._group_for(kind))

    def _recv_op(self, peer, kind):
        buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        return buf, dist.P2POp(dist.irecv, buf, peer, self._group_for(kind))

    # ------------------------------------------------------------------- step
    def run(self, stage_fn, first_inputs=None):
        """first_inputs[m]: what the first stage feeds micro-batch m (ignored elsewhere).
        On the last stage stage_fn returns the micro-batch loss, built so that its backward is
        already multiplied by loss_scale / M.  Returns the mean loss there, None elsewhere."""
        inputs, outputs = {}, {}
        grads_in = {}
        losses = []
        prog = self.program
        separate = bool(self.links)
        # receives in program order; posted[k] = (buffer, handles) once receive k is in flight
        recv_idx = [i for i, st in enumerate(prog) if st.action in (RECV_FWD, RECV_BWD)]
        posted = {}
        next_to_post = 0
        sends = []                     # (tensor, handles) kept until the end of the step

        def post_recv(k, extra_ops=()):
            st = prog[recv_idx[k]]
            fwd = st.action == RECV_FWD
            buf, op = self._recv_op(self.prev if fwd else self.next, "recv_fwd" if fwd else "recv_bwd")
            handles = self._issue(list(extra_ops) + [op])
            posted[k] = (buf, handles)
            self.max_recvs_in_flight = max(self.max_recvs_in_flight, len(posted))
            return handles

        def prefetch(upto_pos):
            """With separate links: post every receive that the program wants at or before position
            upto_pos (the next compute step's input), two in flight at most."""
            nonlocal next_to_post
            while separate and next_to_post < len(recv_idx) and recv_idx[next_to_post] <= upto_pos and len(posted) < 2:
                post_recv(next_to_post)
                next_to_post += 1

        def next_compute_after(i):
            j = i + 1
            while j < len(prog) and prog[j].action not in (FORWARD, BACKWARD):
                j += 1
            return j

        i = 0
        while i < len(prog):
            st = prog[i]
            m = st.microbatch
            if st.action in (RECV_FWD, RECV_BWD):
                k = recv_idx.index(i)
                if k not in posted:
                    post_recv(k)
                    next_to_post = max(next_to_post, k + 1)
                buf, handles = posted.pop(k)
                for w in handles:
                    w.wait()                       # GPU: the compute stream waits; CPU ranks: the host does
                if st.action == RECV_FWD:
                    inputs[m] = buf.requires_grad_(True)
                else:
                    grads_in[m] = buf
            elif st.action == FORWARD:
                prefetch(next_compute_after(i))    # the next pass's input travels while this one computes
                x = first_inputs[m] if self.stage == 0 else inputs[m]
                if self.recompute:
                    with torch.no_grad():
                        y = stage_fn(x, m)
                else:
                    y = stage_fn(x, m)
                outputs[m] = y
                if self.stage == self.S - 1:
                    losses.append(y.detach().float())
            elif st.action == BACKWARD:
                prefetch(next_compute_after(i))
                y = outputs.pop(m)
                if self.recompute:
                    x = first_inputs[m] if self.stage == 0 else inputs[m]
                    y = stage_fn(x, m)             # second forward pass, this time with its graph
                if self.stage == self.S - 1:
                    y.backward()       # stage_fn built the loss with grad_scale = loss_scale / M
                else:
                    y.backward(grads_in.pop(m))
            elif st.action in (SEND_FWD, SEND_BWD):
                if st.action == SEND_FWD:
                    t, peer, kind = outputs[m].detach().contiguous(), self.next, "send_fwd"
                    if self.recompute and self.stage != self.S - 1:
                        outputs[m] = None          # nothing of the first pass is kept but the input
                else:
                    t, peer, kind = inputs.pop(m).grad.contiguous(), self.prev, "send_bwd"
                op = self._send_op(t, peer, kind)
                nxt = prog[i + 1] if i + 1 < len(prog) else None
                if not separate and nxt is not None and nxt.action in (RECV_FWD, RECV_BWD):
                    k = recv_idx.index(i + 1)      # one shared group: the send and the receive behind it go as one batch
                    handles = post_recv(k, extra_ops=[op])
                    next_to_post = max(next_to_post, k + 1)
                else:
                    handles = self._issue([op])
                sends.append((t, handles))
            i += 1
        for t, handles in sends:
            for w in handles:
                w.wait()
        if self.stage == self.S - 1:
            return torch.stack(losses).mean()
        return None

    def bubble_fraction(self) -> float:
        """Idle share of the schedule: (S - 1) / (M + S - 1)."""
        return (self.S - 1) / (self.M + self.S - 1)
