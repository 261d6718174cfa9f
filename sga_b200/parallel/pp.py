"""Pipeline parallelism: the one-forward-one-backward schedule over
point-to-point transfers.

Stage ``p`` holds a contiguous run of layers (``models.gpt.stage_layers``), the
first stage the embedding, the last the final norm, the output layer and the
loss. A step of ``m`` micro-batches runs ``min(P - p - 1, m)`` warm-up
forwards, then alternates one forward with one backward, then drains the
backwards; a stage therefore keeps at most ``P - p`` micro-batches of saved
activations. Activations (``[tokens, hidden]`` bf16) go to the next stage and
their gradients come back with ``torch.distributed`` send / receive pairs on
the library's own streams (NCCL on GPUs, gloo on CPU), posted together where a
stage both sends and receives so that neighbouring stages cannot block each
other; a receive is waited for only when its tensor is needed.

The reference leaves pipeline stages to its external training stack and only
tolerates them (untied embeddings, no always-sync layers:
``sga/runtime.py:71-76``, ``sga/config/validation.py:332-341``); the
data-parallel gradient machinery of each stage runs unchanged on the stage's
own parameters. Combined with tensor parallelism every tensor-parallel rank of a
stage runs this schedule with the same-index rank of the neighbouring stages.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


class Pipeline:
    def __init__(self, model, *, pp_rank: int, pp_size: int, prev_rank: Optional[int], next_rank: Optional[int],
                 group=None):
        self.model = model
        self.pp_rank, self.pp_size = pp_rank, pp_size
        self.prev_rank, self.next_rank = prev_rank, next_rank
        self.group = group
        self.first, self.last = pp_rank == 0, pp_rank == pp_size - 1
        self.transfers = 0

    # ------------------------------------------------------------ transfers
    def _post(self, send: Optional[torch.Tensor], send_to: Optional[int], recv_shape, recv_from: Optional[int]):
        """Posts an optional send and an optional receive together; returns ``(requests, buffer)``."""
        ops, buf = [], None
        dev, dt = self.model.device, torch.bfloat16
        if recv_from is not None:
            buf = torch.empty(recv_shape, dtype=dt, device=dev)
            ops.append(dist.P2POp(dist.irecv, buf, recv_from, self.group))
        if send is not None and send_to is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), send_to, self.group))
        if not ops:
            return [], None
        self.transfers += len(ops)
        return dist.batch_isend_irecv(ops), buf

    @staticmethod
    def _wait(reqs) -> None:
        for r in reqs:
            r.wait()

    # ----------------------------------------------------------- validation
    def run_forward(self, micro_batches):
        """Forward passes only (the validation pass): every micro-batch goes down the stages once, nothing is
        kept for a backward pass and no gradient is written. Returns the micro-batch losses on the last
        stage, an empty list elsewhere."""
        model = self.model
        B, S = micro_batches[0][0].shape
        act_shape = (B * S // getattr(model, "tp_size", 1), model.cfg.hidden)
        losses = []
        for tokens, targets in micro_batches:
            x_in = None
            if not self.first:
                reqs, x_in = self._post(None, None, act_shape, self.prev_rank)
                self._wait(reqs)
            out, ctx = model.stage_forward(tokens, targets, x_in, loss_scale=1.0, write_grad=False)
            ctx.clear()
            if self.last:
                losses.append(out)
            else:
                reqs, _ = self._post(out, self.next_rank, None, None)
                self._wait(reqs)
        return losses

    # ------------------------------------------------------------- schedule
    def run(self, micro_batches, *, loss_scale: float, on_param_done_last: Optional[Callable] = None,
            before_last_backward: Optional[Callable] = None):
        """``micro_batches``: list of ``(tokens [B, S], targets [B, S])``, the same on every stage of a
        data-parallel replica. Returns the list of micro-batch losses (last stage; empty elsewhere).
        ``before_last_backward`` runs right before the step's final backward pass (arming the
        per-bucket gradient synchronisation); ``on_param_done_last`` is passed to that pass."""
        m = len(micro_batches)
        model = self.model
        B, S = micro_batches[0][0].shape
        # under tensor parallelism the activations are sharded by rows: a rank exchanges its own block
        # with the rank of the same tensor-parallel index in the neighbouring stages
        act_shape = (B * S // getattr(model, "tp_size", 1), model.cfg.hidden)
        warm = min(self.pp_size - self.pp_rank - 1, m)
        steady = m - warm
        depth = warm + 1  # micro-batches this stage holds between their forward and their backward
        ctxs, losses = [], []
        f = b = 0

        def forward(x_in):
            nonlocal f
            tokens, targets = micro_batches[f]
            out, ctx = model.stage_forward(tokens, targets, x_in, loss_scale=loss_scale, inflight=f % depth)
            ctxs.append(ctx)
            f += 1
            if self.last:
                losses.append(out)
                return None
            return out

        def backward(dx_out):
            nonlocal b
            ctx = ctxs.pop(0)
            last_one = b == m - 1
            if last_one and before_last_backward is not None:
                before_last_backward()
            dx_in = model.stage_backward(ctx, dx_out, on_param_done_last if last_one else None)
            b += 1
            return dx_in

        # warm-up forwards
        x_in = None
        for _ in range(warm):
            if not self.first:
                reqs, x_in = self._post(None, None, act_shape, self.prev_rank)
                self._wait(reqs)
            out = forward(x_in)
            reqs, _ = self._post(out, self.next_rank, None, None)
            self._wait(reqs)
        # steady state: forward, (send activation | receive its gradient), backward, (send gradient | receive next)
        if steady > 0 and not self.first:
            reqs, x_in = self._post(None, None, act_shape, self.prev_rank)
            self._wait(reqs)
        for i in range(steady):
            out = forward(x_in)
            reqs, dx_out = self._post(out, self.next_rank, act_shape, None if self.last else self.next_rank)
            self._wait(reqs)
            dx_in = backward(dx_out)
            more = i + 1 < steady
            reqs, x_in = self._post(dx_in, self.prev_rank, act_shape,
                                    self.prev_rank if (more and not self.first) else None)
            self._wait(reqs)
        # cool-down backwards
        for _ in range(warm):
            reqs, dx_out = self._post(None, None, act_shape, None if self.last else self.next_rank)
            self._wait(reqs)
            dx_in = backward(dx_out)
            reqs, _ = self._post(dx_in, self.prev_rank, None, None)
            self._wait(reqs)
        assert f == m and b == m and not ctxs
        return losses
