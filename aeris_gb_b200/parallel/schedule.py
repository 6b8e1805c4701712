"""Pipeline schedules as streams of instructions, and the instruction types the engines interpret.

Three schedules, matching what the reference uses:
  * :class:`TrainSchedule` — synchronous 1F1B with alternating forward/backward slots; the reference takes it from
    DeepSpeed (``deepspeed.runtime.pipe.schedule.TrainSchedule``, used at
    src/aeris/parallelism/parallel_engine.py:1200). ``2 (M + S - 1)`` steps, ``max(2, min(S - s, M))`` buffers.
  * :class:`OverlappedTrainSchedule` — the reference's ``LessCustomTrainSchedule``
    (src/aeris/parallelism/schedule.py:169-231): every receive is split into *submit* (posted one step early) and
    *process* (wait + hand over), sends are issued right after the compute; one extra step and one extra buffer.
  * :class:`EnsembleInferenceSchedule` — forward-only fill/drain over the ensemble members; the last stage returns
    each result to stage 0 (src/aeris/parallelism/sp_inference_engine.py:48-101).

Slot arithmetic (derived here, not taken from either code base): at step ``k`` stage ``s`` of ``S`` is in a forward
slot iff ``k`` and ``s`` have the same parity; the forward slot handles micro-batch ``(k - s) / 2`` and the backward
slot micro-batch ``(k + s + 1) / 2 - S``.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Instruction:
    buffer_id: int | None = None

    @property
    def name(self) -> str:
        return type(self).__name__

    @property
    def kwargs(self) -> dict:
        return {} if self.buffer_id is None else {"buffer_id": self.buffer_id}


class LoadMicroBatch(Instruction): pass
class ForwardPass(Instruction): pass
class BackwardPass(Instruction): pass
class SendActivation(Instruction): pass
class RecvActivation(Instruction): pass
class SendGrad(Instruction): pass
class RecvGrad(Instruction): pass
class SubmitRecvActivation(Instruction): pass
class SubmitRecvGrad(Instruction): pass
class ProcessActivation(Instruction): pass
class ProcessGrad(Instruction): pass
class ReduceTiedGrads(Instruction): pass
class ReduceGrads(Instruction): pass
class OptimizerStep(Instruction): pass
class SendResult(Instruction): pass
class ReturnResult(Instruction): pass


# Point-to-point traffic of the training instructions. Every link between two neighbouring stages has two channels,
# one per direction of travel: "down" carries activations (x, then the noise-level embedding dt) from stage s to s + 1,
# "up" carries gradients (of x, then of dt where dt is trainable upstream) from s + 1 to s. A channel is a communicator
# of its own, so its operations all flow one way and the k-th send meets the k-th receive whatever the two ranks do on
# other channels in between. (With one communicator per pair, as NCCL orders the operations of a communicator by issue
# order, the overlapped schedule stalls: stage s issues recv(grad) then send(x), stage s + 1 recv(x) then send(grad),
# and each receive waits for a send queued behind the peer's receive.)
# instruction type -> (channel as seen from the issuing stage, "send" | "recv", "act" | "grad")
def p2p_op(cmd: Instruction) -> tuple[str, str, str] | None:
    return {
        SendActivation: ("down_next", "send", "act"), RecvActivation: ("down_prev", "recv", "act"),
        SubmitRecvActivation: ("down_prev", "recv", "act"),
        SendGrad: ("up_prev", "send", "grad"), RecvGrad: ("up_next", "recv", "grad"),
        SubmitRecvGrad: ("up_next", "recv", "grad"),
    }.get(type(cmd))


class PipeSchedule:
    def __init__(self, micro_batches: int, stages: int, stage_id: int):
        assert 0 <= stage_id < stages and micro_batches >= 1
        self.micro_batches, self.stages, self.stage_id = micro_batches, stages, stage_id

    @property
    def is_first(self) -> bool:
        return self.stage_id == 0

    @property
    def is_last(self) -> bool:
        return self.stage_id == self.stages - 1

    def valid(self, mb: int) -> bool:
        return 0 <= mb < self.micro_batches

    def buffer_idx(self, mb: int) -> int:
        return mb % self.num_pipe_buffers()

    def slot(self, step: int) -> tuple[int, bool]:
        """(micro-batch id, is_forward) of this stage at ``step``; the id may be out of range (idle slot)."""
        s, S = self.stage_id, self.stages
        if (step - s) % 2 == 0:
            return (step - s) // 2, True
        return (step + s + 1) // 2 - S, False

    def num_pipe_buffers(self) -> int:
        raise NotImplementedError

    def steps(self):
        raise NotImplementedError

    def __iter__(self):
        return iter(self.steps())


class TrainSchedule(PipeSchedule):
    def num_pipe_buffers(self) -> int:
        return max(2, min(self.stages - self.stage_id, self.micro_batches))

    def steps(self):
        total = 2 * (self.micro_batches + self.stages - 1)
        prev_mb = -1
        for k in range(total):
            mb, fwd = self.slot(k)
            cmds: list[Instruction] = []
            if fwd:
                # the previous (backward) slot's input gradient goes upstream while the next activation comes in
                if self.valid(prev_mb) and not self.is_first:
                    cmds.append(SendGrad(self.buffer_idx(prev_mb)))
                if self.valid(mb) and not self.is_first:
                    cmds.append(RecvActivation(self.buffer_idx(mb)))
            else:
                if self.valid(mb) and not self.is_last:
                    cmds.append(RecvGrad(self.buffer_idx(mb)))
                if self.valid(prev_mb) and not self.is_last:
                    cmds.append(SendActivation(self.buffer_idx(prev_mb)))
            if (self.is_first or self.is_last) and fwd and self.valid(mb):
                cmds.append(LoadMicroBatch(self.buffer_idx(mb)))
            if self.valid(mb):
                cmds.append(ForwardPass(self.buffer_idx(mb)) if fwd else BackwardPass(self.buffer_idx(mb)))
            if k == total - 1:
                cmds += [ReduceTiedGrads(), ReduceGrads(), OptimizerStep()]
            prev_mb = mb
            yield cmds


class OverlappedTrainSchedule(PipeSchedule):
    def num_pipe_buffers(self) -> int:
        return max(2, min(self.stages - self.stage_id, self.micro_batches) + 1)

    def steps(self):
        total = 2 * (self.micro_batches + self.stages - 1) + 1
        for k in range(total):
            mb, fwd = self.slot(k)
            nxt, _ = self.slot(k + 1)
            cmds: list[Instruction] = []
            if (self.is_first or self.is_last) and fwd and self.valid(mb):
                cmds.append(LoadMicroBatch(self.buffer_idx(mb)))
            # post next step's receive before this step's compute so the transfer overlaps it
            if fwd:
                if self.valid(nxt) and not self.is_last:
                    cmds.append(SubmitRecvGrad(self.buffer_idx(nxt)))
            else:
                if self.valid(nxt) and not self.is_first:
                    cmds.append(SubmitRecvActivation(self.buffer_idx(nxt)))
            if self.valid(mb):
                b = self.buffer_idx(mb)
                if fwd:
                    if not self.is_first:
                        cmds.append(ProcessActivation(b))
                    cmds.append(ForwardPass(b))
                    if not self.is_last:
                        cmds.append(SendActivation(b))
                else:
                    if not self.is_last:
                        cmds.append(ProcessGrad(b))
                    cmds.append(BackwardPass(b))
                    if not self.is_first:
                        cmds.append(SendGrad(b))
            if k == total - 1:
                cmds += [ReduceTiedGrads(), ReduceGrads(), OptimizerStep()]
            yield cmds


class EnsembleInferenceSchedule(PipeSchedule):
    """Forward-only: at step ``k`` stage ``s`` runs member ``k - s``. Stage 0 collects the result of member
    ``k - (S - 1)`` that the last stage sent in the same step."""

    def num_pipe_buffers(self) -> int:
        return 2

    def steps(self):
        S = self.stages
        total = self.micro_batches + S - 1
        for k in range(total):
            mb = k - self.stage_id
            cmds: list[Instruction] = []
            if self.valid(mb):
                b = self.buffer_idx(mb)
                if self.is_first:
                    cmds.append(LoadMicroBatch(b))
                else:
                    cmds.append(RecvActivation(b))
                cmds.append(ForwardPass(b))
                if self.is_last:
                    cmds.append(SendResult(b))
                else:
                    cmds.append(SendActivation(b))
            done = k - (S - 1)
            if self.is_first and self.valid(done):
                cmds.append(ReturnResult(self.buffer_idx(done)))
            yield cmds
