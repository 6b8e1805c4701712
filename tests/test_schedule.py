"""Properties of the pipeline schedules, checked by replaying every stage's instruction stream on a fake wire."""
import pytest
from hypothesis import given, settings, strategies as st

from aeris_gb_b200.parallel import schedule as S


def _replay(cls, M, P):
    """Runs all stages in lock step; sends append to a per-link FIFO, receives pop from it. Returns per-stage logs."""
    scheds = [list(cls(M, P, s).steps()) for s in range(P)]
    n_steps = len(scheds[0])
    assert all(len(x) == n_steps for x in scheds)
    act = {(s, s + 1): [] for s in range(P - 1)}
    grad = {(s + 1, s): [] for s in range(P - 1)}
    posted = [dict(act=None, grad=None) for _ in range(P)]
    fwd_done = [[] for _ in range(P)]
    bwd_done = [[] for _ in range(P)]
    live = [dict() for _ in range(P)]          # buffer -> micro-batch whose activation it holds
    mb_of_buf_in = [dict() for _ in range(P)]
    for k in range(n_steps):
        # two passes: all sends of this step first become visible only after being issued; process in program order
        # but let receives wait for a matching send issued in the same step by running stages in both orders.
        pending = [list(scheds[s][k]) for s in range(P)]
        progress = True
        while progress and any(pending):
            progress = False
            for s in range(P):
                while pending[s]:
                    c = pending[s][0]
                    mb_f, is_f = cls(M, P, s).slot(k)
                    if isinstance(c, (S.RecvActivation, S.ProcessActivation)):
                        if not act[(s - 1, s)]:
                            break
                        mb_of_buf_in[s][c.buffer_id] = act[(s - 1, s)].pop(0)
                    elif isinstance(c, (S.RecvGrad, S.ProcessGrad)):
                        if not grad[(s + 1, s)]:
                            break
                        got = grad[(s + 1, s)].pop(0)
                        assert live[s].get(c.buffer_id) == got, "gradient arrived for a buffer holding another micro-batch"
                    elif isinstance(c, S.SendActivation):
                        act[(s, s + 1)].append(live[s][c.buffer_id])
                    elif isinstance(c, S.SendGrad):
                        grad[(s, s - 1)].append(bwd_done[s][-1])
                    elif isinstance(c, S.LoadMicroBatch):
                        if s == 0:
                            mb_of_buf_in[s][c.buffer_id] = len(fwd_done[s])
                    elif isinstance(c, S.ForwardPass):
                        mb = mb_of_buf_in[s][c.buffer_id] if s > 0 or c.buffer_id in mb_of_buf_in[s] else len(fwd_done[s])
                        assert c.buffer_id not in live[s], "forward into a buffer whose backward has not run"
                        live[s][c.buffer_id] = mb
                        fwd_done[s].append(mb)
                    elif isinstance(c, S.BackwardPass):
                        mb = live[s].pop(c.buffer_id)
                        bwd_done[s].append(mb)
                    pending[s].pop(0)
                    progress = True
        assert not any(pending), f"deadlock at step {k}: {pending}"
    return fwd_done, bwd_done, scheds


@settings(max_examples=60, deadline=None)
@given(M=st.integers(1, 9), P=st.integers(1, 7), overlapped=st.booleans())
def test_1f1b_runs_every_micro_batch_once_and_never_deadlocks(M, P, overlapped):
    cls = S.OverlappedTrainSchedule if overlapped else S.TrainSchedule
    fwd, bwd, scheds = _replay(cls, M, P)
    for s in range(P):
        assert fwd[s] == list(range(M)) and bwd[s] == list(range(M))
        names = [c.name for step in scheds[s] for c in step]
        assert names[-3:] == ["ReduceTiedGrads", "ReduceGrads", "OptimizerStep"]
        assert names.count("OptimizerStep") == 1


def test_step_counts_and_buffers():
    assert len(list(S.TrainSchedule(4, 3, 0).steps())) == 2 * (4 + 3 - 1)
    assert len(list(S.OverlappedTrainSchedule(4, 3, 0).steps())) == 2 * (4 + 3 - 1) + 1
    assert S.TrainSchedule(20, 10, 0).num_pipe_buffers() == 10
    assert S.TrainSchedule(20, 10, 9).num_pipe_buffers() == 2
    assert S.OverlappedTrainSchedule(20, 10, 3).num_pipe_buffers() == 8


def test_first_stage_warmup_depth_is_1f1b():
    # stage 0 of 4 runs 4 forwards before its first backward; the last stage alternates from the start
    names0 = [c.name for step in S.TrainSchedule(8, 4, 0).steps() for c in step if c.name in ("ForwardPass", "BackwardPass")]
    assert names0[:5] == ["ForwardPass"] * 4 + ["BackwardPass"]
    names3 = [c.name for step in S.TrainSchedule(8, 4, 3).steps() for c in step if c.name in ("ForwardPass", "BackwardPass")]
    assert names3[:4] == ["ForwardPass", "BackwardPass", "ForwardPass", "BackwardPass"]


@pytest.mark.parametrize("M,P", [(1, 1), (3, 1), (5, 4), (2, 6)])
def test_ensemble_inference_schedule(M, P):
    seq = [list(S.EnsembleInferenceSchedule(M, P, s).steps()) for s in range(P)]
    assert all(len(x) == M + P - 1 for x in seq)
    for s in range(P):
        names = [c.name for step in seq[s] for c in step]
        assert names.count("ForwardPass") == M
        assert names.count("ReturnResult") == (M if s == 0 else 0)
        assert names.count("SendResult") == (M if s == P - 1 else 0)
    # a result is returned in the step in which the last stage sends it
    for k in range(M + P - 1):
        sent = [c for c in seq[P - 1][k] if c.name == "SendResult"]
        ret = [c for c in seq[0][k] if c.name == "ReturnResult"]
        assert len(sent) == len(ret)


# ---------------------------------------------------------------------------------------------------------------------
# Stream-level replay of the point-to-point traffic the way NCCL executes it: the host enqueues everything without
# blocking; every communicator runs its operations in issue order on a stream of its own; an operation starts once
# the compute kernels queued before it have finished and completes only together with the complementary operation at
# the head of the peer's stream of the same communicator; a compute kernel waits for the receives it consumes.
def _enqueue(cls, M, P, s, directional):
    sched = cls(M, P, s)
    comm, compute, pending, wait_list = {}, [], {}, []
    buf_mb = {}
    for k, cmds in enumerate(sched.steps()):
        for c in cmds:
            op = S.p2p_op(c)
            if op is not None:
                channel, kind, what = op
                lo = s if channel.endswith("next") else s - 1
                key = (lo, channel.split("_")[0]) if directional else (lo,)
                item = dict(kind=kind, what=what, after=len(compute), done=False, rank=s)
                comm.setdefault(key, []).append(item)
                if isinstance(c, (S.RecvActivation, S.RecvGrad)):
                    wait_list.append(item)
                elif kind == "recv":
                    pending[(what, c.buffer_id)] = item
            elif isinstance(c, S.ProcessActivation):
                wait_list.append(pending.pop(("act", c.buffer_id)))
            elif isinstance(c, S.ProcessGrad):
                wait_list.append(pending.pop(("grad", c.buffer_id)))
            elif isinstance(c, (S.ForwardPass, S.BackwardPass)):
                compute.append(dict(needs=wait_list, done=False))
                wait_list = []
    assert not pending
    return comm, compute


def _run_streams(cls, M, P, directional):
    ranks = [_enqueue(cls, M, P, s, directional) for s in range(P)]
    heads = [{k: 0 for k in comm} for comm, _ in ranks]
    chead = [0] * P
    progress = True
    while progress:
        progress = False
        for s, (comm, compute) in enumerate(ranks):
            while chead[s] < len(compute) and all(n["done"] for n in compute[chead[s]]["needs"]):
                compute[chead[s]]["done"] = True
                chead[s] += 1
                progress = True
        for s, (comm, compute) in enumerate(ranks):
            for key, q in comm.items():
                i = heads[s][key]
                if i >= len(q) or chead[s] < q[i]["after"]:
                    continue
                peer = key[0] + 1 if key[0] == s else key[0]
                pq = ranks[peer][0].get(key, [])
                j = heads[peer][key] if key in heads[peer] else 0
                if j >= len(pq) or chead[peer] < pq[j]["after"]:
                    continue
                a, b = q[i], pq[j]
                if {a["kind"], b["kind"]} != {"send", "recv"}:
                    continue                      # two receives (or two sends) face each other: neither can move
                assert a["what"] == b["what"], f"{a} meets {b} on {key}"
                a["done"] = b["done"] = True
                heads[s][key] += 1
                heads[peer][key] += 1
                progress = True
    finished = all(chead[s] == len(ranks[s][1]) for s in range(P)) and \
        all(heads[s][k] == len(q) for s in range(P) for k, q in ranks[s][0].items())
    return finished


@settings(max_examples=80, deadline=None)
@given(M=st.integers(1, 9), P=st.integers(2, 7), overlapped=st.booleans())
def test_one_communicator_per_direction_never_stalls_on_ordered_streams(M, P, overlapped):
    cls = S.OverlappedTrainSchedule if overlapped else S.TrainSchedule
    assert _run_streams(cls, M, P, directional=True)


def test_one_communicator_per_pair_stalls_under_the_overlapped_schedule():
    """Why the links are split by direction: with a single communicator per pair the early receive of stage s
    (gradient) and that of stage s + 1 (activation) face each other at the heads of the two streams."""
    assert _run_streams(S.TrainSchedule, 4, 2, directional=False)
    assert not _run_streams(S.OverlappedTrainSchedule, 4, 2, directional=False)
