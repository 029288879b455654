"""Failure detection without any GPU fault: a rank that stops (host-side) is noticed through the heartbeat store by
the others before their next collective; the step watchdog reports a step that misses its deadline and a device
status word that a kernel set after giving up a bounded wait (here: a fake status reader)."""

import json
import time

import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed


class _Flag:
    def __init__(self):
        self.done = False

    def query(self):
        return self.done


def test_watchdog_deadline_and_completion():
    from cornstarch_b200.utils.watchdog import StepWatchdog

    seen = []
    wd = StepWatchdog(deadline_s=0.2, on_timeout=seen.append, poll_s=0.02)
    ok = _Flag()
    wd.arm(0, ok)
    ok.done = True
    time.sleep(0.1)
    assert not seen
    stuck = _Flag()
    wd.arm(1, stuck)
    time.sleep(0.5)
    wd.close()
    assert len(seen) == 1 and seen[0]["step"] == 1 and seen[0]["reason"] == "deadline"


def test_watchdog_reports_device_status_word():
    from cornstarch_b200.utils.watchdog import StepWatchdog

    status = {"v": 0}
    seen = []
    wd = StepWatchdog(deadline_s=5.0, on_timeout=seen.append, poll_s=0.02, status_reader=lambda: status["v"])
    wd.arm(7, _Flag())
    time.sleep(0.05)
    status["v"] = 5  # what a kernel stores when a peer flag never arrived
    time.sleep(0.2)
    wd.close()
    assert seen and seen[0] == {"step": 7, "reason": "device_status", "status": 5}


def _hb_worker(rank, world):
    from cornstarch_b200.utils.watchdog import Heartbeat, PeerFailure

    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=0.6)
    dist.barrier()
    x = torch.ones(1)
    dist.all_reduce(x)  # a healthy step
    assert hb.failed() == []
    if rank == world - 1:
        hb.stop()       # this rank "dies" between steps: no kernel or collective of its own in flight
        time.sleep(3.0)
        return
    deadline = time.monotonic() + 5
    dead = []
    while time.monotonic() < deadline and not dead:
        time.sleep(0.1)
        dead = hb.failed()
    assert dead == [world - 1], dead
    assert hb.survivors() == list(range(world - 1))
    try:
        hb.check()
        raise AssertionError("check() must raise")
    except PeerFailure as e:
        assert e.ranks == [world - 1]
    hb.stop()
    # the survivors re-plan among themselves: a new group without the dead rank works
    sub = dist.new_group(list(range(world - 1))) if False else None  # (new_group is collective over all ranks: skipped)
    del sub


def test_heartbeat_detects_a_stopped_rank():
    run_distributed(_hb_worker, 3)


def test_step_logger_json_lines(tmp_path):
    from cornstarch_b200.utils.metrics import StepLogger

    p = tmp_path / "steps.jsonl"
    lg = StepLogger(str(p), tokens_per_step=1000, extra={"config": "unit"})
    for i in range(3):
        lg.begin()
        time.sleep(0.01)
        lg.end(loss=1.0 / (i + 1))
    lg.close()
    rows = [json.loads(x) for x in p.read_text().splitlines()]
    assert [r["step"] for r in rows] == [0, 1, 2] and rows[2]["loss"] < rows[0]["loss"]
    assert rows[0]["tokens_per_s"] > 0 and rows[0]["config"] == "unit"


# ------------------------------------------------------------------------------------------------ on the device
import pytest  # noqa: E402


@pytest.mark.gpu
def test_device_wait_runs_out_sets_status_and_optimizer_skips():
    """A bounded device-side wait really runs out: ``csb_cp_wait`` on a local counter that nothing advances, with the
    wait limit set to a few milliseconds.  The kernel gives up by itself, stores ST_TIMEOUT_PEER_FLAG (5) in the status
    word and returns; the context stays usable; the optimizer skips the update of that step on the device;
    ``poll_status`` (no sync) and ``check_status`` (sync) raise."""
    from cornstarch_b200.ops import _native as nat
    from cornstarch_b200.optim.fused_adamw import FusedAdamW
    from cornstarch_b200.parallel import cp_fused  # noqa: F401  (declares csb_cp_wait)

    lib = nat.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    st = nat.status_word(dev)
    st.zero_()
    w = torch.nn.Parameter(torch.randn(256, 64, device=dev).bfloat16())
    opt = FusedAdamW([w], lr=1e-2, max_norm=1.0)
    before = w.detach().clone()
    w.main_grad.fill_(0.5)
    nat.set_wait_limit(0.005)
    try:
        flags = torch.zeros(8, dtype=torch.int32, device=dev)  # counters of two "ranks"; nobody ever writes them
        t0 = time.monotonic()
        nat.check(lib.csb_cp_wait(flags.data_ptr(), 2, 1, st.data_ptr(), nat.stream()), "csb_cp_wait")
        torch.cuda.synchronize()
        assert time.monotonic() - t0 < 1.0  # gave up after ~5 ms, not after the built-in 2 s
        assert int(st.item()) == 5
        opt.step()  # reads the status word on the device: update skipped
        torch.cuda.synchronize()
        assert torch.equal(w.detach(), before)
        with pytest.raises(RuntimeError, match="status 5"):
            for _ in range(50):  # the asynchronous copy enqueued by step() completes within a few polls
                nat.poll_status(dev)
                time.sleep(0.01)
        assert nat.check_status(dev) == 0  # cleared by the raise
        # the context is intact: the next step updates the weights
        nat._POLLS.clear()
        w.main_grad.fill_(0.5)
        opt.step()
        torch.cuda.synchronize()
        assert not torch.equal(w.detach(), before)
        assert nat.check_status(dev) == 0
    finally:
        nat.set_wait_limit(0.0)
        st.zero_()
        nat._POLLS.clear()
