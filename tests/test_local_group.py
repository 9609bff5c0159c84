"""Host collectives of the in-process group on CPU threads: sums, timeout, abort, and the failure paths of the
reference's data-parallel tests (tests/data_parallel.rs:512-570, src/dp/weighting.rs:109-201). No GPU involved."""
import threading
import time
from concurrent.futures import ThreadPoolExecutor

import pytest

import oxidizr_b200 as ox
from oxidizr_b200 import ffi


def run_ranks(world, body, timeout=5.0):
    comms = ox.Communicator.local_group(world, None, timeout=timeout)
    with ThreadPoolExecutor(world) as pool:
        futs = [pool.submit(body, comms[r]) for r in range(world)]
        out = []
        for f in futs:
            try:
                out.append(f.result())
            except Exception as e:  # noqa: BLE001
                out.append(e)
    for c in comms:
        c.destroy()
    return out


def test_counts_and_losses_sum_over_ranks():
    def body(c):
        r = c.rank()
        counts = c.sum_counts(10 + r, 1)
        loss = c.sum_f64([[0.75, 0.5, 0.25][r]])
        c.barrier()
        return counts, loss, c.world_size()
    out = run_ranks(3, body)
    assert all(o == ((33, 3), [1.5], 3) for o in out)
    # src/dp/reduce.rs:88-121: .75 + .5 = 1.25 on both ranks
    out = run_ranks(2, lambda c: c.sum_f64([[0.75, 0.5][c.rank()]]))
    assert out == [[1.25], [1.25]]


def test_mixed_masks_error_on_every_rank():
    # src/dp/weighting.rs: some ranks mask and some do not -> every rank returns the same error
    def body(c):
        masked = c.rank() == 0
        scored, masks = c.sum_counts(5 if masked else 0, 1 if masked else 0)
        return ox.step_weighting(1, c.world_size(), scored, masks)
    out = run_ranks(2, body)
    assert all(isinstance(o, ox.OxzError) and "1 of 2 data-parallel ranks carry a loss mask" in str(o) for o in out)


def test_a_rank_that_never_joins_times_out_the_others():
    # tests/data_parallel.rs:546-570
    def body(c):
        if c.rank() == 1:
            return "stayed away"
        return c.sum_counts(1, 0)
    t0 = time.time()
    out = run_ranks(2, body, timeout=0.3)
    assert time.time() - t0 < 5.0
    assert isinstance(out[0], ox.OxzError) and out[0].status == ffi.ERR_TIMEOUT and "never joined" in str(out[0])
    assert out[1] == "stayed away"


def test_abort_from_another_thread_releases_waiting_ranks_and_the_first_abort_wins():
    # src/dp/launch.rs:133-157: the first failure aborts the group once; peers blocked in a collective get an error
    comms = ox.Communicator.local_group(3, None, timeout=30.0)
    results = {}

    def waiter(r):
        try:
            results[r] = comms[r].sum_counts(1, 0)
        except ox.OxzError as e:
            results[r] = e
    threads = [threading.Thread(target=waiter, args=(r,)) for r in (0, 1)]
    for t in threads:
        t.start()
    time.sleep(0.2)
    comms[2].abort()  # rank 2 failed before joining
    comms[2].abort()  # a second abort is a no-op
    for t in threads:
        t.join(5.0)
        assert not t.is_alive(), "a rank is still blocked after the abort"
    assert all(isinstance(results[r], ox.OxzError) and results[r].status == ffi.ERR_ABORTED for r in (0, 1))
    # the group stays unusable
    with pytest.raises(ox.OxzError, match="aborted"):
        comms[0].barrier()
    for c in comms:
        c.destroy()


def test_negative_count_is_refused_before_the_collective():
    comms = ox.Communicator.local_group(1, None)
    assert comms[0].sum_counts(4, 1) == (4, 1)  # world 1: no collective
    with pytest.raises(ox.OxzError, match="timeout"):
        ox.Communicator.local_group(2, None, timeout=0.0)
    comms[0].destroy()


# ---- the rank launcher (src/dp/launch.rs:296-366: first error wins, panic -> error, no hang)

def test_run_ranks_returns_values_in_rank_order():
    comms = ox.Communicator.local_group(3, None, timeout=5.0)
    out = ox.run_ranks(comms, lambda rank, world, comm: (rank, world, comm.sum_counts(rank, 0)[0]))
    assert out == [(0, 3, 3), (1, 3, 3), (2, 3, 3)]
    one = ox.Communicator.local_group(1, None)
    assert ox.run_ranks(one, lambda rank, world, comm: threading.current_thread() is threading.main_thread()) == [True]
    for c in comms + one:
        c.destroy()


def test_the_first_failure_wins_and_releases_the_blocked_peers():
    comms = ox.Communicator.local_group(3, None, timeout=30.0)

    def body(rank, world, comm):
        comm.sum_counts(1, 0)               # step 1: everyone joins
        if rank == 1:
            raise ox.OxzError(ffi.ERR_DATA, "the loader of this rank ran out of rows")   # tests/data_parallel.rs:512-542
        comm.sum_counts(1, 0)               # the peers block here until the abort
        return rank
    t0 = time.time()
    with pytest.raises(ox.OxzError, match="rank 1 of 3 failed first: the loader of this rank ran out of rows") as info:
        ox.run_ranks(comms, body)
    assert time.time() - t0 < 10.0, "the peers waited for the timeout instead of the abort"
    assert info.value.failed_rank == 1 and info.value.status == ffi.ERR_DATA
    for c in comms:
        c.destroy()


def test_a_panic_becomes_an_error_with_its_rank():
    comms = ox.Communicator.local_group(2, None, timeout=30.0)

    def body(rank, world, comm):
        if rank == 0:
            raise ZeroDivisionError("boom")
        return comm.sum_counts(1, 0)
    with pytest.raises(ox.OxzError, match="rank 0 of 2 failed first: panic: boom"):
        ox.run_ranks(comms, body)
    for c in comms:
        c.destroy()


def test_a_fault_injected_at_the_nth_collective_surfaces_as_that_ranks_error():
    # tests/data_parallel_run.rs:283-394: a wrapper communicator that errors at its N-th count all-reduce
    class FaultyRank:
        def __init__(self, comm, fail_at):
            self.comm, self.calls, self.fail_at = comm, 0, fail_at

        def sum_counts(self, a, b):
            self.calls += 1
            if self.calls == self.fail_at:
                raise ox.OxzError(ffi.ERR_NCCL, f"injected failure at collective {self.calls}")
            return self.comm.sum_counts(a, b)
    comms = ox.Communicator.local_group(2, None, timeout=30.0)

    def body(rank, world, comm):
        c = FaultyRank(comm, 3) if rank == 1 else comm
        return [c.sum_counts(1, 0) for _ in range(5)]
    with pytest.raises(ox.OxzError, match="rank 1 of 2 failed first: injected failure at collective 3") as info:
        ox.run_ranks(comms, body)
    assert info.value.status == ffi.ERR_NCCL
    for c in comms:
        c.destroy()
