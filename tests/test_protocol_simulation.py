"""Host-side simulation of the flag protocol behind the fused all-gather + GEMM (`flb_tp_push`, `flb_gemm_gathered_bf16`,
`parallel/fused_tp.py`): ranks are threads, streams are ordered lists of operations, peer memory is shared Python state, and
every step sleeps a random time, so the interleavings a GPU could produce are sampled.  Checked on every read and write:

  * a consumer only ever reads rows of the call it belongs to (no stale rows, no rows of a later call);
  * a push never overwrites a landing zone that some rank is still reading or has yet to read;
  * nothing waits forever (every wait has a deadline, as on the device).

The model keeps what the device code relies on and nothing else: two landing zones used by call parity; a push of call k
first tells every peer "my call k has begun" and waits for the same word from every peer; it runs behind the point of the main
stream where the gather was started (so behind every consumer that was queued before); after its stores it raises the peer's
arrival word to k; consumers wait for arrival words >= their call.  A variant without the meeting shows that the checks can fail."""

import random
import threading
import time

import pytest

DEADLINE = 20.0


class Violation(AssertionError):
    pass


class Rank:
    def __init__(self, index: int, world: int):
        self.index, self.world = index, world
        self.begun = [0] * world  # begun[p]: the last call whose push rank p reported as begun (written by p)
        self.arrival = [[0] * world for _ in range(2)]  # arrival[half][p]: last call whose rows from p have landed
        self.landing = [[0] * world for _ in range(2)]  # landing[half][p]: which call's rows of p lie there
        self.reading = [None, None]  # per half: the call a consumer is reading right now
        self.consumed = 0  # consumers finish in order on the main stream
        self.lock = threading.Lock()
        self.errors: list = []  # shared by all ranks of a run


def _wait(predicate, what: str, errors: list):
    start = time.monotonic()
    while not predicate():
        if errors:
            raise Violation("stopped: another rank reported a violation")  # like the error word: everybody gives up
        if time.monotonic() - start > DEADLINE:
            raise Violation(f"deadline: {what}")
        time.sleep(0)


def _jitter(rng, scale=0.002):
    time.sleep(rng.random() * scale)


def _push(ranks, me: Rank, call: int, rng, meet: bool):
    half = call & 1
    for peer in ranks:
        if peer is not me:
            peer.begun[me.index] = call
    if meet:
        for peer in ranks:
            if peer is not me:
                _wait(lambda p=peer: me.begun[p.index] >= call, f"rank {me.index} waits for the push of call {call} on rank {peer.index}", me.errors)
    for peer in ranks:
        if peer is me:
            continue
        _jitter(rng)
        with peer.lock:
            if peer.reading[half] is not None:
                raise Violation(f"rank {me.index} overwrites half {half} of rank {peer.index} during its read of call {peer.reading[half]}")
            if peer.consumed < call - 2:
                raise Violation(f"rank {me.index} overwrites half {half} of rank {peer.index} before call {call - 2} was read")
            peer.landing[half][me.index] = call
        _jitter(rng)
        peer.arrival[half][me.index] = call


def _consume(ranks, me: Rank, call: int, rng):
    half = call & 1
    for peer in ranks:
        if peer is not me:
            _wait(lambda p=peer: me.arrival[half][p.index] >= call, f"rank {me.index} waits for rows of rank {peer.index}, call {call}", me.errors)
    with me.lock:
        me.reading[half] = call
    _jitter(rng, 0.004)
    with me.lock:
        for peer in ranks:
            if peer is not me and me.landing[half][peer.index] != call:
                raise Violation(f"rank {me.index} read rows of call {me.landing[half][peer.index]} from rank {peer.index} in call {call}")
        me.reading[half] = None
        me.consumed = call


def _main_stream(ranks, me: Rank, program, seed: int, meet: bool, errors: list, slow: float = 1.0):
    """`program`: list of ("start", call) / ("consume", call) in main-stream order.  A push runs on the side stream: after every
    earlier push of this rank and after everything queued on the main stream before its start."""
    rng = random.Random(seed)
    side = None
    try:
        for kind, call in program:
            _jitter(rng, 0.002 * slow)
            if kind == "start":
                previous = side

                def run(previous=previous, call=call):
                    try:
                        if previous is not None:
                            previous.join(DEADLINE)
                        _push(ranks, me, call, random.Random(seed * 1000 + call), meet)
                    except Violation as e:
                        errors.append(e)

                # the main stream is executed in order by this thread, so "behind this point of the main stream" = now
                side = threading.Thread(target=run)
                side.start()
            else:
                if slow > 1:
                    time.sleep(0.002 * slow)  # a rank that lags behind its peers
                _consume(ranks, me, call, rng)
        if side is not None:
            side.join(DEADLINE)
    except Violation as e:
        errors.append(e)


def _program(calls: int, paired: bool):
    """One gather consumed at once (a linear layer), or two gathers started back to back and consumed afterwards (the MLP's
    backward: output gradient and layer input)."""
    program, call = [], 1
    while call <= calls:
        if paired and call + 1 <= calls:
            program += [("start", call), ("start", call + 1), ("consume", call), ("consume", call + 1)]
            call += 2
        else:
            program += [("start", call), ("consume", call)]
            call += 1
    return program


def _run(world: int, calls: int, paired: bool, meet: bool, seed: int, slow_last_rank: float = 1.0):
    ranks = [Rank(i, world) for i in range(world)]
    errors: list = []
    for rank in ranks:
        rank.errors = errors
    threads = [threading.Thread(target=_main_stream, args=(ranks, rank, _program(calls, paired), seed * 17 + rank.index, meet, errors,
                                                             slow_last_rank if rank.index == world - 1 else 1.0)) for rank in ranks]
    for t in threads:
        t.start()
    for t in threads:
        t.join(DEADLINE * 2)
    assert not any(t.is_alive() for t in threads), "a rank did not finish"
    return errors


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("paired", [False, True])
def test_gather_protocol_holds_under_random_interleavings(world, paired):
    for seed in range(6):
        errors = _run(world, 14, paired, True, seed, slow_last_rank=3.0 if seed % 2 else 1.0)
        assert not errors, errors[0]


def test_the_checks_catch_a_protocol_without_the_meeting():
    """With two gathers in flight (the MLP's backward) and without the "my call has begun" meeting, a fast rank's push of call
    k + 2 can land while a slow rank still has call k to read: the simulation must be able to see that (otherwise the test
    above proves nothing).  With one gather in flight the arrival words alone order everything, so that case cannot fail."""
    found = False
    for seed in range(40):
        if _run(3, 8, True, False, seed, slow_last_rank=4.0):
            found = True
            break
    assert found
