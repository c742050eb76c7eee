"""Model check of the READY / DONE counter protocol of the peer-memory exchanges.

The executor (munet_b200/csrc/engine.cu, lower_linear / lower_mha with tp_exchange 2 to 4) emits,
for exchange number x of a forward, on BOTH ranks:

    wait  DONE  >= seq(x) - 2      the peer has consumed what last sat in receive buffer x & 1
    produce x                      GEMM / attention kernel: writes the PEER's receive buffer x & 1
    signal READY = seq(x)          into the peer's counters
    wait  READY >= seq(x)          what the peer produced for x has arrived here
    consume x                      reduce kernel / unsharded out_proj: reads this rank's buffer x & 1
    signal DONE = seq(x)           into the peer's counters

with seq(x) = (forward - 1) * exchanges_per_forward + x + 1 (munet_b200/csrc/peer_reduce.cu) and
one extra wait DONE >= seq of the previous forward's last exchange at the start of a forward.
This test replays that op list for two ranks under random interleavings and checks the two
properties the design rests on: a consumer always finds the data of ITS exchange in the buffer
(never an older or a newer one), and no schedule dead-locks. It runs on the CPU and models the
protocol only; the kernels are exercised by tests/test_gpu_tp.py.
"""
import random

import pytest


def _ops(per_forward: int, forwards: int):
    ops = []
    for f in range(forwards):
        base = f * per_forward
        ops.append(("wait_done", base))  # start of a forward: everything earlier has been consumed
        for x in range(per_forward):
            seq = base + x + 1
            ops.append(("wait_done", base + max(0, x - 1)))
            ops.append(("produce", seq))
            ops.append(("signal_ready", seq))
            ops.append(("wait_ready", seq))
            ops.append(("consume", seq))
            ops.append(("signal_done", seq))
    return ops


class _Rank:
    def __init__(self, ops, slots=2):
        self.ops, self.pc, self.slots = ops, 0, slots
        self.ready = self.done = 0       # written by the peer only
        self.buf = [None] * slots        # receive buffers: (exchange whose data they hold, consumed?)

    def finished(self):
        return self.pc >= len(self.ops)


def _step(me: _Rank, peer: _Rank) -> bool:
    """Run the next op of `me` if it can; returns False when it is blocked."""
    kind, v = me.ops[me.pc]
    if kind == "wait_done":
        if me.done < v:
            return False
    elif kind == "wait_ready":
        if me.ready < v:
            return False
    elif kind == "produce":
        slot = (v - 1) % me.slots
        # the write lands in the peer's buffer: that must not hold data the peer has yet to consume
        held = peer.buf[slot]
        assert held is None or held[1], f"exchange {v} overwrites unconsumed data of exchange {held[0]}"
        peer.buf[slot] = (v, False)
    elif kind == "signal_ready":
        assert v > peer.ready
        peer.ready = v
    elif kind == "consume":
        slot = (v - 1) % me.slots
        assert me.buf[slot] is not None and me.buf[slot][0] == v, \
            f"exchange {v} reads data of exchange {me.buf[slot]}"
        me.buf[slot] = (v, True)
    elif kind == "signal_done":
        assert v > peer.done
        peer.done = v
    me.pc += 1
    return True


@pytest.mark.parametrize("per_forward", [1, 2, 3, 4, 48])
def test_counters_never_lose_or_overtake_an_exchange(per_forward):
    for seed in range(40):
        rng = random.Random(1000 * per_forward + seed)
        ranks = [_Rank(_ops(per_forward, 3)), _Rank(_ops(per_forward, 3))]
        # long runs of one rank model a rank that is far ahead of the other
        while not all(r.finished() for r in ranks):
            order = [0, 1] if rng.random() < 0.5 else [1, 0]
            burst = rng.choice([1, 1, 2, 5, 50])
            progressed = False
            for i in order:
                for _ in range(burst):
                    if ranks[i].finished() or not _step(ranks[i], ranks[1 - i]):
                        break
                    progressed = True
            assert progressed, f"dead-lock at ops {ranks[0].pc}, {ranks[1].pc}"


def test_a_single_receive_buffer_would_be_overwritten():
    """The model has teeth: the same op list over ONE receive buffer (instead of two used by
    alternate exchanges) lets a rank that runs ahead overwrite data its peer has not consumed."""
    a, b = _Rank(_ops(4, 1), slots=1), _Rank(_ops(4, 1), slots=1)
    with pytest.raises(AssertionError, match="overwrites unconsumed data"):
        for _ in range(400):
            moved = False
            while not a.finished() and _step(a, b):  # rank a runs as far ahead as it may
                moved = True
            if not b.finished() and _step(b, a):
                moved = True
            if not moved:
                break
