"""The flag protocols of the one-sided kernels, explored over every interleaving (host-side model), and proof that the
explorer rejects the broken variants of each protocol."""
import pytest

from maltos_b200.utils import flag_protocol as fp


@pytest.mark.parametrize("world,calls", [(2, 5), (3, 4), (4, 3)])
def test_pull_collective_with_parity_buffers_is_safe(world, calls):
    assert fp.explore(fp.pull_collective(world, calls)).states > 0


def test_pull_collective_broken_variants_are_rejected():
    with pytest.raises(fp.ProtocolViolation, match="overlaps a write"):
        fp.explore(fp.pull_collective(3, 3, double_buffered=False))          # one buffer: recycled under a slow reader
    with pytest.raises(fp.ProtocolViolation, match="expects version"):
        fp.explore(fp.pull_collective(2, 3, publish_before_write=True))      # flag before data


@pytest.mark.parametrize("world,calls", [(2, 5), (3, 3)])
def test_push_into_peer_slots_is_safe(world, calls):
    fp.explore(fp.push_with_back_pressure(world, calls))
    # the "consumed" wait is redundant with two buffers (kernel boundaries already order the reuse) ...
    fp.explore(fp.push_with_back_pressure(world, calls, back_pressure=False))


def test_push_into_a_single_buffer_needs_the_consumed_flag():
    fp.explore(fp.push_with_back_pressure(2, 4, double_buffered=False))
    with pytest.raises(fp.ProtocolViolation):
        fp.explore(fp.push_with_back_pressure(2, 4, double_buffered=False, back_pressure=False))


@pytest.mark.parametrize("world", [2, 3, 4])
def test_alternating_dispatch_buffers_with_one_barrier(world):
    fp.explore(fp.alternating_buffers_with_barrier(world, 3))
    with pytest.raises(fp.ProtocolViolation):
        fp.explore(fp.alternating_buffers_with_barrier(world, 3, buffers=1))


@pytest.mark.parametrize("world", [2, 3])
def test_ring_publish_barriers(world):
    fp.explore(fp.ring_publish(world, 3))                                    # one buffer, backward form: A, B, C
    fp.explore(fp.ring_publish(world, 3, backward=False))                    # one buffer, forward form: A, B
    with pytest.raises(fp.ProtocolViolation, match="overlaps a write"):
        fp.explore(fp.ring_publish(world, 3, backward=False, barrier_before_overwrite=False))
    # what ops/peer_ring.py does: two buffers alternating by call, no barrier in front of the publish
    fp.explore(fp.ring_publish(world, 4, backward=False, buffers=2, barrier_before_overwrite=False))
    fp.explore(fp.ring_publish(world, 3, backward=True, buffers=2, barrier_before_overwrite=False))


@pytest.mark.parametrize("world", [2, 3])
def test_owner_side_reduction_and_parameter_push_need_both_barriers(world):
    assert fp.explore(fp.owner_reduce_and_push(world, 3)).states > 0
    assert fp.explore(fp.owner_reduce_and_push(world, 3, barrier_after_reduce=False)).states > 0      # G3 covers for G2
    with pytest.raises(fp.ProtocolViolation):      # a fast rank's next backward overwrites a bucket that a peer still reads
        fp.explore(fp.owner_reduce_and_push(world, 2, barrier_after_reduce=False, barrier_after_push=False))
    with pytest.raises(fp.ProtocolViolation):      # a rank reads a parameter slice its owner has not stored yet
        fp.explore(fp.owner_reduce_and_push(world, 2, barrier_after_push=False))


def test_explorer_reports_deadlock_and_overlapping_writes():
    with pytest.raises(fp.ProtocolDeadlock):
        fp.explore({"a": [("wait", "never", 1)], "b": [("set", "other", 1)]})
    with pytest.raises(fp.ProtocolViolation, match="overlaps another write"):
        fp.explore({"a": [("write", "cell", 1)], "b": [("write", "cell", 2)]})
    with pytest.raises(fp.ProtocolDeadlock):                                 # a barrier one member never reaches
        fp.explore({"a": [("barrier", "x", ("a", "b"))], "b": []})
