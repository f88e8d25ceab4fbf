"""The host loop's staging policy on a machine without a GPU: a loop created without a fabric
makes no CUDA call; the lane's mirror words are injected, polls are stepped by hand and the
decisions are read back as a log.  The expectations are the behaviour of the reference's
HostLoop::step (csrc/host/host_loop.cpp:82-146): which layer is staged when, the order of the
experts, the two halves, entries switched after the copy landed and back when the layer is done,
a restart on a new program generation, nothing while the lane is idle."""
import numpy as np

from monoserve_b200.host_loop import RawHostLoop, staging_order


def mark(layer, phase):
    return (layer << 8) | phase


def make(layers=4, experts=8, slots=2, order=None):
    loop = RawHostLoop(None, layers, experts, 1024, 512)
    order = order or [[7, 5, 3, 1]] * layers
    loop.add_lane(lane=1, region=2, w13_dst=0, w2_dst=0, slots=slots, tables=0, order=order)
    return loop


def test_stages_the_working_layer_in_order_and_flips_after_landing():
    loop = make()
    loop.inject(0, mark(0, 1))          # layer 0, attention window
    loop.step()
    assert loop.log() == [("copy", 1, 0, 7, 0)]                       # best expert first, half 0, slot 0
    loop.step()                                                      # the copy is still in flight
    assert len(loop.log()) == 1
    loop.step()                                                      # landed: entry switched, next copy issued
    assert loop.log()[1:] == [("flip", 1, 0, 7, 0), ("copy", 1, 0, 5, 1)]
    loop.step(2)
    assert loop.log()[3:] == [("flip", 1, 0, 5, 1)]                  # the half is full (2 slots): nothing more
    loop.step(3)
    assert len(loop.log()) == 4
    s = loop.stats()
    assert (s["copies"], s["flips"], s["restores"], s["bytes"]) == (2, 2, 0, 2 * (1024 + 512))
    loop.close()


def test_moe_window_moves_staging_to_the_next_layer_and_layer_done_gives_the_half_back():
    loop = make()
    loop.inject(0, mark(0, 1))
    loop.step(5)                                                     # layer 0 staged in half 0 (slots 0, 1)
    n0 = len(loop.log())
    loop.inject(0, mark(0, 2))                                       # MoE window of layer 0: its table was read
    loop.step(5)
    assert loop.log()[n0:] == [("copy", 1, 1, 7, 2), ("flip", 1, 1, 7, 2), ("copy", 1, 1, 5, 3), ("flip", 1, 1, 5, 3)]
    n1 = len(loop.log())
    loop.inject(0, mark(0, 3))                                       # layer 0 done: its entries go back to the host
    loop.step()
    got = loop.log()[n1:]
    assert got[:2] == [("restore", 1, 0, 7, 7), ("restore", 1, 0, 5, 5)]
    # the lane now works on layer 1, whose half is full; layer 2 is staged only once layer 1's MoE window began
    assert len(got) == 2
    loop.inject(0, mark(1, 2))
    loop.step()
    assert loop.log()[n1 + 2:] == [("copy", 1, 2, 7, 0)]             # half 0 again, for layer 2
    loop.close()


def test_busy_half_is_not_taken_and_last_layer_stages_nothing_beyond():
    loop = make(layers=2)
    loop.inject(0, mark(1, 2))          # the last layer's MoE window: the next layer does not exist
    loop.step(4)
    assert loop.log() == []
    loop.inject(0, mark(1, 3))          # the program's last layer is done
    loop.step(4)
    assert loop.log() == []
    loop.close()


def test_new_generation_or_idle_lane_starts_over():
    loop = make()
    loop.inject(0, mark(2, 1), gen=1)
    loop.step(5)
    assert [r[0] for r in loop.log()] == ["copy", "flip", "copy", "flip"]
    n = len(loop.log())
    loop.inject(0, mark(0, 1), gen=2)    # another program was published
    loop.step()
    got = loop.log()[n:]
    assert got[:2] == [("restore", 1, 2, 7, 7), ("restore", 1, 2, 5, 5)]
    assert got[2:] == [("copy", 1, 0, 7, 0)]
    loop.step(4)
    n = len(loop.log())
    loop.inject(0, mark(0, 1), gen=2, running=0)    # the lane stopped
    loop.step(3)
    got = loop.log()[n:]
    assert all(r[0] == "restore" for r in got) and len(got) == 2
    loop.step(3)
    assert len(loop.log()) == n + 2, "an idle lane is left alone"
    loop.close()


def test_short_order_and_bad_arguments():
    loop = make(order=[[3], [], [2, 4], [1]])
    loop.inject(0, mark(0, 1))
    loop.step(6)
    assert loop.log() == [("copy", 1, 0, 3, 0), ("flip", 1, 0, 3, 0)]
    loop.inject(0, mark(0, 3))          # layer 1 has nothing to stage
    loop.step(4)
    assert loop.log()[2:] == [("restore", 1, 0, 3, 3)]
    loop.close()
    bad = RawHostLoop(None, 2, 4, 16, 16)
    try:
        bad.add_lane(0, 2, 0, 0, 1, 0, [[9], []])
        raise AssertionError("an expert id beyond the expert count must be refused")
    except RuntimeError as e:
        assert "out of range" in str(e)
    try:
        bad.start()
        raise AssertionError("a loop without a fabric cannot start a thread")
    except RuntimeError:
        pass
    bad.close()


def test_staging_order_skips_hot_experts():
    class W:
        class cfg:
            num_experts = 6
        hot = [[0, 4], []]
    profile = np.array([[5, 1, 9, 3, 8, 2], [1, 1, 1, 1, 1, 1]], dtype=np.float64)
    assert staging_order(profile, W, 0) == [2, 3, 5, 1]
    assert staging_order(None, W, 1) == [0, 1, 2, 3, 4, 5]
