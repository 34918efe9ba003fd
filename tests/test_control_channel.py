"""Control plane without a cluster: master and workers in one process on a free localhost port (threads),
the way the reference tests its distributed coordinator. Failures are injected on the host: a worker that stops
sending heartbeats, a worker that never joins a barrier."""
import threading
import time

from ksanallm_b200.parallel.control_channel import ControlMaster, ControlWorker, split_layers


def test_split_layers():
    assert split_layers(61, 2) == [(0, 31), (31, 61)]
    assert split_layers(32, 4) == [(0, 8), (8, 16), (16, 24), (24, 32)]
    r = split_layers(32, 2, master_offload=4)
    assert r == [(0, 12), (12, 32)]


def test_barrier_layers_blocksync_shutdown():
    m = ControlMaster("127.0.0.1", 0, 3, heartbeat_interval=0.05, heartbeat_timeout=5.0)
    ws = [ControlWorker("127.0.0.1", m.port, r, heartbeat_interval=0.05) for r in (1, 2)]
    assert m.wait_nodes(5.0)
    res = {}

    def worker(w):
        res[("b", w.rank)] = w.barrier("init", 5.0)
        res[("l", w.rank)] = w.wait_layers(5.0)
        res[("k", w.rank)] = w.sync_min("blocks", 1000 + w.rank, 5.0)
        res[("s", w.rank)] = w.wait_shutdown(5.0)

    ts = [threading.Thread(target=worker, args=(w,)) for w in ws]
    for t in ts:
        t.start()
    assert m.barrier("init", 5.0)
    ranges = m.allocate_layers(61, nccl_id="abc")
    assert m.sync_min("blocks", 900, 5.0) == 900
    m.shutdown()
    for t in ts:
        t.join(5.0)
    assert res[("b", 1)] and res[("b", 2)]
    assert res[("l", 1)] == (ranges[1] if isinstance(ranges[1], list) else list(ranges[1]), "abc") or \
        tuple(res[("l", 1)][0]) == tuple(ranges[1])
    assert res[("k", 1)] == 900 and res[("k", 2)] == 900
    assert res[("s", 1)] and res[("s", 2)]
    for w in ws:
        w.close()


def test_heartbeat_loss_is_detected_and_barrier_times_out():
    failed = []
    m = ControlMaster("127.0.0.1", 0, 2, heartbeat_interval=0.05, heartbeat_timeout=0.4, on_failure=failed.append)
    w = ControlWorker("127.0.0.1", m.port, 1, heartbeat_interval=0.05)
    assert m.wait_nodes(5.0)
    time.sleep(0.3)
    assert failed == []
    w.paused = True  # host-side fault injection: the worker goes silent
    t0 = time.time()
    ok = m.barrier("never", 3.0)  # the silent worker never joins: the barrier ends with an error, not a hang
    assert not ok and time.time() - t0 < 3.5
    assert failed == [1]
    m.shutdown()
    w.close()
