"""Native shared-memory broadcast ring: ordering across two reader processes, back-pressure, bounded waits."""
import multiprocessing as mp
import os

import pytest

native = pytest.importorskip("onecat_vllm.utils._native")


def _reader(name, idx, q):
    from onecat_vllm.utils import _native
    r = _native.ShmRing(name, 2, 4, 1 << 16, False)
    got = []
    while True:
        m = r.read(idx, 5000.0)
        if m is None or m == b"stop":
            break
        got.append(len(m))
    q.put((idx, got))


@pytest.mark.timeout(60)
def test_broadcast_order_and_backpressure():
    name = f"/onecat-test-{os.getpid()}"
    ring = native.ShmRing(name, 2, 4, 1 << 16, True)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_reader, args=(name, i, q)) for i in range(2)]
    for p in ps:
        p.start()
    for i in range(300):  # far more messages than chunks: the writer must wait for both readers
        assert ring.write(b"x" * (i + 1), 10000.0)
    assert ring.write(b"stop", 10000.0)
    res = sorted(q.get(timeout=20) for _ in ps)
    for p in ps:
        p.join(10)
    assert all(g == list(range(1, 301)) for _, g in res)
    assert ring.published() == 301


def test_waits_are_bounded():
    name = f"/onecat-test-b-{os.getpid()}"
    ring = native.ShmRing(name, 1, 2, 1024, True)
    assert ring.read(0, 20.0) is None  # nothing published: returns after the timeout
    assert ring.write(b"a", 20.0) and ring.write(b"b", 20.0)
    assert ring.write(b"c", 30.0) is False  # the only reader never consumed chunk 0: writer gives up instead of blocking
    assert ring.read(0, 20.0) == b"a"
    assert ring.write(b"c", 30.0)
    with pytest.raises(Exception):
        ring.write(b"x" * 2000, 10.0)
    buf = bytearray(16)
    assert native.spin_wait_changed(buf, 0, 0, 5.0) is False
