"""Failure detection on the host: heartbeats and membership agreement with CPU ranks (no GPU involved)."""
import multiprocessing as mp
import socket
import time

import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q, behaviour):
    import datetime

    from torch.distributed import TCPStore

    from stellatrain_b200.parallel.heartbeat import HeartbeatMonitor, PeerLostError, agree_on_survivors

    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20),
                     wait_for_workers=False)
    hb = HeartbeatMonitor(store, rank, world, interval_s=0.1, timeout_s=1.0)
    t0 = time.time()
    try:
        for step in range(200):
            if behaviour == "leave" and rank == world - 1 and step == 5:
                hb.announce_leave()              # between steps, nothing in flight
                q.put((rank, "left", step))
                time.sleep(3.0)                  # stay around so that the store (rank 0) outlives the others
                return
            if behaviour == "die" and rank == world - 1 and step == 5:
                hb.close()                       # stops beating without a word, like a killed process
                q.put((rank, "died", step))
                time.sleep(4.0)
                return
            hb.check()
            time.sleep(0.05)
        q.put((rank, "finished", 200))
    except PeerLostError as e:
        members = agree_on_survivors(store, rank, world, e.lost, generation=1, timeout_s=5.0)
        q.put((rank, "lost", (e.lost, members, round(time.time() - t0, 2))))
        time.sleep(1.0 if rank else 3.0)


@pytest.mark.parametrize("behaviour", ["leave", "die"])
def test_peer_loss_is_detected_and_survivors_agree(behaviour):
    world, port = 3, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q, behaviour)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    deadline = time.time() + 40
    while len(results) < world and time.time() < deadline:
        try:
            r, what, info = q.get(timeout=0.5)
            results[r] = (what, info)
        except Exception:  # noqa: BLE001
            pass
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    assert results[2][0] in ("left", "died")
    for r in (0, 1):
        what, (lost, members, elapsed) = results[r]
        assert what == "lost" and lost == [2] and members == [0, 1], results
        assert elapsed < 10.0
