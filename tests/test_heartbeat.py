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


def _ckpt_rank_main(rank, world, port, q, tmp):
    import datetime

    import torch
    import torch.distributed as dist

    from stellatrain_b200.utils import checkpoint

    class _Engine:           # what save() needs of an engine
        def synchronize(self):
            pass

        def state_dict(self):
            return {"world": world, "buckets": [], "param_names": [], "state_partition": "replicated"}

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank,
                            timeout=datetime.timedelta(seconds=30))
    model = torch.nn.Linear(3, 2)
    path = checkpoint.save(f"{tmp}/only0.pt", model, _Engine(), {"step": 1}, all_ranks=False)
    # a collective right behind it: with an unmatched barrier inside save() the ranks would pair this one wrongly or block
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t)
    dist.barrier()
    q.put((rank, path, float(t)))
    dist.destroy_process_group()


def test_checkpoint_written_by_rank_0_only_keeps_the_ranks_in_step(tmp_path):
    import os

    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ckpt_rank_main, args=(r, world, port, q, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    deadline = time.time() + 90
    while len(results) < world and time.time() < deadline:
        try:
            r, path, total = q.get(timeout=0.5)
            results[r] = (path, total)
        except Exception:  # noqa: BLE001
            pass
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
    assert sorted(results) == [0, 1], results
    assert results[0][0] is not None and os.path.exists(results[0][0]) and results[1][0] is None
    assert results[0][1] == results[1][1] == 3.0
    assert not os.path.exists(tmp_path / "only0.rank1.pt")
