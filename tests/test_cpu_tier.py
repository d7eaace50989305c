"""Host-side machinery of the CPU tier: shared memory, TCP ring, multi-process pipeline, failure handling.
Everything here runs on CPU ranks on localhost; failures are injected on the host (a process that
never joins, a sender that drops its messages, a node that exits)."""
import multiprocessing as mp
import os
import socket
import threading
import time

import numpy as np
import pytest
import torch

from stellatrain_b200 import cpu_tier
from stellatrain_b200.ops import oracle as O
from stellatrain_b200.parallel import buckets as B

ext = cpu_tier._load()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shm_manager_offsets_and_barriers():
    session = os.getpid() * 100 + 7
    master = ext.ShmManager(True, session, 0, 2, 1 << 20)
    other = ext.ShmManager(False, session, 1, 2, 1 << 20)
    p = master.alloc(4096)
    off = master.offset_of(p)
    q = other.from_offset(off)
    a = cpu_tier._from_ptr(p, 16); b = cpu_tier._from_ptr(q, 16)
    a.fill_(3.5)
    assert float(b.sum()) == 56.0, "both mappings must see the same bytes"
    assert other.alloc(64) != p and master.data_used() >= 4096 + 64
    with pytest.raises(MemoryError):
        master.alloc(2 << 20)
    t0 = time.time()
    assert master.barrier(200) is False and time.time() - t0 < 2.0     # the other process never arrives
    res = []
    th = threading.Thread(target=lambda: res.append(other.barrier(5000)))
    th.start()
    assert master.barrier(5000) is True
    th.join()
    assert res == [True]
    assert master.arrive(42, 2) is False and master.complete(42) is False
    assert other.arrive(42, 2) is True and master.complete(42) is True
    master.depart(42, 2); other.depart(42, 2)
    del other, master


def _libzmq_path():
    """The libzmq that ships inside pyzmq, if that package is installed."""
    import glob
    import importlib.util

    spec = importlib.util.find_spec("zmq")
    if spec is None or not spec.submodule_search_locations:
        return ""
    root = os.path.dirname(list(spec.submodule_search_locations)[0])
    found = sorted(glob.glob(os.path.join(root, "pyzmq.libs", "libzmq*.so*")))
    return found[0] if found else ""


def _ring(world, port, transport="tcp"):
    boxes = [ext.CommManager("127.0.0.1", port, 5000) for _ in range(world)]
    if transport != "tcp":
        for b in boxes:
            if not b.set_data_transport(transport, _libzmq_path()):
                for x in boxes:
                    x.close()
                pytest.skip("no ZeroMQ library on this machine")
            assert b.data_transport() == transport
    boxes[0].start_server(world)
    oks = [None] * world
    ths = [threading.Thread(target=lambda r=r: oks.__setitem__(r, boxes[r].start_client(r, world, 1))) for r in range(world)]
    [t.start() for t in ths]; [t.join() for t in ths]
    assert oks == [True] * world
    return boxes


def _wait_for(fn, timeout=5.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        v = fn()
        if v:
            return v
        time.sleep(0.01)
    return fn()


def test_comm_ring_stash_narrowing_and_control_plane():
    boxes = _ring(3, free_port())
    try:
        # rank 0 -> 1: message arrives BEFORE its receive is posted (stash), 16-bit indices, fp16 values
        boxes[0].queue_tx(5, "3@1@w!0", [1, 40000, 65535], [0.5, -2.0, 1024.0], 65536, True, 1)
        assert _wait_for(lambda: boxes[1].stashed() == 1)
        boxes[1].post_recv("3@1@w!0")
        (key, flags, idx, val), = boxes[1].drain()
        assert key == "3@1@w!0" and flags == 0x03 and idx == [1, 40000, 65535] and val == [0.5, -2.0, 1024.0]
        # whole aligned blocks travel as block ids and arrive as the same entries
        blk = list(range(64, 80)) + [3] + list(range(160, 176))
        boxes[1].post_recv("blk")
        boxes[0].queue_tx(0, "blk", blk, [float(i) for i in blk], 100000)
        (key, flags, idx, val), = _wait_for(lambda: boxes[1].drain())
        assert flags == 0x18 and idx == list(range(64, 80)) + list(range(160, 176)) + [3] and val == [float(i) for i in idx]
        # wide indices stay 32-bit; priority: the smaller number leaves first
        boxes[1].post_recv("a"); boxes[1].post_recv("b")
        boxes[0].drop_keys_containing("hold", 150)          # stall the sender so both wait in the queue
        boxes[0].queue_tx(0, "hold", [0], [0.0], 10)
        boxes[0].queue_tx(9, "b", [70000], [1.0], 100000)
        boxes[0].queue_tx(1, "a", [70001], [2.0], 100000)
        got = _wait_for(lambda: (lambda d: d if len(d) == 2 else None)(boxes[1].drain() if boxes[1].stashed() >= 0 and time.sleep(0.4) is None else []))
        assert [g[0] for g in got] == ["a", "b"] and got[0][1] == 0 and got[0][2] == [70001]
        # a dropped message never arrives; nothing hangs
        boxes[2].drop_keys_containing("lost")
        boxes[0].post_recv("lost!0")
        boxes[2].queue_tx(0, "lost!0", [1], [1.0], 10)
        time.sleep(0.3)
        assert boxes[0].drain() == []
        # control plane: model relay through the broker, barrier, clock offset, stats
        res = {}
        th = threading.Thread(target=lambda: res.__setitem__("r", boxes[2].recv_init_model("init@0@w", 4)))
        th.start()
        time.sleep(0.1)
        assert boxes[0].send_init_model("init@0@w", [1.0, 2.0, 3.0, 4.0])
        th.join()
        assert res["r"] == (True, [1.0, 2.0, 3.0, 4.0])
        ths = [threading.Thread(target=lambda b=b: res.__setitem__(id(b), b.global_barrier())) for b in boxes]
        [t.start() for t in ths]; [t.join() for t in ths]
        assert all(res[id(b)] for b in boxes)
        assert abs(boxes[1].sync_time(4)) < 50.0
        assert boxes[1].report_stat(100.0, 90.0) and _wait_for(lambda: boxes[0].broker_stats()) == [(1, 100.0, 90.0)]
        assert boxes[0].bytes_sent() > 0 and boxes[1].bytes_received() > 0 and boxes[1].rx_peak_bytes_per_s() > 0
    finally:
        for b in boxes[::-1]:
            b.close()


def test_comm_ring_over_zeromq_push_pull_sockets():
    """The reference's data transport: the ring runs over ZeroMQ PUSH/PULL sockets (library opened at run time), with the
    same keyed messages, the stash for early arrivals, block and 16-bit wire forms and priority order."""
    boxes = _ring(3, free_port(), "zmq")
    try:
        boxes[0].queue_tx(5, "3@1@w!0", [1, 40000, 65535], [0.5, -2.0, 1024.0], 65536, True, 1)
        assert _wait_for(lambda: boxes[1].stashed() == 1)
        boxes[1].post_recv("3@1@w!0")
        (key, flags, idx, val), = boxes[1].drain()
        assert key == "3@1@w!0" and flags == 0x03 and idx == [1, 40000, 65535] and val == [0.5, -2.0, 1024.0]
        blk = list(range(64, 80)) + [3] + list(range(160, 176))
        boxes[2].post_recv("blk")
        boxes[1].queue_tx(0, "blk", blk, [float(i) for i in blk], 100000)
        (key, flags, idx, val), = _wait_for(lambda: boxes[2].drain())
        assert flags == 0x18 and sorted(idx) == sorted(blk) and val == [float(i) for i in idx]
        # a large message (1 MB of entries) and the ring's last hop back to rank 0
        n = 120000
        boxes[0].post_recv("big")
        boxes[2].queue_tx(0, "big", list(range(0, 2 * n, 2)), [1.0] * n, 1 << 20, True, 0, False)
        (key, flags, idx, val), = _wait_for(lambda: boxes[0].drain(), timeout=10.0)
        assert key == "big" and len(idx) == n and idx[-1] == 2 * n - 2
        assert boxes[2].bytes_sent() > 8 * n and boxes[0].bytes_received() > 8 * n
        # the control plane next to it is unchanged
        res = {}
        ths = [threading.Thread(target=lambda b=b: res.__setitem__(id(b), b.global_barrier())) for b in boxes]
        [t.start() for t in ths]; [t.join() for t in ths]
        assert all(res[id(b)] for b in boxes)
    finally:
        for b in boxes[::-1]:
            b.close()


def test_sparse_payload_block_form_round_trip():
    rng = np.random.default_rng(0)
    n = 200000
    blocks = np.sort(rng.choice(n // 16, 40, replace=False))
    idx = []
    for b in blocks[:20]:
        idx += list(range(16 * b, 16 * b + 16))
    idx += [5, 16 * int(blocks[25]) + 3, 7777]                     # loose entries between the blocks
    for b in blocks[20:30]:
        idx += list(range(16 * b, 16 * b + 16))
    idx += list(range(16 * int(blocks[35]), 16 * int(blocks[35]) + 9))   # a truncated block stays loose
    val = rng.standard_normal(len(idx)).astype(np.float32).tolist()
    flags, payload = ext.encode_sparse(idx, val, n)
    loose = len(idx) - 30 * 16
    assert flags == 0x08 | 0x10                                    # block form, 16-bit block ids (n <= 1 Mi)
    assert len(payload) == 8 + 30 * 2 + loose * 4 + len(idx) * 4
    pairs_flags, pairs = ext.encode_sparse(idx, val, n, True, 0, False)
    assert pairs_flags == 0 and len(pairs) == 4 + 8 * len(idx) and len(payload) < 0.56 * len(pairs)
    for f, p in ((flags, payload), (pairs_flags, pairs)):
        gi, gv = ext.decode_sparse(f, p, n)
        assert sorted(zip(gi, gv)) == sorted(zip(idx, val))       # same entries; whole blocks moved to the front
    gi, _ = ext.decode_sparse(flags, payload, n)
    assert gi[:16] == list(range(16 * blocks[0], 16 * blocks[0] + 16))
    # wide block ids above 1 Mi elements, 16-bit loose indices and bf16 values in a small tensor
    big = [16 * 70000 + d for d in range(16)] + [3]
    f2, p2 = ext.encode_sparse(big, [1.0] * 17, 2_000_000)
    assert f2 == 0x08 and ext.decode_sparse(f2, p2, 2_000_000)[0] == big
    small = list(range(32, 48)) + [65535]
    f3, p3 = ext.encode_sparse(small, [0.5] * 17, 65536, True, 2)
    assert f3 == 0x01 | 0x04 | 0x08 | 0x10 and len(p3) == 8 + 2 + 2 + 17 * 2
    assert ext.decode_sparse(f3, p3, 65536) == (small, [0.5] * 17)
    # malformed payloads are refused: truncated, block count beyond the entry count, index outside the tensor
    for bad in (payload[:-1], payload[:4] + (10 ** 6).to_bytes(4, "little") + payload[8:], b"\x01"):
        with pytest.raises(ValueError):
            ext.decode_sparse(flags, bad, n)
    with pytest.raises(ValueError):
        ext.decode_sparse(flags, payload, 1000)
    assert ext.decode_sparse(*ext.encode_sparse([], [], 10)) == ([], [])


def test_paced_sends_hold_the_configured_rate():
    boxes = _ring(2, free_port())
    try:
        n = 4000                                             # 32 KB per message as pairs
        idx, val = list(range(1, 2 * n, 2)), [1.0] * n       # odd indices: no whole block
        boxes[0].set_tx_rate_limit(1_000_000.0, 16 << 10)    # 1 MB/s
        for i in range(8):
            boxes[1].post_recv(f"m{i}")
        t0 = time.time()
        for i in range(8):
            boxes[0].queue_tx(i, f"m{i}", idx, val, 100000)
        got = []
        while len(got) < 8 and time.time() - t0 < 10:
            got += boxes[1].drain()
            time.sleep(0.005)
        dt = time.time() - t0
        assert len(got) == 8
        sent = boxes[0].bytes_sent()
        assert sent > 8 * 32000
        assert 0.7 * (sent - (16 << 10)) / 1e6 <= dt <= 8 * sent / 1e6, (dt, sent)     # ~0.26 s at 1 MB/s; generous above for busy hosts
        boxes[0].set_tx_rate_limit(0.0)
        boxes[1].post_recv("fast")
        t1 = time.time()
        boxes[0].queue_tx(0, "fast", idx, val, 100000)
        assert _wait_for(lambda: boxes[1].drain()) and time.time() - t1 < 1.0
    finally:
        for b in boxes[::-1]:
            b.close()


def test_bandwidth_monitor_and_interfaces():
    m = ext.BandwidthMonitor()
    for _ in range(5):
        m.add(1000)
    assert m.total_bytes() == 5000 and m.peak_bytes_per_s() >= 10000 and m.mean_bytes_per_s() == 5000
    assert any(ip == "127.0.0.1" for _, ip, lo, _ in ext.list_interfaces())
    os.environ["PUBLIC_IP"] = "10.1.2.3"
    try:
        assert ext.pick_local_ip() == "10.1.2.3"
    finally:
        del os.environ["PUBLIC_IP"]


def _oracle_run(world, local_world, steps, method, optimizer, ratio_from=None, weights=None):
    from _cpu_workers import SIZES, synthetic_grad

    params = [torch.full((n,), 0.5) for n in SIZES]
    resid = [[torch.zeros(n) for n in SIZES] for _ in range(world)]
    states = [[O.ThresholdState() for _ in SIZES] for _ in range(world)]
    if optimizer == "sgd":
        cfg, st = O.SGDConfig(lr=0.1, momentum=0.9), [O.SGDState() for _ in SIZES]
    else:
        cfg, st = O.AdamConfig(lr=1e-2), [O.AdamState() for _ in SIZES]
    for step in range(steps):
        for pi, n in enumerate(SIZES):
            k = B.entries_for(n, 0.9 if ratio_from is None or step < ratio_from[0] else ratio_from[1], world)
            streams = []
            for node in range(world):
                g = sum(synthetic_grad(node, l, step, pi, n) for l in range(local_world))
                idx, val, resid[node][pi] = O.compress_step(method, g, resid[node][pi], k, states[node][pi])
                keep = idx < n
                streams.append((idx[keep], val[keep]))
                resid[node][pi] = resid[node][pi][:n]
            dense, touched = O.merge_streams(n, streams, weights or [1.0 / world] * world)
            (O.sparse_sgd if optimizer == "sgd" else O.sparse_adam)(params[pi], dense, touched, cfg, st[pi])
    return params


def _launch(world, local_world, steps, method, optimizer, staleness, mode, join_timeout=90):
    from _cpu_workers import engine_worker

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port, session = free_port(), (os.getpid() % 10000) * 1000 + np.random.randint(0, 900)
    procs = []
    for node in range(world):
        for local in range(local_world):
            p = ctx.Process(target=engine_worker, args=(q, port, session, world, node, local_world, local, steps, method,
                                                        optimizer, staleness, mode))
            p.start()
            procs.append(p)
    results = []
    deadline = time.time() + join_timeout
    while len(results) < len(procs) and time.time() < deadline:
        try:
            results.append(q.get(timeout=0.5))
        except Exception:  # noqa: BLE001 - queue.Empty
            if mode == "die" and sum(p.is_alive() for p in procs) == 0:
                break
    for p in procs:
        p.join(timeout=5)
        if p.is_alive():
            p.kill()
    for node in range(world):
        ext.ShmManager.unlink_session(session + node)
    return results


@pytest.mark.parametrize("method,optimizer,staleness", [("topk", "sgd", 1), ("thresholdv16", "adam", 0), ("thresholdv", "adam", 1)])
def test_two_nodes_two_local_processes_match_oracle(method, optimizer, staleness):
    world, local_world, steps = 2, 2, 6
    results = _launch(world, local_world, steps, method, optimizer, staleness, "ok")
    assert len(results) == 4 and all(r[2] == "ok" for r in results), results
    want = _oracle_run(world, local_world, steps, method, optimizer)
    for node, local, _, out in results:
        assert out["drift"] == 0.0
        assert out["versions"] == [steps] * 3
        assert out["stats_len"] > 100
        for got, w in zip(out["params"], want):
            np.testing.assert_allclose(got, w.numpy(), rtol=2e-5, atol=1e-6)


@pytest.mark.parametrize("mode", ["ok_bundle", "ok_bundle_device"])
def test_two_nodes_two_local_processes_with_a_bundle_match_oracle(mode):
    """The bundle through every stage with company: sliced gather over two local processes, per-member selection on the
    node master, ring exchange of the joined streams between two nodes, merge, optimiser, copy-out into the members."""
    world, local_world, steps = 2, 2, 6
    results = _launch(world, local_world, steps, "thresholdv16", "adam", 1, mode)
    assert len(results) == 4 and all(r[2] == "ok" for r in results), results
    want = _oracle_run(world, local_world, steps, "thresholdv16", "adam")
    for node, local, _, out in results:
        assert out["drift"] == 0.0 and out["versions"] == [steps] * 3
        for got, w in zip(out["params"], want):
            np.testing.assert_allclose(got, w.numpy(), rtol=2e-5, atol=1e-6)


def test_two_nodes_exchange_over_zeromq_like_over_tcp(monkeypatch):
    """The whole host pipeline with the ring on ZeroMQ PUSH/PULL sockets: same parameters as the oracle."""
    lib = _libzmq_path()
    if not lib:
        pytest.skip("no ZeroMQ library on this machine")
    monkeypatch.setenv("STELLATRAIN_DATA_TRANSPORT", "zmq")       # the spawned node processes inherit it
    monkeypatch.setenv("STELLATRAIN_LIBZMQ", lib)
    world, local_world, steps = 2, 1, 5
    results = _launch(world, local_world, steps, "thresholdv16", "adam", 1, "ok")
    assert len(results) == 2 and all(r[2] == "ok" for r in results), results
    want = _oracle_run(world, local_world, steps, "thresholdv16", "adam")
    for node, local, _, out in results:
        assert out["drift"] == 0.0
        for got, w in zip(out["params"], want):
            np.testing.assert_allclose(np.asarray(got), w.numpy(), rtol=2e-5, atol=1e-6)


def test_wire_formats_block_ids_and_bf16_values():
    """threshold-v16 streams as block ids need fewer bytes for the same update; bf16 values keep their rounding error
    in the sender's residual, so replicas still agree exactly and stay close to the fp32 run."""
    world, steps = 2, 6
    runs = {m: _launch(world, 1, steps, "thresholdv16", "adam", 1, m) for m in ("ok", "ok_pairs", "ok_bf16")}
    for m, results in runs.items():
        assert len(results) == 2 and all(r[2] == "ok" for r in results), (m, results)
        assert all(r[3]["drift"] == 0.0 for r in results)
    by = {m: sorted(r[:2] + (r[3],) for r in results)[0][2] for m, results in runs.items()}
    for a, b in zip(by["ok"]["params"], by["ok_pairs"]["params"]):
        np.testing.assert_array_equal(a, b)                         # the wire form does not change the update
    assert by["ok"]["tx_bytes"] < 0.8 * by["ok_pairs"]["tx_bytes"]
    assert by["ok_bf16"]["tx_bytes"] < 0.8 * by["ok"]["tx_bytes"]
    # a rounding error can change which block is selected in a later step, so single elements may differ by one
    # Adam step; on average the two runs stay together
    for a, b in zip(by["ok"]["params"], by["ok_bf16"]["params"]):
        assert float(np.abs(a - b).mean()) < 0.1 * float(np.abs(a - 0.5).mean())


def test_two_nodes_two_local_processes_with_engine_device_copies():
    """Same pipeline, but every process lets the engine copy gradients in and parameters out through the stand-in
    CUDA runtime (copy streams that lag, host callbacks that start the tasks and end the copy-out)."""
    world, local_world, steps = 2, 2, 5
    results = _launch(world, local_world, steps, "thresholdv16", "adam", 1, "ok_device")
    assert len(results) == 4 and all(r[2] == "ok" for r in results), results
    want = _oracle_run(world, local_world, steps, "thresholdv16", "adam")
    for node, local, _, out in results:
        assert out["drift"] == 0.0 and out["versions"] == [steps] * 3
        for got, w in zip(out["params"], want):
            np.testing.assert_allclose(got, w.numpy(), rtol=2e-5, atol=1e-6)


def test_ratio_switch_takes_effect_at_the_same_iteration_on_every_node():
    """An instruction names the iteration from which its compression ratio counts; nodes that learn of it at different
    steps still switch at the same task, so replicas stay equal and match the oracle with the same schedule."""
    world, steps = 2, 6
    results = _launch(world, 1, steps, "topk", "adam", 1, "ok_switch")
    assert len(results) == 2 and all(r[2] == "ok" for r in results), results
    want = _oracle_run(world, 1, steps, "topk", "adam", ratio_from=(3, 0.5))
    for node, local, _, out in results:
        assert out["drift"] == 0.0 and out["versions"] == [steps] * 3
        for got, w in zip(out["params"], want):
            np.testing.assert_allclose(got, w.numpy(), rtol=2e-5, atol=1e-6)


def test_node_weights_follow_the_ring_order():
    """Unequal batch sizes per node: every node merges the streams with the same per-node weights, whichever slot a
    stream arrived in."""
    world, steps = 2, 5
    results = _launch(world, 1, steps, "topk", "sgd", 1, "ok_weights")
    assert len(results) == 2 and all(r[2] == "ok" for r in results), results
    want = _oracle_run(world, 1, steps, "topk", "sgd", weights=[0.25, 0.75])
    for node, local, _, out in results:
        assert out["drift"] == 0.0
        for got, w in zip(out["params"], want):
            np.testing.assert_allclose(got, w.numpy(), rtol=2e-5, atol=1e-6)


def test_cpu_tier_telemetry_closes_the_loop_with_the_controller():
    import torch.nn as nn
    import torch.nn.functional as F

    from stellatrain_b200.control.controller import Controller

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 8))
    eng = cpu_tier.CpuOffloadEngine(model, method="topk", ratio=0.9, optimizer="sgd", optimizer_options={"lr": 0.05},
                                    staleness=1, data_bytes=8 << 20, workers=2)
    ctl = Controller(port=0, host="127.0.0.1", adapt=False).start()
    try:
        srv = ext.TelemetryServer(f"127.0.0.1:{ctl.port}", False, 5000)
        srv.send_global_telemetry(1, 1, [p.numel() for p in model.parameters()], False, False)
        hook = cpu_tier.CpuTierTelemetry(eng, f"127.0.0.1:{ctl.port}", batch_size=16)
        x, y = torch.randn(16, 32), torch.randint(0, 8, (16,))
        shapes = []
        for it in range(20):
            xb, yb = hook.resize_batch(x, y)
            shapes.append(xb.shape[0])
            with hook.step() as marker:
                loss = F.cross_entropy(model(xb), yb)
                marker.backward_begins()
                loss.backward()
            if it == 4:
                hook._on_instruction(since=8, ubatch=24, grad_acc=1, ratio=0.6)     # what the client's callback delivers
        eng.synchronize()
        assert hook.applied == [(8, 24, 0.6)]
        assert shapes[7] == 16 and shapes[8] == 24 and hook.ratio == pytest.approx(0.6)
        assert eng.engine.compression_ratio_at(7) == pytest.approx(0.9) and eng.engine.compression_ratio_at(8) == pytest.approx(0.6)
        assert hook.last["fwd_delay_ms"] > 0.0 and hook.last["bwd_delay_ms"] > 0.0
        assert _wait_for(lambda: ctl.latest_iter >= 15), "reports did not reach the controller"
        assert len(ctl.scoreboard) == 1 and float(ctl.scoreboard.iloc[0]["bwd_ms"]) > 0.0
    finally:
        ctl.close()
        eng.close()


def test_absent_local_process_times_out_instead_of_hanging():
    t0 = time.time()
    results = _launch(1, 2, 2, "topk", "sgd", 1, "absent", join_timeout=40)
    assert time.time() - t0 < 40
    status = {(n, l): s for n, l, s, _ in results}
    assert status[(0, 1)] == "absent"
    assert status[(0, 0)] == "error", results
    assert "did not all reach configure" in [r[3] for r in results if r[2] == "error"][0]


@pytest.mark.parametrize("mode", ["drop", "die"])
def test_lost_peer_surfaces_as_error(mode):
    t0 = time.time()
    results = _launch(2, 1, 5, "topk", "sgd", 0, mode, join_timeout=60)
    assert time.time() - t0 < 60
    by_node = {n: (s, info) for n, l, s, info in results}
    assert by_node[0][0] == "error", results     # node 0 never gets node 1's stream
    assert any(w in by_node[0][1] for w in ("timed out", "failed", "closed")), by_node[0][1]


def _run_single_process_engine(device_copies, staleness, delay_ms=0, steps=6, bundle=False):
    from _cpu_workers import SIZES, synthetic_grad

    if bundle:
        return _run_bundled_engine(device_copies, staleness, delay_ms, steps)

    session = (os.getpid() % 10000) * 1000 + np.random.randint(0, 900)
    if device_copies:
        ext.install_fake_cuda(delay_ms)
    try:
        eng = ext.CpuEngine()
        eng.configure("127.0.0.1", free_port(), 1, 0, session, 1, 0, "thresholdv16", 1, staleness, 0.9, 32 << 20, 20000, 4,
                      False, True, False)
        eng.set_optimizer("adam")
        eng.configure_optimizer("lr", 1e-2)
        params = [torch.full((n,), 0.5) for n in SIZES]            # with device copies these play the device memory
        idxs = [eng.pre_train_init(pi, f"p{pi}", p.numel(), 0, p.data_ptr()) if device_copies else
                eng.pre_train_init(pi, f"p{pi}", p.numel(), p.data_ptr()) for pi, p in enumerate(params)]
        keep = []
        if device_copies:
            assert eng.device_copies_available()
            for pi, p in zip(idxs, params):
                eng.attach_device_param(pi, p.data_ptr())
        for step in range(steps):
            for pi in idxs:
                eng.pre_forward_process(pi)
            for pi in reversed(idxs):
                g = synthetic_grad(0, 0, step, pi, SIZES[pi])
                if device_copies:
                    keep.append(g)                                 # alive until the copy stream has read it
                    eng.post_backward_device(pi, g.data_ptr(), 0)
                else:
                    eng.post_backward_process(pi, g.data_ptr())
        eng.synchronize()
        versions = [eng.model_version(pi) for pi in idxs]
        counters = ext.fake_cuda_counters() if device_copies else None
        del eng
        return [p.clone() for p in params], versions, counters
    finally:
        if device_copies:
            ext.remove_fake_cuda()
        ext.ShmManager.unlink_session(session)


def _run_bundled_engine(device_copies, staleness, delay_ms, steps):
    """The same three tensors registered as ONE parameter with three members (offsets in steps of 16)."""
    from _cpu_workers import SIZES, synthetic_grad

    session = (os.getpid() % 10000) * 1000 + np.random.randint(0, 900)
    if device_copies:
        ext.install_fake_cuda(delay_ms)
    try:
        eng = ext.CpuEngine()
        eng.configure("127.0.0.1", free_port(), 1, 0, session, 1, 0, "thresholdv16", 1, staleness, 0.9, 32 << 20, 20000, 4,
                      False, True, False)
        eng.set_optimizer("adam")
        eng.configure_optimizer("lr", 1e-2)
        params = [torch.full((n,), 0.5) for n in SIZES]
        offsets, total = [], 0
        for n in SIZES:
            offsets.append(total)
            total += (n + 15) // 16 * 16
        init = torch.zeros(total)
        for p, off in zip(params, offsets):
            init[off:off + p.numel()] = p
        idx = eng.pre_train_init(0, "bundle", total, 0, init.data_ptr())
        eng.set_param_members(idx, [f"{pi}@p{pi}" for pi in range(len(SIZES))], offsets, list(SIZES),
                              [] if device_copies else [p.data_ptr() for p in params])
        with pytest.raises(RuntimeError, match="steps of 16"):
            eng.set_param_members(idx, ["a", "b"], [0, 8], [4, 4], [])
        keep = []
        if device_copies:
            eng.attach_device_members(idx, [p.data_ptr() for p in params])
        for step in range(steps):
            eng.pre_forward_process(idx)
            grads = [synthetic_grad(0, 0, step, pi, SIZES[pi]) for pi in range(len(SIZES))]
            keep.append(grads)
            if device_copies:
                eng.post_backward_device_members(idx, [g.data_ptr() for g in grads], 0)
            else:
                for pi in reversed(range(len(SIZES))):
                    eng.post_backward_member(idx, pi, grads[pi].data_ptr())
        eng.synchronize()
        versions = [eng.model_version(idx)] * len(SIZES)
        counters = ext.fake_cuda_counters() if device_copies else None
        assert eng.num_params() == 1
        del eng
        return [p.clone() for p in params], versions, counters
    finally:
        if device_copies:
            ext.remove_fake_cuda()
        ext.ShmManager.unlink_session(session)


@pytest.mark.parametrize("device_copies", [False, True])
def test_a_bundle_of_tensors_is_one_task_with_per_tensor_selection(device_copies):
    """Three tensors as one bundle: one task per iteration (one callback behind the gradient copies, one behind the
    parameter copies), and the same parameters bit for bit as three tasks give, because every member is still selected
    by itself under its own threshold."""
    steps = 6
    want, _, _ = _run_single_process_engine(False, 1, steps=steps)
    got, versions, counters = _run_single_process_engine(device_copies, 1, 2 if device_copies else 0, steps=steps, bundle=True)
    assert versions == [steps] * 3
    if device_copies:
        d2h, h2d, funcs = counters
        assert d2h == 3 * steps and h2d == 3 * steps and funcs == 2 * steps
    for a, b in zip(got, want):
        assert torch.equal(a, b)


@pytest.mark.parametrize("bundle_elems,units", [(0, 4), (1 << 16, 1), (512, 3)])
def test_offload_engine_bundles_small_tensors(bundle_elems, units):
    import torch.nn as nn
    import torch.nn.functional as F

    def run(be):
        torch.manual_seed(5)
        model = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 8))
        eng = cpu_tier.CpuOffloadEngine(model, method="thresholdv16", ratio=0.9, optimizer="adam", optimizer_options={"lr": 1e-2},
                                        staleness=1, data_bytes=8 << 20, workers=2, bundle_elems=be)
        for i in range(6):
            g = torch.Generator().manual_seed(70 + i)
            x, y = torch.randn(16, 32, generator=g), torch.randint(0, 8, (16,), generator=g)
            F.cross_entropy(model(x), y).backward()
        eng.synchronize()
        out = [p.detach().clone() for p in model.parameters()], eng.engine.num_params(), sorted(eng.state_dict()["sparsifier"]["threshold"])
        eng.close()
        return out

    want, n_plain, keys_plain = run(0)
    got, n_units, keys = run(bundle_elems)
    assert n_plain == 4 and n_units == units
    assert keys == keys_plain                       # thresholds stay per tensor, under the tensor's own key
    for a, b in zip(got, want):
        assert torch.equal(a, b)


@pytest.mark.parametrize("staleness,delay_ms", [(0, 0), (1, 0), (1, 3)])
def test_engine_device_copies_against_a_fake_runtime(staleness, delay_ms):
    """The engine's own gradient and parameter copies (event, stream wait, asynchronous copy, host callback) give the
    same parameters as the host path, also when the copy streams lag behind the host by whole iterations."""
    steps = 6
    want, _, _ = _run_single_process_engine(False, staleness, steps=steps)
    got, versions, (d2h, h2d, funcs) = _run_single_process_engine(True, staleness, delay_ms, steps=steps)
    assert versions == [steps] * 3
    assert d2h == 3 * steps and h2d == 3 * steps and funcs == 2 * 3 * steps   # one callback behind every copy
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert any(float((a - 0.5).abs().max()) > 0 for a in got)


@pytest.mark.parametrize("method,optimizer", [("thresholdv16", "adam"), ("topk", "sgd")])
def test_cpu_tier_checkpoint_resumes_bit_for_bit(method, optimizer, tmp_path):
    import torch.nn as nn
    import torch.nn.functional as F

    def make():
        torch.manual_seed(3)
        model = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 8))
        opts = {"lr": 1e-2} if optimizer == "adam" else {"lr": 0.05, "momentum": 0.9}
        return model, cpu_tier.CpuOffloadEngine(model, method=method, ratio=0.9, optimizer=optimizer, optimizer_options=opts,
                                                staleness=1, data_bytes=8 << 20, workers=2)

    def steps(model, lo, hi):
        for i in range(lo, hi):
            g = torch.Generator().manual_seed(50 + i)
            x, y = torch.randn(16, 32, generator=g), torch.randint(0, 8, (16,), generator=g)
            F.cross_entropy(model(x), y).backward()

    model, eng = make()
    steps(model, 0, 5)
    sd = eng.state_dict()
    path = tmp_path / "cpu_tier.pt"
    torch.save(sd, path)
    steps(model, 5, 9)
    eng.synchronize()
    want = [p.detach().clone() for p in model.parameters()]
    eng.close()

    model2, eng2 = make()
    with torch.no_grad():
        for p in model2.parameters():
            p.add_(1.0)                                  # anything but the saved values
    loaded = torch.load(path, weights_only=False)
    assert set(loaded) == {"model", "optimizer", "sparsifier", "engine"} and loaded["optimizer"]["kind"] == optimizer
    assert any(float(r.abs().sum()) > 0 for r in loaded["sparsifier"]["residual"].values())
    eng2.load_state_dict(loaded)
    steps(model2, 5, 9)
    eng2.synchronize()
    for a, b in zip(model2.parameters(), want):
        assert torch.equal(a.detach(), b)
    other = cpu_tier.CpuOffloadEngine(nn.Linear(4, 4), optimizer="sgd" if optimizer == "adam" else "adam", data_bytes=1 << 20, workers=1)
    with pytest.raises(ValueError, match="optimiser"):
        other.load_state_dict(loaded)
    other.close()
    eng2.close()


def test_ring_benchmark_smoke():
    from stellatrain_b200 import bench_cpu_ring as R

    sizes = [65536, 20000]
    pairs = R.run(nodes=2, gbps=0.0, steps=3, warmup=1, wire="pairs", sizes=sizes, ratio=0.9)
    blocks = R.run(nodes=2, gbps=0.0, steps=3, warmup=1, wire="blocks+bf16", sizes=sizes, ratio=0.9)
    assert pairs["ms_per_step"] > 0 and blocks["tx_bytes_per_step_per_node"] < 0.5 * pairs["tx_bytes_per_step_per_node"]


def test_pipeline_overhead_mode_leaves_the_arithmetic_out():
    """STELLATRAIN_SKIP_CRITICAL_PATHS=1: tasks run through every stage, barrier and copy, but nothing is accumulated,
    selected or applied, so the parameters stay as they were and the run measures the pipeline alone."""
    import subprocess
    import sys

    code = """
import os, torch
from stellatrain_b200 import cpu_tier
ext = cpu_tier._load()
eng = ext.CpuEngine()
eng.configure("127.0.0.1", 5555, 1, 0, os.getpid(), 1, 0, "thresholdv16", 1, 1, 0.9, 8 << 20, 20000, 2, False, False, False)
assert eng.skips_critical_paths()
eng.set_optimizer("adam"); eng.configure_optimizer("lr", 1e-2)
p = torch.full((5000,), 0.5)
i = eng.pre_train_init(0, "p", p.numel(), p.data_ptr())
for step in range(4):
    eng.pre_forward_process(i)
    g = torch.randn(5000)
    eng.post_backward_process(i, g.data_ptr())
eng.synchronize()
assert eng.model_version(i) == 4 and bool((p == 0.5).all())
print("ok")
"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120,
                         env={**os.environ, "STELLATRAIN_SKIP_CRITICAL_PATHS": "1", "PYTHONPATH": root})
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stderr[-1500:]
