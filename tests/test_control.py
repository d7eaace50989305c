"""Control plane on CPU: wire format, profile evaluation, optimiser phases, controller round trip with the
native telemetry client, shaped-link schedule."""
import os
import socket
import threading
import time

import numpy as np
import pytest

from stellatrain_b200.control import messages as M
from stellatrain_b200.control.controller import Controller
from stellatrain_b200.control.gp_profile import AnalyticProfile, GPProfile, ProfileMeta, fit_profile, load_profile, matern
from stellatrain_b200.control.optimizer import (BatchRateOptimizer, Phase, TrafficModel, fit_alpha_beta, saturating)
from stellatrain_b200.control.shaper import BandwidthSchedule, TokenBucket


def test_message_roundtrip():
    lt = M.LocalTelemetry(3, 77, M.TrainConfig(32, 2, 0.97), M.Measurement(1, 2, 3, 4, 5, 6))
    raw = M.pack_local(lt)
    magic, mtype, n = M._FRAME.unpack(raw[:12])
    assert magic == M.MAGIC and mtype == M.LOCAL and n == len(raw) - 12
    assert M.parse(mtype, raw[12:]) == lt
    gi = M.GlobalInit(2, 8, False, True, [10, 20, 30])
    raw = M.pack_global_init(gi)
    assert M.parse(M.GLOBAL_INIT, raw[12:]) == gi
    ins = M.Instruction(42, M.TrainConfig(48, 1, 0.9))
    assert M.parse(M.INSTRUCTION, M.pack_instruction(ins)[12:]) == ins
    li = M.LocalInit(1, 0, 1, "NVIDIA B200")
    assert M.parse(M.LOCAL_INIT, M.pack_local_init(li)[12:]) == li


def test_gp_profile_fit_and_io(tmp_path):
    rng = np.random.default_rng(0)
    tb = rng.uniform(64, 1024, 40); bw = rng.uniform(0.2, 2.0, 40)
    truth = lambda a, b: 0.01 * np.log1p(a / 256) + 0.02 / (1 + b)
    prof = fit_profile(tb, bw, truth(tb, bw), ProfileMeta(batch_size=256, max_batch_size=1024, bandwidth=1.0))
    q_tb, q_bw = np.array([200.0, 800.0]), np.array([0.5, 1.5])
    np.testing.assert_allclose(prof.h(q_tb, q_bw), truth(q_tb, q_bw), atol=2e-3)
    prof.save(tmp_path / "p.npz")
    again = load_profile(str(tmp_path / "p.npz"))
    np.testing.assert_allclose(again.h(q_tb, q_bw), prof.h(q_tb, q_bw))
    assert matern(np.array([0.0]), 1.5)[0] == 1.0 and matern(np.array([1.0]), 0.5)[0] == pytest.approx(np.exp(-1))
    with pytest.raises(ValueError):
        load_profile("something.pkl")
    a = AnalyticProfile()
    assert a.h(1024, 1.0)[0] > a.h(128, 1.0)[0] and a.h(256, 0.1)[0] > a.h(256, 10.0)[0]


def test_alpha_beta_fit_recovers_saturation():
    xs = np.array([4, 8, 16, 32, 64, 128]); ys = saturating(40.0, 900.0, xs)
    a, b = fit_alpha_beta(list(zip(xs, ys)), (20.0, 500.0), 1.0, 1.0)
    assert a == pytest.approx(40.0, rel=0.05) and b == pytest.approx(900.0, rel=0.02)


def _rows(batches, ms_per_item, gap=0.0, ratio=0.99):
    return [{"gpu": g, "batch_size": b, "bwd_ms": b * ms_per_item[g] + 2.0, "fwd_ms": 1.0, "comp_ratio": ratio,
             "bwd_fwd_gap_ms": gap, "intra_fwd_gap_ms": 0.0} for g, b in enumerate(batches)]


def test_optimizer_phases_and_heterogeneous_batches():
    it = {"n": 0}
    opt = BatchRateOptimizer(2, 2, TrafficModel([1_000_000] * 10, "tcp"), latest_iter=lambda: it["n"], reoptimize_every=5)
    opt.set_max_batch(0, 64); opt.set_max_batch(1, 64)
    speed = [0.5, 1.0]          # GPU 1 is twice as slow per item
    batches = np.array([8.0, 8.0])
    issued = []
    for step in range(400):
        it["n"] = step
        opt.update(_rows(batches, speed))
        inst = opt.step(step, measured_mbps=400.0)
        if inst is not None:
            issued.append(inst)
            assert inst.iter == step + 3, "effective three iterations after the latest observed one"
            batches = inst.batch.copy()
        if opt.phase == Phase.RUNNING and len(issued) > 12:
            break
    assert opt.phase == Phase.RUNNING
    gaps = np.diff([i.iter for i in issued])
    assert gaps.min() >= 4, "at most one instruction per four observed iterations"
    final = issued[-1]
    assert final.batch[0] > final.batch[1], "the faster GPU gets the larger batch"
    t = opt.iteration_seconds(final.batch)
    assert abs(t[0] - t[1]) / t.max() < 0.35
    assert 0.0 <= final.comp_ratio <= 0.999


def test_allocation_stays_inside_the_sampled_batch_range():
    """A fast GPU that starts at its working batch is only ever measured on the flat part of its curve; the knee is
    then not determined by the samples and the allocation must not go below what was measured."""
    it = {"n": 0}
    opt = BatchRateOptimizer(2, 1, TrafficModel([1_000_000] * 10, "nvlink"), latest_iter=lambda: it["n"], reoptimize_every=5)
    opt.set_max_batch(0, 64); opt.set_max_batch(1, 64)

    def rows(batches):
        out = []
        for g, b in enumerate(batches):
            bwd = (13.0 + 0.3 * max(0.0, b - 24.0)) * (1.0 if g == 0 else 1.6)     # latency-bound below 24 samples
            out.append({"gpu": g, "batch_size": float(b), "bwd_ms": bwd, "fwd_ms": bwd / 2, "comp_ratio": 0.99,
                        "bwd_fwd_gap_ms": 0.0, "intra_fwd_gap_ms": 0.0})
        return out

    batches = np.array([32.0, 32.0])
    issued = []
    for step in range(300):
        it["n"] = step
        opt.update(rows(batches))
        inst = opt.step(step, measured_mbps=20000.0)
        if inst is not None:
            issued.append(inst)
            batches = inst.batch.copy()
        if opt.phase == Phase.RUNNING and len(issued) > 8:
            break
    assert opt.phase == Phase.RUNNING
    assert min(float(b) for i in issued for b in i.batch) >= 32.0, [i.batch for i in issued]
    assert issued[-1].batch[0] >= issued[-1].batch[1]                   # the slower GPU does not get the larger share


def test_compression_follows_bandwidth():
    traffic = TrafficModel([5_000_000] * 20, "nvlink")
    assert traffic.tx_bytes(0.99) == pytest.approx(8 * 20 * 50_000 + 64, rel=1e-3)
    assert traffic.tx_bytes(0.9) > 9 * traffic.tx_bytes(0.99)
    opt = BatchRateOptimizer(2, 2, traffic)
    x = np.array([32.0, 32.0])
    tight, loose = opt._min_ratio_for(x, 50.0), opt._min_ratio_for(x, 5000.0)
    assert tight > loose and tight > 0.9


def test_shipped_b200_profile_changes_the_choice_where_the_sweep_says_so():
    """The profile fitted from the convergence sweep ships for B200 and is what the controller takes when none is named.
    At half the bandwidth of its operating point the sweep needs fewer samples at a total batch of 128 to 256 than at 64
    (longer iterations carry a larger share of the gradient), so on GPUs whose throughput is already flat at 8 samples
    the objective prefers the larger batch; the analytic surrogate, monotone in the batch, stays at the knee."""
    from stellatrain_b200.control.gp_profile import AnalyticProfile, load_profile, shipped_profile_path

    assert shipped_profile_path("NVIDIA GeForce RTX 2080 Ti") is None
    assert isinstance(load_profile(None, "NVIDIA GeForce RTX 2080 Ti"), AnalyticProfile)
    shipped = load_profile(None, "NVIDIA B200")
    assert isinstance(shipped, GPProfile) and shipped.meta.bandwidth == 1.0 and 0.9 < shipped.meta.compression < 0.99
    # one profile per model, as the reference ships them: the one taken for the model closest in size is chosen
    assert shipped_profile_path("NVIDIA B200").name == "b200_gpt2_small.json"
    assert shipped_profile_path("NVIDIA B200", 60e6).name == "b200_resnet152.json"
    assert shipped_profile_path("NVIDIA B200", 110e6).name == "b200_gpt2_small.json"
    assert "resnet50" in load_profile(None, "NVIDIA B200", 25e6).meta.model
    # the fit follows the sweep it was made from (its rows are inside the file); it smooths the sweep's noise
    import json

    rows = json.loads(shipped_profile_path("NVIDIA B200").read_text())["sweep"]
    fitted = [float(shipped.h(tb, gbps / rows["ref_bandwidth_gbps"])[0]) for tb, gbps, _, _, _ in rows["rows"]]
    measured = [h for _, _, _, _, h in rows["rows"]]
    assert float(np.corrcoef(fitted, measured)[0, 1]) > 0.93
    assert max(abs(a - b) for a, b in zip(fitted, measured)) < 0.08
    # less bandwidth never needs fewer samples at a fixed batch, within the noise of the sweep
    assert float(shipped.h(64, 0.25)[0]) > float(shipped.h(64, 2.0)[0]) > float(shipped.h(64, 8.0)[0])

    traffic = TrafficModel([1_000_000] * 100, "nvlink")

    def best_total(profile):
        opt = BatchRateOptimizer(8, 2, traffic, profile)
        opt.alphas[:], opt.betas[:] = 8.0, 400.0                     # flat beyond 8 samples per GPU
        half_width_mbps, conv = 500.0, 1.0                           # objective asks h(total, 0.5)
        return min((64, 128, 256, 512), key=lambda t: opt.objective(np.full(8, t / 8.0), half_width_mbps, conv))

    assert best_total(AnalyticProfile()) == 64
    assert best_total(shipped) in (128, 256)


def test_controller_roundtrip_with_native_client():
    from stellatrain_b200 import cpu_tier

    ext = cpu_tier._load()
    ctl = Controller(port=0, host="127.0.0.1", adapt=True).start()
    try:
        uri = f"tcp://127.0.0.1:{ctl.port}"
        server = ext.TelemetryServer(uri, False, 3000)
        clients = [ext.TelemetryClient(uri, g, "NVIDIA B200", 0, g, 3000) for g in range(2)]
        assert server.send_global_telemetry(1, 2, [1000, 2000, 300000], False, False)
        got = []
        cfg = [ext.TrainConfig(8, 1, 0.99), ext.TrainConfig(8, 1, 0.99)]
        for it in range(120):
            for g, c in enumerate(clients):
                bwd = cfg[g].ubatch_size * (0.5 if g == 0 else 1.0) + 2.0
                c.report(it, cfg[g], [300.0, 300.0, 1.0, bwd, 0.0, 0.0],
                         lambda since, ub, ga, cr, g=g: (got.append((g, since, ub, cr)), setattr(cfg[g], "ubatch_size", ub)))
            time.sleep(0.01)
            if len(got) >= 6:
                break
        assert len(got) >= 2, "the controller must have issued instructions"
        assert all(ub >= 1 and 0.0 <= cr <= 0.999 for _, _, ub, cr in got)
        assert clients[0].sent() > 0 and clients[0].alive()
        assert set(ctl.scoreboard.index) == {0, 1} and ctl.scoreboard.at[0, "gpu"] == "NVIDIA B200"
        # no profile was named: the one fitted for this kind of GPU is in use, in the optimiser too
        assert isinstance(ctl.profile, GPProfile) and ctl.optimizer.profile is ctl.profile
        assert server.terminate()
        del clients, server
    finally:
        ctl.close()


def test_client_survives_controller_loss():
    from stellatrain_b200 import cpu_tier

    ext = cpu_tier._load()
    ctl = Controller(port=0, host="127.0.0.1", adapt=False).start()
    c = ext.TelemetryClient(f"127.0.0.1:{ctl.port}", 0, "cpu", 0, 0, 500)
    c.report(0, ext.TrainConfig(4, 1, 0.9), [0, 0, 1, 2, 0, 0])
    time.sleep(0.1)
    ctl.close(); ctl.stop.set()
    time.sleep(0.5)
    for i in range(5):
        c.report(i + 1, ext.TrainConfig(4, 1, 0.9), [0, 0, 1, 2, 0, 0])   # must not raise or block
    time.sleep(1.2)
    assert c.queued() <= 5
    with pytest.raises(RuntimeError):
        ext.TelemetryClient("127.0.0.1:1", 0, "cpu", 0, 0, 300)


def test_schedule_and_token_bucket():
    s1, s2 = BandwidthSchedule(seed=7), BandwidthSchedule(seed=7)
    ts = np.linspace(0, 100, 200)
    v = [s1.gbps_at(t) for t in ts]
    assert v == [s2.gbps_at(t) for t in ts] and min(v) >= 10.0 and max(v) <= 40.0 and len(set(v)) > 10
    assert BandwidthSchedule(seed=8).gbps_at(0.0) != s1.gbps_at(0.0)
    now = {"t": 0.0}
    tb = TokenBucket(BandwidthSchedule(seed=1, lo_gbps=8.0, hi_gbps=8.0), burst_bytes=1000, clock=lambda: now["t"])
    assert tb.delay_for(1000) == 0.0
    w = tb.delay_for(1_000_000)              # 1 MB at 1 GB/s
    assert w == pytest.approx(1e-3, rel=0.01)
    now["t"] += w + 0.5
    assert tb.delay_for(500) == 0.0


def test_optimizer_state_survives_a_restart():
    """A controller restarted from its state_dict issues the same instructions as one that kept running."""
    import copy
    import pickle

    def make(it):
        o = BatchRateOptimizer(2, 2, TrafficModel([1_000_000] * 10, "tcp"), latest_iter=lambda: it["n"], reoptimize_every=5)
        o.set_max_batch(0, 64); o.set_max_batch(1, 64)
        return o

    it_a, it_b = {"n": 0}, {"n": 0}
    a = make(it_a)
    speed, batches = [0.5, 1.0], np.array([8.0, 8.0])
    for step in range(120):
        it_a["n"] = step
        a.update(_rows(batches, speed))
        inst = a.step(step, measured_mbps=400.0)
        if inst is not None:
            batches = inst.batch.copy()
    sd = pickle.loads(pickle.dumps(a.state_dict()))         # what torch.save would do with checkpoint "extra"
    b = make(it_b)
    b.load_state_dict(copy.deepcopy(sd))
    assert b.phase == a.phase and len(b.history) == len(a.history)
    batches_a, batches_b = batches.copy(), batches.copy()
    for step in range(120, 200):
        it_a["n"] = it_b["n"] = step
        a.update(_rows(batches_a, speed)); b.update(_rows(batches_b, speed))
        ia, ib = a.step(step, measured_mbps=400.0), b.step(step, measured_mbps=400.0)
        assert (ia is None) == (ib is None)
        if ia is not None:
            assert ia.iter == ib.iter and np.allclose(ia.batch, ib.batch) and ia.comp_ratio == pytest.approx(ib.comp_ratio)
            batches_a, batches_b = ia.batch.copy(), ib.batch.copy()


def test_controller_keeps_its_state_across_a_restart(tmp_path):
    from stellatrain_b200.control import messages as M
    from stellatrain_b200.control.controller import Controller

    path = str(tmp_path / "controller.state")
    gi = M.GlobalInit(num_nodes=1, num_gpus=2, param_counts=[1000, 2000], grad_fp16=False, grad_idx_u16=False)
    a = Controller(port=0, host="127.0.0.1", adapt=True, state_path=path)
    try:
        a._on_global_init(gi)
        a.optimizer.alphas[:] = [12.5, 30.0]
        a.optimizer.phase = Phase.RUNNING
        a.latest_iter = 77
        a.save_state()
    finally:
        a.close()
    b = Controller(port=0, host="127.0.0.1", adapt=True, state_path=path)
    try:
        b._on_global_init(gi)
        assert b.optimizer.alphas.tolist() == [12.5, 30.0] and b.optimizer.phase == Phase.RUNNING and b.latest_iter == 77
        # a state file of a job with another number of GPUs is ignored
        b._on_global_init(M.GlobalInit(num_nodes=1, num_gpus=3, param_counts=[1000], grad_fp16=False, grad_idx_u16=False))
        assert len(b.optimizer.alphas) == 3 and b.optimizer.phase == Phase.INIT_WARMUP
    finally:
        b.close()


def test_traffic_model_matches_the_block_wire_format():
    """The controller's byte model of the framed TCP transport follows the encoder: whole blocks of 16 entries behind
    one block id, loose entries as pairs."""
    from stellatrain_b200 import cpu_tier

    ext = cpu_tier._load()
    n, ratio = 400_000, 0.99
    k = 4000
    idx = [j for b in range(0, k // 16) for j in range(64 * b, 64 * b + 16)]
    _, payload = ext.encode_sparse(idx, [1.0] * len(idx), n)
    pairs = TrafficModel([n], "tcp").tx_bytes(ratio)
    blocks = TrafficModel([n], "tcp", grad_block16=True).tx_bytes(ratio)
    header = 24 + 16
    assert abs((blocks - header) - len(payload)) <= 0.05 * len(payload) + 0x42 * 12   # payload + per-segment headers
    assert blocks < 0.56 * pairs
    assert TrafficModel([8], "tcp", grad_block16=True).tx_bytes(0.5) == TrafficModel([8], "tcp").tx_bytes(0.5)


class _FakeKernel:                       # stand-ins whose pickles look like scikit-optimize's to the converter
    def __init__(self, **kw):
        self.__dict__.update(kw)


class Sum(_FakeKernel): pass             # noqa: E701
class Product(_FakeKernel): pass         # noqa: E701
class ConstantKernel(_FakeKernel): pass  # noqa: E701
class Matern(_FakeKernel): pass          # noqa: E701
class WhiteKernel(_FakeKernel): pass     # noqa: E701
class GaussianProcessRegressor(_FakeKernel): pass   # noqa: E701


class OptimizeResult(dict):
    pass


class _Boom:
    def __reduce__(self):
        import os

        return (os.system, ("touch /dev/null/should_never_run",))


def test_profile_converter_reads_a_result_pickle_without_running_it(tmp_path):
    import joblib

    from stellatrain_b200.control import convert_profile as C
    from stellatrain_b200.control.gp_profile import GPProfile, ProfileMeta, fit_profile, load_profile

    meta = ProfileMeta(batch_size=256, max_batch_size=1024, min_batch_size=64, bandwidth=1.0, compression=0.9, model="toy")
    rng = np.random.default_rng(0)
    tb, bw = rng.uniform(64, 1024, 20), rng.uniform(0.1, 1.0, 20)
    want = fit_profile(tb, bw, 0.05 + 0.1 * tb / 1024 + 0.02 / bw, meta, length_scale=(0.4, 0.7), nu=1.5)
    gp = GaussianProcessRegressor(
        X_train_=np.asfortranarray(want.x_train), alpha_=want.alpha, _y_train_mean=np.float64(want.y_mean), _y_train_std=np.float64(want.y_std),
        kernel_=Sum(k1=Product(k1=ConstantKernel(constant_value=1.0), k2=Matern(length_scale=np.array([0.4, 0.7]), nu=1.5)),
                    k2=WhiteKernel(noise_level=0.0)))
    res = OptimizeResult(models=[None, gp], metadata=dict(meta.__dict__), x=[0.1, 0.2], trap=_Boom())
    src = tmp_path / "toy.pkl"
    joblib.dump(res, src, compress=3)          # the container scikit-optimize writes: zlib, arrays as raw payloads

    records = C.read_records(str(src))
    assert isinstance(records["trap"], C.Record) and records["trap"]._name.endswith("system")   # recorded, not called
    got = C.convert(str(src), str(tmp_path / "toy.npz"))
    assert got.nu == 1.5 and got.meta.model == "toy" and got.meta.max_batch_size == 1024
    q_tb, q_bw = np.array([100.0, 512.0, 900.0]), np.array([0.2, 0.5, 1.0])
    np.testing.assert_allclose(got.h(q_tb, q_bw), want.h(q_tb, q_bw), rtol=1e-12)
    np.testing.assert_allclose(load_profile(str(tmp_path / "toy.npz")).h(q_tb, q_bw), want.h(q_tb, q_bw), rtol=1e-12)
    C.convert(str(src), str(tmp_path / "toy.json"))
    np.testing.assert_allclose(GPProfile.load(tmp_path / "toy.json").h(q_tb, q_bw), want.h(q_tb, q_bw), rtol=1e-9)
    with pytest.raises(ValueError):
        load_profile(str(src))                 # the controller itself still refuses pickles
    bad = tmp_path / "bad.pkl"
    joblib.dump({"models": []}, bad)
    with pytest.raises(ValueError):
        C.convert(str(bad))


@pytest.mark.parametrize("name", ["resnet152_frac50_368", "resnet50_frac50_256", "vitb16_frac25_512.v2", "swinb_frac25_512"])
def test_profile_converter_on_published_profiles(name):
    """Where the upstream tree is at hand: its profiles convert, and the converted Gaussian process reproduces its own
    training targets through (K + noise I) alpha = y, which pins kernel, length scales and constant."""
    from pathlib import Path

    from stellatrain_b200.control import convert_profile as C

    here = Path(__file__).resolve().parent.parent
    tree = Path(os.environ.get("STELLATRAIN_REFERENCE") or here.parent / "reference")    # named, else beside this repository
    src = tree / "bayesian" / "profile" / f"{name}.pkl"
    if not src.exists():
        pytest.skip("upstream profiles not available")
    rec = C.read_records(str(src))
    prof = C.profile_from_records(rec)
    gp = rec["models"][-1]
    y = np.asarray(gp.attr("y_train_"), float)
    fit = prof._k(prof.x_train) @ prof.alpha + float(gp.attr("noise_")) * prof.alpha
    np.testing.assert_allclose(fit, y, atol=1e-6)
    assert prof.meta.bandwidth == 1.0 and prof.meta.compression == 0.9 and prof.meta.max_batch_size in (1024.0, 2048.0)
    assert np.isfinite(prof.h(prof.meta.batch_size, 1.0)).all()


def test_client_may_be_destroyed_from_its_own_thread():
    """A callback can own the client (a bound method of the object that holds it).  When the reports still queued in the
    client's thread are the last owners, the client is destroyed on that thread; it must let the thread go instead of
    joining itself (which ends the process with 'Resource deadlock avoided')."""
    import gc

    from stellatrain_b200 import cpu_tier

    ext = cpu_tier._load()
    ctl = Controller(port=0, host="127.0.0.1", adapt=False).start()
    try:
        before = ext.telemetry_clients_destroyed_on_own_thread()

        class Holder:
            def __init__(self):
                self.client = ext.TelemetryClient(f"127.0.0.1:{ctl.port}", 0, "cpu", 0, 0, 2000)
                self.seen = 0

            def on_instruction(self, since, ubatch, grad_acc, ratio):
                self.seen += 1

        for _ in range(5):
            h = Holder()
            for i in range(300):
                h.client.report(i, ext.TrainConfig(4, 1, 0.9), [0, 0, 1, 2, 0, 0], h.on_instruction)
            del h                                       # the queue inside the client's thread now owns the holder
            gc.collect()
        time.sleep(1.0)
        deadline = time.time() + 10
        while ctl.latest_iter < 250 and time.time() < deadline:
            time.sleep(0.05)
        assert ctl.latest_iter >= 250
        deadline = time.time() + 30
        while ext.telemetry_clients_destroyed_on_own_thread() == before and time.time() < deadline:
            time.sleep(0.1)
        assert ext.telemetry_clients_destroyed_on_own_thread() > before      # the situation did arise
    finally:
        ctl.close()


def test_profile_reader_refuses_the_numpy_scalar_detour(tmp_path):
    """numpy's scalar constructor unpickles its payload itself when the dtype is object: a pickle can smuggle a second,
    unrestricted pickle through it.  The reader refuses object-typed scalars and still reads ordinary ones."""
    import pickle

    from stellatrain_b200.control import convert_profile as C

    marker = tmp_path / "ran"

    class Inner:
        def __reduce__(self):
            return (open, (str(marker), "w"))

    inner = pickle.dumps(Inner())

    class Outer:
        def __reduce__(self):
            import numpy._core.multiarray as ma

            return (ma.scalar, (np.dtype("O"), inner))

    bad = tmp_path / "bad.pkl"
    bad.write_bytes(pickle.dumps({"models": [Outer()]}))
    with pytest.raises(pickle.UnpicklingError):
        C.read_records(str(bad))
    assert not marker.exists()
    good = tmp_path / "good.pkl"
    good.write_bytes(pickle.dumps({"x": np.float64(2.5), "n": np.int32(7)}))
    rec = C.read_records(str(good))
    assert float(rec["x"]) == 2.5 and int(rec["n"]) == 7


def test_client_destroyed_with_callbacks_still_queued_does_not_wait_for_itself():
    """Dropping the client on the Python thread while its thread still holds Python callbacks: the destructor joins
    that thread, which needs the interpreter lock to release the callbacks, so the lock must not be held meanwhile."""
    from stellatrain_b200 import cpu_tier

    ext = cpu_tier._load()
    ctl = Controller(port=0, host="127.0.0.1", adapt=False).start()
    try:
        t0 = time.time()
        for _ in range(10):
            c = ext.TelemetryClient(f"127.0.0.1:{ctl.port}", 0, "cpu", 0, 0, 2000)
            for i in range(200):
                c.report(i, ext.TrainConfig(4, 1, 0.9), [0, 0, 1, 2, 0, 0], lambda *a: None)
            del c
        assert time.time() - t0 < 30
    finally:
        ctl.close()


def test_controller_in_a_process_of_its_own_serves_clients_and_terminates():
    """`spawn_controller` starts `python -m stellatrain_b200.control.controller`, waits until it listens, and the
    native server shim and clients work against it; TERMINATE ends the process."""
    from stellatrain_b200 import cpu_tier
    from stellatrain_b200.control.controller import spawn_controller

    ext = cpu_tier._load()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    proc = spawn_controller(port, max_batch=48)
    try:
        uri = f"127.0.0.1:{port}"
        server = ext.TelemetryServer(uri, False, 5000)
        assert server.send_global_telemetry(1, 2, [1000, 2000, 300000], False, False)
        clients = [ext.TelemetryClient(uri, g, "NVIDIA B200", 0, g, 5000) for g in range(2)]
        got = []
        cfg = [ext.TrainConfig(8, 1, 0.99), ext.TrainConfig(8, 1, 0.99)]
        for it in range(200):
            for g, c in enumerate(clients):
                c.report(it, cfg[g], [300.0, 300.0, 1.0, cfg[g].ubatch_size * 0.5 + 2.0, 0.0, 0.0],
                         lambda since, ub, ga, cr, g=g: (got.append((g, since, ub, cr)), setattr(cfg[g], "ubatch_size", ub)))
            time.sleep(0.01)
            if len(got) >= 4:
                break
        assert len(got) >= 2 and all(1 <= ub <= 48 for _, _, ub, _ in got), got      # the batch ceiling reached the child
        assert server.terminate()
        assert proc.wait(timeout=10) == 0
        del clients, server
    finally:
        if proc.poll() is None:
            proc.kill()


def test_single_instance_guard_leaves_other_processes_alone(tmp_path):
    """The pid file of a controller that is long gone may name a process id that belongs to somebody else by now: the
    guard only ends a process that still is a controller."""
    import subprocess
    import sys

    from stellatrain_b200.control import controller as C

    port = 59999
    pid_file = f"/tmp/stellatrain-b200-controller-{port}.pid"
    bystander = subprocess.Popen([sys.executable, "-c", "import time; time.sleep(30)"])
    try:
        with open(pid_file, "w") as f:
            f.write(str(bystander.pid))
        C._single_instance(port)
        time.sleep(0.3)
        assert bystander.poll() is None                       # still running
        assert int(open(pid_file).read()) == os.getpid()      # the file names the new owner
    finally:
        bystander.kill()
        try:
            os.unlink(pid_file)
        except OSError:
            pass
