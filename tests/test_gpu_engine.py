"""Engine-level behaviour on one GPU: dense equivalence, staleness protocol, accumulation, checkpoint."""
import copy

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def small_net():
    torch.manual_seed(0)
    return nn.Sequential(
        nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(), nn.Conv2d(8, 8, 3, padding=1), nn.ReLU(),
        nn.AdaptiveAvgPool2d(4), nn.Flatten(1), nn.Linear(128, 37), nn.ReLU(), nn.Linear(37, 10),
    ).cuda()


def batches(n, bs=16):
    g = torch.Generator(device="cuda").manual_seed(42)
    return [(torch.randn(bs, 3, 16, 16, device="cuda", generator=g),
             torch.randint(0, 10, (bs,), device="cuda", generator=g)) for _ in range(n)]


def make_engine(model, **kw):
    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine

    cfg = EngineConfig(**{"bucket_mb": 0.004, "chunk_elems": 1024, **kw})
    return SparseDPEngine(model, cfg)


@pytest.mark.parametrize("optimizer", ["sgd", "adam"])
def test_keep_everything_equals_dense_optimizer(optimizer):
    model = small_net()
    ref = copy.deepcopy(model)
    eng = make_engine(model, compressor="topk", ratio=0.0, optimizer=optimizer, staleness=0,
                      optimizer_options={"lr": 0.05} if optimizer == "sgd" else {"lr": 1e-2})
    assert len(eng.buckets) > 1
    opt = torch.optim.SGD(ref.parameters(), lr=0.05) if optimizer == "sgd" else torch.optim.Adam(ref.parameters(), lr=1e-2)
    for x, y in batches(5):
        F.cross_entropy(model(x), y).backward()
        opt.zero_grad()
        F.cross_entropy(ref(x), y).backward()
        opt.step()
    eng.synchronize()
    for p, q in zip(model.parameters(), ref.parameters()):
        torch.testing.assert_close(p, q, rtol=1e-4, atol=1e-5)
    eng.close()


def test_staleness_one_sees_updates_up_to_two_iterations_back():
    model = small_net()
    names = [n for n, _ in model.named_parameters()]
    p0 = {n: p.detach().clone() for n, p in model.named_parameters()}
    lr = 0.1
    eng = make_engine(model, compressor="topk", ratio=0.0, optimizer="sgd", staleness=1,
                      optimizer_options={"lr": lr})
    data = batches(5)
    for x, y in data:
        F.cross_entropy(model(x), y).backward()
    eng.synchronize()
    # simulate: gradient j is taken at the parameters that contain updates 0..j-2
    shadow = small_net()
    grads = []
    for j, (x, y) in enumerate(data):
        with torch.no_grad():
            for n, p in shadow.named_parameters():
                p.copy_(p0[n] - lr * sum((g[n] for g in grads[: max(0, j - 1)]), torch.zeros_like(p0[n])))
        shadow.zero_grad()
        F.cross_entropy(shadow(x), y).backward()
        grads.append({n: p.grad.detach().clone() for n, p in shadow.named_parameters()})
    for n, p in model.named_parameters():
        want = p0[n] - lr * sum(g[n] for g in grads)
        torch.testing.assert_close(p, want, rtol=1e-4, atol=1e-5)
    eng.close()


def test_gradient_accumulation_sums_micro_batches():
    model = small_net()
    ref = copy.deepcopy(model)
    eng = make_engine(model, compressor="topk", ratio=0.0, optimizer="sgd", staleness=0, grad_accumulation=2,
                      optimizer_options={"lr": 0.05})
    opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    for x, y in batches(3, bs=16):
        for xm, ym in zip(x.chunk(2), y.chunk(2)):
            F.cross_entropy(model(xm), ym).backward()
        opt.zero_grad()
        for xm, ym in zip(x.chunk(2), y.chunk(2)):
            F.cross_entropy(ref(xm), ym).backward()
        opt.step()
    eng.synchronize()
    for p, q in zip(model.parameters(), ref.parameters()):
        torch.testing.assert_close(p, q, rtol=1e-4, atol=1e-5)
    eng.close()


@pytest.mark.parametrize("compressor", ["thresholdv16", "topk", "thresholdv", "randomk"])
@pytest.mark.parametrize("staleness", [0, 1])
def test_sparse_training_reduces_loss(compressor, staleness):
    torch.manual_seed(3)
    teacher = nn.Linear(32, 10).cuda()
    model = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 10)).cuda()
    eng = make_engine(model, compressor=compressor, ratio=0.9, optimizer="adam", staleness=staleness,
                      optimizer_options={"lr": 1e-2})
    x = torch.randn(256, 32, device="cuda")
    y = teacher(x).argmax(1)
    losses = []
    for _ in range(200):
        loss = F.cross_entropy(model(x), y)
        loss.backward()
        losses.append(float(loss.detach()))
    eng.synchronize()
    eng.check_status()
    assert losses[-1] < 0.5 * losses[0], losses[::20]
    eng.close()


def test_graphed_step_matches_eager():
    from stellatrain_b200.parallel.graphs import GraphedStep

    data = batches(6)
    results = []
    for use_graph in (False, True):
        model = small_net()
        eng = make_engine(model, compressor="topk", ratio=0.9, optimizer="adam", staleness=1)
        step = lambda x, y: _fwd_bwd(model, x, y)
        if not use_graph:
            for x, y in data[:3] + data:     # same number of warm-up steps as the graphed run
                step(x, y)
        else:
            x0, y0 = data[0]
            # warm-up inside GraphedStep runs on its static copies: feed the same three batches
            g = None
            for x, y in data[:2]:
                step(x, y)
            g = GraphedStep(eng, step, data[2], warmup=1)
            for x, y in data:
                g.copy_inputs(x, y)
                g.replay()
        eng.synchronize()
        eng.check_status()
        results.append([p.detach().clone() for p in model.parameters()])
        eng.close()
    for p, q in zip(*results):
        torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


def _fwd_bwd(model, x, y):
    loss = F.cross_entropy(model(x), y)
    loss.backward()
    return loss


def test_checkpoint_resume_is_bit_exact(monkeypatch):
    # cuDNN's weight-gradient kernels may sum in a run-dependent order; pin them for a bit-exact check
    monkeypatch.setattr(torch.backends.cudnn, "deterministic", True)
    monkeypatch.setattr(torch.backends.cudnn, "benchmark", False)
    data = batches(8)
    model = small_net()
    eng = make_engine(model, compressor="thresholdv16", ratio=0.9, optimizer="adam", staleness=1)
    for x, y in data[:4]:
        F.cross_entropy(model(x), y).backward()
    sd = {"engine": eng.state_dict(), "model": copy.deepcopy(model.state_dict())}
    for x, y in data[4:]:
        F.cross_entropy(model(x), y).backward()
    eng.synchronize()
    want = [p.detach().clone() for p in model.parameters()]
    eng.close()

    model2 = small_net()
    eng2 = make_engine(model2, compressor="thresholdv16", ratio=0.9, optimizer="adam", staleness=1)
    eng2.load_state_dict(sd["engine"])
    for x, y in data[4:]:
        F.cross_entropy(model2(x), y).backward()
    eng2.synchronize()
    for p, q in zip(model2.parameters(), want):
        assert torch.equal(p, q)
    eng2.close()


@pytest.mark.parametrize("grad_mode", ["flat", "steal"])
def test_gradient_modes_agree(grad_mode):
    """Flat-buffer gradients and stolen gradient tensors must train identically."""
    data = batches(5)
    model = small_net()
    eng = make_engine(model, compressor="topk", ratio=0.9, optimizer="adam", staleness=1, grad_mode=grad_mode,
                      grad_accumulation=2)
    for x, y in data:
        for xm, ym in zip(x.chunk(2), y.chunk(2)):
            F.cross_entropy(model(xm), ym).backward()
    eng.synchronize()
    eng.check_status()
    got = [p.detach().clone() for p in model.parameters()]
    eng.close()
    key = "_gradient_modes_reference"
    ref = globals().get(key)
    if ref is None:
        globals()[key] = got
    else:
        for p, q in zip(got, ref):
            torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


def test_channels_last_parameters_are_supported():
    model = small_net().to(memory_format=torch.channels_last)
    ref = copy.deepcopy(model)
    eng = make_engine(model, compressor="topk", ratio=0.0, optimizer="sgd", staleness=0, optimizer_options={"lr": 0.05})
    opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    for x, y in batches(3):
        x = x.contiguous(memory_format=torch.channels_last)
        F.cross_entropy(model(x), y).backward()
        opt.zero_grad()
        F.cross_entropy(ref(x), y).backward()
        opt.step()
    eng.synchronize()
    for p, q in zip(model.parameters(), ref.parameters()):
        torch.testing.assert_close(p, q, rtol=1e-4, atol=1e-5)
    eng.close()


def test_wrapper_and_module_api():
    import stellatrain_b200 as st

    st.detach()
    st.configure("127.0.0.1", 29533, 1, 0, 0, 1, 0, "topk", 1, staleness=0)
    st.configure_compression_ratio(0.5)
    st.set_optimizer("sgd")
    st.configure_optimizer("lr", 0.1)
    st.configure_optimizer("momentum", 0.9)
    with pytest.raises(RuntimeError, match="NO OPTION"):
        st.configure_optimizer("b1", 0.5)
    import torchvision

    model = st.FasterDpModelWrapper(torchvision.models.resnet18(num_classes=10).cuda())
    assert isinstance(model.module, nn.Sequential)
    x = torch.randn(4, 3, 64, 64, device="cuda")
    y = torch.randint(0, 10, (4,), device="cuda")
    loader = st.StellaTrainDataLoader([(x, y)] * 3)
    for xb, yb in loader:
        assert loader.is_eoi
        F.cross_entropy(model(xb), yb).backward()
    st.synchronize()
    idx, val = st.compress("probe", torch.randn(10000, device="cuda"), 0.99)
    assert idx.numel() == 100 and val.numel() == 100 and idx.dtype == torch.int32
    assert st.force_model_sync(0, "x", True) == 0.0
    st.detach()


def test_train_driver_checkpoints_and_resumes(tmp_path):
    """The driver on the GPU tier: periodic checkpoint, then a second run that resumes from it."""
    import subprocess
    import sys

    ck = str(tmp_path / "ck.pt")
    base = [sys.executable, "-m", "stellatrain_b200.train", "--tier", "gpu", "--model", "resnet18", "--dataset", "dummy",
            "--num-epochs", "1", "--dummy-length", "8", "--batch-size", "4", "--local-world-size", "1", "--compression", "0.9",
            "--num-classes", "10", "--log-every", "1", "--optim", "adam", "--lr", "1e-3", "--checkpoint", ck]
    first = subprocess.run(base + ["--num-iters", "4", "--checkpoint-every", "2"], capture_output=True, text=True, timeout=600)
    assert first.returncode == 0, first.stderr[-3000:]
    assert "done: 4 iterations" in first.stdout
    second = subprocess.run(base + ["--num-iters", "6", "--resume", ck], capture_output=True, text=True, timeout=600)
    assert second.returncode == 0, second.stderr[-3000:]
    assert "resumed from" in second.stdout and "at iteration 4" in second.stdout
    assert "done: 6 iterations" in second.stdout


def test_telemetry_hook_reports_to_the_controller_and_applies_instructions():
    """Closed loop on one GPU: device-timed measurements reach the controller through the native client, and an
    instruction takes effect at its effective iteration (batch size and compression ratio)."""
    import time

    import torch.nn as nn
    import torch.nn.functional as F

    from stellatrain_b200 import cpu_tier
    from stellatrain_b200.control.controller import Controller
    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine
    from stellatrain_b200.parallel.telemetry import TelemetryHook

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 8)).cuda()
    eng = SparseDPEngine(model, EngineConfig(compressor="topk", ratio=0.9, min_ratio=0.5, optimizer="sgd", staleness=1,
                                             bucket_mb=0.01, chunk_elems=1024, optimizer_options={"lr": 0.05}))
    ctl = Controller(port=0, host="127.0.0.1", adapt=False).start()
    try:
        srv = cpu_tier._load().TelemetryServer(f"127.0.0.1:{ctl.port}", False, 5000)
        srv.send_global_telemetry(1, 1, [p.numel() for p in model.parameters()], False, False)
        hook = TelemetryHook(eng, f"127.0.0.1:{ctl.port}", batch_size=16)
        x, y = torch.randn(16, 32, device="cuda"), torch.randint(0, 8, (16,), device="cuda")
        for it in range(30):
            xb, yb = hook.resize_batch(x, y)
            with hook.step() as marker:
                loss = F.cross_entropy(model(xb), yb)
                marker.backward_begins()
                loss.backward()
            if it == 5:
                hook._on_instruction(since=10, ubatch=24, grad_acc=1, ratio=0.8)    # what the client's callback delivers
            if it == 12:
                assert xb.shape[0] == 24 and eng.cfg.ratio == pytest.approx(0.8)
        eng.synchronize()
        assert hook.applied == [(10, 24, 0.8)]
        assert hook.last["fwd_delay_ms"] > 0.0 and hook.last["bwd_delay_ms"] > 0.0
        deadline = time.time() + 5.0
        while ctl.latest_iter < 20 and time.time() < deadline:
            time.sleep(0.05)
        assert ctl.latest_iter >= 20, "reports did not reach the controller"
        assert len(ctl.scoreboard) == 1 and float(ctl.scoreboard.iloc[0]["bwd_ms"]) > 0.0
    finally:
        ctl.close()
        eng.close()


def test_checkpoint_module_roundtrip_and_world_change(tmp_path):
    """utils.checkpoint on one GPU: save, load into a fresh replica, continue; a file that claims another world
    size is refused unless allow_world_change is given, and then restores parameters and moments only."""
    import torch.nn as nn
    import torch.nn.functional as F

    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine
    from stellatrain_b200.utils import checkpoint

    def make():
        torch.manual_seed(3)
        m = nn.Sequential(nn.Linear(24, 48), nn.ReLU(), nn.Linear(48, 6)).cuda()
        return m, SparseDPEngine(m, EngineConfig(compressor="thresholdv16", ratio=0.9, optimizer="adam", staleness=0,
                                                 bucket_mb=0.01, chunk_elems=1024, optimizer_options={"lr": 1e-2}))

    x, y = torch.randn(32, 24, device="cuda"), torch.randint(0, 6, (32,), device="cuda")
    m1, e1 = make()
    for _ in range(5):
        F.cross_entropy(m1(x), y).backward()
    path = checkpoint.save(str(tmp_path / "ck.pt"), m1, e1, {"global_step": 5})
    m2, e2 = make()
    assert checkpoint.load(path, m2, e2)["global_step"] == 5
    for p, q in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(p, q)
    assert torch.equal(e1.buckets[0].bucket.resid, e2.buckets[0].bucket.resid)
    # a checkpoint from a job of another size
    ck = torch.load(path, weights_only=False)
    ck["world"] = ck["engine"]["world"] = 4
    other = str(tmp_path / "ck4.pt")
    torch.save(ck, other)
    m3, e3 = make()
    with pytest.raises(ValueError):
        checkpoint.load(other, m3, e3)
    checkpoint.load(other, m3, e3, allow_world_change=True)
    for p, q in zip(m1.parameters(), m3.parameters()):
        assert torch.equal(p, q)
    assert torch.equal(e3.buckets[0].bucket.m, e1.buckets[0].bucket.m)
    assert float(e3.buckets[0].bucket.resid.abs().max()) == 0.0        # residuals belong to the old world
    F.cross_entropy(m3(x), y).backward()
    e3.synchronize()
    for e in (e1, e2, e3):
        e.close()


def test_engine_with_debug_checks_trains_like_without():
    import torch.nn as nn
    import torch.nn.functional as F

    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine

    def run(debug):
        torch.manual_seed(5)
        m = nn.Sequential(nn.Linear(40, 80), nn.ReLU(), nn.Linear(80, 5)).cuda()
        e = SparseDPEngine(m, EngineConfig(compressor="thresholdv16", ratio=0.9, optimizer="adam", staleness=1, bucket_mb=0.01,
                                           chunk_elems=1024, optimizer_options={"lr": 1e-2}, debug_checks=debug))
        g = torch.Generator(device="cuda").manual_seed(9)
        x, y = torch.randn(64, 40, device="cuda", generator=g), torch.randint(0, 5, (64,), device="cuda", generator=g)
        for _ in range(12):
            F.cross_entropy(m(x), y).backward()
        e.synchronize()
        e.check_status()
        for row in e.device_timeline():      # device clock of the last select + push and apply of every bucket
            assert 0.0 < row["select_ms"] < 50.0 and 0.0 < row["apply_ms"] < 50.0, row
            assert row["select_epoch"] == row["apply_epoch"] == 12, row
            assert row["select_end_to_apply_start_ms"] is not None
        out = [p.detach().clone() for p in m.parameters()]
        e.close()
        return out

    for a, b in zip(run(False), run(True)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("native_copies", [False, True])
def test_cpu_offload_tier_with_a_cuda_model(native_copies):
    """The CPU-offload tier under a model on the GPU: gradients go to pinned shared slots on a copy stream, the
    C++ pipeline compresses and optimises on the host, updated parameters come back by asynchronous copies, issued
    either by the Python class or by the native engine itself."""
    import torch.nn as nn
    import torch.nn.functional as F

    from stellatrain_b200.cpu_tier import CpuOffloadEngine

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(64, 128), nn.ReLU(), nn.Linear(128, 10)).cuda()
    before = [p.detach().clone() for p in model.parameters()]
    eng = CpuOffloadEngine(model, method="thresholdv16", ratio=0.9, optimizer="adam", optimizer_options={"lr": 1e-2},
                           staleness=1, data_bytes=16 << 20, workers=4, native_copies=native_copies)
    assert all(torch.equal(p, q) for p, q in zip(model.parameters(), before)), "attaching must keep the initial values"
    g = torch.Generator(device="cuda").manual_seed(1)
    x, y = torch.randn(128, 64, device="cuda", generator=g), torch.randint(0, 10, (128,), device="cuda", generator=g)
    losses = []
    for _ in range(25):
        loss = F.cross_entropy(model(x), y)
        loss.backward()
        losses.append(float(loss.detach()))
    eng.synchronize()
    assert all(torch.isfinite(p).all() for p in model.parameters())
    assert any(not torch.equal(p, q) for p, q in zip(model.parameters(), before))
    assert losses[-1] < 0.9 * losses[0]        # the hidden layer has to learn for this, not only the output bias
    assert "Total" in eng.stats_json()
    eng.close()


def _wrapper_run(graph, data, ratio_change_at=None, eager_detour_at=None, drain_and_new_shape_at=None):
    """Train small_net through the wrapper's whole-iteration call; returns the final parameters."""
    import stellatrain_b200 as st

    st.detach()
    st.configure("127.0.0.1", 29541, 1, 0, 0, 1, 0, "thresholdv16", 1, staleness=1)
    st.configure_compression_ratio(0.9)
    torch.backends.cudnn.deterministic = True       # weight-gradient kernels may otherwise sum in a run-dependent order
    st.state().engine_cfg.min_ratio = 0.5
    st.state().engine_cfg.bucket_mb = 0.004
    st.state().engine_cfg.chunk_elems = 1024
    st.set_optimizer("adam")
    st.configure_optimizer("lr", 1e-2)
    net = st.FasterDpModelWrapper(small_net(), sequential=False, graph=graph, graph_warmup=2)
    losses = []
    for i, (x, y) in enumerate(data):
        if ratio_change_at is not None and i == ratio_change_at:
            net.engine.set_compression_ratio(0.8)
        if eager_detour_at is not None and i == eager_detour_at:
            F.cross_entropy(net(x), y).backward()          # the reference's way of running an iteration, in between replays
            continue
        if drain_and_new_shape_at is not None and i >= drain_and_new_shape_at:
            if i == drain_and_new_shape_at + 1:
                st.synchronize()                           # drained pipeline right in front of the capture of a new shape
            x, y = x[: x.shape[0] // 2], y[: y.shape[0] // 2]
        losses.append(float(net.train_step(x, y)))
    st.synchronize()
    net.engine.check_status()
    out = [p.detach().clone() for p in net.parameters()], losses, bool(net._graphs), net.engine.stats.get("graph_replays", 0)
    st.detach()
    from stellatrain_b200.parallel.engine import EngineConfig

    st.state().engine_cfg = EngineConfig()          # the frontend's configuration is process-wide: leave it as found
    return out


class _LinearInGrad(nn.Module):
    """loss = sum_t <p_t, c_t>: the gradient of every tensor is the coefficient tensor handed to forward."""

    def __init__(self, sizes):
        super().__init__()
        g = torch.Generator().manual_seed(7)
        self.ps = nn.ParameterList([nn.Parameter(torch.randn(n, generator=g)) for n in sizes])

    def forward(self, coeffs):
        return sum((p * c).sum() for p, c in zip(self.ps, coeffs))


@pytest.mark.parametrize("native", [True, False])
def test_stolen_gradients_outlive_the_select_that_reads_them(native):
    """In pointer-table mode the select reads autograd's own gradient tensors.  They have to stay allocated until
    that kernel has run, also when it runs late: here the backward pass sits behind a long kernel, the host is far
    ahead, and everything the allocator considers free is taken and overwritten at once.  Exact accounting (what was
    fed equals what moved the parameters plus what is left in the residual) fails on the first gradient that was
    given away too early."""
    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine

    sizes = (5000, 70000, 300, 17, 4096)
    model = _LinearInGrad(sizes).cuda()
    p0 = [p.detach().clone() for p in model.ps]
    eng = SparseDPEngine(model, EngineConfig(compressor="topk", ratio=0.9, optimizer="sgd", staleness=1, bucket_mb=0.5,
                                             chunk_elems=1024, optimizer_options={"lr": 1.0}, native_hooks=native))
    g = torch.Generator(device="cuda").manual_seed(500)
    fed = [torch.zeros_like(p, dtype=torch.float64) for p in p0]
    junk = []
    for step in range(8):
        coeffs = [torch.randn(p.numel(), device="cuda", generator=g) * (0.5 ** (step % 3)) for p in p0]
        for f, c in zip(fed, coeffs):
            f += c.double()
        torch.cuda._sleep(30_000_000)           # about 15 ms of head start for the host
        model(coeffs).backward()
        junk = [torch.full((n,), 1e30, device="cuda") for n in sizes for _ in range(4)]
    eng.synchronize()
    eng.check_status()
    by_name = {n: p for n, p in model.named_parameters()}
    for rt, names in zip(eng.buckets, eng.param_names):
        for seg, name in zip(rt.bucket.layout.segments, names):
            i = int(name.split(".")[-1])
            resid = rt.bucket.resid[seg.off: seg.off + seg.numel].double()
            moved = p0[i].double() - by_name[name].detach().double()
            assert float((fed[i] - resid - moved).abs().max()) < 1e-4, (name, step)
    del junk
    eng.close()


@pytest.mark.parametrize("grad_mode", ["steal", "flat"])
@pytest.mark.parametrize("native", [True, False])
def test_a_select_that_runs_late_still_reads_its_own_iterations_gradients(native, grad_mode):
    """A shaped link holds every select for about 20 ms while an iteration of this small model takes far less, so the
    host and the compute stream are an iteration ahead of the sparse stream all the time.  The select of iteration i
    must nevertheless read the gradients of iteration i: the bucket's table of gradient addresses (or its flat
    gradient buffer) may only be rewritten once that select has read it.  Exact accounting shows a gradient that was
    dropped or taken twice."""
    from stellatrain_b200.control.shaper import BandwidthSchedule, DeviceTokenBucket
    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine

    sizes = (5000, 70000, 300, 17, 4096)
    model = _LinearInGrad(sizes).cuda()
    p0 = [p.detach().clone() for p in model.ps]
    eng = SparseDPEngine(model, EngineConfig(compressor="topk", ratio=0.9, optimizer="sgd", staleness=1, bucket_mb=0.5,
                                             chunk_elems=1024, optimizer_options={"lr": 1.0}, native_hooks=native,
                                             grad_mode=grad_mode))
    sched = BandwidthSchedule(seed=1, lo_gbps=0.025, hi_gbps=0.025, period_s=10.0)       # about 3 MB/s
    eng.set_link_shaper(DeviceTokenBucket(sched, eng.device, burst_bytes=1 << 12), destinations=1)
    g = torch.Generator(device="cuda").manual_seed(500)
    fed = [torch.zeros_like(p, dtype=torch.float64) for p in p0]
    for step in range(8):
        coeffs = [torch.randn(p.numel(), device="cuda", generator=g) * (0.5 ** (step % 3)) for p in p0]
        for f, c in zip(fed, coeffs):
            f += c.double()
        model(coeffs).backward()
    eng.synchronize()
    eng.check_status()
    assert eng.shaper.stats()["waited_s"] > 0.02            # the link did hold the selects back
    by_name = {n: p for n, p in model.named_parameters()}
    for rt, names in zip(eng.buckets, eng.param_names):
        for seg, name in zip(rt.bucket.layout.segments, names):
            i = int(name.split(".")[-1])
            resid = rt.bucket.resid[seg.off: seg.off + seg.numel].double()
            moved = p0[i].double() - by_name[name].detach().double()
            assert float((fed[i] - resid - moved).abs().max()) < 1e-4, name
    eng.close()


@pytest.mark.parametrize("scenario", ["plain", "ratio_change", "eager_detour", "drain_and_new_shape"])
def test_wrapper_train_step_graph_equals_eager(scenario):
    """The captured iteration is the product path of the wrapper: same parameters as eager launches, also across a
    change of the compression ratio (the capture goes stale, one eager iteration, a new capture) and across an
    iteration run the reference's way between replays (gradient addresses of eager steps never reach a replay), and
    when a new batch shape meets a pipeline that was just drained (one more eager iteration, then the capture)."""
    data = batches(12)
    kw = {"ratio_change": dict(ratio_change_at=7), "eager_detour": dict(eager_detour_at=8),
          "drain_and_new_shape": dict(drain_and_new_shape_at=6)}.get(scenario, {})
    p_eager, l_eager, captured_e, _ = _wrapper_run(False, data, **kw)
    p_graph, l_graph, captured_g, replays = _wrapper_run(True, data, **kw)
    assert not captured_e and captured_g and replays >= 5
    for p, q in zip(p_eager, p_graph):
        torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)
    assert l_graph[-1] == pytest.approx(l_eager[-1], rel=1e-4)


def test_device_token_bucket_paces_a_stream_also_inside_a_graph():
    """The shaper on the device: payloads beyond the burst hold the stream for bytes / rate, measured with the GPU's
    own clock, both launched directly and replayed from a captured graph."""
    from stellatrain_b200 import _build
    from stellatrain_b200.control.shaper import BandwidthSchedule, DeviceTokenBucket

    C = _build.load_extension("_C")
    dev = torch.device("cuda:0")
    sched = BandwidthSchedule(seed=1, lo_gbps=8.0, hi_gbps=8.0, period_s=10.0)      # 1 GB/s flat
    stamps = torch.zeros(2, dtype=torch.int64, device=dev)
    s = torch.cuda.Stream()
    for captured in (False, True):
        tb = DeviceTokenBucket(sched, dev, burst_bytes=1 << 16)
        def burst():
            C.stamp(stamps.data_ptr(), torch.cuda.current_stream().cuda_stream)
            for _ in range(10):
                tb.take(1_000_000, torch.cuda.current_stream())       # 10 MB at 1 GB/s: about 10 ms
            C.stamp(stamps.data_ptr() + 8, torch.cuda.current_stream().cuda_stream)
        with torch.cuda.stream(s):
            if captured:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s):
                    burst()
                g.replay()
            else:
                burst()
        torch.cuda.synchronize()
        ms = float(stamps[1] - stamps[0]) / 1e6
        st = tb.stats()
        assert st["sent_bytes"] == 10_000_000
        assert 8.0 < ms < 14.0, (captured, ms)
        assert tb.achieved_gbps() == pytest.approx(8.0, rel=0.25)


class _CoefficientNet(nn.Module):
    """loss = sum <p, c>: the gradient is the coefficient tensor, independent of the parameters."""

    def __init__(self):
        super().__init__()
        g = torch.Generator().manual_seed(3)
        self.ps = nn.ParameterList([nn.Parameter(torch.randn(n, generator=g)) for n in (3000, 700, 64)])

    def forward(self, coeffs):
        return sum((p * c).sum() for p, c in zip(self.ps, coeffs))


@pytest.mark.parametrize("staleness", [0, 1])
def test_rank_weights_switch_at_a_named_iteration_without_draining(staleness):
    """Merge weights that count from iteration s on: with learning rate 1 and gradients that do not depend on the
    parameters, the run that halves its weight at s ends exactly halfway between the run that stops at s and the
    run that never switches."""
    steps, since = 9, 4

    def run(n_steps, switch):
        model = _CoefficientNet().cuda()
        eng = make_engine(model, compressor="topk", ratio=0.9, optimizer="sgd", staleness=staleness,
                          optimizer_options={"lr": 1.0}, bucket_mb=0.008)
        g = torch.Generator(device="cuda").manual_seed(77)
        for i in range(n_steps):
            if switch and i == 2:
                eng.set_rank_weights([0.5], from_iteration=since)      # announced early, counts from `since`
            model([torch.randn(p.numel(), device="cuda", generator=g) for p in model.ps]).backward()
        eng.synchronize()
        eng.check_status()
        out = [p.detach().clone() for p in model.ps]
        eng.close()
        return out

    full, half, head = run(steps, False), run(steps, True), run(since, False)
    for a, b, c in zip(full, half, head):
        torch.testing.assert_close(b - c, 0.5 * (a - c), rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError):
        model = _CoefficientNet().cuda()
        eng = make_engine(model, compressor="topk", ratio=0.9, optimizer="sgd")
        model([torch.randn(p.numel(), device="cuda") for p in model.ps]).backward()
        eng.set_rank_weights([1.0], from_iteration=0)
