"""Peer-memory exchange on 2+ GPUs: one process per GPU, NCCL only for rendezvous and barriers."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn(fn, world, *args, env=None):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = []
    for r in range(world):
        p = ctx.Process(target=_entry, args=(fn, r, world, port, q, env or {}, args))
        p.start()
        procs.append(p)
    import time

    deadline = time.time() + 240          # for all ranks together: a hung rank costs GPU time on every GPU of the box
    for p in procs:
        p.join(timeout=max(1.0, deadline - time.time()))
    results = {}
    while not q.empty():
        r, ok, payload = q.get()
        results[r] = (ok, payload)
    hung = [r for r, p in enumerate(procs) if p.is_alive()]
    for p in procs:
        if p.is_alive():
            p.kill()
    if hung:
        # a rank that failed leaves the others waiting in their next collective: say what it died of
        died = "\n".join(f"rank {r} failed:\n{payload}" for r, (ok, payload) in sorted(results.items()) if not ok)
        pytest.fail(f"ranks {hung} did not finish" + (f"; {died}" if died else f"; finished: {sorted(results)}"))
    assert len(results) == world, f"missing results: {sorted(results)}"
    for r in range(world):
        ok, payload = results[r]
        assert ok, f"rank {r} failed:\n{payload}"
    return [results[r][1] for r in range(world)]


def _entry(fn, rank, world, port, q, env, args):
    import traceback

    import faulthandler

    faulthandler.dump_traceback_later(200, exit=False)      # a rank that hangs says where, before the parent ends it
    os.environ.update(env)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank,
                                device_id=torch.device("cuda", rank))
        out = fn(rank, world, *args)
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, True, out))
    except Exception:  # noqa: BLE001
        q.put((rank, False, traceback.format_exc()))


def _net():
    import torch.nn as nn

    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(48, 96), nn.ReLU(), nn.Linear(96, 96), nn.ReLU(), nn.Linear(96, 10)).cuda()


def _data(rank, steps, bs=32):
    g = torch.Generator(device="cuda").manual_seed(1000 + rank)
    return [(torch.randn(bs, 48, device="cuda", generator=g), torch.randint(0, 10, (bs,), device="cuda", generator=g))
            for _ in range(steps)]


def _worker_dense_equivalence(rank, world, transport, multicast):
    import torch.distributed as dist
    import torch.nn.functional as F

    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine

    model = _net()
    eng = SparseDPEngine(model, EngineConfig(compressor="topk", ratio=0.0, optimizer="sgd", staleness=0,
                                             divide_k_by_world=False, bucket_mb=0.02, chunk_elems=1024,
                                             transport=transport, multicast=multicast,
                                             optimizer_options={"lr": 0.1}))
    steps = 4
    mine = _data(rank, steps)
    for x, y in mine:
        F.cross_entropy(model(x), y).backward()
    eng.synchronize()
    drift = eng.replica_drift()
    # dense reference: mean over ranks of the per-rank mean gradient == one big batch of equal shards
    ref = _net()
    opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    everyone = [_data(r, steps) for r in range(world)]
    for s in range(steps):
        opt.zero_grad()
        x = torch.cat([everyone[r][s][0] for r in range(world)])
        y = torch.cat([everyone[r][s][1] for r in range(world)])
        F.cross_entropy(ref(x), y).backward()
        opt.step()
    err = max(float((p - q).abs().max()) for p, q in zip(model.parameters(), ref.parameters()))
    info = {"drift": drift, "err": err, "backend": eng.pool.backend if eng.pool else "local",
            "mc": bool(eng.pool and eng.pool.mc_ptr)}
    eng.close()
    return info


@pytest.mark.parametrize("transport,multicast", [("peer", False), ("peer", True), ("nccl", False)])
def test_exchange_equals_dense_data_parallel(transport, multicast):
    world = min(torch.cuda.device_count(), 4)
    outs = _spawn(_worker_dense_equivalence, world, transport, multicast)
    for o in outs:
        assert o["err"] < 1e-4, outs
        assert o["drift"] <= 1e-6, outs      # replicas may differ only by atomic-add rounding order


def _worker_sparse_parity(rank, world, compressor, staleness, partition="replicated", wire="wide", deterministic=False):
    import torch.nn.functional as F

    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine

    model = _net()
    if rank != 0:   # broadcast_init must overwrite this
        with torch.no_grad():
            for p in model.parameters():
                p.add_(1.0)
    eng = SparseDPEngine(model, EngineConfig(compressor=compressor, ratio=0.9, optimizer="adam", staleness=staleness,
                                             bucket_mb=0.02, chunk_elems=1024, optimizer_options={"lr": 1e-2},
                                             state_partition=partition, wire_format=wire,
                                             deterministic_merge=deterministic))
    first = None
    for x, y in _data(rank, 30):
        loss = F.cross_entropy(model(x), y)
        loss.backward()
        first = first if first is not None else float(loss.detach())
    eng.synchronize()
    eng.check_status()
    drift = eng.replica_drift()
    state_elems = sum(rt.bucket.m.numel() for rt in eng.buckets)
    total_elems = sum(rt.bucket.layout.n_total for rt in eng.buckets)
    checksum = float(sum(p.detach().double().sum() for p in model.parameters()))
    eng.close()
    return {"drift": drift, "first": first, "last": float(loss.detach()), "state_elems": state_elems,
            "total_elems": total_elems, "checksum": checksum}


@pytest.mark.parametrize("compressor", ["thresholdv16", "topk", "thresholdv"])
@pytest.mark.parametrize("staleness", [0, 1])
def test_sparse_replicas_stay_in_sync(compressor, staleness):
    world = min(torch.cuda.device_count(), 4)
    outs = _spawn(_worker_sparse_parity, world, compressor, staleness)
    for o in outs:
        assert o["drift"] <= 1e-5, outs
        assert o["first"] == pytest.approx(outs[0]["first"], rel=0.5)


@pytest.mark.parametrize("multicast", [True, False])
@pytest.mark.parametrize("staleness", [0, 1])
def test_partitioned_optimizer_state(staleness, multicast):
    """Every tensor's optimiser state on one rank; owners store the new values into all replicas."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs 2 GPUs")
    env = {} if multicast else {"STELLATRAIN_NVLS": "0"}
    # Three or more contributions to one element add up in an order that differs from run to run, and a selection by
    # threshold turns one unit in the last place into a different choice of blocks a few steps later: two runs are
    # only comparable when the merge adds in rank order.
    par = _spawn(_worker_sparse_parity, world, "thresholdv16", staleness, "owner", "wide", True, env=env)
    rep = _spawn(_worker_sparse_parity, world, "thresholdv16", staleness, "replicated", "wide", True, env=env)
    for o in par:
        assert o["drift"] == 0.0, par                      # values are copied from the owner, never recomputed
        assert o["state_elems"] < o["total_elems"], par
    assert sum(o["state_elems"] for o in par) <= par[0]["total_elems"] + 16 * world * 8
    # same training trajectory as with replicated state, up to the order of floating-point additions
    assert par[0]["checksum"] == pytest.approx(rep[0]["checksum"], rel=1e-4, abs=1e-3)
    assert par[0]["last"] == pytest.approx(rep[0]["last"], rel=1e-2, abs=1e-3)


class _LinearInGrad(torch.nn.Module):
    """loss = sum_t <p_t, c_t>: the gradient of every tensor is the coefficient tensor handed to forward, whatever the
    parameters are, so a run's gradients are known exactly and do not depend on how earlier updates were rounded."""

    SIZES = (5000, 70000, 300, 17, 4096)      # below and above the 65536-element limit of the narrow format

    def __init__(self):
        super().__init__()
        g = torch.Generator().manual_seed(7)
        self.ps = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(n, generator=g)) for n in self.SIZES])

    def forward(self, coeffs):
        return sum((p * c).sum() for p, c in zip(self.ps, coeffs))


def _worker_mass_conservation(rank, world, partition, wire, compressor):
    import torch.distributed as dist

    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine

    model = _LinearInGrad().cuda()
    p0 = [p.detach().clone() for p in model.ps]
    eng = SparseDPEngine(model, EngineConfig(compressor=compressor, ratio=0.9, optimizer="sgd", staleness=1, bucket_mb=0.5,
                                             chunk_elems=1024, optimizer_options={"lr": 1.0}, state_partition=partition,
                                             wire_format=wire))
    g = torch.Generator(device="cuda").manual_seed(500 + rank)
    fed = [torch.zeros_like(p, dtype=torch.float64) for p in p0]
    for step in range(12):
        coeffs = [torch.randn(p.numel(), device="cuda", generator=g) * (0.5 ** (step % 3)) for p in p0]
        model(coeffs).backward()
        for f, c in zip(fed, coeffs):
            f += c.double()
    eng.synchronize()
    eng.check_status()
    drift = eng.replica_drift()
    # What this rank has not sent yet sits in its residual; everything else was sent, merged with weight 1/world and
    # applied with learning rate 1, so  world * (p0 - p)  ==  sum over ranks of (fed - residual)  element for element.
    worst, scale = 0.0, 0.0
    by_name = {n: p for n, p in model.named_parameters()}
    for rt, names in zip(eng.buckets, eng.param_names):
        for seg, name in zip(rt.bucket.layout.segments, names):
            i = int(name.split(".")[-1])
            resid = rt.bucket.resid[seg.off: seg.off + seg.numel].double()
            sent = fed[i] - resid
            dist.all_reduce(sent)
            moved = (p0[i].double() - by_name[name].detach().double()) * world
            worst = max(worst, float((sent - moved).abs().max()))
            scale = max(scale, float(sent.abs().max()))
    narrow_segments = sum(rt.bucket.layout.is_narrow(s) for rt in eng.buckets for s in rt.bucket.layout.segments)
    eng.close()
    return {"drift": drift, "worst": worst, "scale": scale, "narrow_segments": narrow_segments}


@pytest.mark.parametrize("compressor", ["topk", "thresholdv16"])
@pytest.mark.parametrize("wire", ["wide", "narrow"])
@pytest.mark.parametrize("partition", ["replicated", "owner"])
def test_mass_conservation(partition, wire, compressor):
    """Nothing is lost on the way: sent + residual equals the sum of the gradients on every rank, and the parameters
    moved by exactly the mean of what was sent.  With the narrow wire format (u16 index, bf16 value for tensors below
    65536 elements) the rounding error of every value must have stayed in the sender's residual: a lost error shows
    up here as a mismatch of 2^-9 of the value, four orders of magnitude over the bound."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs 2 GPUs")
    outs = _spawn(_worker_mass_conservation, world, partition, wire, compressor)
    for o in outs:
        assert o["drift"] <= (0.0 if partition == "owner" else 1e-5), outs
        assert o["scale"] > 1.0, outs                        # the run did send something
        assert o["worst"] <= 2e-5 * max(1.0, o["scale"]), outs
        assert o["narrow_segments"] == (4 if wire == "narrow" else 0), outs


@pytest.mark.parametrize("partition", ["replicated", "owner"])
def test_narrow_wire_format_trains_like_wide(partition):
    """Training with 4-byte entries follows the wide format: same loss to a few per cent, replicas in step."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs 2 GPUs")
    narrow = _spawn(_worker_sparse_parity, world, "topk", 1, partition, "narrow", True)
    wide = _spawn(_worker_sparse_parity, world, "topk", 1, partition, "wide", True)
    for o in narrow:
        assert o["drift"] <= (0.0 if partition == "owner" else 1e-5), narrow
    assert narrow[0]["last"] == pytest.approx(wide[0]["last"], rel=5e-2, abs=5e-3)


def _worker_gathered_checkpoint(rank, world, tmp):
    import torch.nn.functional as F

    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine
    from stellatrain_b200.utils import checkpoint

    def make():
        model = _net()
        return model, SparseDPEngine(model, EngineConfig(compressor="topk", ratio=0.9, optimizer="adam", staleness=1,
                                                         bucket_mb=0.02, chunk_elems=1024, optimizer_options={"lr": 1e-2},
                                                         state_partition="owner"))

    m1, e1 = make()
    data = _data(rank, 12)
    for x, y in data[:6]:
        F.cross_entropy(m1(x), y).backward()
    path = checkpoint.save(f"{tmp}/gathered.pt", m1, e1, {"global_step": 6}, gather=True)
    single = os.path.exists(f"{tmp}/gathered.pt") and not os.path.exists(f"{tmp}/gathered.rank0.pt")
    m2, e2 = make()
    extra = checkpoint.load(f"{tmp}/gathered.pt", m2, e2)
    same_params = all(torch.equal(p, q) for p, q in zip(m1.parameters(), m2.parameters()))
    same_state = all(torch.equal(a.bucket.m, b.bucket.m) and torch.equal(a.bucket.v, b.bucket.v)
                     for a, b in zip(e1.buckets, e2.buckets))
    for x, y in data[6:]:
        loss = F.cross_entropy(m2(x), y)
        loss.backward()
    e2.synchronize()
    e2.check_status()
    drift = e2.replica_drift()
    e1.close(); e2.close()
    return {"single": single, "step": extra["global_step"], "same_params": same_params, "same_state": same_state,
            "drift": drift, "wrote": path is not None}


def test_gathered_checkpoint_of_partitioned_state(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs 2 GPUs")
    outs = _spawn(_worker_gathered_checkpoint, world, str(tmp_path))
    for r, o in enumerate(outs):
        assert o["single"] and o["step"] == 6 and o["same_params"] and o["same_state"], outs
        assert o["drift"] == 0.0 and o["wrote"] == (r == 0), outs


def _worker_grouped(rank, world, group_size, sparse):
    import torch.nn.functional as F

    from stellatrain_b200.control.shaper import BandwidthSchedule, TokenBucket
    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine

    model = _net()
    lr = 0.05
    cfg = EngineConfig(compressor="topk", ratio=0.9 if sparse else 0.0, optimizer="sgd", staleness=0 if not sparse else 1,
                       divide_k_by_world=sparse, bucket_mb=0.02, chunk_elems=1024, group_size=group_size,
                       optimizer_options={"lr": lr})
    eng = SparseDPEngine(model, cfg)
    if sparse:
        eng.set_link_shaper(TokenBucket(BandwidthSchedule(seed=3, lo_gbps=0.05, hi_gbps=0.2), burst_bytes=1 << 12))
    steps = 4
    for x, y in _data(rank, steps):
        F.cross_entropy(model(x), y).backward()
    eng.synchronize()
    eng.check_status()
    drift = eng.replica_drift()
    out = {"drift": drift, "owned": [sum(not s.skip for s in rt.bucket.layout.segments) for rt in eng.buckets],
           "shaped": getattr(eng, "shaped_bytes", 0)}
    if not sparse:
        # sum inside a group, mean over groups  ==  group_size * (mean over all ranks)
        ref = _net()
        opt = torch.optim.SGD(ref.parameters(), lr=lr * group_size)
        everyone = [_data(r, steps) for r in range(world)]
        for s in range(steps):
            opt.zero_grad()
            x = torch.cat([everyone[r][s][0] for r in range(world)])
            y = torch.cat([everyone[r][s][1] for r in range(world)])
            F.cross_entropy(ref(x), y).backward()
            opt.step()
        out["err"] = max(float((p.detach() - q.detach()).abs().max()) for p, q in zip(model.parameters(), ref.parameters()))
    eng.close()
    return out


@pytest.mark.parametrize("sparse", [False, True])
def test_grouped_mode(sparse):
    """Two groups of two ranks: dense reduction inside a group by tensor owners, sparse exchange between all."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    outs = _spawn(_worker_grouped, 4, 2, sparse)
    for o in outs:
        assert o["drift"] <= 1e-6, outs
        if not sparse:
            assert o["err"] < 1e-4, outs
        else:
            assert o["shaped"] > 0
    # ownership is a partition inside each group
    assert [a + b for a, b in zip(outs[0]["owned"], outs[1]["owned"])] == [a + b for a, b in zip(outs[2]["owned"], outs[3]["owned"])]


def _worker_link_probe(rank, world):
    from stellatrain_b200 import _build
    from stellatrain_b200.parallel import symm

    C = _build.load_extension("_C")
    dev = torch.device("cuda", rank)
    n = 1 << 24
    pool = symm.allocate(n * 4 + 4096, dev, None)
    dst = torch.empty(n, device=dev)
    out = torch.tensor([0, 2**63 - 1, 0], dtype=torch.int64, device=dev)
    ctr = torch.zeros(1, dtype=torch.int32, device=dev)
    peer = (rank + 1) % world
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        out.copy_(torch.tensor([0, 2**63 - 1, 0], dtype=torch.int64))
        C.link_probe(dst.data_ptr(), pool.peer_addr(peer, 0), n, out.data_ptr(), ctr.data_ptr(), s)
        torch.cuda.synchronize()
    ns = int(out[0])
    return {"gbps": n * 4 * 8 / ns, "backend": pool.backend}


def test_link_probe_measures_nvlink():
    outs = _spawn(_worker_link_probe, 2)
    for o in outs:
        assert 100.0 < o["gbps"] < 20000.0, outs      # a peer copy over NVLink: hundreds of GB/s


def _worker_missing_peer(rank, world):
    """Rank 1 leaves between steps (host-side decision); rank 0's next step must end with a timeout
    status instead of a hang.  Plain peer stores only (NVLS disabled by the environment)."""
    import torch.distributed as dist
    import torch.nn.functional as F

    from stellatrain_b200.parallel.engine import EngineConfig, SparseDPEngine
    from stellatrain_b200.parallel.gpu_bucket import SparseStepError

    model = _net()
    eng = SparseDPEngine(model, EngineConfig(compressor="topk", ratio=0.9, optimizer="sgd", staleness=0,
                                             bucket_mb=1.0, timeout_s=1.0, multicast=False))
    data = _data(rank, 3)
    for x, y in data[:2]:
        F.cross_entropy(model(x), y).backward()
    eng.synchronize()
    dist.barrier()
    outcome = "skipped"
    if rank != 1:
        x, y = data[2]
        F.cross_entropy(model(x), y).backward()
        try:
            eng.synchronize()
            outcome = "no error"
        except SparseStepError as e:
            outcome = f"status {e.code}"
    torch.cuda.synchronize()
    eng.close()
    return outcome


def test_missing_peer_times_out_cleanly():
    outs = _spawn(_worker_missing_peer, 2, env={"STELLATRAIN_NVLS": "0", "NCCL_NVLS_ENABLE": "0"})
    assert outs[1] == "skipped"
    assert outs[0] == "status 2", outs
