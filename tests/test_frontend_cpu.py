"""Frontend pieces that need no GPU: model cutting, micro-batch loader, bucket planning, CPU-tier driver."""
import copy
import subprocess
import sys

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from stellatrain_b200.models import GPT, build_model, synthetic_batch, to_sequential
from stellatrain_b200.parallel import buckets as B
from stellatrain_b200.utils.loader import StellaTrainDataLoader, current_micro_step


@pytest.mark.parametrize("name", ["resnet18", "vgg11", "vit_b_32", "swin_t"])
def test_to_sequential_computes_the_same_function(name):
    torch.manual_seed(0)
    m = build_model(name, 10).eval()
    seq = to_sequential(m).eval()
    x = torch.randn(2, 3, 224, 224)
    with torch.no_grad():
        torch.testing.assert_close(seq(x), m(x), rtol=1e-5, atol=1e-5)
    assert {id(p) for p in seq.parameters()} == {id(p) for p in m.parameters()}


def test_gpt_sequential_and_loss():
    torch.manual_seed(0)
    m = GPT.from_name("gpt2-tiny").eval()
    seq = to_sequential(m).eval()
    x, y = synthetic_batch("gpt2-tiny", 3, seq_len=32)
    with torch.no_grad():
        logits, loss = m(x, y)
        l2, loss2 = seq((x, y))
    torch.testing.assert_close(l2, logits)
    torch.testing.assert_close(loss2, loss)
    assert abs(float(loss) - np.log(257)) < 0.5
    assert GPT.from_name("gpt2", vocab_size=50257).num_parameters() == pytest.approx(124.4e6, rel=0.01)
    with pytest.raises(NotImplementedError):
        to_sequential(nn.ModuleDict({"a": nn.Linear(2, 2)}))


def test_micro_batch_loader():
    data = [(torch.arange(8).view(8, 1), torch.arange(8), {"m": torch.ones(8, 2)}, "tag")] * 2
    loader = StellaTrainDataLoader(data, gradient_accumulation=4)
    seen = []
    for x, y, d, tag in loader:
        seen.append((current_micro_step(), x.shape[0], d["m"].shape[0], tag, loader.is_eoi))
    assert [s[0] for s in seen] == [0, 1, 2, 3] * 2 and all(s[1] == 2 and s[2] == 2 and s[3] == "tag" for s in seen)
    assert [s[4] for s in seen] == [False, False, False, True] * 2
    assert current_micro_step() == -1 and len(loader) == 8
    with pytest.raises(ValueError):
        list(StellaTrainDataLoader([(torch.zeros(3, 1),)], gradient_accumulation=4))


def test_bucket_planning_and_entry_rule():
    assert B.entries_for(1000, 0.99, 1) == 10 and B.entries_for(1000, 0.99, 8) == 1 and B.entries_for(50, 0.99, 8) == 1
    assert B.entries_for(0, 0.5, 1) == 0 and B.entries_for(1000, 0.0, 1) == 1000
    numels = [10, 5000, 17, 70000, 3]
    groups = B.plan_buckets(numels, 6000)
    assert [i for g in groups for i in g] == list(range(5)) and groups[0] == [0, 1, 2] and groups[1] == [3]
    lay = B.BucketLayout([str(i) for i in range(5)], numels, chunk_elems=4096)
    lay.set_ratio(0.9, 1)
    offs = [s.off for s in lay.segments]
    assert all(o % 16 == 0 for o in offs) and lay.n_total % 16 == 0
    chunks = lay.chunk_table()
    assert chunks["len"].sum() == lay.n_total and (chunks["len"] % 16 == 0).all() and chunks["len"].max() <= 4096
    segs = lay.seg_table()
    assert segs["k"].tolist() == [1, 500, 1, 7000, 1] and segs["out_off"].tolist() == [0, 1, 501, 502, 7502] and lay.cap == 7503
    covered = np.zeros(lay.n_total, bool)
    for c in chunks:
        assert not covered[c["start"]: c["start"] + c["len"]].any()
        covered[c["start"]: c["start"] + c["len"]] = True
        s = lay.segments[c["seg"]]
        assert s.off <= c["start"] and c["start"] + c["len"] <= s.off + s.n_pad
    assert covered.all()


def test_cpu_tier_trains_a_model_on_host_tensors():
    from stellatrain_b200.cpu_tier import CpuOffloadEngine

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 4))
    ref = copy.deepcopy(model)
    eng = CpuOffloadEngine(model, method="topk", ratio=1e-9, optimizer="sgd", optimizer_options={"lr": 0.1}, staleness=0,
                           data_bytes=8 << 20, workers=2)
    # ratio ~ 0 keeps (almost) everything: equals dense SGD up to the one entry per tensor it may drop
    opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    x, y = torch.randn(64, 16), torch.randint(0, 4, (64,))
    for _ in range(5):
        F.cross_entropy(model(x), y).backward()
        opt.zero_grad(); F.cross_entropy(ref(x), y).backward(); opt.step()
    eng.synchronize()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert (p - q).abs().max() < 5e-2
    assert "Total" in eng.stats_json()
    eng.close()


def test_train_driver_cpu_tier_end_to_end():
    out = subprocess.run([sys.executable, "-m", "stellatrain_b200.train", "--tier", "cpu", "--model", "resnet18", "--dataset", "dummy",
                          "--num-epochs", "1", "--dummy-length", "3", "--batch-size", "2", "--local-world-size", "1",
                          "--compression", "0.9", "--num-classes", "10", "--log-every", "1"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "done: 3 iterations" in out.stdout


def test_train_driver_cpu_tier_checkpoint_and_resume(tmp_path):
    ck = str(tmp_path / "cpu.pt")
    base = [sys.executable, "-m", "stellatrain_b200.train", "--tier", "cpu", "--model", "resnet18", "--dataset", "dummy",
            "--num-epochs", "1", "--dummy-length", "4", "--batch-size", "2", "--local-world-size", "1", "--compression", "0.9",
            "--num-classes", "10", "--log-every", "1", "--checkpoint", ck]
    out = subprocess.run(base + ["--num-iters", "2"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "done: 2 iterations" in out.stdout
    out = subprocess.run(base + ["--resume", ck, "--num-iters", "4"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "resumed from" in out.stdout and "at iteration 2" in out.stdout and "done: 4 iterations" in out.stdout


def test_train_driver_real_dataset_through_a_loader_process(tmp_path):
    """ImageNet-100 builder (class list next to the data), the loader in a child process, CPU tier."""
    np = pytest.importorskip("numpy")
    Image = pytest.importorskip("PIL.Image")
    classes = ["n01440764", "n01443537"]
    for c in classes + ["n09999999"]:                       # the third class is not on the list and must be ignored
        d = tmp_path / "train" / c
        d.mkdir(parents=True)
        for i in range(4):
            Image.fromarray((np.random.rand(40, 40, 3) * 255).astype("uint8")).save(d / f"{i}.jpg")
    (tmp_path / "imagenet100.txt").write_text("\n".join(classes) + "\n")
    out = subprocess.run([sys.executable, "-m", "stellatrain_b200.train", "--tier", "cpu", "--model", "resnet18", "--dataset",
                          "imagenet100", "--imagenet-root", str(tmp_path), "--num-epochs", "1", "--batch-size", "2",
                          "--local-world-size", "1", "--compression", "0.9", "--num-classes", "2", "--log-every", "1",
                          "--num-workers", "1", "--loader", "subprocess"], capture_output=True, text=True, timeout=400)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "done: 4 iterations" in out.stdout               # 8 listed images, batches of 2


def test_fasterdp_named_calls_drive_the_cpu_tier(tmp_path):
    """The reference's call sequence (configure, ratio, optimiser, wrapper, loader, backward, synchronize) with
    tier="cpu": the native host pipeline does the update."""
    script = tmp_path / "run.py"
    script.write_text("""
import os, torch, torchvision, torch.nn.functional as F
import stellatrain_b200 as fasterdp
fasterdp.configure("127.0.0.1", 5555, 1, 0, os.getpid(), 1, 0, "thresholdv16", 2, tier="cpu")
fasterdp.configure_compression_ratio(0.9)
fasterdp.set_optimizer("adam"); fasterdp.configure_optimizer("lr", 1e-2)
torch.manual_seed(0)
model = fasterdp.FasterDpModelWrapper(torchvision.models.resnet18(num_classes=10))
before = [p.detach().clone() for p in model.parameters()]
x, y = torch.randn(8, 3, 32, 32), torch.randint(0, 10, (8,))
losses = []
for _ in range(6):
    for xb, yb in fasterdp.StellaTrainDataLoader([(x, y)]):       # two micro-batches of four
        loss = F.cross_entropy(model(xb), yb); loss.backward(); losses.append(float(loss.detach()))
fasterdp.synchronize()
assert type(model.engine).__name__ == "CpuOffloadEngine"
assert any(not torch.equal(a, b.detach()) for a, b in zip(before, model.parameters()))
assert losses[-1] < losses[0], losses
assert model.step() is None or True
fasterdp.configure_compression_ratio(0.8)                          # reaches the running engine
assert abs(model.engine.engine.compression_ratio_at(10**6) - 0.8) < 1e-9
sd = model.engine.state_dict(); assert set(sd) == {"model", "optimizer", "sparsifier", "engine"}
fasterdp.detach()
print("ok", losses[0], losses[-1])
""")
    out = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=300,
                         env={**__import__("os").environ, "PYTHONPATH": str(__import__("pathlib").Path(__file__).resolve().parent.parent)})
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip().splitlines()[-1].startswith("ok")


def test_reference_arm_reports_unavailable():
    import json

    out = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--steps", "3", "--warmup", "3"],
                         capture_output=True, text=True, timeout=400)
    assert out.returncode == 0
    d = json.loads(out.stdout.strip().splitlines()[-1])
    # without a GPU (or without the out-of-tree build) the arm says why it cannot run; with both it reports a number
    assert d["impl"] == "reference" and ("unavailable" in d or d["value"] > 0)


def test_reference_arm_starts_local_rank_0_first_and_reports_every_rank():
    """Failure path of the arm on a box without GPUs: local rank 0 brings the pool up, only then the second rank
    starts; both fail at their first CUDA call and the line names each rank's exit and the host's limits."""
    import json
    import os
    from pathlib import Path

    import torch

    root = Path(__file__).resolve().parent.parent
    if torch.cuda.is_available() or not list((root / "baseline" / "_ref").glob("fasterdp*.so")):
        pytest.skip("needs the out-of-tree build of the reference and no GPU")
    env = {**os.environ, "WORLD_SIZE": "2", "RANK": "0", "REFERENCE_ARM_ASSUME_GPUS": "2", "REFERENCE_ARM_TIMEOUT_S": "120"}
    out = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300, cwd=root, env=env)
    assert out.returncode == 0
    d = json.loads(out.stdout.strip().splitlines()[-1])
    why = d["unavailable"]
    assert d["impl"] == "reference" and d["n_gpus"] == 2
    assert "Starting SHM Master OK" in why and "[local rank 0:" in why and "[local rank 1:" in why
    assert "/dev/shm" in why and "pool need" in why


def test_reference_pool_arithmetic():
    """ResNet-152 (58.3 M parameters): one master copy and two gradient slots per GPU fit the reference's 4 GiB chunk
    up to 8 local GPUs, and no further."""
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("bench_mod", Path(__file__).resolve().parent.parent / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    n = 58_348_708
    assert mod.reference_pool_need(n, 8) < mod.REFERENCE_POOL_BYTES < mod.reference_pool_need(n, 9)
    assert mod.reference_pool_need(n, 4) < 2.3e9


def test_merge_state_shards_reassembles_full_moments():
    import torch

    from stellatrain_b200.utils.checkpoint import merge_state_shards

    n = 64
    full_m, full_v = torch.arange(n, dtype=torch.float32), torch.arange(n, dtype=torch.float32) * 2
    ranges = [(0, 16), (16, 48), (48, 48), (48, 64)]
    sds = []
    for lo, hi in ranges:
        pad = max(hi - lo, 16)
        m, v = torch.zeros(pad), torch.zeros(pad)
        m[: hi - lo], v[: hi - lo] = full_m[lo:hi], full_v[lo:hi]
        sds.append({"param_names": [["w"]], "world": 4, "state_partition": "owner",
                    "buckets": [{"param": torch.ones(n), "m": m, "v": v, "state_range": (lo, hi), "stamp": torch.zeros(pad)}]})
    out = merge_state_shards(sds)
    b = out["buckets"][0]
    assert torch.equal(b["m"], full_m) and torch.equal(b["v"], full_v)
    assert b["state_range"] == (0, n) and out["state_partition"] == "replicated"


def test_package_entry_point_reports_build_state():
    out = subprocess.run([sys.executable, "-m", "stellatrain_b200"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    import json

    rep = json.loads(out.stdout)
    assert rep["extensions"]["_Ccpu"]["built"] and rep["cpu_simd"] in ("scalar", "avx2", "avx512")


def test_train_driver_two_local_ranks_with_heartbeat():
    """Two processes of one node share gradients and the master copy through shared memory; the heartbeat monitor
    runs between steps and every rank announces that it leaves at the end."""
    out = subprocess.run([sys.executable, "-m", "stellatrain_b200.train", "--tier", "cpu", "--model", "resnet18", "--dataset", "dummy",
                          "--num-epochs", "1", "--dummy-length", "3", "--batch-size", "2", "--local-world-size", "2",
                          "--compression", "0.9", "--num-classes", "10", "--log-every", "1", "--heartbeat", "5"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "done: 3 iterations" in out.stdout


def test_state_partition_and_narrow_wire_layout():
    """Layout rules of the partitioned optimiser state and of the narrow wire format (pure Python)."""
    import numpy as np

    from stellatrain_b200.parallel import buckets as B

    lay = B.BucketLayout(["a", "b", "c", "d", "e", "f"], [5000, 70000, 130, 40000, 16, 9000], chunk_elems=1024, narrow_wire=True)
    lay.set_ratio(0.9, 4)
    owners = lay.assign_state_owners(4)
    assert owners == sorted(owners) and set(owners) <= set(range(4))            # consecutive tensors, one range per rank
    ranges = [lay.state_range(r) for r in range(4)]
    assert ranges[0][0] == 0 and ranges[-1][1] == lay.n_total
    assert all(ranges[r][1] == ranges[r + 1][0] for r in range(3) if ranges[r + 1] != (0, 0))
    bounds = lay.owner_bounds(4)
    assert bounds[0] == 0 and bounds[-1] == lay.cap and bounds == sorted(bounds)
    for r in range(4):                                                           # entry ranges match the tensors owned
        assert bounds[r + 1] - bounds[r] == sum(s.k for s in lay.segments if s.owner == r)
    segs = lay.seg_table()
    assert [(int(x) >> 8) & 0xFF for x in segs["reserved"]] == owners
    assert [bool(int(x) & 2) for x in segs["reserved"]] == [True, False, True, True, True, True]   # 70000 elements stay wide
    assert lay.wire_bytes() == sum(s.k * (4 if s.n_pad < 65536 else 8) for s in lay.segments)
    wide = B.BucketLayout(["a"], [1000], chunk_elems=1024)
    wide.set_ratio(0.9, 1)
    assert wide.wire_bytes() == 8 * wide.cap and not any(int(x) & 2 for x in wide.seg_table()["reserved"])
    # more ranks than tensors: some ranks own nothing, the bounds still tile the stream
    few = B.BucketLayout(["a", "b"], [100000, 50], chunk_elems=1024)
    few.set_ratio(0.9, 4)
    few.assign_state_owners(4)
    assert [few.state_range(r) for r in range(4)].count((0, 0)) == 2 and few.owner_bounds(4)[-1] == few.cap
    assert isinstance(np.asarray(few.owner_bounds(4)), np.ndarray)


def test_cpu_tier_drops_nan_gradients():
    """A step whose gradients are NaN leaves parameters and residuals untouched (the NaN is dropped in the gather
    stage); training continues normally afterwards."""
    from stellatrain_b200.cpu_tier import CpuOffloadEngine

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 4))
    eng = CpuOffloadEngine(model, method="topk", ratio=0.5, optimizer="sgd", optimizer_options={"lr": 0.1}, staleness=0,
                           data_bytes=8 << 20, workers=2)
    x, y = torch.randn(32, 16), torch.randint(0, 4, (32,))
    before = [p.detach().clone() for p in model.parameters()]
    (F.cross_entropy(model(x), y) * float("nan")).backward()
    eng.synchronize()
    for p, q in zip(model.parameters(), before):
        assert torch.equal(p, q) and torch.isfinite(p).all()
    F.cross_entropy(model(x), y).backward()
    eng.synchronize()
    assert any(not torch.equal(p, q) for p, q in zip(model.parameters(), before))
    assert all(torch.isfinite(p).all() for p in model.parameters())
    eng.close()
