"""Data utilities and helpers (counterparts of the reference's util/dataloader.py, util/datasets.py,
util/transforms.py, util/util.py) on the CPU."""
import json
from argparse import Namespace
from pathlib import Path

import pytest
import torch
import torch.nn as nn

from stellatrain_b200.utils import dataloader as D
from stellatrain_b200.utils import misc as U
from stellatrain_b200.utils.transforms import RandomCutmix, RandomMixup


def test_meters_accuracy_and_byte_accounting():
    m = U.AverageMeter()
    m.update(2.0, 3); m.update(4.0, 1)
    assert m.val == 4.0 and m.count == 4 and m.avg == pytest.approx(2.5)
    out = torch.tensor([[0.1, 0.7, 0.2], [0.8, 0.1, 0.1], [0.2, 0.3, 0.5], [0.3, 0.4, 0.3]])
    top1, top2 = U.accuracy(out, torch.tensor([1, 0, 1, 2]), (1, 2))
    assert float(top1) == pytest.approx(50.0) and float(top2) == pytest.approx(75.0)
    soft = torch.nn.functional.one_hot(torch.tensor([1, 0, 1, 2]), 3).float()
    assert float(U.accuracy(out, soft)[0]) == pytest.approx(50.0)          # soft labels are reduced to their argmax
    t = torch.zeros(10, 4)
    assert U.get_logical_bytes(t) == 160 and U.get_bytes([t, {"a": t[:5]}]) >= 160
    assert U.get_shape({"x": t, "y": [t[:2]]}) == {"x": (10, 4), "y": [(2, 4)]}


def test_run_directory_helpers(tmp_path):
    class Writer:
        log_dir = str(tmp_path / "run")

    script = tmp_path / "launch.sh"
    script.write_text("echo hi\n")
    U.copy_script_file(Writer(), str(script))
    U.log_current_config(Writer(), Namespace(lr=0.1, model="resnet18", path=Path("/x")))
    assert (tmp_path / "run" / "scripts" / "launch.sh").read_text() == "echo hi\n"
    cfg = json.loads((tmp_path / "run" / "config.json").read_text())
    assert cfg == {"lr": 0.1, "model": "resnet18", "path": "/x"} and (tmp_path / "run" / "cmdline.txt").exists()


def test_exponential_moving_average_follows_the_parameters():
    net = nn.Linear(3, 2)
    ema = U.ExponentialMovingAverage(net, decay=0.5)
    with torch.no_grad():
        start = net.weight.clone()
        net.weight.add_(1.0)
    ema.update_parameters(net)     # the first update copies
    with torch.no_grad():
        net.weight.add_(2.0)
    ema.update_parameters(net)
    assert torch.allclose(ema.module.weight, 0.5 * (start + 1.0) + 0.5 * (start + 3.0))


@pytest.mark.parametrize("cls", [RandomMixup, RandomCutmix])
def test_batch_mixes_keep_shapes_and_label_mass(cls):
    torch.manual_seed(0)
    x, y = torch.randn(8, 3, 16, 16), torch.randint(0, 5, (8,))
    same_x, same_y = cls(5, p=0.0)(x, y)
    assert torch.equal(same_x, x) and torch.equal(same_y.argmax(1), y)
    mx, my = cls(5, p=1.0, alpha=1.0)(x, y)
    assert mx.shape == x.shape and my.shape == (8, 5)
    assert torch.allclose(my.sum(1), torch.ones(8), atol=1e-6) and float(my.max()) <= 1.0
    assert not torch.equal(mx, x)
    with pytest.raises(TypeError):
        cls(5)(torch.zeros(8, 16), y)
    with pytest.raises(ValueError):
        cls(0)


def test_cutmix_pastes_a_box_and_weights_labels_by_area():
    torch.manual_seed(1)
    x = torch.arange(4.0).view(4, 1, 1, 1).expand(4, 1, 8, 8).contiguous()      # sample i is the constant i
    y = torch.arange(4)
    mx, my = RandomCutmix(4, p=1.0)(x, y)
    for i in range(4):
        other = (i - 1) % 4                                  # the batch is rolled by one
        frac_other = float((mx[i] == float(other)).float().mean())
        assert set(mx[i].unique().tolist()) <= {float(i), float(other)}
        assert float(my[i, other]) == pytest.approx(frac_other, abs=1e-6)
        assert float(my[i, i]) == pytest.approx(1.0 - frac_other, abs=1e-6)


def test_loaders_and_generators():
    ds = torch.utils.data.TensorDataset(torch.arange(20.0).view(20, 1), torch.arange(20))
    fast = D.FastDataLoader(ds, batch_size=5, num_workers=0, shuffle=False)
    for _ in range(2):                                       # the wrapped iterator survives epochs
        seen = torch.cat([yb for _, yb in fast])
        assert seen.tolist() == list(range(20)) and len(fast) == 4
    pre = D.PrefetchLoader(fast, device=None)
    assert sum(xb.shape[0] for xb, _ in pre) == 20 and len(pre) == 4
    gen = D.DummyInputGenerator(4, length=3, input_shape=32, num_class=7, seed=1)
    batches = list(gen)
    assert len(batches) == len(gen) == 3 and batches[0][0].shape == (4, 3, 32, 32) and int(batches[0][1].max()) < 7
    assert torch.equal(batches[0][0], batches[2][0])
    assert D.DummyInputGenerator(4, length=1, input_shape=8, num_class=7, soft_labels=True).y.shape == (4, 7)
    tok = D.DummyTokenGenerator(2, seq_len=16, vocab=50, length=2)
    x, y = next(iter(tok))
    assert x.shape == y.shape == (2, 16) and torch.equal(x[:, 1:], y[:, :-1])
    assert len(D.build_dummy_dataloader(None, 4, length=5, num_classes=3)) == 5
    sampler = D.get_sampler(ds, world_size=2, rank=1, shuffle=False)
    assert len(list(iter(sampler))) == 10


def test_imagenet100_keeps_only_listed_classes(tmp_path):
    PIL = pytest.importorskip("PIL.Image")
    from stellatrain_b200.utils.datasets import ImageNet100

    for wnid in ("n01", "n02", "n03"):
        d = tmp_path / "train" / wnid
        d.mkdir(parents=True)
        PIL.new("RGB", (8, 8), (10, 20, 30)).save(d / "a.png")
    (tmp_path / "imagenet100.txt").write_text("n01 tench\nn03 shark\n")
    ds = ImageNet100(str(tmp_path), "train")
    assert ds.classes == ["n01", "n03"] and len(ds) == 2
    (tmp_path / "imagenet100.txt").write_text("n99 nothing\n")
    with pytest.raises(FileNotFoundError):
        ImageNet100(str(tmp_path), "train")                  # none of the listed classes is present


def _small_loader():
    ds = torch.utils.data.TensorDataset(torch.arange(24, dtype=torch.float32).view(12, 2), torch.arange(12))
    return torch.utils.data.DataLoader(ds, batch_size=4)


def _broken_loader():
    raise OSError("no such dataset")


class _Stalls:
    def __len__(self):
        return 1

    def __iter__(self):
        import time

        time.sleep(60)
        yield None


def test_loader_in_a_child_process():
    sub = D.SuperFastDataLoader(_small_loader, depth=2, epochs=2)
    try:
        assert len(sub) == 3
        for _ in range(2):                                   # two epochs come from the same child
            got = list(sub)
            assert [b[1].tolist() for b in got] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11]]
            assert got[2][0].tolist() == [[16.0, 17.0], [18.0, 19.0], [20.0, 21.0], [22.0, 23.0]]
    finally:
        sub.close()
    assert not sub._proc.is_alive()
    with pytest.raises(RuntimeError, match="no such dataset"):
        D.SuperFastDataLoader(_broken_loader)
    stalled = D.SuperFastDataLoader(_Stalls, timeout_s=1.0)   # a child that never delivers: an error, not a hang
    try:
        with pytest.raises(RuntimeError, match="no batch"):
            next(iter(stalled))
    finally:
        stalled.close()
    assert not stalled._proc.is_alive()
