"""Data loaders of the training driver (role of the reference's util/dataloader.py:11-218).

* ``FastDataLoader``: a ``DataLoader`` whose worker processes survive across epochs (repeat sampler).
* ``PrefetchLoader``: produces batches in a background thread and copies them to the device from pinned
  memory on a side stream, so that the host-to-device copy of batch i+1 overlaps step i.
* ``SuperFastDataLoader``: runs a whole loader in a child process and hands batches over through shared
  memory (util/dataloader.py:41-71), for pipelines whose Python-side decoding would otherwise compete
  with the training loop for the interpreter lock; wrap it in a ``PrefetchLoader`` for the device copy.
* ``DummyInputGenerator``: one fixed random batch repeated ``length`` times (images N(0,1), labels uniform).
* builders for ImageNet, ImageNet-100, CIFAR-10/100 and dummy data with a ``DistributedSampler``.
"""
from __future__ import annotations

import queue
import threading
from typing import Callable, Iterator, Optional

import torch
from torch.utils.data import DataLoader, DistributedSampler


class _RepeatSampler:
    def __init__(self, sampler) -> None:
        self.sampler = sampler

    def __iter__(self):
        while True:
            yield from iter(self.sampler)


class FastDataLoader(DataLoader):
    """Keeps one iterator (and its workers) alive for the life of the loader."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        object.__setattr__(self, "batch_sampler", _RepeatSampler(self.batch_sampler))
        self._iterator = super().__iter__()

    def __len__(self) -> int:
        return len(self.batch_sampler.sampler)

    def __iter__(self) -> Iterator:
        for _ in range(len(self)):
            yield next(self._iterator)


class PrefetchLoader:
    def __init__(self, loader, device: Optional[torch.device] = None, depth: int = 2,
                 channels_last: bool = False) -> None:
        self.loader, self.device, self.depth, self.channels_last = loader, device, depth, channels_last

    def __len__(self) -> int:
        return len(self.loader)

    def _to_device(self, obj, stream):
        if isinstance(obj, torch.Tensor):
            if self.device is None or self.device.type != "cuda":
                return obj
            src = obj if obj.is_pinned() else obj.pin_memory()
            with torch.cuda.stream(stream):
                out = src.to(self.device, non_blocking=True)
                if self.channels_last and out.dim() == 4:
                    out = out.contiguous(memory_format=torch.channels_last)
            return out
        if isinstance(obj, (list, tuple)):
            return type(obj)(self._to_device(o, stream) for o in obj)
        return obj

    def __iter__(self) -> Iterator:
        q: "queue.Queue" = queue.Queue(maxsize=self.depth)
        stream = torch.cuda.Stream(self.device) if (self.device is not None and self.device.type == "cuda") else None
        done = object()

        def produce() -> None:
            try:
                for batch in self.loader:
                    moved = self._to_device(batch, stream)
                    ev = None
                    if stream is not None:
                        ev = torch.cuda.Event()
                        ev.record(stream)
                    q.put((moved, ev))
            except Exception as e:  # noqa: BLE001 - surfaced in the consumer
                q.put((e, None))
            q.put((done, None))

        t = threading.Thread(target=produce, daemon=True, name="PrefetchLoader")
        t.start()
        while True:
            item, ev = q.get()
            if item is done:
                break
            if isinstance(item, Exception):
                raise item
            if ev is not None:
                cur = torch.cuda.current_stream(self.device)
                cur.wait_event(ev)
                self._record_stream(item, cur)     # allocated on the copy stream, used on this one
            yield item

    def _record_stream(self, obj, stream) -> None:
        if isinstance(obj, torch.Tensor):
            if obj.is_cuda:
                obj.record_stream(stream)
        elif isinstance(obj, (list, tuple)):
            for o in obj:
                self._record_stream(o, stream)


def _loader_process(factory: Callable, out, stop, epochs: int, parent_pid: int) -> None:
    """Body of the child process of ``SuperFastDataLoader``."""
    import os

    torch.set_num_threads(1)
    try:
        loader = factory()
        out.put(("len", len(loader) if hasattr(loader, "__len__") else -1))
        for _ in range(epochs):
            for batch in loader:
                if stop.is_set():
                    return
                out.put(("batch", batch))
            out.put(("end", None))
    except Exception as e:  # noqa: BLE001 - reported to the parent
        out.put(("error", f"{type(e).__name__}: {e}"))
    # tensors travel as file descriptors that the parent fetches from this process when it unpickles a batch:
    # stay until the parent says it is done (or is gone: this process is not a daemon, its loader may have workers)
    while not stop.wait(timeout=1.0):
        if os.getppid() != parent_pid:
            return


class SuperFastDataLoader:
    """A loader that lives in a child process.

    ``factory`` is a picklable callable that builds the loader inside the child (a loader with worker processes
    cannot be pickled once it runs).  The child is not a daemon, because a loader inside it needs worker processes of
    its own; ``close()`` ends it, and a finalizer does the same when this process exits.  Batches come back through a bounded queue; tensors travel in shared memory,
    so the parent does not copy them.  ``len()`` is the child's loader length.  Every wait has a limit: a child that
    dies or stalls raises ``RuntimeError`` in the parent instead of blocking the training loop forever.
    """

    def __init__(self, factory: Callable, depth: int = 4, epochs: int = 1 << 30, timeout_s: float = 300.0,
                 start_method: str = "spawn") -> None:
        import torch.multiprocessing as tmp

        ctx = tmp.get_context(start_method)
        self._q = ctx.Queue(maxsize=depth)
        self._stop = ctx.Event()
        self._timeout = timeout_s
        import multiprocessing.util as mp_util
        import os

        # not a daemon: a DataLoader inside the child needs worker processes of its own
        self._proc = ctx.Process(target=_loader_process, args=(factory, self._q, self._stop, epochs, os.getpid()),
                                 daemon=False, name="SuperFastDataLoader")
        self._proc.start()
        # runs when this process ends, before multiprocessing waits for its non-daemonic children, also in a process
        # that multiprocessing itself started (those skip atexit handlers)
        self._finalizer = mp_util.Finalize(self, SuperFastDataLoader._shutdown, args=(self._proc, self._q, self._stop),
                                           exitpriority=20)
        kind, value = self._get(max(timeout_s, 120.0))     # starting an interpreter and importing torch takes a while
        if kind == "error":
            self.close()
            raise RuntimeError(f"the loader process failed to start: {value}")
        self._len = int(value)

    def _get(self, limit: Optional[float] = None):
        waited, limit = 0.0, (self._timeout if limit is None else limit)
        while True:
            try:
                return self._q.get(timeout=0.5)
            except queue.Empty:
                waited += 0.5
                if not self._proc.is_alive() and self._q.empty():
                    raise RuntimeError("the loader process exited") from None
                if waited >= limit:
                    raise RuntimeError(f"no batch from the loader process within {limit:.0f} s") from None

    def __len__(self) -> int:
        if self._len < 0:
            raise TypeError("the wrapped loader has no length")
        return self._len

    def __iter__(self) -> Iterator:
        while True:
            kind, value = self._get()
            if kind == "end":
                return
            if kind == "error":
                raise RuntimeError(f"the loader process failed: {value}")
            yield value

    @staticmethod
    def _shutdown(proc, q, stop) -> None:
        if not proc.is_alive():
            return
        stop.set()
        try:
            while True:                      # unblock a child that waits for room in the queue
                q.get_nowait()
        except (queue.Empty, OSError, ValueError):
            pass
        proc.join(timeout=5)
        if proc.is_alive():
            proc.terminate()                 # this exact child, by handle
            proc.join(timeout=5)

    def close(self) -> None:
        self._finalizer()                    # runs _shutdown once



class DummyInputGenerator:
    """``length`` copies of one random batch (util/dataloader.py:74-86 uses soft labels of shape
    (B, classes); ``soft_labels`` selects that form, hard labels are the default here)."""

    def __init__(self, batch_size: int, length: int = 128, input_shape: int = 224, num_class: int = 100,
                 device: str = "cpu", soft_labels: bool = False, seed: int = 0) -> None:
        g = torch.Generator().manual_seed(seed)
        self.x = torch.randn(batch_size, 3, input_shape, input_shape, generator=g)
        self.y = torch.rand(batch_size, num_class, generator=g) if soft_labels else \
            torch.randint(0, num_class, (batch_size,), generator=g)
        if device != "cpu":
            self.x, self.y = self.x.to(device), self.y.to(device)
        else:
            self.x, self.y = self.x.pin_memory() if torch.cuda.is_available() else self.x, self.y
        self.length = length

    def __len__(self) -> int:
        return self.length

    def __iter__(self):
        for _ in range(self.length):
            yield self.x, self.y


class DummyTokenGenerator:
    """Token ids uniform over the vocabulary with next-token targets, one fixed batch repeated."""

    def __init__(self, batch_size: int, seq_len: int = 1024, vocab: int = 50257, length: int = 128, seed: int = 0) -> None:
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, vocab, (batch_size, seq_len + 1), generator=g)
        self.x, self.y, self.length = ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), length

    def __len__(self) -> int:
        return self.length

    def __iter__(self):
        for _ in range(self.length):
            yield self.x, self.y


def get_sampler(dataset, world_size: Optional[int], rank: Optional[int], shuffle: bool = True):
    if world_size is None or world_size <= 1:
        return None
    return DistributedSampler(dataset, num_replicas=world_size, rank=rank, shuffle=shuffle)


_dataset_cache: dict = {}


def _loader(dataset, batch_size, num_workers, pin_memory, split, collate_fn, world_size, rank, worker_init_fn):
    sampler = get_sampler(dataset, world_size, rank, shuffle=(split == "train"))
    return FastDataLoader(dataset, batch_size=batch_size, shuffle=(sampler is None and split == "train"), sampler=sampler,
                          num_workers=num_workers, pin_memory=pin_memory, drop_last=(split == "train"),
                          collate_fn=collate_fn, worker_init_fn=worker_init_fn,
                          persistent_workers=num_workers > 0)


def _imagenet_transform(split: str):
    import torchvision.transforms as T

    norm = T.Normalize(mean=[0.485, 0.456, 0.406], std=[0.229, 0.224, 0.225])
    if split == "train":
        return T.Compose([T.RandomResizedCrop(224), T.RandomHorizontalFlip(), T.ToTensor(), norm])
    return T.Compose([T.Resize(256), T.CenterCrop(224), T.ToTensor(), norm])


def build_imagenet_dataloader(imagenet_dir, batch_size, num_workers, pin_memory=True, split="train", collate_fn=None,
                              world_size=None, rank=None, worker_init_fn=None):
    from torchvision.datasets import ImageFolder

    key = ("imagenet", imagenet_dir, split)
    if key not in _dataset_cache:
        _dataset_cache[key] = ImageFolder(f"{imagenet_dir}/{split}", _imagenet_transform(split))
    return _loader(_dataset_cache[key], batch_size, num_workers, pin_memory, split, collate_fn, world_size, rank, worker_init_fn)


def build_imagenet100_dataloader(imagenet_dir, batch_size, num_workers, pin_memory=True, split="train", collate_fn=None,
                                 world_size=None, rank=None, worker_init_fn=None):
    from .datasets import ImageNet100

    key = ("imagenet100", imagenet_dir, split)
    if key not in _dataset_cache:
        _dataset_cache[key] = ImageNet100(imagenet_dir, split, _imagenet_transform(split))
    return _loader(_dataset_cache[key], batch_size, num_workers, pin_memory, split, collate_fn, world_size, rank, worker_init_fn)


def _cifar_transform(split: str, mean, std):
    import torchvision.transforms as T

    norm = T.Normalize(mean, std)
    if split == "train":
        return T.Compose([T.RandomCrop(32, padding=4), T.RandomHorizontalFlip(), T.ToTensor(), norm])
    return T.Compose([T.ToTensor(), norm])


def build_cifar100_dataloader(cifar_dir, batch_size, num_workers, pin_memory=True, split="train", collate_fn=None,
                              world_size=None, rank=None, worker_init_fn=None):
    from torchvision.datasets import CIFAR100

    key = ("cifar100", cifar_dir, split)
    if key not in _dataset_cache:
        _dataset_cache[key] = CIFAR100(cifar_dir, train=(split == "train"), download=False,
                                       transform=_cifar_transform(split, (0.5071, 0.4865, 0.4409), (0.2673, 0.2564, 0.2762)))
    return _loader(_dataset_cache[key], batch_size, num_workers, pin_memory, split, collate_fn, world_size, rank, worker_init_fn)


def build_cifar10_dataloader(cifar_dir, batch_size, num_workers, pin_memory=True, split="train", collate_fn=None,
                             world_size=None, rank=None, worker_init_fn=None):
    from torchvision.datasets import CIFAR10

    key = ("cifar10", cifar_dir, split)
    if key not in _dataset_cache:
        _dataset_cache[key] = CIFAR10(cifar_dir, train=(split == "train"), download=False,
                                      transform=_cifar_transform(split, (0.4914, 0.4822, 0.4465), (0.2470, 0.2435, 0.2616)))
    return _loader(_dataset_cache[key], batch_size, num_workers, pin_memory, split, collate_fn, world_size, rank, worker_init_fn)


def build_dummy_dataloader(_root, batch_size, num_workers=0, pin_memory=True, num_classes=100, split="train",
                           collate_fn=None, world_size=None, rank=None, worker_init_fn=None, length: int = 128):
    return DummyInputGenerator(batch_size, length=length, num_class=num_classes, seed=rank or 0)
