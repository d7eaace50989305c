"""One local rank of the reference arm of ``bench.py`` (``--impl reference``).

Runs the unmodified reference (kaist-ina/stellatrain, built out of tree into ``baseline/_ref``) through its own
public API, the way its driver does (backend/test/test_end_to_end.py:15-85): ``fasterdp.configure`` with the
``thresholdv16`` compressor (or another one it accepts), ``configure_compression_ratio``,
``FasterDpModelWrapper`` around the torchvision model, ``set_optimizer`` / ``configure_optimizer``, ``StellaTrainDataLoader`` around the batches, forward, cross entropy,
backward, and ``fasterdp.synchronize`` at the end.  Nothing of this package is imported here.

One node (``WORLD_SIZE=1``) with ``--local-world`` processes, one per GPU, which is the reference's single-machine
mode: gradients of the local GPUs are summed on the host, sparsified once, applied by its sparse optimiser on the host
and copied back.  Data: a fixed set of synthetic host batches in pinned memory, copied to the device every step.

Prints one JSON line: {"ms": device-timed milliseconds of the timed steps, "steps": K, "loss": last loss}.
"""
import argparse
import json
import os
import sys
import time


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-dir", required=True)
    ap.add_argument("--local-rank", type=int, required=True)
    ap.add_argument("--local-world", type=int, required=True)
    ap.add_argument("--session", type=int, required=True)
    ap.add_argument("--port", type=int, default=5555)
    ap.add_argument("--model", default="resnet152")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--num-classes", type=int, default=100)
    ap.add_argument("--ratio", type=float, default=0.99)
    ap.add_argument("--method", default="thresholdv16", help="compressor name given to fasterdp.configure")
    ap.add_argument("--optimizer", default="adam")
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--momentum", type=float, default=0.0)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()

    sys.path.insert(0, a.ref_dir)
    import torch
    import torch.nn.functional as F
    import torchvision

    import fasterdp                                            # the reference's binding
    from model_wrapper import FasterDpModelWrapper, StellaTrainDataLoader   # the reference's frontend

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    fasterdp.configure("127.0.0.1", a.port, 1, 0, a.session, a.local_world, a.local_rank, a.method, 1)
    torch.cuda.set_device(a.local_rank)
    fasterdp.configure_compression_ratio(a.ratio)

    torch.manual_seed(1234)
    model = getattr(torchvision.models, a.model)(num_classes=a.num_classes).to("cuda")
    model = FasterDpModelWrapper(model)
    model.train()
    model.to("cuda")
    fasterdp.set_optimizer(a.optimizer)
    fasterdp.configure_optimizer("lr", a.lr)
    if a.optimizer == "sgd":
        fasterdp.configure_optimizer("momentum", a.momentum)
        fasterdp.configure_optimizer("smart_momentum", False)

    gen = torch.Generator().manual_seed(100 + a.local_rank)
    host = [(torch.randn(a.batch, 3, 224, 224, generator=gen).pin_memory(),
             torch.randint(0, a.num_classes, (a.batch,), generator=gen).pin_memory()) for _ in range(4)]

    def batches(n):
        for i in range(n):
            yield host[i % len(host)]

    def run(n):
        loss = None
        loader = StellaTrainDataLoader(enumerate(batches(n)))
        for _idx, (data, target) in loader:
            data, target = data.cuda(non_blocking=True), target.cuda(non_blocking=True)
            loss = F.cross_entropy(model(data), target)
            loss.backward()
        return loss

    fasterdp.barrier()
    run(max(1, a.warmup))
    torch.cuda.synchronize()
    fasterdp.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    loss = run(a.steps)
    fasterdp.synchronize()                                     # the last updates are part of the measured work
    e1.record()
    torch.cuda.synchronize()
    out = {"ms": e0.elapsed_time(e1), "wall_ms": (time.time() - t0) * 1e3, "steps": a.steps,
           "loss": float(loss.detach().cpu()), "local_rank": a.local_rank}
    print("REFERENCE_ARM_RESULT " + json.dumps(out), flush=True)
    os._exit(0)                                                # the engine's threads do not stop by themselves


if __name__ == "__main__":
    main()
