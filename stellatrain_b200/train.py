"""Training driver (role of the reference's backend/test/test_end_to_end.py:15-163).

    python -m stellatrain_b200.train --model resnet152 --dataset dummy --num-epochs 1 --batch-size 32 \
        --compression 0.99 --optim adam --lr 1e-3 --local-world-size 8

One process per local GPU is spawned (or ``--manual-spawn <local_rank>`` starts exactly one, e.g. under a
debugger).  Environment, as in the reference's launch scripts (test_script.sh:32-40): MASTER_ADDR,
MASTER_PORT, WORLD_SIZE (groups / nodes), RANK (group rank).  ``--tier cpu`` trains through the
CPU-offload tier instead of the GPU-resident engine.
"""
from __future__ import annotations

import argparse
import os
import time

import torch
import torch.multiprocessing as mp
import torch.nn.functional as F


def train_worker(local_rank: int, master_pid: int, local_world_size: int, args: argparse.Namespace) -> None:
    import stellatrain_b200 as st
    from stellatrain_b200.models.registry import build_model, is_language_model
    from stellatrain_b200.utils import dataloader as D
    from stellatrain_b200.utils.misc import AverageMeter

    master_addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    master_port = int(os.environ.get("MASTER_PORT", "5555"))
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    use_cuda = torch.cuda.is_available() and args.tier == "gpu"
    lm = is_language_model(args.model)
    model = build_model(args.model, args.num_classes)
    global_rank, global_world = rank * local_world_size + local_rank, world_size * local_world_size

    if args.tier == "gpu":
        st.configure(master_addr, master_port, world_size, rank, master_pid, local_world_size, local_rank,
                     args.compressor, args.gradient_accumulation, staleness=args.staleness)
        st.configure_compression_ratio(args.compression)
        st.state().engine_cfg.state_partition = args.state_partition
        st.state().engine_cfg.wire_format = args.wire_format
        st.set_optimizer(args.optim)
        # linear scaling rule of the reference driver (test_end_to_end.py:48-52)
        lr = args.lr / 256.0 * global_world * args.batch_size if args.scale_lr else args.lr
        st.configure_optimizer("lr", lr)
        if args.optim == "sgd":
            st.configure_optimizer("momentum", args.momentum)
        dev = torch.device("cuda", torch.cuda.current_device())
        model = model.to(dev)
        if args.channels_last and not lm:
            model = model.to(memory_format=torch.channels_last)
        net = st.FasterDpModelWrapper(model, sequential=not lm, graph=args.graph, graph_warmup=args.graph_warmup)
        sync, engine_of = st.synchronize, (lambda: net.engine)
    else:
        from stellatrain_b200.cpu_tier import CpuOffloadEngine

        dev = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
        model = model.to(dev)
        eng = CpuOffloadEngine(model, master_addr=master_addr, master_port=master_port, world_size=world_size, rank=rank,
                               session=master_pid, local_world_size=local_world_size, local_rank=local_rank,
                               method=args.compressor, gradient_accumulation=args.gradient_accumulation,
                               staleness=args.staleness, ratio=args.compression, optimizer=args.optim,
                               wire_blocks=not args.no_wire_blocks, wire_values=args.wire_values,
                               data_transport=args.data_transport, bundle_elems=args.bundle_elems,
                               optimizer_options={"lr": args.lr, **({"momentum": args.momentum} if args.optim == "sgd" else {})})
        net, sync, engine_of = model, eng.synchronize, (lambda: eng)

    builders = {"imagenet": (D.build_imagenet_dataloader, args.imagenet_root), "imagenet100": (D.build_imagenet100_dataloader, args.imagenet_root),
                "cifar100": (D.build_cifar100_dataloader, args.cifar100_root), "cifar10": (D.build_cifar10_dataloader, args.cifar10_root)}
    full_batch = args.batch_size * args.gradient_accumulation
    if args.dataset == "dummy":
        base = D.DummyTokenGenerator(full_batch, args.seq_len, length=args.dummy_length, seed=global_rank) if lm else \
            D.DummyInputGenerator(full_batch, length=args.dummy_length, num_class=args.num_classes, seed=global_rank)
    else:
        fn, root = builders[args.dataset]
        if args.loader == "subprocess":
            # the whole input pipeline in a child process (the reference's SuperFastDataLoader, util/dataloader.py:41-71)
            import functools

            base = D.SuperFastDataLoader(functools.partial(fn, root, full_batch, args.num_workers, world_size=global_world,
                                                           rank=global_rank), epochs=args.num_epochs)
        else:
            base = fn(root, full_batch, args.num_workers, world_size=global_world, rank=global_rank)
    hook = None
    if args.telemetry_uri and args.tier == "gpu":
        from stellatrain_b200.parallel.telemetry import TelemetryHook

        net._ensure_engine()
        # under captured iterations every applied ratio change costs an eager iteration and a new capture
        hook = TelemetryHook(net.engine, args.telemetry_uri, args.batch_size, ratio_min_interval=(48 if args.graph else 0))
    elif args.telemetry_uri:
        from stellatrain_b200.cpu_tier import CpuTierTelemetry

        hook = CpuTierTelemetry(eng, args.telemetry_uri, args.batch_size, gpu_id=global_rank, rank=rank, local_rank=local_rank)

    meter, global_step, t_start = AverageMeter(), 0, time.time()
    if args.resume and args.tier == "gpu":
        from stellatrain_b200.utils import checkpoint

        net._ensure_engine()
        extra = checkpoint.load(args.resume, net.module, net.engine, allow_world_change=args.allow_world_change)
        global_step = int(extra.get("global_step", 0))
        if global_rank == 0:
            print(f"resumed from {args.resume} at iteration {global_step}", flush=True)
    def save_cpu_tier(step: int) -> None:
        # optimiser state and thresholds live in each node's master process; one file per node
        sd = eng.state_dict()
        if local_rank == 0:
            sd["extra"] = {"global_step": step}
            target = args.checkpoint if world_size == 1 else f"{args.checkpoint}.node{rank}"
            torch.save(sd, target + ".tmp")
            os.replace(target + ".tmp", target)

    if args.resume and args.tier == "cpu":
        source = args.resume if world_size == 1 else f"{args.resume}.node{rank}"
        sd = torch.load(source, map_location="cpu", weights_only=False)
        eng.load_state_dict(sd)
        global_step = int(sd.get("extra", {}).get("global_step", 0))
        if global_rank == 0:
            print(f"resumed from {args.resume} at iteration {global_step}", flush=True)
    monitor = None
    if args.heartbeat and global_world > 1:
        import datetime

        from torch.distributed import TCPStore

        from stellatrain_b200.parallel.heartbeat import HeartbeatMonitor

        store = TCPStore(master_addr, master_port + 7, global_world, is_master=(global_rank == 0),
                         timeout=datetime.timedelta(seconds=60), wait_for_workers=False)
        monitor = HeartbeatMonitor(store, global_rank, global_world, interval_s=args.heartbeat / 4.0, timeout_s=args.heartbeat)
    for epoch in range(args.num_epochs):
        loader = st.StellaTrainDataLoader(D.PrefetchLoader(base, dev if dev.type == "cuda" else None,
                                                           channels_last=args.channels_last and not lm),
                                          gradient_accumulation=args.gradient_accumulation)
        for idx, (data, target) in enumerate(loader):
            if args.num_iters is not None and global_step >= args.num_iters:
                break
            if dev.type != "cuda":
                pass
            if hook is not None:
                data, target = hook.resize_batch(data, target)
            if args.tier == "gpu" and args.graph and args.gradient_accumulation == 1:
                # the wrapper owns the whole iteration: eager at first, then captured once and replayed
                loss = hook.run(net, data, target) if hook is not None else net.train_step(data, target)
            else:
                ctx = hook.step() if hook is not None else None
                marker = ctx.__enter__() if ctx is not None else None
                loss = net(data, target)[1] if lm else F.cross_entropy(net(data), target)
                if marker is not None:
                    marker.backward_begins()
                loss.backward()
                if ctx is not None:
                    ctx.__exit__(None, None, None)
            if loader.is_eoi:
                global_step += 1
                if monitor is not None:
                    # between steps, before kernels that would wait for a missing peer are launched; a lost
                    # peer ends this job with PeerLostError, the survivors restart from the last checkpoint
                    # with --resume --allow-world-change
                    monitor.check()
                if args.checkpoint and args.checkpoint_every and args.tier == "gpu" and global_step % args.checkpoint_every == 0:
                    from stellatrain_b200.utils import checkpoint

                    checkpoint.save(args.checkpoint, net.module, net.engine, {"global_step": global_step})
                if args.checkpoint and args.checkpoint_every and args.tier == "cpu" and global_step % args.checkpoint_every == 0:
                    save_cpu_tier(global_step)
                if global_step % args.log_every == 0:
                    meter.update(float(loss.detach()))
                    if global_rank == 0:
                        rate = global_step * args.batch_size * args.gradient_accumulation * global_world / (time.time() - t_start)
                        print(f"epoch {epoch} step {global_step} loss {meter.val:.4f} ({rate:.0f} samples/s)", flush=True)
        if args.tier == "gpu":
            net.step()
    if hasattr(base, "close"):
        base.close()       # a loader in a child process: this process cannot exit while that child lives
    sync()
    if args.checkpoint and args.tier == "gpu":
        from stellatrain_b200.utils import checkpoint

        checkpoint.save(args.checkpoint, net.module, net.engine, {"global_step": global_step})
    if args.checkpoint and args.tier == "cpu":
        save_cpu_tier(global_step)
    if monitor is not None:
        monitor.announce_leave()
    if global_rank == 0:
        print(f"done: {global_step} iterations in {time.time() - t_start:.1f} s", flush=True)
    if args.tier == "gpu":
        st.barrier()


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    p.add_argument("--model", default="resnet18")
    p.add_argument("--optim", default="sgd", choices=["sgd", "adam"])
    p.add_argument("--num-classes", type=int, default=100)
    p.add_argument("--num-iters", type=int, default=None)
    p.add_argument("--batch-size", type=int, default=72, help="per-device batch size")
    p.add_argument("--num-epochs", type=int, default=100)
    p.add_argument("--compression", type=float, default=0.95, help="fraction of gradient entries dropped")
    p.add_argument("--compressor", default="thresholdv16", choices=["thresholdv16", "thresholdv", "topk", "randomk"])
    p.add_argument("--staleness", type=int, default=1, choices=[0, 1])
    p.add_argument("--tier", default="gpu", choices=["gpu", "cpu"])
    p.add_argument("--manual-spawn", type=int, default=None)
    p.add_argument("--local-world-size", type=int, default=max(1, torch.cuda.device_count()))
    p.add_argument("--local-master-pid", type=int, default=os.getpid())
    p.add_argument("--lr", type=float, default=0.00625)
    p.add_argument("--scale-lr", action="store_true", help="lr / 256 * world * batch, as the reference driver does")
    p.add_argument("--momentum", type=float, default=0.9)
    p.add_argument("--imagenet-root", default="/datasets/imagenet")
    p.add_argument("--cifar100-root", default="/datasets/cifar100")
    p.add_argument("--cifar10-root", default="/datasets/cifar10")
    p.add_argument("--dataset", default="imagenet100", choices=["imagenet", "imagenet100", "cifar100", "cifar10", "dummy"])
    p.add_argument("--dummy-length", type=int, default=128)
    p.add_argument("--seq-len", type=int, default=1024)
    p.add_argument("--num-workers", type=int, default=8)
    p.add_argument("--gradient-accumulation", type=int, default=1)
    p.add_argument("--channels-last", action="store_true")
    p.add_argument("--graph", action="store_true",
                   help="GPU tier: capture the iteration in a CUDA graph after --graph-warmup eager iterations and replay it")
    p.add_argument("--graph-warmup", type=int, default=3)
    p.add_argument("--telemetry-uri", default=None,
                   help="controller address: host:port or tcp://host:port (this package's frames), zmq://host:port (the "
                        "reference's protobuf messages over ZeroMQ, e.g. its own batch_rate_alloc.py)")
    p.add_argument("--checkpoint", default=None, help="written at the end and every --checkpoint-every iterations")
    p.add_argument("--checkpoint-every", type=int, default=0)
    p.add_argument("--resume", default=None, help="checkpoint to start from")
    p.add_argument("--allow-world-change", action="store_true", help="resume on a different number of ranks")
    p.add_argument("--heartbeat", type=float, default=0.0, help="seconds of silence after which a rank counts as lost (0: off)")
    p.add_argument("--state-partition", default="replicated", choices=["replicated", "owner"])
    p.add_argument("--loader", default="inline", choices=["inline", "subprocess"],
                   help="real datasets: build and run the DataLoader in this process or in a child process")
    p.add_argument("--wire-format", default="wide", choices=["wide", "narrow"])
    p.add_argument("--wire-values", default="fp32", choices=["fp32", "fp16", "bf16"],
                   help="CPU tier: value type of the messages between nodes (the rounding error stays in the residual)")
    p.add_argument("--no-wire-blocks", action="store_true",
                   help="CPU tier: send (index, value) pairs even where 16 aligned indices could travel as one block id")
    p.add_argument("--data-transport", default="tcp", choices=["tcp", "zmq"],
                   help="CPU tier: the gradient ring between nodes over framed TCP or over ZeroMQ PUSH/PULL sockets")
    p.add_argument("--bundle-elems", type=int, default=1 << 16,
                   help="CPU tier: tensors below this many elements share one task per bundle of about that size; 0 gives "
                        "one task per tensor, as in the reference")
    p.add_argument("--log-every", type=int, default=10)
    return p


def main() -> None:
    args = build_parser().parse_args()
    if args.dataset == "imagenet":
        args.num_classes = 1000
    elif args.dataset == "cifar10":
        args.num_classes = 10
    print(f"per-device batch size is {args.batch_size}", flush=True)
    if args.manual_spawn is not None:
        train_worker(args.manual_spawn, args.local_master_pid, args.local_world_size, args)
    else:
        mp.spawn(train_worker, args=(os.getpid(), args.local_world_size, args), nprocs=args.local_world_size, join=True)


if __name__ == "__main__":
    main()
