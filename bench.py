#!/usr/bin/env python
"""Headline benchmark: ResNet-152 sparse data-parallel training throughput (images/s) on N B200s.

Configuration (the reference's smoke workload shape, backend/test/test_end_to_end.py:21-52, at the
baseline's operating point): torchvision ResNet-152 with a 100-class head, fp32, batch 32 per GPU,
synthetic 3x224x224 N(0,1) images with uniform labels, threshold-v16 compression keeping 1 % of the
gradient entries with error feedback, sparse Adam lr 1e-3, bounded staleness 1, random-init weights.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints ONE JSON line.  ``value`` is device-timed (CUDA events, max over ranks) with inputs already
on the device; ``e2e`` is the same loop through the public API with, every step, the host-to-device copy
of the batch from pinned memory and a device-to-host read of the loss inside the timed region.
Other arms: ``--impl reference`` (the unmodified reference, built out of tree by ``baseline/build_reference.sh`` and
driven through its own API; prints an ``unavailable`` line with the cause when it cannot run), ``--impl nccl_sparse``
(same kernels, streams moved by ncclAllGather), ``--impl ddp`` (dense all-reduce + torch.optim.Adam),
``--impl dense_single`` / ``dense_graph`` (plain PyTorch on one GPU) and ``--impl cpu_offload`` (this package's CPU tier)
as baselines.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

REFERENCE_UNAVAILABLE = (
    "the reference is a CMake project without setup.py/pyproject.toml, so `pip install --target baseline/_ref "
    "<reference tree>` fails with \"Neither 'setup.py' nor 'pyproject.toml' found\"; "
    "baseline/build_reference.sh builds it with CMake instead"
)


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl_sparse", "ddp", "dense_single", "dense_graph", "cpu_offload"],
                    help="dense_graph: plain PyTorch step with capturable Adam/SGD captured in one CUDA graph (1 GPU), the "
                         "strongest dense baseline for the N = 1 point")
    ap.add_argument("--model", default="resnet152")
    ap.add_argument("--batch", type=int, default=32, help="per-GPU batch size")
    ap.add_argument("--num-classes", type=int, default=100)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--compressor", default="thresholdv16")
    ap.add_argument("--ratio", type=float, default=0.99, help="fraction of gradient entries dropped")
    ap.add_argument("--optimizer", default="adam")
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--staleness", type=int, default=1)
    ap.add_argument("--bucket-mb", type=float, default=64.0)
    ap.add_argument("--graph", type=int, default=1, help="capture the training step in a CUDA graph")
    ap.add_argument("--channels-last", type=int, default=1, help="NHWC memory format for vision models")
    ap.add_argument("--amp", default="none", choices=["none", "bf16"])
    ap.add_argument("--no-multicast", action="store_true")
    ap.add_argument("--grad-mode", default="steal", choices=["steal", "flat"])
    ap.add_argument("--momentum", type=float, default=0.0)
    ap.add_argument("--group-size", type=int, default=1, help="ranks per group (grouped two-level mode)")
    ap.add_argument("--state-partition", default="replicated", choices=["replicated", "owner"],
                    help="owner: optimiser state of every tensor on one rank, new values stored into all replicas")
    ap.add_argument("--shape-gbps", default=None, help="lo:hi[:seed] emulated cross-group link, e.g. 10:40:0")
    ap.add_argument("--shape-destinations", type=int, default=None,
                    help="charge every stream for this many ranks outside the own group (rehearsal of a shaped link on fewer GPUs)")
    ap.add_argument("--shape-share", type=float, default=None, help="this rank's share of the scheduled rate (default 1 / group size)")
    ap.add_argument("--controller", type=int, default=0, help="run the telemetry controller and apply its instructions")
    ap.add_argument("--adapt-batch", type=int, default=0, help="with --controller: also apply the per-GPU batch sizes it assigns")
    ap.add_argument("--slow-ranks-ms", type=float, default=0.0,
                    help="hold the upper half of the ranks for this long in every iteration (unequal GPUs for --adapt-batch)")
    ap.add_argument("--native-copies", type=int, default=1,
                    help="cpu_offload arm: 1 lets the native engine issue the device copies itself")
    ap.add_argument("--native-hooks", type=int, default=1, help="0: Python hooks instead of the native step engine (eager mode comparison)")
    ap.add_argument("--skip-e2e", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def arm_watchdog(seconds: float) -> None:
    """Hard limit for the whole run: dump every thread's stack and leave without running destructors,
    so that a stuck rank can never hold the GPUs until an outer limit kills the job."""
    import faulthandler
    import threading

    def fire() -> None:
        sys.stderr.write(f"[bench] watchdog: no result after {seconds:.0f}s, aborting\n")
        faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        sys.stderr.flush()
        os._exit(3)

    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()


def _exit_text(rc) -> str:
    """A child's return code in words: 'exit 0', 'signal SIGBUS', 'still running (killed at the limit)'."""
    import signal

    if rc is None:
        return "still running (killed at the limit)"
    if rc < 0:
        try:
            return f"signal {signal.Signals(-rc).name}"
        except ValueError:
            return f"signal {-rc}"
    return f"exit {rc}"


def _host_limits() -> str:
    """What the machine offers to a pipeline that lives in host memory: shared-memory file system, RAM, cores."""
    parts = []
    try:
        v = os.statvfs("/dev/shm")
        parts.append(f"/dev/shm {v.f_bavail * v.f_frsize >> 20} MiB free of {v.f_blocks * v.f_frsize >> 20} MiB")
    except OSError as e:
        parts.append(f"/dev/shm: {e}")
    try:
        with open("/proc/meminfo") as f:
            mem = {ln.split(":")[0]: ln.split()[1] for ln in f if ln.startswith(("MemTotal", "MemAvailable"))}
        parts.append(f"RAM {int(mem.get('MemAvailable', 0)) >> 10} MiB available of {int(mem.get('MemTotal', 0)) >> 10} MiB")
    except (OSError, ValueError):
        pass
    for path in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            with open(path) as f:
                parts.append(f"cgroup memory limit {f.read().strip()}")
            break
        except OSError:
            continue
    parts.append(f"{len(os.sched_getaffinity(0))} cores")
    return ", ".join(parts)


# Pinned pool the reference carves its tensors from: ONE chunk of 4 GiB that never grows
# (backend/src/engine/config.h:24, backend/src/engine/shm_manager.cpp:217-219, 330-370).
REFERENCE_POOL_BYTES = 4 << 30


def reference_pool_need(n_params: int, local_world: int) -> int:
    """Bytes the reference takes from its pool for one model: the master copy of every parameter
    (backend/src/engine/core.cpp:807-830) plus, per local GPU, two gradient slots of every tensor
    (backend/src/engine/core.cpp:963-1008), each start rounded up to 16 bytes."""
    return n_params * 4 * (1 + 2 * local_world) + 16 * 1024 * (1 + 2 * local_world)


def run_reference_arm(args: argparse.Namespace) -> None:
    """The unmodified reference, built out of tree into ``baseline/_ref`` (recipe in ``baseline/build_reference.sh``),
    driven through its own API by ``baseline/reference_arm.py``: one node, one process per GPU.  Local rank 0 is
    started first and the others only once its shared-memory pool exists, the order in which the reference's own
    driver brings its local ranks up (backend/test/test_end_to_end.py:160-163): a local rank that finds the metadata
    segment before rank 0 has filled it in reads a chunk count of zero and stops at
    backend/src/engine/shm_manager.cpp:186.  Any failure, a time-out included, ends in the ``unavailable`` line,
    which carries every rank's exit code or signal, the head and tail of its log, and the host's limits."""
    import glob
    import signal

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return                      # the other launcher ranks have nothing to do: rank 0 owns all local processes
    here = os.path.dirname(os.path.abspath(__file__))
    ref_dir = os.path.join(here, "baseline", "_ref")

    def unavailable(why: str) -> None:
        print(json.dumps({"impl": "reference", "n_gpus": world, "unavailable": " ".join(why.split())[:6000]}), flush=True)

    if not glob.glob(os.path.join(ref_dir, "fasterdp*.so")) or not os.path.exists(os.path.join(ref_dir, "model_wrapper.py")):
        unavailable(REFERENCE_UNAVAILABLE + "; no out-of-tree build under baseline/_ref either")
        return
    lm = args.model.startswith("gpt")
    if lm or args.amp != "none" or args.compressor not in ("thresholdv16", "thresholdv", "topk"):
        unavailable("the reference's driver path is torchvision models in fp32 with one of its compressors thresholdv16, "
                    "thresholdv, topk (backend/test/test_end_to_end.py:21-45, backend/src/engine/core.cpp:110-118); this "
                    "configuration is outside it")
        return
    try:
        import torch

        have = torch.cuda.device_count()
    except Exception as e:  # noqa: BLE001
        have = 0
        sys.stderr.write(f"[bench] torch: {e!r}\n")
    have = int(os.environ.get("REFERENCE_ARM_ASSUME_GPUS", have))    # tests of the launch and failure path on a CPU box
    if have < world:
        unavailable(f"{world} GPUs asked for, {have} visible")
        return
    # The pool is a file in /dev/shm that the reference sizes to 4 GiB without reserving it: where the file system is
    # smaller than what the run touches, the process that touches the first missing page dies of SIGBUS without a word.
    try:
        import torchvision

        n_params = sum(p.numel() for p in getattr(torchvision.models, args.model)(num_classes=args.num_classes).parameters())
    except Exception as e:  # noqa: BLE001
        unavailable(f"cannot size the model: {e!r}")
        return
    need = reference_pool_need(n_params, world)
    if need > REFERENCE_POOL_BYTES:
        unavailable(f"{args.model} on {world} local GPUs needs {need >> 20} MiB of the reference's pinned pool (one parameter "
                    f"copy and two gradient slots per GPU, backend/src/engine/core.cpp:807-830, 963-1008); the pool is one "
                    f"chunk of {REFERENCE_POOL_BYTES >> 20} MiB that never grows (backend/src/engine/config.h:24, "
                    f"backend/src/engine/shm_manager.cpp:217-219) and its allocator throws when it is full (shm_manager.cpp:355-367)")
        return
    vfs = os.statvfs("/dev/shm")
    shm_free = vfs.f_bavail * vfs.f_frsize
    if shm_free < need + (64 << 20) + (64 << 20):      # 64 MiB metadata segment (config.h:23) and some slack
        unavailable(f"{args.model} on {world} local GPUs touches {need >> 20} MiB of the reference's pool in /dev/shm "
                    f"(+64 MiB of metadata); this box: {_host_limits()}")
        return
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = ref_dir + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT", "MASTER_ADDR", "OMP_NUM_THREADS"):
        env.pop(k, None)            # the reference reads the first ones as NODE rank and NODE count; the launcher's
                                    # OMP_NUM_THREADS=1 would slow the ATen calls of its host pipeline
    sampler = ClockSampler(0)
    sampler.start()
    deadline = time.time() + float(os.environ.get("REFERENCE_ARM_TIMEOUT_S", "360"))
    straggler_s = float(os.environ.get("REFERENCE_ARM_STRAGGLER_S", "45"))
    max_attempts = int(os.environ.get("REFERENCE_ARM_ATTEMPTS", "3"))

    def attempt(no: int):
        """One run of all local ranks.  Returns (results, reason, per-rank text).  The reference has no time-outs of
        its own and its pipeline can lose a wake-up (it polls its barriers every 100 ms and re-broadcasts every 5 s for
        that reason, backend/src/engine/core.cpp:464-484, 1124-1128), so a rank can sit in ``synchronize`` for good
        after the others have finished: a rank that is still running ``straggler_s`` after the first one has
        reported ends the attempt."""
        session = os.getpid() * 8 + no
        port = int(os.environ.get("MASTER_PORT", "29500")) + 31 + no
        env_a = dict(env, WORLD_SIZE="1", RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs, logs = [], []

        def start(lr: int) -> None:
            log = open(os.path.join(here, "baseline", f".reference_arm_{lr}.log"), "w+")
            logs.append(log)
            procs.append(subprocess.Popen(
                [sys.executable, os.path.join(here, "baseline", "reference_arm.py"), "--ref-dir", ref_dir, "--local-rank", str(lr),
                 "--local-world", str(world), "--session", str(session), "--port", str(port), "--model", args.model,
                 "--batch", str(args.batch), "--num-classes", str(args.num_classes), "--ratio", str(args.ratio),
                 "--optimizer", args.optimizer, "--lr", str(args.lr), "--momentum", str(args.momentum), "--method", args.compressor,
                 "--steps", str(args.steps), "--warmup", str(max(3, args.warmup))],
                stdout=log, stderr=subprocess.STDOUT, env=env_a, start_new_session=True))

        def log_text(i: int) -> str:
            logs[i].flush()
            with open(logs[i].name) as f:
                return f.read()

        start(0)
        pool_file = f"/dev/shm/fasterdp-shm-data-{session}-0"
        master_up = False
        while time.time() < deadline and procs[0].poll() is None:
            if os.path.exists(pool_file) and "Starting SHM Master OK" in log_text(0):
                master_up = True
                break
            time.sleep(0.1)
        if master_up:
            for lr in range(1, world):
                start(lr)
        reason, first_done = "", None
        while master_up and any(p.poll() is None for p in procs):
            now = time.time()
            if now > deadline:
                reason = "timed out"
                break
            if any(p.poll() not in (None, 0) for p in procs):
                time.sleep(2.0)         # one rank failed: the others would wait for it forever
                reason = "a rank failed"
                break
            if first_done is None and any(p.poll() == 0 for p in procs):
                first_done = now
            if first_done is not None and now - first_done > straggler_s:
                reason = f"a rank was still running {straggler_s:.0f} s after another had finished"
                break
            time.sleep(0.2)
        if not master_up:
            reason = "local rank 0 did not bring its shared-memory pool up"
        codes = [p.poll() for p in procs]
        for p in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGKILL)      # exactly the process group this call started
                except ProcessLookupError:
                    pass
                p.wait()
        limits = _host_limits()         # before the pool's files go: what was left while the run had its pages
        for f in glob.glob(f"/dev/shm/fasterdp-shm-*-{session}*") + glob.glob(f"/dev/shm/sem.fasterdp-sem-{session}*"):
            try:
                os.unlink(f)
            except OSError:
                pass
        results, tails = [], []
        for i, log in enumerate(logs):
            log.seek(0)
            text = log.read()
            log.close()
            body = text if len(text) <= 1536 else text[:512] + " [...] " + text[-1024:]
            tails.append(f"[local rank {i}: {_exit_text(codes[i])}] {body}")
            for line in text.splitlines():
                if line.startswith("REFERENCE_ARM_RESULT "):
                    results.append(json.loads(line[len("REFERENCE_ARM_RESULT "):]))
        if len(results) == world:
            return results, "", ""
        return None, f"{reason or 'a rank ended without a result'}; {len(results)} of {world} processes finished; host: {limits}", " | ".join(tails)

    results, failures, detail = None, [], ""
    for no in range(max_attempts):
        if no and deadline - time.time() < 90:
            failures.append("no time left for another attempt")
            break
        results, why, detail_now = attempt(no)
        if results is not None:
            break
        failures.append(f"attempt {no + 1}: {why}")
        detail = detail_now
    clocks = sampler.stop()
    if results is None:
        unavailable(f"pool need {need >> 20} MiB; " + "; ".join(failures) + "; last attempt: " + detail)
        return
    ms = max(r["ms"] for r in results)
    per_step = ms / args.steps
    value = args.batch * world / (per_step / 1e3)
    h2d = args.batch * 3 * 224 * 224 * 4 + args.batch * 8
    out = {
        "metric": f"{args.model} training throughput, sparse data parallel ({args.compressor} keeping {(1 - args.ratio) * 100:g}% of "
                  f"gradient entries, error feedback, sparse {args.optimizer})",
        "impl": "reference", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (torch defaults: TF32 cuDNN convolutions)",
        "data": "synthetic N(0,1) images / uniform labels, random-init weights",
        "config": {"model": args.model, "global_batch": args.batch * world, "per_gpu_batch": args.batch, "seq_len": None,
                   "parallelism": f"dp{world}", "compressor": args.compressor, "kept_fraction": 1 - args.ratio,
                   "optimizer": args.optimizer, "lr": args.lr, "staleness": 1,
                   "transport": "reference: one node, pinned shared memory, CPU pipeline",
                   "build": "unmodified sources, CMake RelWithDebInfo, out of tree (baseline/build_reference.sh)",
                   "l2": "per-step working set exceeds the 126 MB L2; no flush needed"},
        "clocks": clocks,
        # the reference's loop copies every batch from pinned host memory itself; it reads no loss back
        "e2e": {"value": value, "unit": "images/s", "ms_per_step": per_step, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "final_loss": results[0]["loss"],
        # the reference can hang in its own synchronize; such an attempt is ended and the run repeated
        "attempts": len(failures) + 1, "failed_attempts": failures,
    }
    print(json.dumps(out), flush=True)


def main() -> None:
    args = parse_args()
    arm_watchdog(float(os.environ.get("BENCH_WATCHDOG_S", "420")))
    if args.impl == "reference":
        run_reference_arm(args)
        return

    # Libraries (NCCL's version banner, for one) write to the process's stdout; the contract is ONE JSON
    # line there, so everything but that line goes to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    import stellatrain_b200 as st
    from stellatrain_b200.models.registry import build_model, is_language_model, synthetic_batch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
        args.gpus = world
    master_addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    master_port = int(os.environ.get("MASTER_PORT", "29500"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    torch.manual_seed(1234)
    # the controller's batch sizes bring new input shapes at run time: no exhaustive search of convolution algorithms
    # for each of them (tens of seconds for ResNet-152, during which the other ranks' bounded waits run out)
    torch.backends.cudnn.benchmark = not args.adapt_batch

    lm = is_language_model(args.model)
    if args.impl == "cpu_offload":
        args.channels_last, args.graph = 0, 0      # the CPU tier reads and writes contiguous parameters, eagerly
    model = build_model(args.model, args.num_classes).to(dev)
    if args.channels_last and not lm:
        model = model.to(memory_format=torch.channels_last)
    n_params = sum(p.numel() for p in model.parameters())

    engine = None
    cpu_engine = None
    opt = None
    if args.impl == "cpu_offload":
        # The reference's own pipeline shape, built from this package's CPU tier: gradients leave the GPU into
        # pinned shared memory, are reduced, sparsified and applied by the sparse optimiser on the host, and the
        # parameters come back; one node, one process per GPU.
        from stellatrain_b200.cpu_tier import CpuOffloadEngine

        if world > 1:
            dist.init_process_group("nccl", init_method=f"tcp://{master_addr}:{master_port}", world_size=world,
                                    rank=rank, device_id=dev)
        session = (os.getppid() if world > 1 else os.getpid()) % 1000000 + 1000000
        need = int(n_params * 4 * (2 + 2 * world) * 1.25) + (72 << 20)
        vfs = os.statvfs("/dev/shm")
        if vfs.f_bavail * vfs.f_frsize < need + (256 << 20):
            if rank == 0:
                os.write(json_fd, (json.dumps({"impl": "cpu_offload", "unavailable":
                         f"/dev/shm has {vfs.f_bavail * vfs.f_frsize >> 20} MiB free, the pinned pool needs {need >> 20} MiB"}) + "\n").encode())
            return
        options = {"lr": args.lr}
        if args.optimizer == "sgd" and args.momentum:
            options["momentum"] = args.momentum
        cpu_engine = CpuOffloadEngine(model, master_addr=master_addr, master_port=master_port + 23, world_size=1, rank=0,
                                      session=session, local_world_size=world, local_rank=rank, method=args.compressor,
                                      staleness=args.staleness, ratio=args.ratio, optimizer=args.optimizer,
                                      optimizer_options=options, timeout_ms=120000,
                                      native_copies=bool(args.native_copies))
        net = model
    elif args.impl in ("ours", "nccl_sparse"):
        st.configure(master_addr, master_port, 1, 0, os.getpid(), world, rank, args.compressor, 1,
                     staleness=args.staleness, transport=("nccl" if args.impl == "nccl_sparse" else None))
        st.configure_compression_ratio(args.ratio)
        st.set_optimizer(args.optimizer)
        st.configure_optimizer("lr", args.lr)
        if args.optimizer == "sgd" and args.momentum:
            st.configure_optimizer("momentum", args.momentum)
        st.state().engine_cfg.group_size = args.group_size
        st.state().engine_cfg.state_partition = args.state_partition
        if args.controller:
            st.state().engine_cfg.min_ratio = min(args.ratio, 0.9)      # room for the controller to lower the ratio
        st.state().engine_cfg.bucket_mb = args.bucket_mb
        st.state().engine_cfg.multicast = not args.no_multicast
        st.state().engine_cfg.grad_mode = args.grad_mode
        st.state().engine_cfg.native_hooks = bool(args.native_hooks)
        if args.adapt_batch:
            # ranks capture their new batch shapes at different speeds: give the device-side waits room for it
            st.state().engine_cfg.timeout_s = 120.0
        if args.impl == "nccl_sparse":
            args.graph = 0            # the library collective between the kernel chains is not captured
        net = st.FasterDpModelWrapper(model, sequential=False, graph=bool(args.graph), graph_warmup=max(3, args.warmup - 2),
                                      autocast_dtype=(torch.bfloat16 if args.amp == "bf16" else None))
        net._ensure_engine()
        engine = net.engine
        if args.shape_gbps:
            from stellatrain_b200.control.shaper import BandwidthSchedule

            parts = args.shape_gbps.split(":")
            sched = BandwidthSchedule(seed=int(parts[2]) if len(parts) > 2 else 0, lo_gbps=float(parts[0]), hi_gbps=float(parts[1]))
            if args.shape_share is not None:
                from stellatrain_b200.control.shaper import DeviceTokenBucket

                sched = DeviceTokenBucket(sched, dev, share=args.shape_share)
            engine.set_link_shaper(sched, destinations=args.shape_destinations)   # token bucket on the device: works inside the captured step too
        if args.slow_ranks_ms > 0 and rank >= (world + 1) // 2:
            from stellatrain_b200 import _build

            hold = torch.tensor([int(args.slow_ranks_ms * 1e6)], dtype=torch.int64, device=dev)
            plain = net._loss_of

            def slowed(*inputs):
                _build.load_extension("_C").delay(hold.data_ptr(), 1_000_000_000, torch.cuda.current_stream().cuda_stream)
                return plain(*inputs)

            net._loss_of = slowed
    else:
        if world > 1:
            dist.init_process_group("nccl", init_method=f"tcp://{master_addr}:{master_port}", world_size=world,
                                    rank=rank, device_id=dev)
        net = model
        if args.impl == "ddp" and world > 1:
            net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], gradient_as_bucket_view=True)
        if args.impl == "dense_graph" and world > 1:
            raise SystemExit("--impl dense_graph is a single-GPU arm")
        opt = (torch.optim.Adam(model.parameters(), lr=args.lr, capturable=(args.impl == "dense_graph"))
               if args.optimizer == "adam" else torch.optim.SGD(model.parameters(), lr=args.lr, momentum=0.9))

    gen = torch.Generator().manual_seed(100 + rank)
    n_host = 4
    host_batches = []
    for _ in range(n_host):
        x, y = synthetic_batch(args.model, args.batch, args.num_classes, args.seq_len, generator=gen)
        host_batches.append((x.pin_memory(), y.pin_memory()))
    dev_x = host_batches[0][0].to(dev)
    dev_y = host_batches[0][1].to(dev)
    if args.channels_last and not lm:
        dev_x = dev_x.contiguous(memory_format=torch.channels_last)
    h2d_bytes = sum(t.numel() * t.element_size() for t in host_batches[0])
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    amp = torch.autocast("cuda", dtype=torch.bfloat16) if args.amp == "bf16" else None

    def fwd_bwd(x, y, marker=None):
        if amp is not None:
            with amp:
                loss = net(x, y)[1] if lm else F.cross_entropy(net(x), y)
        else:
            loss = net(x, y)[1] if lm else F.cross_entropy(net(x), y)
        if marker is not None:
            marker.backward_begins()
        loss.backward()
        return loss

    hook = None
    controller = None
    if args.controller and engine is not None:
        from stellatrain_b200.control.controller import Controller
        from stellatrain_b200.parallel.telemetry import TelemetryHook

        ctl_port = master_port + 17
        if rank == 0:
            controller = Controller(port=ctl_port, host="127.0.0.1", adapt=True,
                                    max_batch=(2 * args.batch if args.adapt_batch else args.batch)).start()
            from stellatrain_b200 import cpu_tier
            srv = cpu_tier._load().TelemetryServer(f"127.0.0.1:{ctl_port}", False, 5000)
            srv.send_global_telemetry(max(1, world // max(1, args.group_size)), world,
                                      [p.numel() for p in model.parameters()], False, False)
        if world > 1:
            dist.barrier()
        hook = TelemetryHook(engine, f"127.0.0.1:{ctl_port}", args.batch, apply_batch=bool(args.adapt_batch),
                             ratio_min_interval=(48 if args.graph else 0))
        if world > 1:
            # Nobody trains before everybody is registered.  The controller lives in rank 0's interpreter here: once
            # rank 0's first step has kernels waiting for a peer's stream, a call of its main thread that waits for
            # the device while it holds the interpreter lock keeps the controller from answering that very peer.
            dist.barrier()

    sparse_arm = engine is not None      # this package's engine: the wrapper owns the iteration (eager or captured)

    samples = [0]       # samples this rank really processed (the controller may change the per-GPU batch)

    def train_step(x, y):
        if sparse_arm:
            if hook is not None:
                if args.adapt_batch:
                    x, y = hook.resize_batch(x, y)
                samples[0] += x.shape[0]
                return hook.run(net, x, y)
            samples[0] += x.shape[0]
            return net.train_step(x, y)
        samples[0] += x.shape[0]
        loss = fwd_bwd(x, y)
        if opt is not None:
            opt.step()
            opt.zero_grad(set_to_none=False)
        return loss

    dense_graph, dense_loss = None, None
    if args.impl == "dense_graph":
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                train_step(dev_x, dev_y)
        torch.cuda.current_stream().wait_stream(side)
        dense_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(dense_graph):
            dense_loss = train_step(dev_x, dev_y)

    def run_step_device():
        if dense_graph is not None:
            dense_graph.replay()
            return dense_loss
        return train_step(dev_x, dev_y)

    # End to end, the way a user feeds the model: the package's PrefetchLoader copies batch i+1 from pinned host
    # memory on a side stream while step i runs; every step still has its own host-to-device copy and ends with
    # a device-to-host read of its loss.
    e2e_iter = None

    def run_step_e2e(i):
        x, y = next(e2e_iter)
        if dense_graph is not None:
            dev_x.copy_(x, non_blocking=True)
            dev_y.copy_(y, non_blocking=True)
            dense_graph.replay()
            loss = dense_loss
        else:
            loss = train_step(x, y)
        loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the step's result is read on the host
        return float(loss_host[0])

    def sync_all():
        if engine is not None:
            engine.synchronize()
        if cpu_engine is not None:
            cpu_engine.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        sampler = ClockSampler(local_rank)
        sampler.start()
        launches0 = engine.kernels_launched() if engine is not None else 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        if engine is not None:
            engine.synchronize()     # the last updates are part of the measured work
        if cpu_engine is not None:
            cpu_engine.synchronize()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            dist.barrier()
        launches = (engine.kernels_launched() - launches0) if engine is not None else 0
        return ms, clocks, launches

    for i in range(max(3, args.warmup)):
        run_step_device()
    if sparse_arm and net.graph:
        # the wrapper captures the iteration after its eager warm-up: make sure that lies before the timed region
        for i in range(8):
            if net._graphs:
                break
            run_step_device()
        if not net._graphs:
            sys.stderr.write("[bench] the step was not captured; running eagerly\n")
            args.graph = 0
    samples0 = samples[0]
    ms, clocks, launches = timed(lambda i: run_step_device(), args.steps)
    per_step = ms / args.steps
    unit_per_step = args.batch * world * (args.seq_len if lm else 1)
    if args.adapt_batch and world >= 1:
        # unequal, changing batches: count what was processed
        done = torch.tensor([float(samples[0] - samples0)], device=dev)
        if world > 1:
            dist.all_reduce(done)
        unit_per_step = float(done.item()) / args.steps * (args.seq_len if lm else 1)
    value = unit_per_step / (per_step / 1e3)

    e2e = None
    if not args.skip_e2e:
        from stellatrain_b200.utils.dataloader import PrefetchLoader

        e2e_warm = 3
        e2e_iter = iter(PrefetchLoader((host_batches[i % n_host] for i in range(e2e_warm + args.steps + 4)), dev, depth=2,
                                       channels_last=bool(args.channels_last and not lm)))
        for i in range(e2e_warm):
            run_step_e2e(i)
        ms2, clocks2, _ = timed(run_step_e2e, args.steps)
        e2e = {"value": unit_per_step / (ms2 / args.steps / 1e3), "unit": "tokens/s" if lm else "images/s",
               "ms_per_step": ms2 / args.steps, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4,
               "clocks": clocks2}

    final_loss = float(run_step_device().detach())
    if engine is not None:
        engine.synchronize()
        engine.check_status()
    if cpu_engine is not None:
        cpu_engine.synchronize()
        cpu_engine.close()

    # The sparse path inside the step, from the device-clock stamps that the kernels of the last step wrote themselves:
    # select + push and scatter + apply of every bucket, and the select chain against the memory roofline at the measured
    # copy bandwidth.  Bytes per element: the one-pass chain reads gradient and residual and writes the residual (12), the
    # two-pass chain reads the residual once more (16); 4 more where the consumed gradients are zeroed ("flat" gradient
    # mode).  In the step these kernels share the GPU with the backward pass, so the fraction is a lower bound of what the
    # kernels reach alone (profiles/ has those numbers).  Never allowed to break the result line.
    sparse_path = None
    if engine is not None:
        try:
            rows = engine.device_timeline()
            sel, app = sum(r["select_ms"] for r in rows), sum(r["apply_ms"] for r in rows)
            hbm_gbs, peaks_src = 6650.0, "fallback"
            peaks_file = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
            if os.path.exists(peaks_file):
                with open(peaks_file) as f:
                    hbm_gbs, peaks_src = float(json.load(f)["hbm_gbs"]), "measured"
            one_pass = all(getattr(rt.bucket, "last_select_fused", False) for rt in engine.buckets)
            per_elem = (12 if one_pass else 16) + (4 if engine.cfg.grad_mode == "flat" else 0)
            sparse_path = {"buckets": len(rows), "select_push_ms": sel, "scatter_apply_ms": app,
                           "share_of_step": (sel + app) / per_step if per_step > 0 else None,
                           "select_chain": "one-pass" if one_pass else "two-pass", "select_bytes_per_element": per_elem,
                           "select_bytes": per_elem * n_params,
                           "select_fraction_of_copy_bandwidth": (per_elem * n_params / (sel * 1e-3) / (hbm_gbs * 1e9)) if sel > 0 else None,
                           "copy_bandwidth_gbs": hbm_gbs, "of": peaks_src,
                           "nvlink_bytes_per_step": int(sum(rt.bucket.layout.wire_bytes() for rt in engine.buckets) * max(world - 1, 0))}
        except Exception as e:  # noqa: BLE001
            sparse_path = {"error": repr(e)}

    if rank == 0:
        out = {
            "metric": f"{args.model} training throughput, sparse data parallel ({args.compressor} keeping "
                      f"{(1 - args.ratio) * 100:g}% of gradient entries, error feedback, sparse {args.optimizer})",
            "impl": args.impl,
            "value": value, "unit": "tokens/s" if lm else "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 autocast" if args.amp == "bf16" else "fp32 (torch defaults: TF32 cuDNN convolutions)",
            "data": "synthetic N(0,1) images / uniform labels, random-init weights" if not lm
                    else "synthetic uniform token ids, random-init weights",
            "config": {
                "model": args.model, "params": n_params, "global_batch": args.batch * world,
                "per_gpu_batch": args.batch, "seq_len": args.seq_len if lm else None, "parallelism": f"dp{world}",
                "compressor": args.compressor, "kept_fraction": 1 - args.ratio, "optimizer": args.optimizer,
                "lr": args.lr, "staleness": args.staleness, "bucket_mb": args.bucket_mb,
                "transport": engine.transport if engine is not None else
                             ("pinned shared memory, host pipeline, copies by the " + ("native engine" if args.native_copies else "Python class")
                              if cpu_engine is not None else args.impl), "group_size": args.group_size,
                "state_partition": args.state_partition, "shaped_link_gbps": args.shape_gbps,
                "controller": ({"instructions_applied": len(hook.applied), "initial_ratio": args.ratio, "final_ratio": engine.cfg.ratio,
                                "ratio_trajectory": [(s_, r_) for s_, _b, r_ in hook.applied][-12:],
                                "final_batch": hook.batch_size} if hook is not None else None),
                "shaper": ({"gbps_achieved_this_rank": engine.shaper.achieved_gbps(),
                            "gbps_scheduled_mean_this_rank": engine.shaper.scheduled_mean_gbps(),
                            "ranks_sharing_the_link": engine.group_size, "waited_s": engine.shaper.stats()["waited_s"],
                            "bytes_per_step_this_rank": engine.shaped_bytes_per_step()}
                           if engine is not None and engine.shaper is not None else None),
                "multicast": bool(engine is not None and engine.pool is not None and engine.pool.mc_ptr),
                "native_step_engine": bool(engine is not None and engine.native is not None),
                "cuda_graph": bool(args.graph and net._graphs) if engine is not None else (args.impl == "dense_graph"), "channels_last": bool(args.channels_last), "grad_mode": args.grad_mode,
                "l2": "per-step working set (233 MB of parameters plus activations) exceeds the 126 MB L2; no flush needed",
            },
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": final_loss, "sparse_path": sparse_path,
        }
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(out) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:  # noqa: BLE001 - report, then leave without touching communicators again
        import traceback

        traceback.print_exc()
        sys.stderr.flush()
        sys.stdout.flush()
        os._exit(1)
