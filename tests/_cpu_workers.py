"""Worker entry points for multi-process tests of the CPU tier (importable for the spawn start method)."""
import ctypes
import os
import sys
import traceback

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SIZES = [1000, 37, 4096]


def synthetic_grad(node, local, step, pi, n):
    g = torch.Generator().manual_seed(1_000_003 * node + 10_007 * local + 101 * step + pi)
    return torch.randn(n, generator=g) * 1e-2


def engine_worker(q, port, session_base, world, node, local_world, local, steps, method, optimizer, staleness, mode):
    """mode: 'ok' | 'ok_bf16' (bf16 values on the wire) | 'ok_pairs' (no block ids on the wire) | 'ok_switch' (the compression ratio changes from iteration 3 on; the nodes learn
    of it at different steps) | 'ok_weights' (node 0 counts a quarter, node 1 three quarters in the merge) | 'ok_device' (the
    engine copies gradients and parameters itself, through the stand-in CUDA runtime) | 'ok_bundle' (the three tensors
    registered as one bundle, host gradients) | 'ok_bundle_device' (the bundle with the engine's own copies) | 'absent' (never
    configures) | 'drop' (node 1 drops its gradient sends) | 'die' (node 1 exits mid-run)"""
    try:
        from stellatrain_b200 import cpu_tier

        ext = cpu_tier._load()
        ext.set_log_level(3)
        if mode == "absent" and local == local_world - 1:
            q.put((node, local, "absent", None))
            return
        eng = ext.CpuEngine()
        wire = {"ok_bf16": (True, 2), "ok_pairs": (False, 0)}.get(mode)
        device = mode in ("ok_device", "ok_bundle_device")
        bundle = mode in ("ok_bundle", "ok_bundle_device")
        if device:
            ext.install_fake_cuda(1)
        if mode.startswith("ok") and mode not in ("ok_switch", "ok_weights"):
            mode = "ok"
        timeout_ms = 4000 if mode != "ok" else 30000
        eng.configure("127.0.0.1", port, world, node, session_base + node, local_world, local, method, 1, staleness,
                      0.9, 32 << 20, timeout_ms, 4, False, True, mode == "ok")
        if wire is not None:
            eng.configure_wire(*wire)
        eng.set_optimizer(optimizer)
        eng.configure_optimizer("lr", 0.1 if optimizer == "sgd" else 1e-2)
        if optimizer == "sgd":
            eng.configure_optimizer("momentum", 0.9)
        params = [torch.full((n,), 0.5 + node + local) for n in SIZES]   # only node 0 / local 0 values must survive
        if bundle:
            offsets, total = [], 0
            for n in SIZES:
                offsets.append(total)
                total += (n + 15) // 16 * 16
            init = torch.zeros(total)
            for p, off in zip(params, offsets):
                init[off:off + p.numel()] = p
            b = eng.pre_train_init(0, "bundle", total, 0, init.data_ptr())
            eng.set_param_members(b, [f"{pi}@p{pi}" for pi in range(len(SIZES))], offsets, list(SIZES),
                                  [] if device else [p.data_ptr() for p in params])
            if device:
                master = torch.frombuffer((ctypes.c_float * total).from_address(eng.master_param(b)), dtype=torch.float32)
                for p, off in zip(params, offsets):
                    p.copy_(master[off:off + p.numel()])
                eng.attach_device_members(b, [p.data_ptr() for p in params])
            idxs = [b]
        elif device:
            idxs = [eng.pre_train_init(pi, f"p{pi}", p.numel(), 0, p.data_ptr()) for pi, p in enumerate(params)]
            for pi, p in zip(idxs, params):
                p.copy_(torch.frombuffer((ctypes.c_float * p.numel()).from_address(eng.master_param(pi)),
                                         dtype=torch.float32))      # what a framework does after registration
                eng.attach_device_param(pi, p.data_ptr())
        else:
            idxs = [eng.pre_train_init(pi, f"p{pi}", p.numel(), p.data_ptr()) for pi, p in enumerate(params)]
        keep = []
        if mode == "drop" and node == 1:
            eng.drop_tx_containing("@")
        if mode == "ok_weights":
            eng.set_node_weights([0.25, 0.75])
            mode = "ok"
        switch = mode == "ok_switch"
        if switch:
            mode = "ok"
        for step in range(steps):
            if switch and step == 1 + node:
                eng.configure_compression_ratio_from(3, 0.5)
            if mode == "die" and node == 1 and step == 2:
                os._exit(0)
            for pi in idxs:
                eng.pre_forward_process(pi)
            if bundle:
                grads = [synthetic_grad(node, local, step, pi, SIZES[pi]) for pi in range(len(SIZES))]
                keep.append(grads)
                if device:
                    eng.post_backward_device_members(idxs[0], [g.data_ptr() for g in grads], 0)
                else:
                    for pi in reversed(range(len(SIZES))):
                        eng.post_backward_member(idxs[0], pi, grads[pi].data_ptr())
                continue
            for pi in reversed(idxs):
                g = synthetic_grad(node, local, step, pi, SIZES[pi])
                if device:
                    keep.append(g)
                    eng.post_backward_device(pi, g.data_ptr(), 0)
                else:
                    eng.post_backward_process(pi, g.data_ptr())
        eng.synchronize()
        drift = max(eng.force_model_sync(pi, True) for pi in idxs)
        stats = eng.stats_json(False)
        eng.barrier()
        q.put((node, local, "ok", {"params": [p.numpy().copy() for p in params], "drift": drift,
                                   "versions": [eng.model_version(pi) for pi in idxs] * (len(SIZES) if bundle else 1),
                                   "stats_len": len(stats),
                                   "tx_bytes": eng.comm_bytes()[0]}))
        del eng
    except Exception as e:  # noqa: BLE001
        q.put((node, local, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()[-600:]}"))
