"""Shared test helpers: tiny configs and a CPU multi-rank launcher (gloo)."""
import os
import socket
import traceback

import torch
import torch.multiprocessing as mp

from dawn_srw_b200.config import preset


def tiny_config(version="spatial-r1-v4.1", **over):
    cfg = preset("40M", model_version=version, d_model=64, n_layers=2, n_heads=4, d_route=16,
                 n_qk=40, n_v=56, n_know=120)
    cfg.model.vocab_size, cfg.model.max_seq_len = 500, 32
    cfg.model.dropout = cfg.model.router_dropout = 0.0
    t = cfg.training
    t.batch_size, t.log_interval, t.val_interval, t.checkpoint_interval = 4, 0, 0, 0
    cfg.data.synthetic, cfg.data.synthetic_sequences = True, 64
    for k, v in over.items():
        if hasattr(cfg.model, k):
            setattr(cfg.model, k, v)
        else:
            setattr(cfg.training, k, v)
    return cfg


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _plain(x):
    """Tensors -> numpy so results survive the child process exiting."""
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy()
    if isinstance(x, dict):
        return {k: _plain(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_plain(v) for v in x)
    return x


def _tensors(x):
    import numpy as np
    if isinstance(x, np.ndarray):
        return torch.from_numpy(x)
    if isinstance(x, dict):
        return {k: _tensors(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_tensors(v) for v in x)
    return x


def _entry(rank, world, port, fn, args, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        out = fn(rank, world, *args)
        q.put((rank, "ok", _plain(out)))
    except Exception:
        q.put((rank, "err", traceback.format_exc()))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_ranks(fn, world, *args, timeout=240):
    """Run ``fn(rank, world, *args)`` in ``world`` CPU processes; returns the
    per-rank results (ordered by rank) or raises with the failing traceback."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(world):
            rank, status, out = q.get(timeout=timeout)
            if status == "err":
                raise RuntimeError(f"rank {rank} failed:\n{out}")
            res[rank] = out
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
    return [_tensors(res[r]) for r in range(world)]
