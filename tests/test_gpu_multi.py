"""Kernels that talk over NVLink, on 2 GPUs of one box (skipped with fewer).
Child processes, NCCL only for set-up, NVLS off."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _spawn(fn, world, *args):
    import torch.multiprocessing as mp
    from helpers import free_port
    port = free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_child, args=(fn, r, world, port, q, args)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(world):
            r, status, val = q.get(timeout=300)
            if status != "ok":
                raise RuntimeError(f"rank {r} failed:\n{val}")
            out[r] = val
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.terminate()
    return [out[r] for r in range(world)]


def _child(fn, rank, world, port, q, args):
    import traceback
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    try:
        import torch.distributed as dist
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
        val = fn(rank, world, *args)
        torch.cuda.synchronize()
        dist.barrier()
        q.put((rank, "ok", val))
        dist.destroy_process_group()
    except Exception:
        q.put((rank, "err", traceback.format_exc()))


def _barrier_and_scatter(rank, world):
    import torch.distributed as dist
    from dawn_srw_b200.ops import cuda_backend as CB
    from dawn_srw_b200.parallel.symm import SymmWorkspace
    dev = torch.device("cuda", rank)
    ws = SymmWorkspace(None, dev)
    for _ in range(5):
        ws.barrier()
    torch.cuda.synchronize()
    CB.check_status()
    # fused GEMM -> reduce-scatter against NCCL reduce_scatter of the same products,
    # with fp32 and with bf16 receive slots (N = 520: ragged last column tile)
    rows, N, K = 256, 520, 384
    M = rows * world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    A = torch.randn(M, K, device=dev, generator=g).bfloat16()
    B = torch.randn(N, K, device=dev, generator=g).bfloat16()
    rs = torch.rand(M, device=dev, generator=g) + 0.5
    full = (A.float() @ B.float().t()) * rs[:, None]
    ref = torch.empty(rows, N, device=dev)
    dist.reduce_scatter_tensor(ref, full.contiguous())
    errs = []
    for name, dt, tol_scale in (("f32", torch.float32, 1.0), ("bf16", torch.bfloat16, 400.0)):
        buf = ws.alloc("rs_" + name, (world * rows, N), dt)
        buf.local.fill_(float("nan"))             # every element must be overwritten
        for it in range(2):                       # twice: buffers are reused across calls
            ws.barrier()
            CB.ext().gemm_scatter(A, False, B, False, buf.ptrs, rank, rows, N, dt == torch.bfloat16,
                                  1.0, rs, CB.status_word(dev), None, [])
            ws.barrier()                          # every rank's stores have landed
            got = CB.ext().sum_slabs(buf.local, world, False)
            torch.cuda.synchronize()
            errs.append(((got - ref).norm() / ref.norm()).item() / tol_scale)
    CB.check_status()
    return max(errs)


def test_peer_barrier_and_fused_gemm_reduce_scatter():
    _need(2)
    errs = _spawn(_barrier_and_scatter, 2)
    assert max(errs) < 1e-5, errs


def _fused_vs_nccl(rank, world, version, U_total):
    """One sequence+pool-sharded SRW op: in-kernel collectives vs NCCL collectives."""
    from dawn_srw_b200.ops import cuda_backend as CB
    from dawn_srw_b200.ops.backend import ParallelCtx
    from dawn_srw_b200.ops.gates import gate_spec_for
    from dawn_srw_b200.parallel.topology import PoolShard
    import torch.distributed as dist
    dev = torch.device("cuda", rank)
    spec = gate_spec_for(version)
    Tl, R, U, r, D = 512, 2, U_total, 64, 128
    g = torch.Generator(device=dev).manual_seed(7)             # same full tensors on every rank
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    nz = torch.nn.functional.normalize
    emb_f, read_f, write_f = nz(rn(U, r), dim=-1), nz(rn(U, D), dim=-1), nz(rn(U, D), dim=-1)
    x_f, h_f, off_f, w_f = rn(world * Tl, D), rn(world * Tl, R, r), rn(world * Tl, R) * 0.3 - 0.3, rn(world * Tl, R, D)
    sh = PoolShard(rank, world)
    lo, hi, padded = sh.slice_of(U)

    def local_pool(t):
        out = torch.zeros(padded, t.shape[1], device=dev)
        out[: hi - lo] = t[lo:hi]
        return out
    rows = slice(rank * Tl, (rank + 1) * Tl)
    pctx = ParallelCtx(shard_group=dist.group.WORLD, dp_group=None, n_total=U, n_valid=hi - lo,
                       seq_sharded=True)
    res = {}
    for name, fused in (("nccl", False), ("fused", True)):
        be = CB.CudaBackend(fused_comm=fused)
        ps = [t.clone().requires_grad_(True) for t in
              (local_pool(emb_f), local_pool(read_f), local_pool(write_f), x_f[rows], h_f[rows], off_f[rows])]
        sc = torch.tensor(1.7, device=dev, requires_grad=True)          # learnable pool scale
        pool = be.prepare_pool(ps[0], ps[1], ps[2], spec, pctx)
        out = be.srw(ps[3], ps[4], ps[5], pool, spec, pctx=pctx, want_diag=False, out_scale=sc)
        ((out.stacked() * w_f[rows]).sum() + 3.0 * out.lb).backward()
        torch.cuda.synchronize()
        res[name] = [out.stacked().detach(), out.lb.detach(), out.den.detach()] + \
            [p.grad.clone() for p in ps] + [sc.grad.clone()]
    CB.check_status()
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()
    names = ["out", "lb", "den", "demb", "dread", "dwrite", "dx", "dh", "doff", "dscale"]
    return {n: rel(a, b) for n, a, b in zip(names, res["fused"], res["nccl"])}


@pytest.mark.parametrize("version,units", [("spatial-r1-v4.0.1", 300), ("spatial-r1-v3.9.4", 300),
                                           ("spatial-r1-v4.0.1", 1301)])    # 1301: 256-wide kernels
def test_fused_all_gather_and_reduce_scatter_match_nccl_path(version, units):
    _need(2)
    outs = _spawn(_fused_vs_nccl, 2, version, units)
    for o in outs:
        for k, v in o.items():
            # same kernels and math; differences: fp32 (fused) vs bf16 (NCCL) partial sums
            # (dscale is one scalar summed with heavy cancellation)
            assert v < (0.25 if k == "dscale" else 2e-2), (k, v, o)


def _group_vs_oracle(rank, world, version, n_qk, n_v):
    """The Q/K + V group of an attention block, sequence- and pool-sharded over
    ``world`` GPUs through the kernels with fused collectives, against a
    single-process fp32 oracle (unsharded pools, all tokens) computed on every rank."""
    from dawn_srw_b200.ops import cuda_backend as CB
    from dawn_srw_b200.ops.backend import ParallelCtx, ReferenceBackend
    from dawn_srw_b200.ops.gates import gate_spec_for
    from dawn_srw_b200.parallel.topology import PoolShard
    import torch.distributed as dist
    dev = torch.device("cuda", rank)
    spec = gate_spec_for(version)
    Tl, r, D = 256, 64, 128
    T = world * Tl
    g = torch.Generator(device=dev).manual_seed(11)            # same full tensors on every rank
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    q = lambda t: t.bfloat16().float()
    nz = torch.nn.functional.normalize
    pools_f = {n: [q(nz(rn(U, r), dim=-1)), q(nz(rn(U, D), dim=-1)), q(nz(rn(U, D), dim=-1))]
               for n, U in (("qk", n_qk), ("v", n_v))}
    x_f = q(rn(T, D))
    h_f = {"qk": q(rn(T, 2, r)), "v": q(rn(T, 1, r))}
    off_f = {"qk": rn(T, 2) * 0.3 - 0.3, "v": rn(T, 1) * 0.3 - 0.3}
    w_f = {"qk": rn(T, 2, D), "v": rn(T, 1, D)}
    scale0 = {"qk": 1.7, "v": 0.6}
    rows = slice(rank * Tl, (rank + 1) * Tl)
    sh = PoolShard(rank, world)

    def local_rows(t, U):
        lo, hi, padded = sh.slice_of(U)
        out = torch.zeros(padded, t.shape[1], device=dev)
        out[: hi - lo] = t[lo:hi]
        return out, lo, hi
    # ---- sharded, on the kernels
    be = CB.CudaBackend(fused_comm=True)
    leaves, calls, slices = {}, [], {}
    for n, U in (("qk", n_qk), ("v", n_v)):
        loc = [local_rows(t, U) for t in pools_f[n]]
        lo, hi = loc[0][1], loc[0][2]
        slices[n] = (lo, hi)
        ps = [l[0].clone().requires_grad_(True) for l in loc]
        hh, oo = h_f[n][rows].clone().requires_grad_(True), off_f[n][rows].clone().requires_grad_(True)
        sc = torch.tensor(scale0[n], device=dev, requires_grad=True)
        pctx = ParallelCtx(shard_group=dist.group.WORLD, dp_group=None, n_total=U, n_valid=hi - lo,
                           seq_sharded=True)
        leaves[n] = ps + [hh, oo, sc]
        calls.append(dict(h=hh, tau_off=oo, pool=be.prepare_pool(ps[0], ps[1], ps[2], spec, pctx),
                          pctx=pctx, out_scale=sc))
    xs = x_f[rows].clone().requires_grad_(True)
    res = be.srw_group(xs, calls, spec, want_diag=False)
    loss = sum((rs.stacked() * w_f[n][rows]).sum() + 3.0 * rs.lb + 2.0 * rs.dead_penalty
               for n, rs in zip(("qk", "v"), res))
    loss.backward()
    torch.cuda.synchronize()
    CB.check_status()
    # ---- oracle: everything on one rank in fp32; the objective is the sum of the ranks' losses
    rb = ReferenceBackend(torch.float32)
    xo = x_f.clone().requires_grad_(True)
    oleaves, total = {}, 0.0
    for n in ("qk", "v"):
        ps = [t.clone().requires_grad_(True) for t in pools_f[n]]
        hh, oo = h_f[n].clone().requires_grad_(True), off_f[n].clone().requires_grad_(True)
        sc = torch.tensor(scale0[n], device=dev, requires_grad=True)
        oleaves[n] = ps + [hh, oo, sc]
        ro = rb.srw(xo, hh, oo, rb.prepare_pool(ps[0], ps[1], ps[2], spec, ParallelCtx()), spec,
                    pctx=ParallelCtx(), want_diag=False, out_scale=sc)
        total = total + (ro.stacked() * w_f[n]).sum() + world * (3.0 * ro.lb + 2.0 * ro.dead_penalty)
        oleaves[n].append(ro)
    total.backward()
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()
    out = {"dx": rel(xs.grad, xo.grad[rows])}
    for n, rs in zip(("qk", "v"), res):
        lo, hi = slices[n]
        ro = oleaves[n][-1]
        out[f"{n}.out"] = rel(rs.stacked(), ro.stacked()[rows])
        out[f"{n}.lb"] = abs(float(rs.lb) - float(ro.lb))
        out[f"{n}.den"] = rel(rs.den, ro.den[rows])
        for k, name in enumerate(("demb", "dread", "dwrite")):
            out[f"{n}.{name}"] = rel(leaves[n][k].grad[: hi - lo], oleaves[n][k].grad[lo:hi])
            out[f"{n}.{name}_pad"] = float(leaves[n][k].grad[hi - lo:].abs().max()) if \
                leaves[n][k].shape[0] > hi - lo else 0.0
        out[f"{n}.dh"] = rel(leaves[n][3].grad, oleaves[n][3].grad[rows])
        out[f"{n}.doff"] = rel(leaves[n][4].grad, oleaves[n][4].grad[rows])
        # the scale gradient is a sum over ALL tokens of the group: all-reduce the partial sums
        gs = leaves[n][5].grad.clone()
        dist.all_reduce(gs)
        terms = float((ro.stacked().abs() * w_f[n].abs()).sum() / scale0[n])
        out[f"{n}.dscale"] = abs(float(gs) - float(oleaves[n][5].grad)) / terms
    return out


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("version,n_qk,n_v", [
    ("spatial-r1-v4.0.1", 1580, 2600),      # 1580 is not a multiple of 8: padded shards
    ("spatial-r1-v4.0.1", 4100, 5000),      # every shard runs the 256-wide kernels up to 8 ranks
    ("spatial-r1-v3.9.4", 4100, 5000),
    ("spatial-r1-v4.1", 4100, 5000),        # dead-unit penalty on the fused path
    ("spatial-r1-v4.0.1+regs", 4100, 5000), # peers' rows copied through registers instead of bounce buffers
    ("spatial-r1-v4.0.1", 1030, 1100),      # 2 ranks: 520 padded rows each, the last rank holds 510 (< 512) units
])
def test_sharded_route_group_matches_single_process_fp32_oracle(world, version, n_qk, n_v, monkeypatch):
    _need(world)
    if version.endswith("+regs"):
        version = version[: -len("+regs")]
        monkeypatch.setenv("DSB_GATHER_REGS_MIN_UNITS", "1")      # the spawned ranks inherit it
        monkeypatch.setenv("DSB_SPREAD_GATHER_RANKS", "2")         # and every kernel of a group gathers its own rows
    outs = _spawn(_group_vs_oracle, world, version, n_qk, n_v)
    sharp = ("demb", "dh", "doff")     # flow through d(gate)/d(score): bf16 rounding moves scores across the kink
    for o in outs:
        for k, v in o.items():
            leaf = k.split(".")[-1]
            if leaf.endswith("_pad"):
                assert v == 0.0, (k, v)                      # padded unit rows receive no gradient
            elif leaf == "lb":
                assert v < 2e-3, (k, v, o)
            elif leaf == "dscale":
                assert v < 2e-3, (k, v, o)
            else:
                assert v < (0.08 if leaf in sharp else 2e-2), (k, v, o)


def test_peer_barrier_times_out_when_a_peer_never_arrives():
    """One GPU plays a two-rank world in which the other rank's flag is never
    written: the wait runs out, the status word reports it, the context lives."""
    _need(1)
    from dawn_srw_b200.ops import cuda_backend as CB
    dev = torch.device("cuda", 0)
    pad0 = torch.zeros(64, dtype=torch.int32, device=dev)
    pad1 = torch.zeros(64, dtype=torch.int32, device=dev)      # stands in for the absent peer's pad
    pads = torch.tensor([pad0.data_ptr(), pad1.data_ptr()], dtype=torch.int64, device=dev)
    st = CB.status_word(dev)
    st.zero_()
    CB.ext().peer_barrier(pads, 0, 2, 1, 0, st, 20_000_000)     # ~10 ms budget
    torch.cuda.synchronize()
    assert int(st.item()) == 3
    with pytest.raises(RuntimeError):
        CB.check_status()
    assert int(st.item()) == 0                                  # cleared; the GPU is still usable
    x = torch.ones(4, device=dev)
    assert float((x + 1).sum()) == 8.0


def _small_allreduce(rank, world):
    import torch.distributed as dist
    from dawn_srw_b200.ops import cuda_backend as CB
    from dawn_srw_b200.parallel.symm import SymmWorkspace
    dev = torch.device("cuda", rank)
    ws = SymmWorkspace(None, dev)
    ws.enable_small_allreduce()
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    errs = []
    for n in (1, 7, 256, 4096, 4097, 30000, 65536, 131072, 100001, 3, 9000):   # repeated calls reuse the two halves
        x = torch.randn(n, device=dev, generator=g)
        ref = x.clone()
        dist.all_reduce(ref)
        ws.all_reduce_small(x)
        errs.append(float((x - ref).abs().max()))
        # every rank holds bit-identical sums
        both = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(both, x)
        assert all(torch.equal(both[0], b) for b in both)
    torch.cuda.synchronize()
    CB.check_status()
    return max(errs)


def test_small_allreduce_kernel_matches_nccl():
    _need(2)
    errs = _spawn(_small_allreduce, 2)
    assert max(errs) < 1e-5, errs


def _zero_peer_vs_library(rank, world):
    """PartitionedAdamW with the peer-memory kernels against the same class on
    NCCL collectives and against replicated AdamW + all-reduce."""
    from dawn_srw_b200.ops import cuda_backend as CB
    from dawn_srw_b200.parallel.grad_sync import GradSync
    from dawn_srw_b200.parallel.topology import init_topology
    from dawn_srw_b200.parallel.zero import PartitionedAdamW
    from dawn_srw_b200.train.optimizer import DawnAdamW
    dev = torch.device("cuda", rank)
    topo = init_topology(pool_shards=1, seq_shard=False)
    shapes = {"router.proj_know.weight": (130, 70), "router.proj_know.bias": (70,),
              "neuron_pool.know_read": (1001, 33), "layers.0.norm1.weight": (70,),
              "token_emb.weight": (513, 70)}
    g0 = torch.Generator(device=dev).manual_seed(1)
    init = {n: torch.randn(*s, device=dev, generator=g0) for n, s in shapes.items()}
    sets = []
    for _ in range(3):
        sets.append([(n, torch.nn.Parameter(v.clone())) for n, v in init.items()])
    opts = [PartitionedAdamW(sets[0], topo, lr=1e-2, accumulation_steps=2, peer_kernels=True),
            PartitionedAdamW(sets[1], topo, lr=1e-2, accumulation_steps=2, peer_kernels=False),
            DawnAdamW(sets[2], lr=1e-2, accumulation_steps=2, grad_sync=GradSync(topo), fused=True)]
    gr = torch.Generator(device=dev).manual_seed(100 + rank)           # rank-specific gradients
    for step in range(6):
        grads = {n: torch.randn(*s, device=dev, generator=gr) * 3 for n, s in shapes.items()}
        for named, opt in zip(sets, opts):
            for n, p in named:
                if p.grad is None:
                    p.grad = grads[n].clone()
                else:
                    p.grad.add_(grads[n])
            opt.step()
            opt.zero_grad()
    torch.cuda.synchronize()
    CB.check_status()
    out = {"gn": [float(o.last_grad_norm) for o in opts], "count": [o.count for o in opts]}
    out["peer_vs_lib"] = max(float((a - b).abs().max()) for (_, a), (_, b) in zip(sets[0], sets[1]))
    out["peer_vs_replicated"] = max(float((a - b).abs().max()) for (_, a), (_, b) in zip(sets[0], sets[2]))
    out["params"] = torch.cat([p.detach().reshape(-1) for _, p in sets[0]]).cpu().numpy()
    return out


def test_partitioned_adamw_peer_kernels():
    _need(2)
    outs = _spawn(_zero_peer_vs_library, 2)
    for o in outs:
        assert o["count"] == [3, 3, 3]
        assert abs(o["gn"][0] - o["gn"][1]) < 1e-3 and abs(o["gn"][0] - o["gn"][2]) < 1e-3
        assert o["peer_vs_lib"] < 2e-6 and o["peer_vs_replicated"] < 2e-6, o
    import numpy as np
    assert np.array_equal(outs[0]["params"], outs[1]["params"])       # replicas stay identical
