"""The communication kernels on ONE GPU: several ranks' buffers live on the same
device and one launch plays one rank at a time.  Only kernels that never wait on
another launch are used this way (scatter stores, slab sums, the partitioned
optimizer's two phases, a world-of-one all-reduce); the flag-waiting paths with
real peers are in tests/test_gpu_multi.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cb():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dawn_srw_b200.ops import cuda_backend
    return cuda_backend


def test_scatter_gemm_and_slab_sum_emulating_three_ranks(cb):
    """Reduce-scatter of three ranks' partial products: every 'rank' runs the
    scatter GEMM into the same three receive buffers (slot = its rank, owner
    order rotated by rank), then each owner sums its slots."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    W, rows, N, K = 3, 256, 200, 136
    M = W * rows
    e, st = cb.ext(), cb.status_word(dev)
    for dt in (torch.float32, torch.bfloat16):
        recv = [torch.full((W * rows, N), float("nan"), device=dev, dtype=dt) for _ in range(W)]
        ptrs = [r.data_ptr() for r in recv]
        want = torch.zeros(M, N, device=dev)
        for rank in range(W):
            A = torch.randn(M, K, device=dev, generator=g).bfloat16()
            B = torch.randn(N, K, device=dev, generator=g).bfloat16()
            rs = torch.rand(M, device=dev, generator=g) + 0.5
            e.gemm_scatter(A, False, B, False, ptrs, rank, rows, N, dt == torch.bfloat16, 1.0, rs, st, None, [])
            want += (A.float() @ B.float().t()) * rs[:, None]
        for owner in range(W):
            assert not torch.isnan(recv[owner].float()).any()          # every slot row was written
            got = e.sum_slabs(recv[owner], W, False)
            ref = want[owner * rows:(owner + 1) * rows]
            rel = ((got - ref).norm() / ref.norm()).item()
            assert rel < (2e-5 if dt == torch.float32 else 4e-3), (dt, owner, rel)
    cb.check_status()


def test_partitioned_optimizer_kernels_emulating_two_ranks(cb):
    """zero_reduce + zero_adam_scatter with both replicas' flat buffers on one
    device, against replicated AdamW on the averaged gradient."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    W, n = 2, 4096 + 512
    sl = n // W
    e = cb.ext()
    p0 = torch.randn(n, device=dev, generator=g)
    params = [p0.clone() for _ in range(W)]
    grads = [torch.randn(n, device=dev, generator=g) for _ in range(W)]
    p_ptrs = torch.tensor([p.data_ptr() for p in params], dtype=torch.int64, device=dev)
    g_ptrs = torch.tensor([x.data_ptr() for x in grads], dtype=torch.int64, device=dev)
    ms = [torch.zeros(sl, device=dev) for _ in range(W)]
    vs = [torch.zeros(sl, device=dev) for _ in range(W)]
    sq = torch.zeros(1, device=dev)
    owns = []
    for rank in range(W):                                      # phase 1 on every rank
        own = torch.empty(sl, device=dev)
        e.zero_reduce(g_ptrs, W, rank * sl, sl, 1.0 / W, own, sq)
        owns.append(own)
    gmean = (grads[0] + grads[1]) / W
    assert torch.allclose(torch.cat(owns), gmean, atol=1e-6)
    assert abs(float(sq) - float(gmean.square().sum())) < 1e-2
    clip = torch.ones(1, device=dev)
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    for rank in range(W):                                      # phase 2 on every rank
        e.zero_adam_scatter(p_ptrs, W, rank, rank * sl, sl, owns[rank], ms[rank], vs[rank], clip,
                            lr, b1, b2, eps, wd, 1 - b1, 1 - b2)
    m = (1 - b1) * gmean
    v = (1 - b2) * gmean * gmean
    upd = (m / (1 - b1)) / ((v / (1 - b2)).sqrt() + eps) + wd * p0
    want = p0 - lr * upd
    for p in params:                                           # both replicas hold the full update
        assert torch.allclose(p, want, atol=2e-6)


def test_small_allreduce_world_of_one_and_its_timeout(cb):
    dev = torch.device("cuda")
    e, st = cb.ext(), cb.status_word(dev)
    st.zero_()
    cap = 8192
    stage = torch.zeros(2 * cap, device=dev)
    pads = torch.zeros(1024, dtype=torch.int32, device=dev)
    stage_dev = torch.tensor([stage.data_ptr()], dtype=torch.int64, device=dev)
    pads_dev = torch.tensor([pads.data_ptr()], dtype=torch.int64, device=dev)
    x = torch.arange(5000, device=dev, dtype=torch.float32)
    for epoch in (1, 2, 3):
        y = x.clone()
        e.small_allreduce(stage_dev, pads_dev, 0, 1, epoch, 512, y, y, cap, st, 0)
        assert torch.equal(y, x)                               # the sum over a world of one
    # a two-rank world whose peer never signals: bounded wait, status 3, context alive
    other = torch.zeros(2 * cap, device=dev)
    pads2 = torch.zeros(1024, dtype=torch.int32, device=dev)
    stage2 = torch.tensor([stage.data_ptr(), other.data_ptr()], dtype=torch.int64, device=dev)
    pads_pair = torch.tensor([pads.data_ptr(), pads2.data_ptr()], dtype=torch.int64, device=dev)
    y = x[:100].clone()
    e.small_allreduce(stage2, pads_pair, 0, 2, 7, 512, y, y, cap, st, 20_000_000)
    torch.cuda.synchronize()
    assert int(st.item()) == 3
    with pytest.raises(RuntimeError):
        cb.check_status()
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0
