import pytest
import torch

from dawn_srw_b200.ops.gates import GateSpec, gate_backward, gate_forward, gate_spec_for
from dawn_srw_b200.ops.srw_ref import prepare_pool_ref, srw_pool_ref

VERSIONS = ["spatial-r1-v3.9.4", "spatial-r1-v4.0.1", "spatial-r1-v4.1"]


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_manual_gate_backward_matches_autograd(kind):
    torch.manual_seed(kind)
    spec = GateSpec(kind=kind, sharpness=20.0)   # softer sigmoid keeps fp64 autograd comparable
    s = torch.randn(7, 2, 33, dtype=torch.float64, requires_grad=True)
    tau = (torch.randn(7, 2, 1, dtype=torch.float64) * 0.3).requires_grad_(True)
    sd = (torch.rand(7, 2, 1, dtype=torch.float64) + 0.5).requires_grad_(True)
    g, dterm, _ = gate_forward(spec, s, tau, sd)
    dg = torch.randn_like(g)
    dden = torch.randn(7, 2, 1, dtype=torch.float64)
    (g * dg).sum().add((dterm * dden).sum()).backward()
    ds, dtau, dsig_z = gate_backward(spec, s.detach(), tau.detach(), sd.detach(), dg, dden)
    assert torch.allclose(ds, s.grad, atol=1e-9)
    assert torch.allclose(dtau, tau.grad, atol=1e-9)
    if kind == 1:   # d sigma = sum(ds * -z) = dsig_z with z = (s - tau) / sigma
        assert torch.allclose(dsig_z, sd.grad, atol=1e-9)


def _inputs(T=12, R=2, U=50, r=8, D=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    return rn(T, D), rn(T, R, r), rn(T, R) * 0.3 - 0.3, rn(U, r), rn(U, D), rn(U, D)


@pytest.mark.parametrize("version", VERSIONS)
def test_chunked_equals_dense(version):
    spec = gate_spec_for(version)
    x, h, off, emb, read, write = _inputs()
    e, r_, w = prepare_pool_ref(emb, read, write, spec, torch.float32)
    a = srw_pool_ref(x, h, off, e, r_, w, spec)
    b = srw_pool_ref(x, h, off, e, r_, w, spec, chunk_size=7, use_checkpoint=True)
    assert torch.allclose(a.out, b.out, atol=1e-5)
    assert torch.allclose(a.lb, b.lb, atol=1e-6)
    for k in a.diag:
        assert torch.allclose(a.diag[k], b.diag[k], atol=1e-4), k


@pytest.mark.parametrize("version", VERSIONS)
def test_padding_rows_contribute_nothing(version):
    spec = gate_spec_for(version)
    x, h, off, emb, read, write = _inputs(U=37)
    e, r_, w = prepare_pool_ref(emb, read, write, spec, torch.float32)
    a = srw_pool_ref(x, h, off, e, r_, w, spec)
    pad = lambda t: torch.cat([t, torch.randn(11, t.shape[1])])
    b = srw_pool_ref(x, h, off, pad(e), pad(r_), pad(w), spec, n_valid=37, n_total=37)
    assert torch.allclose(a.out, b.out, atol=1e-6)
    assert torch.allclose(a.lb, b.lb) and torch.allclose(a.dead_penalty, b.dead_penalty)
    assert torch.allclose(a.diag["active_n_mean"], b.diag["active_n_mean"])


def test_paired_routes_equal_two_single_routes():
    spec = gate_spec_for("spatial-r1-v4.0.1")
    x, h, off, emb, read, write = _inputs()
    e, r_, w = prepare_pool_ref(emb, read, write, spec, torch.float32)
    both = srw_pool_ref(x, h, off, e, r_, w, spec, want_diag=False)
    for i in range(2):
        one = srw_pool_ref(x, h[:, i:i + 1], off[:, i:i + 1], e, r_, w, spec, want_diag=False)
        assert torch.allclose(both.out[:, i], one.out[:, 0], atol=1e-6)


def test_output_formula_v41():
    """out = ((g * xr) @ write) / max(sum intensity, 1)."""
    spec = gate_spec_for("spatial-r1-v4.1")
    x, h, off, emb, read, write = _inputs(R=1)
    res = srw_pool_ref(x, h, off, emb, read, write, spec, return_gates=True)
    s = h[:, 0] @ emb.t()
    mu, sd = s.mean(-1, keepdim=True), s.std(-1, unbiased=False, keepdim=True) + 1e-8
    m = s - (mu + off * sd) - 0.5
    act = torch.sigmoid(500 * m)
    inten = 1e-4 + (m - 0.01).clamp(0, 10)
    want = ((act * inten) * (x @ read.t())) @ write / inten.sum(-1, keepdim=True).clamp(min=1)
    assert torch.allclose(res.out[:, 0], want, atol=1e-5)
    assert torch.allclose(res.gates[:, 0], act * inten, atol=1e-6)


def test_unit_mask_zeroes_units():
    spec = gate_spec_for("spatial-r1-v4.0.1")
    x, h, off, emb, read, write = _inputs(R=1)
    e, r_, w = prepare_pool_ref(emb, read, write, spec, torch.float32)
    mask = torch.ones(50)
    mask[::2] = 0
    a = srw_pool_ref(x, h, off, e, r_, w, spec, unit_mask=mask, return_gates=True)
    assert float(a.gates[..., ::2].abs().max()) == 0.0


def test_dead_penalty_has_gradient():
    spec = gate_spec_for("spatial-r1-v4.1")
    x, h, off, emb, read, write = _inputs(R=1)
    emb = emb.clone().requires_grad_(True)
    res = srw_pool_ref(x, h, off + 5.0, emb, read, write, spec)   # tau far up: everything dead
    assert float(res.diag["dead_count"]) > 0
    res.dead_penalty.backward()
    assert emb.grad is not None and float(emb.grad.abs().sum()) > 0


@pytest.mark.parametrize("normalize", [False, True])
def test_gram_statistics_and_their_gradient(normalize):
    """mean_U(s) and mean_U(s^2) as quadratic forms in h (the CUDA backend's
    replacement for the first pass over all scores), and the gradient that
    reaches emb through the Gram matrix and the pool preparation."""
    from dawn_srw_b200.ops.backend import PreparedPool
    from dawn_srw_b200.ops.cuda_backend import _PoolPrepFn
    torch.manual_seed(1)
    U, r, D, T = 40, 8, 12, 9
    emb = torch.randn(U, r, requires_grad=True)
    read = torch.randn(U, D, requires_grad=True)
    write = torch.randn(U, D, requires_grad=True)
    h = torch.randn(T, r).bfloat16().float().requires_grad_(True)
    holder = PreparedPool(None, None, None)
    anchor, gram, esum = _PoolPrepFn.apply(emb, read, write, holder, normalize, U)
    mu = h @ (esum / U)
    m2 = ((h @ gram) * h).sum(-1) / U
    w1, w2 = torch.randn(T), torch.randn(T)
    # pool gradients that the SRW calls of a step would have accumulated
    acc = [torch.randn(U, r), torch.randn(U, D), torch.randn(U, D)]
    holder.g_emb += acc[0]; holder.g_read += acc[1]; holder.g_write += acc[2]
    ((mu * w1).sum() + (m2 * w2).sum() + anchor.sum() * 0).backward()
    got = [emb.grad.clone(), read.grad.clone(), write.grad.clone(), h.grad.clone()]

    # oracle: the same quantities straight from the scores, bf16 cast with a
    # straight-through gradient
    emb2, read2, write2 = (t.detach().clone().requires_grad_(True) for t in (emb, read, write))
    h2 = h.detach().clone().requires_grad_(True)

    def prep(w):
        n = w / (torch.linalg.vector_norm(w, dim=-1, keepdim=True) + 1e-8) if normalize else w
        return n + (n.bfloat16().float() - n).detach()
    e_c, r_c, w_c = prep(emb2), prep(read2), prep(write2)
    s = h2 @ e_c.t()
    loss = (s.mean(-1) * w1).sum() + ((s * s).mean(-1) * w2).sum()
    loss = loss + (e_c * acc[0]).sum() + (r_c * acc[1]).sum() + (w_c * acc[2]).sum()
    loss.backward()
    assert torch.allclose(mu, s.mean(-1), atol=1e-5) and torch.allclose(m2, (s * s).mean(-1), atol=1e-5)
    for a, b in zip(got, (emb2.grad, read2.grad, write2.grad, h2.grad)):
        assert torch.allclose(a, b, atol=2e-5), float((a - b).abs().max())


def test_out_scale_and_route_accessors():
    """``out_scale`` multiplies the route outputs inside the backend call and
    ``route(i)`` / ``stacked()`` agree whichever way a backend stores them."""
    from dawn_srw_b200.ops.backend import ParallelCtx, ReferenceBackend
    from dawn_srw_b200.ops.gates import gate_spec_for
    from dawn_srw_b200.ops.srw_ref import SRWResult
    torch.manual_seed(0)
    spec = gate_spec_for("spatial-r1-v4.0.1")
    be = ReferenceBackend(torch.float32)
    T, R, U, r, D = 12, 2, 40, 8, 16
    emb, read, write = torch.randn(U, r), torch.randn(U, D), torch.randn(U, D)
    x, h, off = torch.randn(T, D), torch.randn(T, R, r), torch.zeros(T, R)
    pool = be.prepare_pool(emb, read, write, spec, ParallelCtx())
    a = be.srw(x, h, off, pool, spec, want_diag=False)
    sc = torch.tensor(2.5, requires_grad=True)
    b = be.srw(x, h, off, pool, spec, want_diag=False, out_scale=sc)
    assert torch.allclose(b.out, a.out * 2.5)
    assert torch.equal(b.route(1), b.out[:, 1]) and torch.equal(b.stacked(), b.out)
    b.out.sum().backward()
    assert torch.allclose(sc.grad, a.out.sum())
    listed = SRWResult(out=None, lb=a.lb, dead_penalty=a.dead_penalty, outs=[a.out[:, 0], a.out[:, 1]])
    assert torch.equal(listed.route(0), a.out[:, 0]) and torch.equal(listed.stacked(), a.out)


def test_score_statistics_node_matches_autograd_of_the_plain_formula():
    """tau / 1/sigma / column sums from the Gram matrix, forward and all gradients,
    against autograd through explicit scores; a zero h row (router dropout, padded
    rows) must give finite gradients."""
    from dawn_srw_b200.ops.score_stats import score_stats
    torch.manual_seed(3)
    T, R, r, U = 37, 2, 16, 50
    emb = torch.nn.functional.normalize(torch.randn(U, r), dim=-1)
    h0 = torch.randn(T, R, r).bfloat16().float()
    h0[5, 1] = 0.0
    off0 = torch.randn(T, R) * 0.4
    wt, wi, wh, wb = torch.randn(T, R), torch.randn(T, R), torch.randn(r), torch.randn(T, R, r).bfloat16().float()

    def loss(tau, isd, hsum, hb):
        return (tau * wt).sum() + (isd * wi).sum() * 1e-2 + (hsum * wh).sum() + (hb.float() * wb).sum()
    # node under test
    h, off = h0.clone().requires_grad_(True), off0.clone().requires_grad_(True)
    ef = emb.clone().requires_grad_(True)
    gram, esum = ef.t() @ ef, ef.sum(0)
    loss(*score_stats(h, off, gram, esum, U)).backward()
    got = [h.grad.clone(), off.grad.clone(), ef.grad.clone()]
    # plain formula through the scores
    h2, off2, ef2 = h0.clone().requires_grad_(True), off0.clone().requires_grad_(True), emb.clone().requires_grad_(True)
    s = h2 @ ef2.t()                                                    # [T,R,U]
    mu = s.mean(-1)
    var = (s * s).mean(-1) - mu * mu
    sd = torch.sqrt(var.clamp_min(1e-12)) + 1e-8
    loss(mu + off2 * sd, 1.0 / sd, h2.sum(dim=(0, 1)), h2).backward()
    want = [h2.grad, off2.grad, ef2.grad]
    for name, a, b in zip(("dh", "doff", "demb"), got, want):
        assert torch.isfinite(a).all(), name
        # the zero row sits exactly at the variance floor, where the two formulations may
        # legitimately differ; everywhere else they agree to fp32 round-off
        if name == "dh":
            a, b = a.clone(), b.clone()
            a[5, 1], b[5, 1] = 0.0, 0.0
        assert torch.allclose(a, b, rtol=2e-3, atol=2e-4), (name, (a - b).abs().max())


def test_forward_only_row_statistics_agree_with_the_autograd_node():
    """The generation path's route-major statistics (rows ri * T + t) are the node's
    values in another order."""
    from dawn_srw_b200.ops.score_stats import score_stats, score_stats_rows
    torch.manual_seed(4)
    T, R, r, U = 6, 2, 16, 40
    emb = torch.nn.functional.normalize(torch.randn(U, r), dim=-1)
    gram, esum = emb.t() @ emb, emb.sum(0)
    h, off = torch.randn(T, R, r), torch.randn(T, R) * 0.3
    tau, isd, _, hb = score_stats(h, off, gram, esum, U)
    tau2, isd2, hb2 = score_stats_rows(h, off, gram, esum, U)
    assert torch.allclose(tau2, tau.t().reshape(-1), atol=1e-6)
    assert torch.allclose(isd2, isd.t().reshape(-1), rtol=1e-6)
    assert torch.equal(hb2, hb.transpose(0, 1).reshape(R * T, r))


def test_prepared_pool_is_freed_without_a_backward_pass():
    """A forward pass with gradients enabled that is never followed by backward (an
    exception, a skipped non-finite step) must not keep its prepared pools alive: the
    preparation node of the graph does not point back at the pool."""
    import gc
    import weakref
    from dawn_srw_b200.ops.backend import ParallelCtx
    from dawn_srw_b200.ops.cuda_backend import CudaBackend
    from dawn_srw_b200.ops.gates import gate_spec_for
    spec = gate_spec_for("spatial-r1-v4.0.1")
    be = CudaBackend()
    emb, read, write = (torch.randn(50, d, requires_grad=True) for d in (16, 32, 32))
    refs = []
    for _ in range(3):
        pool = be.prepare_pool(emb, read, write, spec, ParallelCtx())
        assert pool.emb.dtype == torch.bfloat16 and pool.g_write is not None
        refs.append(weakref.ref(pool.tensors))
        del pool
    gc.collect()
    assert all(r() is None for r in refs)
