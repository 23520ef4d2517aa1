import torch

from dawn_srw_b200.models import inference as I
from dawn_srw_b200.models.dawn import DAWN

KW = dict(vocab_size=200, d_model=32, n_layers=2, n_heads=4, max_seq_len=24, d_route=8, n_qk=24,
          n_v=30, n_know=50, dropout_rate=0.0, router_dropout=0.0)


def _model(version="spatial-r1-v4.1"):
    m = DAWN(**KW, model_version=version, seed=1)
    m.eval()
    return m


def test_prefill_matches_training_forward_logits():
    for version in ("spatial-r1-v4.1", "spatial-r1-v4.0.1", "spatial-r1-v3.9.4"):
        m = _model(version)
        ids = torch.randint(1, 200, (2, 12))
        logits, ck, cv, n = I.prefill(m, ids)
        with torch.no_grad():
            ref = m(ids, want_diag=False)["logits"]
        assert n == 12 and ck.shape == (2, 2, 4, 24, 8)
        assert torch.allclose(logits, ref, atol=1e-4), version


def test_decode_step_equals_full_forward():
    m = _model()
    ids = torch.randint(1, 200, (2, 10))
    logits, ck, cv, n = I.prefill(m, ids[:, :6])
    for t in range(6, 10):
        lg, ck, cv, n = I.decode_step(m, ids[:, t], ck, cv, n)
        with torch.no_grad():
            ref = m(ids[:, : t + 1], want_diag=False)["logits"][:, -1]
        assert torch.allclose(lg, ref, atol=2e-4), t
    assert n == 10


def test_generate_and_sampling_filters():
    m = _model()
    ids = torch.randint(1, 200, (1, 4))
    g = torch.Generator().manual_seed(0)
    seq, info = I.generate(m, ids, max_new_tokens=5, temperature=0.8, top_k=10, generator=g)
    assert seq.shape == (1, 9) and info["new_tokens"] == 5 and info["tokens_per_sec"] > 0
    greedy, _ = I.generate(m, ids, max_new_tokens=3, temperature=0.0)
    greedy2, _ = I.generate(m, ids, max_new_tokens=3, temperature=0.0)
    assert torch.equal(greedy, greedy2)
    lg = torch.tensor([[0.0, 5.0, 4.0, -1.0]])
    picks = {int(I.sample_token(lg, 1.0, top_k=2, generator=g)) for _ in range(50)}
    assert picks <= {1, 2}
    picks = {int(I.sample_token(lg, 1.0, top_p=0.5, generator=g)) for _ in range(50)}
    assert picks == {1}


def test_vectorized_eval_masks_pad_id_zero():
    m = _model()
    ids = torch.randint(1, 200, (2, 12))
    ids[:, 8:] = 0
    loss, ppl, acc, n = I.vectorized_eval(m, [ids, ids])
    assert n == 2 * 2 * 7 and ppl > 1.0 and 0.0 <= acc <= 100.0
    with torch.no_grad():
        lab = torch.where(ids > 0, ids, torch.full_like(ids, -100))
        ref = float(m(ids, labels=lab, want_diag=False)["loss"])
    assert abs(loss - ref) < 1e-5


def test_analysis_forward_gate_shapes_and_normalisation():
    m = _model("spatial-r1-v4.0.1")
    ids = torch.randint(1, 200, (2, 6))
    out = I.analysis_forward(m, ids, mode="full")
    assert out["gate_Q"].shape == (2, 2, 6, 24) and out["gate_Know"].shape == (2, 2, 6, 50)
    assert out["gate_V_raw"].shape == (2, 2, 6, 30)
    s = out["gate_Know"].sum(-1)
    assert torch.all((s - 1).abs().lt(1e-4) | s.eq(0))
    assert out["attn_out_norm"].shape == (2,)
    with torch.no_grad():
        assert torch.allclose(out["logits"], m(ids, want_diag=False)["logits"], atol=1e-4)


def test_suppressed_forward():
    m = _model()
    ids = torch.randint(1, 200, (2, 6))
    none = I.build_suppressed_forward(m, {})(ids)
    with torch.no_grad():
        assert torch.allclose(none, m(ids, want_diag=False)["logits"], atol=1e-4)
    mask = torch.zeros(50, dtype=torch.bool)
    mask[:40] = True
    some = I.build_suppressed_forward(m, {"know": mask})(ids)
    assert not torch.allclose(some, none, atol=1e-5)
    alln = I.build_suppressed_forward(m, {"know": torch.ones(50, dtype=torch.bool)})(ids)
    assert torch.isfinite(alln).all()


def test_health_and_weight_analysis_and_flops():
    m = _model()
    h = I.neuron_health(m)
    assert abs(h["know_emb_norm_mean"] - 1.0) < 1e-4 and h["qk_read_dead"] == 0
    assert abs(h["tau_know_bias"] + 0.5) < 1e-6
    w = I.weight_analysis(m)
    assert 0 < w["know_write_effective_rank"] <= 32 + 1e-3 and w["qk_emb_cos_abs_mean"] < 1.0
    big = DAWN(**{**KW, "d_model": 384, "n_layers": 12, "n_heads": 6, "d_route": 128, "n_qk": 1580,
                  "n_v": 2600, "n_know": 25200, "vocab_size": 30522, "max_seq_len": 512})
    f = I.estimate_flops_per_token(big)
    # 0.79 GF/token when the scores are counted twice (two sweeps); one sweep here
    scores = 2 * 128 * (2 * 1580 + 2600 + 25200)
    assert abs((f["total"] + 12 * scores) / 1e9 - 0.79) < 0.01


def test_dense_baseline_kv_cache_matches_full_forward():
    from dawn_srw_b200.models.baseline import VanillaTransformer
    m = VanillaTransformer(vocab_size=200, d_model=32, d_ff=64, n_layers=2, n_heads=4, max_seq_len=24,
                           dropout_rate=0.0, seed=2)
    m.eval()
    ids = torch.randint(1, 200, (2, 10))
    logits, ck, cv, n = I.prefill(m, ids[:, :6])
    with torch.no_grad():
        assert torch.allclose(logits, m(ids[:, :6])["logits"], atol=1e-4)
    for t in range(6, 10):
        lg, ck, cv, n = I.decode_step(m, ids[:, t], ck, cv, n)
        with torch.no_grad():
            ref = m(ids[:, : t + 1])["logits"][:, -1]
        assert torch.allclose(lg, ref, atol=2e-4), t
    out, stats = I.generate(m, ids[:, :4], max_new_tokens=5, temperature=0.0)
    assert out.shape == (2, 9) and stats["new_tokens"] == 5


def test_prepared_pools_are_cached_until_a_parameter_changes():
    m = _model("spatial-r1-v4.0.1")
    ids = torch.randint(1, 200, (1, 8))
    a, *_ = I.prefill(m, ids)
    pools1 = m._inference_pools[1]
    b, *_ = I.prefill(m, ids)
    assert m._inference_pools[1] is pools1 and torch.equal(a, b)       # reused
    with torch.no_grad():
        m.neuron_pool.know_write.mul_(1.5)                             # in-place update bumps the version
    c, *_ = I.prefill(m, ids)
    assert m._inference_pools[1] is not pools1 and not torch.allclose(a, c)
    with torch.no_grad():
        ref = m(ids, want_diag=False)["logits"]
    assert torch.allclose(c, ref, atol=1e-4)
