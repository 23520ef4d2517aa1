import torch

from dawn_srw_b200.models.dawn import DAWN
from dawn_srw_b200.models.baseline import VanillaTransformer
from dawn_srw_b200.ops import reference as R

KW = dict(vocab_size=300, d_model=32, n_layers=2, n_heads=4, max_seq_len=16, d_route=8, n_qk=24,
          n_v=30, n_know=50)


def test_forward_keys_and_shapes():
    m = DAWN(**KW, dropout_rate=0.0, router_dropout=0.0)
    ids = torch.randint(0, 300, (3, 16))
    r = m(ids, labels=ids)
    for k in ("loss", "correct", "valid_count", "per_token_ce", "valid_mask", "aux_loss",
              "attn_aux", "know_aux", "dead_penalty", "attn_tau_offset", "know_tau_offset",
              "know_active", "attn_qk_active", "attn_v_active", "attn_score_std", "know_gate_entropy",
              "qk_emb_norm_mean", "know_emb_norm", "per_layer_attn_out_norm", "debug_residual_norm",
              "attn_int_max", "know_int_cap_frac", "attn_tau_std"):
        assert k in r, k
    assert r["attn_tau_offset"].shape == (2, 3, 16, 3) and r["know_tau_offset"].shape == (2, 3, 16, 1)
    assert r["per_token_ce"].shape == (3, 15) and r["attn_tau_std"].shape == (3,)
    assert "logits" not in r
    r2 = m(ids)
    assert r2["logits"].shape == (3, 16, 300)


def test_sequence_longer_than_max_raises():
    m = DAWN(**KW)
    try:
        m(torch.zeros(1, 17, dtype=torch.long))
    except ValueError:
        return
    raise AssertionError("expected ValueError")


def test_layer_recompute_gives_same_loss_and_grads():
    ids = torch.randint(0, 300, (2, 16))
    grads = []
    for ck in (False, True):
        m = DAWN(**KW, dropout_rate=0.0, router_dropout=0.0, gradient_checkpointing=ck, seed=3)
        m.train()
        r = m(ids, labels=ids, want_diag=False)
        (r["loss"] + 0.1 * r["aux_loss"] + 0.1 * r["dead_penalty"]).backward()
        grads.append({n: p.grad.clone() for n, p in m.named_parameters()})
    for n in grads[0]:
        assert torch.allclose(grads[0][n], grads[1][n], atol=1e-6), n


def test_eval_has_no_dropout_scaling():
    """An earlier version of the reference scaled activations by 1/keep at eval."""
    m = DAWN(**KW, dropout_rate=0.5, router_dropout=0.5)
    m.eval()
    ids = torch.randint(0, 300, (2, 16))
    a = m(ids, labels=ids, want_diag=False)["loss"]
    b = m(ids, labels=ids, want_diag=False)["loss"]
    m0 = DAWN(**KW, dropout_rate=0.0, router_dropout=0.0)
    m0.load_state_dict(m.state_dict())
    m0.eval()
    c = m0(ids, labels=ids, want_diag=False)["loss"]
    assert float(a) == float(b) == float(c)
    x = torch.randn(4, 4)
    assert torch.equal(R.dropout(x, 0.9, False), x)


def test_labels_minus_100_are_ignored():
    m = DAWN(**KW, dropout_rate=0.0, router_dropout=0.0)
    ids = torch.randint(0, 300, (2, 16))
    lab = ids.clone()
    lab[:, 8:] = -100
    r = m(ids, labels=lab, want_diag=False)
    assert int(r["valid_count"]) == 2 * 7
    assert float(r["per_token_ce"][:, 7:].abs().sum()) == 0.0


def test_v394_has_no_scale_params_and_reports_tau_reg():
    m = DAWN(**KW, model_version="spatial-r1-v3.9.4")
    names = dict(m.named_parameters())
    assert "neuron_pool.qk_scale" not in names
    ids = torch.randint(0, 300, (2, 16))
    assert "tau_reg" in m(ids, labels=ids, want_diag=False)
    m41 = DAWN(**KW)
    assert "neuron_pool.know_scale" in dict(m41.named_parameters())


def test_baseline_transformer_interface():
    m = VanillaTransformer(vocab_size=300, d_model=32, d_ff=64, n_layers=2, n_heads=4, max_seq_len=16,
                           dropout_rate=0.0)
    ids = torch.randint(0, 300, (2, 16))
    r = m(ids, labels=ids)
    assert float(r["aux_loss"]) == 0.0 and r["loss"].requires_grad
    r["loss"].backward()
    assert m(ids)["logits"].shape == (2, 16, 300)
