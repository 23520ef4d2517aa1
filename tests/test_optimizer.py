import math

import torch

from dawn_srw_b200.models.dawn import DAWN
from dawn_srw_b200.train.optimizer import DawnAdamW, warmup_cosine, wd_group_of


def test_schedule_values():
    lr, warm, total = 1e-3, 10, 110
    assert warmup_cosine(0, lr, warm, total) == 1e-4
    assert abs(warmup_cosine(5, lr, warm, total) - (1e-4 + 9e-4 * 0.5)) < 1e-12
    assert abs(warmup_cosine(10, lr, warm, total) - 1e-3) < 1e-12
    assert abs(warmup_cosine(60, lr, warm, total) - (1e-4 + 9e-4 * 0.5)) < 1e-12
    assert abs(warmup_cosine(110, lr, warm, total) - 1e-4) < 1e-12
    assert abs(warmup_cosine(500, lr, warm, total) - 1e-4) < 1e-12


def test_weight_decay_groups():
    assert wd_group_of("neuron_pool.know_read") == "pool"
    assert wd_group_of("neuron_pool.qk_emb") == "pool"
    assert wd_group_of("neuron_pool.qk_scale") == "none"
    assert wd_group_of("router.proj_attn.weight") == "base"
    assert wd_group_of("router.proj_attn.bias") == "none"
    assert wd_group_of("layers.3.norm1.weight") == "none"
    assert wd_group_of("norm.weight") == "none"
    assert wd_group_of("layers.0.attn.expand_O.weight") == "base"
    assert wd_group_of("token_emb.weight") == "base"
    m = DAWN(vocab_size=50, d_model=16, n_layers=2, n_heads=2, max_seq_len=8, d_route=4, n_qk=8, n_v=8, n_know=8)
    opt = DawnAdamW(m.named_parameters(), lr=1e-3, fused=False)
    assert len(opt.groups["pool"]) == 9
    assert len(opt.groups["base"]) == 2 + 2 + 2 + 2     # embeddings, 2 proj, 2 tau kernels, 2 O-proj


def test_step_matches_formula():
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(5, 3))
    b = torch.nn.Parameter(torch.randn(3))
    opt = DawnAdamW([("router.proj_know.weight", p), ("router.proj_know.bias", b)], lr=0.1,
                    weight_decay=0.1, schedule=lambda s: 0.1 * (s + 1), clip_norm=1.0, fused=False)
    p0, b0 = p.detach().clone(), b.detach().clone()
    gp, gb = torch.randn(5, 3) * 3, torch.randn(3) * 3
    p.grad, b.grad = gp.clone(), gb.clone()
    opt.step()
    norm = math.sqrt(float(gp.square().sum() + gb.square().sum()))
    sc = 1.0 / max(norm, 1.0)
    for w0, g, w, wd in ((p0, gp, p, 0.1), (b0, gb, b, 0.0)):
        g = g * sc
        m, v = 0.1 * g, 0.05 * g * g
        upd = (m / 0.1) / ((v / 0.05).sqrt() + 1e-8) + wd * w0
        assert torch.allclose(w.detach(), w0 - 0.1 * upd, atol=1e-6)
    assert abs(float(opt.last_grad_norm) - norm) < 1e-4
    p.grad, b.grad = gp.clone(), gb.clone()
    opt.step()
    assert abs(opt.last_lr - 0.2) < 1e-12       # schedule counts optimizer steps from 0


def test_gradient_accumulation_averages():
    w1 = torch.nn.Parameter(torch.ones(4))
    w2 = torch.nn.Parameter(torch.ones(4))
    o1 = DawnAdamW([("w.weight", w1)], lr=0.1, accumulation_steps=2, fused=False)
    o2 = DawnAdamW([("w.weight", w2)], lr=0.1, fused=False)
    ga, gb = torch.tensor([1., 2, 3, 4]) * 0.1, torch.tensor([4., 3, 2, 1]) * 0.1
    w1.grad = ga.clone()
    assert o1.step() is False
    w1.grad = gb.clone()
    assert o1.step() is True
    w2.grad = (ga + gb) / 2
    o2.step()
    assert torch.allclose(w1, w2, atol=1e-7) and o1.count == 1


def test_state_dict_roundtrip():
    w = torch.nn.Parameter(torch.randn(4))
    o = DawnAdamW([("w.weight", w)], lr=0.1, fused=False)
    w.grad = torch.randn(4)
    o.step()
    sd = o.state_dict()
    w2 = torch.nn.Parameter(w.detach().clone())
    o2 = DawnAdamW([("w.weight", w2)], lr=0.1, fused=False)
    o2.load_state_dict(sd)
    g = torch.randn(4)
    w.grad, w2.grad = g.clone(), g.clone()
    o.step(), o2.step()
    assert torch.equal(w, w2)
