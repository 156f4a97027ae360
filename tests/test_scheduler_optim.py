import torch

from tests.tiny import TINY


def _lrs(total, warm, decay):
    from torchure_b200.optim import WarmupStableDecay

    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=1.0)
    sch = WarmupStableDecay(opt, total_steps=total, warmup_ratio=warm, decay_ratio=decay)
    used = []
    for _ in range(total):
        used.append(opt.param_groups[0]["lr"])
        opt.step()
        sch.step()
    return used, sch.get_last_lr()[0]


def test_wsd_values():
    used, after = _lrs(20, 0.2, 0.25)
    want = [0.25, 0.5, 0.75] + [1.0] * 13 + [0.8, 0.6, 0.4, 0.2]
    torch.testing.assert_close(torch.tensor(used), torch.tensor(want))
    assert after == 0.0
    used, after = _lrs(100, 0.001, 0.1)
    assert all(abs(u - 1.0) < 1e-12 for u in used[:91])
    torch.testing.assert_close(torch.tensor(used[91:]), torch.tensor([0.9 - 0.1 * i for i in range(9)]))
    assert after == 0.0


def test_wsd_state_dict_keys_and_roundtrip():
    from torchure_b200.optim import WarmupStableDecay

    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=1.0)
    sch = WarmupStableDecay(opt, total_steps=10, warmup_ratio=0.1, decay_ratio=0.2)
    for _ in range(4):
        opt.step()
        sch.step()
    sd = sch.state_dict()
    for key in ("total_steps", "warmup_ratio", "decay_ratio", "base_lrs", "last_epoch", "_last_lr"):
        assert key in sd
    sch2 = WarmupStableDecay(torch.optim.SGD([p], lr=1.0), total_steps=10, warmup_ratio=0.1, decay_ratio=0.2)
    sch2.load_state_dict(sd)
    assert sch2.last_epoch == 4 and sch2.get_last_lr() == sch.get_last_lr()


def test_cosine_is_real():
    from torchure_b200.optim.scheduler import cosine_scale

    assert cosine_scale(0, 100, 0.1, 0.0) == 0.1
    assert abs(cosine_scale(10, 100, 0.1, 0.0) - 1.0) < 1e-12
    assert cosine_scale(99, 100, 0.1, 0.1) < 0.11


def test_param_groups_and_adamw_matches_torch():
    from torchure_b200.models import Qwen3
    from torchure_b200.optim import build_optimizer

    torch.manual_seed(0)
    a = Qwen3(**TINY)
    a.init_weights()
    b = Qwen3(**TINY)
    b.load_state_dict(a.state_dict())
    cfg = {"lr": 3e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "fused": True}
    opt = build_optimizer(a, "adamw", cfg)
    assert [g["weight_decay"] for g in opt.param_groups] == [0.1, 0.0]
    assert all(p.dim() >= 2 for p in opt.param_groups[0]["params"])
    assert all(p.dim() < 2 for p in opt.param_groups[1]["params"])
    decay = [p for p in b.parameters() if p.dim() >= 2]
    nodecay = [p for p in b.parameters() if p.dim() < 2]
    ref = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": nodecay, "weight_decay": 0.0}],
                            lr=3e-3, betas=(0.9, 0.95))
    ids = torch.randint(0, TINY["vocab_size"], (2, 16))
    for _ in range(3):
        for m, o in ((a, opt), (b, ref)):
            o.zero_grad()
            m(ids).float().pow(2).mean().backward()
            o.step()
    for p, q in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(p, q)
    sd = opt.state_dict()
    assert set(sd["state"][0].keys()) == {"step", "exp_avg", "exp_avg_sq"}


def test_grad_scale_hook_equals_prescaled_grads():
    from torchure_b200.optim import AdamW

    torch.manual_seed(0)
    p1 = torch.nn.Parameter(torch.randn(4, 4))
    p2 = torch.nn.Parameter(p1.detach().clone())
    g = torch.randn(4, 4)
    o1, o2 = AdamW([p1], lr=1e-2), AdamW([p2], lr=1e-2)
    p1.grad = g.clone()
    o1.set_grad_scale(torch.tensor(0.25))
    o1.step()
    p2.grad = g * 0.25
    o2.step()
    torch.testing.assert_close(p1, p2)
