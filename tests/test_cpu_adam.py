"""Native host AdamW against torch.optim.AdamW (fp32 and bf16 parameters)."""
import torch


def test_cpu_offload_adam_matches_torch_adamw():
    from loongforge_b200.optim.cpu_offload import CPUOffloadAdam

    torch.manual_seed(0)
    a = torch.nn.Sequential(torch.nn.Linear(33, 17), torch.nn.Linear(17, 5))
    b = torch.nn.Sequential(torch.nn.Linear(33, 17), torch.nn.Linear(17, 5))
    b.load_state_dict(a.state_dict())
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref = torch.optim.AdamW([{"params": [p for p in a.parameters() if p.dim() > 1]},
                             {"params": [p for p in a.parameters() if p.dim() <= 1], "weight_decay": 0.0}], **kw)
    opt = CPUOffloadAdam(b.parameters(), **kw)
    for _ in range(5):
        x = torch.randn(8, 33)
        for m, o in ((a, ref), (b, opt)):
            o.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert torch.allclose(pa, pb, atol=2e-6, rtol=1e-5), (pa - pb).abs().max()


def test_cpu_offload_adam_bf16_params_keep_fp32_master():
    from loongforge_b200.optim.cpu_offload import CPUOffloadAdam

    p = torch.nn.Parameter(torch.ones(1000, dtype=torch.bfloat16))
    opt = CPUOffloadAdam([p], lr=1e-4, weight_decay=0.0)
    for _ in range(30):  # each update is far below bf16 resolution at 1.0, the master accumulates them
        p.grad = torch.ones_like(p)
        opt.step()
    assert abs(float(opt.state[0]["master"][0]) - (1.0 - 30e-4)) < 1e-5
    assert float(p[0]) < 1.0
    sd = opt.state_dict()
    opt2 = CPUOffloadAdam([torch.nn.Parameter(torch.ones(1000, dtype=torch.bfloat16))], lr=1e-4)
    opt2.load_state_dict(sd)
    assert opt2.step_count == 30 and torch.equal(opt2.state[0]["m"], opt.state[0]["m"])
