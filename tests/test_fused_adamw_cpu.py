"""FusedAdamW keeps torch.optim.AdamW's statements and state layout (CPU path here; the kernel path has a GPU test)."""

import torch

from pear_b200.train.fused_adamw import FusedAdamW


def _run(opt_cls, device="cpu", steps=3, **kw):
    torch.manual_seed(0)
    p = [torch.nn.Parameter(torch.randn(37, 5, device=device)), torch.nn.Parameter(torch.randn(11, device=device))]
    opt = opt_cls(p, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, **kw)
    g = torch.Generator(device=device).manual_seed(1)
    for _ in range(steps):
        for x in p:
            x.grad = torch.randn(x.shape, device=device, generator=g)
        opt.step()
    return [x.detach().clone() for x in p], opt


def test_matches_torch_adamw_and_shares_its_state_layout():
    a, oa = _run(FusedAdamW)
    b, ob = _run(torch.optim.AdamW, foreach=False, fused=False)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, atol=1e-6, rtol=1e-5)
    sa, sb = oa.state_dict()["state"], ob.state_dict()["state"]
    assert sa.keys() == sb.keys() and all(set(sa[k]) == set(sb[k]) for k in sa)
    ob.load_state_dict(oa.state_dict())  # a run may switch between the two
