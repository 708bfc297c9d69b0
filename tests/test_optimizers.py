"""StreamedAdamW against torch.optim.AdamW bit for bit (the reference's own bar: tests/trainer/test_streamed_adamw_on_gpu.py),
with a chunk size small enough that the staging slots wrap; FusedAdamW's kernel with bf16 gradients."""

import pytest
import torch

from pear_b200.train.streamed_adamw import StreamedAdamW


def _run(opt_cls, device, steps=4, **kw):
    g = torch.Generator(device=device).manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(257, 33, device=device, generator=g)), torch.nn.Parameter(torch.randn(19, device=device, generator=g)),
          torch.nn.Parameter(torch.randn(3, 5, 7, device=device, generator=g))]
    opt = opt_cls(ps, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, **kw)
    for _ in range(steps):
        for x in ps:
            x.grad = torch.randn(x.shape, device=device, generator=g)
        opt.step()
    return [x.detach().clone() for x in ps], opt


def test_streamed_adamw_bit_exact_cpu():
    a, opt = _run(StreamedAdamW, "cpu", chunk_bytes=8 * 100)  # 100 elements per chunk: 85 chunks for the first parameter
    b, _ = _run(torch.optim.AdamW, "cpu", foreach=False)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    # the moments live flat in host memory, one pair per parameter
    for p in opt.param_groups[0]["params"]:
        assert opt.state[p]["exp_avg"].numel() == p.numel() and not opt.state[p]["exp_avg"].is_cuda


@pytest.mark.gpu
def test_streamed_adamw_bit_exact_gpu():
    """Moments in pinned host memory, three staging slots, copy streams on both sides of the update: 85 chunks per step make
    every slot wrap many times; the parameters equal torch.optim.AdamW's bit for bit after four steps."""
    a, opt = _run(StreamedAdamW, "cuda", chunk_bytes=8 * 100)
    b, _ = _run(torch.optim.AdamW, "cuda", foreach=False, fused=False)
    torch.cuda.synchronize()
    for x, y in zip(a, b):
        assert torch.equal(x, y), float((x - y).abs().max())
    for p in opt.param_groups[0]["params"]:
        assert opt.state[p]["exp_avg"].is_pinned()


@pytest.mark.gpu
def test_fused_adamw_bf16_gradients():
    """The kernel reads bf16 gradients (what the bf16 reduce-scatter leaves) and scales them by `grad_scale`: equal to the
    fp32 update fed with the same bf16-rounded, scaled gradients."""
    from pear_b200.ops import lib as kl
    from pear_b200.train.fused_adamw import FusedAdamW

    def run(fused: bool):
        g = torch.Generator(device="cuda").manual_seed(1)
        ps = [torch.nn.Parameter(torch.randn(1000, 37, device="cuda", generator=g)), torch.nn.Parameter(torch.randn(13, device="cuda", generator=g))]
        opt = (FusedAdamW if fused else torch.optim.AdamW)(ps, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, **({} if fused else dict(foreach=False, fused=False)))
        for _ in range(3):
            for x in ps:
                gr = torch.randn(x.shape, device="cuda", generator=g).to(torch.bfloat16)
                if fused:
                    x.grad_dtype = None  # torch checks a gradient's dtype against the parameter's unless told otherwise
                    x.grad = gr
                else:
                    x.grad = gr.float() * 0.25
            if fused:
                opt.step(grad_scale=0.25)
            else:
                opt.step()
        return [x.detach().clone() for x in ps]

    before = kl.LAUNCH_COUNT
    a = run(True)
    assert kl.LAUNCH_COUNT == before + 6  # the kernel ran, not the torch statements
    b = run(False)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, atol=1e-6, rtol=1e-5), float((x - y).abs().max())
