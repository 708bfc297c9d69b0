"""The operand split behind the head's logits GEMM: three bf16 products laid side by side along K reproduce the fp32
product to ~2^-16 (the GEMM itself runs on the GPU; here the concatenated operands are multiplied in fp64)."""

import torch

from pear_b200.ops.gemm import split_operand


def test_three_term_bf16_split_is_close_to_the_fp32_product():
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(64, 256, generator=g), torch.randn(96, 256, generator=g)
    ac, bc = split_operand(a, "a"), split_operand(b, "b")
    assert ac.dtype == torch.bfloat16 and ac.shape == (64, 768) and bc.shape == (96, 768)
    want = a.double() @ b.double().t()
    got = ac.double() @ bc.double().t()
    plain = a.to(torch.bfloat16).double() @ b.to(torch.bfloat16).double().t()
    err, err_plain = ((got - want).norm() / want.norm()).item(), ((plain - want).norm() / want.norm()).item()
    assert err < 2e-5 and err < err_plain / 50
