"""The backward of the delta-rule chunk loop is the same recurrence run in reverse with W and Kt swapped: checked on
CPU (torch statement of the kernel) against autograd of the plain chunked scan."""

import torch

from pear_b200.ops import kernels as K
from pear_b200.ops import reference as ref


def test_scan_loop_backward_equals_autograd_of_the_chunked_scan():
    g = torch.Generator().manual_seed(0)
    t, hk, hv, d = 150, 1, 2, 128
    q = ref.l2norm(torch.randn(t, hk, d, generator=g)) * d ** -0.5
    k = ref.l2norm(torch.randn(t, hk, d, generator=g))
    v = torch.randn(t, hv, 32, generator=g)
    gate = -torch.rand(t, hv, generator=g) * 0.2
    beta = torch.rand(t, hv, generator=g)
    s0 = torch.randn(hv, 32, d, generator=g) * 0.1
    w_o, w_s = torch.randn(t, hv, 32, generator=g), torch.randn(hv, 32, d, generator=g)

    def run(fn):
        leaves = [x.clone().double().requires_grad_(True) for x in (q, k, v, gate, beta, s0)]
        o, s = fn(*[x.float() for x in leaves])
        ((o * w_o).sum() + (s * w_s).sum()).backward()
        return o, s, [x.grad for x in leaves]

    def through_loop_function(q_, k_, v_, g_, b_, s_):
        op = ref.gdn_chunk_operands(q_, k_, v_, g_, b_)
        o, s = K._ScanLoop.apply(op["W"], op["U"], op["Qe"], op["A"], op["Kt"], op["gamma"], s_)
        return o.permute(1, 2, 0, 3).reshape(op["n"] * 64, hv, 32)[:t], s

    o1, s1, g1 = run(through_loop_function)
    o2, s2, g2 = run(ref.gdn_chunked)
    assert (o1 - o2).abs().max() < 1e-5 and (s1 - s2).abs().max() < 1e-5
    for name, a, b in zip(("q", "k", "v", "g", "beta", "s0"), g1, g2):
        assert ((a - b).norm() / (b.norm() + 1e-12)).item() < 1e-4, name
