import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nesterov,wd,momentum", [(False, 0.0, 0.0), (False, 5e-4, 0.9), (True, 5e-4, 0.9)])
def test_fused_sgd_matches_torch(nesterov, wd, momentum):
    from grace_b200.optim import FusedSGD

    torch.manual_seed(0)
    dev = torch.device("cuda")
    shapes = [(64, 3, 3, 3), (64,), (1000, 77), (5,)]
    ref_params = [torch.randn(s, device=dev, requires_grad=True) for s in shapes]
    my_params = [p.detach().clone().requires_grad_(True) for p in ref_params]
    ref = torch.optim.SGD(ref_params, lr=0.1, momentum=momentum, weight_decay=wd, nesterov=nesterov)
    mine = FusedSGD(my_params, lr=0.1, momentum=momentum, weight_decay=wd, nesterov=nesterov)
    for step in range(4):
        for p, q in zip(ref_params, my_params):
            g = torch.randn_like(p)
            p.grad = g.clone()
            if q.grad is None:
                q.grad = g.clone()
            else:
                q.grad.copy_(g)
        ref.step()
        mine.step()
        for p, q in zip(ref_params, my_params):
            torch.testing.assert_close(q, p, rtol=1e-6, atol=1e-6)
