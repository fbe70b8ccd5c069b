"""cxg_column_sum (the bias gradient of the layers): against float64, run-to-run identical, through autograd."""
import pytest
import torch

from helpers import randn, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,width", [(1, 1), (5, 47), (1000, 128), (70001, 64), (3000, 300), (257, 1024), (0, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_column_sum(cuda, n, width, dtype):
    import cxgnncomp_backend as be
    x = randn((n, width), n + width, dtype=dtype)
    got = be.column_sum(x.cuda())
    assert got.dtype == torch.float32 and got.shape == (width,)
    want = x.double().sum(0)
    if n == 0:
        assert bool((got == 0).all())
        return
    assert float((got.cpu().double() - want).abs().max()) <= 1e-5 * float(x.double().abs().sum(0).max()) + 1e-30
    assert torch.equal(got, be.column_sum(x.cuda()))


def test_bias_add_autograd(cuda):
    import cxgnncomp_backend as be
    y = randn((4000, 4, 32), 1).cuda().requires_grad_(True)
    b = randn((4, 32), 2).cuda().requires_grad_(True)
    out = be.bias_add(y, b)
    assert torch.equal(out, y + b)
    go = randn((4000, 4, 32), 3).cuda()
    out.backward(go)
    assert torch.equal(y.grad, go)
    assert rel_err(b.grad.cpu(), go.cpu().double().sum(0)) < 1e-5
    # a bias over the last dimension only, and shapes the kernel does not cover, take the torch expression
    y2 = randn((10, 3, 8), 4).cuda().requires_grad_(True)
    b2 = randn((8,), 5).cuda().requires_grad_(True)
    be.bias_add(y2, b2).sum().backward()
    assert torch.allclose(b2.grad.cpu(), torch.full((8,), 30.0))
