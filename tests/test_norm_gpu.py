"""Residual add + RMSNorm kernel (b200_residual_rmsnorm) against plain torch."""
import pytest
import torch
import torch.nn.functional as F

from sparser_faster_llms_b200 import _lib, norm

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.mark.parametrize("m,d", [(1, 2048), (32, 2048), (5, 4096), (3, 264), (7, 8192)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_matches_torch(m, d, with_delta):
    gen = torch.Generator().manual_seed(m * d)
    x = torch.randn(m, 1, d, generator=gen).to(torch.bfloat16).to(DEV)
    delta = (torch.randn(m, 1, d, generator=gen) * 0.3).to(torch.bfloat16).to(DEV)
    w = (1 + 0.1 * torch.randn(d, generator=gen)).to(torch.bfloat16).to(DEV)
    dl = delta if with_delta else None
    x_out, h = norm.residual_rmsnorm(x, dl, w, 1e-5)
    want_x, want_h = norm.reference(x, dl, w, 1e-5)
    torch.cuda.synchronize()
    assert torch.equal(x_out, want_x)               # the sum is a single bf16 rounding
    assert x.data_ptr() != x_out.data_ptr() or not with_delta
    # normalised values: the fp32 sum of squares may be grouped differently -> one bf16 ulp
    assert torch.allclose(h.float(), want_h.float(), rtol=2 ** -7, atol=1e-6)
    assert (h != want_h).float().mean() < 0.02
    lib = F.rms_norm(want_x, (d,), w, 1e-5)
    assert torch.allclose(h.float(), lib.float(), rtol=2 ** -6, atol=1e-6)


def test_in_place_and_argument_errors():
    x = torch.randn(4, 2048).to(torch.bfloat16).to(DEV)
    delta = torch.randn(4, 2048).to(torch.bfloat16).to(DEV)
    w = torch.ones(2048, dtype=torch.bfloat16, device=DEV)
    want_x, want_h = norm.reference(x, delta, w, 1e-5)
    x_out, h = norm.residual_rmsnorm(x, delta, w, 1e-5, inplace=True)
    torch.cuda.synchronize()
    assert x_out.data_ptr() == x.data_ptr() and torch.equal(x, want_x)
    assert torch.allclose(h.float(), want_h.float(), rtol=2 ** -7, atol=1e-6)
    with pytest.raises(ValueError):
        norm.residual_rmsnorm(x, delta[:2], w, 1e-5)
    with pytest.raises(ValueError):   # D not a multiple of 8
        _lib.call("b200_residual_rmsnorm", DEV, x.data_ptr(), None, w.data_ptr(), 1e-5, None,
                  delta.data_ptr(), 4, 2044)
    with pytest.raises(ValueError):   # h_out aliases x
        _lib.call("b200_residual_rmsnorm", DEV, x.data_ptr(), None, w.data_ptr(), 1e-5, None,
                  x.data_ptr(), 4, 2048)
    with pytest.raises(RuntimeError):
        norm.residual_rmsnorm(x.cpu(), None, w.cpu(), 1e-5)
