"""128-point Walsh-Hadamard pre-conditioning kernel against the oracle's restatement of normalized_fwht
(r2omni/sspa/runtime/int2_reference.py:18-31): same butterfly order, so the rounded result is bit-exact."""
import pytest
import torch

import r2omni_b200 as R
from oracle import sspa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 128), (7, 128), (2, 130, 128), (4, 28, 33, 128)])
def test_fwht_matches_the_oracle_bit_for_bit(dtype, shape):
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * torch.exp(torch.randn(shape[-1], generator=g))).to(dtype)
    want = O.fwht128(x).to(dtype)
    got = R.triton_fwht_128(x.cuda())
    assert got.dtype == dtype and got.shape == x.shape
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))
    # in place through `output`, and twice is the identity up to rounding
    y = x.cuda()
    assert R.triton_fwht_128(y, output=y) is y
    assert torch.equal(y, got)
    back = R.triton_fwht_128(got).float().cpu()
    assert (back - x.float()).abs().max() <= 2.0 ** -6 * x.float().abs().max()


def test_fwht_argument_errors_follow_the_reference():
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        R.triton_fwht_128(x)
    with pytest.raises(ValueError):
        R.triton_fwht_128(torch.zeros(4, 128, dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError):
        R.triton_fwht_128(torch.zeros(4, 128, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        R.triton_fwht_128(torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda"),
                          output=torch.zeros(4, 128, dtype=torch.float16, device="cuda"))
    empty = R.triton_fwht_128(torch.zeros(0, 128, dtype=torch.bfloat16, device="cuda"))
    assert empty.shape == (0, 128)
