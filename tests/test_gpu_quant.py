"""CUDA quantisers vs the oracle: bit-exact bytes and scale bits (through the C ABI)."""
import numpy as np
import pytest
import torch

from oracle import fp8_spec as S

pytestmark = pytest.mark.gpu


def bits(t):
    return t.contiguous().view(torch.uint8 if t.element_size() == 1 else torch.int32).cpu()


@pytest.fixture(scope="module")
def ops(built_library):
    from nano_qwen_b200 import ops
    ops.init()
    return ops


@pytest.mark.parametrize("m,k", [(1, 128), (7, 1024), (16, 4096), (129, 3072), (64, 12288), (300, 256),
                                 (5, 192), (3, 100), (2, 17), (33, 4096 + 64)])
def test_act_quant_bit_exact(ops, m, k):
    g = torch.Generator().manual_seed(m * 1000 + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    xq_ref, sx_ref = S.quantize_act_group128(x)
    xq, sx = ops.act_quant(x.cuda())
    torch.cuda.synchronize()
    assert xq.shape == (m, k) and sx.shape == sx_ref.shape
    assert torch.equal(bits(sx), bits(sx_ref))
    assert torch.equal(bits(xq) & 0x7F, bits(xq_ref) & 0x7F)      # sign of an exact zero is not significant
    nz = (bits(xq_ref) & 0x7F) != 0
    assert torch.equal(bits(xq)[nz], bits(xq_ref)[nz])


def test_act_quant_bit_exact_over_many_scales(ops):
    """16 M elements, per-row magnitudes from 2^-60 to 2^60: the reciprocal-based exact division agrees
    with the IEEE divide of the oracle on every byte."""
    g = torch.Generator().manual_seed(2024)
    x = torch.randn(4096, 4096, generator=g)
    x = x * torch.exp2(torch.randint(-60, 61, (4096, 1), generator=g).float()) * (1 + torch.rand(4096, 1, generator=g))
    x = x.to(torch.bfloat16)
    xq_ref, sx_ref = S.quantize_act_group128(x)
    xq, sx = ops.act_quant(x.cuda())
    assert torch.equal(bits(sx), bits(sx_ref))
    assert torch.equal(bits(xq) & 0x7F, bits(xq_ref) & 0x7F)
    nz = (bits(xq_ref) & 0x7F) != 0
    assert torch.equal(bits(xq)[nz], bits(xq_ref)[nz])


def test_act_quant_edge_values(ops):
    x = torch.zeros(6, 256, dtype=torch.bfloat16)
    x[0, :128] = 1.0
    x[0, 128] = 448.0
    x[0, 129] = -3.0
    x[1, 5] = -2.0
    x[3, :] = torch.finfo(torch.bfloat16).max                      # huge values: scale ~7.6e35, q = 448
    x[4, 0], x[4, 1] = 1.0, 2.0 ** -10                             # lands between e4m3 subnormal steps after scaling
    x[5, 0], x[5, 1], x[5, 2] = 1.0, 1.0 / 448 * 2 ** -9 * 1.5, 1e-30    # subnormal midpoint, underflow to zero
    xq_ref, sx_ref = S.quantize_act_group128(x)
    xq, sx = ops.act_quant(x.cuda())
    assert torch.equal(bits(sx), bits(sx_ref))
    assert torch.equal(bits(xq) & 0x7F, bits(xq_ref) & 0x7F)
    assert sx[2, 0].item() == np.float32(1e-10) / np.float32(448)  # all-zero group


def test_act_quant_strided_input_and_large(ops):
    g = torch.Generator().manual_seed(3)
    big = torch.randn(2048, 4096 + 256, generator=g).to(torch.bfloat16)
    view = big[:, 128:128 + 4096]                                  # row stride != K
    xq_ref, sx_ref = S.quantize_act_group128(view)
    xq, sx = ops.act_quant(big.cuda()[:, 128:128 + 4096])
    assert torch.equal(bits(sx), bits(sx_ref))
    assert torch.equal(bits(xq) & 0x7F, bits(xq_ref) & 0x7F)


@pytest.mark.parametrize("n,k", [(128, 128), (1024, 2048), (4096, 1024), (130, 200), (256, 100), (384, 4096 + 64)])
def test_weight_quant_bit_exact(ops, n, k):
    g = torch.Generator().manual_seed(n + k)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    wq_ref, sw_ref = S.quantize_weight_block128(w)
    wq, sw = ops.weight_quant(w.cuda())
    assert torch.equal(bits(sw), bits(sw_ref))
    assert torch.equal(bits(wq) & 0x7F, bits(wq_ref) & 0x7F)


def test_quantisers_leave_status_clean(ops):
    from nano_qwen_b200 import _cabi
    torch.cuda.synchronize()
    assert _cabi.device_status()["code"] == 0
