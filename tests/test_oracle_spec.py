"""The oracle's arithmetic specification, pinned by known answers and properties (CPU)."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from oracle import fp8_spec as S


def test_decode_table_matches_torch():
    tab = S.e4m3_decode_table()
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(tab), np.isnan(ref))
    assert np.array_equal(tab[~np.isnan(tab)], ref[~np.isnan(ref)])
    assert tab[0x7E] == 448.0 and tab[0x01] == 2.0 ** -9 and tab[0x08] == 2.0 ** -6


def test_numpy_encoder_matches_torch_cast_on_all_midpoints():
    tab = S.e4m3_decode_table()
    fin = np.sort(tab[~np.isnan(tab)])
    mids = ((fin[:-1].astype(np.float64) + fin[1:]) / 2).astype(np.float32)
    rng = np.random.default_rng(0)
    x = np.concatenate([fin, mids, np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf)),
                        np.clip(rng.standard_normal(100000).astype(np.float32) * 100, -448, 448),
                        rng.standard_normal(100000).astype(np.float32) * 0.01])
    ours = S.e4m3_encode_rne(x)
    theirs = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    # +0/-0 codes may differ in sign only for exact zeros produced by rounding
    assert np.array_equal(ours & 0x7F, theirs & 0x7F)
    nz = (ours & 0x7F) != 0
    assert np.array_equal(ours[nz], theirs[nz])


def test_act_quant_known_answers():
    x = torch.zeros(3, 256, dtype=torch.bfloat16)
    x[0, :128] = 1.0                      # amax 1 -> scale 1/448, q = 448 everywhere
    x[0, 128] = 448.0                     # scale exactly 1.0
    x[0, 129] = -3.0
    x[1, 5] = -2.0                        # negative amax element
    # row 2 all zero: scale = 1e-10/448, q = 0
    xq, sx = S.quantize_act_group128(x)
    assert sx.shape == (3, 2)
    assert sx[0, 0].item() == np.float32(1.0) / np.float32(448.0)
    assert torch.all(xq[0, :128].float() == 448.0)
    assert sx[0, 1].item() == 1.0 and xq[0, 128].float().item() == 448.0 and xq[0, 129].float().item() == -3.0
    assert xq[1, 5].float().item() == -448.0 and sx[1, 0].item() == np.float32(2.0) / np.float32(448.0)
    assert sx[2, 0].item() == np.float32(1e-10) / np.float32(448.0)
    assert torch.all(xq[2].float() == 0)


def test_weight_quant_known_answers_and_ragged_edges():
    w = torch.zeros(130, 200, dtype=torch.bfloat16)
    w[0, 0] = 0.5
    w[129, 199] = -0.25                   # lives in the ragged corner block (1, 1)
    wq, sw = S.quantize_weight_block128(w)
    assert wq.shape == (130, 200) and sw.shape == (2, 2)
    assert sw[0, 0].item() == np.float32(0.5) / np.float32(448.0)
    assert sw[1, 1].item() == np.float32(0.25) / np.float32(448.0)
    assert wq[0, 0].float().item() == 448.0 and wq[129, 199].float().item() == -448.0
    assert sw[0, 1].item() == np.float32(1e-10) / np.float32(448.0)


@settings(max_examples=40, deadline=None)
@given(m=st.integers(1, 5), k=st.integers(1, 300), scale=st.sampled_from([1e-4, 0.02, 1.0, 37.0, 3e4]),
       seed=st.integers(0, 2 ** 16))
def test_act_quant_properties(m, k, scale, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(m, k, generator=g) * scale).to(torch.bfloat16)
    xq, sx = S.quantize_act_group128(x)
    assert xq.shape == (m, k) and sx.shape == (m, (k + 127) // 128)
    q = xq.float()
    assert not torch.isnan(q).any() and q.abs().max() <= 448.0
    # the amax element of every group maps to +-448 and the scale is amax/448
    xf = x.float()
    for gi in range(sx.shape[1]):
        seg = xf[:, gi * 128:(gi + 1) * 128]
        amax = seg.abs().amax(dim=1)
        assert torch.equal(sx[:, gi], amax.clamp(min=1e-10) / 448.0)
        hit = q[:, gi * 128:(gi + 1) * 128].abs().amax(dim=1)
        assert torch.all((hit == 448.0) | (amax == 0))
    # the numpy encoder agrees with the torch cast used by the quantiser
    s_full = sx.repeat_interleave(128, dim=1)[:, :k]
    again = S.e4m3_encode_rne((xf / s_full).numpy())
    mine = xq.view(torch.uint8).numpy()
    assert np.array_equal(again & 0x7F, mine & 0x7F)
    # dequantisation error is bounded by half an e4m3 step (2^-4 relative) of the group amax
    err = (S.dequantize_act(xq, sx) - xf).abs()
    bound = (sx * 448.0 * 2.0 ** -4).repeat_interleave(128, dim=1)[:, :k] + 1e-30
    assert torch.all(err <= bound)


def test_quantising_representable_values_is_exact():
    """Values already on the e4m3 grid of their group survive a round trip bit-exactly."""
    tab = torch.from_numpy(S.e4m3_decode_table())
    vals = tab[~torch.isnan(tab)]
    g = torch.Generator().manual_seed(1)
    idx = torch.randint(0, vals.numel(), (4, 256), generator=g)
    q0 = vals[idx]
    q0[:, 0] = 448.0
    q0[:, 128] = -448.0                   # pin each group's amax to 448 -> scale = s exactly
    s = torch.tensor([[0.5, 2.0 ** -7]]).expand(4, 2)
    x = (q0 * s.repeat_interleave(128, dim=1)).to(torch.bfloat16)
    assert torch.equal(x.float(), q0 * s.repeat_interleave(128, dim=1))   # representable in bf16
    xq, sx = S.quantize_act_group128(x)
    assert torch.equal(sx, s.contiguous())
    assert torch.equal(xq.float(), q0)


@pytest.mark.parametrize("m,n,k", [(4, 256, 512), (3, 130, 200), (16, 1024, 2048)])
def test_tile_promotion_agrees_with_dequant_matmul(m, n, k):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    b = torch.randn(n, generator=g).to(torch.bfloat16)
    xq, sx = S.quantize_act_group128(x)
    wq, sw = S.quantize_weight_block128(w)
    y0 = S.linear_dequant_matmul(xq, sx, wq, sw, b)
    y1 = S.linear_tile_promotion(xq, sx, wq, sw, b)
    assert S.max_rel_err(y1, y0) <= 4e-3          # same math, fp32 summation order only
    # and quantisation itself costs a few percent against the unquantised layer
    y_unq = torch.nn.functional.linear(x.float(), w.float(), b.float())
    assert 1e-3 < S.max_rel_err(y0, y_unq) < 0.1
