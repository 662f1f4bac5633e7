"""The oracle against fixtures produced by the reference's own modules (CPU).

``tests/golden/*.json|npz`` were written by ``tests/golden/make_golden.py``,
which drives nano_qwen's ``layers/linear.py`` classes; nothing here reads the
reference at run time.
"""
import json
import os

import numpy as np
import pytest
import torch

from oracle import fp8_spec as S, ref_linear as R, synth
from conftest import GOLDEN


def expand(segs):
    out = []
    for dst, src, n in segs:
        assert dst == len(out)
        out.extend(range(src, src + n))
    return out


@pytest.fixture(scope="module")
def sharding():
    with open(os.path.join(GOLDEN, "sharding.json")) as f:
        return json.load(f)


def index_coded(n, k):
    return torch.arange(n, dtype=torch.float32).unsqueeze(1) * k + torch.arange(k, dtype=torch.float32)


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_oracle_sharding_matches_reference_loaders(sharding, tp):
    cases = sharding["cases"]
    for rank in range(tp):
        gold = sharding[f"tp{tp}"][rank]
        c = cases["column"]
        full = index_coded(c["N"], c["K"])
        mine = R.column_shard(full, rank, tp)
        g = gold["column"]["weight"]
        assert list(mine.shape) == g["shape"]
        assert torch.equal(mine, full[expand(g["rows"])][:, expand(g["cols"])])
        assert R.column_shard(torch.arange(c["N"]), rank, tp).tolist() == expand(gold["column"]["bias"]["rows"])

        c = cases["merged"]
        full = index_coded(sum(c["sizes"]), c["K"])
        parts = list(full.split(c["sizes"], 0))
        g = gold["merged"]["weight"]
        assert torch.equal(R.merged_column_param(parts, rank, tp), full[expand(g["rows"])][:, expand(g["cols"])])

        c = cases["qkv"]
        nq, nk = c["heads"] * c["head"], c["kv"] * c["head"]
        full = index_coded(nq + 2 * nk, c["K"])
        g = gold["qkv"]["weight"]
        mine = R.qkv_param(full[:nq], full[nq:nq + nk], full[nq + nk:], rank, tp)
        assert torch.equal(mine, full[expand(g["rows"])][:, expand(g["cols"])])
        assert R.qkv_output_size(c["head"], c["heads"], c["kv"]) == nq + 2 * nk
        assert gold["qkv"]["num_heads"] == R.divide(c["heads"], tp)

        c = cases["row"]
        full = index_coded(c["N"], c["K"])
        g = gold["row"]["weight"]
        assert torch.equal(R.row_shard(full, rank, tp), full[expand(g["rows"])][:, expand(g["cols"])])
        assert R.row_shard(torch.arange(c["N"]), rank, tp).tolist() == expand(gold["row"]["bias"]["rows"])


def test_divide_rejects_non_divisible():
    assert R.divide(12, 4) == 3
    with pytest.raises(AssertionError):
        R.divide(10, 4)


@pytest.fixture(scope="module")
def stack06():
    weights, acts = synth.make_stack("qwen3-0.6b", 16, seed=0)
    q = {}
    for name in synth.LAYER_ORDER:
        wq, sw = S.quantize_weight_block128(weights[name])
        xq, sx = S.quantize_act_group128(acts[name])
        q[name] = (xq, sx, wq, sw)
    return weights, acts, q


def test_seeded_inputs_reproduce(stack06):
    weights, acts, q = stack06
    with np.load(os.path.join(GOLDEN, "linear_tp1.npz")) as z:
        for name in synth.LAYER_ORDER:
            assert synth.digest(weights[name].view(torch.int16)) == str(z[f"sha_w_{name}"])
            assert synth.digest(acts[name].view(torch.int16)) == str(z[f"sha_x_{name}"])
            assert synth.digest(q[name][2].view(torch.uint8)) == str(z[f"sha_wq_{name}"])
            assert synth.digest(q[name][0].view(torch.uint8)) == str(z[f"sha_xq_{name}"])


def test_oracle_linear_matches_reference_forward_tp1(stack06):
    """Dequantise-then-``F.linear`` equals what the reference's modules returned."""
    _, _, q = stack06
    with np.load(os.path.join(GOLDEN, "linear_tp1.npz")) as z:
        for name in synth.LAYER_ORDER:
            gold = torch.from_numpy(z[f"y_{name}_r0"]).view(torch.bfloat16)
            mine = S.linear_dequant_matmul(*q[name])
            assert mine.shape == gold.shape
            assert S.max_rel_err(mine, gold) <= 2e-3, name       # same op; CPU BLAS blocking may differ
            assert S.max_rel_err(S.linear_tile_promotion(*q[name]), gold) <= 5e-3, name


def test_oracle_tp2_matches_reference_forward(stack06):
    """Column shards concatenate per rank; row shards sum (the reference ran these under 2 gloo ranks)."""
    _, _, q = stack06
    shapes = synth.STACKS["qwen3-0.6b"]
    with np.load(os.path.join(GOLDEN, "linear_tp2.npz")) as z:
        for rank in range(2):
            xq, sx, wq, sw = q["qkv"]
            wd, xd = S.dequantize_weight(wq, sw), S.dequantize_act(xq, sx)
            nq = shapes["qkv"][1] - 2048
            w_r = R.qkv_param(wd[:nq], wd[nq:nq + 1024], wd[nq + 1024:], rank, 2)
            gold = torch.from_numpy(z[f"y_qkv_r{rank}"]).view(torch.bfloat16)
            assert S.max_rel_err(R.column_forward(xd, w_r).to(torch.bfloat16), gold) <= 2e-3

            xq, sx, wq, sw = q["gate_up"]
            wd, xd = S.dequantize_weight(wq, sw), S.dequantize_act(xq, sx)
            half = shapes["gate_up"][1] // 2
            w_r = R.merged_column_param([wd[:half], wd[half:]], rank, 2)
            gold = torch.from_numpy(z[f"y_gate_up_r{rank}"]).view(torch.bfloat16)
            assert S.max_rel_err(R.column_forward(xd, w_r).to(torch.bfloat16), gold) <= 2e-3

            for name in ("o_proj", "down"):
                xq, sx, wq, sw = q[name]
                wd, xd = S.dequantize_weight(wq, sw), S.dequantize_act(xq, sx)
                gold = torch.from_numpy(z[f"y_{name}_r{rank}"]).view(torch.bfloat16)
                assert S.max_rel_err(R.row_forward(xd, wd, None, 2).to(torch.bfloat16), gold) <= 2e-3
