"""Host logic of the drop-in layers on CPU: constructors, attributes, loaders, error behaviour.

Expected shard placement comes from ``tests/golden/sharding.json`` (recorded
from the reference's own ``weight_loader`` methods under real gloo ranks).
"""
import json
import os

import pytest
import torch

from conftest import GOLDEN
from test_golden_reference import expand

FP8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def sharding():
    with open(os.path.join(GOLDEN, "sharding.json")) as f:
        return json.load(f)


@pytest.fixture()
def fake_tp(monkeypatch, single_rank_group):
    """Makes the layer module see an arbitrary (rank, world size)."""
    from nano_qwen_b200.layers import linear as L

    def set_tp(rank, size):
        monkeypatch.setattr(L.dist, "get_rank", lambda *a, **k: rank)
        monkeypatch.setattr(L.dist, "get_world_size", lambda *a, **k: size)
        return L
    return set_tp


def byte_coded(n, k):
    """A float8 tensor whose bytes identify (row, col) well enough to detect any misplacement."""
    r = torch.arange(n, dtype=torch.int64).unsqueeze(1)
    c = torch.arange(k, dtype=torch.int64).unsqueeze(0)
    b = ((r * 131 + c * 31 + (r // 7) * 3) % 126).to(torch.uint8)     # 0..125: finite, positive
    return b.view(FP8)


def block_coded(nb, kb):
    return (torch.arange(nb, dtype=torch.float32).unsqueeze(1) * 1000 + torch.arange(kb, dtype=torch.float32) + 1)


def block_rows(rows):
    assert len(rows) % 128 == 0
    out = [rows[i] // 128 for i in range(0, len(rows), 128)]
    for i, b in enumerate(out):       # every 128-row group must be one aligned checkpoint block
        assert rows[i * 128] % 128 == 0 and rows[i * 128 + 127] == rows[i * 128] + 127
    return out


def as_bytes(t):
    return t.contiguous().view(torch.uint8)


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_loaders_place_fp8_weights_and_block_scales_like_the_reference(sharding, fake_tp, tp):
    cases = sharding["cases"]
    for rank in range(tp):
        L = fake_tp(rank, tp)
        gold = sharding[f"tp{tp}"][rank]

        # ---- column ----
        c = cases["column"]
        m = L.ColumnParallelLinear(c["K"], c["N"], bias=True)
        w, s = byte_coded(c["N"], c["K"]), block_coded(c["N"] // 128, c["K"] // 128)
        m.weight.weight_loader(m.weight, w)
        m.weight_scale_inv.weight_loader(m.weight_scale_inv, s)
        m.bias.weight_loader(m.bias, torch.arange(c["N"], dtype=torch.float32))
        g = gold["column"]["weight"]
        rows, cols = expand(g["rows"]), expand(g["cols"])
        assert list(m.weight.shape) == g["shape"] and m.weight.dtype == FP8
        assert torch.equal(as_bytes(m.weight.data), as_bytes(w)[rows][:, cols])
        assert torch.equal(m.weight_scale_inv.data, s[block_rows(rows)])
        assert m.bias.data.tolist() == expand(gold["column"]["bias"]["rows"])
        assert (m.tp_dim, m.tp_rank, m.tp_size) == (0, rank, tp)

        # ---- merged (gate_up) ----
        c = cases["merged"]
        m = L.MergedColumnParallelLinear(c["K"], c["sizes"])
        n_all = sum(c["sizes"])
        w, s = byte_coded(n_all, c["K"]), block_coded(n_all // 128, c["K"] // 128)
        off = 0
        for i, sz in enumerate(c["sizes"]):
            m.weight.weight_loader(m.weight, w[off:off + sz], i)
            m.weight_scale_inv.weight_loader(m.weight_scale_inv, s[off // 128:(off + sz) // 128], i)
            off += sz
        g = gold["merged"]["weight"]
        rows, cols = expand(g["rows"]), expand(g["cols"])
        assert list(m.weight.shape) == g["shape"] and m.output_sizes == c["sizes"] and m.bias is None
        assert torch.equal(as_bytes(m.weight.data), as_bytes(w)[rows][:, cols])
        assert torch.equal(m.weight_scale_inv.data, s[block_rows(rows)])

        # ---- qkv ----
        c = cases["qkv"]
        m = L.QKVParallelLinear(c["K"], c["head"], c["heads"], c["kv"])
        nq, nk = c["heads"] * c["head"], c["kv"] * c["head"]
        w, s = byte_coded(nq + 2 * nk, c["K"]), block_coded((nq + 2 * nk) // 128, c["K"] // 128)
        for sid, lo, hi in (("q", 0, nq), ("k", nq, nq + nk), ("v", nq + nk, nq + 2 * nk)):
            m.weight.weight_loader(m.weight, w[lo:hi], sid)
            m.weight_scale_inv.weight_loader(m.weight_scale_inv, s[lo // 128:hi // 128], sid)
        g = gold["qkv"]["weight"]
        rows, cols = expand(g["rows"]), expand(g["cols"])
        assert torch.equal(as_bytes(m.weight.data), as_bytes(w)[rows][:, cols])
        assert torch.equal(m.weight_scale_inv.data, s[block_rows(rows)])
        assert (m.head_size, m.num_heads, m.num_kv_heads) == (c["head"], gold["qkv"]["num_heads"], gold["qkv"]["num_kv_heads"])
        with pytest.raises(AssertionError):
            m.weight.weight_loader(m.weight, w[:nq], "x")

        # ---- row ----
        c = cases["row"]
        m = L.RowParallelLinear(c["K"], c["N"], bias=True)
        w, s = byte_coded(c["N"], c["K"]), block_coded(c["N"] // 128, c["K"] // 128)
        m.weight.weight_loader(m.weight, w)
        m.weight_scale_inv.weight_loader(m.weight_scale_inv, s)
        m.bias.weight_loader(m.bias, torch.arange(c["N"], dtype=torch.float32))
        g = gold["row"]["weight"]
        rows, cols = expand(g["rows"]), expand(g["cols"])
        assert list(m.weight.shape) == g["shape"]
        assert torch.equal(as_bytes(m.weight.data), as_bytes(w)[rows][:, cols])
        assert cols[0] % 128 == 0 and len(cols) % 128 == 0
        assert torch.equal(m.weight_scale_inv.data, s[:, cols[0] // 128:(cols[0] + len(cols)) // 128])
        assert m.bias.data.tolist() == expand(gold["row"]["bias"]["rows"])      # bias is replicated
        assert (m.tp_dim, m.tp_rank, m.tp_size) == (1, rank, tp)

        # ---- replicated ----
        c = cases["replicated"]
        m = L.ReplicatedLinear(c["K"], c["N"], bias=True)
        w = byte_coded(c["N"], c["K"])
        m.weight.weight_loader(m.weight, w)
        assert torch.equal(as_bytes(m.weight.data), as_bytes(w)) and m.tp_dim is None


def test_constructor_rejects_non_divisible_tp(fake_tp):
    L = fake_tp(0, 3)
    with pytest.raises(AssertionError):
        L.ColumnParallelLinear(256, 1024)
    with pytest.raises(AssertionError):
        L.RowParallelLinear(1024, 256)
    with pytest.raises(AssertionError):
        L.QKVParallelLinear(256, 128, 16, 8)


def test_misaligned_scale_shards_are_rejected(fake_tp):
    L = fake_tp(1, 2)
    m = L.ColumnParallelLinear(256, 384)          # 192 rows per rank: block scales would straddle ranks
    with pytest.raises(AssertionError, match="aligned"):
        m.weight_scale_inv.weight_loader(m.weight_scale_inv, torch.ones(3, 2))


def test_parameters_follow_the_loader_protocol(fake_tp):
    """Every loadable parameter is reachable by name and carries ``weight_loader`` (nano_qwen utils/loader.py:20-28)."""
    L = fake_tp(0, 1)
    m = torch.nn.ModuleDict({"qkv_proj": L.QKVParallelLinear(256, 128, 4, 2, bias=True),
                             "down_proj": L.RowParallelLinear(200, 256)})       # K not a multiple of 16
    for name in ("qkv_proj.weight", "qkv_proj.weight_scale_inv", "qkv_proj.bias", "down_proj.weight",
                 "down_proj.weight_scale_inv"):
        p = m.get_parameter(name)
        assert callable(p.weight_loader) and not p.requires_grad
    assert m["down_proj"].bias is None
    w = m["down_proj"].weight
    assert w.shape == (256, 200) and w.stride(0) % 16 == 0        # row stride padded for TMA
    assert m["down_proj"].weight_scale_inv.shape == (2, 2)


def test_forward_on_cpu_raises_instead_of_falling_back(fake_tp):
    L = fake_tp(0, 1)
    m = L.ColumnParallelLinear(128, 128)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        m(torch.zeros(2, 128, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        m.weight.weight_loader(m.weight, torch.zeros(128, 128, dtype=torch.bfloat16))   # quantise-on-load needs CUDA
