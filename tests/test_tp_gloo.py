"""Tensor-parallel host logic under real multi-rank gloo groups on CPU.

The CUDA kernels cannot run here, so the ONE call into them
(``LinearBase._linear``) is replaced, inside these tests only, by the oracle's
evaluation of the same FP8 linear.  What is under test is everything around
it: construction under a real world size, shard loading, bias-on-rank-0 and
the row-parallel all-reduce, checked against the reference's own 2-rank run
(``tests/golden/linear_tp2.npz``).
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import GOLDEN, ROOT, free_port


def _oracle_linear(self, x, bias):
    from oracle import fp8_spec as S
    xq, sx = S.quantize_act_group128(x.to(torch.bfloat16))
    return S.linear_tile_promotion(xq, sx, self.weight.data, self.weight_scale_inv.data,
                                   None if bias is None else bias.data)


def _worker(rank, world, port, out_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nano_qwen_b200.layers import linear as L
        from oracle import fp8_spec as S, synth
        L.LinearBase._linear = _oracle_linear
        weights, acts = synth.make_stack("qwen3-0.6b", 16, seed=0)
        shapes = synth.STACKS["qwen3-0.6b"]
        q = {n: S.quantize_weight_block128(weights[n]) for n in synth.LAYER_ORDER}
        res = {}

        K, N = shapes["qkv"]
        qkv = L.QKVParallelLinear(K, 128, N // 128 - 16, 8)
        wq, sw = q["qkv"]
        nq = N - 2048
        for sid, lo, hi in (("q", 0, nq), ("k", nq, nq + 1024), ("v", nq + 1024, N)):
            qkv.weight.weight_loader(qkv.weight, wq[lo:hi], sid)
            qkv.weight_scale_inv.weight_loader(qkv.weight_scale_inv, sw[lo // 128:hi // 128], sid)
        res["qkv"] = qkv(acts["qkv"])

        K, N = shapes["gate_up"]
        gu = L.MergedColumnParallelLinear(K, [N // 2, N // 2])
        wq, sw = q["gate_up"]
        for i in range(2):
            gu.weight.weight_loader(gu.weight, wq[i * N // 2:(i + 1) * N // 2], i)
            gu.weight_scale_inv.weight_loader(gu.weight_scale_inv, sw[i * N // 256:(i + 1) * N // 256], i)
        res["gate_up"] = gu(acts["gate_up"])

        for name in ("o_proj", "down"):
            K, N = shapes[name]
            row = L.RowParallelLinear(K, N, bias=True)
            wq, sw = q[name]
            row.weight.weight_loader(row.weight, wq)
            row.weight_scale_inv.weight_loader(row.weight_scale_inv, sw)
            row.bias.weight_loader(row.bias, torch.full((N,), 0.5))
            ks = K // world
            res[name] = row(acts[name][:, rank * ks:(rank + 1) * ks].contiguous())
        np.savez(out_path.format(rank=rank), **{k: v.to(torch.bfloat16).view(torch.int16).numpy() for k, v in res.items()})
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_rank_layers_match_the_reference_two_rank_run(tmp_path):
    from oracle import fp8_spec as S
    out = str(tmp_path / "r{rank}.npz")
    mp.spawn(_worker, args=(2, free_port(), out), nprocs=2, join=True)
    with np.load(os.path.join(GOLDEN, "linear_tp2.npz")) as gold:
        got = [np.load(out.format(rank=r)) for r in range(2)]
        for r in range(2):
            for name in ("qkv", "gate_up"):
                mine = torch.from_numpy(got[r][name]).view(torch.bfloat16)
                ref = torch.from_numpy(gold[f"y_{name}_r{r}"]).view(torch.bfloat16)
                assert mine.shape == ref.shape
                assert S.max_rel_err(mine, ref) <= 5e-3, (name, r)
            for name in ("o_proj", "down"):
                mine = torch.from_numpy(got[r][name]).view(torch.bfloat16)
                ref = torch.from_numpy(gold[f"y_{name}_r{r}"]).view(torch.bfloat16).float() + 0.5   # bias once, not twice
                assert S.max_rel_err(mine, ref.to(torch.bfloat16)) <= 1e-2, (name, r)
        # all-reduce: both ranks hold the same reduced tensor
        for name in ("o_proj", "down"):
            assert np.array_equal(got[0][name], got[1][name])


def _absent_rank_worker(rank, world, port, out_path):
    """Rank 1 never reaches the row-parallel forward; rank 0 must learn of it on the host and carry on."""
    import datetime
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from nano_qwen_b200.layers import linear as L
    L.LinearBase._linear = _oracle_linear
    row = L.RowParallelLinear(256, 128)
    row.weight.weight_loader(row.weight, torch.zeros(128, 256).to(torch.float8_e4m3fn))
    dist.barrier()                                   # both ranks are up: the failure happens between steps
    if rank == 1:
        time.sleep(8)                                # stays away for longer than the group's time limit, then leaves
        os._exit(0)
    t0 = time.perf_counter()
    try:
        row(torch.ones(4, 128))
        verdict = "no error"
    except RuntimeError as e:                        # the collective's time limit ends the wait with an error
        verdict = "timeout reported" if time.perf_counter() - t0 < 7.5 else "late: " + str(e)[:80]
    with open(out_path, "w") as f:
        f.write(verdict)
    os._exit(0)                                      # the group is broken: leave without the collective teardown


@pytest.mark.timeout(120)
def test_a_rank_that_never_arrives_is_reported_on_the_host(tmp_path):
    """Failure detection without a GPU fault: the peer is lost between steps, the survivor's next all-reduce ends
    with an error inside the process group's time limit instead of waiting for ever."""
    out = str(tmp_path / "verdict.txt")
    mp.spawn(_absent_rank_worker, args=(2, free_port(), out), nprocs=2, join=True)
    assert open(out).read() == "timeout reported"
