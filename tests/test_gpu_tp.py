"""Tensor-parallel layers on 2 GPUs with NCCL against the reference's own 2-rank run (skipped on 1-GPU boxes)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import GOLDEN, ROOT, free_port

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nano_qwen_b200 import ops
        from nano_qwen_b200.layers import linear as L
        from oracle import fp8_spec as S, synth
        ops.init()
        weights, acts = synth.make_stack("qwen3-0.6b", 16, seed=0)
        shapes = synth.STACKS["qwen3-0.6b"]
        q = {n: S.quantize_weight_block128(weights[n]) for n in synth.LAYER_ORDER}
        torch.set_default_device("cuda")
        torch.set_default_dtype(torch.bfloat16)
        K, N = shapes["qkv"]
        qkv = L.QKVParallelLinear(K, 128, N // 128 - 16, 8)
        K, N = shapes["gate_up"]
        gu = L.MergedColumnParallelLinear(K, [N // 2, N // 2])
        rows = {name: L.RowParallelLinear(*shapes[name]) for name in ("o_proj", "down")}
        torch.set_default_device("cpu")
        torch.set_default_dtype(torch.float32)
        res = {}
        wq, sw = q["qkv"]
        N = shapes["qkv"][1]
        nq = N - 2048
        for sid, lo, hi in (("q", 0, nq), ("k", nq, nq + 1024), ("v", nq + 1024, N)):
            qkv.weight.weight_loader(qkv.weight, wq[lo:hi], sid)
            qkv.weight_scale_inv.weight_loader(qkv.weight_scale_inv, sw[lo // 128:hi // 128], sid)
        res["qkv"] = qkv(acts["qkv"].cuda())
        wq, sw = q["gate_up"]
        N = shapes["gate_up"][1]
        for i in range(2):
            gu.weight.weight_loader(gu.weight, wq[i * N // 2:(i + 1) * N // 2], i)
            gu.weight_scale_inv.weight_loader(gu.weight_scale_inv, sw[i * N // 256:(i + 1) * N // 256], i)
        res["gate_up"] = gu(acts["gate_up"].cuda())
        for name, row in rows.items():
            wq, sw = q[name]
            row.weight.weight_loader(row.weight, wq)
            row.weight_scale_inv.weight_loader(row.weight_scale_inv, sw)
            ks = shapes[name][0] // world
            x = acts[name][:, rank * ks:(rank + 1) * ks].contiguous().cuda()
            res[name] = row(x)
            # the same call captured in a CUDA graph (the all-reduce included), as the model runner does for decode
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                row(x)
            torch.cuda.current_stream().wait_stream(side)
            with torch.cuda.graph(g):
                yg = row(x)
            g.replay()
            torch.cuda.synchronize()
            res[name + "_graph"] = yg.clone()
            del g, yg                                       # a graph holding an NCCL collective pins the communicator
        # chunked GEMM / all-reduce pipeline of prefill-sized batches against the single-shot path
        big = torch.randn(4096, shapes["down"][0] // world, generator=torch.Generator().manual_seed(5 + rank)).to(torch.bfloat16).cuda()
        row = rows["down"]
        single = row(big)
        row.overlap_chunks = 2
        piped = row(big)
        torch.cuda.synchronize()
        # same sums up to fp32 summation order (the chunked launches may split K differently)
        err = (piped.float() - single.float()).abs().max() / single.float().abs().max()
        res["pipelined_close_to_single"] = (err <= 8e-3).to(torch.int16).reshape(1)
        # ---- Qwen3-32B-shaped row layer (down_proj, K = 25600 split over the ranks) against the unsharded product ----
        K32, N32 = synth.STACKS["qwen3-32b"]["down"]
        g32 = torch.Generator(device="cuda").manual_seed(4242)            # same seed on every rank: same tensors
        w32 = (torch.randn(N32, K32, generator=g32, device="cuda") * 0.02).to(torch.bfloat16)
        wq32, sw32 = ops.weight_quant(w32)
        del w32
        torch.set_default_device("cuda")
        torch.set_default_dtype(torch.bfloat16)
        row32 = L.RowParallelLinear(K32, N32)
        torch.set_default_device("cpu")
        torch.set_default_dtype(torch.float32)
        row32.weight.weight_loader(row32.weight, wq32)
        row32.weight_scale_inv.weight_loader(row32.weight_scale_inv, sw32)
        ok32 = 1
        for m32 in (1, 64, 2048):
            x32 = torch.randn(m32, K32, generator=g32, device="cuda").to(torch.bfloat16)
            full = ops.fp8_linear(x32, wq32, sw32)                         # one GPU, whole K
            ks = K32 // world
            part = row32(x32[:, rank * ks:(rank + 1) * ks].contiguous())   # this rank's K-slice + the sum over ranks
            torch.cuda.synchronize()
            err = float((part.float() - full.float()).abs().max() / full.float().abs().max())
            ok32 &= int(err <= 8e-3)                                       # partials are rounded to bf16 before the sum
        res["row_32b_matches_unsharded"] = torch.tensor([ok32], dtype=torch.int16)
        del row32, wq32, sw32
        # ---- the peer-memory sum (decode-sized outputs) against NCCL's all-reduce ----
        from nano_qwen_b200.layers import p2p_reduce
        from nano_qwen_b200 import _cabi
        reducer = p2p_reduce.get_reducer()
        assert reducer is not None, "the row layers above should have created the peer-memory reducer"
        gen = torch.Generator(device="cuda").manual_seed(100 + rank)
        worst = 0.0
        for it, n in enumerate([8, 1024, 16 * 1024, 64 * 4096, 256 * 4096, 8 * 5120, 40, 64 * 4096]):
            # back-to-back calls of changing size, nothing but the kernels' own handshake between them
            t = torch.randn(n, generator=gen, device="cuda").to(torch.bfloat16)
            want = t.clone()
            dist.all_reduce(want)
            assert reducer.fits(t), n
            got_t = reducer.reduce_(t.clone())
            worst = max(worst, float((got_t.float() - want.float()).abs().max() / want.float().abs().max()))
        res["p2p_vs_nccl_ok"] = torch.tensor([1 if worst <= 2 ** -7 else 0], dtype=torch.int16)
        # a graph that holds nothing but one row layer, replayed with fresh inputs: the call counter lives on the device
        row = rows["o_proj"]
        xs = torch.zeros(16, shapes["o_proj"][0] // world, dtype=torch.bfloat16, device="cuda")
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            row(xs)
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(g):
            yg = row(xs)
        replay_ok = 1
        for it in range(6):
            xs.copy_(torch.randn(xs.shape, generator=gen, device="cuda").to(torch.bfloat16))
            g.replay()
            row.p2p_reduce = False
            ref = row(xs)                                   # eager GEMM + NCCL
            row.p2p_reduce = True
            torch.cuda.synchronize()
            err = float((yg.float() - ref.float()).abs().max() / ref.float().abs().max())
            replay_ok &= int(err <= 2 ** -7)
        res["p2p_graph_replays_ok"] = torch.tensor([replay_ok], dtype=torch.int16)
        res["p2p_result_for_rank_equality"] = yg.clone().reshape(-1)
        del g, yg
        torch.cuda.synchronize()
        res["device_status"] = torch.tensor([_cabi.device_status()["code"]], dtype=torch.int16)
        np.savez(out_path.format(rank=rank), **{k: v.cpu().view(torch.int16).numpy() for k, v in res.items()})
        dist.barrier()
    except BaseException:
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
        os._exit(1)
    # leave without the communicator teardown (it can block behind captured collectives)
    sys.stdout.flush()
    os._exit(0)


@pytest.mark.timeout(300)
def test_two_gpu_layers_match_the_reference_two_rank_run(tmp_path, built_library):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from oracle import fp8_spec as S
    out = str(tmp_path / "r{rank}.npz")
    mp.spawn(_worker, args=(2, free_port(), out), nprocs=2, join=True)
    with np.load(os.path.join(GOLDEN, "linear_tp2.npz")) as gold:
        got = [np.load(out.format(rank=r)) for r in range(2)]
        for r in range(2):
            for name in ("qkv", "gate_up", "o_proj", "down"):
                mine = torch.from_numpy(got[r][name]).view(torch.bfloat16)
                ref = torch.from_numpy(gold[f"y_{name}_r{r}"]).view(torch.bfloat16)
                assert S.max_rel_err(mine, ref) <= 2e-2, (name, r)
            for name in ("o_proj", "down"):
                assert np.array_equal(got[r][name], got[r][name + "_graph"]), name     # graph replay == eager
            assert int(got[r]["pipelined_close_to_single"][0]) == 1
            assert int(got[r]["row_32b_matches_unsharded"][0]) == 1
            assert int(got[r]["p2p_vs_nccl_ok"][0]) == 1
            assert int(got[r]["p2p_graph_replays_ok"][0]) == 1
            assert int(got[r]["device_status"][0]) == 0
        assert np.array_equal(got[0]["p2p_result_for_rank_equality"], got[1]["p2p_result_for_rank_equality"])
        for name in ("o_proj", "down"):
            assert np.array_equal(got[0][name], got[1][name])                          # both ranks hold the sum
