"""The allocation-free linear entry point against the ordinary one (collected last on purpose).

``nq_fp8_linear_noalloc`` serves hosts that cannot give the library scratch memory: it keeps the quantised
activations in a fixed array inside the library image.  Here it is called twice in a row through the C ABI,
with different inputs, and each result is compared with ``nq_fp8_linear`` (caller-allocated scratch) on the
same inputs and with the CPU oracle.  The second call checks that nothing left in the shared array by the first one leaks into it.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

PARITY = 2e-2     # the tolerance of the other GEMM tests; the two entry points run the same kernels


@pytest.fixture(scope="module")
def lib(built_library):
    from nano_qwen_b200 import _cabi, ops
    ops.init()
    return _cabi.lib()


def _call_noalloc(lib, x, wq, sw, bias, y):
    from nano_qwen_b200 import _cabi
    m, k = x.shape
    n = wq.shape[0]
    st = lib.nq_fp8_linear_noalloc(x.data_ptr(), x.stride(0), wq.data_ptr(), wq.stride(0), sw.data_ptr(), sw.stride(0),
                                   None if bias is None else bias.data_ptr(), y.data_ptr(), y.stride(0), m, n, k,
                                   0, 0, torch.cuda.current_stream().cuda_stream)
    _cabi.check(st, "nq_fp8_linear_noalloc")


def test_noalloc_entry_matches_the_ordinary_one_twice_in_a_row(lib):
    from nano_qwen_b200 import ops
    from oracle import fp8_spec as S
    gen = torch.Generator(device="cuda").manual_seed(99)
    n, k = 1024, 2048
    w = (torch.randn(n, k, generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    wq, sw = ops.weight_quant(w)
    bias = torch.randn(n, generator=gen, device="cuda").to(torch.bfloat16)
    for m, use_bias in ((200, True), (24, False)):          # second call: fewer tokens than the first left behind
        x = torch.randn(m, k, generator=gen, device="cuda").to(torch.bfloat16)
        expect = ops.fp8_linear(x, wq, sw, bias if use_bias else None)
        y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        _call_noalloc(lib, x, wq, sw, bias if use_bias else None, y)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before       # the call took nothing from the allocator
        assert not torch.isnan(y.float()).any()
        assert S.max_rel_err(y.cpu(), expect.cpu()) <= PARITY
        assert torch.equal(y, expect)                        # same kernels, same scratch contents: same bits
        # and against the CPU oracle (dequantise both operands, fp32 matmul, bf16 out), not only against the sibling entry
        xq_ref, sx_ref = S.quantize_act_group128(x.cpu())
        ref = S.linear_dequant_matmul(xq_ref, sx_ref, wq.cpu(), sw.cpu(), bias.cpu() if use_bias else None)
        assert S.max_rel_err(y.cpu(), ref) <= PARITY


def test_noalloc_entry_refuses_sizes_beyond_its_array(lib):
    k = 4096
    m = (8 << 20) // k + 1                                   # one token too many for the 8 MiB of e4m3 bytes
    x = torch.zeros(m, k, dtype=torch.bfloat16, device="cuda")
    wq = torch.zeros(128, k, dtype=torch.uint8, device="cuda")
    sw = torch.ones(1, k // 128, device="cuda")
    y = torch.zeros(m, 128, dtype=torch.bfloat16, device="cuda")
    st = lib.nq_fp8_linear_noalloc(x.data_ptr(), k, wq.data_ptr(), k, sw.data_ptr(), k // 128, None, y.data_ptr(), 128,
                                   m, 128, k, 0, 0, None)
    assert st == -3                                          # NQ_ERR_WORKSPACE, nothing launched
    assert lib.nq_status_string(st).startswith(b"workspace")
