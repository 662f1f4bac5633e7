"""The CPU restatement of SiluAndMul / RMSNorm / GemmaRMSNorm against the reference modules' own outputs
(``tests/golden/fused_ops.npz``, made by ``tests/golden/make_golden.py``): bit for bit."""
import os

import numpy as np
import torch

from conftest import GOLDEN
from oracle import ref_fused as R


def _load():
    with np.load(os.path.join(GOLDEN, "fused_ops.npz")) as z:
        return {k: torch.from_numpy(z[k].copy()).view(torch.bfloat16) for k in z.files}


def test_silu_and_mul_equals_reference_module():
    g = _load()
    assert torch.equal(R.silu_and_mul(g["silu_in"]).view(torch.int16), g["silu_out"].view(torch.int16))


def test_rms_norms_equal_reference_modules():
    g = _load()
    for name, gemma in (("rms", False), ("gemma", True)):
        out = R.rms_norm(g["norm_x"], g[name + "_w"], 1e-6, None, gemma)
        assert torch.equal(out.view(torch.int16), g[name + "_out"].view(torch.int16)), name
        out, res = R.rms_norm(g["norm_x"], g[name + "_w"], 1e-6, g["norm_res"], gemma)
        assert torch.equal(out.view(torch.int16), g[name + "_add_out"].view(torch.int16)), name
        assert torch.equal(res.view(torch.int16), g[name + "_add_res"].view(torch.int16)), name


def test_eager_mode_is_the_reference_arithmetic_and_fp8_mode_has_no_cpu_fallback():
    """``emit_fp8=False`` is the reference's eager op (bit-equal to its modules' outputs); ``emit_fp8=True`` belongs to
    the FP8 path and refuses anything but a CUDA bf16 tensor instead of quietly computing something else."""
    import pytest
    from nano_qwen_b200.layers.activation import SiluAndMul
    from nano_qwen_b200.layers.layernorm import GemmaRMSNorm, RMSNorm
    g = _load()
    assert torch.equal(SiluAndMul(emit_fp8=False)(g["silu_in"]).view(torch.int16), g["silu_out"].view(torch.int16))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        SiluAndMul()(g["silu_in"])
    for name, cls in (("rms", RMSNorm), ("gemma", GemmaRMSNorm)):
        mod = cls(1024, eps=1e-6).to(torch.bfloat16)
        mod.weight.data.copy_(g[name + "_w"])
        out, res = mod(g["norm_x"], g["norm_res"])
        assert torch.equal(out.view(torch.int16), g[name + "_add_out"].view(torch.int16)), name
        assert torch.equal(res.view(torch.int16), g[name + "_add_res"].view(torch.int16)), name
        fp8_mod = cls(1024, eps=1e-6, emit_fp8=True).to(torch.bfloat16)
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            fp8_mod(g["norm_x"], g["norm_res"])
