"""FP8 checkpoint ingestion end to end: ``*.safetensors`` files -> loader loop -> drop-in layers.

A synthetic block-FP8 checkpoint of a tiny Qwen3-dense-shaped model (``oracle/synth_checkpoint.py``: separate
q/k/v and gate/up projections as ``weight`` float8_e4m3fn + ``weight_scale_inv`` fp32, unquantised embeddings, norms
and ``lm_head``) is written to disk and loaded through the restatement of nano_qwen's ``load_model``
(``oracle/ref_loader.py``, following ``utils/loader.py:12-28``) into a module tree built from
``nano_qwen_b200.layers``.  Expected placement comes from ``tests/golden/checkpoint_digests.json``: the reference's
own ``load_model`` and modules, run under real gloo ranks on the dequantised variant of the same checkpoint.

CPU part (here): every rank of tp 1/2/4/8 ends up with weights whose dequantised values are bit-equal to the
reference rank's parameters.  GPU part (marked gpu): the loaded layers' forward against the reference modules'
outputs on probe activations.
"""
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import fp8_spec as S, ref_loader, synth, synth_checkpoint as CK

FP8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def checkpoint_dir(tmp_path_factory):
    return CK.write(str(tmp_path_factory.mktemp("ckpt") / "fp8"), seed=0, quantised=True)


@pytest.fixture(scope="module")
def golden_digests():
    with open(os.path.join(GOLDEN, "checkpoint_digests.json")) as f:
        return json.load(f)


def fp32_digest(t: torch.Tensor) -> str:
    return synth.digest(t.float().contiguous().view(torch.uint8))


def check_against_reference_rank(model, gold: dict):
    """Every parameter the reference rank holds is present here with the same values (FP8 weights after dequantisation)."""
    seen = 0
    for name, want in gold.items():
        param = model.get_parameter(name)
        if param.dtype == FP8:
            scales = model.get_parameter(name + "_scale_inv")
            assert scales.dtype == torch.float32
            value = S.dequantize_weight(param.data.cpu(), scales.data.cpu())
        else:
            value = param.data.cpu()
        assert fp32_digest(value) == want, name
        seen += 1
    assert seen == len(gold) and seen >= 4 * CK.LAYERS + 3


def test_checkpoint_files_hold_fp8_weights_and_block_scales(checkpoint_dir):
    from safetensors import safe_open
    files = sorted(os.listdir(checkpoint_dir))
    assert len(files) == 2 and all(f.endswith(".safetensors") for f in files)
    kinds = {}
    for f in files:
        with safe_open(os.path.join(checkpoint_dir, f), "pt", "cpu") as h:
            for k in h.keys():
                kinds[k] = h.get_tensor(k).dtype
    assert kinds["model.layers.0.self_attn.q_proj.weight"] == FP8
    assert kinds["model.layers.1.mlp.down_proj.weight_scale_inv"] == torch.float32
    assert kinds["lm_head.weight"] == torch.bfloat16 and kinds["model.norm.weight"] == torch.bfloat16
    assert not any("qkv_proj" in k or "gate_up_proj" in k for k in kinds)     # packed only inside the model


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_loader_loop_fills_every_rank_like_the_reference(checkpoint_dir, golden_digests, monkeypatch,
                                                         single_rank_group, tp):
    from nano_qwen_b200.layers import linear as L
    for rank in range(tp):
        monkeypatch.setattr(L.dist, "get_rank", lambda *a, **k: rank)
        monkeypatch.setattr(L.dist, "get_world_size", lambda *a, **k: tp)
        model = CK.build_tree(L, rank, tp)
        touched = ref_loader.load_model(model, checkpoint_dir)
        # every parameter of the tree was written at least once, scales included
        assert set(touched) == {n for n, _ in model.named_parameters()}
        qkv = model.model.layers[0].self_attn.qkv_proj
        assert qkv.weight.dtype == FP8 and qkv.weight.shape == ((CK.HEADS + 2 * CK.KV_HEADS) * CK.HEAD_DIM // tp, CK.HIDDEN)
        assert qkv.weight_scale_inv.shape == (qkv.weight.shape[0] // 128, CK.HIDDEN // 128)
        check_against_reference_rank(model, golden_digests[f"tp{tp}"][rank])


def test_resolve_follows_the_packed_mapping():
    assert ref_loader.resolve("model.layers.0.mlp.up_proj.weight_scale_inv", CK.PACKED) == \
        ("model.layers.0.mlp.gate_up_proj.weight_scale_inv", (1,))
    assert ref_loader.resolve("model.layers.1.self_attn.k_proj.weight", CK.PACKED) == \
        ("model.layers.1.self_attn.qkv_proj.weight", ("k",))
    assert ref_loader.resolve("model.layers.1.self_attn.o_proj.weight", CK.PACKED) == \
        ("model.layers.1.self_attn.o_proj.weight", ())
    assert ref_loader.resolve("lm_head.weight", {}) == ("lm_head.weight", ())


@pytest.mark.gpu
def test_loaded_layers_forward_like_the_reference_modules(checkpoint_dir, golden_digests, built_library,
                                                          single_rank_group):
    """tp = 1 on the device: checkpoint -> loader -> CUDA modules -> forward, against the outputs of the reference's
    modules (fp32 on CPU, dequantised operands); <= 2e-2."""
    from nano_qwen_b200 import ops
    from nano_qwen_b200.layers import linear as L
    ops.init()
    torch.set_default_device("cuda")
    torch.set_default_dtype(torch.bfloat16)
    try:
        model = CK.build_tree(L, 0, 1)
    finally:
        torch.set_default_device("cpu")
        torch.set_default_dtype(torch.float32)
    ref_loader.load_model(model, checkpoint_dir)              # CPU tensors from the files are copied into CUDA params
    assert model.model.layers[1].mlp.down_proj.weight.is_cuda
    check_against_reference_rank(model, golden_digests["tp1"][0])
    with np.load(os.path.join(GOLDEN, "checkpoint_probe_tp1.npz")) as gold:
        for name, x in CK.probe_inputs().items():
            y = model.model.get_submodule(name)(x.cuda())
            torch.cuda.synchronize()
            want = torch.from_numpy(gold[f"{name}_r0"]).view(torch.bfloat16)
            assert y.shape == want.shape and y.dtype == torch.bfloat16
            assert S.max_rel_err(y.cpu(), want) <= 2e-2, name
