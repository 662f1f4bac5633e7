"""CPU restatement of nano_qwen's checkpoint loading loop.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  In a deployment the caller of the drop-in layers'
``weight_loader`` methods is the reference's own ``load_model`` (``src/nano_qwen/utils/loader.py:12-28``), which
stays as it is.  The reference is not present where the GPU tests run, so the tests drive the layers with this
restatement of that loop instead.  It is checked against the real ``load_model`` by the fixture script
(``tests/golden/make_golden.py``): both load the same synthetic checkpoint and must place the same bytes.

What the loop does, per tensor of every ``*.safetensors`` file under ``path`` (opened on the CPU):

* if a key of ``model.packed_modules_mapping`` occurs in the tensor's name (first match in dictionary order,
  ``loader.py:17-24``), the name is rewritten (key -> packed parameter's module name), the parameter is looked up
  with ``model.get_parameter`` and its ``weight_loader(param, tensor, shard_id)`` is called;
* otherwise (``loader.py:25-28``) the parameter of that very name gets ``weight_loader(param, tensor)``, or a plain
  ``param.data.copy_(tensor)`` when it carries no loader (``default_weight_loader``, ``loader.py:8-9``).

The same substring rule covers ``<module>.weight_scale_inv`` tensors of FP8 block checkpoints: ``q_proj`` occurs in
``...q_proj.weight_scale_inv`` too, so the scale tensor reaches ``qkv_proj.weight_scale_inv`` with shard id ``"q"``.
"""
from __future__ import annotations

import glob
import os

import torch
from safetensors import safe_open
from torch import nn


def plain_copy(param: nn.Parameter, tensor: torch.Tensor) -> None:
    """What a parameter without a ``weight_loader`` attribute gets (``loader.py:8-9``)."""
    param.data.copy_(tensor)


def resolve(name: str, packed: dict) -> tuple[str, tuple]:
    """Parameter name and extra loader arguments for a checkpoint tensor name (``loader.py:17-26``)."""
    for key, (target, shard_id) in packed.items():
        if key in name:
            return name.replace(key, target), (shard_id,)
    return name, ()


def load_model(model: nn.Module, path: str) -> list[str]:
    """Feeds every tensor of the checkpoint directory to its parameter's loader; returns the parameter names hit."""
    packed = getattr(model, "packed_modules_mapping", {})
    touched = []
    for file in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        with safe_open(file, "pt", "cpu") as f:
            for name in f.keys():
                param_name, extra = resolve(name, packed)
                param = model.get_parameter(param_name)
                loader = getattr(param, "weight_loader", plain_copy) if not extra else param.weight_loader
                loader(param, f.get_tensor(name), *extra)
                touched.append(param_name)
    return touched
