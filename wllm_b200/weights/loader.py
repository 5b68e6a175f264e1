"""Weights from safetensors, by tensor name.

The model says which tensors it reads (name, shape, kind); the folder's
`*.safetensors` files say which they hold.  Before anything is copied the two lists
are compared, and one `WeightError` names every missing tensor, every unexpected
one and every wrong shape.  The reference raises on missing and unexpected names
after loading everything into host memory (src/wllm/models/llama.py:640-649); here
tensors are read one at a time and go straight to the device.

Element types: matrices and tables are held in the model's type (bfloat16 serving,
float32 for the true 32-bit path).  A vector (norm gain) that the file stores in
32-bit stays 32-bit under either; other vectors follow the model's type.  Integer
tensors become int32.
"""
from __future__ import annotations

import glob
import os

import torch
from safetensors import safe_open

_SAFE_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
                "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8}


class WeightError(RuntimeError):
    """The checkpoint does not hold what the model reads."""


def _open_folder(folder: str):
    files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not files:
        raise WeightError(f"{folder}: no .safetensors file (a model folder holds config.json and model.safetensors)")
    handles, where = [], {}
    for path in files:
        f = safe_open(path, framework="pt", device="cpu")
        handles.append(f)
        for name in f.keys():
            where[name] = f
    return handles, where


def check_names(expected: list, where: dict, folder: str) -> None:
    want = {ps.name: ps for ps in expected}
    missing = sorted(n for n in want if n not in where)
    unexpected = sorted(n for n in where if n not in want)
    wrong = []
    for name, ps in want.items():
        if name in where:
            shape = tuple(where[name].get_slice(name).get_shape())
            if shape != tuple(ps.shape):
                wrong.append(f"{name}: expected {tuple(ps.shape)}, file has {shape}")
    if missing or unexpected or wrong:
        lines = [f"{folder}: the checkpoint does not match the model"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(lines))


def convert(t: torch.Tensor, kind: str, model_dtype: torch.dtype) -> torch.Tensor:
    if not t.is_floating_point():
        return t.to(torch.int32)
    if kind == "vector" and t.dtype == torch.float32:
        return t
    return t.to(model_dtype)


def load_weights(model, folder: str, device) -> None:
    """Fill `model` (a ComposedModel) from the safetensors files of `folder`."""
    handles, where = _open_folder(folder)
    specs = model.param_specs()
    check_names(specs, where, folder)
    kinds = {ps.name: ps.kind for ps in specs}

    def fetch(name: str) -> torch.Tensor:
        return convert(where[name].get_tensor(name), kinds[name], model.dtype).to(device)
    model.load(fetch)
    del handles
