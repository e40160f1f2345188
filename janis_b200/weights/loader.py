"""Loading a model's tensors by name, and writing a model folder of random ones.

A model states which tensors it expects (`TensorSpec` by checkpoint name); the
loader compares that with what the folder holds and raises ONE error that lists
every missing tensor, every unexpected tensor and every wrong shape.  What is
loaded is kept as stored where it can be: BF16 stays bfloat16, F16 becomes
bfloat16, anything stored in 32-bit floating point stays float32, integer
tables become int32.  The parts widen to float32 themselves when the engine
runs its 32-bit path.

The reference loads tensor by tensor through `File.Get(name)` and fails on the
first missing one (`safetensors/safetensors.go:180-192`, `qwen/embed.go:40-50`);
it has no random-weights mode (`inkling2/testdata/gen_fixture.py` makes its
fixtures for another architecture).
"""
from __future__ import annotations

import fnmatch
import hashlib
import json
import os
from dataclasses import dataclass
from typing import Iterable, Mapping

import torch

from .safetensors import ModelFiles, SafetensorsError, open_model, write_safetensors


class WeightsError(ValueError):
    """The folder's tensors do not match what the model expects."""


@dataclass(frozen=True)
class TensorSpec:
    """One expected tensor: its shape, whether it is an integer table, and how
    the random-weights mode draws it (normal with `init_std`)."""
    shape: tuple[int, ...]
    integer: bool = False
    init_std: float = 0.02


_FLOATS = {"F64", "F32", "F16", "BF16"}
_INTS = {"I64", "I32", "I16", "I8", "U8", "U16", "U32"}


def check_tensors(expected: Mapping[str, TensorSpec], files: ModelFiles,
                  ignorable: Iterable[str] = ()) -> None:
    """Raise one WeightsError naming all that is missing, unexpected or misshapen."""
    have = set(files.names())
    want = set(expected)
    ignorable = tuple(ignorable)
    missing = sorted(want - have)
    unexpected = sorted(n for n in have - want if not any(fnmatch.fnmatch(n, p) for p in ignorable))
    wrong = []
    for n in sorted(want & have):
        info, spec = files.info(n), expected[n]
        if tuple(info.shape) != tuple(spec.shape):
            wrong.append(f"{n}: expected shape {list(spec.shape)}, found {list(info.shape)}")
        elif spec.integer and info.dtype not in _INTS:
            wrong.append(f"{n}: expected an integer table, found dtype {info.dtype}")
        elif not spec.integer and info.dtype not in _FLOATS:
            wrong.append(f"{n}: expected floating point, found dtype {info.dtype}")
    if not (missing or unexpected or wrong):
        return
    lines = ["model weights do not match the configuration:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}):")
        lines += [f"    {n}  {list(expected[n].shape)}" for n in missing]
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}):")
        lines += [f"    {n}  {list(files.info(n).shape)}" for n in unexpected]
    if wrong:
        lines.append(f"  wrong shape or dtype ({len(wrong)}):")
        lines += [f"    {w}" for w in wrong]
    raise WeightsError("\n".join(lines))


def stored_to_kept(t: torch.Tensor, integer: bool) -> torch.Tensor:
    """The dtype a tensor is kept in after loading (see the module text)."""
    if integer:
        return t.to(torch.int32)
    if t.dtype in (torch.float32, torch.float64):
        return t.to(torch.float32)
    return t.to(torch.bfloat16)


def load_tensors(model_dir: str, expected: Mapping[str, TensorSpec], device,
                 ignorable: Iterable[str] = ()) -> dict[str, torch.Tensor]:
    """Check the folder against `expected`, then bring every expected tensor to `device`."""
    try:
        files = open_model(model_dir)
    except SafetensorsError as e:
        raise WeightsError(str(e)) from e
    try:
        check_tensors(expected, files, ignorable)
        out = {}
        for name, spec in expected.items():
            out[name] = stored_to_kept(files.read(name), spec.integer).to(device)
        return out
    finally:
        files.close()


# ----------------------------------------------------------------------------
# random weights
# ----------------------------------------------------------------------------

def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, spec: TensorSpec, seed: int, device="cpu",
                  dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The tensor that (seed, name) names: each tensor has a generator of its own, so
    the values do not depend on which other tensors are drawn, nor in what order."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if spec.integer:
        return torch.randint(0, 2 ** 15, spec.shape, generator=g, device=device, dtype=torch.int32)
    t = torch.empty(spec.shape, device=device, dtype=torch.float32)
    t.normal_(0.0, spec.init_std, generator=g)
    return t.to(dtype)


def random_tensors(expected: Mapping[str, TensorSpec], seed: int, device="cpu",
                   dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    return {n: random_tensor(n, s, seed, device, dtype) for n, s in expected.items()}


def write_model_folder(model_dir: str, config_dict: dict, tensors: Mapping[str, torch.Tensor],
                       metadata: dict[str, str] | None = None) -> None:
    """config.json and model.safetensors, the two files a model folder is."""
    os.makedirs(model_dir, exist_ok=True)
    tmp = os.path.join(model_dir, f"config.json.tmp.{os.getpid()}")
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=2, sort_keys=True)
        f.write("\n")
    os.replace(tmp, os.path.join(model_dir, "config.json"))
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      {n: t.detach().cpu() for n, t in tensors.items()}, metadata)
