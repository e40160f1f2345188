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


def _signed64(c: int) -> int:
    c &= 0xFFFF_FFFF_FFFF_FFFF
    return c - (1 << 64) if c >= (1 << 63) else c


_GAMMA, _MUL1, _MUL2 = _signed64(0x9E3779B97F4A7C15), _signed64(0xBF58476D1CE4E5B9), _signed64(0x94D049BB133111EB)
_CHUNK = 1 << 24                 # elements drawn at a time (the 64-bit intermediates of a whole embedding would not fit)


def _hash64(counter: torch.Tensor) -> torch.Tensor:
    """The splitmix64 finaliser over int64 values (two's-complement wrap-around; shifts made logical by masks)."""
    z = counter * _GAMMA
    z = (z ^ ((z >> 30) & 0x3_FFFF_FFFF)) * _MUL1
    z = (z ^ ((z >> 27) & 0x1F_FFFF_FFFF)) * _MUL2
    return z ^ ((z >> 31) & 0x1_FFFF_FFFF)


def _bell(key: int, start: int, n: int, device) -> torch.Tensor:
    """n values of mean 0 and variance 1, those of elements start .. start + n - 1 of the tensor `key` names:
    the sum of twelve 16-bit fields of three hashes of the element's index, a bell curve that stands in for the
    normal distribution (same mean and variance, kurtosis 2.9, nothing beyond 6 standard deviations).  Integer
    arithmetic and exact float steps only, so every device computes the same bits."""
    i = torch.arange(start, start + n, dtype=torch.int64, device=device)
    total = torch.zeros(n, dtype=torch.int64, device=device)
    for j in (1, 2, 3):
        z = _hash64(i * 4 + (j + key))
        for shift in (0, 16, 32, 48):
            total += (z >> shift) & 0xFFFF
    # twelve uniforms on [0, 1): mean 6 x 65535 / 65536 (subtracted exactly), variance 12 / 12 (up to 2^-32)
    return (total - 6 * 65535).to(torch.float32) * (1.0 / 65536.0)


def random_tensor(name: str, spec: TensorSpec, seed: int, device="cpu",
                  dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The tensor that (seed, name) names, the same bits on every device: a counter-based generator keyed by the
    seed, the name and the element's index, so the values depend neither on which other tensors are drawn, nor
    on their order, nor on where they are drawn."""
    key = _tensor_seed(seed, name) >> 3           # room for the counters' low bits within 63 bits
    n = 1
    for d in spec.shape:
        n *= int(d)
    if spec.integer:
        out = torch.empty(n, device=device, dtype=torch.int32)
        for a in range(0, n, _CHUNK):
            m = min(_CHUNK, n - a)
            i = torch.arange(a, a + m, dtype=torch.int64, device=device)
            out[a:a + m] = (_hash64(i * 4 + (1 + key)) & 0x7FFF).to(torch.int32)
        return out.view(spec.shape)
    out = torch.empty(n, device=device, dtype=dtype)
    std = float(spec.init_std)
    for a in range(0, n, _CHUNK):
        m = min(_CHUNK, n - a)
        out[a:a + m] = (_bell(key, a, m, device) * std).to(dtype)
    return out.view(spec.shape)


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
