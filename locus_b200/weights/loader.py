"""Loading weights by tensor name, and the random-weights mode.

The loader matches the tensors a model's parts declare against the tensors a source
offers, and reports everything that is wrong in one error: missing tensors, unexpected
tensors and wrong shapes (the reference raises one ``gguf::Error`` per case:
"missing tensor: N", "unexpected shape for tensor: N",
src/locus/model/gguf_load.hpp:34-86).

Element types.  In a bfloat16 model a parameter is kept in bfloat16 when its checkpoint
tensors are stored in 16 bits, and stays float32 when they are stored in 32 bits; integer
tensors become int32.  In a float32 model every floating tensor is float32.

The random-weights mode writes a model folder (config.json + model.safetensors) from a
configuration and a seed: linear and embedding weights N(0, 0.02), biases N(0, 0.02), norm
weights 1 + N(0, 0.01); each tensor has its own generator seeded by (seed, tensor name), so
values do not depend on the order of generation.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, List, Tuple

import torch

from ..config.base import find_arch
from .safetensors_io import write_safetensors


class WeightError(ValueError):
    """The source does not fit the model; the message lists every problem."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong: List[str]) -> None:
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong
        lines = [f"weights do not fit the model: {len(missing)} missing, {len(unexpected)} unexpected, "
                 f"{len(wrong)} with a wrong shape or element type"]

        def block(title, items):
            if items:
                lines.append(f"  {title}:")
                lines.extend(f"    {i}" for i in items[:40])
                if len(items) > 40:
                    lines.append(f"    ... and {len(items) - 40} more")

        block("missing tensors", missing)
        block("unexpected tensors", unexpected)
        block("wrong shape or type", wrong)
        super().__init__("\n".join(lines))


_FLOAT16 = (torch.bfloat16, torch.float16)
_FLOAT32 = (torch.float32, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def _param_dtype(model_dtype: torch.dtype, stored: List[torch.dtype]) -> torch.dtype:
    if all(d in _INTS for d in stored):
        return torch.int32
    if model_dtype == torch.float32:
        return torch.float32
    return torch.float32 if any(d in _FLOAT32 for d in stored) else torch.bfloat16


def load_weights(model, source) -> None:
    """Fill every parameter of ``model`` from ``source`` (``names()``, ``info(name)``,
    ``tensor(name)``), on the model's device."""
    wanted = model.tensor_sources()
    by_name: Dict[str, Tuple[object, object]] = {}
    for part, src in wanted:
        by_name[src.name] = (part, src)
    have = set(source.names())
    ignorable = set(model.ignorable_tensor_names())
    missing = sorted(n for n in by_name if n not in have)
    unexpected = sorted(n for n in have if n not in by_name and n not in ignorable
                        and not n.endswith("rotary_emb.inv_freq"))
    wrong = []
    for n, (_, src) in by_name.items():
        if n in have:
            dt, shape = source.info(n)
            if tuple(shape) != tuple(src.shape):
                wrong.append(f"{n}: stored {tuple(shape)}, the model wants {tuple(src.shape)}")
            elif dt not in _FLOAT16 + _FLOAT32 + _INTS:
                wrong.append(f"{n}: element type {dt} is not loadable")
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, sorted(wrong))

    # element type of each parameter from the storage types of its tensors
    stored: Dict[Tuple[int, str], List[torch.dtype]] = {}
    for part, src in wanted:
        stored.setdefault((id(part), src.param), []).append(source.info(src.name)[0])
    parts = {id(p): p for p, _ in wanted}
    for (pid, pname), dts in stored.items():
        part = parts[pid]
        shape = part.param_shapes()[pname]
        part.params[pname] = torch.empty(shape, dtype=_param_dtype(model.dtype, dts), device=model.device)
    for part in model.all_parts():
        for pname in part.param_shapes():
            if pname not in part.params:
                raise WeightError([f"(no tensor fills parameter {pname} of {part.prefix})"], [], [])
    for part, src in wanted:
        dest = part.params[src.param]
        flat = dest.view(-1, dest.shape[-1]) if dest.dim() >= 2 else dest
        t = source.tensor(src.name)
        n0 = src.shape[0]
        flat[src.row0 : src.row0 + n0].copy_(t.reshape(flat[src.row0 : src.row0 + n0].shape)
                                             .to(device=model.device, dtype=dest.dtype))
    model.loaded = True


# ---------------------------------------------------------------------------
# random weights


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(seed: int, name: str, shape, init: str, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """The random-weights mode's value of tensor ``name``: float32 draws, rounded to ``dtype``."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    t = torch.randn(tuple(shape), generator=g, dtype=torch.float32, device=device)
    if init == "norm":
        t = 1.0 + 0.01 * t
    elif init in ("linear", "bias"):
        t = 0.02 * t
    else:
        raise ValueError(f"unknown init kind {init!r}")
    return t.to(dtype)


class RandomSource:
    """A weight source that draws each tensor when asked (on ``device``), without a file."""

    def __init__(self, model, seed: int, dtype: torch.dtype, device="cpu") -> None:
        self.seed, self.dtype, self.device = seed, dtype, device
        self._src = {s.name: s for _, s in model.tensor_sources()}

    def names(self):
        return list(self._src)

    def info(self, name):
        return self.dtype, tuple(self._src[name].shape)

    def tensor(self, name):
        s = self._src[name]
        return random_tensor(self.seed, name, s.shape, s.init, self.dtype, self.device)


def write_random_model(raw_config: dict, seed: int, out_dir: str, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` with seeded random weights."""
    from ..config.base import arch_name_of
    from ..models.model import Model

    entry = find_arch(arch_name_of(raw_config))
    cfg = entry.parse_config(raw_config)
    model = Model(entry.build_plan(cfg), torch.float32, "cpu")
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw_config, f, indent=1)
    sources = [s for _, s in model.tensor_sources()]
    by_name = {s.name: s for s in sources}
    write_safetensors(
        os.path.join(out_dir, "model.safetensors"),
        [(s.name, tuple(s.shape), dtype) for s in sources],
        lambda n: random_tensor(seed, n, by_name[n].shape, by_name[n].init, dtype),
        metadata={"format": "pt", "seed": str(seed)},
    )
    return out_dir
