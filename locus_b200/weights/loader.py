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
weights 1 + N(0, 0.01); every element is a function of (seed, tensor name, element index) alone
(``random_init``), so values depend neither on the order of generation nor on the device that draws.
"""
from __future__ import annotations

import fnmatch
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
    ``tensor(name)``), on the model's device.  Parts that name the same checkpoint tensor as the whole
    of a parameter (a head tied to the embedding) share one device tensor."""
    wanted = model.tensor_sources()
    by_name: Dict[str, List[Tuple[object, object]]] = {}
    for part, src in wanted:
        by_name.setdefault(src.name, []).append((part, src))
    have = set(source.names())
    ignorable = tuple(getattr(model.plan, "ignorable_tensors", ()))
    missing = sorted(n for n in by_name if n not in have)
    unexpected = sorted(n for n in have if n not in by_name and not any(fnmatch.fnmatchcase(n, pat) for pat in ignorable))
    wrong = []
    for n, users in by_name.items():
        if n in have:
            dt, shape = source.info(n)
            for _, src in users:
                if tuple(shape) != tuple(src.shape):
                    wrong.append(f"{n}: stored {tuple(shape)}, the model wants {tuple(src.shape)}")
            if dt not in _FLOAT16 + _FLOAT32 + _INTS:
                wrong.append(f"{n}: element type {dt} is not loadable")
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, sorted(set(wrong)))

    # element type of each parameter from the storage types of its tensors
    stored: Dict[Tuple[int, str], List[torch.dtype]] = {}
    for part, src in wanted:
        stored.setdefault((id(part), src.param), []).append(source.info(src.name)[0])
    parts = {id(p): p for p, _ in wanted}

    def whole(part, src) -> bool:
        return src.row0 == 0 and tuple(src.shape) == tuple(part.param_shapes()[src.param])

    shared: Dict[str, torch.Tensor] = {}   # checkpoint tensor -> the device tensor that holds all of it
    filled = set()
    for part, src in wanted:
        if whole(part, src) and src.name in shared:
            part.params[src.param] = shared[src.name]
            filled.add((id(part), src.param))
            continue
        key = (id(part), src.param)
        if src.param not in part.params or key not in filled:
            shape = part.param_shapes()[src.param]
            part.params[src.param] = torch.empty(shape, dtype=_param_dtype(model.dtype, stored[key]),
                                                 device=model.device)
            filled.add(key)
        dest = part.params[src.param]
        flat = dest.view(-1, dest.shape[-1]) if dest.dim() >= 2 else dest
        t = source.tensor(src.name)
        n0 = src.shape[0]
        flat[src.row0 : src.row0 + n0].copy_(t.reshape(flat[src.row0 : src.row0 + n0].shape)
                                             .to(device=model.device, dtype=dest.dtype))
        if whole(part, src):
            shared[src.name] = dest
    for part in model.all_parts():
        for pname in part.param_shapes():
            if (id(part), pname) not in filled:
                raise WeightError([f"(no tensor fills parameter {pname} of {part.prefix})"], [], [])
    model.loaded = True


# ---------------------------------------------------------------------------
# random weights


from .random_init import random_tensor  # noqa: E402  (the draw itself: same bits on every device)


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


def write_random_model(raw_config: dict, seed: int, out_dir: str, dtype: torch.dtype = torch.bfloat16,
                       device="cpu") -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` with seeded random weights.
    ``device``: where the values are drawn (the same bits everywhere; a GPU draws a large model in
    seconds where the host takes minutes)."""
    from ..config.base import arch_name_of
    from ..models.model import Model

    entry = find_arch(arch_name_of(raw_config))
    cfg = entry.parse_config(raw_config)
    model = Model(entry.build_plan(cfg), torch.float32, "cpu")
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw_config, f, indent=1)
    by_name = {}
    for _, s in model.tensor_sources():
        by_name.setdefault(s.name, s)   # a tensor that two parts name (a tied head) is written once
    sources = list(by_name.values())
    write_safetensors(
        os.path.join(out_dir, "model.safetensors"),
        [(s.name, tuple(s.shape), dtype) for s in sources],
        lambda n: random_tensor(seed, n, by_name[n].shape, by_name[n].init, dtype, device).cpu(),
        metadata={"format": "pt", "seed": str(seed)},
    )
    return out_dir
