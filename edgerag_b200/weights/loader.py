"""Weights by tensor name: from a model folder's safetensors, or random from a seed.

The reference copies tensors attribute by attribute out of a loaded library module
(edgerag/core/model.py:274-295) and reports a wrong shape per tensor (edgerag/core/linear.py:85-98).
Here the model lists the tensors it needs (``WeightSpec``: name, shape, kind), the loader finds
each under the prefixes a checkpoint may carry (in ``model.safetensors``, or in the shards that
``model.safetensors.index.json`` names), and **one** error reports every missing tensor,
every unexpected tensor and every wrong shape together.

Element types follow the spec's kind: matrices are cast to the engine's element type (bfloat16
when serving, float32 on the 32-bit path); ``vector32`` tensors are held in float32; ``keep``
leaves a tensor stored in 32-bit as it is; integer tables become int32.
"""

from __future__ import annotations

import hashlib
import json
import warnings
from pathlib import Path
from typing import Iterable

import torch

from ..parts.base import WeightSpec
from .safetensors_io import SafetensorsFile, write_safetensors


class WeightsError(ValueError):
    """The checkpoint does not fit the model.  The message lists every offender."""

    def __init__(self, where: str, missing: list[str], unexpected: list[str],
                 wrong_shape: list[tuple[str, tuple, tuple]], wrong_type: list[tuple[str, str]] = (),
                 note: str = "") -> None:
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_type = list(wrong_shape), list(wrong_type)
        lines = [f"{where}: the checkpoint does not fit the model" + (f" ({note})" if note else "")]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_type:
            lines.append(f"  wrong element types ({len(self.wrong_type)}): " + ", ".join(
                f"{n} is {t}" for n, t in self.wrong_type))
        super().__init__("\n".join(lines))


def _target_dtype(kind: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if kind == "vector32":
        return torch.float32
    if kind == "keep" and stored in (torch.float32, torch.int32):
        return stored
    return compute


class _Checkpoint:
    """The tensors of a model folder by name: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` lists (``{"weight_map": {tensor name: shard file}}``), which is
    how checkpoints too large for one file are stored."""

    def __init__(self, folder: Path) -> None:
        self.where = str(folder / "model.safetensors")
        self.files: list[SafetensorsFile] = []
        self.file_of: dict[str, SafetensorsFile] = {}
        single, index = folder / "model.safetensors", folder / "model.safetensors.index.json"
        try:
            if single.is_file() or not index.is_file():
                self._open(single)            # (a missing file raises the container's own error)
                return
            self.where = str(index)
            try:
                weight_map = json.loads(index.read_text())["weight_map"]
                assert isinstance(weight_map, dict) and weight_map
            except (json.JSONDecodeError, KeyError, AssertionError, UnicodeDecodeError) as exc:
                raise WeightsError(self.where, [], [], [], note=f"not a shard index with a weight_map ({exc!r})") from exc
            lost = sorted({str(f) for f in weight_map.values() if not (folder / str(f)).is_file()})
            if lost:
                raise WeightsError(self.where, [], [], [], note="shard files that the index names are absent: " + ", ".join(lost))
            opened = {shard: self._open(folder / shard) for shard in sorted({str(f) for f in weight_map.values()})}
            # the index decides where a name is read from; a tensor it names must be in that shard
            stray = sorted(n for n, shard in weight_map.items() if n not in opened[str(shard)].entries)
            if stray:
                raise WeightsError(self.where, stray, [], [], note="the index names tensors that their shard does not hold")
            self.file_of = {n: opened[str(shard)] for n, shard in weight_map.items()}
            for f in opened.values():          # tensors a shard holds beyond the index are reported as unexpected
                for n in f.names():
                    self.file_of.setdefault(n, f)
        except Exception:
            self.close()
            raise

    def _open(self, path: Path) -> SafetensorsFile:
        f = SafetensorsFile(path)
        self.files.append(f)
        for n in f.names():
            self.file_of.setdefault(n, f)
        return f

    def names(self) -> set[str]:
        return set(self.file_of)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.file_of[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self.file_of[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.file_of[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()

    def __enter__(self) -> "_Checkpoint":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def load_safetensors(folder: str | Path, specs: Iterable[WeightSpec], compute_dtype: torch.dtype,
                     device: torch.device, name_prefixes: tuple[str, ...] = ("model.text_model.", "model.", ""),
                     ignored_prefixes: tuple[str, ...] = ()) -> dict[str, torch.Tensor]:
    """``{model-relative name: tensor on device}`` for every spec, from ``folder/model.safetensors`` or
    from the shards listed in ``folder/model.safetensors.index.json``."""
    specs = list(specs)
    with _Checkpoint(Path(folder)) as f, warnings.catch_warnings():
        warnings.filterwarnings("ignore", message=".*non-writable.*")
        path = f.where
        stored = f.names()
        found: dict[str, str] = {}
        for s in specs:
            for prefix in name_prefixes:
                if prefix + s.name in stored:
                    found[s.name] = prefix + s.name
                    break
        missing = [s.name for s in specs if s.name not in found and not (s.fallback and s.fallback in found)]
        used = set(found.values())
        unexpected = sorted(n for n in stored - used if not any(n.startswith(p) for p in ignored_prefixes))
        wrong_shape = [(found[s.name], f.shape(found[s.name]), tuple(s.shape)) for s in specs
                       if s.name in found and f.shape(found[s.name]) != tuple(s.shape)]
        wrong_type = []
        for s in specs:
            if s.name in found:
                is_float = f.dtype(found[s.name]).is_floating_point
                if (s.kind == "int") == is_float:
                    wrong_type.append((found[s.name], str(f.dtype(found[s.name]))))
        if missing or unexpected or wrong_shape or wrong_type:
            raise WeightsError(str(path), missing, unexpected, wrong_shape, wrong_type)
        out: dict[str, torch.Tensor] = {}
        for s in specs:
            if s.name in found:
                t = f.tensor(found[s.name])
                out[s.name] = t.to(device=device, dtype=_target_dtype(s.kind, t.dtype, compute_dtype)).contiguous()
        for s in specs:
            if s.name not in out:
                out[s.name] = out[s.fallback]  # a tied head shares the embedding table
    return out


def random_tensors(specs: Iterable[WeightSpec], seed: int, std: float = 0.02, norm_jitter: float = 0.0,
                   compute_dtype: torch.dtype = torch.float32, device: torch.device | str = "cpu",
                   share_fallbacks: bool = True) -> dict[str, torch.Tensor]:
    """Seeded random weights: matrices ``N(0, std)``, vectors ``1 + norm_jitter * N(0, 1)``.

    Each tensor has a generator of its own, seeded from ``seed`` and the tensor's name, and is drawn
    in float32 on the CPU before the cast, so the values do not depend on the order of the specs or
    on the device.  A spec with a fallback (a tied head) shares the fallback's tensor.
    """
    out: dict[str, torch.Tensor] = {}
    specs = list(specs)
    names = {s.name for s in specs}
    for s in specs:
        if s.fallback and share_fallbacks and s.fallback in names:
            continue
        digest = hashlib.sha256(f"{seed}:{s.name}".encode()).digest()
        gen = torch.Generator().manual_seed(int.from_bytes(digest[:8], "little") >> 1)
        if s.kind == "int":
            t = torch.randint(0, 2, s.shape, generator=gen, dtype=torch.int32)
        elif len(s.shape) == 1:
            t = 1.0 + norm_jitter * torch.randn(s.shape, generator=gen)
        else:
            t = std * torch.randn(s.shape, generator=gen)
        out[s.name] = t.to(device=device, dtype=_target_dtype(s.kind, t.dtype, compute_dtype)).contiguous()
    for s in specs:
        if s.name not in out:
            out[s.name] = out[s.fallback]
    return out


def write_model_folder(folder: str | Path, raw_config: dict, specs: Iterable[WeightSpec], seed: int,
                       std: float = 0.02, norm_jitter: float = 0.0, dtype: torch.dtype = torch.bfloat16,
                       name_prefix: str = "model.") -> Path:
    """The random-weights mode: write ``config.json`` and ``model.safetensors`` for a configuration.

    Tensors get the names a checkpoint of the architecture has (``model.`` + the model-relative
    name; ``lm_head.weight`` without prefix; a tied head is not written).
    """
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw_config, indent=1))
    specs = list(specs)
    tensors = random_tensors(specs, seed, std, norm_jitter, compute_dtype=torch.float32, share_fallbacks=True)
    names = {s.name for s in specs}
    stored: dict[str, torch.Tensor] = {}
    for s in specs:
        if s.fallback and s.fallback in names:
            continue
        t = tensors[s.name]
        if t.is_floating_point():
            t = t.to(torch.float32 if (s.kind == "keep") else dtype)
        stored[s.name if s.name.startswith("lm_head.") else name_prefix + s.name] = t
    write_safetensors(folder / "model.safetensors", stored, metadata={"format": "pt", "seed": seed})
    return folder
