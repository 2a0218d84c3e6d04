"""Where tensors come from: the safetensors files of a model folder, or a seeded generator.

Reading is by tensor name, as in the reference's loader
(src/cloud_engine/weights.py:81-94: every ``*.safetensors`` file of the folder, sorted,
opened on the CPU, a name present in two files is an error).  The reference has no
random weights; ``RandomSource`` is this framework's: one generator per tensor, seeded
from (seed, tensor name), so a tensor's values do not depend on which other tensors
exist or in which order they are drawn.
"""

from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Any

from ..parts.base import TensorSpec


class WeightsError(Exception):
    """The tensors of a model folder do not fit the model: lists every fault at once."""

    def __init__(self, message: str, *, missing=(), unexpected=(), wrong_shape=(), duplicate=()):
        super().__init__(message)
        self.missing = tuple(missing)
        self.unexpected = tuple(unexpected)
        self.wrong_shape = tuple(wrong_shape)
        self.duplicate = tuple(duplicate)


class SafetensorsSource:
    def __init__(self, model_dir: str | Path) -> None:
        import safetensors

        self.model_dir = Path(model_dir)
        paths = sorted(self.model_dir.glob("*.safetensors"))
        if not paths:
            raise FileNotFoundError(f"no *.safetensors found in {self.model_dir}")
        self._where: dict[str, Path] = {}
        self._shapes: dict[str, tuple[int, ...]] = {}
        self._handles: dict[Path, Any] = {}
        duplicates: list[str] = []
        for path in paths:
            handle = safetensors.safe_open(str(path), framework="pt", device="cpu")
            self._handles[path] = handle
            for name in handle.keys():  # noqa: SIM118 - safetensors API
                if name in self._where:
                    duplicates.append(f"{name} (in {self._where[name].name} and {path.name})")
                    continue
                self._where[name] = path
                self._shapes[name] = tuple(handle.get_slice(name).get_shape())
        if duplicates:
            raise WeightsError(
                "tensors stored more than once: " + "; ".join(duplicates), duplicate=duplicates
            )

    def names(self) -> list[str]:
        return sorted(self._where)

    def shape(self, name: str) -> tuple[int, ...]:
        return self._shapes[name]

    def get(self, name: str) -> Any:
        return self._handles[self._where[name]].get_tensor(name)


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


class RandomSource:
    """Seeded random tensors for a name table: weights and biases N(0, std), norm gains
    1 + N(0, std); drawn in float32 and rounded to ``store_dtype`` (bfloat16 by default, so a
    32-bit run and a bfloat16 run of the same folder start from identical values).

    ``scales`` maps a piece of a tensor name to a factor: every tensor whose name contains the
    piece is multiplied by it before rounding (``{".q_proj.": 1.9, ".k_proj.": 1.9}`` spreads
    attention scores, which N(0, 0.02) weights leave close to uniform)."""

    def __init__(self, table: dict[str, TensorSpec], seed: int, std: float = 0.02,
                 store_dtype: str = "bfloat16", vector_dtype: str | None = None,
                 device: str = "cpu", scales: dict[str, float] | None = None) -> None:
        self.table = dict(table)
        self.seed = int(seed)
        self.std = float(std)
        self.store_dtype = store_dtype
        self.vector_dtype = vector_dtype or store_dtype
        self.device = device
        self.scales = dict(scales or {})

    def names(self) -> list[str]:
        return sorted(self.table)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.table[name].shape)

    def get(self, name: str) -> Any:
        import torch

        spec = self.table[name]
        generator = torch.Generator(device=self.device)
        generator.manual_seed(_tensor_seed(self.seed, name))
        if spec.init == "zeros":
            values = torch.zeros(spec.shape, dtype=torch.float32, device=self.device)
        else:
            values = torch.empty(spec.shape, dtype=torch.float32, device=self.device)
            values.normal_(0.0, self.std, generator=generator)
            if spec.init == "gain":
                values += 1.0
            elif spec.init != "normal":
                raise ValueError(f"tensor {name}: unknown init {spec.init!r}")
        for piece, factor in self.scales.items():
            if piece in name:
                values *= factor
        dtype = self.vector_dtype if spec.role == "vector" else self.store_dtype
        return values.to(getattr(torch, dtype))
