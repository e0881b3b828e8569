"""Weights by tensor name, checked against what the model declares.

One error lists everything that is wrong with a checkpoint: tensors the model needs
and the files lack, tensors the files hold and the model does not know, and tensors
of the wrong shape.  The reference copies whatever bytes arrive under a name
(src/model/linear.cuh:67-75) and only rejects unknown names (src/model/model.cuh:138-141).

Dtypes: matrices are held in the compute dtype (bfloat16 for serving); small tensors
(norm weights and the like) stored in 32-bit stay 32-bit; integer tables become
int32.  With the float32 compute dtype every floating tensor is widened to fp32.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from ..parts.base import WeightSpec
from .safetensors_io import SafetensorsError, SafetensorsFile, model_files


class WeightError(ValueError):
    """Everything that is wrong with a checkpoint, in one message: missing tensors, unexpected tensors, wrong
    shapes, and other problems (a tensor that cannot be read, a floating tensor where an integer table belongs).
    A stored dtype that differs from the one the tensor is held in is not an error: the tensor is converted
    (see ``target_dtype``)."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[str], other: List[str] = ()):
        self.missing, self.unexpected, self.wrong_shape, self.other = list(missing), list(unexpected), list(wrong_shape), list(other)
        lines = ["the checkpoint does not fit the model:"]

        def section(title: str, items: List[str]) -> None:
            if items:
                lines.append(f"  {title} ({len(items)}):")
                lines.extend(f"    {x}" for x in items[:40])
                if len(items) > 40:
                    lines.append(f"    ... and {len(items) - 40} more")

        section("missing tensors", self.missing)
        section("unexpected tensors", self.unexpected)
        section("wrong shapes", self.wrong_shape)
        section("other problems", self.other)
        super().__init__("\n".join(lines))


def target_dtype(spec: WeightSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.role == "table" or not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if spec.role == "vector" and stored in (torch.float32, torch.float64):
        return torch.float32
    return compute


def check_and_place(named: Iterable[Tuple[str, torch.Tensor]], expected: Mapping[str, WeightSpec],
                    compute: torch.dtype, device: "torch.device | str",
                    ignore: Optional[Callable[[str], bool]] = None) -> Dict[str, torch.Tensor]:
    """Checks every (name, tensor) against ``expected`` and moves it to the device in its
    target dtype.  Raises one :class:`WeightError` for all problems."""
    out: Dict[str, torch.Tensor] = {}
    unexpected: List[str] = []
    wrong: List[str] = []
    other: List[str] = []
    for name, t in named:
        spec = expected.get(name)
        if spec is None:
            if not (ignore and ignore(name)):
                unexpected.append(name)
            continue
        if name in out:
            other.append(f"{name}: given twice")
            continue
        if tuple(t.shape) != tuple(spec.shape):
            wrong.append(f"{name}: stored {tuple(t.shape)}, the model needs {tuple(spec.shape)}")
            continue
        if spec.role != "table" and not t.dtype.is_floating_point:
            other.append(f"{name}: stored as {t.dtype}, a floating tensor is needed")
            continue
        out[name] = t.to(device=device, dtype=target_dtype(spec, t.dtype, compute)).contiguous()
    missing = [n for n in expected if n not in out and not any(w.startswith(n + ":") for w in wrong + other)]
    if missing or unexpected or wrong or other:
        raise WeightError(sorted(missing), sorted(unexpected), sorted(wrong), sorted(other))
    return out


def iter_checkpoint(model_dir: str, adapt: Optional[Callable[[str, torch.Tensor], List[Tuple[str, torch.Tensor]]]] = None):
    for path in model_files(model_dir):
        f = SafetensorsFile(path)
        for name in f.names():
            t = f.tensor(name)
            if adapt is None:
                yield name, t
            else:
                yield from adapt(name, t)


def load_checkpoint(model_dir: str, expected: Mapping[str, WeightSpec], compute: torch.dtype,
                    device: "torch.device | str",
                    adapt: Optional[Callable[[str, torch.Tensor], List[Tuple[str, torch.Tensor]]]] = None,
                    ignore: Optional[Callable[[str], bool]] = None) -> Dict[str, torch.Tensor]:
    try:
        return check_and_place(iter_checkpoint(model_dir, adapt), expected, compute, device, ignore)
    except SafetensorsError as e:
        raise WeightError([], [], [], [str(e)]) from None
