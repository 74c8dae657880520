"""From a model folder to tensors on the device, by tensor name.

The tensors a model needs are declared by its parts (`TensorDecl`); this file
checks a checkpoint against those declarations, and lists everything that is
missing, unexpected or of the wrong shape in one error before anything is
allocated (`src/microinfer/weights.py:139-150` does the same from config.json).
All tensors then go into ONE device allocation at 256-byte aligned offsets
(`src/microinfer/engine.py:88-103`, `src/core_kernels/include/microinfer/
kernels.h:110`).

Types on the device. With `dtype="bfloat16"`: what is stored in bfloat16 or
float16 is kept in bfloat16; a tensor stored in 32 bits stays in 32 bits; tables
of integers are int32. With `dtype="float32"` every number is widened to
float32, which is exact for all three stored types.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..errors import allocate
from .decl import TensorDecl
from .safetensors_io import STORED, SafetensorsFile, WeightError

ALIGNMENT = 256


def device_dtype(stored: str, mode: str) -> torch.dtype:
    """The type a tensor stored as `stored` has on the device in mode `mode`."""
    if stored in ("I32", "I64"):
        return torch.int32
    if mode == "float32":
        return torch.float32
    if mode == "bfloat16":
        return torch.float32 if stored == "F32" else torch.bfloat16
    raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {mode!r}")


class Checkpoint:
    """The safetensors files of a folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` names."""

    def __init__(self, folder):
        self.folder = Path(folder)
        index = self.folder / "model.safetensors.index.json"
        single = self.folder / "model.safetensors"
        self.files: dict[str, SafetensorsFile] = {}
        self.where: dict[str, str] = {}
        if single.is_file():
            self.files[single.name] = SafetensorsFile(single)
            self.where = {name: single.name for name in self.files[single.name].infos}
        elif index.is_file():
            weight_map = json.loads(index.read_text()).get("weight_map", {})
            for shard in sorted(set(weight_map.values())):
                self.files[shard] = SafetensorsFile(self.folder / shard)
            for shard, f in self.files.items():
                for name in f.infos:
                    self.where[name] = shard
        else:
            raise WeightError(f"{self.folder} holds neither model.safetensors nor "
                              "model.safetensors.index.json")

    def info(self, name: str):
        return self.files[self.where[name]].infos[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].tensor(name)

    def names(self):
        return list(self.where)


def check_tensors(checkpoint: Checkpoint, decls: list[TensorDecl], source: str,
                  ignore=()) -> None:
    """Raise one WeightError that lists every missing tensor, every unexpected
    tensor and every wrong shape or kind; silent if the checkpoint holds exactly
    what `decls` say. Names that match one of the shell-style patterns in `ignore`
    (an architecture's buffers that some exporters write and no part reads) are
    not counted as unexpected."""
    from fnmatch import fnmatchcase
    expected = {d.name: d for d in decls}
    found = {n for n in checkpoint.names()
             if n in expected or not any(fnmatchcase(n, pattern) for pattern in ignore)}
    missing = [f"    {n}: missing (shape {tuple(expected[n].shape)})"
               for n in expected if n not in found]
    unexpected = [f"    {n}: unexpected, not implied by {source} "
                  f"(shape {checkpoint.info(n).shape})" for n in sorted(found - set(expected))]
    wrong = []
    for n, d in expected.items():
        if n not in found:
            continue
        info = checkpoint.info(n)
        if tuple(info.shape) != tuple(d.shape):
            wrong.append(f"    {n}: shape {tuple(info.shape)}, {source} implies {tuple(d.shape)}")
        elif d.integer != (info.dtype in ("I32", "I64")):
            wrong.append(f"    {n}: stored as {info.dtype}, expected "
                         f"{'integers' if d.integer else 'numbers'}")
    if missing or unexpected or wrong:
        raise WeightError(
            f"{checkpoint.folder} does not hold what {source} describes "
            f"({len(missing)} missing, {len(unexpected)} unexpected, {len(wrong)} wrong); "
            "nothing was allocated:\n" + "\n".join(missing + unexpected + wrong))


class WeightArena:
    """One device allocation holding every tensor of a model, and views into it."""

    def __init__(self, decls: list[TensorDecl], dtypes: dict[str, torch.dtype], device):
        self.offsets: dict[str, int] = {}
        self.dtypes = dtypes
        self.decls = {d.name: d for d in decls}
        self.groups: dict[str, list[str]] = {}
        end, previous = 0, None
        for d in decls:
            nbytes = _numel(d.shape) * dtypes[d.name].itemsize
            joins = (d.group is not None and previous is not None and previous.group == d.group
                     and tuple(previous.shape[1:]) == tuple(d.shape[1:])
                     and dtypes[previous.name] == dtypes[d.name])
            start = end if joins else -(-end // ALIGNMENT) * ALIGNMENT
            if d.group is not None:
                if joins:
                    self.groups[d.group].append(d.name)
                elif d.group not in self.groups:
                    self.groups[d.group] = [d.name]
                else:               # a second run of the same group name: not contiguous
                    self.groups[d.group].append(None)
            self.offsets[d.name] = start
            end = start + nbytes
            previous = d
        self.nbytes = -(-end // ALIGNMENT) * ALIGNMENT
        raw = allocate(lambda: torch.empty(self.nbytes + ALIGNMENT, dtype=torch.uint8,
                                           device=device),
                       "the model's weights", self.nbytes + ALIGNMENT)
        shift = -raw.data_ptr() % ALIGNMENT          # device allocations are aligned already
        self.buffer = raw[shift:shift + max(self.nbytes, 1)]

    def view(self, name: str) -> torch.Tensor:
        d, dtype = self.decls[name], self.dtypes[name]
        nbytes = _numel(d.shape) * dtype.itemsize
        start = self.offsets[name]
        return self.buffer[start:start + nbytes].view(dtype).reshape(tuple(d.shape))

    def group_view(self, group: str):
        """The members of `group` as one tensor (joined along the first axis), or
        None if they could not be laid back to back."""
        names = self.groups.get(group)
        if not names or None in names:
            return None
        first = self.decls[names[0]]
        rows = sum(self.decls[n].shape[0] for n in names)
        dtype = self.dtypes[names[0]]
        nbytes = rows * _numel(first.shape[1:]) * dtype.itemsize
        start = self.offsets[names[0]]
        return self.buffer[start:start + nbytes].view(dtype).reshape((rows,) + tuple(first.shape[1:]))


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def load_checkpoint(folder, decls: list[TensorDecl], mode: str, device,
                    source: str = "config.json", ignore=()):
    """Check, allocate, copy. Returns the arena; nothing is allocated unless the
    whole checkpoint fits the declarations, and a NaN or infinity in any tensor
    is refused by name (`src/microinfer/weights.py:153-174`)."""
    checkpoint = Checkpoint(folder)
    check_tensors(checkpoint, decls, source, ignore)
    dtypes = {d.name: device_dtype(checkpoint.info(d.name).dtype, mode) for d in decls}
    arena = WeightArena(decls, dtypes, device)
    bad = []
    for d in decls:
        host = checkpoint.tensor(d.name)
        if host.is_floating_point() and host.numel():
            if not bool(torch.isfinite(host).all()):
                bad.append(f"    {d.name}: holds NaN or infinity")
                continue
        arena.view(d.name).copy_(host.to(dtypes[d.name]))
    if bad:
        raise WeightError(f"{checkpoint.folder} holds values that are not numbers:\n"
                          + "\n".join(bad))
    return arena
