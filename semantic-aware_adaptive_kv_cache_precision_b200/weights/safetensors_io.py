"""Reading and writing safetensors files, without any library for the format.

The format, as the reference's reader has it (`src/microinfer/weights.py:51-58,
61-78`): eight bytes of little-endian header length, a JSON header that gives
`dtype`, `shape` and `data_offsets` for every tensor name (and an optional
`__metadata__`), then the data. Files are memory-mapped, so a checkpoint is
never held in host memory as a whole.
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch


class WeightError(RuntimeError):
    """A checkpoint that cannot be loaded; the message lists every problem."""


#: dtype name in the file -> (torch dtype, bytes per element)
STORED = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8),
}
_NAME_OF = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
            torch.int32: "I32", torch.int64: "I64"}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple
    begin: int
    end: int


class SafetensorsFile:
    """One file's header, and its tensors on demand as CPU torch tensors that
    view the mapped file (read-only: copy before writing to them)."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise WeightError(f"{self.path} does not exist")
        size = self.path.stat().st_size
        with open(self.path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise WeightError(f"{self.path}: {size} bytes is too short for a safetensors file")
            (length,) = struct.unpack("<Q", head)
            if length <= 0 or length > 100_000_000 or 8 + length > size:
                raise WeightError(f"{self.path}: its first eight bytes announce a header of "
                                  f"{length} bytes, which a safetensors file of {size} bytes "
                                  "cannot have")
            try:
                header = json.loads(f.read(length))
            except (json.JSONDecodeError, UnicodeDecodeError):
                raise WeightError(f"{self.path}: the header is not JSON; "
                                  "not a safetensors file") from None
        self.base = 8 + length
        self.infos: dict[str, TensorInfo] = {}
        problems = []
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                begin, end = meta["data_offsets"]
                info = TensorInfo(name, meta["dtype"], tuple(int(s) for s in meta["shape"]),
                                  int(begin), int(end))
            except (KeyError, TypeError, ValueError):
                problems.append(f"    {name}: malformed header entry {meta!r}")
                continue
            if info.dtype not in STORED:
                problems.append(f"    {name}: dtype {info.dtype} is not supported "
                                f"(supported: {', '.join(sorted(STORED))})")
                continue
            want = int(np.prod(info.shape, dtype=np.int64)) * STORED[info.dtype][1]
            if info.end - info.begin != want:
                problems.append(f"    {name}: {info.end - info.begin} bytes of data for shape "
                                f"{info.shape} {info.dtype}, which needs {want}")
            self.infos[name] = info
        if problems:
            raise WeightError(f"{self.path} has a bad header:\n" + "\n".join(problems))
        needed = self.base + max((i.end for i in self.infos.values()), default=0)
        if size < needed:
            raise WeightError(f"{self.path.name} is cut short: its header places tensors up to "
                              f"byte {needed:,}, the file ends at byte {size:,}")
        self._map = None

    def _mapped(self):
        if self._map is None:
            with open(self.path, "rb") as f:
                self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return self._map

    def tensor(self, name: str) -> torch.Tensor:
        info = self.infos[name]
        dtype, width = STORED[info.dtype]
        count = (info.end - info.begin) // width
        if count == 0:
            return torch.empty(info.shape, dtype=dtype)
        arr = np.frombuffer(self._mapped(), dtype=np.uint8, count=info.end - info.begin,
                            offset=self.base + info.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # the buffer is read-only; it is only read
            flat = torch.frombuffer(arr, dtype=torch.uint8)
        return flat.view(dtype).reshape(info.shape)


def write_safetensors(path, tensors, metadata: dict | None = None) -> None:
    """Write `tensors` (name -> CPU torch tensor, or a callable that makes one, so
    that a large model is written one tensor at a time) to `path`."""
    names = list(tensors)
    made = {}
    header, offset = {}, 0
    plan = []
    for name in names:
        value = tensors[name]
        if callable(value):
            shape, dtype = value.shape, value.dtype
        else:
            value = value.detach().cpu().contiguous()
            made[name] = value
            shape, dtype = tuple(value.shape), value.dtype
        if dtype not in _NAME_OF:
            raise WeightError(f"{name}: cannot store dtype {dtype}")
        nbytes = int(np.prod(shape, dtype=np.int64)) * STORED[_NAME_OF[dtype]][1]
        header[name] = {"dtype": _NAME_OF[dtype], "shape": list(shape),
                        "data_offsets": [offset, offset + nbytes]}
        plan.append((name, nbytes))
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, nbytes in plan:
            value = made.get(name)
            if value is None:
                value = tensors[name]().detach().cpu().contiguous()
            data = value.view(torch.uint8).numpy().tobytes() if value.numel() else b""
            if len(data) != nbytes:
                raise WeightError(f"{name}: made {len(data)} bytes, header promised {nbytes}")
            f.write(data)
