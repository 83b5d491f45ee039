"""Reading and writing safetensors files directly.

The format: an 8-byte little-endian header length, a JSON header mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the
end of the header), then the raw little-endian data.  A model folder holds either
``model.safetensors`` or ``model.safetensors.index.json`` whose ``weight_map`` names
the shard of each tensor (the reference reads that index for tensor names at
thinruntime/model_arch.py:873-889; it converts the data to its own archive first,
src/convert_hf.rs:790-846, a step this library does not have).
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import torch


class WeightError(ValueError):
    """A checkpoint that cannot be read or does not fit the model."""


TORCH_DTYPES: dict[str, torch.dtype] = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
SAFETENSORS_NAMES = {v: k for k, v in TORCH_DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str                # safetensors dtype string
    shape: tuple[int, ...]
    file: Path
    begin: int                # absolute byte offsets in ``file``
    end: int


class SafetensorsFile:
    """One open ``.safetensors`` file: its entries and zero-copy views of the data."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        if not self.path.is_file():
            raise WeightError(f"weight file {self.path} does not exist")
        self._file = self.path.open("rb")
        size = self.path.stat().st_size
        if size < 8:
            raise WeightError(f"{self.path} is too small to be a safetensors file")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if 8 + header_len > size:
            raise WeightError(f"{self.path}: header length {header_len} exceeds the file size {size}")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise WeightError(f"{self.path}: header is not valid JSON: {exc}") from exc
        base = 8 + header_len
        self.entries: dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            begin, end = meta["data_offsets"]
            if meta["dtype"] not in TORCH_DTYPES:
                raise WeightError(f"{self.path}: tensor {name!r} has unsupported dtype {meta['dtype']!r}")
            shape = tuple(int(s) for s in meta["shape"])
            count = 1
            for s in shape:
                count *= s
            width = torch.empty((), dtype=TORCH_DTYPES[meta["dtype"]]).element_size()
            if end - begin != count * width or base + end > size:
                raise WeightError(
                    f"{self.path}: tensor {name!r} of shape {list(shape)} and dtype {meta['dtype']} "
                    f"needs {count * width} bytes but its data range holds {end - begin}"
                )
            self.entries[name] = TensorEntry(name, meta["dtype"], shape, self.path, base + begin, base + end)
        self._mmap = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the file's bytes (read-only memory: copy before writing)."""
        entry = self.entries[name]
        if entry.end == entry.begin:
            return torch.empty(entry.shape, dtype=TORCH_DTYPES[entry.dtype])
        view = memoryview(self._mmap)[entry.begin : entry.end]
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            flat = torch.frombuffer(view, dtype=TORCH_DTYPES[entry.dtype])
        return flat.reshape(entry.shape)

    def close(self) -> None:
        if self._mmap is not None:
            try:
                self._mmap.close()
            except BufferError:
                pass  # tensors still view it; the OS unmaps when they go
            self._mmap = None
        self._file.close()


class Checkpoint:
    """All tensors of a model folder, whichever shard holds them."""

    def __init__(self, folder: str | Path):
        self.folder = Path(folder)
        single = self.folder / "model.safetensors"
        index = self.folder / "model.safetensors.index.json"
        self.files: list[SafetensorsFile] = []
        if single.is_file():
            self.files.append(SafetensorsFile(single))
        elif index.is_file():
            weight_map = json.loads(index.read_text(encoding="utf-8")).get("weight_map", {})
            for shard in sorted(set(weight_map.values())):
                if not (self.folder / shard).is_file():
                    raise WeightError(f"{index} names shard {shard!r}, which is missing from {self.folder}")
                self.files.append(SafetensorsFile(self.folder / shard))
        else:
            raise WeightError(f"{self.folder} holds neither model.safetensors nor model.safetensors.index.json")
        self.entries: dict[str, TensorEntry] = {}
        self._owner: dict[str, SafetensorsFile] = {}
        for file in self.files:
            for name, entry in file.entries.items():
                if name in self.entries:
                    raise WeightError(f"tensor {name!r} is stored in both {self.entries[name].file.name} and {file.path.name}")
                self.entries[name] = entry
                self._owner[name] = file

    def tensor(self, name: str) -> torch.Tensor:
        return self._owner[name].tensor(name)

    def close(self) -> None:
        for file in self.files:
            file.close()


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) in the order given."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    blobs = []
    for name, tensor in tensors.items():
        if tensor.dtype not in SAFETENSORS_NAMES:
            raise WeightError(f"cannot store tensor {name!r} of dtype {tensor.dtype}")
        tensor = tensor.detach().cpu().contiguous()
        size = tensor.numel() * tensor.element_size()
        header[name] = {
            "dtype": SAFETENSORS_NAMES[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + size],
        }
        blobs.append(tensor)
        offset += size
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * (-len(encoded) % 8)
    with Path(path).open("wb") as out:
        out.write(struct.pack("<Q", len(encoded)))
        out.write(encoded)
        for tensor in blobs:
            if tensor.numel():
                out.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes())
