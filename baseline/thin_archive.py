"""Writing a ``.thin`` archive, the only container random-unknown-username/Thintensor loads.

Its Rust converter cannot be built here (no cargo), so the reference arm of the benchmark and the
script that made the golden logits write the archive themselves, from the layout the reference's
reader documents (thinruntime/archive.py:9-13, 99-208): an 88-byte header
``"<8sIIQQQQQ32s"`` (magic, header length, version, manifest offset and length, page-table offset,
page count, data offset, a hash the reader does not check), a JSON manifest, a page table of
``u16 id length, id, "<QQQI32s"`` records (offset, stored size, raw size, flags, checksum), and the
raw pages.  This is test and benchmark plumbing; nothing of the library uses it.
"""
from __future__ import annotations

import hashlib
import json
import struct
from pathlib import Path
from typing import Callable, Sequence

import torch

PAGE_DTYPES = {"F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2)}


def llama_manifest_model(*, hidden: int, layers: int, heads: int, kv_heads: int, head_dim: int, inter: int, vocab: int, eps: float,
                         theta: float, tied: bool, max_pos: int, scaling: dict | None = None, bias: bool = False) -> dict:
    """The ``model`` block of the manifest for a Llama dense decoder, with the keys the reference's
    runtime reads."""
    model = {
        "model_type": "llama", "arch": "LlamaForCausalLM", "hidden_size": hidden, "layers": layers, "heads": heads,
        "kv_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter, "vocab_size": vocab,
        "rms_norm_eps": eps, "norm_eps": eps, "norm_kind": "rms_norm", "rope_theta": theta, "tie_word_embeddings": tied,
        "activation": "silu", "max_position_embeddings": max_pos,
    }
    if bias:
        model.update({"attention_bias": True, "mlp_bias": True})
    if scaling:
        model.update({"rope_variant": "llama3", "rope_scaling": scaling, "rope_parameters": dict(scaling, rope_theta=theta),
                      "original_max_position_embeddings": scaling["original_max_position_embeddings"]})
    return model


def write_thin(path: Path, model: dict, specs: Sequence[tuple[str, tuple[int, ...]]], page_dtype: str,
               tensor_of: Callable[[str, tuple[int, ...]], torch.Tensor]) -> None:
    """Write pages ``specs`` (name, shape) in ``page_dtype`` ("F32" or "BF16").  ``tensor_of`` is
    called once per page, in order, while the file is written, so that a model of gigabytes never
    stands in host memory whole.  Page checksums are taken from the names: the reader does not
    verify them, but pages with equal (checksum, shape, dtype) would share one device tensor."""
    dtype, width = PAGE_DTYPES[page_dtype]
    pages = []
    for name, shape in specs:
        count = 1
        for d in shape:
            count *= d
        layer = int(name.split(".")[2]) if name.startswith("model.layers.") else None
        pages.append({"id": name, "kind": "tensor", "layer": layer, "op": name.rsplit(".", 2)[-2], "dtype": page_dtype,
                      "shape": list(shape), "backend_layout": "row_major", "size": count * width,
                      "checksum": hashlib.sha256(name.encode()).hexdigest()})
    manifest = json.dumps({"format": "thin", "version": 0, "model": model, "execution_tape": [], "pages": pages, "memory_plan": {}}).encode("utf-8")
    record = struct.calcsize("<QQQI32s")
    table_off = 88 + len(manifest)
    data_off = table_off + sum(2 + len(p["id"].encode()) + record for p in pages)
    table, offset = b"", data_off
    for page in pages:
        ident = page["id"].encode()
        table += struct.pack("<H", len(ident)) + ident + struct.pack("<QQQI32s", offset, page["size"], page["size"], 0, bytes(32))
        offset += page["size"]
    with Path(path).open("wb") as out:
        out.write(struct.pack("<8sIIQQQQQ32s", b"THINv0\0\0", 88, 0, 88, len(manifest), table_off, len(pages), data_off, bytes(32)))
        out.write(manifest)
        out.write(table)
        for (name, shape), page in zip(specs, pages):
            raw = tensor_of(name, tuple(shape)).to(dtype).contiguous()
            raw = raw.view(torch.int16 if width == 2 else torch.int32).numpy().tobytes()
            if len(raw) != page["size"]:
                raise ValueError(f"page {name}: {len(raw)} bytes for a declared shape of {shape}")
            out.write(raw)
