"""Checkpoint files -> device tensors: a safetensors reader with the loader vocabulary of the reference.

Mirror of `GpuWeights::from_dir / from_single_file / from_index / take`
(crates/layers/src/weights.rs:473-520, 847-880): the files are memory-mapped and parsed on the host
(no device allocation), and a tensor is uploaded when a layer loader takes it — through a pinned
staging buffer, bytes exactly as stored (what `take_keep_dtype` does for the int4 scales and biases).
The on-disk format is the public safetensors layout: an 8-byte little-endian header length, a JSON
header `{name: {dtype, shape, data_offsets}}`, then the tensors' bytes.  `write_safetensors` exists for
tests and synthetic checkpoints.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch

from .layers import GpuWeights

# safetensors dtype -> (bytes per element, torch dtype the bytes are handed over as)
_DTYPES = {
    "BF16": (2, torch.bfloat16), "F16": (2, torch.float16), "F32": (4, torch.float32), "F64": (8, torch.float64),
    "U32": (4, torch.int32),            # packed int4 codes: same bits, torch has no general uint32 kernels
    "I32": (4, torch.int32), "I64": (8, torch.int64), "U8": (1, torch.uint8), "I8": (1, torch.int8),
    "F8_E4M3": (1, torch.uint8),        # e4m3 bytes are handled as bytes by the fp8 loader
    "BOOL": (1, torch.bool),
}
_NUMPY_TO_ST = {np.dtype(np.uint32): "U32", np.dtype(np.int32): "I32", np.dtype(np.float32): "F32",
                np.dtype(np.float16): "F16", np.dtype(np.uint8): "U8", np.dtype(np.int64): "I64"}


class SafetensorsFile:
    """One memory-mapped shard: `entries[name] = (dtype string, shape, begin, end)`."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise ValueError(f"{path}: not a safetensors file (too short)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise ValueError(f"{path}: header length {hlen} exceeds the file")
        header = json.loads(self._f.read(hlen).decode("utf-8"))
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            dtype, shape, (b0, b1) = e["dtype"], tuple(int(d) for d in e["shape"]), e["data_offsets"]
            if dtype not in _DTYPES:
                raise ValueError(f"{path}: tensor `{name}` has unsupported dtype {dtype}")
            want = _DTYPES[dtype][0] * int(np.prod(shape, dtype=np.int64)) if shape else _DTYPES[dtype][0]
            if b1 - b0 != want or self._base + b1 > size:
                raise ValueError(f"{path}: tensor `{name}` spans {b1 - b0} bytes, its shape needs {want}")
            self.entries[name] = (dtype, shape, int(b0), int(b1))

    def bytes_of(self, name: str) -> memoryview:
        _, _, b0, b1 = self.entries[name]
        return memoryview(self._mm)[self._base + b0:self._base + b1]

    def close(self) -> None:
        self._mm.close()
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, object], metadata: Optional[dict] = None) -> None:
    """`tensors[name]` is a numpy array, or `(uint16 array, "BF16")` / `(uint8 array, "F8_E4M3")` for the
    dtypes numpy does not have.  Data is laid out in name order, unpadded."""
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name]
        if isinstance(t, tuple):
            arr, dtype = np.ascontiguousarray(t[0]), t[1]
        else:
            arr = np.ascontiguousarray(t)
            dtype = _NUMPY_TO_ST[arr.dtype]
        raw = arr.tobytes()
        if len(raw) != _DTYPES[dtype][0] * arr.size:
            raise ValueError(f"`{name}`: {arr.dtype} does not store {dtype}")
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)


class CheckpointWeights(GpuWeights):
    """`GpuWeights` backed by memory-mapped safetensors shards: `take` uploads, `contains` probes the
    headers.  Tensors handed in directly (device tensors) take precedence, as in the base class."""

    STAGING_BYTES = 64 << 20

    def __init__(self, files: Iterable[SafetensorsFile], device, scale_dtype: Optional[torch.dtype] = torch.bfloat16):
        super().__init__({}, scale_dtype)
        self.device = torch.device(device)
        self._files = list(files)
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self._files:
            for name in f.entries:
                self._where[name] = f
        self._staging: Optional[torch.Tensor] = None

    # ---- GpuWeights::from_dir (weights.rs:473-492)
    @classmethod
    def from_dir(cls, directory: str, device, scale_dtype: Optional[torch.dtype] = torch.bfloat16) -> "CheckpointWeights":
        index = os.path.join(directory, "model.safetensors.index.json")
        single = os.path.join(directory, "model.safetensors")
        if os.path.exists(index):
            return cls.from_index(index, device, scale_dtype)
        if os.path.exists(single):
            return cls.from_single_file(single, device, scale_dtype)
        shards = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors")) if os.path.isdir(directory) else []
        if shards:
            return cls([SafetensorsFile(os.path.join(directory, f)) for f in shards], device, scale_dtype)
        raise FileNotFoundError(f"No safetensors files found in {directory}")

    @classmethod
    def from_single_file(cls, path: str, device, scale_dtype: Optional[torch.dtype] = torch.bfloat16) -> "CheckpointWeights":
        return cls([SafetensorsFile(path)], device, scale_dtype)

    @classmethod
    def from_index(cls, index_path: str, device, scale_dtype: Optional[torch.dtype] = torch.bfloat16) -> "CheckpointWeights":
        with open(index_path) as f:
            weight_map = json.load(f).get("weight_map")
        if not isinstance(weight_map, dict):
            raise ValueError(f"{index_path}: no `weight_map`")
        directory = os.path.dirname(os.path.abspath(index_path))
        files = {name: SafetensorsFile(os.path.join(directory, name)) for name in sorted(set(weight_map.values()))}
        gw = cls(files.values(), device, scale_dtype)
        for tensor, shard in weight_map.items():
            if tensor not in files[shard].entries:
                raise KeyError(f"{index_path}: `{tensor}` is not in shard {shard}")
            gw._where[tensor] = files[shard]
        return gw

    def names(self):
        return sorted(set(self._where) | set(self._t))

    def contains(self, name: str) -> bool:
        return name in self._t or name in self._where

    def _upload(self, name: str) -> torch.Tensor:
        f = self._where[name]
        dtype, shape, _, _ = f.entries[name]
        raw = f.bytes_of(name)
        with warnings.catch_warnings():                                  # the mapping is read-only and only ever read
            warnings.simplefilter("ignore", UserWarning)
            host = torch.frombuffer(raw, dtype=torch.uint8) if len(raw) else torch.empty(0, dtype=torch.uint8)
        if self.device.type == "cuda":
            dev = torch.empty(len(raw), dtype=torch.uint8, device=self.device)
            if self._staging is None:
                self._staging = torch.empty(self.STAGING_BYTES, dtype=torch.uint8, pin_memory=True)
            for off in range(0, len(raw), self.STAGING_BYTES):          # mmap -> pinned -> device, chunked
                n = min(self.STAGING_BYTES, len(raw) - off)
                self._staging[:n].copy_(host[off:off + n])
                dev[off:off + n].copy_(self._staging[:n], non_blocking=True)
                torch.cuda.current_stream(self.device).synchronize()   # the staging buffer is reused
        else:
            dev = host.clone()
        return dev.view(_DTYPES[dtype][1]).reshape(shape)

    def take(self, name: str) -> torch.Tensor:
        if name in self._t:
            self._where.pop(name, None)
            return self._t.pop(name)
        if name not in self._where:
            raise KeyError(f"tensor `{name}` not found in checkpoint")
        t = self._upload(name)
        del self._where[name]
        return t

    def peek(self, name: str) -> torch.Tensor:
        if name not in self._t:
            if name not in self._where:
                raise KeyError(f"tensor `{name}` not found in checkpoint")
            self._t[name] = self._upload(name)      # uploaded once, kept until taken
        return self._t[name]

    def close(self) -> None:
        for f in self._files:
            f.close()
