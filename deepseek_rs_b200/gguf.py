"""Host-side mirror of the reference's GGUF reader for the tensors of the routed-expert path.

``GgufFile`` follows ``GgufFile`` of engine/src/gguf.rs:12-122 (``open``, ``find``, ``tensor_data``, ``tensors``) over
the C ABI (``dsmoe_gguf_*``); ``GgufBuilder`` writes small GGUF v3 images in memory the way the reference's parser
tests do (engine/tests/gguf_parse.rs:12-77), which is how the tests here get files without a model on disk.
"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass

import numpy as np

from . import _lib


class GgufError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"dsmoe status {code}: {msg}")
        self.code = code


@dataclass
class TensorMeta:
    """engine/src/model.rs:79-97"""
    name: str
    type: int
    dims: list
    offset: int
    bytes: int
    host_ptr: int


class GgufFile:
    def __init__(self, path: str | None = None, data: bytes | np.ndarray | None = None):
        self.lib = _lib.load()
        self.g = C.c_void_p()
        if data is not None:
            self._keep = np.frombuffer(data, np.uint8) if not isinstance(data, np.ndarray) else np.ascontiguousarray(data)
            rc = self.lib.dsmoe_gguf_open_memory(C.c_void_p(self._keep.ctypes.data), self._keep.size, C.byref(self.g))
        else:
            rc = self.lib.dsmoe_gguf_open(path.encode(), C.byref(self.g))
        if rc != 0:
            msg = self.lib.dsmoe_gguf_last_error(self.g).decode() if self.g else "allocation failed"
            self.close()
            raise GgufError(rc, msg)

    @classmethod
    def open(cls, path: str) -> "GgufFile":
        return cls(path=path)

    def close(self):
        if getattr(self, "g", None):
            self.lib.dsmoe_gguf_close(self.g)
            self.g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise GgufError(rc, self.lib.dsmoe_gguf_last_error(self.g).decode())

    @staticmethod
    def _meta(t: _lib.GgufTensor) -> TensorMeta:
        return TensorMeta(t.name.decode(), int(t.type), [int(t.dims[i]) for i in range(t.n_dims)], int(t.offset), int(t.bytes),
                          int(t.host_data))

    @property
    def data_offset(self) -> int:
        return int(self.lib.dsmoe_gguf_data_offset(self.g))

    @property
    def tensors(self) -> list:
        out, t = [], _lib.GgufTensor()
        for i in range(int(self.lib.dsmoe_gguf_tensor_count(self.g))):
            self._check(self.lib.dsmoe_gguf_tensor_at(self.g, i, C.byref(t)))
            out.append(self._meta(t))
        return out

    def find(self, name: str):
        """engine/src/gguf.rs:118-121: the tensor's metadata or None."""
        t = _lib.GgufTensor()
        rc = self.lib.dsmoe_gguf_find_tensor(self.g, name.encode(), C.byref(t))
        if rc == _lib.ERR_STATE:
            return None
        self._check(rc)
        return self._meta(t)

    def tensor_data(self, t: TensorMeta) -> np.ndarray:
        """engine/src/gguf.rs:111-116: the tensor's bytes (a copy)."""
        buf = (C.c_uint8 * t.bytes).from_address(t.host_ptr)
        return np.frombuffer(buf, np.uint8).copy()

    def upload_experts(self, kernels, gguf_layer: int, expert_begin: int = 0, expert_count: int | None = None,
                       layout: int = _lib.LAYOUT_ROWSOA):
        """Validates and copies one layer's expert tensors (or the shard [expert_begin, expert_begin + expert_count))
        to new torch tensors on the kernels' device; returns (gate, up, down)."""
        import torch

        cfg = kernels.cfg
        n = cfg.n_expert - expert_begin if expert_count is None else expert_count
        gu, dn = C.c_uint64(0), C.c_uint64(0)
        self._check(self.lib.dsmoe_gguf_expert_shard_bytes(C.byref(cfg), n, C.byref(gu), C.byref(dn)))
        dev = torch.device("cuda", kernels.device)
        gate = torch.empty(gu.value, dtype=torch.uint8, device=dev)
        up = torch.empty(gu.value, dtype=torch.uint8, device=dev)
        down = torch.empty(dn.value, dtype=torch.uint8, device=dev)
        staging = torch.empty(max(gu.value, dn.value), dtype=torch.uint8, device=dev) if layout == _lib.LAYOUT_ROWSOA else None
        p = lambda t: None if t is None else C.c_void_p(t.data_ptr())
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._check(self.lib.dsmoe_gguf_upload_experts(self.g, C.byref(cfg), stream, gguf_layer, expert_begin, n, layout,
                                                      p(gate), p(up), p(down), p(staging)))
        torch.cuda.current_stream().synchronize()
        return gate, up, down


class GgufBuilder:
    """A GGUF v3 image in memory: header, optional metadata, tensor table, 32-byte aligned data section."""

    def __init__(self, version: int = 3):
        self.version, self.kv, self.infos, self.data = version, [], [], bytearray()

    @staticmethod
    def _str(s: str) -> bytes:
        b = s.encode()
        return struct.pack("<Q", len(b)) + b

    def add_kv_u32(self, key: str, value: int):
        self.kv.append(self._str(key) + struct.pack("<II", 4, value))

    def add_kv_string_array(self, key: str, values):
        self.kv.append(self._str(key) + struct.pack("<IIQ", 9, 8, len(values)) + b"".join(self._str(v) for v in values))

    def add_tensor(self, name: str, type_id: int, dims, payload: bytes | np.ndarray | None = None, offset: int | None = None):
        """dims: fastest dimension first. payload: the tensor's bytes (appended to the data section, 32-byte aligned);
        None declares a tensor without data (for table-only tests), at ``offset``."""
        if payload is not None:
            pad = (-len(self.data)) % 32
            self.data += b"\0" * pad
            offset = len(self.data)
            self.data += bytes(payload) if not isinstance(payload, np.ndarray) else payload.tobytes()
        info = self._str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        self.infos.append(info + struct.pack("<IQ", type_id, offset or 0))

    def build(self, extra_data_bytes: int = 0) -> bytes:
        head = struct.pack("<IIQQ", 0x46554747, self.version, len(self.infos), len(self.kv))
        body = head + b"".join(self.kv) + b"".join(self.infos)
        body += b"\0" * ((-len(body)) % 32)
        return body + bytes(self.data) + b"\0" * extra_data_bytes
