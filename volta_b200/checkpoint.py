"""Optimizer-state checkpoints in Volta's own ``StateDict`` file format.

Volta saves model weights as ``BTreeMap<String, TensorData { data: Vec<f32>, shape: Vec<usize> }>``
encoded with bincode 2 ``config::standard()`` (src/io.rs:15-22,151-166) but never saves
optimizer state (m, v, t, velocity are private, src/nn/optim/adam.rs:5-14).  This module
writes the state of a ``volta_b200`` optimizer into that same container, so that
``volta::io::load_state_dict`` can read the file and a resumed run continues bit-identically:

    optimizer.kind            shape [1]   0 Adam, 1 SGD, 2 Muon
    optimizer.t               shape [1]   Adam's step counter (exact below 2^24)
    optimizer.state0.<i>      parameter i's shape: Adam m / SGD velocity / Muon velocity
    optimizer.state1.<i>      parameter i's shape: Adam v

The same dictionary can be written as a SafeTensors file, the other container Volta reads and
writes (``save_safetensors`` / ``load_safetensors``, src/io.rs:280-345: every tensor F32).
SafeTensors: u64 little-endian header length, a JSON header ``{name: {"dtype", "shape",
"data_offsets": [begin, end]}}`` padded with spaces to a multiple of 8 bytes, then the tensors'
bytes back to back in header order.

bincode ``standard()``: little endian; unsigned integers as varints (< 251: one byte; 251 +
u16; 252 + u32; 253 + u64); f32 as four bytes; ``Vec``/``String``/map = varint length + items;
``BTreeMap`` iterates in key order (byte-wise string order).
"""
from __future__ import annotations

import json
import struct
from typing import Dict, Tuple

import numpy as np

StateDict = Dict[str, Tuple[np.ndarray, Tuple[int, ...]]]


def _put_varint(out: bytearray, v: int) -> None:
    if v < 0:
        raise ValueError("unsigned only")
    if v < 251:
        out.append(v)
    elif v < 1 << 16:
        out.append(251)
        out += struct.pack("<H", v)
    elif v < 1 << 32:
        out.append(252)
        out += struct.pack("<I", v)
    else:
        out.append(253)
        out += struct.pack("<Q", v)


def _get_varint(buf: memoryview, pos: int) -> Tuple[int, int]:
    tag = buf[pos]
    if tag < 251:
        return tag, pos + 1
    if tag == 251:
        return struct.unpack_from("<H", buf, pos + 1)[0], pos + 3
    if tag == 252:
        return struct.unpack_from("<I", buf, pos + 1)[0], pos + 5
    if tag == 253:
        return struct.unpack_from("<Q", buf, pos + 1)[0], pos + 9
    raise ValueError(f"unsupported varint tag {tag}")


def encode_state_dict(state: StateDict) -> bytes:
    """bincode(standard) bytes of a Volta ``StateDict``."""
    out = bytearray()
    _put_varint(out, len(state))
    for key in sorted(state, key=lambda k: k.encode("utf-8")):
        data, shape = state[key]
        kb = key.encode("utf-8")
        _put_varint(out, len(kb))
        out += kb
        arr = np.ascontiguousarray(data, dtype="<f4").reshape(-1)
        _put_varint(out, arr.size)
        out += arr.tobytes()
        _put_varint(out, len(shape))
        for s in shape:
            _put_varint(out, int(s))
    return bytes(out)


def decode_state_dict(blob: bytes) -> StateDict:
    buf = memoryview(blob)
    n, pos = _get_varint(buf, 0)
    state: StateDict = {}
    for _ in range(n):
        klen, pos = _get_varint(buf, pos)
        key = bytes(buf[pos:pos + klen]).decode("utf-8")
        pos += klen
        dlen, pos = _get_varint(buf, pos)
        data = np.frombuffer(buf, dtype="<f4", count=dlen, offset=pos).astype(np.float32)
        pos += 4 * dlen
        slen, pos = _get_varint(buf, pos)
        shape = []
        for _ in range(slen):
            s, pos = _get_varint(buf, pos)
            shape.append(s)
        state[key] = (data, tuple(shape))
    if pos != len(blob):
        raise ValueError("trailing bytes after the state dict")
    return state


def encode_safetensors(state: StateDict) -> bytes:
    """SafeTensors image of a state dict: all tensors F32, in key order (src/io.rs:321-345)."""
    header = {}
    offset = 0
    blobs = []
    for key in sorted(state, key=lambda k: k.encode("utf-8")):
        data, shape = state[key]
        flat = np.ascontiguousarray(data, dtype="<f4").reshape(-1)
        if int(np.prod(shape, dtype=np.int64)) != flat.size:
            raise ValueError(f"{key}: shape {shape} does not hold {flat.size} elements")
        header[key] = {"dtype": "F32", "shape": [int(d) for d in shape],
                       "data_offsets": [offset, offset + flat.size * 4]}
        offset += flat.size * 4
        blobs.append(flat.tobytes())
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    return struct.pack("<Q", len(text)) + text + b"".join(blobs)


def decode_safetensors(blob: bytes) -> StateDict:
    """Inverse of :func:`encode_safetensors`; accepts any SafeTensors file whose tensors are F32."""
    if len(blob) < 8:
        raise ValueError("SafeTensors file shorter than its length field")
    (n,) = struct.unpack_from("<Q", blob, 0)
    if 8 + n > len(blob):
        raise ValueError("SafeTensors header runs past the end of the file")
    header = json.loads(bytes(blob[8:8 + n]).decode("utf-8"))
    base = 8 + n
    out: StateDict = {}
    for key in sorted((k for k in header if k != "__metadata__"), key=lambda k: k.encode("utf-8")):
        info = header[key]
        if info["dtype"] != "F32":
            raise ValueError(f"{key}: dtype {info['dtype']} (optimizer state is F32)")
        begin, end = info["data_offsets"]
        shape = tuple(int(d) for d in info["shape"])
        if end - begin != 4 * int(np.prod(shape, dtype=np.int64)) or base + end > len(blob):
            raise ValueError(f"{key}: data_offsets do not match the shape or the file")
        out[key] = (np.frombuffer(blob, dtype="<f4", count=(end - begin) // 4, offset=base + begin).copy(), shape)
    return out


_KINDS = {"Adam": 0, "SGD": 1, "Muon": 2}


def optimizer_state_dict(opt) -> StateDict:
    """Collects an optimizer's state (this rank's part on a sharded engine; the rest is zero)."""
    kind = type(opt).__name__
    state: StateDict = {"optimizer.kind": (np.array([_KINDS[kind]], np.float32), (1,))}
    if kind == "Adam":
        t = opt.t
        if t >= 1 << 24:
            raise ValueError("t does not fit an f32 exactly")
        state["optimizer.t"] = (np.array([t], np.float32), (1,))
    n_states = 2 if kind == "Adam" else 1
    for i, p in enumerate(opt.params):
        for which in range(n_states):
            try:
                arr = opt.state(i, which)
            except Exception:  # SGD without momentum has no state buffer
                continue
            state[f"optimizer.state{which}.{i}"] = (arr, tuple(p.shape))
    return state


def _is_safetensors(path: str, fmt: str) -> bool:
    if fmt not in ("auto", "bincode", "safetensors"):
        raise ValueError("format is 'auto', 'bincode' or 'safetensors'")
    return fmt == "safetensors" or (fmt == "auto" and path.endswith(".safetensors"))


def save_optimizer_state(opt, path: str, format: str = "auto") -> None:
    """``format='auto'`` writes SafeTensors for ``*.safetensors`` and bincode otherwise."""
    state = optimizer_state_dict(opt)
    with open(path, "wb") as fh:
        fh.write(encode_safetensors(state) if _is_safetensors(path, format) else encode_state_dict(state))


def load_optimizer_state(opt, path: str, format: str = "auto") -> None:
    with open(path, "rb") as fh:
        blob = fh.read()
    state = decode_safetensors(blob) if _is_safetensors(path, format) else decode_state_dict(blob)
    kind = type(opt).__name__
    if int(state["optimizer.kind"][0][0]) != _KINDS[kind]:
        raise ValueError("checkpoint was written by a different optimizer kind")
    if kind == "Adam":
        opt.t = int(state["optimizer.t"][0][0])
    for key, (data, shape) in state.items():
        if key.startswith("optimizer.state"):
            which, idx = key[len("optimizer.state"):].split(".")
            if tuple(shape) != tuple(opt.params[int(idx)].shape):
                raise ValueError(f"{key}: shape {shape} does not match the parameter")
            opt.load_state(int(idx), int(which), data)
