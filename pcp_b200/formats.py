"""Disk formats of the reference's Shepherd, so that a run on this backend can be resumed by (or resume from) a PCP
Shepherd (Backend.save_checkpoint / load_checkpoint for the parameters, Backend.load_recovery for parameters plus the
Nesterov velocities of this rank's shard): the model checkpoint `checkpoint_<step>.bin` (src/algorithms/diloco.zig:590-628) and the recovery file
`recovery/shepherd_state.bin` (diloco.zig:1063-1107, read back at :1110-1180).  Little-endian throughout.

    PCPCHECK file:  "PCPCHECK"  u32 version (= 1)  u32 n_tensors
                    per tensor: u8 rank, rank x i64 dims, u64 n_bytes, raw parameter bytes (f32 or bf16)
    PCP_RES file:   "PCP_RES"   u32 n_tensors, per tensor: u64 n_bytes, raw bytes
                    u64 optimizer bytes: the Nesterov velocities, f32, tensor after tensor
                    (src/optimizers/nesterov.zig:101-113)
                    u64 data-manager bytes (opaque here: kept and written back verbatim)
"""
from __future__ import annotations

import struct
from typing import List, Optional, Sequence, Tuple

import numpy as np

CHECKPOINT_MAGIC = b"PCPCHECK"
CHECKPOINT_VERSION = 1
RECOVERY_MAGIC = b"PCP_RES"
RECOVERY_FILENAME = "shepherd_state.bin"


class FormatError(ValueError):
    pass


def split_flat(flat: np.ndarray, shapes: Sequence[Sequence[int]]) -> List[np.ndarray]:
    """The flat parameter vector (artefact argument order, as the C ABI hands it out) as one array per tensor."""
    out, at = [], 0
    for s in shapes:
        n = int(np.prod(s)) if len(s) else 1
        out.append(np.ascontiguousarray(flat[at:at + n]).reshape(s))
        at += n
    if at != flat.size:
        raise FormatError(f"{flat.size} values for shapes that hold {at}")
    return out


def write_checkpoint(path: str, tensors: Sequence[np.ndarray]) -> None:
    """tensors: one array per parameter in argument order; float32, or uint16 holding bf16 bit patterns."""
    with open(path, "wb") as f:
        f.write(CHECKPOINT_MAGIC)
        f.write(struct.pack("<II", CHECKPOINT_VERSION, len(tensors)))
        for t in tensors:
            t = np.ascontiguousarray(t)
            if t.dtype not in (np.float32, np.uint16):
                raise FormatError("checkpoint tensors are float32 or bf16 bit patterns (uint16)")
            f.write(struct.pack("<B", t.ndim))
            for d in t.shape:
                f.write(struct.pack("<q", int(d)))
            raw = t.tobytes()
            f.write(struct.pack("<Q", len(raw)))
            f.write(raw)


def read_checkpoint(path: str) -> List[np.ndarray]:
    """-> one array per tensor: float32 if the byte count is 4 per element, uint16 (bf16 bits) if it is 2."""
    with open(path, "rb") as f:
        data = f.read()
    if data[:8] != CHECKPOINT_MAGIC:
        raise FormatError("not a PCPCHECK file")
    version, n = struct.unpack_from("<II", data, 8)
    if version != CHECKPOINT_VERSION:
        raise FormatError(f"checkpoint version {version} is not supported")
    at, out = 16, []
    for _ in range(n):
        (rank,) = struct.unpack_from("<B", data, at); at += 1
        shape = struct.unpack_from(f"<{rank}q", data, at); at += 8 * rank
        (nbytes,) = struct.unpack_from("<Q", data, at); at += 8
        if at + nbytes > len(data):
            raise FormatError("truncated checkpoint")
        numel = int(np.prod(shape)) if rank else 1
        if nbytes == 4 * numel:
            arr = np.frombuffer(data, np.float32, numel, at)
        elif nbytes == 2 * numel:
            arr = np.frombuffer(data, np.uint16, numel, at)
        else:
            raise FormatError(f"{nbytes} bytes for a tensor of {numel} elements")
        out.append(arr.reshape(shape).copy()); at += nbytes
    return out


def write_recovery(path: str, tensors: Sequence[np.ndarray], velocities: Optional[Sequence[np.ndarray]],
                   data_manager_state: bytes = b"") -> None:
    with open(path, "wb") as f:
        f.write(RECOVERY_MAGIC)
        f.write(struct.pack("<I", len(tensors)))
        for t in tensors:
            raw = np.ascontiguousarray(t).tobytes()
            f.write(struct.pack("<Q", len(raw)))
            f.write(raw)
        opt = b"".join(np.ascontiguousarray(v, np.float32).tobytes() for v in velocities) if velocities is not None else b""
        f.write(struct.pack("<Q", len(opt)))
        f.write(opt)
        f.write(struct.pack("<Q", len(data_manager_state)))
        f.write(data_manager_state)


def read_recovery(path: str, shapes: Sequence[Sequence[int]]) -> Tuple[List[np.ndarray], Optional[List[np.ndarray]], bytes]:
    """-> (parameter tensors, velocities or None, data-manager bytes).  The file carries no shapes (the Shepherd
    takes them from the model it was started with, diloco.zig:1145-1150); `shapes` plays that part."""
    with open(path, "rb") as f:
        data = f.read()
    if data[:7] != RECOVERY_MAGIC:
        raise FormatError("not a PCP_RES file")
    (n,) = struct.unpack_from("<I", data, 7)
    if n not in (0, len(shapes)):
        raise FormatError(f"{n} tensors in the file, {len(shapes)} in the model")
    at, tensors = 11, []
    for i in range(n):
        (nbytes,) = struct.unpack_from("<Q", data, at); at += 8
        numel = int(np.prod(shapes[i])) if len(shapes[i]) else 1
        dt = np.float32 if nbytes == 4 * numel else np.uint16 if nbytes == 2 * numel else None
        if dt is None or at + nbytes > len(data):
            raise FormatError("tensor size does not match the model (CorruptSaveFile)")
        tensors.append(np.frombuffer(data, dt, numel, at).reshape(shapes[i]).copy()); at += nbytes
    (opt_len,) = struct.unpack_from("<Q", data, at); at += 8
    velocities = None
    if opt_len:
        want = 4 * sum(int(np.prod(s)) if len(s) else 1 for s in shapes)
        if opt_len < want or at + opt_len > len(data):
            raise FormatError("optimizer state shorter than the velocities (CorruptSaveFile)")      # nesterov.zig:122
        velocities, o = [], at
        for s in shapes:
            numel = int(np.prod(s)) if len(s) else 1
            velocities.append(np.frombuffer(data, np.float32, numel, o).reshape(s).copy()); o += 4 * numel
        at += opt_len
    (dm_len,) = struct.unpack_from("<Q", data, at); at += 8
    return tensors, velocities, bytes(data[at:at + dm_len])
