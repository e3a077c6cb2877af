"""Checkpoint / recovery file formats against byte layouts written out by hand from the reference's writer
(src/algorithms/diloco.zig:590-628, 1063-1107) and round trips."""
import os
import struct

import numpy as np
import pytest

from pcp_b200.formats import (FormatError, read_checkpoint, read_recovery, split_flat, write_checkpoint, write_recovery)


def test_checkpoint_bytes_match_the_reference_layout(tmp_path):
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    b = np.array([0x3F80, 0xBF80, 0x4000], dtype=np.uint16)          # bf16 1.0, -1.0, 2.0
    p = os.path.join(tmp_path, "checkpoint_7.bin")
    write_checkpoint(p, [a, b])
    want = b"PCPCHECK" + struct.pack("<I", 1) + struct.pack("<I", 2)
    want += struct.pack("<B", 2) + struct.pack("<qq", 2, 3) + struct.pack("<Q", 24) + a.tobytes()
    want += struct.pack("<B", 1) + struct.pack("<q", 3) + struct.pack("<Q", 6) + b.tobytes()
    assert open(p, "rb").read() == want
    got = read_checkpoint(p)
    assert got[0].dtype == np.float32 and np.array_equal(got[0], a)
    assert got[1].dtype == np.uint16 and np.array_equal(got[1], b)


def test_checkpoint_rejects_foreign_and_truncated_files(tmp_path):
    p = os.path.join(tmp_path, "x.bin")
    open(p, "wb").write(b"NOTACHECKPOINT!!")
    with pytest.raises(FormatError):
        read_checkpoint(p)
    write_checkpoint(p, [np.zeros((4, 4), np.float32)])
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-8])
    with pytest.raises(FormatError):
        read_checkpoint(p)


def test_recovery_bytes_and_round_trip(tmp_path):
    shapes = [(2, 2), (3,)]
    params = [np.arange(4, dtype=np.float32).reshape(2, 2), np.array([1, 2, 3], np.float32)]
    vel = [np.full((2, 2), 0.5, np.float32), np.array([-1, 0, 1], np.float32)]
    p = os.path.join(tmp_path, "shepherd_state.bin")
    write_recovery(p, params, vel, b"DM")
    want = b"PCP_RES" + struct.pack("<I", 2)
    want += struct.pack("<Q", 16) + params[0].tobytes() + struct.pack("<Q", 12) + params[1].tobytes()
    want += struct.pack("<Q", 28) + vel[0].tobytes() + vel[1].tobytes()
    want += struct.pack("<Q", 2) + b"DM"
    assert open(p, "rb").read() == want
    t, v, dm = read_recovery(p, shapes)
    assert all(np.array_equal(x, y) for x, y in zip(t, params))
    assert all(np.array_equal(x, y) for x, y in zip(v, vel)) and dm == b"DM"
    with pytest.raises(FormatError):
        read_recovery(p, [(2, 2), (4,)])


def test_split_flat_follows_argument_order():
    flat = np.arange(10, dtype=np.float32)
    parts = split_flat(flat, [(2, 3), (4,)])
    assert parts[0].shape == (2, 3) and parts[1].tolist() == [6, 7, 8, 9]
    with pytest.raises(FormatError):
        split_flat(flat, [(2, 3)])
