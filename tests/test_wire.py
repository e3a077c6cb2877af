"""Shepherd <-> worker message formats (host side, no GPU): envelope text and framing, the StartInnerLoop payload, the
chunked parameter / update transfers and a round trip Shepherd -> worker -> Shepherd over them."""
import base64
import json
import os
import struct

import numpy as np
import pytest

from pcp_b200 import wire
from pcp_b200.wire import ChunkReassembler, Envelope, InnerLoopTask, WireError


def test_envelope_text_is_the_struct_in_field_order():
    # what std.json.stringify(MessageEnvelope, .{}) writes for these values (src/network/message.zig:46-57): compact,
    # fields in declaration order, data last
    env = Envelope(7, "worker", 0, "shepherd", "StartInnerLoop", 41, {"tau": 10, "dtype": "bf16"}, 1, 3, 2, 9)
    want = (b'{"recipient_node":7,"recipient_service":"worker","sender_node":0,"sender_service":"shepherd",'
            b'"msg_type":"StartInnerLoop","msg_id":41,"protocol_version":1,"request_id":3,"round_id":2,"task_id":9,'
            b'"data":{"tau":10,"dtype":"bf16"}}')
    assert env.to_json() == want
    framed = env.frame()
    assert framed[:4] == struct.pack("<I", len(want)) and framed[4:] == want
    back, nxt = wire.unframe(framed + b"\x05\x00")
    assert back == env and nxt == len(framed)
    assert wire.unframe(framed[:-1]) == (None, 0) and wire.unframe(framed[:3]) == (None, 0)


def test_envelope_errors():
    good = json.loads(Envelope(1, "worker", 0, "shepherd", "Heartbeat", 1, None).to_json())
    with pytest.raises(WireError):
        Envelope.from_json(json.dumps(dict(good, protocol_version=2)).encode())
    bad = dict(good)
    del bad["msg_type"]
    with pytest.raises(WireError):
        Envelope.from_json(json.dumps(bad).encode())
    with pytest.raises(WireError):
        Envelope.from_json(b"{not json")
    with pytest.raises(WireError):
        wire.unframe(struct.pack("<I", 0xFFFFFFFF) + b"x")
    # request / round / task ids default to 0 when absent (older senders)
    old = {k: v for k, v in good.items() if k not in ("request_id", "round_id", "task_id")}
    assert Envelope.from_json(json.dumps(old).encode()).round_id == 0


def test_start_inner_loop_payload_round_trip_and_defaults():
    t = InnerLoopTask(offset=4096, length=1 << 20, chunk_id=3, data_path="/data/tokens.bin", tau=50, tokenizer="u16",
                      sampling="fifo", dtype="bf16", effective_batch_size=64, raw_params=True)
    p = t.payload()
    assert list(p) == ["raw_params", "offset", "length", "chunk_id", "data_path", "tau", "tokenizer", "sampling",
                       "effective_batch_size", "use_in_graph_accumulation", "dtype"]
    assert InnerLoopTask.from_payload(json.loads(json.dumps(p))) == t
    assert t.accumulation_steps(32) == 2
    with pytest.raises(WireError):
        t.accumulation_steps(48)
    inline = InnerLoopTask(0, 10, 0, "d", 1, params=b"\x00\x01\x02\x03")
    q = inline.payload()
    assert q["params"] == base64.b64encode(b"\x00\x01\x02\x03").decode() and "raw_params" not in q
    assert InnerLoopTask.from_payload(q).params == b"\x00\x01\x02\x03"
    # optional keys of another JSON type fall back to the defaults; unknown dtypes mean f32
    r = InnerLoopTask.from_payload({"raw_params": True, "offset": 0, "length": 1, "chunk_id": 0, "data_path": "d", "tau": 2,
                                    "tokenizer": 5, "dtype": "f64", "effective_batch_size": "x"})
    assert (r.tokenizer, r.sampling, r.dtype, r.effective_batch_size, r.accumulation_steps(8)) == ("char", "random", "f32", None, 1)
    for missing in ("offset", "length", "chunk_id", "data_path", "tau"):
        bad = dict(p)
        del bad[missing]
        with pytest.raises(WireError):
            InnerLoopTask.from_payload(bad)
    with pytest.raises(WireError):
        InnerLoopTask.from_payload(dict(p, tau="10"))
    with pytest.raises(WireError):
        InnerLoopTask.from_payload({"offset": 0, "length": 1, "chunk_id": 0, "data_path": "d", "tau": 2, "params": "***"})


def test_chunk_sizes_and_message_ids():
    blob = os.urandom(2 * wire.CHUNK_SIZE + 12345)
    pays = list(wire.weight_chunk_payloads(blob))
    assert [p["chunk_index"] for p in pays] == [0, 1, 2] and all(p["total_chunks"] == 3 and p["total_bytes"] == len(blob) for p in pays)
    assert [len(base64.b64decode(p["data"])) for p in pays] == [wire.CHUNK_SIZE, wire.CHUNK_SIZE, 12345]
    req = Envelope(4, "worker", 0, "shepherd", wire.START_INNER_LOOP, 1000, {}, 1, 11, 5, 6)
    msgs = wire.update_messages(req, 4, blob, 2.5, chunk_id=5)
    assert [m.msg_type for m in msgs] == [wire.UPDATE_CHUNK] * 3 + [wire.INNER_LOOP_COMPLETE]
    assert [m.msg_id for m in msgs] == [1001, 1002, 1003, 1004]
    assert all((m.recipient_node, m.recipient_service, m.sender_node, m.sender_service) == (0, "shepherd", 4, "worker") for m in msgs)
    assert all((m.request_id, m.round_id, m.task_id) == (11, 5, 6) for m in msgs)
    assert list(msgs[0].data) == ["chunk_index", "total_chunks", "total_bytes", "data", "loss", "chunk_id"]
    assert msgs[-1].data == {"chunk_id": 5, "loss": 2.5, "chunked": True}
    # an empty delta still completes
    assert [m.msg_type for m in wire.update_messages(req, 4, b"", 0.0, 0)] == [wire.INNER_LOOP_COMPLETE]


def test_reassembly_restart_and_errors():
    r = ChunkReassembler()
    a, b = os.urandom(2500), os.urandom(1800)
    pa, pb = list(wire.weight_chunk_payloads(a, 1000)), list(wire.weight_chunk_payloads(b, 1000))
    assert r.add(9, pa[0]) is False and r.add(9, pa[1]) is False
    # a new first chunk under the same key drops the stale transfer
    assert r.add(9, pb[0]) is False and r.add(9, pb[1]) is True
    assert r.take(9) == (b, 0.0, 0) and r.take(9) is None
    with pytest.raises(WireError):
        r.add(10, pa[1])                                  # no first chunk
    with pytest.raises(WireError):
        r.add(9, {"chunk_index": 0})
    with pytest.raises(WireError):
        r.add(9, dict(pa[0], data="@@"))
    # two transfers interleaved under different keys
    for x, y in zip(pa, list(wire.weight_chunk_payloads(a[::-1], 1000))):
        r.add("k1", x)
        r.add("k2", y)
    assert r.take("k1")[0] == a and r.take("k2")[0] == a[::-1]


def test_round_trip_shepherd_worker_shepherd():
    """Parameters out in WeightChunk messages, a StartInnerLoop naming them, a worker that reassembles, 'trains' and
    answers in UpdateChunk messages, and the Shepherd-side reassembly of the delta: bytes and loss survive."""
    rng = np.random.default_rng(0)
    master = rng.standard_normal(70_000).astype(np.float32)
    stream = bytearray()
    for i, p in enumerate(wire.weight_chunk_payloads(master.tobytes(), 64 * 1024)):
        stream += Envelope(2, "worker", 0, "shepherd", wire.WEIGHT_CHUNK, 500 + i, p, 1, 77, 3, 0).frame()
    task = InnerLoopTask(0, 4096, 12, "tokens.bin", 5, "u16", "fifo", "f32", raw_params=True)
    stream += Envelope(2, "worker", 0, "shepherd", wire.START_INNER_LOOP, 600, task.payload(), 1, 77, 3, 13).frame()

    # worker
    weights, at, replies = ChunkReassembler(), 0, bytearray()
    while True:
        env, at = wire.unframe(bytes(stream), at)
        if env is None:
            break
        if env.msg_type == wire.WEIGHT_CHUNK:
            weights.add(env.request_id, env.data)
        elif env.msg_type == wire.START_INNER_LOOP:
            got = InnerLoopTask.from_payload(env.data)
            assert got == task
            theta0 = np.frombuffer(weights.take(env.request_id)[0], np.float32)
            theta = theta0 * np.float32(0.5)                     # stand-in for the inner loop
            delta = (theta0 - theta).astype(np.float32)
            for m in wire.update_messages(env, 2, delta.tobytes(), 3.25, got.chunk_id, 64 * 1024):
                replies += m.frame()
    assert at == len(stream)

    # Shepherd
    updates, at, result = ChunkReassembler(), 0, None
    while True:
        env, at = wire.unframe(bytes(replies), at)
        if env is None:
            break
        if env.msg_type == wire.UPDATE_CHUNK:
            updates.add(wire.shepherd_key(env), env.data)
        elif env.msg_type == wire.INNER_LOOP_COMPLETE:
            assert env.data["chunked"] is True and (env.request_id, env.round_id, env.task_id) == (77, 3, 13)
            result = updates.take(wire.shepherd_key(env))
    blob, loss, chunk_id = result
    np.testing.assert_array_equal(np.frombuffer(blob, np.float32), master - master * np.float32(0.5))
    assert (loss, chunk_id) == (3.25, 12)
