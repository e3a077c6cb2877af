"""Message formats of the Shepherd <-> worker TCP protocol for the training path, so that a node running this backend
can take part in a cluster of reference nodes: the envelope and its length-prefixed framing
(src/network/message.zig:46-72, src/network/tcp_stream.zig:22-98), the START_INNER_LOOP payload
(src/algorithms/diloco.zig:767-800, parsed at src/nodes/workers/worker.zig:866-946), the chunked parameter broadcast
WEIGHT_CHUNK (src/nodes/controllers/shepherd.zig:841-879, reassembled at worker.zig:491-556) and the chunked update
UPDATE_CHUNK followed by INNER_LOOP_COMPLETE (worker.zig:1413-1478, reassembled at shepherd.zig:565-643).

Host side only: bytes in, bytes out.  The compute between a START_INNER_LOOP and its reply is Backend.inner_loop."""
from __future__ import annotations

import base64
import json
import struct
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Tuple

PROTOCOL_VERSION = 1                 # message.zig:6
CHUNK_SIZE = 10 * 1024 * 1024        # worker.zig:1414, shepherd.zig:842
MAX_MESSAGE_SIZE = 4000 * 1024 * 1024  # tcp_stream.zig:61

START_INNER_LOOP = "StartInnerLoop"  # message.zig:219-237
INNER_LOOP_COMPLETE = "InnerLoopComplete"
WEIGHT_CHUNK = "WeightChunk"
UPDATE_CHUNK = "UpdateChunk"


class WireError(ValueError):
    pass


@dataclass
class Envelope:
    """MessageEnvelope (message.zig:46-57); JSON keys in the struct's field order, as std.json.stringify writes them."""
    recipient_node: int
    recipient_service: str
    sender_node: int
    sender_service: str
    msg_type: str
    msg_id: int
    data: Any
    protocol_version: int = PROTOCOL_VERSION
    request_id: int = 0
    round_id: int = 0
    task_id: int = 0

    _ORDER = ("recipient_node", "recipient_service", "sender_node", "sender_service", "msg_type", "msg_id",
              "protocol_version", "request_id", "round_id", "task_id", "data")

    def to_json(self) -> bytes:
        return json.dumps({k: getattr(self, k) for k in self._ORDER}, separators=(",", ":")).encode()

    @classmethod
    def from_json(cls, raw: bytes) -> "Envelope":
        try:
            d = json.loads(raw)
        except json.JSONDecodeError as e:
            raise WireError(f"envelope is not JSON: {e}") from None
        missing = [k for k in ("recipient_node", "recipient_service", "sender_node", "sender_service", "msg_type",
                               "msg_id", "data") if k not in d]
        if missing:
            raise WireError(f"envelope lacks {missing}")
        env = cls(**{k: d[k] for k in cls._ORDER if k in d})
        if env.protocol_version != PROTOCOL_VERSION:          # tcp_stream.zig:83-87
            raise WireError(f"protocol version {env.protocol_version}, expected {PROTOCOL_VERSION}")
        return env

    def frame(self) -> bytes:
        """u32 little-endian length, then the JSON text (tcp_stream.zig:22-47)."""
        body = self.to_json()
        if len(body) > MAX_MESSAGE_SIZE:
            raise WireError("message exceeds the size limit")
        return struct.pack("<I", len(body)) + body


def unframe(buf: bytes, at: int = 0) -> Tuple[Optional[Envelope], int]:
    """One envelope from a byte stream: (envelope, next offset), or (None, at) while the frame is incomplete."""
    if len(buf) - at < 4:
        return None, at
    (n,) = struct.unpack_from("<I", buf, at)
    if n > MAX_MESSAGE_SIZE:
        raise WireError("length prefix exceeds the size limit")
    if len(buf) - at - 4 < n:
        return None, at
    return Envelope.from_json(buf[at + 4:at + 4 + n]), at + 4 + n


def reply_to(msg: Envelope, sender_node: int, msg_type: str, msg_id: int, data: Any) -> Envelope:
    """A worker's message to the Shepherd carrying the request / round / task ids of `msg` (worker.zig contextFromMessage)."""
    return Envelope(0, "shepherd", sender_node, "worker", msg_type, msg_id, data, PROTOCOL_VERSION, msg.request_id,
                    msg.round_id, msg.task_id)


# ------------------------------------------------------------------------------------------------------------
# START_INNER_LOOP
# ------------------------------------------------------------------------------------------------------------
@dataclass
class InnerLoopTask:
    offset: int
    length: int
    chunk_id: int
    data_path: str
    tau: int
    tokenizer: str = "char"
    sampling: str = "random"
    dtype: str = "f32"
    effective_batch_size: Optional[int] = None
    use_in_graph_accumulation: bool = False
    raw_params: bool = False                 # parameters come by WEIGHT_CHUNK messages of the same request id
    params: Optional[bytes] = None           # else inline, base64 in the payload

    def payload(self) -> Dict[str, Any]:
        """diloco.zig:767-793 (key order as put there)."""
        p: Dict[str, Any] = {}
        if self.raw_params:
            p["raw_params"] = True
        else:
            p["params"] = base64.b64encode(self.params or b"").decode()
        p.update(offset=self.offset, length=self.length, chunk_id=self.chunk_id, data_path=self.data_path, tau=self.tau,
                 tokenizer=self.tokenizer, sampling=self.sampling)
        if self.effective_batch_size is not None:
            p["effective_batch_size"] = self.effective_batch_size
        p["use_in_graph_accumulation"] = self.use_in_graph_accumulation
        p["dtype"] = self.dtype
        return p

    @classmethod
    def from_payload(cls, p: Dict[str, Any]) -> "InnerLoopTask":
        """worker.zig:866-946: offset, length, chunk_id, data_path and tau are required integers / strings, the rest
        fall back to their defaults when absent or of another JSON type."""
        if not isinstance(p, dict):
            raise WireError("StartInnerLoop payload must be an object")

        def need(key, typ):
            if key not in p:
                raise WireError(f"missing {key}")
            if not isinstance(p[key], typ) or isinstance(p[key], bool):
                raise WireError(f"invalid {key}")
            return p[key]

        def opt(key, typ, default):
            v = p.get(key, default)
            return v if isinstance(v, typ) else default

        t = cls(offset=need("offset", int), length=need("length", int), chunk_id=need("chunk_id", int),
                data_path=need("data_path", str), tau=need("tau", int), tokenizer=opt("tokenizer", str, "char"),
                sampling=opt("sampling", str, "random"), dtype=opt("dtype", str, "f32"),
                use_in_graph_accumulation=opt("use_in_graph_accumulation", bool, False),
                raw_params=opt("raw_params", bool, False))
        if t.dtype not in ("bf16", "f16"):
            t.dtype = "f32"
        ebs = p.get("effective_batch_size")
        t.effective_batch_size = ebs if isinstance(ebs, int) and not isinstance(ebs, bool) else None
        if not t.raw_params:
            text = need("params", str)
            try:
                t.params = base64.b64decode(text, validate=True)
            except (ValueError, TypeError):
                raise WireError("params is not base64") from None
        return t

    def accumulation_steps(self, micro_batch: int) -> int:
        """worker.zig:921-933."""
        eff = self.effective_batch_size if self.effective_batch_size is not None else micro_batch
        if eff % micro_batch:
            raise WireError("effective batch size is not a multiple of the micro batch")
        return eff // micro_batch


# ------------------------------------------------------------------------------------------------------------
# chunked transfers: WEIGHT_CHUNK (Shepherd -> worker) and UPDATE_CHUNK + INNER_LOOP_COMPLETE (worker -> Shepherd)
# ------------------------------------------------------------------------------------------------------------
def _slices(n: int, chunk_size: int) -> Iterator[Tuple[int, int, int, int]]:
    total = (n + chunk_size - 1) // chunk_size
    for i in range(total):
        yield i, total, i * chunk_size, min((i + 1) * chunk_size, n)


def weight_chunk_payloads(blob: bytes, chunk_size: int = CHUNK_SIZE) -> Iterator[Dict[str, Any]]:
    """shepherd.zig:841-873: 10 MB slices, base64; keys chunk_index, total_chunks, data, total_bytes."""
    view = memoryview(blob)
    for i, total, lo, hi in _slices(len(view), chunk_size):
        yield {"chunk_index": i, "total_chunks": total, "data": base64.b64encode(view[lo:hi]).decode(),
               "total_bytes": len(view)}


def update_messages(request: Envelope, node_id: int, delta: bytes, loss: float, chunk_id: int,
                    chunk_size: int = CHUNK_SIZE) -> List[Envelope]:
    """What a worker sends after its inner loop (worker.zig:1413-1478): the delta blob in UPDATE_CHUNK messages with ids
    request.msg_id + 1 + i, then INNER_LOOP_COMPLETE {chunk_id, loss, chunked: true} with id request.msg_id + 1 + n."""
    view = memoryview(delta)
    out, total = [], 0
    for i, total, lo, hi in _slices(len(view), chunk_size):
        data = {"chunk_index": i, "total_chunks": total, "total_bytes": len(view),
                "data": base64.b64encode(view[lo:hi]).decode(), "loss": float(loss), "chunk_id": chunk_id}
        out.append(reply_to(request, node_id, UPDATE_CHUNK, request.msg_id + 1 + i, data))
    out.append(reply_to(request, node_id, INNER_LOOP_COMPLETE, request.msg_id + 1 + total,
                        {"chunk_id": chunk_id, "loss": float(loss), "chunked": True}))
    return out


@dataclass
class _Transfer:
    total_bytes: int
    expected: int
    received: int = 0
    parts: List[bytes] = field(default_factory=list)
    loss: float = 0.0
    chunk_id: int = 0


class ChunkReassembler:
    """Receiver of either chunked transfer.  A transfer starts at chunk_index 0 (dropping a stale one under the same key,
    worker.zig:504-511 / shepherd.zig:588-593), every chunk is appended in arrival order, and the blob is complete when
    `total_chunks` chunks have arrived.  Keys: the request id on a worker (worker.zig:497), (worker, request, round,
    task) on the Shepherd (updateKeyForMessage)."""

    def __init__(self):
        self._open: Dict[Any, _Transfer] = {}
        self._done: Dict[Any, _Transfer] = {}

    def add(self, key, payload: Dict[str, Any]) -> bool:
        """Returns True when this chunk completed the transfer."""
        try:
            idx, total, nbytes, b64 = (payload["chunk_index"], payload["total_chunks"], payload["total_bytes"],
                                       payload["data"])
        except (KeyError, TypeError):
            raise WireError("chunk payload lacks chunk_index / total_chunks / total_bytes / data") from None
        if idx == 0:
            self._open.pop(key, None)
            self._done.pop(key, None)
            t = _Transfer(int(nbytes), int(total))
            loss = payload.get("loss", 0.0)
            t.loss = float(loss) if isinstance(loss, (int, float)) and not isinstance(loss, bool) else 0.0
            t.chunk_id = int(payload.get("chunk_id", 0))
            self._open[key] = t
        t = self._open.get(key)
        if t is None:
            raise WireError("chunk without a first chunk (MissingChunkState)")
        try:
            t.parts.append(base64.b64decode(b64, validate=True))
        except (ValueError, TypeError):
            raise WireError("chunk data is not base64") from None
        t.received += 1
        if t.received == t.expected:
            self._done[key] = self._open.pop(key)
            return True
        return False

    def take(self, key) -> Optional[Tuple[bytes, float, int]]:
        """(blob, loss, chunk_id) of a completed transfer, once (shepherd.zig takeReassembledUpdateForMessage)."""
        t = self._done.pop(key, None)
        if t is None:
            return None
        return b"".join(t.parts), t.loss, t.chunk_id


def shepherd_key(msg: Envelope) -> Tuple[int, int, int, int]:
    return (msg.sender_node, msg.request_id, msg.round_id, msg.task_id)
