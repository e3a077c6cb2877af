"""ctypes binding of libpcp_b200.so, mirroring the reference's worker backend.

Method names follow src/backends/iree.zig (IreeBackend) and src/backends/worker_backend.zig
(WorkerBackend vtable) so that code written against the reference reads the same:

    IreeBackend.init / deinit                 -> Backend(device_id) / close()
    moveToDevice / allocateZerosDevice        -> move_to_device / allocate_zeros_device
    loadSession                               -> load_session
    executeWithDeviceBuffers                  -> execute_with_device_buffers
    readToHost                                -> read_to_host
    execute / executeFunction                 -> execute
    executeTrainingStep                       -> execute_training_step
    DeviceBuffer.retain/release/byteLength    -> DeviceBuffer.retain/release/byte_length

Errors raise BackendError (the reference maps every runtime failure to error.IreeRuntimeError);
the numeric code is kept in `.code`.  There is no CPU fallback: without the shared library or
without a B200 the constructor raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

F32, F64, F16, BF16, I32, I64, BOOL = range(7)
DTYPE_SIZE = {F32: 4, F64: 8, F16: 2, BF16: 2, I32: 4, I64: 8, BOOL: 1}
_NP_DTYPE = {F32: np.float32, F64: np.float64, F16: np.float16, BF16: np.uint16, I32: np.int32, I64: np.int64,
             BOOL: np.uint8}
IPC_HANDLE_BYTES = 64

E_INVALID, E_CUDA, E_ARTIFACT, E_FUNCTION, E_CHUNK_TOO_SMALL, E_CHUNK_EXHAUSTED, E_STATE, E_TOO_LARGE = range(1, 9)

LIB_PATH = os.environ.get("PCPB_LIBRARY") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libpcp_b200.so")

EXPORTS = [
    "pcpb_create", "pcpb_destroy", "pcpb_backend_type", "pcpb_last_error", "pcpb_free", "pcpb_load_artifact",
    "pcpb_inspect_artifact", "pcpb_graph_describe", "pcpb_num_params", "pcpb_param_shape", "pcpb_model_info", "pcpb_buffer_from_host", "pcpb_buffer_zeros",
    "pcpb_buffer_retain", "pcpb_buffer_release", "pcpb_buffer_nbytes", "pcpb_execute", "pcpb_read_to_host",
    "pcpb_execute_host", "pcpb_op_gemm", "pcpb_fifo_get_batch", "pcpb_set_adam", "pcpb_worker_begin_round", "pcpb_worker_set_tokens", "pcpb_worker_step",
    "pcpb_worker_end_round", "pcpb_inner_loop", "pcpb_worker_read_state", "pcpb_synchronize", "pcpb_outer_export",
    "pcpb_outer_attach_ipc", "pcpb_outer_attach_local", "pcpb_outer_prepare", "pcpb_outer_apply",
    "pcpb_launch_count", "pcpb_worker_last_loss", "pcpb_timer_start", "pcpb_timer_stop", "pcpb_profile_enable",
    "pcpb_profile_read", "pcpb_adamw_step_noalloc", "pcpb_stream_begin", "pcpb_stream_send", "pcpb_stream_outer",
    "pcpb_stream_outer_start", "pcpb_stream_outer_wait",
    "pcpb_stream_merge", "pcpb_prng_seed", "pcpb_prng_next", "pcpb_prng_uint_at_most", "pcpb_random_window_starts",
    "pcpb_random_get_batch", "pcpb_char_tokenizer_build", "pcpb_char_encode", "pcpb_char_decode",
    "pcpb_init_master_elems", "pcpb_init_master", "pcpb_worker_write_state", "pcpb_worker_set_sampling",
    "pcpb_adjoint_status", "pcpb_rollout_num_params", "pcpb_rollout_create", "pcpb_rollout_destroy", "pcpb_rollout_last_error",
    "pcpb_rollout_load_weights", "pcpb_rollout_random_weights", "pcpb_rollout_generate", "pcpb_rollout_read_logits",
    "pcpb_rollout_launch_count",
]
ADJ_CLAMPED, ADJ_INTERNAL = 1, 2
CHAR_VOCAB_MAX = 65


class BackendError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"pcp_b200 error {code}: {message}")
        self.code = code


class AdamConf(C.Structure):
    _fields_ = [("learning_rate", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("epsilon", C.c_float),
                ("weight_decay", C.c_float), ("max_grad_norm", C.c_float)]


class InnerCfg(C.Structure):
    _fields_ = [("tau", C.c_int), ("accumulation_steps", C.c_int), ("param_dtype", C.c_int),
                ("persist_adam", C.c_int), ("tokens_on_device", C.c_int)]


class OuterCfg(C.Structure):
    _fields_ = [("learning_rate", C.c_float), ("momentum", C.c_float), ("param_dtype", C.c_int)]


class Prng(C.Structure):
    """pcpb_prng: the generator of the random-window datasets and of the master initialisation."""
    _fields_ = [("s", C.c_uint64 * 4)]


class RolloutCfg(C.Structure):
    _fields_ = [("vocab", C.c_int), ("d_model", C.c_int), ("n_layer", C.c_int), ("n_head", C.c_int), ("n_kv_head", C.c_int),
                ("head_dim", C.c_int), ("d_ff", C.c_int), ("max_seq", C.c_int), ("page_tokens", C.c_int), ("max_batch", C.c_int),
                ("max_prompt", C.c_int), ("rope_theta", C.c_float), ("rms_eps", C.c_float)]


class StreamCfg(C.Structure):
    _fields_ = [("num_fragments", C.c_int), ("alpha", C.c_float), ("learning_rate", C.c_float), ("momentum", C.c_float)]


_lib = None


def load_library(path: str | None = None):
    """Loads the shared library (no GPU needed for loading) and declares the signatures."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise BackendError(E_CUDA, f"{p} not found: build it with `python -m pcp_b200.build` "
                                   "(there is no CPU fallback)")
    lib = C.CDLL(p)
    vp, i, sz = C.c_void_p, C.c_int, C.c_size_t
    lib.pcpb_create.argtypes = [i, C.POINTER(vp)]
    lib.pcpb_destroy.argtypes = [vp]; lib.pcpb_destroy.restype = None
    lib.pcpb_backend_type.argtypes = [vp]; lib.pcpb_backend_type.restype = C.c_char_p
    lib.pcpb_last_error.argtypes = [vp]; lib.pcpb_last_error.restype = C.c_char_p
    lib.pcpb_free.argtypes = [vp]; lib.pcpb_free.restype = None
    lib.pcpb_load_artifact.argtypes = [vp, vp, sz]
    lib.pcpb_inspect_artifact.argtypes = [vp, sz, C.POINTER(C.c_int64), C.c_char_p, sz]
    lib.pcpb_graph_describe.argtypes = [vp, sz, i, C.POINTER(vp), C.c_char_p, sz]
    lib.pcpb_num_params.argtypes = [vp]
    lib.pcpb_param_shape.argtypes = [vp, i, C.POINTER(C.c_int64), C.POINTER(i)]
    lib.pcpb_model_info.argtypes = [vp, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                    C.POINTER(i), C.POINTER(C.c_int64)]
    lib.pcpb_buffer_from_host.argtypes = [vp, vp, sz, C.POINTER(C.c_int64), i, i, C.POINTER(vp)]
    lib.pcpb_buffer_zeros.argtypes = [vp, C.POINTER(C.c_int64), i, i, C.POINTER(vp)]
    lib.pcpb_buffer_retain.argtypes = [vp]; lib.pcpb_buffer_retain.restype = None
    lib.pcpb_buffer_release.argtypes = [vp]; lib.pcpb_buffer_release.restype = None
    lib.pcpb_buffer_nbytes.argtypes = [vp]; lib.pcpb_buffer_nbytes.restype = sz
    lib.pcpb_execute.argtypes = [vp, C.c_char_p, C.POINTER(vp), sz, C.POINTER(C.POINTER(vp)), C.POINTER(sz)]
    lib.pcpb_read_to_host.argtypes = [vp, vp, vp, sz]
    lib.pcpb_execute_host.argtypes = [vp, C.c_char_p, C.POINTER(vp), C.POINTER(sz), C.POINTER(C.POINTER(C.c_int64)),
                                      C.POINTER(i), C.POINTER(i), sz, C.POINTER(C.POINTER(vp)),
                                      C.POINTER(C.POINTER(sz)), C.POINTER(sz)]
    ll = C.c_longlong
    lib.pcpb_op_gemm.argtypes = [vp, i, vp, ll, ll, vp, ll, ll, vp, ll, vp, vp, i, i, i, i]
    lib.pcpb_fifo_get_batch.argtypes = [vp, vp, sz, C.POINTER(sz), C.POINTER(vp), C.POINTER(vp)]
    lib.pcpb_set_adam.argtypes = [vp, C.POINTER(AdamConf)]
    lib.pcpb_worker_begin_round.argtypes = [vp, C.POINTER(InnerCfg), vp, sz]
    lib.pcpb_worker_set_tokens.argtypes = [vp, vp, sz]
    lib.pcpb_worker_step.argtypes = [vp]
    lib.pcpb_worker_end_round.argtypes = [vp, vp, sz, vp, sz]
    lib.pcpb_inner_loop.argtypes = [vp, C.POINTER(InnerCfg), vp, sz, vp, sz, vp, sz, vp]
    lib.pcpb_worker_read_state.argtypes = [vp, i, vp, sz]
    lib.pcpb_synchronize.argtypes = [vp]
    lib.pcpb_outer_export.argtypes = [vp, vp]
    lib.pcpb_outer_attach_ipc.argtypes = [vp, i, i, vp]
    lib.pcpb_outer_attach_local.argtypes = [vp, i, i, C.POINTER(vp)]
    lib.pcpb_outer_prepare.argtypes = [vp, C.POINTER(OuterCfg)]
    lib.pcpb_outer_apply.argtypes = [vp, C.POINTER(OuterCfg), C.POINTER(i), i, C.POINTER(C.c_double)]
    lib.pcpb_launch_count.argtypes = [vp]; lib.pcpb_launch_count.restype = C.c_longlong
    lib.pcpb_worker_last_loss.argtypes = [vp, C.POINTER(C.c_float)]
    lib.pcpb_timer_start.argtypes = [vp]
    lib.pcpb_timer_stop.argtypes = [vp, C.POINTER(C.c_double)]
    lib.pcpb_stream_begin.argtypes = [vp, C.POINTER(StreamCfg)]
    lib.pcpb_stream_send.argtypes = [vp, i]
    lib.pcpb_stream_outer.argtypes = [vp, i, C.POINTER(C.c_double)]
    lib.pcpb_stream_outer_start.argtypes = [vp, i]
    lib.pcpb_stream_outer_wait.argtypes = [vp, i, C.POINTER(C.c_double)]
    lib.pcpb_stream_merge.argtypes = [vp, i]
    lib.pcpb_profile_enable.argtypes = [vp, i]
    lib.pcpb_profile_read.argtypes = [vp, C.POINTER(C.c_longlong), C.POINTER(C.c_double), C.POINTER(C.c_double)]
    lib.pcpb_adamw_step_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ll, C.POINTER(AdamConf), C.c_float,
                                            C.c_char_p, sz]
    u64 = C.c_uint64
    lib.pcpb_prng_seed.argtypes = [C.POINTER(Prng), u64]; lib.pcpb_prng_seed.restype = None
    lib.pcpb_prng_next.argtypes = [C.POINTER(Prng)]; lib.pcpb_prng_next.restype = u64
    lib.pcpb_prng_uint_at_most.argtypes = [C.POINTER(Prng), u64]; lib.pcpb_prng_uint_at_most.restype = u64
    lib.pcpb_random_window_starts.argtypes = [C.POINTER(Prng), sz, sz, sz, C.POINTER(u64)]
    lib.pcpb_random_get_batch.argtypes = [vp, C.POINTER(Prng), vp, i, sz, C.POINTER(vp), C.POINTER(vp)]
    lib.pcpb_char_tokenizer_build.argtypes = [vp, sz, vp, C.POINTER(i), C.POINTER(i)]
    lib.pcpb_char_encode.argtypes = [vp, i, vp, sz, vp]
    lib.pcpb_char_decode.argtypes = [vp, i, vp, sz, vp]
    lib.pcpb_init_master_elems.argtypes = [u64, i, sz, vp, sz]
    lib.pcpb_init_master.argtypes = [vp, u64, i, vp, sz]
    lib.pcpb_worker_write_state.argtypes = [vp, i, vp, sz]
    lib.pcpb_worker_set_sampling.argtypes = [vp, i, u64]
    if hasattr(lib, "pcpb_rollout_create"):
        rc = C.POINTER(RolloutCfg)
        lib.pcpb_rollout_num_params.argtypes = [rc]; lib.pcpb_rollout_num_params.restype = C.c_longlong
        lib.pcpb_rollout_create.argtypes = [i, rc, C.POINTER(vp)]
        lib.pcpb_rollout_destroy.argtypes = [vp]; lib.pcpb_rollout_destroy.restype = None
        lib.pcpb_rollout_last_error.argtypes = [vp]; lib.pcpb_rollout_last_error.restype = C.c_char_p
        lib.pcpb_rollout_load_weights.argtypes = [vp, vp, sz, i]
        lib.pcpb_rollout_random_weights.argtypes = [vp, u64, C.c_float]
        lib.pcpb_rollout_generate.argtypes = [vp, vp, vp, i, i, i, C.c_int64, C.c_float, vp, vp, vp, C.POINTER(C.c_double),
                                              C.POINTER(C.c_double)]
        lib.pcpb_rollout_read_logits.argtypes = [vp, i, vp, sz]
        lib.pcpb_rollout_launch_count.argtypes = [vp]; lib.pcpb_rollout_launch_count.restype = C.c_longlong
    if hasattr(lib, "pcpb_adjoint_status"):              # absent from older builds of the library (PCPB_LIBRARY)
        lib.pcpb_adjoint_status.argtypes = [vp, C.POINTER(i), i]
    if path is None:
        _lib = lib
    return lib


class RandomGenerator:
    """std.Random.DefaultPrng stand-in of the library (xoshiro256++ / SplitMix64; unpinned against Zig's)."""

    def __init__(self, seed: int):
        self._lib = load_library()
        self.state = Prng()
        self._lib.pcpb_prng_seed(C.byref(self.state), seed)

    def next(self) -> int:
        return int(self._lib.pcpb_prng_next(C.byref(self.state)))

    def uint_at_most(self, at_most: int) -> int:
        return int(self._lib.pcpb_prng_uint_at_most(C.byref(self.state), at_most))

    def window_starts(self, n_tokens: int, batch: int, block: int) -> np.ndarray:
        out = np.empty(batch, np.uint64)
        rc = self._lib.pcpb_random_window_starts(C.byref(self.state), n_tokens, batch, block,
                                                 out.ctypes.data_as(C.POINTER(C.c_uint64)))
        if rc:
            raise BackendError(rc, "ChunkTooSmall" if rc == E_CHUNK_TOO_SMALL else "bad arguments")
        return out


class CharTokenizer:
    """CharTokenizer of src/data/loader.zig:12-89 (host function of the library)."""

    def __init__(self, text: bytes):
        self._lib = load_library()
        raw = np.frombuffer(text, np.uint8)
        self._chars = np.zeros(CHAR_VOCAB_MAX, np.uint8)
        n, ign = C.c_int(), C.c_int()
        rc = self._lib.pcpb_char_tokenizer_build(raw.ctypes.data, raw.size, self._chars.ctypes.data, C.byref(n), C.byref(ign))
        if rc:
            raise BackendError(rc, "char tokenizer: bad arguments")
        self.vocab_size, self.ignored = n.value, ign.value

    @property
    def chars(self):
        return [int(c) for c in self._chars[: self.vocab_size]]

    def encode(self, text: bytes) -> np.ndarray:
        raw = np.frombuffer(text, np.uint8)
        out = np.empty(raw.size, np.uint32)
        rc = self._lib.pcpb_char_encode(self._chars.ctypes.data, self.vocab_size, raw.ctypes.data, raw.size, out.ctypes.data)
        if rc:
            raise BackendError(rc, "char encode: bad arguments")
        return out

    def decode(self, tokens) -> bytes:
        tok = np.ascontiguousarray(tokens, np.uint32)
        out = np.empty(tok.size, np.uint8)
        rc = self._lib.pcpb_char_decode(self._chars.ctypes.data, self.vocab_size, tok.ctypes.data, tok.size, out.ctypes.data)
        if rc:
            raise BackendError(rc, "UnknownToken")
        return out.tobytes()


def init_master_elems(seed: int, n: int, dtype=F32) -> np.ndarray:
    """n elements of 0.02 * N(0,1) (src/algorithms/diloco.zig:513-586): float32 values or bf16 bit patterns."""
    lib = load_library()
    out = np.empty(n, np.float32 if dtype == F32 else np.uint16)
    rc = lib.pcpb_init_master_elems(seed, dtype, n, out.ctypes.data, out.nbytes)
    if rc:
        raise BackendError(rc, "init_master: bad arguments")
    return out


def inspect_artifact(artifact) -> dict:
    """Model facts of a forward graph, parsed on the host (no GPU needed)."""
    lib = load_library()
    raw = artifact.encode() if isinstance(artifact, str) else artifact
    facts = (C.c_int64 * 12)()
    err = C.create_string_buffer(512)
    rc = lib.pcpb_inspect_artifact(raw, len(raw), facts, err, 512)
    if rc:
        raise BackendError(rc, err.value.decode())
    keys = ["vocab", "d_model", "n_layer", "n_head", "n_kv_head", "head_dim", "d_ff", "batch", "block", "dtype",
            "num_tensors", "total_params"]
    out = dict(zip(keys, [int(x) for x in facts]))
    out["family"] = "graph" if out["d_model"] == 0 else "fused"      # graph: run op by op by the general front end
    return out


def graph_describe(artifact, with_gradients: bool = True, with_plan: bool = False) -> str:
    """The general front end's tensor program of a forward graph as text, with_plan: followed by the executor's plan
    of it (see include/pcp_b200.h); no GPU needed."""
    lib = load_library()
    raw = artifact.encode() if isinstance(artifact, str) else artifact
    text = C.c_void_p()
    err = C.create_string_buffer(512)
    rc = lib.pcpb_graph_describe(raw, len(raw), 2 if with_plan else (1 if with_gradients else 0), C.byref(text), err, 512)
    if rc:
        raise BackendError(rc, err.value.decode())
    try:
        return C.string_at(text).decode()
    finally:
        lib.pcpb_free(text)


NOALLOC_MAX_ELEMS = 1 << 26


def adamw_step_noalloc(p, g, m, v, p_out, m_out, v_out, n, conf: AdamConf, timestep: float, stream=None):
    """AdamW on caller-owned device memory without any allocation (see include/pcp_b200.h).  Arguments are raw
    device addresses (ints); `stream` a cudaStream_t value or None.  The work is enqueued, not waited for."""
    lib = load_library()
    err = C.create_string_buffer(256)
    rc = lib.pcpb_adamw_step_noalloc(stream, p, g, m, v, p_out, m_out, v_out, n, C.byref(conf), timestep, err, 256)
    if rc:
        raise BackendError(rc, err.value.decode())


class DeviceBuffer:
    """One reference to a device buffer (src/backends/iree.zig:53-69)."""

    def __init__(self, lib, handle, shape=None, dtype=None):
        self._lib, self.handle, self.shape, self.dtype = lib, handle, shape, dtype
        self._refs = 1                      # references this object holds on the native buffer

    def retain(self):
        self._lib.pcpb_buffer_retain(self.handle)
        self._refs += 1

    def release(self):
        if self.handle:
            self._lib.pcpb_buffer_release(self.handle)
            self._refs -= 1
            if self._refs == 0:
                self.handle = None

    def byte_length(self):
        return self._lib.pcpb_buffer_nbytes(self.handle)


def _as_bytes_array(x):
    a = np.ascontiguousarray(x)
    return a, a.ctypes.data, a.nbytes


class Backend:
    def __init__(self, device_id: int = 0):
        self._lib = load_library()
        h = C.c_void_p()
        rc = self._lib.pcpb_create(device_id, C.byref(h))
        self._h = h
        if rc:
            msg = self._lib.pcpb_last_error(h).decode() if h else "allocation failed"
            if h:
                self._lib.pcpb_destroy(h)
            self._h = None
            raise BackendError(rc, msg)
        self._artifact = None

    # -- plumbing
    def _check(self, rc):
        if rc:
            raise BackendError(rc, self._lib.pcpb_last_error(self._h).decode())

    def close(self):
        if getattr(self, "_h", None):
            self._lib.pcpb_destroy(self._h)
            self._h = None

    deinit = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def get_backend_type(self):
        return self._lib.pcpb_backend_type(self._h).decode()

    @property
    def launch_count(self):
        return int(self._lib.pcpb_launch_count(self._h))

    # -- artefact
    def load_session(self, artifact):
        if isinstance(artifact, str):
            artifact = artifact.encode()
        self._artifact_raw = artifact
        self._artifact = C.create_string_buffer(artifact, len(artifact))      # keeps (ptr, len) stable
        self._check(self._lib.pcpb_load_artifact(self._h, C.cast(self._artifact, C.c_void_p), len(artifact)))

    def _ensure_session(self, artifact):
        if artifact is None:
            return
        raw = artifact.encode() if isinstance(artifact, str) else artifact
        if self._artifact is None or self._artifact_raw != raw:
            self.load_session(raw)

    def num_params(self):
        return self._lib.pcpb_num_params(self._h)

    def param_shapes(self):
        out = []
        shp = (C.c_int64 * 8)()
        rank = C.c_int()
        for k in range(self.num_params()):
            self._check(self._lib.pcpb_param_shape(self._h, k, shp, C.byref(rank)))
            out.append(tuple(shp[j] for j in range(rank.value)))
        return out

    def model_info(self):
        b, t, v, n = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64()
        dt = C.c_int()
        self._check(self._lib.pcpb_model_info(self._h, C.byref(b), C.byref(t), C.byref(v), C.byref(dt), C.byref(n)))
        return {"batch": b.value, "block": t.value, "vocab": v.value, "dtype": dt.value, "total_params": n.value}

    # -- buffers
    def move_to_device(self, data, shape, dtype) -> DeviceBuffer:
        a, ptr, nbytes = _as_bytes_array(data)
        shp = (C.c_int64 * max(len(shape), 1))(*shape)
        h = C.c_void_p()
        self._check(self._lib.pcpb_buffer_from_host(self._h, ptr, nbytes, shp, len(shape), dtype, C.byref(h)))
        return DeviceBuffer(self._lib, h, tuple(shape), dtype)

    def allocate_zeros_device(self, shape, dtype) -> DeviceBuffer:
        shp = (C.c_int64 * max(len(shape), 1))(*shape)
        h = C.c_void_p()
        self._check(self._lib.pcpb_buffer_zeros(self._h, shp, len(shape), dtype, C.byref(h)))
        return DeviceBuffer(self._lib, h, tuple(shape), dtype)

    def read_to_host(self, buf: DeviceBuffer, dtype=None, shape=None) -> np.ndarray:
        n = buf.byte_length()
        raw = np.empty(n, dtype=np.uint8)
        self._check(self._lib.pcpb_read_to_host(self._h, buf.handle, raw.ctypes.data, n))
        dt = dtype if dtype is not None else buf.dtype
        if dt is None:
            return raw
        out = raw.view(_NP_DTYPE[dt])
        shp = shape if shape is not None else buf.shape
        return out.reshape(shp) if shp is not None else out

    # -- execution
    def execute_with_device_buffers(self, artifact, fn_name: str, inputs):
        self._ensure_session(artifact)
        arr = (C.c_void_p * max(len(inputs), 1))(*[b.handle for b in inputs])
        out = C.POINTER(C.c_void_p)()
        n = C.c_size_t()
        self._check(self._lib.pcpb_execute(self._h, fn_name.encode(), arr, len(inputs), C.byref(out), C.byref(n)))
        res = [DeviceBuffer(self._lib, C.c_void_p(out[k])) for k in range(n.value)]
        self._lib.pcpb_free(out)
        return res

    def execute(self, artifact, fn_name: str, inputs_data, input_shapes, input_dtypes=None):
        """Host bytes in, host bytes out (list of uint8 arrays)."""
        self._ensure_session(artifact)
        n = len(inputs_data)
        keep = [_as_bytes_array(x) for x in inputs_data]
        ptrs = (C.c_void_p * n)(*[k[1] for k in keep])
        sizes = (C.c_size_t * n)(*[k[2] for k in keep])
        shp_arrs = [(C.c_int64 * max(len(s), 1))(*s) for s in input_shapes]
        shps = (C.POINTER(C.c_int64) * n)(*[C.cast(a, C.POINTER(C.c_int64)) for a in shp_arrs])
        ranks = (C.c_int * n)(*[len(s) for s in input_shapes])
        dts = (C.c_int * n)(*input_dtypes) if input_dtypes is not None else None
        out = C.POINTER(C.c_void_p)()
        onb = C.POINTER(C.c_size_t)()
        no = C.c_size_t()
        self._check(self._lib.pcpb_execute_host(self._h, fn_name.encode(), ptrs, sizes, shps, ranks, dts, n,
                                                C.byref(out), C.byref(onb), C.byref(no)))
        res = []
        for k in range(no.value):
            res.append(np.ctypeslib.as_array(C.cast(out[k], C.POINTER(C.c_uint8)), shape=(onb[k],)).copy())
            self._lib.pcpb_free(out[k])
        self._lib.pcpb_free(out)
        self._lib.pcpb_free(onb)
        return res

    def execute_function(self, artifact, function_name, inputs, shapes, dtypes=None):
        return self.execute(artifact, function_name, inputs, shapes, dtypes)

    def execute_training_step(self, artifact, inputs, shapes, dtypes=None):
        return self.execute(artifact, "main", inputs, shapes, dtypes)

    def op_gemm(self, A, sam, sak, B, sbk, sbn, Cbuf, ldc, M, N, K, epilogue=0, R=None, C2=None, path=0):
        self._check(self._lib.pcpb_op_gemm(self._h, path, A.handle, sam, sak, B.handle, sbk, sbn, Cbuf.handle, ldc,
                                           R.handle if R else None, C2.handle if C2 else None, M, N, K, epilogue))

    def fifo_get_batch(self, tokens: np.ndarray, cursor: int):
        """-> (inputs DeviceBuffer, targets DeviceBuffer, new cursor); tokens: host uint16 array."""
        tok = np.ascontiguousarray(tokens, dtype=np.uint16)
        cur = C.c_size_t(cursor)
        x, y = C.c_void_p(), C.c_void_p()
        self._check(self._lib.pcpb_fifo_get_batch(self._h, tok.ctypes.data, tok.size, C.byref(cur), C.byref(x), C.byref(y)))
        info = self.model_info()
        shp = (info["batch"], info["block"])
        return DeviceBuffer(self._lib, x, shp, I64), DeviceBuffer(self._lib, y, shp, I64), cur.value

    def random_get_batch(self, gen: RandomGenerator, tokens: np.ndarray):
        """-> (inputs DeviceBuffer, targets DeviceBuffer); tokens: host uint16 or uint32 array (the worker's chunk)."""
        tok = np.ascontiguousarray(tokens)
        if tok.dtype not in (np.uint16, np.uint32):
            raise ValueError("tokens must be uint16 or uint32")
        x, y = C.c_void_p(), C.c_void_p()
        self._check(self._lib.pcpb_random_get_batch(self._h, C.byref(gen.state), tok.ctypes.data, tok.dtype.itemsize,
                                                    tok.size, C.byref(x), C.byref(y)))
        info = self.model_info()
        shp = (info["batch"], info["block"])
        return DeviceBuffer(self._lib, x, shp, I64), DeviceBuffer(self._lib, y, shp, I64)

    def init_master(self, seed: int = 12345, param_dtype=F32) -> np.ndarray:
        """The Shepherd's initial master parameters for the loaded model as a blob for worker_begin_round."""
        P = self.model_info()["total_params"]
        out = np.empty(P, np.float32 if param_dtype == F32 else np.uint16)
        self._check(self._lib.pcpb_init_master(self._h, seed, param_dtype, out.ctypes.data, out.nbytes))
        return out

    def worker_set_sampling(self, mode: str = "fifo", seed: int = 0):
        self._check(self._lib.pcpb_worker_set_sampling(self._h, {"fifo": 0, "random": 1}[mode], seed))

    def set_adam(self, learning_rate=1e-3, beta1=0.9, beta2=0.999, epsilon=1e-8, weight_decay=0.01,
                 max_grad_norm=1.0):
        conf = AdamConf(learning_rate, beta1, beta2, epsilon, weight_decay, max_grad_norm)
        self._check(self._lib.pcpb_set_adam(self._h, C.byref(conf)))

    def synchronize(self):
        self._check(self._lib.pcpb_synchronize(self._h))

    def adjoint_status(self, clear=True) -> int:
        """Bits ADJ_CLAMPED / ADJ_INTERNAL: whether the reference's finite guard or +-100 clamp on adjoint edges
        (src/autodiff/engine.zig:604-702) was active since the last clear."""
        f = C.c_int()
        self._check(self._lib.pcpb_adjoint_status(self._h, C.byref(f), int(clear)))
        return f.value

    # -- fused worker round (Worker.handleStartInnerLoop, src/nodes/workers/worker.zig:855-1480)
    def worker_begin_round(self, tau, params_blob=None, param_dtype=F32, accumulation_steps=1, persist_adam=False,
                           tokens_on_device=False):
        cfg = InnerCfg(tau, accumulation_steps, param_dtype, int(persist_adam), int(tokens_on_device))
        if params_blob is None:
            self._check(self._lib.pcpb_worker_begin_round(self._h, C.byref(cfg), None, 0))
        else:
            a, ptr, nbytes = _as_bytes_array(params_blob)
            self._check(self._lib.pcpb_worker_begin_round(self._h, C.byref(cfg), ptr, nbytes))

    def worker_set_tokens(self, tokens=None, device_ptr=None, n_tokens=None):
        if device_ptr is not None:
            self._check(self._lib.pcpb_worker_set_tokens(self._h, device_ptr, n_tokens))
            return
        self._tokens = np.ascontiguousarray(tokens, dtype=np.uint16)          # must outlive the round
        self._check(self._lib.pcpb_worker_set_tokens(self._h, self._tokens.ctypes.data, self._tokens.size))

    def worker_step(self):
        self._check(self._lib.pcpb_worker_step(self._h))

    def worker_last_loss(self) -> float:
        v = C.c_float()
        self._check(self._lib.pcpb_worker_last_loss(self._h, C.byref(v)))
        return v.value

    def timer_start(self):
        self._check(self._lib.pcpb_timer_start(self._h))

    def timer_stop(self) -> float:
        ms = C.c_double()
        self._check(self._lib.pcpb_timer_stop(self._h, C.byref(ms)))
        return ms.value

    def profile_enable(self, on=True):
        self._check(self._lib.pcpb_profile_enable(self._h, int(on)))

    def profile_read(self):
        n, ms, fl = C.c_longlong(), C.c_double(), C.c_double()
        self._check(self._lib.pcpb_profile_read(self._h, C.byref(n), C.byref(ms), C.byref(fl)))
        return {"launches": n.value, "ms": ms.value, "flops": fl.value}

    def worker_end_round(self, steps, param_dtype=F32, want_delta=True, out=None):
        """-> (delta blob, per-step losses).  `out`: a caller-owned array for the delta (e.g. a view of pinned host
        memory, which the device -> host copy fills at full PCIe rate and without first-touch page faults)."""
        P = self.model_info()["total_params"]
        losses = np.zeros(max(steps, 1), dtype=np.float32)
        if want_delta:
            dt = np.float32 if param_dtype == F32 else np.uint16
            if out is not None:
                if out.dtype != dt or out.size != P or not out.flags["C_CONTIGUOUS"]:
                    raise ValueError("out must be a contiguous array of the delta's dtype and length")
                delta = out
            else:
                delta = np.empty(P, dtype=dt)
            self._check(self._lib.pcpb_worker_end_round(self._h, delta.ctypes.data, delta.nbytes, losses.ctypes.data, steps))
        else:
            delta = None
            self._check(self._lib.pcpb_worker_end_round(self._h, None, 0, losses.ctypes.data, steps))
        return delta, losses[:steps]

    def inner_loop(self, params_blob, tokens, tau, param_dtype=F32, accumulation_steps=1):
        cfg = InnerCfg(tau, accumulation_steps, param_dtype, 0, 0)
        a, ptr, nbytes = _as_bytes_array(params_blob)
        tok = np.ascontiguousarray(tokens, dtype=np.uint16)
        P = self.model_info()["total_params"]
        delta = np.empty(P, dtype=np.float32 if param_dtype == F32 else np.uint16)
        losses = np.zeros(max(tau, 1), dtype=np.float32)
        self._check(self._lib.pcpb_inner_loop(self._h, C.byref(cfg), ptr, nbytes, tok.ctypes.data, tok.size,
                                              delta.ctypes.data, delta.nbytes, losses.ctypes.data))
        return delta, losses[:tau]

    def worker_read_state(self, which: str):
        sel = {"params": 0, "m": 1, "v": 2, "delta": 3, "master": 4, "velocity": 5, "grads": 6}[which]
        n = self.model_info()["total_params"] if sel != 5 else self._shard_len
        out = np.empty(n, dtype=np.float32)
        self._check(self._lib.pcpb_worker_read_state(self._h, sel, out.ctypes.data, n))
        return out

    def worker_write_state(self, which: str, values):
        sel = {"params": 0, "m": 1, "v": 2, "delta": 3, "master": 4, "velocity": 5}[which]
        a = np.ascontiguousarray(values, np.float32)
        self._check(self._lib.pcpb_worker_write_state(self._h, sel, a.ctypes.data, a.size))

    def load_recovery(self, path: str):
        """Restores a run from the Shepherd's recovery file (src/algorithms/diloco.zig:1063-1107): the master
        parameters become the next round's start and this rank's slice of the Nesterov velocities is written into
        its shard (attach the outer step first).  -> (parameter blob dtype code, data-manager bytes)."""
        from . import formats
        from .diloco import shard_range
        params, vels, data_manager = formats.read_recovery(path, self.param_shapes())
        if not params:
            raise BackendError(1, "recovery file holds no parameters")
        flat = np.concatenate([t.reshape(-1) for t in params])
        dt = BF16 if flat.dtype == np.uint16 else F32
        master = (flat.astype(np.uint32) << 16).view(np.float32) if dt == BF16 else flat.astype(np.float32)
        self.worker_write_state("master", master)
        if vels is not None and hasattr(self, "_shard_len"):
            v = np.concatenate([np.asarray(t, np.float32).reshape(-1) for t in vels])
            lo, hi = shard_range(v.size, self._world, self._rank)
            shard = np.zeros(self._shard_len, np.float32)
            shard[: hi - lo] = v[lo:hi]
            self.worker_write_state("velocity", shard)
        return dt, data_manager

    # -- checkpoints in the reference's file format (pcp_b200/formats.py)
    def save_checkpoint(self, path: str, param_dtype=F32):
        """Writes the master parameters on the device as a `checkpoint_<step>.bin` file of the reference
        (src/algorithms/diloco.zig:590-628): f32, or bf16 bit patterns (truncated, as the Shepherd keeps them)."""
        from . import formats
        flat = self.worker_read_state("master")
        if param_dtype == BF16:
            flat = (flat.view(np.uint32) >> 16).astype(np.uint16)
        formats.write_checkpoint(path, formats.split_flat(flat, self.param_shapes()))

    def load_checkpoint(self, path: str):
        """-> (parameter blob for worker_begin_round, its dtype code), checked against the loaded artefact's shapes."""
        from . import formats
        tensors = formats.read_checkpoint(path)
        shapes = self.param_shapes()
        if [tuple(t.shape) for t in tensors] != [tuple(s) for s in shapes]:
            raise BackendError(1, "checkpoint shapes do not match the artefact")
        dts = {t.dtype for t in tensors}
        if len(dts) != 1:
            raise BackendError(1, "checkpoint mixes parameter dtypes")
        blob = np.concatenate([t.reshape(-1) for t in tensors])
        return blob, (BF16 if blob.dtype == np.uint16 else F32)

    # -- outer step
    def outer_export(self) -> bytes:
        buf = C.create_string_buffer(2 * IPC_HANDLE_BYTES)
        self._check(self._lib.pcpb_outer_export(self._h, buf))
        return buf.raw

    def _set_shard(self, world, rank=0):
        self._world, self._rank = world, rank
        P = self.model_info()["total_params"]
        s = (P + world - 1) // world
        self._shard_len = (s + 255) // 256 * 256

    def outer_attach_ipc(self, rank, world, all_handles: bytes):
        self._check(self._lib.pcpb_outer_attach_ipc(self._h, rank, world, all_handles))
        self._set_shard(world, rank)

    def outer_attach_local(self, rank, peers):
        arr = (C.c_void_p * len(peers))(*[p._h for p in peers])
        self._check(self._lib.pcpb_outer_attach_local(self._h, rank, len(peers), arr))
        self._set_shard(len(peers), rank)

    def outer_prepare(self, learning_rate=0.7, momentum=0.9, param_dtype=F32):
        cfg = OuterCfg(learning_rate, momentum, param_dtype)
        self._check(self._lib.pcpb_outer_prepare(self._h, C.byref(cfg)))

    # ---- streaming DiLoCo (worker.zig:2207-2610): fragment-wise send / outer step / merge inside a round ----
    def stream_begin(self, num_fragments=4, alpha=0.5, learning_rate=0.7, momentum=0.9):
        cfg = StreamCfg(num_fragments, alpha, learning_rate, momentum)
        self._check(self._lib.pcpb_stream_begin(self._h, C.byref(cfg)))

    def stream_send(self, fragment: int):
        self._check(self._lib.pcpb_stream_send(self._h, int(fragment)))

    def stream_outer(self, fragment: int) -> float:
        ms = C.c_double()
        self._check(self._lib.pcpb_stream_outer(self._h, int(fragment), C.byref(ms)))
        return ms.value

    def stream_outer_start(self, fragment: int):
        """The fragment's outer step on a side stream; returns at once (pair with stream_outer_wait before the merge)."""
        self._check(self._lib.pcpb_stream_outer_start(self._h, int(fragment)))

    def stream_outer_wait(self, fragment: int) -> float:
        ms = C.c_double(0.0)
        self._check(self._lib.pcpb_stream_outer_wait(self._h, int(fragment), C.byref(ms)))
        return ms.value

    def stream_merge(self, fragment: int):
        self._check(self._lib.pcpb_stream_merge(self._h, int(fragment)))

    def outer_apply(self, learning_rate=0.7, momentum=0.9, param_dtype=F32, contributors=None) -> float:
        cfg = OuterCfg(learning_rate, momentum, param_dtype)
        ms = C.c_double()
        if contributors is None:
            self._check(self._lib.pcpb_outer_apply(self._h, C.byref(cfg), None, 0, C.byref(ms)))
        else:
            arr = (C.c_int * len(contributors))(*contributors)
            self._check(self._lib.pcpb_outer_apply(self._h, C.byref(cfg), arr, len(contributors), C.byref(ms)))
        return ms.value


class Rollout:
    """GenerationEngine of the reference (src/nodes/workers/generation_engine.zig) on the device: batched prefill, paged
    KV cache, greedy decode, for a Qwen3-shaped bf16 model.  Method names follow the reference:
    ensureDeviceWeights -> ensure_device_weights, generateRollout -> generate_rollout."""

    def __init__(self, device_id: int, vocab, d_model, n_layer, n_head, n_kv_head, head_dim, d_ff, max_seq, max_batch=16,
                 max_prompt=None, page_tokens=16, rope_theta=1e6, rms_eps=1e-6):
        self._lib = load_library()
        self.cfg = RolloutCfg(vocab, d_model, n_layer, n_head, n_kv_head, head_dim, d_ff, max_seq, page_tokens, max_batch,
                              max_prompt if max_prompt is not None else max_seq, rope_theta, rms_eps)
        h = C.c_void_p()
        rc = self._lib.pcpb_rollout_create(device_id, C.byref(self.cfg), C.byref(h))
        self._h = h
        if rc:
            msg = self._lib.pcpb_rollout_last_error(h).decode() if h else "allocation failed"
            if h:
                self._lib.pcpb_rollout_destroy(h)
            self._h = None
            raise BackendError(rc, msg)

    def _check(self, rc):
        if rc:
            raise BackendError(rc, self._lib.pcpb_rollout_last_error(self._h).decode())

    def close(self):
        if getattr(self, "_h", None):
            self._lib.pcpb_rollout_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def num_params(self) -> int:
        return int(self._lib.pcpb_rollout_num_params(C.byref(self.cfg)))

    @property
    def launch_count(self) -> int:
        return int(self._lib.pcpb_rollout_launch_count(self._h))

    def ensure_device_weights(self, blob: np.ndarray):
        """blob: all weights concatenated in argument order, float32 or uint16 (bf16 bit patterns)."""
        a = np.ascontiguousarray(blob)
        if a.dtype not in (np.float32, np.uint16):
            raise ValueError("weight blob must be float32 or bf16 bit patterns (uint16)")
        self._check(self._lib.pcpb_rollout_load_weights(self._h, a.ctypes.data, a.nbytes, F32 if a.dtype == np.float32 else BF16))

    def random_weights(self, seed: int = 0, std: float = 0.02):
        self._check(self._lib.pcpb_rollout_random_weights(self._h, seed, std))

    def generate_rollout(self, prompts, max_new_tokens: int, eos_token: int = -1, temperature: float = 0.0):
        """prompts: list of token-id lists.  -> (list of generated token lists, list of finish reasons, (prefill ms,
        decode ms))."""
        B = len(prompts)
        stride = max(1, max(len(p) for p in prompts))
        buf = np.zeros((B, stride), np.int64)
        lens = np.zeros(B, np.int32)
        for b, p in enumerate(prompts):
            buf[b, :len(p)] = p
            lens[b] = len(p)
        out = np.zeros((B, max_new_tokens), np.int64)
        n = np.zeros(B, np.int32)
        why = np.zeros(B, np.int32)
        pm, dm = C.c_double(), C.c_double()
        self._check(self._lib.pcpb_rollout_generate(self._h, buf.ctypes.data, lens.ctypes.data, B, stride, max_new_tokens, eos_token,
                                                    temperature, out.ctypes.data, n.ctypes.data, why.ctypes.data, C.byref(pm),
                                                    C.byref(dm)))
        return ([out[b, :n[b]].tolist() for b in range(B)], ["stop" if w else "length" for w in why], (pm.value, dm.value))

    def read_logits(self, row: int) -> np.ndarray:
        out = np.empty(self.cfg.vocab, np.float32)
        self._check(self._lib.pcpb_rollout_read_logits(self._h, row, out.ctypes.data, out.size))
        return out
