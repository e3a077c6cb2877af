/* pcp_b200 — C ABI of the B200 execution backend for PCP's training hot path.
 *
 * Drop-in boundary: what the reference's worker reaches through its backend object
 * (src/backends/worker_backend.zig:11-41 vtable, src/backends/iree.zig:53-442 concrete methods,
 * pointer-cast at src/nodes/workers/worker.zig:1105).  Every entry point returns 0 on success or a
 * non-zero PCPB_E_* code; the message is available from pcpb_last_error().  Nothing aborts, traps or
 * falls back to the CPU.  A backend instance is not thread-safe (neither is the reference's); several
 * instances per process are supported, one per GPU process is the normal deployment
 * (src/nodes/node_manager.zig:65-107).
 *
 * The artefact given to pcpb_load_artifact is the forward StableHLO text of the model (the text the
 * Shepherd holds before compiling, src/algorithms/diloco.zig:153), of the nanochat family (RMSNorm, RoPE,
 * QK-norm, ReLU^2, soft-capped loss) or the nanoGPT family (LayerNorm, learned positions, ReLU or tanh-GELU MLP,
 * biased head).  The backend recognises the model from the @main signature, the RoPE table resources, the
 * soft-cap constant and the activation's ops, and implements for it the functions the reference's graph builder emits
 * (src/compiler/graph_builder.zig:56-278), including the sanitiser's and the autodiff engine's guard
 * terms (src/compiler/sanitizer.zig:8-111, src/autodiff/vjp_rules.zig), with fused kernels.  Any other forward graph
 * (parameters..., ids [B,T] i64, targets [B,T] i64) -> scalar loss over the StableHLO ops of the reference's exports
 * runs through the general front end: the same functions, one kernel per op of the program pcpb_graph_describe shows.
 * What neither path can run is refused with PCPB_E_ARTIFACT and a reason.
 */
#ifndef PCP_B200_H
#define PCP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct pcpb_backend pcpb_backend;
typedef struct pcpb_buffer pcpb_buffer;

/* Element types, numbered like DType in src/core/tensor.zig:9-62. */
enum pcpb_dtype { PCPB_F32 = 0, PCPB_F64 = 1, PCPB_F16 = 2, PCPB_BF16 = 3, PCPB_I32 = 4, PCPB_I64 = 5, PCPB_BOOL = 6 };

enum pcpb_status {
  PCPB_OK = 0,
  PCPB_E_INVALID = 1,      /* bad argument, shape or dtype                               */
  PCPB_E_CUDA = 2,         /* a CUDA call failed (the reference: error.IreeRuntimeError)  */
  PCPB_E_ARTIFACT = 3,     /* artefact not recognised / not loaded                        */
  PCPB_E_FUNCTION = 4,     /* unknown function name                                       */
  PCPB_E_CHUNK_TOO_SMALL = 5,   /* src/data/loader.zig:559 ChunkTooSmall                  */
  PCPB_E_CHUNK_EXHAUSTED = 6,   /* src/data/loader.zig:560 ChunkExhausted                 */
  PCPB_E_STATE = 7,        /* call sequence error (e.g. step before begin_round)          */
  PCPB_E_TOO_LARGE = 8     /* size beyond a fixed capacity                                */
};

/* IreeBackend.init / deinit  (src/backends/iree.zig:84,153): device by ordinal. */
int pcpb_create(int device_ordinal, pcpb_backend** out);
void pcpb_destroy(pcpb_backend* b);
/* WorkerBackend.getBackendType (src/backends/worker_backend.zig:33): always "cuda". */
const char* pcpb_backend_type(const pcpb_backend* b);
const char* pcpb_last_error(const pcpb_backend* b);
void pcpb_free(void* p);

/* IreeBackend.loadSession (src/backends/iree.zig:213): (re)loads iff (ptr, len) differ from the cached
 * artefact; the bytes are borrowed only for the duration of the call (they are parsed, not retained). */
int pcpb_load_artifact(pcpb_backend* b, const void* bytes, size_t n);

/* ModelInspector.inspect without a device (src/mlir/model_introspection.zig:251-312): parses the artefact and
 * writes vocab, d_model, layers, heads, kv_heads, head_dim, mlp width, batch, block, model dtype, number of
 * parameter tensors, total parameter count into facts[12].  err (may be NULL) receives the reason on failure.
 * For a graph of neither fused family (run op by op by the general front end) d_model, layers, heads, kv_heads,
 * head_dim and mlp width are 0, and vocab is the first parameter's row count. */
int pcpb_inspect_artifact(const void* bytes, size_t n, int64_t* facts, char* err, size_t err_cap);

/* The general front end's view of a forward graph, for graphs outside the two fused families: what the reference's
 * AD engine does when it emits the gradient function next to the forward function (src/autodiff/engine.zig:196-348,
 * rules src/autodiff/vjp_rules.zig, adjoint edges engine.zig:604-702), after the stability patches of
 * src/compiler/sanitizer.zig:8-244.  Writes the tensor program (one line per value and per op; forward ops first, then,
 * if with_gradients, the gradient ops for every argument but the last two) as text into *text_out (release with
 * pcpb_free).  with_gradients = 2 appends the executor's plan of that program: per value where it is stored (arena
 * offset, the ops that define and release it), per op whether it runs, was folded into the constants, dropped or fused.
 * Needs no device.  A graph pcpb_inspect_artifact reports with d_model = 0 is run from this program
 * (one kernel per op); PCPB_FRONTEND=graph in the environment sends every graph that way, PCPB_FRONTEND=fused none. */
int pcpb_graph_describe(const void* bytes, size_t n, int with_gradients, char** text_out, char* err, size_t err_cap);

/* Model facts recovered from the artefact (src/mlir/model_introspection.zig:251-312: parameters are all
 * @main arguments except the last two).  shape_out receives up to 8 dims. */
int pcpb_num_params(const pcpb_backend* b);
int pcpb_param_shape(const pcpb_backend* b, int index, int64_t* shape_out, int* rank_out);
int pcpb_model_info(const pcpb_backend* b, int64_t* batch, int64_t* block, int64_t* vocab, int* model_dtype,
                    int64_t* total_params);

/* IreeBackend.moveToDevice / allocateZerosDevice (src/backends/iree.zig:166,198) and
 * DeviceBuffer.retain / release / byteLength (:53-69). */
int pcpb_buffer_from_host(pcpb_backend* b, const void* src, size_t nbytes, const int64_t* shape, int rank, int dtype,
                          pcpb_buffer** out);
int pcpb_buffer_zeros(pcpb_backend* b, const int64_t* shape, int rank, int dtype, pcpb_buffer** out);
void pcpb_buffer_retain(pcpb_buffer* buf);
void pcpb_buffer_release(pcpb_buffer* buf);
size_t pcpb_buffer_nbytes(const pcpb_buffer* buf);

/* IreeBackend.executeWithDeviceBuffers (src/backends/iree.zig:256): blocking; inputs are borrowed; each
 * returned buffer carries one reference owned by the caller; the returned array is freed with pcpb_free.
 * Functions (the names src/compiler/graph_builder.zig:56-278 and :435-726 emit):
 *   compute_gradients              (params f32..., ids[B,T], targets[B,T]) -> (grads f32..., loss)
 *   compute_gradients_accumulated  (params f32..., ids[S,B,T], targets[S,B,T]) -> (sum of grads f32..., sum of losses);
 *                                  S is taken from the byte length of ids; the caller divides by S
 *                                  (src/nodes/workers/worker.zig:1134-1187)
 *   apply_optimizer                (p..., g..., m..., v..., t) -> (p'..., m'..., v'...), hyper-parameters of pcpb_set_adam
 *   accumulate_gradients           (acc..., grads...) -> (acc + grads ...)
 *   model_forward_pass, main       (params model dtype..., ids, targets) -> loss
 *   model_forward_pass_grad        (params model dtype..., ids, targets, dloss) -> (grads model dtype...)
 * Every function except apply_optimizer and accumulate_gradients stages its parameters in the buffers of the fused
 * worker path and is refused with PCPB_E_STATE between pcpb_worker_begin_round and pcpb_worker_end_round. */
int pcpb_execute(pcpb_backend* b, const char* fn, pcpb_buffer* const* in, size_t n_in, pcpb_buffer*** out, size_t* n_out);

/* IreeBackend.readToHost (src/backends/iree.zig:315): blocking device -> host copy. */
int pcpb_read_to_host(pcpb_backend* b, const pcpb_buffer* buf, void* dst, size_t nbytes);

/* IreeBackend.execute / WorkerBackend.executeFunction (src/backends/iree.zig:336, worker_backend.zig:24):
 * host bytes in, host bytes out.  out[i] and the two arrays are freed with pcpb_free. */
int pcpb_execute_host(pcpb_backend* b, const char* fn, const void* const* in, const size_t* in_nbytes,
                      const int64_t* const* shapes, const int* ranks, const int* dtypes, size_t n_in, void*** out,
                      size_t** out_nbytes, size_t* n_out);

/* One contraction of the op surface (stablehlo.dot_general as the reference's graphs use it, src/core/ops.zig and
 * matmulVJP src/autodiff/vjp_rules.zig:426-496), on device buffers of the loaded model's dtype:
 *   C[M,N] = epilogue(sum_k A(m,k) B(k,n)),  A(m,k) = A[m*sam + k*sak],  B(k,n) = B[k*sbk + n*sbn]
 * epilogue: 0 store, 1 residual add (R), 2 store + relu^2 into C2, 3 relu^2 backward at R, 4 weight gradient (f32 C),
 *           5 store + relu into C2, 6 relu backward at R, 7 add bias R[N], 8 store + tanh-GELU into C2,
 *           9 tanh-GELU backward at R (tanhVJP src/autodiff/vjp_rules.zig:1692 and the multiply / add rules, in closed form).
 * path: 0 = pick (tensor cores when the shape allows), 1 = generic kernel, 2 = tensor-core kernel or error. */
int pcpb_op_gemm(pcpb_backend* b, int path, const pcpb_buffer* A, long long sam, long long sak, const pcpb_buffer* B,
                 long long sbk, long long sbn, pcpb_buffer* C, long long ldc, const pcpb_buffer* R, pcpb_buffer* C2,
                 int M, int N, int K, int epilogue);

/* Dataset.getBatch of the FIFO u16 dataset (U16TokenDatasetFifo.getBatchImpl, src/data/loader.zig:555-589),
 * with the widening to i64 done on the device: consumes B*T+1 tokens of the host chunk at *cursor, returns the
 * [B,T] i64 inputs and 1-shifted targets as device buffers and advances *cursor by B*T+1.
 * PCPB_E_CHUNK_TOO_SMALL / PCPB_E_CHUNK_EXHAUSTED as in the reference. */
int pcpb_fifo_get_batch(pcpb_backend* b, const uint16_t* tokens, size_t n_tokens, size_t* cursor,
                        pcpb_buffer** inputs, pcpb_buffer** targets);

/* ---- random-window batching, character tokenizer, master initialisation (host side) ---------------------------
 * The generator stands in for Zig 0.13's std.Random.DefaultPrng, which the reference draws from but does not ship:
 * xoshiro256++ seeded through SplitMix64, bounded integers by Lemire's multiply-shift with rejection, normals by
 * Box-Muller.  UNPINNED against the Zig standard library: the same distributions, not the same sequences. */
typedef struct pcpb_prng { uint64_t s[4]; } pcpb_prng;
void pcpb_prng_seed(pcpb_prng* g, uint64_t seed);                       /* std.Random.DefaultPrng.init(seed) */
uint64_t pcpb_prng_next(pcpb_prng* g);
uint64_t pcpb_prng_uint_at_most(pcpb_prng* g, uint64_t at_most);        /* random.uintAtMost(usize, at_most) */
/* One window start per batch row, uniform in [0, n_tokens - block - 1]; PCPB_E_CHUNK_TOO_SMALL when
 * n_tokens <= block + 1 (src/data/loader.zig:289-291, 379-381, 469-471). */
int pcpb_random_window_starts(pcpb_prng* g, size_t n_tokens, size_t batch, size_t block, uint64_t* starts_out);
/* Dataset.getBatch of the random-window datasets (U16TokenDataset, TextDataset, ByteTextDataset .getBatchImpl,
 * src/data/loader.zig:457-486, 276-307, 366-397): draws the loaded model's B window starts from `g`, gathers the
 * windows of the host chunk (token_bytes 2: u16 stream; 4: u32 tokens of the char / byte tokenizers) and returns the
 * [B,T] i64 inputs and 1-shifted targets as device buffers (widening on the device). */
int pcpb_random_get_batch(pcpb_backend* b, pcpb_prng* g, const void* tokens, int token_bytes, size_t n_tokens,
                          pcpb_buffer** inputs, pcpb_buffer** targets);
/* CharTokenizer (src/data/loader.zig:12-89): vocabulary = the distinct bytes of the text, ascending, at most 65
 * (vocab_chars_out has room for PCPB_CHAR_VOCAB_MAX entries; *ignored_chars_out, optional, counts the bytes beyond);
 * encode maps unknown bytes to token 0; decode refuses unknown tokens with PCPB_E_INVALID (UnknownToken). */
#define PCPB_CHAR_VOCAB_MAX 65
int pcpb_char_tokenizer_build(const uint8_t* text, size_t n, uint8_t* vocab_chars_out, int* vocab_size_out,
                              int* ignored_chars_out);
int pcpb_char_encode(const uint8_t* vocab_chars, int vocab_size, const uint8_t* text, size_t n, uint32_t* tokens_out);
int pcpb_char_decode(const uint8_t* vocab_chars, int vocab_size, const uint32_t* tokens, size_t n, uint8_t* text_out);
/* DiLoCo.initializeMasterParameters (src/algorithms/diloco.zig:513-586): every element of every tensor, in argument
 * order from one generator, is 0.02 * N(0,1) in f32; PCPB_BF16 keeps the upper 16 bits (truncation).  The reference
 * seeds with 12345.  pcpb_init_master fills the parameter blob of the loaded artefact (what
 * pcpb_worker_begin_round takes); pcpb_init_master_elems needs no backend. */
int pcpb_init_master_elems(uint64_t seed, int dtype, size_t n, void* out, size_t out_bytes);
int pcpb_init_master(const pcpb_backend* b, uint64_t seed, int dtype, void* blob_out, size_t blob_bytes);

/* AdamW constants of apply_optimizer (src/optimizers/adam_mlir.zig:10-19; the reference bakes them into the
 * compiled module, src/algorithms/diloco.zig:205-211).  Defaults: lr 1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0. */
typedef struct pcpb_adam_conf {
  float learning_rate, beta1, beta2, epsilon, weight_decay, max_grad_norm;
} pcpb_adam_conf;
int pcpb_set_adam(pcpb_backend* b, const pcpb_adam_conf* conf);

/* ---- fused worker path: Worker.handleStartInnerLoop (src/nodes/workers/worker.zig:855-1480) kept on the
 * device.  Same semantics: Adam state reset at the start of a round (unless persist_adam), tau steps of
 * FIFO batch -> compute_gradients (accumulation_steps micro-batches, summed, scaled by 1/steps) ->
 * apply_optimizer, NaN heal of m/v, delta = initial - final (bf16: truncated), last step's loss. */
typedef struct pcpb_inner_cfg {
  int tau;
  int accumulation_steps;   /* >= 1 */
  int param_dtype;          /* PCPB_F32 | PCPB_BF16: dtype of the parameter / delta blobs */
  int persist_adam;         /* 0 = reference behaviour (reset every round) */
  int tokens_on_device;     /* 0: `tokens` is host memory, each step's window is copied in the step;
                               1: `tokens` is a device pointer */
} pcpb_inner_cfg;

/* Start a round.  params_blob: host bytes of all parameters concatenated in argument order in param_dtype
 * (the START_INNER_LOOP payload, src/algorithms/diloco.zig:665-667), or NULL to continue from the master
 * parameters already on the device (after pcpb_outer_apply). */
int pcpb_worker_begin_round(pcpb_backend* b, const pcpb_inner_cfg* cfg, const void* params_blob, size_t blob_bytes);
/* Attach the token chunk of this round (U16TokenDatasetFifo, src/data/loader.zig:500-553); cursor = 0. */
int pcpb_worker_set_tokens(pcpb_backend* b, const uint16_t* tokens, size_t n_tokens);
/* One inner step, enqueued without host synchronisation.  loss_slot: index in the per-round loss record. */
int pcpb_worker_step(pcpb_backend* b);
/* Finish: heal, delta.  delta_out (host, may be NULL) receives the delta blob in param_dtype; losses (host,
 * may be NULL) receives one f32 per step done this round. */
int pcpb_worker_end_round(pcpb_backend* b, void* delta_out, size_t delta_bytes, float* losses, size_t n_losses);
/* The whole of handleStartInnerLoop in one call. */
int pcpb_inner_loop(pcpb_backend* b, const pcpb_inner_cfg* cfg, const void* params_blob, size_t blob_bytes,
                    const uint16_t* tokens, size_t n_tokens, void* delta_out, size_t delta_bytes, float* losses);
/* Current f32 working parameters / Adam state of the fused path, for checks (flat, argument order). */
int pcpb_worker_read_state(pcpb_backend* b, int which /*0 params,1 m,2 v,3 delta,4 master,5 velocity,6 grads*/,
                           float* dst, size_t n);
/* Overwrites one of those states from host memory (same selectors and lengths; 3 = the delta this rank publishes to
 * the outer step, 5 = this rank's velocity shard, which needs pcpb_outer_attach_* first).  This is how a run resumed
 * from a recovery file restores the Nesterov velocities (src/algorithms/diloco.zig:1063-1107) and, for persist_adam,
 * the Adam moments; writing the parameters (0) also refreshes their model-dtype copy. */
int pcpb_worker_write_state(pcpb_backend* b, int which, const float* src, size_t n);
/* Batch sampling of the fused path: 0 = FIFO (U16TokenDatasetFifo, the default, bit-exact), 1 = random windows
 * (U16TokenDataset.getBatchImpl, src/data/loader.zig:457-486) drawn from a generator seeded with `seed`
 * (src/data/loader.zig:439).  Takes effect at the next pcpb_worker_set_tokens. */
int pcpb_worker_set_sampling(pcpb_backend* b, int mode, uint64_t seed);
/* Adjoint-edge status.  The reference's AD engine passes every adjoint through a finite guard (non-finite -> 0) and
 * a clamp to [-100, 100] before accumulating it (src/autodiff/engine.zig:604-702).  The kernels do the same on every
 * adjoint they hold as a value of its own: the loss gradient, the outputs of every backward GEMM (activation and weight
 * gradients), the row and element values of the RMSNorm / QK-norm / RoPE / LayerNorm / activation backward, the
 * attention gradients dQ, dK, dV.  Inside the fused attention backward dP and dS are not clamped edge by edge (its
 * softmax backward is in closed form); their magnitude is checked instead.  flags receives, since the last clear and
 * for the device of this backend (the word is shared by the backends on one device):
 *   bit 0 (PCPB_ADJ_CLAMPED)   some adjoint was non-finite or beyond +-100 and was guarded / clamped: results follow the
 *                              reference's clamped arithmetic at every edge listed above
 *   bit 1 (PCPB_ADJ_INTERNAL)  an adjoint inside the fused attention backward was beyond +-100: from there on the
 *                              gradients are those of the unclamped softmax backward, clamped where they leave the kernel
 * 0 means no guard or clamp of the reference was active: gradients are those of the reference's engine.  Blocks.
 * A graph run by the general front end applies every guard and clamp as an op of its program, exactly where the engine
 * does; nothing is approximated there and nothing is recorded: the flags stay 0 for it. */
#define PCPB_ADJ_CLAMPED 1
#define PCPB_ADJ_INTERNAL 2
int pcpb_adjoint_status(pcpb_backend* b, int* flags, int clear);
/* Blocks until everything enqueued by this backend has run; returns the first asynchronous error. */
int pcpb_synchronize(pcpb_backend* b);

/* ---- DiLoCo outer step on the box: DiLoCo.accumulateAndApplyGradients + Nesterov.update
 * (src/algorithms/diloco.zig:828-1060, src/optimizers/nesterov.zig:70-98) as a reduce-scatter / update /
 * all-gather over peer memory.  Rank r owns elements [r*S, (r+1)*S) of the master parameters and velocity.
 * Sequence per round, with a host barrier across ranks where marked:
 *   pcpb_outer_prepare (all ranks)  -> barrier -> pcpb_outer_apply (all ranks) -> barrier
 * After it every rank's round-start parameters hold the new master. */
typedef struct pcpb_outer_cfg {
  float learning_rate;      /* 0.7 in the reference (src/algorithms/diloco.zig:218-221) */
  float momentum;
  int param_dtype;          /* PCPB_BF16: master and deltas truncated to bf16 precision */
} pcpb_outer_cfg;
#define PCPB_IPC_HANDLE_BYTES 64
/* Bytes to publish to the other ranks: 2 IPC handles (delta buffer, round-start parameter buffer). */
int pcpb_outer_export(pcpb_backend* b, void* handles_out /* 2*PCPB_IPC_HANDLE_BYTES */);
/* world ranks; all_handles: world * 2 * PCPB_IPC_HANDLE_BYTES gathered in rank order (own entry ignored).
 * Attaching again with the same (rank, world) keeps this rank's velocity shard; a different membership starts the
 * shard at zero and the host restores the re-sharded velocities with pcpb_worker_write_state(5)
 * (pcp_b200/diloco.py: DilocoGroup.regroup), so that a worker leaving between rounds does not reset the momentum the
 * reference's Shepherd would have kept (src/algorithms/diloco.zig:418-444, src/optimizers/nesterov.zig:70-98). */
int pcpb_outer_attach_ipc(pcpb_backend* b, int rank, int world, const void* all_handles);
/* Same-process variant (several backends in one process): peers[w] for every rank, own entry included. */
int pcpb_outer_attach_local(pcpb_backend* b, int rank, int world, pcpb_backend* const* peers);
int pcpb_outer_prepare(pcpb_backend* b, const pcpb_outer_cfg* cfg);
/* contributors: ranks whose deltas are averaged (NULL = all), the divisor is their count
 * (src/algorithms/diloco.zig:970). */
int pcpb_outer_apply(pcpb_backend* b, const pcpb_outer_cfg* cfg, const int* contributors, int n_contributors,
                     double* device_ms);

/* ---- Streaming DiLoCo: fragment-wise outer step --------------------------------------------------------------
 * Replaces the worker's extractAndSendFragment / receiveAndMergeFragment (src/nodes/workers/worker.zig:2396-2479,
 * 2482-2610) and the Shepherd's accumulateFragmentGradients / applyFragmentUpdate
 * (src/algorithms/streaming_diloco.zig:425-520).  Tensor i (artefact argument order) belongs to fragment
 * i % num_fragments (worker.zig:2417).  The calls are made inside a round opened with pcpb_worker_begin_round
 * (tau = the number of streaming steps; Adam state persists over the whole loop as in worker.zig:2249-2345), between
 * pcpb_worker_step calls, on the schedule of worker.zig:2213-2239 (pcp_b200/diloco.py restates it):
 *   pcpb_stream_begin   once after pcpb_worker_begin_round: snapshot <- parameters (worker.zig:2124-2176); the
 *                       round-start buffer serves as this rank's replica of the master parameters
 *   pcpb_stream_send    delta[fragment] = snapshot - parameters, snapshot <- parameters; returns when the delta
 *                       is visible to the peers
 *   (barrier)
 *   pcpb_stream_outer   this rank's shard of the fragment: sum of the ranks' deltas in rank order / world,
 *                       Nesterov on master and velocity (no non-finite filter, no truncation: f32 as the
 *                       reference's streaming path), new master written into every rank's replica
 *   (barrier)
 *   pcpb_stream_merge   overlap_tau steps later: parameters[fragment] <- alpha*parameters + (1-alpha)*master,
 *                       snapshot <- the blend
 * pcpb_stream_outer_start / pcpb_stream_outer_wait split pcpb_stream_outer so that the fragment's reduction and
 * Nesterov step run on a side stream under the next overlap_tau training steps, as the reference overlaps its
 * network round trip with them (worker.zig:2213-2239): start after the barrier that follows the send; wait (then a
 * barrier, since every rank writes into every replica) before the merge.  pcpb_stream_merge refuses a fragment whose
 * outer step was started and not waited for.
 * Needs pcpb_outer_attach_* first (same peer mapping and sharding as the DiLoCo outer step). */
typedef struct pcpb_stream_cfg {
  int num_fragments;        /* 4 in the reference (worker.zig:179) */
  float alpha;              /* blend weight of the local parameters */
  float learning_rate;      /* Nesterov, as pcpb_outer_cfg */
  float momentum;
} pcpb_stream_cfg;
int pcpb_stream_begin(pcpb_backend* b, const pcpb_stream_cfg* cfg);
int pcpb_stream_send(pcpb_backend* b, int fragment);
int pcpb_stream_outer(pcpb_backend* b, int fragment, double* device_ms);
int pcpb_stream_outer_start(pcpb_backend* b, int fragment);
int pcpb_stream_outer_wait(pcpb_backend* b, int fragment, double* device_ms);
int pcpb_stream_merge(pcpb_backend* b, int fragment);

/* Loss of the most recent pcpb_worker_step, read back to the host (blocks until that step has run): the
 * per-step loss read of the reference's inner loop (src/nodes/workers/worker.zig:1246). */
int pcpb_worker_last_loss(pcpb_backend* b, float* loss);

/* Device-side timing on the backend's own stream (CUDA events): start / stop bracket whatever the backend
 * enqueues in between; stop blocks until the work has run and returns the elapsed milliseconds. */
int pcpb_timer_start(pcpb_backend* b);
int pcpb_timer_stop(pcpb_backend* b, double* ms);

/* Per-kernel accounting of the tensor-core GEMM: while enabled every launch is bracketed by CUDA events.
 * pcpb_profile_read blocks, then returns the number of launches, their summed duration and their summed
 * algorithmic FLOPs (2*M*N*K each) since the last enable, and keeps profiling on. */
int pcpb_profile_enable(pcpb_backend* b, int on);
int pcpb_profile_read(pcpb_backend* b, long long* launches, double* total_ms, double* total_flops);

/* AdamW step that allocates nothing.  It has no counterpart in the reference; it exists for hosts that cannot
 * let a library allocate device memory on their behalf: runtimes that give out slices of one arena reserved up
 * front and account for every byte (memory-planned runtimes; the reference compiles for one and bounds the size of a
 * single allocation at compile time, --iree-stream-resource-max-allocation-size in src/mlir/context.zig:238-239), and
 * services whose step loop rules out allocation calls because cudaMalloc / cudaFree synchronise the device.
 * The regular apply_optimizer entry allocates its outputs and a descriptor table per call; this one works on
 * tensors the caller owns and keeps its reduction scratch in a fixed array inside the library image.
 *
 *   p, g, m, v        device pointers, n f32 elements each (one tensor); p_out, m_out, v_out receive the update
 *                     (they may alias p, m, v)
 *   stream            a cudaStream_t, or NULL for the default stream; the call enqueues and returns, it does not wait
 *   conf, timestep    as pcpb_set_adam / the f32 step counter of apply_optimizer (1.0 at the first step)
 *   err, err_cap      optional buffer for the error text
 *
 * n may not exceed PCPB_NOALLOC_MAX_ELEMS (PCPB_E_TOO_LARGE otherwise).  The scratch array (about 64 KB) is held
 * by every GPU that loads the library until the process exits.  All calls share it and it keeps what the last call
 * left: the call re-initialises everything it reads, but two calls whose GPU work overlaps race on it, so callers
 * serialise them.  The first call on a device (the current device of the calling thread) looks up the array's
 * device address once; make that first call before beginning any stream capture. */
/* 2^26 = 67,108,864 elements.  Large enough for every layer tensor of the models in scope (the biggest, the d20 MLP
 * matrices, hold 5120 x 1280 = 6,553,600); NOT large enough for a 65536-row embedding or LM head at d_model 1280
 * (83,886,080 elements): those two tensors of nanochat-d20 are refused, callers split them by rows (the clip norm is
 * per tensor, so a split changes it) or use the regular entry point for them. */
#define PCPB_NOALLOC_MAX_ELEMS (1ll << 26)
int pcpb_adamw_step_noalloc(void* stream, const float* p, const float* g, const float* m, const float* v, float* p_out,
                            float* m_out, float* v_out, long long n, const pcpb_adam_conf* conf, float timestep,
                            char* err, size_t err_cap);

/* ---- rollout generation: GenerationEngine.generateRolloutStreaming (src/nodes/workers/generation_engine.zig:174-332)
 * with the sampler's greedy branch (src/core/math.zig:21-73), kept on the device.  The reference feeds one token per
 * call to a compiled decode step of a Qwen3-shaped model (tools/export_qwen3_generation.py) and keeps a dense KV cache
 * on the host; here all prompts of a batch are prefilled at once, the cache is paged and stays in HBM, and every
 * further token is one CUDA graph launch.  The arithmetic per token is the exported step's, including its property
 * that a token attends to the cache as it was before the step (its own slot reads as a zero key and zero value).
 * bf16 model, greedy decoding only (temperature < 1e-6); up to 16 sequences per engine. */
typedef struct pcpb_rollout pcpb_rollout;
typedef struct pcpb_rollout_cfg {
  int vocab, d_model, n_layer, n_head, n_kv_head, head_dim, d_ff;
  int max_seq;              /* positions per sequence: prompt + generated (the reference's MAX_SEQ_LEN) */
  int page_tokens;          /* tokens per KV-cache page */
  int max_batch;            /* sequences generated together, <= 16 */
  int max_prompt;           /* longest prompt; the prefill buffers hold max_batch * max_prompt token rows */
  float rope_theta, rms_eps;
} pcpb_rollout_cfg;
/* Number of weights of a configuration, in the argument order of the exported function (= named_parameters() of the
 * Hugging Face model): embed, per layer q k v o q_norm k_norm gate up down input_ln post_ln, norm, lm_head. */
long long pcpb_rollout_num_params(const pcpb_rollout_cfg* cfg);
int pcpb_rollout_create(int device_ordinal, const pcpb_rollout_cfg* cfg, pcpb_rollout** out);
void pcpb_rollout_destroy(pcpb_rollout* r);
const char* pcpb_rollout_last_error(const pcpb_rollout* r);
/* GenerationEngine.ensureDeviceWeights (generation_engine.zig:80-122): the weight blob, tensor after tensor, PCPB_F32
 * (the reference's blob; rounded to bf16 on the device) or PCPB_BF16. */
int pcpb_rollout_load_weights(pcpb_rollout* r, const void* blob, size_t nbytes, int dtype);
/* Benchmark set-up only: fills the matrices with N(0, std) and the norm weights with 1 on the device (the baseline
 * configuration's random weights; 8 x 10^9 values would take minutes to draw on the host). */
int pcpb_rollout_random_weights(pcpb_rollout* r, uint64_t seed, float std);
/* prompts: batch rows of prompt_stride token ids, row b holding prompt_lens[b] of them (0 = empty prompt: generation
 * starts from token 0 at position 0, generation_engine.zig:233-240).  tokens_out: batch x max_new_tokens, row b holds
 * n_generated[b] tokens (the rest 0); finish_reason[b] (optional): 0 "length", 1 "stop" (eos_token was produced).
 * prefill_ms / decode_ms (optional): device time of the prompt pass with the first token, and of the remaining steps. */
int pcpb_rollout_generate(pcpb_rollout* r, const int64_t* prompts, const int* prompt_lens, int batch, int prompt_stride,
                          int max_new_tokens, int64_t eos_token, float temperature, int64_t* tokens_out, int* n_generated,
                          int* finish_reason, double* prefill_ms, double* decode_ms);
/* Logits (as f32) of sequence `row` at the most recent step, for checks. */
int pcpb_rollout_read_logits(pcpb_rollout* r, int row, float* dst, size_t n);
long long pcpb_rollout_launch_count(const pcpb_rollout* r);

/* Kernel counters of this backend: launches enqueued since creation, by the library's own kernels. */
long long pcpb_launch_count(const pcpb_backend* b);

#ifdef __cplusplus
}
#endif
#endif /* PCP_B200_H */
