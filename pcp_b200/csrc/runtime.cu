// Backend runtime + C ABI (include/pcp_b200.h).
#include "runtime.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/pcp_b200.h"
#include "common.cuh"
#include "attn_flash.h"
#include "attn_tc.h"
#include "gemm_tc.h"

using namespace pcpb;

namespace {

#define CK(b, call)                                                                          \
  do {                                                                                       \
    cudaError_t e__ = (call);                                                                \
    if (e__ != cudaSuccess) {                                                                \
      char m__[512];                                                                         \
      snprintf(m__, sizeof m__, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
      (b)->err = m__;                                                                        \
      return PCPB_E_CUDA;                                                                    \
    }                                                                                        \
  } while (0)

#define KL(b, n, call) do { (b)->launches += (n); CK(b, call); } while (0)

int fail(pcpb_backend* b, int code, const std::string& msg) {
  if (b) b->err = msg;
  return code;
}

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

size_t numel_of(const int64_t* shape, int rank) {
  size_t n = 1;
  for (int i = 0; i < rank; ++i) n *= (size_t)shape[i];
  return n;
}

void block_release(Block* blk) {
  if (blk && blk->refs.fetch_sub(1) == 1) {
    DeviceGuard g(blk->device);
    cudaFree(blk->ptr);
    delete blk;
  }
}

pcpb_buffer* make_view(pcpb_backend* b, Block* blk, void* ptr, size_t nbytes, const int64_t* shape, int rank, int dtype) {
  pcpb_buffer* buf = new pcpb_buffer();
  buf->owner = b; buf->block = blk; buf->ptr = ptr; buf->nbytes = nbytes;
  buf->shape.assign(shape, shape + rank); buf->dtype = dtype;
  blk->refs.fetch_add(1);
  return buf;
}

int alloc_block(pcpb_backend* b, size_t bytes, Block** out) {
  Block* blk = new Block();
  blk->bytes = bytes; blk->device = b->device;
  cudaError_t e = cudaMalloc(&blk->ptr, bytes ? bytes : 1);
  if (e != cudaSuccess) { delete blk; b->err = std::string("cudaMalloc failed: ") + cudaGetErrorString(e); return PCPB_E_CUDA; }
  *out = blk;
  return PCPB_OK;
}

// ------------------------------------------------------------------------------------------------
// workspace
// ------------------------------------------------------------------------------------------------
void free_workspace(pcpb_backend* b) {
  if (b->side_stream) cudaStreamSynchronize(b->side_stream);     // a fragment's outer step may still use the buffers
  b->frag_pending.clear();
  for (void* p : b->ws.allocs) cudaFree(p);
  b->ws = Workspace();
  if (b->gx) { graph_exec_destroy(b->gx); b->gx = nullptr; }
  if (b->tokens_stage) { cudaFree(b->tokens_stage); b->tokens_stage = nullptr; b->stage_cap = 0; }
  if (b->window_stage) { cudaFree(b->window_stage); b->window_stage = nullptr; b->window_stage_cap = 0; }
  if (b->starts_dev) { cudaFree(b->starts_dev); b->starts_dev = nullptr; }
  for (void* p : b->ipc_opened) cudaIpcCloseMemHandle(p);
  b->ipc_opened.clear(); b->peer_delta.clear(); b->peer_theta0.clear();
  if (b->velocity) { cudaFree(b->velocity); b->velocity = nullptr; }
  b->velocity_init = false; b->have_master = false; b->in_round = false;
  b->snapshot = nullptr; b->stream_fragments = 0;      // the snapshot lived in the workspace
}

template <typename P>
int wsalloc(pcpb_backend* b, P** out, size_t bytes) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    char m[256];
    snprintf(m, sizeof m, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    b->err = m;
    return PCPB_E_CUDA;
  }
  b->ws.allocs.push_back(p);
  *out = (P*)p;
  // PCPB_POISON=1 fills every workspace buffer with 0xFF bytes (NaN patterns), so that a kernel reading memory it
  // never wrote shows up in the parity tests instead of depending on what the allocator handed out.
  static const bool poison = [] { const char* e = getenv("PCPB_POISON"); return e && e[0] == '1'; }();
  if (poison && cudaMemset(p, 0xFF, bytes ? bytes : 16) != cudaSuccess) { b->err = "poisoning a workspace buffer failed"; return PCPB_E_CUDA; }
  return PCPB_OK;
}
#define WS(b, ptr, bytes) do { int r__ = wsalloc(b, &(ptr), (bytes)); if (r__) return r__; } while (0)

// optimiser tables of the flat parameter layout
int build_flat_tables(pcpb_backend* b) {
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  const size_t es = dtype_size(c.dtype);
  const int nseg = (int)c.params.size();
  std::vector<TensorSeg> segs(nseg);
  std::vector<int> c2s;
  for (int i = 0; i < nseg; ++i) {
    const TensorInfo& t = c.params[i];
    TensorSeg& s = segs[i];
    s.p = w.theta + t.offset; s.g = w.grads + t.offset; s.m = w.mstate + t.offset; s.v = w.vstate + t.offset;
    s.p_out = w.theta + t.offset; s.m_out = w.mstate + t.offset; s.v_out = w.vstate + t.offset;
    s.shadow = (c.dtype == DT_F32) ? nullptr : (void*)((char*)w.shadow + (size_t)t.offset * es);
    s.n = t.numel; s.first_chunk = (int)c2s.size();
    s.num_chunks = (int)((t.numel + ADAM_CHUNK - 1) / ADAM_CHUNK);
    for (int k = 0; k < s.num_chunks; ++k) c2s.push_back(i);
  }
  w.nchunks = (int)c2s.size();
  WS(b, w.segs, sizeof(TensorSeg) * nseg); WS(b, w.chunk2seg, sizeof(int) * c2s.size());
  WS(b, w.partial, 4 * c2s.size()); WS(b, w.normsq, 4 * (size_t)nseg); WS(b, w.heal_flags, 4 * (size_t)nseg * 2);
  CK(b, cudaMemcpy(w.segs, segs.data(), sizeof(TensorSeg) * nseg, cudaMemcpyHostToDevice));
  CK(b, cudaMemcpy(w.chunk2seg, c2s.data(), sizeof(int) * c2s.size(), cudaMemcpyHostToDevice));
  return PCPB_OK;
}

int build_workspace(pcpb_backend* b) {
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  const size_t P = (size_t)c.total_params, M = (size_t)c.M(), d = (size_t)c.d, F = (size_t)c.F;
  const size_t dkv = (size_t)c.dkv(), es = dtype_size(c.dtype);
  WS(b, w.theta, P * 4); WS(b, w.theta0, P * 4); WS(b, w.mstate, P * 4); WS(b, w.vstate, P * 4);
  WS(b, w.grads, P * 4); WS(b, w.delta, P * 4);
  if (c.dtype == DT_F32) w.shadow = w.theta; else WS(b, w.shadow, P * es);
  if (c.family == FAMILY_GRAPH) {
    // general front end: the values of the program live in the executor's own arena
    WS(b, w.loss, 4); WS(b, w.count, 4); WS(b, w.ids, M * 8); WS(b, w.targets, M * 8);
    int r = build_flat_tables(b);
    if (r) return r;
    WS(b, w.tc_err, sizeof(int));
    CK(b, cudaMemset(w.tc_err, 0, sizeof(int)));
    // f32 graphs: buffers of the split-operand tensor-core path for the un-batched products of tensor-core shape
    // (PCPB_F32_TC=0 keeps them on the general kernel)
    {
      const char* e = getenv("PCPB_F32_TC");
      size_t ab = 0, cc = 0;
      for (const GOp& op : b->graph.ops) {
        if (op.kind != G_DOT || !op.a.empty()) continue;
        const GValue &x = b->graph.vals[op.in[0]], &y = b->graph.vals[op.in[1]];
        long long K = 1;
        for (int64_t i : op.c) K *= x.shape[i];
        const long long Mm = x.numel / K, Nn = y.numel / K;
        if (Mm % 128 || Nn % 128 || K % 64) continue;
        ab = std::max<size_t>(ab, (size_t)std::max<long long>(Mm, Nn) * (size_t)K * 12);
        cc = std::max<size_t>(cc, (size_t)Mm * (size_t)Nn * 4);
      }
      if (c.dtype == DT_F32 && !(e && e[0] == '0') && ab && 2 * ab + cc <= ((size_t)24 << 30)) {
        WS(b, w.pk_a, ab); WS(b, w.pk_b, ab); WS(b, w.pk_c, cc);
        w.pk_ab_bytes = ab; w.pk_c_bytes = cc;
        const size_t want = (size_t)64 << 20;
        WS(b, w.tc_scratch, want); w.tc_scratch_bytes = want;
      }
    }
    std::vector<int64_t> offs;
    for (const TensorInfo& t : c.params) offs.push_back(t.offset);
    const std::string why = graph_exec_create(b->graph, (int)c.params.size(), offs, b->stream, &b->gx);
    if (!why.empty()) return fail(b, PCPB_E_ARTIFACT, "the general front end cannot run this graph: " + why);
    w.ready = true;
    return PCPB_OK;
  }
  w.xs.resize(c.L + 1);
  for (auto& x : w.xs) WS(b, x, M * d * es);
  w.layers.resize(c.L);
  for (auto& l : w.layers) {
    WS(b, l.h1, M * d * es); WS(b, l.qkv, M * (d + 2 * dkv) * es); WS(b, l.qkn, M * (d + dkv) * es);
    WS(b, l.o, M * d * es); WS(b, l.xmid, M * d * es); WS(b, l.h2, M * d * es);
    WS(b, l.u, M * F * es); WS(b, l.a, M * F * es);
    WS(b, l.t1, M * 4); WS(b, l.t2, M * 4); WS(b, l.tq, M * (size_t)(c.H + c.Hkv) * 4);
    WS(b, l.mrow, (size_t)c.B * c.H * c.T * 4); WS(b, l.lrow, (size_t)c.B * c.H * c.T * 4);
    if (c.family == FAMILY_NANOGPT) {
      WS(b, l.mu1, M * 4); WS(b, l.mu2, M * 4); WS(b, l.m64_1, M * 8); WS(b, l.m64_2, M * 8);
    }
  }
  if (c.family == FAMILY_NANOGPT) {
    WS(b, w.muf, M * 4); WS(b, w.m64f, M * 8);
    WS(b, w.ln_partial, layernorm_bwd_scratch_floats((int)M, (int)d) * 4);
    WS(b, w.cs_partial, colsum_scratch_floats((int)M, (int)c.V) * 4);
  }
  WS(b, w.t0, M * 4); WS(b, w.tf, M * 4); WS(b, w.rowloss, M * 4); WS(b, w.count, 4); WS(b, w.loss, 4);
  WS(b, w.hf, M * d * es); WS(b, w.logits, M * (size_t)c.V * es);
  WS(b, w.dx, M * d * es); WS(b, w.dh, M * d * es); WS(b, w.du, M * F * es); WS(b, w.dout, M * d * es);
  WS(b, w.dqkn, M * (d + dkv) * es); WS(b, w.dqkv, M * (d + 2 * dkv) * es); WS(b, w.dkv_acc, M * 2 * dkv * 4);
  WS(b, w.drow, (size_t)c.B * c.H * c.T * 4 * 5);                    // D per row, then a float4 record per row
  WS(b, w.ids, M * 8); WS(b, w.targets, M * 8);
  if (!c.rope_cos.empty()) {
    WS(b, w.d_cos, c.rope_cos.size() * 2); WS(b, w.d_sin, c.rope_sin.size() * 2);
    CK(b, cudaMemcpy(w.d_cos, c.rope_cos.data(), c.rope_cos.size() * 2, cudaMemcpyHostToDevice));
    CK(b, cudaMemcpy(w.d_sin, c.rope_sin.data(), c.rope_sin.size() * 2, cudaMemcpyHostToDevice));
  }
  {
    int r = build_flat_tables(b);
    if (r) return r;
  }
  // tensor-core GEMM scratch (split-K slabs of the weight-gradient GEMMs) and error word
  if (c.dtype == DT_BF16) {
    const int Mi = (int)M, di = (int)d, Fi = (int)F, wqi = (int)(d + 2 * dkv), Vi = (int)c.V;
    size_t want = 0;
    const int shapes[5][2] = {{wqi, di}, {di, di}, {Fi, di}, {di, Fi}, {Vi, di}};
    for (auto& s : shapes) { size_t x = gemm_tc_scratch_wanted(s[0], s[1], Mi); if (x > want) want = x; }
    if (want) { WS(b, w.tc_scratch, want); w.tc_scratch_bytes = want; }
  }
  // f32 models: buffers of the split-operand tensor-core path (gemm()), sized for the widest layer GEMM of the model;
  // PCPB_F32_TC=0 keeps f32 models on the SIMT kernel
  {
    const char* e = getenv("PCPB_F32_TC");
    long long wide = std::max<long long>(std::max<long long>(F, d + 2 * dkv), d);
    // the LM head too when its width is a tile multiple and the buffers stay within 24 GB
    if (c.V % 128 == 0 && (size_t)M * std::max<long long>(wide, c.V) * 28 <= ((size_t)24 << 30)) wide = std::max<long long>(wide, c.V);
    const size_t ab = (size_t)M * wide * 12, cc = (size_t)M * wide * 4;
    if (c.dtype == DT_F32 && !(e && e[0] == '0') && M % 128 == 0 && d % 128 == 0 && 2 * ab + cc <= ((size_t)24 << 30)) {
      WS(b, w.pk_a, ab); WS(b, w.pk_b, ab); WS(b, w.pk_c, cc);
      w.pk_ab_bytes = ab; w.pk_c_bytes = cc;
      const size_t want = (size_t)64 << 20;                     // split-K slabs of the narrow (weight-gradient) products
      WS(b, w.tc_scratch, want); w.tc_scratch_bytes = want;
    }
  }
  // the embedding gradient is a sort + segmented sum (no float atomics); PCPB_EMBED_ATOMIC=1 keeps the atomic scatter
  {
    const char* e = getenv("PCPB_EMBED_ATOMIC");
    if (!(e && e[0] == '1')) {
      w.emb_scratch_bytes = embed_scatter_scratch_bytes((int)M, (int)d);
      WS(b, w.emb_scratch, w.emb_scratch_bytes);
    }
  }
  WS(b, w.tc_err, sizeof(int));
  CK(b, cudaMemset(w.tc_err, 0, sizeof(int)));
  w.ready = true;
  return PCPB_OK;
}

// The tensor-core GEMM records a non-zero code when one of its bounded waits ran out.
int check_tc_error(pcpb_backend* b) {
  int code = 0;
  CK(b, cudaMemcpy(&code, b->ws.tc_err, sizeof(int), cudaMemcpyDeviceToHost));
  if (code) {
    cudaMemset(b->ws.tc_err, 0, sizeof(int));
    return fail(b, PCPB_E_CUDA, "a tensor-core kernel gave up waiting on a barrier (role " + std::to_string(code) + "); results of this call are invalid");
  }
  return PCPB_OK;
}

// Collect the durations of the profiled launches recorded so far (blocks on the stream).
int drain_profile(pcpb_backend* b) {
  if (!b->prof_used) return PCPB_OK;
  CK(b, cudaStreamSynchronize(b->stream));
  for (size_t i = 0; i + 1 < b->prof_used; i += 2) {
    float ms = 0.f;
    CK(b, cudaEventElapsedTime(&ms, b->prof_events[i], b->prof_events[i + 1]));
    b->prof_ms += ms;
  }
  b->prof_used = 0;
  return PCPB_OK;
}

// ------------------------------------------------------------------------------------------------
// GEMM dispatch: tensor-core kernel when the shape qualifies, generic kernel otherwise
// ------------------------------------------------------------------------------------------------
// f32 product of tensor-core shape: operands as sums of three bf16 pieces, one bf16 GEMM over 6 K with the exact
// products accumulated in f32, then the generic kernel's epilogue on the f32 result (kernels.h).  *done = false when the
// shape or the buffers do not allow it (nothing was launched then).
int gemm_f32_split(pcpb_backend* b, const GemmArgs& g, bool* done) {
  *done = false;
  if (!b->force_generic && b->cfg.dtype == DT_F32 && b->ws.pk_a && g.M % 128 == 0 && g.N % 128 == 0 && g.K % 64 == 0 &&
      (size_t)g.M * g.K * 12 <= b->ws.pk_ab_bytes && (size_t)g.N * g.K * 12 <= b->ws.pk_ab_bytes &&
      (size_t)g.M * g.N * 4 <= b->ws.pk_c_bytes) {
    GemmArgs t;
    t.A = b->ws.pk_a; t.sam = 6LL * g.K; t.sak = 1; t.B = b->ws.pk_b; t.sbk = 1; t.sbn = 6LL * g.K;
    t.C = b->ws.pk_c; t.ldc = g.N; t.R = nullptr; t.C2 = nullptr; t.M = g.M; t.N = g.N; t.K = 6 * g.K; t.epi = EPI_RAWF32; t.clip = 0.f;
    t.scratch = b->ws.tc_scratch; t.scratch_bytes = b->ws.tc_scratch_bytes; t.err_word = b->ws.tc_err;
    if (gemm_tc_supported(t)) {
      KL(b, 1, launch_split3_pack(b->stream, (const float*)g.A, g.sam, g.sak, g.M, g.K, 0, b->ws.pk_a));
      KL(b, 1, launch_split3_pack(b->stream, (const float*)g.B, g.sbn, g.sbk, g.N, g.K, 1, b->ws.pk_b));
      KL(b, gemm_tc_launches(t), launch_gemm_tc(b->stream, t));
      KL(b, 1, launch_gemm_epilogue_f32(b->stream, g, b->ws.pk_c));
      *done = true;
    }
  }
  return PCPB_OK;
}

int gemm(pcpb_backend* b, GemmArgs g) {
  g.scratch = b->ws.tc_scratch; g.scratch_bytes = b->ws.tc_scratch_bytes; g.err_word = b->ws.tc_err;
  if (!b->force_generic && b->cfg.dtype == DT_BF16 && gemm_tc_supported(g)) {
    if (b->profiling) {
      // the pool grows instead of being drained: collecting durations needs a stream synchronisation, which must
      // not land inside a region the caller is timing
      while (b->prof_used + 2 > b->prof_events.size()) {
        cudaEvent_t ev = nullptr;
        CK(b, cudaEventCreate(&ev));
        b->prof_events.push_back(ev);
      }
      cudaEvent_t e0 = b->prof_events[b->prof_used], e1 = b->prof_events[b->prof_used + 1];
      CK(b, cudaEventRecord(e0, b->stream));
      KL(b, gemm_tc_launches(g), launch_gemm_tc(b->stream, g));
      CK(b, cudaEventRecord(e1, b->stream));
      b->prof_used += 2;
      b->prof_flops += 2.0 * g.M * g.N * g.K;
      b->prof_launches += 1;
      return PCPB_OK;
    }
    KL(b, gemm_tc_launches(g), launch_gemm_tc(b->stream, g));
    return PCPB_OK;
  }
  {
    bool done = false;
    int r = gemm_f32_split(b, g, &done);
    if (r || done) return r;
  }
  KL(b, 1, launch_gemm_generic(b->stream, b->cfg.dtype, g));
  return PCPB_OK;
}

GemmArgs mk(const void* A, long long sam, long long sak, const void* B, long long sbk, long long sbn, void* C,
            long long ldc, int M, int N, int K, int epi, const void* R = nullptr, void* C2 = nullptr) {
  GemmArgs g;
  g.A = A; g.sam = sam; g.sak = sak; g.B = B; g.sbk = sbk; g.sbn = sbn; g.C = C; g.ldc = ldc; g.R = R; g.C2 = C2;
  g.M = M; g.N = N; g.K = K; g.epi = epi; g.clip = 100.f;
  return g;
}
#define G(b, ...) do { int r__ = gemm(b, mk(__VA_ARGS__)); if (r__) return r__; } while (0)
// activation-gradient product (dot_general VJP output): stored through the adjoint-edge guard and clamp
#define GA(b, ...) do { GemmArgs g__ = mk(__VA_ARGS__); g__.adj = 1; int r__ = gemm(b, g__); if (r__) return r__; } while (0)

// ------------------------------------------------------------------------------------------------
// one forward (+ backward) of the model on the parameters in `wts` (model dtype, flat)
// ------------------------------------------------------------------------------------------------
int forward_backward_gpt(pcpb_backend* b, const void* wts, const long long* ids, const long long* targets, float* grads,
                         float* loss_out, bool backward, float seed);

// Any other graph: the tensor program of the general front end, one kernel per op; un-batched bf16 products of
// tensor-core shape go through the tcgen05 GEMM.
int forward_backward_graph(pcpb_backend* b, const void* wts, const long long* ids, const long long* targets, float* grads,
                           float* loss_out, bool backward, float seed) {
  GraphBind bind;
  bind.params = wts; bind.data = {ids, targets}; bind.seed = seed; bind.grads = grads; bind.loss_out = loss_out;
  bind.backward = backward;
  int hook_rc = PCPB_OK;
  auto dot2d = [&](int dt, const GemmArgs& g0) -> int {
    GemmArgs g = g0;
    g.scratch = b->ws.tc_scratch; g.scratch_bytes = b->ws.tc_scratch_bytes; g.err_word = b->ws.tc_err;
    if (b->force_generic) return 1;
    if (dt == DT_F32 && b->cfg.dtype == DT_F32) {
      bool done = false;
      if ((hook_rc = gemm_f32_split(b, g, &done))) return 2;
      return done ? 0 : 1;
    }
    if (dt != DT_BF16 || !gemm_tc_supported(g)) return 1;
    b->launches += gemm_tc_launches(g);
    if (launch_gemm_tc(b->stream, g) != cudaSuccess) { hook_rc = PCPB_E_CUDA; return 2; }
    return 0;
  };
  const std::string why = graph_exec_run(b->gx, b->stream, bind, dot2d, &b->launches);
  if (!why.empty()) return fail(b, hook_rc ? hook_rc : PCPB_E_CUDA, "general front end: " + why);
  return PCPB_OK;
}

// seed: d(loss), 1 for compute_gradients; model_forward_pass_grad passes the caller's value, which then flows through
// every adjoint edge (and its clamp) like in the reference's gradient function
int forward_backward(pcpb_backend* b, const void* wts, const long long* ids, const long long* targets, float* grads,
                     float* loss_out, bool backward, float seed = 1.f) {
  if (b->cfg.family == FAMILY_NANOGPT) return forward_backward_gpt(b, wts, ids, targets, grads, loss_out, backward, seed);
  if (b->cfg.family == FAMILY_GRAPH) return forward_backward_graph(b, wts, ids, targets, grads, loss_out, backward, seed);
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  cudaStream_t st = b->stream;
  const int dt = c.dtype, M = (int)c.M(), d = (int)c.d, F = (int)c.F, V = (int)c.V, H = (int)c.H, Hkv = (int)c.Hkv;
  const int hd = (int)c.hd, dkv = (int)c.dkv(), L = (int)c.L, Tn = (int)c.T, wq = d + 2 * dkv;
  const size_t es = dtype_size(dt);
  auto W = [&](int i) { return (const void*)((const char*)wts + (size_t)c.params[i].offset * es); };
  auto GR = [&](int i) { return grads + c.params[i].offset; };
  // 1/sqrt(hd): f64 constant converted to the model dtype (exporter idiom)
  float scale = (float)(1.0 / sqrt((double)hd));
  if (dt == DT_BF16) {
    uint32_t u; memcpy(&u, &scale, 4);
    u = (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u;
    memcpy(&scale, &u, 4);
  }

  KL(b, 1, launch_embed_norm_fwd(st, dt, W(0), ids, M, d, V, w.xs[0], w.t0));
  for (int l = 0; l < L; ++l) {
    LayerActs& a = w.layers[l];
    const int pq = 1 + 6 * l;
    KL(b, 1, launch_rmsnorm_fwd(st, dt, w.xs[l], M, d, a.h1, a.t1));
    G(b, a.h1, d, 1, W(pq), 1, d, a.qkv, wq, M, wq, d, EPI_STORE);
    KL(b, 1, launch_rope_qknorm_fwd(st, dt, a.qkv, w.d_cos, w.d_sin, M, Tn, H, Hkv, hd, a.qkn, a.tq));
    FlashArgs fa{};
    fa.qkn = a.qkn; fa.qkv = a.qkv; fa.o = a.o; fa.mrow = a.mrow; fa.lrow = a.lrow;
    fa.B = (int)c.B; fa.T = Tn; fa.H = H; fa.Hkv = Hkv; fa.hd = hd; fa.scale = scale;
    const bool fast = !b->force_generic && dt == DT_BF16 && b->attn_path != 2;
    if (fast && b->attn_path == 0 && attn_tc_supported(fa)) {
      KL(b, 1, launch_attn_tc_fwd(st, fa, w.tc_err));
    } else if (fast && flash_supported(fa)) {
      KL(b, 1, launch_flash_fwd(st, fa));
    } else {
      AttnArgs at{};
      at.qkn = a.qkn; at.qkv = a.qkv; at.o = a.o; at.mrow = a.mrow; at.lrow = a.lrow;
      at.B = (int)c.B; at.T = Tn; at.H = H; at.Hkv = Hkv; at.hd = hd; at.scale = scale;
      if (!b->force_generic && attn_f32_supported(dt, at)) KL(b, 1, launch_attn_f32_fwd(st, at));
      else KL(b, 1, launch_attn_fwd_generic(st, dt, at));
    }
    G(b, a.o, d, 1, W(pq + 3), 1, d, a.xmid, d, M, d, d, EPI_RESID, w.xs[l]);
    KL(b, 1, launch_rmsnorm_fwd(st, dt, a.xmid, M, d, a.h2, a.t2));
    G(b, a.h2, d, 1, W(pq + 4), 1, d, a.u, F, M, F, d, EPI_RELU2, nullptr, a.a);
    G(b, a.a, F, 1, W(pq + 5), 1, F, w.xs[l + 1], d, M, d, F, EPI_RESID, a.xmid);
  }
  const int ph = 1 + 6 * L;
  KL(b, 1, launch_rmsnorm_fwd(st, dt, w.xs[L], M, d, w.hf, w.tf));
  G(b, w.hf, d, 1, W(ph), 1, d, w.logits, V, M, V, d, EPI_STORE);
  KL(b, 1, launch_count_valid(st, targets, M, c.ignore_index, w.count));
  KL(b, 1, launch_softcap_ce(st, dt, w.logits, targets, M, V, c.softcap, c.ignore_index, w.count, w.rowloss,
                             backward ? 1 : 0, seed));
  KL(b, 1, launch_loss_finalize(st, w.rowloss, M, w.count, loss_out));
  if (!backward) return PCPB_OK;

  // ---- backward ----
  GA(b, w.logits, V, 1, W(ph), d, 1, w.dh, d, M, d, V, EPI_STORE);                  // d hf
  G(b, w.logits, 1, V, w.hf, d, 1, GR(ph), d, V, d, M, EPI_WGRAD);                 // d lm_head
  KL(b, 1, launch_rmsnorm_bwd(st, dt, w.xs[L], w.tf, w.dh, nullptr, M, d, w.dx));
  for (int l = L - 1; l >= 0; --l) {
    LayerActs& a = w.layers[l];
    const int pq = 1 + 6 * l;
    // MLP
    G(b, w.dx, d, 1, W(pq + 5), F, 1, w.du, F, M, F, d, EPI_DRELU2, a.u);           // du
    G(b, w.dx, 1, d, a.a, F, 1, GR(pq + 5), F, d, F, M, EPI_WGRAD);                 // d mlp.c_proj [d,F]
    G(b, w.du, 1, F, a.h2, d, 1, GR(pq + 4), d, F, d, M, EPI_WGRAD);                // d c_fc [F,d]
    GA(b, w.du, F, 1, W(pq + 4), d, 1, w.dh, d, M, d, F, EPI_STORE);                 // d h2
    KL(b, 1, launch_rmsnorm_bwd(st, dt, a.xmid, a.t2, w.dh, w.dx, M, d, w.dx));
    // attention
    GA(b, w.dx, d, 1, W(pq + 3), d, 1, w.dout, d, M, d, d, EPI_STORE);               // d o
    G(b, w.dx, 1, d, a.o, d, 1, GR(pq + 3), d, d, d, M, EPI_WGRAD);                 // d c_proj
    FlashArgs fa{};
    fa.qkn = a.qkn; fa.qkv = a.qkv; fa.o = a.o; fa.mrow = a.mrow; fa.lrow = a.lrow;
    fa.B = (int)c.B; fa.T = Tn; fa.H = H; fa.Hkv = Hkv; fa.hd = hd; fa.scale = scale;
    fa.dout = w.dout; fa.dqkn = w.dqkn; fa.dqkv = w.dqkv; fa.drow = w.drow;
    fa.stat4 = reinterpret_cast<float4*>(w.drow + (size_t)c.B * c.H * c.T);
    const bool fast = !b->force_generic && dt == DT_BF16 && b->attn_path != 2;
    if (fast && b->attn_path == 0 && attn_tc_supported(fa)) {
      KL(b, 3, launch_attn_tc_bwd(st, fa, w.tc_err));
    } else if (fast && flash_supported(fa)) {
      KL(b, 3, launch_flash_bwd(st, fa));
    } else {
      AttnArgs at{};
      at.qkn = a.qkn; at.qkv = a.qkv; at.o = a.o; at.mrow = a.mrow; at.lrow = a.lrow;
      at.B = (int)c.B; at.T = Tn; at.H = H; at.Hkv = Hkv; at.hd = hd; at.scale = scale;
      at.dout = w.dout; at.dqkn = w.dqkn; at.dqkv = w.dqkv; at.dkv_acc = w.dkv_acc;
      if (!b->force_generic && attn_f32_supported(dt, at)) KL(b, 3, launch_attn_f32_bwd(st, at, w.dkv_acc));
      else KL(b, 3, launch_attn_bwd_generic(st, dt, at));
    }
    KL(b, 1, launch_rope_qknorm_bwd(st, dt, a.qkv, w.dqkn, a.tq, w.d_cos, w.d_sin, M, Tn, H, Hkv, hd, w.dqkv));
    G(b, w.dqkv, 1, wq, a.h1, d, 1, GR(pq), d, wq, d, M, EPI_WGRAD);                // d c_q,c_k,c_v (contiguous)
    GA(b, w.dqkv, wq, 1, W(pq), d, 1, w.dh, d, M, d, wq, EPI_STORE);                 // d h1
    KL(b, 1, launch_rmsnorm_bwd(st, dt, w.xs[l], a.t1, w.dh, w.dx, M, d, w.dx));
  }
  CK(b, cudaMemsetAsync(GR(0), 0, (size_t)c.params[0].numel * 4, st));
  if (w.emb_scratch) {
    // per-position gradient rows into dh (free by now), then summed per token in position order
    KL(b, 1, launch_embed_norm_bwd_rows(st, dt, W(0), ids, M, d, V, w.dx, w.t0, w.dh));
    KL(b, 4, launch_embed_scatter_sorted(st, dt, ids, M, d, V, w.dh, w.emb_scratch, w.emb_scratch_bytes, GR(0)));
  } else {
    KL(b, 1, launch_embed_norm_bwd(st, dt, W(0), ids, M, d, V, w.dx, w.t0, GR(0)));
  }
  KL(b, 1, launch_round_guard_f32(st, dt, GR(0), (size_t)c.params[0].numel, 100.f));
  return PCPB_OK;
}


// Attention of either family on the (qkn, qkv) buffers; picks tcgen05, mma.sync or the generic kernels.
int attention_fwd(pcpb_backend* b, LayerActs& a, float scale) {
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  const int dt = c.dtype;
  FlashArgs fa{};
  fa.qkn = a.qkn; fa.qkv = a.qkv; fa.o = a.o; fa.mrow = a.mrow; fa.lrow = a.lrow;
  fa.B = (int)c.B; fa.T = (int)c.T; fa.H = (int)c.H; fa.Hkv = (int)c.Hkv; fa.hd = (int)c.hd; fa.scale = scale;
  const bool fast = !b->force_generic && dt == DT_BF16 && b->attn_path != 2;
  if (fast && b->attn_path == 0 && attn_tc_supported(fa)) { KL(b, 1, launch_attn_tc_fwd(b->stream, fa, w.tc_err)); return PCPB_OK; }
  if (fast && flash_supported(fa)) { KL(b, 1, launch_flash_fwd(b->stream, fa)); return PCPB_OK; }
  AttnArgs at{};
  at.qkn = a.qkn; at.qkv = a.qkv; at.o = a.o; at.mrow = a.mrow; at.lrow = a.lrow;
  at.B = fa.B; at.T = fa.T; at.H = fa.H; at.Hkv = fa.Hkv; at.hd = fa.hd; at.scale = scale;
  if (!b->force_generic && attn_f32_supported(dt, at)) KL(b, 1, launch_attn_f32_fwd(b->stream, at));
  else KL(b, 1, launch_attn_fwd_generic(b->stream, dt, at));
  return PCPB_OK;
}
int attention_bwd(pcpb_backend* b, LayerActs& a, float scale) {
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  const int dt = c.dtype;
  FlashArgs fa{};
  fa.qkn = a.qkn; fa.qkv = a.qkv; fa.o = a.o; fa.mrow = a.mrow; fa.lrow = a.lrow;
  fa.B = (int)c.B; fa.T = (int)c.T; fa.H = (int)c.H; fa.Hkv = (int)c.Hkv; fa.hd = (int)c.hd; fa.scale = scale;
  fa.dout = w.dout; fa.dqkn = w.dqkn; fa.dqkv = w.dqkv; fa.drow = w.drow;
    fa.stat4 = reinterpret_cast<float4*>(w.drow + (size_t)c.B * c.H * c.T);
  const bool fast = !b->force_generic && dt == DT_BF16 && b->attn_path != 2;
  if (fast && b->attn_path == 0 && attn_tc_supported(fa)) { KL(b, 3, launch_attn_tc_bwd(b->stream, fa, w.tc_err)); return PCPB_OK; }
  if (fast && flash_supported(fa)) { KL(b, 3, launch_flash_bwd(b->stream, fa)); return PCPB_OK; }
  AttnArgs at{};
  at.qkn = a.qkn; at.qkv = a.qkv; at.o = a.o; at.mrow = a.mrow; at.lrow = a.lrow;
  at.B = fa.B; at.T = fa.T; at.H = fa.H; at.Hkv = fa.Hkv; at.hd = fa.hd; at.scale = scale;
  at.dout = w.dout; at.dqkn = w.dqkn; at.dqkv = w.dqkv; at.dkv_acc = w.dkv_acc;
  if (!b->force_generic && attn_f32_supported(dt, at)) KL(b, 3, launch_attn_f32_bwd(b->stream, at, w.dkv_acc));
  else KL(b, 3, launch_attn_bwd_generic(b->stream, dt, at));
  return PCPB_OK;
}

// nanoGPT family: learned position embedding, LayerNorm (gamma, beta), fused c_attn, ReLU or tanh-GELU MLP, lm_head with bias,
// plain cross entropy ignoring targets == -100 (models/nanogpt_small.mlir, models/nanogpt_medium_bf16.mlir).
int forward_backward_gpt(pcpb_backend* b, const void* wts, const long long* ids, const long long* targets, float* grads,
                         float* loss_out, bool backward, float seed) {
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  cudaStream_t st = b->stream;
  const int dt = c.dtype, M = (int)c.M(), d = (int)c.d, F = (int)c.F, V = (int)c.V, L = (int)c.L, Tn = (int)c.T;
  const int wq = 3 * d, Bn = (int)c.B;
  const size_t es = dtype_size(dt);
  const bool gelu = (c.activation == ACT_GELU_TANH);
  auto W = [&](int i) { return (const void*)((const char*)wts + (size_t)c.params[i].offset * es); };
  auto GR = [&](int i) { return grads + c.params[i].offset; };
  float scale = (float)(1.0 / sqrt((double)c.hd));
  if (dt == DT_BF16) {
    uint32_t u; memcpy(&u, &scale, 4);
    u = (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u;
    memcpy(&scale, &u, 4);
  }
  KL(b, 1, launch_embed_pos_fwd(st, dt, W(0), W(1), ids, M, Tn, d, V, w.xs[0]));
  for (int l = 0; l < L; ++l) {
    LayerActs& a = w.layers[l];
    const int p0 = 2 + 8 * l;                       // ln1.w ln1.b c_attn c_proj ln2.w ln2.b c_fc mlp.c_proj
    KL(b, 1, launch_layernorm_fwd(st, dt, w.xs[l], W(p0), W(p0 + 1), M, d, a.h1, a.mu1, a.t1, a.m64_1));
    G(b, a.h1, d, 1, W(p0 + 2), 1, d, a.qkv, wq, M, wq, d, EPI_STORE);
    KL(b, 1, launch_copy_cols(st, dt, a.qkv, wq, a.qkn, 2 * d, M, 2 * d));          // q|k in the attention layout
    int r = attention_fwd(b, a, scale);
    if (r) return r;
    G(b, a.o, d, 1, W(p0 + 3), 1, d, a.xmid, d, M, d, d, EPI_RESID, w.xs[l]);
    KL(b, 1, launch_layernorm_fwd(st, dt, a.xmid, W(p0 + 4), W(p0 + 5), M, d, a.h2, a.mu2, a.t2, a.m64_2));
    G(b, a.h2, d, 1, W(p0 + 6), 1, d, a.u, F, M, F, d, gelu ? EPI_GELU : EPI_RELU, nullptr, a.a);
    G(b, a.a, F, 1, W(p0 + 7), 1, F, w.xs[l + 1], d, M, d, F, EPI_RESID, a.xmid);
  }
  const int pf = 2 + 8 * L;                         // ln_f.w ln_f.b lm_head.w lm_head.b
  KL(b, 1, launch_layernorm_fwd(st, dt, w.xs[L], W(pf), W(pf + 1), M, d, w.hf, w.muf, w.tf, w.m64f));
  G(b, w.hf, d, 1, W(pf + 2), 1, d, w.logits, V, M, V, d, EPI_BIAS, W(pf + 3));
  KL(b, 1, launch_count_valid(st, targets, M, c.ignore_index, w.count));
  KL(b, 1, launch_softcap_ce(st, dt, w.logits, targets, M, V, 0.f, c.ignore_index, w.count, w.rowloss, backward ? 1 : 0, seed));
  KL(b, 1, launch_loss_finalize(st, w.rowloss, M, w.count, loss_out));
  if (!backward) return PCPB_OK;

  KL(b, 2, launch_colsum(st, dt, w.logits, M, V, w.cs_partial, GR(pf + 3)));       // d lm_head.b
  GA(b, w.logits, V, 1, W(pf + 2), d, 1, w.dh, d, M, d, V, EPI_STORE);              // d hf
  G(b, w.logits, 1, V, w.hf, d, 1, GR(pf + 2), d, V, d, M, EPI_WGRAD);             // d lm_head.w
  KL(b, 2, launch_layernorm_bwd(st, dt, w.xs[L], W(pf), w.muf, w.tf, w.m64f, w.dh, nullptr, M, d, w.dx, w.ln_partial,
                                GR(pf), GR(pf + 1)));
  for (int l = L - 1; l >= 0; --l) {
    LayerActs& a = w.layers[l];
    const int p0 = 2 + 8 * l;
    G(b, w.dx, d, 1, W(p0 + 7), F, 1, w.du, F, M, F, d, gelu ? EPI_DGELU : EPI_DRELU, a.u);           // du
    G(b, w.dx, 1, d, a.a, F, 1, GR(p0 + 7), F, d, F, M, EPI_WGRAD);                // d mlp.c_proj
    G(b, w.du, 1, F, a.h2, d, 1, GR(p0 + 6), d, F, d, M, EPI_WGRAD);               // d c_fc
    GA(b, w.du, F, 1, W(p0 + 6), d, 1, w.dh, d, M, d, F, EPI_STORE);                // d h2
    KL(b, 2, launch_layernorm_bwd(st, dt, a.xmid, W(p0 + 4), a.mu2, a.t2, a.m64_2, w.dh, w.dx, M, d, w.dx, w.ln_partial,
                                  GR(p0 + 4), GR(p0 + 5)));
    GA(b, w.dx, d, 1, W(p0 + 3), d, 1, w.dout, d, M, d, d, EPI_STORE);              // d o
    G(b, w.dx, 1, d, a.o, d, 1, GR(p0 + 3), d, d, d, M, EPI_WGRAD);                // d c_proj
    int r = attention_bwd(b, a, scale);
    if (r) return r;
    KL(b, 1, launch_copy_cols(st, dt, w.dqkn, 2 * d, w.dqkv, wq, M, 2 * d));       // dq|dk next to dv
    G(b, w.dqkv, 1, wq, a.h1, d, 1, GR(p0 + 2), d, wq, d, M, EPI_WGRAD);           // d c_attn
    GA(b, w.dqkv, wq, 1, W(p0 + 2), d, 1, w.dh, d, M, d, wq, EPI_STORE);            // d h1
    KL(b, 2, launch_layernorm_bwd(st, dt, w.xs[l], W(p0), a.mu1, a.t1, a.m64_1, w.dh, w.dx, M, d, w.dx, w.ln_partial,
                                  GR(p0), GR(p0 + 1)));
  }
  CK(b, cudaMemsetAsync(GR(0), 0, (size_t)c.params[0].numel * 4, st));
  if (w.emb_scratch) {
    KL(b, 1, launch_embed_pos_bwd(st, dt, ids, Bn, Tn, d, V, w.dx, nullptr, GR(1)));        // position-embedding gradient only
    KL(b, 4, launch_embed_scatter_sorted(st, dt, ids, M, d, V, w.dx, w.emb_scratch, w.emb_scratch_bytes, GR(0)));
  } else {
    KL(b, 1, launch_embed_pos_bwd(st, dt, ids, Bn, Tn, d, V, w.dx, GR(0), GR(1)));
  }
  KL(b, 1, launch_round_guard_f32(st, dt, GR(0), (size_t)(c.params[0].numel + c.params[1].numel), 100.f));
  return PCPB_OK;
}

// Random-window batch of the loaded model's [B,T] into (ids, targets): the starts come from `g` on the host, the
// gather and the widening run on the device.  Host chunks: the B windows of T+1 tokens are gathered into a staging
// buffer first, so that only (T+1)*B tokens cross PCIe.
int random_batch_into(pcpb_backend* b, pcpb_prng* g, const void* tokens, int token_bytes, size_t n_tokens,
                      bool on_device, long long* ids, long long* targets) {
  const ModelConfig& c = b->cfg;
  const size_t B = (size_t)c.B, T = (size_t)c.T;
  std::vector<uint64_t> starts(B);
  const int rc = pcpb_random_window_starts(g, n_tokens, B, T, starts.data());
  if (rc == PCPB_E_CHUNK_TOO_SMALL) return fail(b, rc, "ChunkTooSmall: token chunk not longer than T+1");
  if (rc) return fail(b, rc, "bad random-batch arguments");
  if (!b->starts_dev) CK(b, cudaMalloc(&b->starts_dev, B * 8));
  const void* base = tokens;
  if (!on_device) {
    const size_t wlen = T + 1, need = B * wlen * (size_t)token_bytes;
    if (b->window_stage_cap < need) {
      if (b->window_stage) { CK(b, cudaStreamSynchronize(b->stream)); cudaFree(b->window_stage); b->window_stage = nullptr; }
      CK(b, cudaMalloc(&b->window_stage, need));
      b->window_stage_cap = need;
    }
    // the previous step's copy out of the host gather buffer must have been issued completely: a copy from pageable
    // memory is staged before cudaMemcpyAsync returns, so the buffer can be refilled here
    b->window_host.resize((need + 1) / 2);
    char* dst = (char*)b->window_host.data();
    for (size_t i = 0; i < B; ++i) {
      memcpy(dst + i * wlen * token_bytes, (const char*)tokens + starts[i] * (size_t)token_bytes, wlen * token_bytes);
      starts[i] = i * wlen;
    }
    CK(b, cudaMemcpyAsync(b->window_stage, dst, need, cudaMemcpyHostToDevice, b->stream));
    base = b->window_stage;
  }
  CK(b, cudaMemcpyAsync(b->starts_dev, starts.data(), B * 8, cudaMemcpyHostToDevice, b->stream));
  KL(b, 1, launch_window_batch(b->stream, base, token_bytes, b->starts_dev, (int)B, (long long)T, ids, targets));
  return PCPB_OK;
}

AdamHyper hyper_at(const pcpb_backend* b, float t) {
  AdamHyper h = b->adam;
  h.m_corr = fmaxf(1.f - powf(h.beta1, t), h.eps);
  h.v_corr = fmaxf(1.f - powf(h.beta2, t), h.eps);
  return h;
}

int require_loaded(pcpb_backend* b) {
  if (!b) return PCPB_E_INVALID;
  if (!b->loaded || !b->ws.ready) return fail(b, PCPB_E_ARTIFACT, "no artefact loaded (call pcpb_load_artifact first)");
  return PCPB_OK;
}

}  // namespace

// =================================================================================================
// C ABI
// =================================================================================================
extern "C" {

int pcpb_create(int device_ordinal, pcpb_backend** out) {
  if (!out) return PCPB_E_INVALID;
  *out = nullptr;
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  pcpb_backend* b = new pcpb_backend();
  b->device = device_ordinal;
  b->adam.lr = 1e-3f; b->adam.beta1 = 0.9f; b->adam.beta2 = 0.999f; b->adam.eps = 1e-8f; b->adam.wd = 0.01f;
  b->adam.max_norm = 1.0f; b->adam.m_corr = b->adam.v_corr = 1.f;
  const char* fg = getenv("PCPB_FORCE_GENERIC");
  b->force_generic = fg && fg[0] == '1';
  const char* ap = getenv("PCPB_ATTN");                 // "flash": mma.sync kernels, "generic": SIMT kernels
  b->attn_path = (ap && !strcmp(ap, "flash")) ? 1 : ((ap && !strcmp(ap, "generic")) ? 2 : 0);
  *out = b;                       // returned even on failure so that the message can be read
  if (e != cudaSuccess || ndev == 0)
    return fail(b, PCPB_E_CUDA, std::string("no CUDA device: ") + cudaGetErrorString(e));
  if (device_ordinal < 0 || device_ordinal >= ndev) return fail(b, PCPB_E_INVALID, "device ordinal out of range");
  CK(b, cudaSetDevice(device_ordinal));
  cudaDeviceProp prop;
  CK(b, cudaGetDeviceProperties(&prop, device_ordinal));
  if (prop.major != 10)
    return fail(b, PCPB_E_CUDA, "this library is built for sm_100a (B200) only; found compute capability " +
                                    std::to_string(prop.major) + "." + std::to_string(prop.minor));
  CK(b, cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking));
  CK(b, cudaEventCreate(&b->ev0));
  CK(b, cudaEventCreate(&b->ev1));
  CK(b, cudaEventCreate(&b->tm0));
  CK(b, cudaEventCreate(&b->tm1));
  return PCPB_OK;
}

void pcpb_destroy(pcpb_backend* b) {
  if (!b) return;
  DeviceGuard g(b->device);
  if (b->stream) cudaStreamSynchronize(b->stream);
  free_workspace(b);
  for (cudaEvent_t e : b->prof_events) cudaEventDestroy(e);
  if (b->tm0) cudaEventDestroy(b->tm0);
  if (b->tm1) cudaEventDestroy(b->tm1);
  for (cudaEvent_t e : b->frag_ev) if (e) cudaEventDestroy(e);
  if (b->side_stream) cudaStreamDestroy(b->side_stream);
  if (b->ev0) cudaEventDestroy(b->ev0);
  if (b->ev1) cudaEventDestroy(b->ev1);
  if (b->stream) cudaStreamDestroy(b->stream);
  delete b;
}

const char* pcpb_backend_type(const pcpb_backend*) { return "cuda"; }
const char* pcpb_last_error(const pcpb_backend* b) { return b ? b->err.c_str() : "null backend"; }
void pcpb_free(void* p) { free(p); }
long long pcpb_launch_count(const pcpb_backend* b) { return b ? b->launches : 0; }

// Describes a graph the family recogniser refused as a FAMILY_GRAPH model: parameters = all @main arguments but the
// last two (src/mlir/model_introspection.zig:251-312), which are the i64 [B, T] inputs; the result is the scalar loss.
static std::string general_model(const void* bytes, size_t n, ModelConfig* c, Graph* graph) {
  std::string why = graph_parse((const char*)bytes, n, true, graph);
  if (!why.empty()) return why;
  const int n_args = (int)graph->args.size();
  if (n_args < 3) return "@main needs parameters and two data inputs";
  const GValue &ids = graph->vals[graph->args[n_args - 2]], &tg = graph->vals[graph->args[n_args - 1]];
  if (ids.dt != DT_I64 || tg.dt != DT_I64 || ids.shape != tg.shape || ids.shape.size() != 2) return "the last two arguments must be i64 [B, T]";
  const GValue& ret = graph->vals[graph->ret];
  if (ret.numel != 1 || !(ret.dt == DT_F32 || ret.dt == DT_BF16 || ret.dt == DT_F64)) return "@main must return a scalar loss";
  *c = ModelConfig();
  c->family = FAMILY_GRAPH;
  c->dtype = graph->vals[graph->args[0]].dt;
  if (c->dtype != DT_F32 && c->dtype != DT_BF16) return "parameters must be f32 or bf16";
  c->B = ids.shape[0]; c->T = ids.shape[1];
  int64_t off = 0;
  for (int i = 0; i < n_args - 2; ++i) {
    const GValue& v = graph->vals[graph->args[i]];
    if (v.dt != c->dtype) return "parameters of different element types";
    TensorInfo t;
    t.shape = v.shape; t.numel = v.numel; t.offset = off;
    off += v.numel;
    c->params.push_back(t);
  }
  c->total_params = off;
  if (c->params[0].shape.size() == 2) c->V = c->params[0].shape[0];      // the token table comes first in the exports
  return graph_add_gradients(graph, n_args - 2, 1, -100.f, 100.f);
}

// The two fused families first; anything else (or everything, with PCPB_FRONTEND=graph) through the general front end.
static std::string recognise(const void* bytes, size_t n, ModelConfig* c, Graph* graph) {
  const char* e = getenv("PCPB_FRONTEND");
  const bool force = e && strcmp(e, "graph") == 0;
  std::string why = force ? std::string("general front end forced") : parse_artifact((const char*)bytes, n, c);
  if (why.empty()) return "";
  if (e && strcmp(e, "fused") == 0) return why;
  const std::string why2 = general_model(bytes, n, c, graph);
  if (why2.empty()) return "";
  return force ? why2 : why + "; general front end: " + why2;
}

int pcpb_load_artifact(pcpb_backend* b, const void* bytes, size_t n) {
  if (!b || !bytes || n == 0) return fail(b, PCPB_E_INVALID, "null artefact");
  if (!b->stream) return fail(b, PCPB_E_CUDA, "backend has no device");
  if (b->loaded && b->art_ptr == bytes && b->art_len == n) return PCPB_OK;     // same (ptr, len): keep the session
  DeviceGuard g(b->device);
  ModelConfig c;
  Graph graph;
  std::string why = recognise(bytes, n, &c, &graph);
  if (!why.empty()) return fail(b, PCPB_E_ARTIFACT, "artefact not recognised: " + why);
  CK(b, cudaStreamSynchronize(b->stream));
  free_workspace(b);
  b->cfg = c;
  b->graph = std::move(graph);
  b->loaded = false;
  int r = build_workspace(b);
  if (r) { free_workspace(b); return r; }
  b->art_ptr = bytes; b->art_len = n; b->loaded = true;
  return PCPB_OK;
}

int pcpb_inspect_artifact(const void* bytes, size_t n, int64_t* facts, char* err, size_t err_cap) {
  if (!bytes || !facts) return PCPB_E_INVALID;
  ModelConfig c;
  Graph graph;
  std::string why = recognise(bytes, n, &c, &graph);
  if (!why.empty()) {
    if (err && err_cap) snprintf(err, err_cap, "%s", why.c_str());
    return PCPB_E_ARTIFACT;
  }
  const int64_t f[12] = {c.V, c.d, c.L, c.H, c.Hkv, c.hd, c.F, c.B, c.T, c.dtype, (int64_t)c.params.size(), c.total_params};
  memcpy(facts, f, sizeof f);
  if (err && err_cap) err[0] = 0;
  return PCPB_OK;
}

int pcpb_graph_describe(const void* bytes, size_t n, int with_gradients, char** text_out, char* err, size_t err_cap) {
  if (!bytes || !text_out) return PCPB_E_INVALID;
  *text_out = nullptr;
  Graph g;
  std::string why = graph_parse((const char*)bytes, n, true, &g);
  if (why.empty() && with_gradients) {
    if (g.args.size() < 3) why = "@main needs parameters and two data inputs";
    else why = graph_add_gradients(&g, (int)g.args.size() - 2, 1, -100.f, 100.f);
  }
  if (!why.empty()) {
    if (err && err_cap) snprintf(err, err_cap, "%s", why.c_str());
    return PCPB_E_ARTIFACT;
  }
  std::string s = graph_dump(g);
  if (with_gradients == 2) {
    // the executor's plan of the same program (constant folding, dropped and fused ops, arena layout), no device needed
    std::vector<int64_t> offs;
    int64_t off = 0;
    for (size_t i = 0; i + 2 < g.args.size(); ++i) { offs.push_back(off); off += g.vals[g.args[i]].numel; }
    std::string plan;
    why = graph_exec_plan_text(g, (int)g.args.size() - 2, offs, &plan);
    if (!why.empty()) {
      if (err && err_cap) snprintf(err, err_cap, "%s", why.c_str());
      return PCPB_E_ARTIFACT;
    }
    s += plan;
  }
  char* out = (char*)malloc(s.size() + 1);
  if (!out) return PCPB_E_INVALID;
  memcpy(out, s.c_str(), s.size() + 1);
  *text_out = out;
  if (err && err_cap) err[0] = 0;
  return PCPB_OK;
}

int pcpb_num_params(const pcpb_backend* b) { return (b && b->loaded) ? (int)b->cfg.params.size() : -1; }

int pcpb_param_shape(const pcpb_backend* b, int index, int64_t* shape_out, int* rank_out) {
  if (!b || !b->loaded || index < 0 || index >= (int)b->cfg.params.size() || !shape_out || !rank_out) return PCPB_E_INVALID;
  const auto& s = b->cfg.params[index].shape;
  *rank_out = (int)s.size();
  for (size_t i = 0; i < s.size() && i < 8; ++i) shape_out[i] = s[i];
  return PCPB_OK;
}

int pcpb_model_info(const pcpb_backend* b, int64_t* batch, int64_t* block, int64_t* vocab, int* model_dtype,
                    int64_t* total_params) {
  if (!b || !b->loaded) return PCPB_E_ARTIFACT;
  if (batch) *batch = b->cfg.B;
  if (block) *block = b->cfg.T;
  if (vocab) *vocab = b->cfg.V;
  if (model_dtype) *model_dtype = b->cfg.dtype;
  if (total_params) *total_params = b->cfg.total_params;
  return PCPB_OK;
}

int pcpb_set_adam(pcpb_backend* b, const pcpb_adam_conf* c) {
  if (!b || !c) return PCPB_E_INVALID;
  b->adam.lr = c->learning_rate; b->adam.beta1 = c->beta1; b->adam.beta2 = c->beta2; b->adam.eps = c->epsilon;
  b->adam.wd = c->weight_decay; b->adam.max_norm = c->max_grad_norm;
  return PCPB_OK;
}

// ---- buffers -----------------------------------------------------------------------------------
int pcpb_buffer_from_host(pcpb_backend* b, const void* src, size_t nbytes, const int64_t* shape, int rank, int dtype,
                          pcpb_buffer** out) {
  if (!b || !out || (rank > 0 && !shape) || rank < 0 || rank > 8) return fail(b, PCPB_E_INVALID, "bad buffer arguments");
  if (!b->stream) return fail(b, PCPB_E_CUDA, "backend has no device");
  if (dtype < 0 || dtype > PCPB_BOOL) return fail(b, PCPB_E_INVALID, "unknown dtype");
  const size_t want = numel_of(shape, rank) * dtype_size(dtype);
  if (nbytes != want) return fail(b, PCPB_E_INVALID, "byte length does not match shape and dtype");
  if (nbytes && !src) return fail(b, PCPB_E_INVALID, "null source");
  DeviceGuard g(b->device);
  Block* blk = nullptr;
  int r = alloc_block(b, nbytes, &blk);
  if (r) return r;
  if (nbytes) {
    cudaError_t e = cudaMemcpyAsync(blk->ptr, src, nbytes, cudaMemcpyHostToDevice, b->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(b->stream);
    if (e != cudaSuccess) { block_release(blk); return fail(b, PCPB_E_CUDA, std::string("H2D copy failed: ") + cudaGetErrorString(e)); }
  }
  *out = make_view(b, blk, blk->ptr, nbytes, shape, rank, dtype);
  block_release(blk);             // the view holds the only reference now
  return PCPB_OK;
}

int pcpb_buffer_zeros(pcpb_backend* b, const int64_t* shape, int rank, int dtype, pcpb_buffer** out) {
  if (!b || !out || (rank > 0 && !shape) || rank < 0 || rank > 8) return fail(b, PCPB_E_INVALID, "bad buffer arguments");
  if (!b->stream) return fail(b, PCPB_E_CUDA, "backend has no device");
  if (dtype < 0 || dtype > PCPB_BOOL) return fail(b, PCPB_E_INVALID, "unknown dtype");
  DeviceGuard g(b->device);
  const size_t nbytes = numel_of(shape, rank) * dtype_size(dtype);
  Block* blk = nullptr;
  int r = alloc_block(b, nbytes, &blk);
  if (r) return r;
  cudaError_t e = cudaMemsetAsync(blk->ptr, 0, nbytes, b->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(b->stream);
  if (e != cudaSuccess) { block_release(blk); return fail(b, PCPB_E_CUDA, std::string("memset failed: ") + cudaGetErrorString(e)); }
  *out = make_view(b, blk, blk->ptr, nbytes, shape, rank, dtype);
  block_release(blk);
  return PCPB_OK;
}

void pcpb_buffer_retain(pcpb_buffer* buf) { if (buf) buf->refs.fetch_add(1); }
void pcpb_buffer_release(pcpb_buffer* buf) {
  if (buf && buf->refs.fetch_sub(1) == 1) { block_release(buf->block); delete buf; }
}
size_t pcpb_buffer_nbytes(const pcpb_buffer* buf) { return buf ? buf->nbytes : 0; }

int pcpb_read_to_host(pcpb_backend* b, const pcpb_buffer* buf, void* dst, size_t nbytes) {
  if (!b || !buf || (!dst && nbytes)) return fail(b, PCPB_E_INVALID, "bad read arguments");
  if (nbytes != buf->nbytes) return fail(b, PCPB_E_INVALID, "read length does not match the buffer");
  DeviceGuard g(b->device);
  CK(b, cudaMemcpyAsync(dst, buf->ptr, nbytes, cudaMemcpyDeviceToHost, b->stream));
  CK(b, cudaStreamSynchronize(b->stream));
  return PCPB_OK;
}

int pcpb_adjoint_status(pcpb_backend* b, int* flags, int clear) {
  if (!b || !b->stream || !flags) return PCPB_E_INVALID;
  DeviceGuard g(b->device);
  int total = 0, one = 0;
  cudaError_t (*fetch[])(cudaStream_t, int*, bool) = {adj_status_fetch_kernels, adj_status_fetch_kernels_gpt, adj_status_fetch_gemm_tc,
                                                      adj_status_fetch_attn_tc, adj_status_fetch_attn_flash,
                                                      adj_status_fetch_attn_f32};
  for (auto f : fetch) {
    one = 0;
    CK(b, f(b->stream, &one, clear != 0));
    total |= one;
  }
  *flags = total;
  return PCPB_OK;
}

int pcpb_synchronize(pcpb_backend* b) {
  if (!b || !b->stream) return PCPB_E_INVALID;
  DeviceGuard g(b->device);
  CK(b, cudaStreamSynchronize(b->stream));
  return (b->loaded && b->ws.ready) ? check_tc_error(b) : PCPB_OK;
}

// ---- execute -----------------------------------------------------------------------------------
static int check_param_inputs(pcpb_backend* b, pcpb_buffer* const* in, size_t first, int dtype, const char* what) {
  const ModelConfig& c = b->cfg;
  for (size_t i = 0; i < c.params.size(); ++i) {
    const pcpb_buffer* x = in[first + i];
    if (!x) return fail(b, PCPB_E_INVALID, std::string("null input buffer in ") + what);
    if (x->dtype != dtype || x->nbytes != (size_t)c.params[i].numel * dtype_size(dtype))
      return fail(b, PCPB_E_INVALID, std::string(what) + ": buffer " + std::to_string(i) + " has the wrong dtype or size");
  }
  return PCPB_OK;
}

static int gather_flat(pcpb_backend* b, pcpb_buffer* const* in, size_t first, void* flat, size_t es) {
  const ModelConfig& c = b->cfg;
  for (size_t i = 0; i < c.params.size(); ++i)
    CK(b, cudaMemcpyAsync((char*)flat + (size_t)c.params[i].offset * es, in[first + i]->ptr,
                          (size_t)c.params[i].numel * es, cudaMemcpyDeviceToDevice, b->stream));
  return PCPB_OK;
}

static int flat_views(pcpb_backend* b, Block* blk, int dtype, pcpb_buffer** out) {
  const ModelConfig& c = b->cfg;
  const size_t es = dtype_size(dtype);
  for (size_t i = 0; i < c.params.size(); ++i)
    out[i] = make_view(b, blk, (char*)blk->ptr + (size_t)c.params[i].offset * es, (size_t)c.params[i].numel * es,
                       c.params[i].shape.data(), (int)c.params[i].shape.size(), dtype);
  return PCPB_OK;
}

int pcpb_execute(pcpb_backend* b, const char* fn, pcpb_buffer* const* in, size_t n_in, pcpb_buffer*** out, size_t* n_out) {
  int r = require_loaded(b);
  if (r) return r;
  if (!fn || !out || !n_out || (n_in && !in)) return fail(b, PCPB_E_INVALID, "bad execute arguments");
  *out = nullptr; *n_out = 0;
  DeviceGuard g(b->device);
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  const size_t N = c.params.size(), P = (size_t)c.total_params, es = dtype_size(c.dtype);
  const std::string name(fn);
  const int64_t scalar_shape[1] = {0};
  auto data_ok = [&](const pcpb_buffer* x) { return x && x->dtype == PCPB_I64 && x->nbytes == (size_t)c.M() * 8; };

  // These functions stage their inputs in the fused worker's live buffers (parameters, model-dtype copy,
  // gradients).  Inside an open round that would silently replace the round's working parameters, so they are
  // refused until pcpb_worker_end_round.
  const bool stages_params = name == "compute_gradients" || name == "compute_gradients_accumulated" ||
                             name == "model_forward_pass" || name == "main" || name == "model_forward_pass_grad";
  if (stages_params && b->in_round)
    return fail(b, PCPB_E_STATE, name + " cannot run inside an open worker round (it would overwrite the round's working "
                                        "parameters): call pcpb_worker_end_round first");
  if (name == "compute_gradients_accumulated") {
    // GraphBuilder.buildAccumulatedTrainingGraph (src/compiler/graph_builder.zig:435-726): params f32..., ids and
    // targets folded as [S, B, T]; an scf.for over the S micro-batches sums the f32 gradients and the losses.  The
    // caller (src/nodes/workers/worker.zig:1134-1187) divides both by S afterwards.
    if (n_in != N + 2) return fail(b, PCPB_E_INVALID, "compute_gradients_accumulated expects params..., ids[S,B,T], targets[S,B,T]");
    if ((r = check_param_inputs(b, in, 0, PCPB_F32, "compute_gradients_accumulated"))) return r;
    const size_t mb = (size_t)c.M() * 8;
    const pcpb_buffer *bi = in[N], *bt = in[N + 1];
    if (!bi || !bt || bi->dtype != PCPB_I64 || bt->dtype != PCPB_I64 || bi->nbytes == 0 || bi->nbytes % mb ||
        bt->nbytes != bi->nbytes)
      return fail(b, PCPB_E_INVALID, "ids/targets must be i64 [S,B,T] with S >= 1");
    const size_t S = bi->nbytes / mb;
    if ((r = gather_flat(b, in, 0, w.theta, 4))) return r;
    if (c.dtype != DT_F32) KL(b, 1, launch_convert_f32(b->stream, c.dtype, w.theta, w.shadow, P));
    Block *gb = nullptr, *lb = nullptr;
    if ((r = alloc_block(b, P * 4, &gb))) return r;
    if ((r = alloc_block(b, 4, &lb))) { block_release(gb); return r; }
    cudaError_t e = cudaMemsetAsync(gb->ptr, 0, P * 4, b->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(lb->ptr, 0, 4, b->stream);
    for (size_t s = 0; s < S && r == PCPB_OK && e == cudaSuccess; ++s) {
      r = forward_backward(b, w.shadow, (const long long*)bi->ptr + s * (size_t)c.M(),
                           (const long long*)bt->ptr + s * (size_t)c.M(), w.grads, w.loss, true);
      if (r) break;
      b->launches += 2;
      e = launch_axpy_f32(b->stream, (float*)gb->ptr, w.grads, 1.f, P);
      if (e == cudaSuccess) e = launch_axpy_f32(b->stream, (float*)lb->ptr, w.loss, 1.f, 1);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(b->stream);
    if (r == PCPB_OK && e != cudaSuccess) r = fail(b, PCPB_E_CUDA, std::string("compute_gradients_accumulated failed: ") + cudaGetErrorString(e));
    if (r == PCPB_OK) r = check_tc_error(b);
    if (r) { block_release(gb); block_release(lb); return r; }
    pcpb_buffer** o = (pcpb_buffer**)malloc(sizeof(pcpb_buffer*) * (N + 1));
    flat_views(b, gb, PCPB_F32, o);
    o[N] = make_view(b, lb, lb->ptr, 4, scalar_shape, 0, PCPB_F32);
    block_release(gb); block_release(lb);
    *out = o; *n_out = N + 1;
    return PCPB_OK;
  }
  if (name == "compute_gradients") {
    if (n_in != N + 2) return fail(b, PCPB_E_INVALID, "compute_gradients expects params..., ids, targets");
    if ((r = check_param_inputs(b, in, 0, PCPB_F32, "compute_gradients"))) return r;
    if (!data_ok(in[N]) || !data_ok(in[N + 1])) return fail(b, PCPB_E_INVALID, "ids/targets must be i64 [B,T]");
    if ((r = gather_flat(b, in, 0, w.theta, 4))) return r;
    if (c.dtype != DT_F32) KL(b, 1, launch_convert_f32(b->stream, c.dtype, w.theta, w.shadow, P));
    Block *gb = nullptr, *lb = nullptr;
    if ((r = alloc_block(b, P * 4, &gb))) return r;
    if ((r = alloc_block(b, 4, &lb))) { block_release(gb); return r; }
    r = forward_backward(b, w.shadow, (const long long*)in[N]->ptr, (const long long*)in[N + 1]->ptr, (float*)gb->ptr,
                         (float*)lb->ptr, true);
    cudaError_t e = cudaStreamSynchronize(b->stream);
    if (r == PCPB_OK && e != cudaSuccess) r = fail(b, PCPB_E_CUDA, std::string("compute_gradients failed: ") + cudaGetErrorString(e));
    if (r == PCPB_OK) r = check_tc_error(b);
    if (r) { block_release(gb); block_release(lb); return r; }
    pcpb_buffer** o = (pcpb_buffer**)malloc(sizeof(pcpb_buffer*) * (N + 1));
    flat_views(b, gb, PCPB_F32, o);
    o[N] = make_view(b, lb, lb->ptr, 4, scalar_shape, 0, PCPB_F32);
    block_release(gb); block_release(lb);
    *out = o; *n_out = N + 1;
    return PCPB_OK;
  }
  if (name == "model_forward_pass" || name == "main" || name == "model_forward_pass_grad") {
    const bool grad = (name == "model_forward_pass_grad");
    if (n_in != N + 2 + (grad ? 1 : 0)) return fail(b, PCPB_E_INVALID, name + ": wrong number of inputs");
    if ((r = check_param_inputs(b, in, 0, c.dtype, name.c_str()))) return r;
    if (!data_ok(in[N]) || !data_ok(in[N + 1])) return fail(b, PCPB_E_INVALID, "ids/targets must be i64 [B,T]");
    if ((r = gather_flat(b, in, 0, w.shadow, es))) return r;
    // seed: d(loss) given by the caller (a scalar of the loss's type, f32); it enters at the loss and passes through
    // the guard and clamp of every adjoint edge like any other adjoint
    float seed = 1.f;
    if (grad) {
      if (!in[N + 2] || in[N + 2]->nbytes != 4 || in[N + 2]->dtype != PCPB_F32)
        return fail(b, PCPB_E_INVALID, "model_forward_pass_grad: the loss gradient must be one f32");
      CK(b, cudaMemcpyAsync(&seed, in[N + 2]->ptr, 4, cudaMemcpyDeviceToHost, b->stream));
      CK(b, cudaStreamSynchronize(b->stream));
    }
    Block* lb = nullptr;
    if ((r = alloc_block(b, 4, &lb))) return r;
    r = forward_backward(b, w.shadow, (const long long*)in[N]->ptr, (const long long*)in[N + 1]->ptr, w.grads,
                         (float*)lb->ptr, grad, seed);
    if (r) { block_release(lb); return r; }
    pcpb_buffer** o = nullptr;
    if (grad) {
      // gradients are returned in the model dtype
      Block* gb = nullptr;
      if ((r = alloc_block(b, P * es, &gb))) { block_release(lb); return r; }
      if (c.dtype == DT_F32) CK(b, cudaMemcpyAsync(gb->ptr, w.grads, P * 4, cudaMemcpyDeviceToDevice, b->stream));
      else KL(b, 1, launch_convert_f32(b->stream, c.dtype, w.grads, gb->ptr, P));
      o = (pcpb_buffer**)malloc(sizeof(pcpb_buffer*) * N);
      flat_views(b, gb, c.dtype, o);
      block_release(gb); block_release(lb);
      *n_out = N;
    } else {
      o = (pcpb_buffer**)malloc(sizeof(pcpb_buffer*));
      o[0] = make_view(b, lb, lb->ptr, 4, scalar_shape, 0, PCPB_F32);
      block_release(lb);
      *n_out = 1;
    }
    cudaError_t e = cudaStreamSynchronize(b->stream);
    if (e != cudaSuccess) {
      for (size_t i = 0; i < *n_out; ++i) pcpb_buffer_release(o[i]);
      free(o); *n_out = 0;
      return fail(b, PCPB_E_CUDA, name + " failed: " + cudaGetErrorString(e));
    }
    *out = o;
    return PCPB_OK;
  }
  if (name == "apply_optimizer") {
    if (n_in != 4 * N + 1) return fail(b, PCPB_E_INVALID, "apply_optimizer expects p..., g..., m..., v..., t");
    for (int k = 0; k < 4; ++k)
      if ((r = check_param_inputs(b, in, k * N, PCPB_F32, "apply_optimizer"))) return r;
    if (!in[4 * N] || in[4 * N]->nbytes != 4) return fail(b, PCPB_E_INVALID, "timestep must be one f32");
    float t = 1.f;
    CK(b, cudaMemcpyAsync(&t, in[4 * N]->ptr, 4, cudaMemcpyDeviceToHost, b->stream));
    CK(b, cudaStreamSynchronize(b->stream));
    Block* ob[3] = {nullptr, nullptr, nullptr};
    for (int k = 0; k < 3; ++k)
      if ((r = alloc_block(b, P * 4, &ob[k]))) { for (int j = 0; j < k; ++j) block_release(ob[j]); return r; }
    std::vector<TensorSeg> segs(N);
    std::vector<int> c2s;
    for (size_t i = 0; i < N; ++i) {
      TensorSeg& s = segs[i];
      s.p = (const float*)in[i]->ptr; s.g = (const float*)in[N + i]->ptr;
      s.m = (const float*)in[2 * N + i]->ptr; s.v = (const float*)in[3 * N + i]->ptr;
      s.p_out = (float*)ob[0]->ptr + c.params[i].offset; s.m_out = (float*)ob[1]->ptr + c.params[i].offset;
      s.v_out = (float*)ob[2]->ptr + c.params[i].offset; s.shadow = nullptr;
      s.n = c.params[i].numel; s.first_chunk = (int)c2s.size();
      s.num_chunks = (int)((s.n + ADAM_CHUNK - 1) / ADAM_CHUNK);
      for (int k = 0; k < s.num_chunks; ++k) c2s.push_back((int)i);
    }
    TensorSeg* dsegs = nullptr;
    cudaError_t e = cudaMalloc(&dsegs, sizeof(TensorSeg) * N);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dsegs, segs.data(), sizeof(TensorSeg) * N, cudaMemcpyHostToDevice, b->stream);
    if (e == cudaSuccess) {
      b->launches += 3;
      e = launch_adamw(b->stream, -1, dsegs, (int)N, w.chunk2seg, (int)c2s.size(), w.partial, w.normsq, hyper_at(b, t));
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(b->stream);
    if (dsegs) cudaFree(dsegs);
    if (e != cudaSuccess) {
      for (int k = 0; k < 3; ++k) block_release(ob[k]);
      return fail(b, PCPB_E_CUDA, std::string("apply_optimizer failed: ") + cudaGetErrorString(e));
    }
    pcpb_buffer** o = (pcpb_buffer**)malloc(sizeof(pcpb_buffer*) * 3 * N);
    for (int k = 0; k < 3; ++k) { flat_views(b, ob[k], PCPB_F32, o + k * N); block_release(ob[k]); }
    *out = o; *n_out = 3 * N;
    return PCPB_OK;
  }
  if (name == "accumulate_gradients") {
    if (n_in != 2 * N) return fail(b, PCPB_E_INVALID, "accumulate_gradients expects acc..., grads...");
    for (int k = 0; k < 2; ++k)
      if ((r = check_param_inputs(b, in, k * N, PCPB_F32, "accumulate_gradients"))) return r;
    Block* ob = nullptr;
    if ((r = alloc_block(b, P * 4, &ob))) return r;
    if ((r = gather_flat(b, in, 0, ob->ptr, 4))) { block_release(ob); return r; }
    for (size_t i = 0; i < N; ++i) {
      b->launches += 1;
      cudaError_t e = launch_axpy_f32(b->stream, (float*)ob->ptr + c.params[i].offset, (const float*)in[N + i]->ptr, 1.f,
                                      (size_t)c.params[i].numel);
      if (e != cudaSuccess) { block_release(ob); return fail(b, PCPB_E_CUDA, cudaGetErrorString(e)); }
    }
    cudaError_t e = cudaStreamSynchronize(b->stream);
    if (e != cudaSuccess) { block_release(ob); return fail(b, PCPB_E_CUDA, std::string("accumulate_gradients failed: ") + cudaGetErrorString(e)); }
    pcpb_buffer** o = (pcpb_buffer**)malloc(sizeof(pcpb_buffer*) * N);
    flat_views(b, ob, PCPB_F32, o);
    block_release(ob);
    *out = o; *n_out = N;
    return PCPB_OK;
  }
  return fail(b, PCPB_E_FUNCTION, "unknown function: " + name);
}

int pcpb_execute_host(pcpb_backend* b, const char* fn, const void* const* in, const size_t* in_nbytes,
                      const int64_t* const* shapes, const int* ranks, const int* dtypes, size_t n_in, void*** out,
                      size_t** out_nbytes, size_t* n_out) {
  int r = require_loaded(b);
  if (r) return r;
  if (!in || !in_nbytes || !shapes || !ranks || !out || !out_nbytes || !n_out)
    return fail(b, PCPB_E_INVALID, "bad execute_host arguments");
  std::vector<pcpb_buffer*> bufs(n_in, nullptr);
  auto drop = [&]() { for (auto* x : bufs) pcpb_buffer_release(x); };
  for (size_t i = 0; i < n_in; ++i) {
    // dtypes == NULL: all f32 except the last two inputs, which are i64 (src/backends/iree.zig:463-486)
    const int dt = dtypes ? dtypes[i] : (i + 2 >= n_in ? PCPB_I64 : PCPB_F32);
    r = pcpb_buffer_from_host(b, in[i], in_nbytes[i], shapes[i], ranks[i], dt, &bufs[i]);
    if (r) { drop(); return r; }
  }
  pcpb_buffer** o = nullptr;
  size_t no = 0;
  r = pcpb_execute(b, fn, bufs.data(), n_in, &o, &no);
  drop();
  if (r) return r;
  void** host = (void**)malloc(sizeof(void*) * (no ? no : 1));
  size_t* nb = (size_t*)malloc(sizeof(size_t) * (no ? no : 1));
  for (size_t i = 0; i < no; ++i) {
    nb[i] = o[i]->nbytes;
    host[i] = malloc(nb[i] ? nb[i] : 1);
    if (r == PCPB_OK) r = pcpb_read_to_host(b, o[i], host[i], nb[i]);
    pcpb_buffer_release(o[i]);
  }
  free(o);
  if (r) { for (size_t i = 0; i < no; ++i) free(host[i]); free(host); free(nb); return r; }
  *out = host; *out_nbytes = nb; *n_out = no;
  return PCPB_OK;
}

int pcpb_op_gemm(pcpb_backend* b, int path, const pcpb_buffer* A, long long sam, long long sak, const pcpb_buffer* B,
                 long long sbk, long long sbn, pcpb_buffer* C, long long ldc, const pcpb_buffer* R, pcpb_buffer* C2,
                 int M, int N, int K, int epilogue) {
  int r = require_loaded(b);
  if (r) return r;
  if (!A || !B || !C || M < 0 || N < 0 || K < 0 || epilogue < EPI_STORE || epilogue > EPI_DGELU)
    return fail(b, PCPB_E_INVALID, "bad gemm arguments");
  if ((epilogue == EPI_RESID || epilogue == EPI_DRELU2 || epilogue == EPI_DRELU || epilogue == EPI_BIAS || epilogue == EPI_DGELU) && !R)
    return fail(b, PCPB_E_INVALID, "this epilogue needs R");
  if ((epilogue == EPI_RELU2 || epilogue == EPI_RELU || epilogue == EPI_GELU) && !C2) return fail(b, PCPB_E_INVALID, "this epilogue needs C2");
  DeviceGuard g(b->device);
  const size_t es = dtype_size(b->cfg.dtype);
  // extents touched by the strided views must lie inside the buffers
  auto span = [](long long r0, long long s0, long long r1, long long s1) { return (r0 > 0 ? (r0 - 1) * s0 : 0) + (r1 > 0 ? (r1 - 1) * s1 : 0) + 1; };
  if (M && N && K) {
    if ((size_t)span(M, sam, K, sak) * es > A->nbytes || (size_t)span(K, sbk, N, sbn) * es > B->nbytes)
      return fail(b, PCPB_E_INVALID, "operand view exceeds its buffer");
    const size_t ces = (epilogue == EPI_WGRAD) ? 4 : es;
    if ((size_t)span(M, ldc, N, 1) * ces > C->nbytes) return fail(b, PCPB_E_INVALID, "output view exceeds its buffer");
    const size_t r_need = (epilogue == EPI_BIAS) ? (size_t)N * es : (size_t)span(M, ldc, N, 1) * es;
    if (R && r_need > R->nbytes) return fail(b, PCPB_E_INVALID, "R view exceeds its buffer");
    if (C2 && (size_t)span(M, ldc, N, 1) * es > C2->nbytes) return fail(b, PCPB_E_INVALID, "C2 view exceeds its buffer");
  }
  GemmArgs ga = mk(A->ptr, sam, sak, B->ptr, sbk, sbn, C->ptr, ldc, M, N, K, epilogue, R ? R->ptr : nullptr, C2 ? C2->ptr : nullptr);
  ga.scratch = b->ws.tc_scratch; ga.scratch_bytes = b->ws.tc_scratch_bytes; ga.err_word = b->ws.tc_err;
  if (path == 1) KL(b, 1, launch_gemm_generic(b->stream, b->cfg.dtype, ga));
  else if (path == 2) {
    if (b->cfg.dtype != DT_BF16 || !gemm_tc_supported(ga)) return fail(b, PCPB_E_INVALID, "shape not supported by the tensor-core kernel");
    KL(b, gemm_tc_launches(ga), launch_gemm_tc(b->stream, ga));
  } else if ((r = gemm(b, ga))) return r;
  CK(b, cudaStreamSynchronize(b->stream));
  return check_tc_error(b);
}

int pcpb_fifo_get_batch(pcpb_backend* b, const uint16_t* tokens, size_t n_tokens, size_t* cursor,
                        pcpb_buffer** inputs, pcpb_buffer** targets) {
  int r = require_loaded(b);
  if (r) return r;
  if (!tokens || !cursor || !inputs || !targets) return fail(b, PCPB_E_INVALID, "bad get_batch arguments");
  DeviceGuard g(b->device);
  const ModelConfig& c = b->cfg;
  const size_t BT = (size_t)c.M(), needed = BT + 1;
  if (n_tokens < needed) return fail(b, PCPB_E_CHUNK_TOO_SMALL, "ChunkTooSmall: token chunk shorter than B*T+1");
  if (*cursor + needed > n_tokens) return fail(b, PCPB_E_CHUNK_EXHAUSTED, "ChunkExhausted: not enough tokens left for a batch");
  Block *xb = nullptr, *yb = nullptr, *tb = nullptr;
  if ((r = alloc_block(b, BT * 8, &xb))) return r;
  if ((r = alloc_block(b, BT * 8, &yb))) { block_release(xb); return r; }
  if ((r = alloc_block(b, needed * 2, &tb))) { block_release(xb); block_release(yb); return r; }
  cudaError_t e = cudaMemcpyAsync(tb->ptr, tokens + *cursor, needed * 2, cudaMemcpyHostToDevice, b->stream);
  if (e == cudaSuccess) { b->launches += 1; e = launch_fifo_batch(b->stream, (const uint16_t*)tb->ptr, 0, (long long)BT, (long long*)xb->ptr, (long long*)yb->ptr); }
  if (e == cudaSuccess) e = cudaStreamSynchronize(b->stream);
  block_release(tb);
  if (e != cudaSuccess) { block_release(xb); block_release(yb); return fail(b, PCPB_E_CUDA, std::string("get_batch failed: ") + cudaGetErrorString(e)); }
  const int64_t shp[2] = {c.B, c.T};
  *inputs = make_view(b, xb, xb->ptr, BT * 8, shp, 2, PCPB_I64);
  *targets = make_view(b, yb, yb->ptr, BT * 8, shp, 2, PCPB_I64);
  block_release(xb); block_release(yb);
  *cursor += needed;
  return PCPB_OK;
}

int pcpb_random_get_batch(pcpb_backend* b, pcpb_prng* g, const void* tokens, int token_bytes, size_t n_tokens,
                          pcpb_buffer** inputs, pcpb_buffer** targets) {
  int r = require_loaded(b);
  if (r) return r;
  if (!g || !tokens || !inputs || !targets || (token_bytes != 2 && token_bytes != 4))
    return fail(b, PCPB_E_INVALID, "bad get_batch arguments");
  DeviceGuard dg(b->device);
  const ModelConfig& c = b->cfg;
  const size_t BT = (size_t)c.M();
  Block *xb = nullptr, *yb = nullptr;
  if ((r = alloc_block(b, BT * 8, &xb))) return r;
  if ((r = alloc_block(b, BT * 8, &yb))) { block_release(xb); return r; }
  r = random_batch_into(b, g, tokens, token_bytes, n_tokens, false, (long long*)xb->ptr, (long long*)yb->ptr);
  if (r == PCPB_OK && cudaStreamSynchronize(b->stream) != cudaSuccess) r = fail(b, PCPB_E_CUDA, "get_batch failed");
  if (r) { block_release(xb); block_release(yb); return r; }
  const int64_t shp[2] = {c.B, c.T};
  *inputs = make_view(b, xb, xb->ptr, BT * 8, shp, 2, PCPB_I64);
  *targets = make_view(b, yb, yb->ptr, BT * 8, shp, 2, PCPB_I64);
  block_release(xb); block_release(yb);
  return PCPB_OK;
}

int pcpb_init_master(const pcpb_backend* b, uint64_t seed, int dtype, void* blob_out, size_t blob_bytes) {
  if (!b || !b->loaded) return PCPB_E_ARTIFACT;
  return pcpb_init_master_elems(seed, dtype, (size_t)b->cfg.total_params, blob_out, blob_bytes);
}

int pcpb_worker_set_sampling(pcpb_backend* b, int mode, uint64_t seed) {
  if (!b) return PCPB_E_INVALID;
  if (mode != 0 && mode != 1) return fail(b, PCPB_E_INVALID, "sampling mode must be 0 (fifo) or 1 (random)");
  b->sampling = mode;
  pcpb_prng_seed(reinterpret_cast<pcpb_prng*>(b->prng_state), seed);
  return PCPB_OK;
}

int pcpb_worker_write_state(pcpb_backend* b, int which, const float* src, size_t n) {
  int r = require_loaded(b);
  if (r) return r;
  DeviceGuard g(b->device);
  Workspace& w = b->ws;
  const size_t P = (size_t)b->cfg.total_params;
  float* dst = nullptr;
  size_t len = P;
  switch (which) {
    case 0: dst = w.theta; break;
    case 1: dst = w.mstate; break;
    case 2: dst = w.vstate; break;
    case 3: dst = w.delta; break;
    case 4: dst = w.theta0; break;
    case 5: dst = b->velocity; len = (size_t)b->shard_len; break;
    default: return fail(b, PCPB_E_INVALID, "this state cannot be written");
  }
  if (!dst) return fail(b, PCPB_E_STATE, "that state does not exist yet");
  if (n != len || !src) return fail(b, PCPB_E_INVALID, "state length mismatch");
  CK(b, cudaMemcpyAsync(dst, src, n * 4, cudaMemcpyHostToDevice, b->stream));
  if (which == 0 && b->cfg.dtype != DT_F32) KL(b, 1, launch_convert_f32(b->stream, b->cfg.dtype, w.theta, w.shadow, P));
  if (which == 4) b->have_master = true;
  CK(b, cudaStreamSynchronize(b->stream));
  return PCPB_OK;
}

// ---- fused worker round ---------------------------------------------------------------------------
int pcpb_worker_begin_round(pcpb_backend* b, const pcpb_inner_cfg* cfg, const void* params_blob, size_t blob_bytes) {
  int r = require_loaded(b);
  if (r) return r;
  if (!cfg || cfg->tau < 0 || cfg->accumulation_steps < 1) return fail(b, PCPB_E_INVALID, "bad inner-loop configuration");
  if (cfg->param_dtype != PCPB_F32 && cfg->param_dtype != PCPB_BF16) return fail(b, PCPB_E_INVALID, "param_dtype must be f32 or bf16");
  DeviceGuard g(b->device);
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  const size_t P = (size_t)c.total_params;
  if (params_blob) {
    const size_t want = P * dtype_size(cfg->param_dtype);
    if (blob_bytes != want) return fail(b, PCPB_E_INVALID, "parameter blob has the wrong length");
    if (cfg->param_dtype == PCPB_F32) {
      CK(b, cudaMemcpyAsync(w.theta0, params_blob, want, cudaMemcpyHostToDevice, b->stream));
    } else {
      // bf16 blob -> f32 by widening (<<16), src/nodes/workers/worker.zig:1025-1087; staged through w.grads
      CK(b, cudaMemcpyAsync(w.grads, params_blob, want, cudaMemcpyHostToDevice, b->stream));
      KL(b, 1, launch_widen_to_f32(b->stream, DT_BF16, w.grads, w.theta0, P));
    }
  } else if (!b->have_master) {
    return fail(b, PCPB_E_STATE, "no parameter blob given and no master parameters on the device yet");
  }
  CK(b, cudaMemcpyAsync(w.theta, w.theta0, P * 4, cudaMemcpyDeviceToDevice, b->stream));
  if (c.dtype != DT_F32) KL(b, 1, launch_convert_f32(b->stream, c.dtype, w.theta, w.shadow, P));
  b->tau = cfg->tau; b->accumulation_steps = cfg->accumulation_steps; b->param_dtype = cfg->param_dtype;
  b->persist_adam = cfg->persist_adam; b->tokens_on_device = cfg->tokens_on_device;
  if (!cfg->persist_adam || !b->have_master) {
    CK(b, cudaMemsetAsync(w.mstate, 0, P * 4, b->stream));
    CK(b, cudaMemsetAsync(w.vstate, 0, P * 4, b->stream));
    b->timestep = 1.f;
  }
  if (cfg->accumulation_steps > 1 && !w.gacc) WS(b, w.gacc, P * 4);
  const int need = cfg->tau > 0 ? cfg->tau : 1;
  if (w.loss_capacity < need) { WS(b, w.loss_record, (size_t)need * 4); w.loss_capacity = need; }
  CK(b, cudaMemsetAsync(w.loss_record, 0, (size_t)w.loss_capacity * 4, b->stream));
  b->steps_done = 0; b->cursor = 0; b->in_round = true; b->have_master = true;
  return PCPB_OK;
}

int pcpb_worker_set_tokens(pcpb_backend* b, const uint16_t* tokens, size_t n_tokens) {
  int r = require_loaded(b);
  if (r) return r;
  if (!tokens && n_tokens) return fail(b, PCPB_E_INVALID, "null token pointer");
  b->tokens_src = tokens; b->n_tokens = n_tokens; b->cursor = 0;
  return PCPB_OK;
}

int pcpb_worker_step(pcpb_backend* b) {
  int r = require_loaded(b);
  if (r) return r;
  if (!b->in_round) return fail(b, PCPB_E_STATE, "pcpb_worker_step outside a round");
  DeviceGuard g(b->device);
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  const size_t P = (size_t)c.total_params, BT = (size_t)c.M(), needed = BT + 1;
  if (b->steps_done >= w.loss_capacity) return fail(b, PCPB_E_STATE, "more steps than tau in this round");
  const int acc = b->accumulation_steps;
  if (b->sampling == 0 && b->n_tokens < needed) return fail(b, PCPB_E_CHUNK_TOO_SMALL, "ChunkTooSmall: token chunk shorter than B*T+1");
  float* loss_slot = w.loss_record + b->steps_done;
  for (int a = 0; a < acc; ++a) {
    if (b->sampling == 1) {
      if ((r = random_batch_into(b, reinterpret_cast<pcpb_prng*>(b->prng_state), b->tokens_src, 2, b->n_tokens,
                                 b->tokens_on_device != 0, w.ids, w.targets)))
        return r;
    } else {
    if (b->cursor + needed > b->n_tokens) return fail(b, PCPB_E_CHUNK_EXHAUSTED, "ChunkExhausted: not enough tokens left for a batch");
    const uint16_t* win;
    long long cur;
    if (b->tokens_on_device) { win = b->tokens_src; cur = (long long)b->cursor; }
    else {
      if (b->stage_cap < needed) {
        if (b->tokens_stage) { CK(b, cudaStreamSynchronize(b->stream)); cudaFree(b->tokens_stage); b->tokens_stage = nullptr; }
        CK(b, cudaMalloc(&b->tokens_stage, needed * 2));
        b->stage_cap = needed;
      }
      CK(b, cudaMemcpyAsync(b->tokens_stage, b->tokens_src + b->cursor, needed * 2, cudaMemcpyHostToDevice, b->stream));
      win = b->tokens_stage; cur = 0;
    }
    KL(b, 1, launch_fifo_batch(b->stream, win, cur, (long long)BT, w.ids, w.targets));
    b->cursor += needed;
    }
    if ((r = forward_backward(b, w.shadow, w.ids, w.targets, w.grads, w.loss, true))) return r;
    KL(b, 1, launch_axpy_f32(b->stream, loss_slot, w.loss, 1.f, 1));
    if (acc > 1) {
      if (a == 0) CK(b, cudaMemsetAsync(w.gacc, 0, P * 4, b->stream));
      KL(b, 1, launch_axpy_f32(b->stream, w.gacc, w.grads, 1.f, P));
    }
  }
  if (acc > 1) {
    const float s = 1.0f / (float)acc;
    KL(b, 1, launch_scale_f32(b->stream, loss_slot, s, 1));
    KL(b, 1, launch_scale_f32(b->stream, w.gacc, s, P));
    CK(b, cudaMemcpyAsync(w.grads, w.gacc, P * 4, cudaMemcpyDeviceToDevice, b->stream));
  }
  KL(b, 3, launch_adamw(b->stream, c.dtype == DT_F32 ? -1 : c.dtype, w.segs, (int)c.params.size(), w.chunk2seg, w.nchunks,
                        w.partial, w.normsq, hyper_at(b, b->timestep)));
  b->timestep += 1.f;
  b->steps_done += 1;
  return PCPB_OK;
}

int pcpb_worker_end_round(pcpb_backend* b, void* delta_out, size_t delta_bytes, float* losses, size_t n_losses) {
  int r = require_loaded(b);
  if (r) return r;
  if (!b->in_round) return fail(b, PCPB_E_STATE, "pcpb_worker_end_round outside a round");
  DeviceGuard g(b->device);
  const ModelConfig& c = b->cfg;
  Workspace& w = b->ws;
  const size_t P = (size_t)c.total_params;
  const int N = (int)c.params.size();
  // NaN / Inf heal of the Adam state, per tensor (src/nodes/workers/worker.zig:1346-1369)
  CK(b, cudaMemsetAsync(w.heal_flags, 0, sizeof(int) * N, b->stream));
  for (int i = 0; i < N; ++i) {
    KL(b, 1, launch_check_finite(b->stream, w.mstate + c.params[i].offset, (size_t)c.params[i].numel, w.heal_flags + i));
    KL(b, 1, launch_check_finite(b->stream, w.vstate + c.params[i].offset, (size_t)c.params[i].numel, w.heal_flags + i));
  }
  std::vector<int> flags(N, 0);
  CK(b, cudaMemcpyAsync(flags.data(), w.heal_flags, sizeof(int) * N, cudaMemcpyDeviceToHost, b->stream));
  CK(b, cudaStreamSynchronize(b->stream));
  bool healed = false;
  for (int i = 0; i < N; ++i)
    if (flags[i]) {
      CK(b, cudaMemsetAsync(w.mstate + c.params[i].offset, 0, (size_t)c.params[i].numel * 4, b->stream));
      CK(b, cudaMemsetAsync(w.vstate + c.params[i].offset, 0, (size_t)c.params[i].numel * 4, b->stream));
      healed = true;
    }
  if (healed) b->timestep = 1.f;
  KL(b, 1, launch_delta(b->stream, w.theta0, w.theta, w.delta, P, b->param_dtype == PCPB_BF16 ? 1 : 0));
  if (delta_out) {
    const size_t want = P * dtype_size(b->param_dtype);
    if (delta_bytes != want) return fail(b, PCPB_E_INVALID, "delta buffer has the wrong length");
    if (b->param_dtype == PCPB_F32) {
      CK(b, cudaMemcpyAsync(delta_out, w.delta, want, cudaMemcpyDeviceToHost, b->stream));
    } else {
      // truncated values are exactly representable: the rounding convert reproduces the high halves
      KL(b, 1, launch_convert_f32(b->stream, DT_BF16, w.delta, w.grads, P));
      CK(b, cudaMemcpyAsync(delta_out, w.grads, want, cudaMemcpyDeviceToHost, b->stream));
    }
  }
  if (losses && n_losses) {
    const size_t n = n_losses < (size_t)b->steps_done ? n_losses : (size_t)b->steps_done;
    if (n) CK(b, cudaMemcpyAsync(losses, w.loss_record, n * 4, cudaMemcpyDeviceToHost, b->stream));
  }
  CK(b, cudaStreamSynchronize(b->stream));
  if (b->side_stream) CK(b, cudaStreamSynchronize(b->side_stream));
  b->frag_pending.assign(b->frag_pending.size(), 0);
  b->in_round = false;
  return check_tc_error(b);
}

int pcpb_inner_loop(pcpb_backend* b, const pcpb_inner_cfg* cfg, const void* params_blob, size_t blob_bytes,
                    const uint16_t* tokens, size_t n_tokens, void* delta_out, size_t delta_bytes, float* losses) {
  int r = pcpb_worker_begin_round(b, cfg, params_blob, blob_bytes);
  if (r) return r;
  if ((r = pcpb_worker_set_tokens(b, tokens, n_tokens))) return r;
  for (int s = 0; s < cfg->tau; ++s)
    if ((r = pcpb_worker_step(b))) { b->in_round = false; return r; }
  return pcpb_worker_end_round(b, delta_out, delta_bytes, losses, (size_t)cfg->tau);
}

int pcpb_worker_read_state(pcpb_backend* b, int which, float* dst, size_t n) {
  int r = require_loaded(b);
  if (r) return r;
  DeviceGuard g(b->device);
  Workspace& w = b->ws;
  const size_t P = (size_t)b->cfg.total_params;
  const float* src = nullptr;
  size_t len = P;
  switch (which) {
    case 0: src = w.theta; break;
    case 1: src = w.mstate; break;
    case 2: src = w.vstate; break;
    case 3: src = w.delta; break;
    case 4: src = w.theta0; break;
    case 5: src = b->velocity; len = (size_t)b->shard_len; break;
    case 6: src = w.grads; break;
    default: return fail(b, PCPB_E_INVALID, "unknown state selector");
  }
  if (!src) return fail(b, PCPB_E_STATE, "that state does not exist yet");
  if (n != len || !dst) return fail(b, PCPB_E_INVALID, "state length mismatch");
  CK(b, cudaMemcpyAsync(dst, src, n * 4, cudaMemcpyDeviceToHost, b->stream));
  CK(b, cudaStreamSynchronize(b->stream));
  return PCPB_OK;
}

int pcpb_worker_last_loss(pcpb_backend* b, float* loss) {
  int r = require_loaded(b);
  if (r) return r;
  if (!loss) return fail(b, PCPB_E_INVALID, "null loss pointer");
  if (b->steps_done < 1) return fail(b, PCPB_E_STATE, "no step done in this round");
  DeviceGuard g(b->device);
  CK(b, cudaMemcpyAsync(loss, b->ws.loss_record + (b->steps_done - 1), 4, cudaMemcpyDeviceToHost, b->stream));
  CK(b, cudaStreamSynchronize(b->stream));
  return PCPB_OK;
}

int pcpb_timer_start(pcpb_backend* b) {
  if (!b || !b->stream) return PCPB_E_INVALID;
  DeviceGuard g(b->device);
  CK(b, cudaEventRecord(b->tm0, b->stream));
  return PCPB_OK;
}

int pcpb_timer_stop(pcpb_backend* b, double* ms) {
  if (!b || !b->stream || !ms) return PCPB_E_INVALID;
  DeviceGuard g(b->device);
  CK(b, cudaEventRecord(b->tm1, b->stream));
  CK(b, cudaEventSynchronize(b->tm1));
  float f = 0.f;
  CK(b, cudaEventElapsedTime(&f, b->tm0, b->tm1));
  *ms = f;
  return PCPB_OK;
}

int pcpb_profile_enable(pcpb_backend* b, int on) {
  if (!b || !b->stream) return PCPB_E_INVALID;
  DeviceGuard g(b->device);
  if (on && b->prof_events.empty()) {
    b->prof_events.resize(2048);
    for (auto& e : b->prof_events) CK(b, cudaEventCreate(&e));
  }
  int r = drain_profile(b);
  if (r) return r;
  b->profiling = on != 0;
  b->prof_flops = 0.0; b->prof_ms = 0.0; b->prof_launches = 0; b->prof_used = 0;
  return PCPB_OK;
}

int pcpb_profile_read(pcpb_backend* b, long long* launches, double* total_ms, double* total_flops) {
  if (!b || !b->stream) return PCPB_E_INVALID;
  DeviceGuard g(b->device);
  int r = drain_profile(b);
  if (r) return r;
  if (launches) *launches = b->prof_launches;
  if (total_ms) *total_ms = b->prof_ms;
  if (total_flops) *total_flops = b->prof_flops;
  return PCPB_OK;
}

// ---- outer step --------------------------------------------------------------------------------------
static int setup_shard(pcpb_backend* b, int rank, int world) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(b, PCPB_E_INVALID, "world must be 1..8 and 0 <= rank < world");
  const long long P = b->cfg.total_params;
  long long S = (P + world - 1) / world;
  S = (S + 255) / 256 * 256;                 // shard length, a multiple of 256 elements
  // the same (rank, world) again: the shard, and with it the momentum of the outer optimiser, is kept; another
  // membership starts at zero and the host writes the re-sharded velocities (pcpb_worker_write_state, selector 5)
  const bool keep = b->velocity && b->velocity_init && b->rank == rank && b->world == world && b->shard_len == S;
  b->rank = rank; b->world = world; b->shard_len = S;
  if (!keep) {
    if (b->velocity) { CK(b, cudaStreamSynchronize(b->stream)); cudaFree(b->velocity); b->velocity = nullptr; }
    CK(b, cudaMalloc(&b->velocity, (size_t)S * 4));
    CK(b, cudaMemset(b->velocity, 0, (size_t)S * 4));
  }
  b->velocity_init = true;
  b->peer_delta.assign(world, nullptr); b->peer_theta0.assign(world, nullptr);
  b->peer_delta[rank] = b->ws.delta; b->peer_theta0[rank] = b->ws.theta0;
  return PCPB_OK;
}

int pcpb_outer_export(pcpb_backend* b, void* handles_out) {
  int r = require_loaded(b);
  if (r) return r;
  if (!handles_out) return fail(b, PCPB_E_INVALID, "null handle buffer");
  DeviceGuard g(b->device);
  static_assert(sizeof(cudaIpcMemHandle_t) <= PCPB_IPC_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  memset(handles_out, 0, 2 * PCPB_IPC_HANDLE_BYTES);
  CK(b, cudaIpcGetMemHandle(&h, b->ws.delta));
  memcpy(handles_out, &h, sizeof h);
  CK(b, cudaIpcGetMemHandle(&h, b->ws.theta0));
  memcpy((char*)handles_out + PCPB_IPC_HANDLE_BYTES, &h, sizeof h);
  return PCPB_OK;
}

int pcpb_outer_attach_ipc(pcpb_backend* b, int rank, int world, const void* all_handles) {
  int r = require_loaded(b);
  if (r) return r;
  if (!all_handles) return fail(b, PCPB_E_INVALID, "null handles");
  DeviceGuard g(b->device);
  for (void* p : b->ipc_opened) cudaIpcCloseMemHandle(p);
  b->ipc_opened.clear();
  if ((r = setup_shard(b, rank, world))) return r;
  for (int w = 0; w < world; ++w) {
    if (w == rank) continue;
    cudaIpcMemHandle_t h;
    void* p = nullptr;
    memcpy(&h, (const char*)all_handles + (size_t)w * 2 * PCPB_IPC_HANDLE_BYTES, sizeof h);
    CK(b, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    b->ipc_opened.push_back(p); b->peer_delta[w] = (float*)p;
    memcpy(&h, (const char*)all_handles + (size_t)w * 2 * PCPB_IPC_HANDLE_BYTES + PCPB_IPC_HANDLE_BYTES, sizeof h);
    CK(b, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    b->ipc_opened.push_back(p); b->peer_theta0[w] = (float*)p;
  }
  return PCPB_OK;
}

int pcpb_outer_attach_local(pcpb_backend* b, int rank, int world, pcpb_backend* const* peers) {
  int r = require_loaded(b);
  if (r) return r;
  if (!peers) return fail(b, PCPB_E_INVALID, "null peers");
  DeviceGuard g(b->device);
  if ((r = setup_shard(b, rank, world))) return r;
  for (int w = 0; w < world; ++w) {
    if (!peers[w] || !peers[w]->loaded || peers[w]->cfg.total_params != b->cfg.total_params)
      return fail(b, PCPB_E_INVALID, "peer backend missing or loaded with a different model");
    if (peers[w]->device != b->device) {
      int can = 0;
      CK(b, cudaDeviceCanAccessPeer(&can, b->device, peers[w]->device));
      if (!can) return fail(b, PCPB_E_CUDA, "no peer access between the devices");
      cudaError_t e = cudaDeviceEnablePeerAccess(peers[w]->device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) CK(b, e);
      cudaGetLastError();
    }
    b->peer_delta[w] = peers[w]->ws.delta; b->peer_theta0[w] = peers[w]->ws.theta0;
  }
  return PCPB_OK;
}

int pcpb_outer_prepare(pcpb_backend* b, const pcpb_outer_cfg* cfg) {
  int r = require_loaded(b);
  if (r) return r;
  if (!cfg) return fail(b, PCPB_E_INVALID, "null outer configuration");
  DeviceGuard g(b->device);
  // the delta was produced by pcpb_worker_end_round; this call only makes it visible (stream drained)
  if (b->in_round) return fail(b, PCPB_E_STATE, "round still open: call pcpb_worker_end_round first");
  CK(b, cudaStreamSynchronize(b->stream));
  return PCPB_OK;
}

int pcpb_outer_apply(pcpb_backend* b, const pcpb_outer_cfg* cfg, const int* contributors, int n_contributors,
                     double* device_ms) {
  int r = require_loaded(b);
  if (r) return r;
  if (!cfg) return fail(b, PCPB_E_INVALID, "null outer configuration");
  if (!b->velocity_init) return fail(b, PCPB_E_STATE, "outer step not attached (pcpb_outer_attach_*)");
  DeviceGuard g(b->device);
  const long long P = b->cfg.total_params, S = b->shard_len;
  const long long off = (long long)b->rank * S;
  const long long n = off >= P ? 0 : (P - off < S ? P - off : S);
  OuterArgs a{};
  int nc = 0;
  if (contributors) {
    if (n_contributors < 1 || n_contributors > b->world) return fail(b, PCPB_E_INVALID, "bad contributor list");
    for (int i = 0; i < n_contributors; ++i) {
      const int w = contributors[i];
      if (w < 0 || w >= b->world || !b->peer_delta[w]) return fail(b, PCPB_E_INVALID, "contributor rank not attached");
      a.deltas[nc++] = b->peer_delta[w] + off;
    }
  } else {
    for (int w = 0; w < b->world; ++w) {
      if (!b->peer_delta[w]) return fail(b, PCPB_E_STATE, "a peer is not attached");
      a.deltas[nc++] = b->peer_delta[w] + off;
    }
  }
  a.ncontrib = nc; a.vel = b->velocity; a.master = b->ws.theta0 + off;
  a.nouts = 0;
  for (int w = 0; w < b->world; ++w)
    if (w != b->rank) a.outs[a.nouts++] = b->peer_theta0[w] + off;
  a.n = n; a.lr = cfg->learning_rate; a.mu = cfg->momentum; a.trunc = cfg->param_dtype == PCPB_BF16 ? 1 : 0;
  CK(b, cudaEventRecord(b->ev0, b->stream));
  KL(b, 1, launch_nesterov_shard(b->stream, a));
  CK(b, cudaEventRecord(b->ev1, b->stream));
  CK(b, cudaStreamSynchronize(b->stream));
  if (device_ms) { float ms = 0.f; CK(b, cudaEventElapsedTime(&ms, b->ev0, b->ev1)); *device_ms = ms; }
  b->have_master = true;
  return PCPB_OK;
}

// ---- streaming DiLoCo ----------------------------------------------------------------------------------------
static int stream_check(pcpb_backend* b, int fragment) {
  int r = require_loaded(b);
  if (r) return r;
  if (!b->snapshot || b->stream_fragments < 1) return fail(b, PCPB_E_STATE, "streaming not started (pcpb_stream_begin)");
  if (!b->in_round) return fail(b, PCPB_E_STATE, "streaming calls belong inside a round");
  if (fragment < 0 || fragment >= b->stream_fragments) return fail(b, PCPB_E_INVALID, "fragment index out of range");
  return PCPB_OK;
}

int pcpb_stream_begin(pcpb_backend* b, const pcpb_stream_cfg* cfg) {
  int r = require_loaded(b);
  if (r) return r;
  if (!cfg || cfg->num_fragments < 1) return fail(b, PCPB_E_INVALID, "bad streaming configuration");
  if (!b->in_round) return fail(b, PCPB_E_STATE, "pcpb_stream_begin must follow pcpb_worker_begin_round");
  if (!b->velocity_init) return fail(b, PCPB_E_STATE, "outer step not attached (pcpb_outer_attach_*)");
  DeviceGuard g(b->device);
  const size_t P = (size_t)b->cfg.total_params;
  if (!b->snapshot) WS(b, b->snapshot, P * 4);
  CK(b, cudaMemcpyAsync(b->snapshot, b->ws.theta, P * 4, cudaMemcpyDeviceToDevice, b->stream));
  b->stream_fragments = cfg->num_fragments; b->stream_alpha = cfg->alpha;
  b->stream_lr = cfg->learning_rate; b->stream_mu = cfg->momentum;
  return PCPB_OK;
}

int pcpb_stream_send(pcpb_backend* b, int fragment) {
  int r = stream_check(b, fragment);
  if (r) return r;
  DeviceGuard g(b->device);
  Workspace& w = b->ws;
  const auto& ps = b->cfg.params;
  for (size_t i = (size_t)fragment; i < ps.size(); i += (size_t)b->stream_fragments) {
    const size_t off = (size_t)ps[i].offset, n = (size_t)ps[i].numel;
    KL(b, 1, launch_stream_delta(b->stream, b->snapshot + off, w.theta + off, w.delta + off, n));
  }
  CK(b, cudaStreamSynchronize(b->stream));
  return PCPB_OK;
}

// The fragment's outer step of this rank's shard, enqueued on `st` between the two events.
static int stream_outer_enqueue(pcpb_backend* b, int fragment, cudaStream_t st, cudaEvent_t e0, cudaEvent_t e1) {
  const long long P = b->cfg.total_params, S = b->shard_len;
  const long long s_lo = (long long)b->rank * S < P ? (long long)b->rank * S : P;
  const long long s_hi = s_lo + S < P ? s_lo + S : P;
  for (int w = 0; w < b->world; ++w)
    if (!b->peer_delta[w]) return fail(b, PCPB_E_STATE, "a peer is not attached");
  const auto& ps = b->cfg.params;
  CK(b, cudaEventRecord(e0, st));
  for (size_t i = (size_t)fragment; i < ps.size(); i += (size_t)b->stream_fragments) {
    // the part of tensor i that lies in this rank's shard
    const long long lo = ps[i].offset > s_lo ? ps[i].offset : s_lo;
    const long long t_hi = ps[i].offset + ps[i].numel;
    const long long hi = t_hi < s_hi ? t_hi : s_hi;
    if (hi <= lo) continue;
    OuterArgs a{};
    for (int w = 0; w < b->world; ++w) a.deltas[a.ncontrib++] = b->peer_delta[w] + lo;
    a.vel = b->velocity + (lo - s_lo); a.master = b->ws.theta0 + lo;
    for (int w = 0; w < b->world; ++w)
      if (w != b->rank) a.outs[a.nouts++] = b->peer_theta0[w] + lo;
    a.n = hi - lo; a.lr = b->stream_lr; a.mu = b->stream_mu; a.trunc = 0; a.keep_nonfinite = 1;
    KL(b, 1, launch_nesterov_shard(st, a));
  }
  CK(b, cudaEventRecord(e1, st));
  return PCPB_OK;
}

static bool frag_is_pending(const pcpb_backend* b, int fragment) {
  return (size_t)fragment < b->frag_pending.size() && b->frag_pending[fragment];
}

int pcpb_stream_outer(pcpb_backend* b, int fragment, double* device_ms) {
  int r = stream_check(b, fragment);
  if (r) return r;
  if (frag_is_pending(b, fragment)) return fail(b, PCPB_E_STATE, "an outer step of this fragment is still pending (pcpb_stream_outer_wait)");
  DeviceGuard g(b->device);
  if ((r = stream_outer_enqueue(b, fragment, b->stream, b->ev0, b->ev1))) return r;
  CK(b, cudaStreamSynchronize(b->stream));
  if (device_ms) { float ms = 0.f; CK(b, cudaEventElapsedTime(&ms, b->ev0, b->ev1)); *device_ms = ms; }
  return PCPB_OK;
}

int pcpb_stream_outer_start(pcpb_backend* b, int fragment) {
  int r = stream_check(b, fragment);
  if (r) return r;
  if (frag_is_pending(b, fragment)) return fail(b, PCPB_E_STATE, "an outer step of this fragment is still pending (pcpb_stream_outer_wait)");
  DeviceGuard g(b->device);
  if (!b->side_stream) CK(b, cudaStreamCreateWithFlags(&b->side_stream, cudaStreamNonBlocking));
  if (b->frag_ev.size() < 2 * (size_t)b->stream_fragments) {
    const size_t old = b->frag_ev.size();
    b->frag_ev.resize(2 * (size_t)b->stream_fragments, nullptr);
    for (size_t i = old; i < b->frag_ev.size(); ++i) CK(b, cudaEventCreate(&b->frag_ev[i]));
  }
  if (b->frag_pending.size() < (size_t)b->stream_fragments) b->frag_pending.resize((size_t)b->stream_fragments, 0);
  if ((r = stream_outer_enqueue(b, fragment, b->side_stream, b->frag_ev[2 * fragment], b->frag_ev[2 * fragment + 1]))) return r;
  b->frag_pending[fragment] = 1;
  return PCPB_OK;
}

int pcpb_stream_outer_wait(pcpb_backend* b, int fragment, double* device_ms) {
  int r = stream_check(b, fragment);
  if (r) return r;
  if (!frag_is_pending(b, fragment)) return fail(b, PCPB_E_STATE, "no outer step of this fragment was started (pcpb_stream_outer_start)");
  DeviceGuard g(b->device);
  CK(b, cudaEventSynchronize(b->frag_ev[2 * fragment + 1]));
  b->frag_pending[fragment] = 0;
  if (device_ms) { float ms = 0.f; CK(b, cudaEventElapsedTime(&ms, b->frag_ev[2 * fragment], b->frag_ev[2 * fragment + 1])); *device_ms = ms; }
  return PCPB_OK;
}

int pcpb_stream_merge(pcpb_backend* b, int fragment) {
  int r = stream_check(b, fragment);
  if (r) return r;
  if (frag_is_pending(b, fragment)) return fail(b, PCPB_E_STATE, "the fragment's outer step is still pending (pcpb_stream_outer_wait)");
  DeviceGuard g(b->device);
  Workspace& w = b->ws;
  const ModelConfig& c = b->cfg;
  for (size_t i = (size_t)fragment; i < c.params.size(); i += (size_t)b->stream_fragments) {
    const size_t off = (size_t)c.params[i].offset, n = (size_t)c.params[i].numel;
    KL(b, 1, launch_stream_merge(b->stream, w.theta + off, w.theta0 + off, b->snapshot + off, b->stream_alpha, n));
    if (c.dtype != DT_F32)
      KL(b, 1, launch_convert_f32(b->stream, c.dtype, w.theta + off, (char*)w.shadow + off * dtype_size(c.dtype), n));
  }
  return PCPB_OK;
}

}  // extern "C"
