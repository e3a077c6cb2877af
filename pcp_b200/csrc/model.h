// Artefact recogniser: recovers the model configuration of a nanochat-family forward graph from its
// StableHLO text (the @main signature, the RoPE table resources and the soft-cap constant).
#pragma once
#include <stdint.h>
#include <string>
#include <vector>

namespace pcpb {

struct TensorInfo {
  std::vector<int64_t> shape;
  int64_t numel = 0;
  int64_t offset = 0;      // element offset in the flat parameter buffer (argument order)
};

// FAMILY_GRAPH: not one of the two recognised architectures; run op by op by the general front end (graph.h).  Only the
// fields dtype, B, T, params, total_params (and V when the first parameter is a [V, d] table) are meaningful then.
enum { FAMILY_NANOCHAT = 0, FAMILY_NANOGPT = 1, FAMILY_GRAPH = 2 };
enum { ACT_NATIVE = 0, ACT_GELU_TANH = 1 };     // native: ReLU^2 (nanochat) / ReLU (nanoGPT)

struct ModelConfig {
  int family = FAMILY_NANOCHAT;
  int dtype = 0;           // DT_F32 | DT_BF16 (model dtype)
  int64_t V = 0, d = 0, L = 0, H = 0, Hkv = 0, hd = 0, F = 0, B = 0, T = 0;
  int activation = ACT_NATIVE;
  float softcap = 15.f;
  long long ignore_index = -1;
  // nanochat: wte, per layer q k v proj fc proj2, lm_head
  // nanoGPT:  wte, wpe, per layer ln1.w ln1.b c_attn c_proj ln2.w ln2.b c_fc mlp.c_proj, ln_f.w ln_f.b lm_head.w lm_head.b
  std::vector<TensorInfo> params;
  int64_t total_params = 0;
  std::vector<uint16_t> rope_cos, rope_sin;   // [T, hd/2] bf16 bit patterns
  int64_t dkv() const { return Hkv * hd; }
  int64_t M() const { return B * T; }
};

// Returns an empty string on success, else the reason the text was not recognised.
std::string parse_artifact(const char* text, size_t n, ModelConfig* out);

}  // namespace pcpb
