// Host-side data functions of the training path: the pseudo-random generator behind random-window batching and
// master-parameter initialisation, the character tokenizer, and the master initialiser itself.
//
// The reference draws from Zig 0.13's std.Random.DefaultPrng (call sites src/data/loader.zig:257,289,347,379,439,469
// and src/algorithms/diloco.zig:519,543), which is not part of the reference tree.  What is implemented here is the
// published construction that generator is documented to be: xoshiro256++ (Blackman & Vigna) with its four state
// words filled by SplitMix64 from the 64-bit seed, and Lemire's nearly-divisionless method for a bounded integer.
// The standard normal is drawn with the Box-Muller transform in double precision, not with the reference's ziggurat
// tables.  Sequences are therefore UNPINNED against the Zig standard library: window starts and initial parameters
// follow the same distributions, not the same bits, as a reference run with the same seed.  FIFO batching
// (pcpb_fifo_get_batch) is the bit-exact path.
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../../include/pcp_b200.h"

namespace {

inline uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

inline uint64_t splitmix64(uint64_t* s) {
  uint64_t z = (*s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

}  // namespace

extern "C" {

void pcpb_prng_seed(pcpb_prng* g, uint64_t seed) {
  if (!g) return;
  uint64_t s = seed;
  for (int i = 0; i < 4; ++i) g->s[i] = splitmix64(&s);
}

uint64_t pcpb_prng_next(pcpb_prng* g) {
  uint64_t* s = g->s;
  const uint64_t result = rotl64(s[0] + s[3], 23) + s[0];
  const uint64_t t = s[1] << 17;
  s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3];
  s[2] ^= t;
  s[3] = rotl64(s[3], 45);
  return result;
}

// Uniform integer in [0, at_most]: multiply-shift with rejection of the biased low products (Lemire 2019).
uint64_t pcpb_prng_uint_at_most(pcpb_prng* g, uint64_t at_most) {
  if (at_most == UINT64_MAX) return pcpb_prng_next(g);
  const uint64_t range = at_most + 1;
  uint64_t x = pcpb_prng_next(g);
  __uint128_t m = (__uint128_t)x * range;
  uint64_t low = (uint64_t)m;
  if (low < range) {
    const uint64_t threshold = (0 - range) % range;
    while (low < threshold) {
      x = pcpb_prng_next(g);
      m = (__uint128_t)x * range;
      low = (uint64_t)m;
    }
  }
  return (uint64_t)(m >> 64);
}

// One window start per row, uniform in [0, n_tokens - block - 1]; a chunk of at most block + 1 tokens is refused
// (src/data/loader.zig:289-291, 379-381, 469-471).
int pcpb_random_window_starts(pcpb_prng* g, size_t n_tokens, size_t batch, size_t block, uint64_t* starts_out) {
  if (!g || (!starts_out && batch)) return PCPB_E_INVALID;
  for (size_t i = 0; i < batch; ++i) {
    if (n_tokens <= block + 1) return PCPB_E_CHUNK_TOO_SMALL;
    starts_out[i] = pcpb_prng_uint_at_most(g, (uint64_t)(n_tokens - block - 1));
  }
  return PCPB_OK;
}

// CharTokenizer.initFromFile (src/data/loader.zig:21-61): the distinct bytes of the text in ascending order; the
// first 65 of them are the vocabulary, token = rank.
int pcpb_char_tokenizer_build(const uint8_t* text, size_t n, uint8_t* vocab_chars_out, int* vocab_size_out,
                              int* ignored_chars_out) {
  if ((!text && n) || !vocab_chars_out || !vocab_size_out) return PCPB_E_INVALID;
  bool seen[256] = {};
  for (size_t i = 0; i < n; ++i) seen[text[i]] = true;
  int count = 0, ignored = 0;
  for (int c = 0; c < 256; ++c) {
    if (!seen[c]) continue;
    if (count < PCPB_CHAR_VOCAB_MAX) vocab_chars_out[count++] = (uint8_t)c;
    else ++ignored;
  }
  *vocab_size_out = count;
  if (ignored_chars_out) *ignored_chars_out = ignored;
  return PCPB_OK;
}

// CharTokenizer.encode (src/data/loader.zig:68-78): a byte outside the vocabulary becomes token 0.
int pcpb_char_encode(const uint8_t* vocab_chars, int vocab_size, const uint8_t* text, size_t n, uint32_t* tokens_out) {
  if (!vocab_chars || vocab_size < 0 || vocab_size > PCPB_CHAR_VOCAB_MAX || (!text && n) || (!tokens_out && n))
    return PCPB_E_INVALID;
  uint32_t map[256];
  memset(map, 0, sizeof map);
  for (int i = 0; i < vocab_size; ++i) map[vocab_chars[i]] = (uint32_t)i;
  for (size_t i = 0; i < n; ++i) tokens_out[i] = map[text[i]];
  return PCPB_OK;
}

// CharTokenizer.decode (src/data/loader.zig:80-86): a token outside the vocabulary is an error (UnknownToken).
int pcpb_char_decode(const uint8_t* vocab_chars, int vocab_size, const uint32_t* tokens, size_t n, uint8_t* text_out) {
  if (!vocab_chars || vocab_size < 0 || vocab_size > PCPB_CHAR_VOCAB_MAX || (!tokens && n) || (!text_out && n))
    return PCPB_E_INVALID;
  for (size_t i = 0; i < n; ++i) {
    if (tokens[i] >= (uint32_t)vocab_size) return PCPB_E_INVALID;
    text_out[i] = vocab_chars[tokens[i]];
  }
  return PCPB_OK;
}

// DiLoCo.initializeMasterParameters (src/algorithms/diloco.zig:513-586): one generator over all tensors in argument
// order, every element 0.02 * N(0,1) computed in f32; bf16 keeps the upper 16 bits (truncation), f32 the value.
int pcpb_init_master_elems(uint64_t seed, int dtype, size_t n, void* out, size_t out_bytes) {
  if (dtype != PCPB_F32 && dtype != PCPB_BF16) return PCPB_E_INVALID;
  if ((!out && n) || out_bytes != n * (dtype == PCPB_F32 ? 4u : 2u)) return PCPB_E_INVALID;
  pcpb_prng g;
  pcpb_prng_seed(&g, seed);
  const float scale = 0.02f;
  const double two_pi = 6.283185307179586476925286766559;
  const double inv53 = 1.0 / 9007199254740992.0;      // 2^-53
  size_t i = 0;
  while (i < n) {
    const double u1 = (double)((pcpb_prng_next(&g) >> 11) + 1) * inv53;     // (0, 1]
    const double u2 = (double)(pcpb_prng_next(&g) >> 11) * inv53;           // [0, 1)
    const double r = sqrt(-2.0 * log(u1));
    const double z[2] = {r * cos(two_pi * u2), r * sin(two_pi * u2)};
    for (int k = 0; k < 2 && i < n; ++k, ++i) {
      const float v = (float)z[k] * scale;
      if (dtype == PCPB_F32) ((float*)out)[i] = v;
      else { uint32_t u; memcpy(&u, &v, 4); ((uint16_t*)out)[i] = (uint16_t)(u >> 16); }
    }
  }
  return PCPB_OK;
}

}  // extern "C"
