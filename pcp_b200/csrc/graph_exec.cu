// Executor of the general StableHLO front end: planning (host) and the per-op kernels.  See graph_exec.h / graph.h.
//
// Element semantics follow the StableHLO specification as the reference's runtime implements it for these graphs:
// bf16 ops compute in f32 and round once to bf16, f64 stays f64, integer division truncates, reductions of f32 / bf16
// accumulate in f32.  Every kernel is a grid-stride loop over the elements of its result; index arithmetic for the
// strided ops (transpose, broadcast, slice, concatenate, reduce) is a mixed-radix walk over at most 8 dimensions.
#include "graph_exec.h"

#include <math.h>
#include <string.h>

#include <map>
#include <type_traits>

#include "common.cuh"

namespace pcpb {

namespace {

constexpr int MAX_RANK = 8;
constexpr int TPB = 256;

// ------------------------------------------------------------------------------------------------
// element types
// ------------------------------------------------------------------------------------------------
template <typename T> struct TT;
template <> struct TT<float> { typedef float C; static constexpr bool is_fp = true; };
template <> struct TT<bf16> { typedef float C; static constexpr bool is_fp = true; };
template <> struct TT<double> { typedef double C; static constexpr bool is_fp = true; };
template <> struct TT<long long> { typedef long long C; static constexpr bool is_fp = false; };
template <> struct TT<int> { typedef long long C; static constexpr bool is_fp = false; };
template <> struct TT<uint8_t> { typedef long long C; static constexpr bool is_fp = false; };      // i1

template <typename T> __device__ __forceinline__ typename TT<T>::C ld(const T* p, long long i) { return (typename TT<T>::C)p[i]; }
template <> __device__ __forceinline__ float ld<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }

template <typename T, typename C> __device__ __forceinline__ T narrow(C c) {
  if constexpr (std::is_same<T, bf16>::value) return __float2bfloat16_rn((float)c);
  else if constexpr (std::is_same<T, uint8_t>::value) return (uint8_t)(c != 0);
  else return (T)c;
}

// ------------------------------------------------------------------------------------------------
// kernels
// ------------------------------------------------------------------------------------------------
#define GRID_STRIDE(i, n) for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (n); i += (long long)gridDim.x * blockDim.x)

template <typename T> __global__ void k_fill(T* out, long long n, double f, long long iv) {
  T v;
  if constexpr (TT<T>::is_fp) {
    if constexpr (std::is_same<T, double>::value) v = f; else v = narrow<T, float>((float)f);
  } else v = narrow<T, long long>(iv);
  GRID_STRIDE(i, n) out[i] = v;
}

template <typename T> __global__ void k_iota(T* out, long long n, long long inner, long long extent) {
  GRID_STRIDE(i, n) out[i] = narrow<T, long long>((i / inner) % extent);
}

template <typename C> __device__ __forceinline__ C unary_fp(int sub, C x) {
  switch (sub) {
    case U_RSQRT: return C(1) / sqrt(x);
    case U_SQRT: return sqrt(x);
    case U_EXP: return exp(x);
    case U_LOG: return log(x);
    case U_TANH: return tanh(x);
    case U_LOGISTIC: return C(1) / (C(1) + exp(-x));
    case U_NEG: return -x;
    case U_CEIL: return ceil(x);
    case U_FLOOR: return floor(x);
    case U_SIN: return sin(x);
    case U_COS: return cos(x);
    default: return fabs(x);
  }
}

// An adjoint-edge guard (G_GUARD_CLAMP) that is the only reader of an element-wise result runs inside the producing
// kernel: the result is rounded to its element type as the producing op does, then guarded and clamped, then stored.
struct Post { int on, clamp; float lo, hi; };

template <typename T, typename C> __device__ __forceinline__ T finish(C r, const Post& p) {
  T t = narrow<T, C>(r);
  if constexpr (TT<T>::is_fp) {
    if (p.on) {
      C g = ld(&t, 0);
      if (!((g - g) == C(0))) g = C(0);
      if (p.clamp) g = (C)fminf(fmaxf((float)g, p.lo), p.hi);
      t = narrow<T, C>(g);
    }
  }
  return t;
}

template <typename T> __global__ void k_unary(int sub, const T* in, T* out, long long n, Post post) {
  typedef typename TT<T>::C C;
  GRID_STRIDE(i, n) {
    const C x = ld(in, i);
    if constexpr (TT<T>::is_fp) out[i] = finish<T, C>(unary_fp<C>(sub, x), post);
    else out[i] = narrow<T, C>(sub == U_NEG ? -x : (sub == U_ABS ? (x < 0 ? -x : x) : x));
  }
}

template <typename C> __device__ __forceinline__ C pow_fp(C x, C e) {
  // the cases the exporters produce, exact like the CPU library's fast paths; pow() otherwise
  if (e == C(2)) return x * x;
  if (e == C(3)) return (x * x) * x;
  if (e == C(1)) return x;
  if (e == C(0.5)) return sqrt(x);
  return pow(x, e);
}

// How a binary op reads an operand: the tensor itself, a broadcast that was not materialised (one value per run of
// `inner` elements, one value per position inside such a run, or one value for all), or a splat constant.
enum : int { O_DIRECT = 0, O_PER_RUN, O_IN_RUN, O_SCALAR, O_IMM };
struct Opnd { int mode; unsigned inner; double imm; long long iimm; };

template <typename T> __device__ __forceinline__ typename TT<T>::C ldo(const T* p, long long i, const Opnd& o) {
  typedef typename TT<T>::C C;
  switch (o.mode) {
    case O_DIRECT: return ld(p, i);
    case O_PER_RUN: return ld(p, (long long)((unsigned)i / o.inner));
    case O_IN_RUN: return ld(p, (long long)((unsigned)i % o.inner));
    case O_SCALAR: return ld(p, 0);
    default:
      if constexpr (TT<T>::is_fp) return (C)o.imm; else return (C)o.iimm;
  }
}

template <typename T> __global__ void k_binary(int sub, const T* a, const T* b, T* out, long long n, Post post, Opnd oa, Opnd ob) {
  typedef typename TT<T>::C C;
  GRID_STRIDE(i, n) {
    const C x = ldo(a, i, oa), y = ldo(b, i, ob);
    C r;
    if constexpr (TT<T>::is_fp) {
      switch (sub) {
        case B_ADD: r = x + y; break;
        case B_SUB: r = x - y; break;
        case B_MUL: r = x * y; break;
        case B_DIV: r = x / y; break;
        case B_POW: r = pow_fp<C>(x, y); break;
        case B_MAX: r = (x != x || y != y) ? (x + y) : (x > y ? x : y); break;       // NaN propagates
        default: r = (x != x || y != y) ? (x + y) : (x < y ? x : y); break;
      }
    } else {
      switch (sub) {
        case B_ADD: r = x + y; break;
        case B_SUB: r = x - y; break;
        case B_MUL: r = x * y; break;
        case B_DIV: r = y == 0 ? 0 : x / y; break;
        case B_MAX: r = x > y ? x : y; break;
        case B_MIN: r = x < y ? x : y; break;
        case B_AND: r = x & y; break;
        case B_OR: r = x | y; break;
        default: r = 0; break;
      }
    }
    out[i] = finish<T, C>(r, post);
  }
}

template <typename T> __global__ void k_compare(int dir, const T* a, const T* b, uint8_t* out, long long n, Opnd oa, Opnd ob) {
  typedef typename TT<T>::C C;
  GRID_STRIDE(i, n) {
    const C x = ldo(a, i, oa), y = ldo(b, i, ob);
    bool r;
    switch (dir) {
      case C_EQ: r = x == y; break;
      case C_NE: r = x != y; break;
      case C_GE: r = x >= y; break;
      case C_GT: r = x > y; break;
      case C_LE: r = x <= y; break;
      default: r = x < y; break;
    }
    out[i] = r;
  }
}

// a_imm / b_imm: that operand is a splat constant, given as the bits of one element
template <typename U> __global__ void k_select(const uint8_t* pred, const U* a, const U* b, U* out, long long n, int a_imm, int b_imm, U av, U bv) {
  GRID_STRIDE(i, n) out[i] = pred[i] ? (a_imm ? av : a[i]) : (b_imm ? bv : b[i]);
}

template <typename TI, typename TO> __global__ void k_convert(const TI* in, TO* out, long long n) {
  typedef typename TT<TI>::C CI;
  GRID_STRIDE(i, n) {
    const CI x = ld(in, i);
    if constexpr (TT<TI>::is_fp && !TT<TO>::is_fp) {
      if constexpr (std::is_same<TO, uint8_t>::value) out[i] = (uint8_t)(x != CI(0));
      else out[i] = (TO)(long long)trunc(x);
    } else if constexpr (std::is_same<TO, bf16>::value) out[i] = __float2bfloat16_rn((float)x);     // via f32, like the CPU library
    else out[i] = narrow<TO, CI>(x);
  }
}

// adjoint edge (src/autodiff/engine.zig:622-682): (g - g) == 0 ? g : 0, then clamp in f32 and back to the element type
template <typename T> __global__ void k_guard_clamp(const T* in, T* out, long long n, int clamp, float lo, float hi) {
  typedef typename TT<T>::C C;
  GRID_STRIDE(i, n) {
    C g = ld(in, i);
    if (!((g - g) == C(0))) g = C(0);
    if (clamp) g = (C)fminf(fmaxf((float)g, lo), hi);
    out[i] = narrow<T, C>(g);
  }
}

struct NdDesc {            // walk over `rank` dimensions of extents dim[], the other side's strides in stride[]
  int rank;
  long long dim[MAX_RANK], stride[MAX_RANK], offset;
};

// out[i] = in[offset + sum coord_k * stride_k]: transpose, broadcast_in_dim, slice
template <typename U> __global__ void k_gather_nd(const U* in, U* out, long long n, NdDesc d) {
  GRID_STRIDE(i, n) {
    long long rem = i, src = d.offset;
    for (int k = d.rank - 1; k >= 0; --k) { src += (rem % d.dim[k]) * d.stride[k]; rem /= d.dim[k]; }
    out[i] = in[src];
  }
}

// The same walk with 32-bit arithmetic, one warp per run of the innermost dimension: the mixed-radix decomposition is
// done once per run instead of once per element (the divisions, not the loads, bound the element-wise form).
template <typename U> __global__ void k_gather_rows_nd(const U* in, U* out, unsigned n_rows, unsigned inner, NdDesc d) {
  const unsigned lane = threadIdx.x & 31, warps = (gridDim.x * blockDim.x) >> 5;
  const long long s_in = d.stride[d.rank - 1];
  for (unsigned row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < n_rows; row += warps) {
    unsigned rem = row;
    long long src = d.offset;
    for (int k = d.rank - 2; k >= 0; --k) { const unsigned dk = (unsigned)d.dim[k]; src += (long long)(rem % dk) * d.stride[k]; rem /= dk; }
    U* o = out + (size_t)row * inner;
    for (unsigned c = lane; c < inner; c += 32) o[c] = in[src + (long long)c * s_in];
  }
}

// out[offset + sum coord_k * stride_k] = in[i]: concatenate (one launch per operand), pad
template <typename U> __global__ void k_scatter_nd(const U* in, U* out, long long n, NdDesc d) {
  GRID_STRIDE(i, n) {
    long long rem = i, dst = d.offset;
    for (int k = d.rank - 1; k >= 0; --k) { dst += (rem % d.dim[k]) * d.stride[k]; rem /= d.dim[k]; }
    out[dst] = in[i];
  }
}

struct RedDesc {
  int krank, rrank;
  long long kdim[MAX_RANK], kstr[MAX_RANK], rdim[MAX_RANK], rstr[MAX_RANK];
  long long n_out, n_red;
};

// GROUP threads per result element (1 or 32); f32 / bf16 accumulate in f32, f64 in f64, integers in i64; the result is
// rounded to the element type and then combined with the init value, as "reduce then op with init" evaluates
template <typename T, int KIND, int GROUP> __global__ void k_reduce(const T* in, const T* init, T* out, RedDesc d) {
  typedef typename TT<T>::C C;
  const long long gid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long o = gid / GROUP;
  const int lane = (int)(gid % GROUP);
  if (o >= d.n_out) return;                                  // GROUP == 32: a whole warp leaves together
  long long base = 0, rem = o;
  for (int k = d.krank - 1; k >= 0; --k) { base += (rem % d.kdim[k]) * d.kstr[k]; rem /= d.kdim[k]; }
  C acc;
  if constexpr (KIND == R_ADD) acc = C(0);
  else if constexpr (TT<T>::is_fp) acc = (C)(-INFINITY);
  else acc = (C)(-0x7FFFFFFFFFFFFFFFLL - 1);
  for (long long r = lane; r < d.n_red; r += GROUP) {
    long long off = base, q = r;
    for (int k = d.rrank - 1; k >= 0; --k) { off += (q % d.rdim[k]) * d.rstr[k]; q /= d.rdim[k]; }
    const C x = ld(in, off);
    if constexpr (KIND == R_ADD) acc += x; else acc = (x > acc || x != x) ? x : acc;
  }
  if constexpr (GROUP == 32) {
    for (int s = 16; s > 0; s >>= 1) {
      const C y = __shfl_xor_sync(0xffffffffu, acc, s);
      if constexpr (KIND == R_ADD) acc += y; else acc = (y > acc || y != y) ? y : acc;
    }
  }
  if (lane == 0) {
    const T rounded = narrow<T, C>(acc);
    const C a = ld(&rounded, 0), b = ld(init, 0);
    out[o] = narrow<T, C>(KIND == R_ADD ? a + b : ((b > a || b != b) ? b : a));
  }
}

// Reduction over the leading dimensions of a row-major tensor seen as [n_red][n_out] (bias / LayerNorm parameter /
// position-table gradients): a block owns 32 columns and one chunk of rows, 8 row lanes per column, so that every load
// instruction of a warp reads 128 contiguous bytes; per-chunk partials go to scratch [chunks][n_out] and a second kernel
// adds them in chunk order (no atomics: the same bits every run).
template <typename T, int KIND> __global__ void __launch_bounds__(256) k_reduce_cols(const T* in, typename TT<T>::C* partial,
                                                                                     long long n_red, long long n_out, long long rows_per_chunk) {
  typedef typename TT<T>::C C;
  __shared__ C sm[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long col = blockIdx.x * 32LL + tx;
  const long long r0 = blockIdx.y * rows_per_chunk, r1 = (r0 + rows_per_chunk < n_red) ? r0 + rows_per_chunk : n_red;
  C acc;
  if constexpr (KIND == R_ADD) acc = C(0);
  else if constexpr (TT<T>::is_fp) acc = (C)(-INFINITY);
  else acc = (C)(-0x7FFFFFFFFFFFFFFFLL - 1);
  if (col < n_out)
    for (long long r = r0 + ty; r < r1; r += 8) {
      const C x = ld(in, r * n_out + col);
      if constexpr (KIND == R_ADD) acc += x; else acc = (x > acc || x != x) ? x : acc;
    }
  sm[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && col < n_out) {
    for (int k = 1; k < 8; ++k) {
      const C y = sm[k][tx];
      if constexpr (KIND == R_ADD) acc += y; else acc = (y > acc || y != y) ? y : acc;
    }
    partial[blockIdx.y * n_out + col] = acc;
  }
}

template <typename T, int KIND> __global__ void k_reduce_cols_finish(const typename TT<T>::C* partial, const T* init, T* out, int chunks, long long n_out) {
  typedef typename TT<T>::C C;
  GRID_STRIDE(o, n_out) {
    C acc = partial[o];
    for (int k = 1; k < chunks; ++k) {
      const C y = partial[(long long)k * n_out + o];
      if constexpr (KIND == R_ADD) acc += y; else acc = (y > acc || y != y) ? y : acc;
    }
    const T rounded = narrow<T, C>(acc);
    const C a = ld(&rounded, 0), b = ld(init, 0);
    out[o] = narrow<T, C>(KIND == R_ADD ? a + b : ((b > a || b != b) ? b : a));
  }
}

struct DotDesc { long long ab, am, ak, bb, bk, bn; int M, N, K; };

// C[b, m, n] = sum_k A[b, m, k] B[b, k, n] over strided operands; 64 x 64 tile per block, 4 x 4 per thread, k in order
template <typename T> __global__ void __launch_bounds__(256) k_dot(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ Cm, DotDesc s) {
  typedef typename TT<T>::C C;
  __shared__ C As[16][65], Bs[16][65];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const long long bz = blockIdx.z;
  const T* Ab = A + bz * s.ab;
  const T* Bb = B + bz * s.bb;
  C acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = C(0);
  for (int k0 = 0; k0 < s.K; k0 += 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      int mm, kk;
      if (s.ak == 1) { kk = e % 16; mm = e / 16; } else { mm = e % 64; kk = e / 64; }
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < s.M && gk < s.K) ? ld(Ab, gm * s.am + gk * s.ak) : C(0);
      int nn, k2;
      if (s.bn == 1) { nn = e % 64; k2 = e / 64; } else { k2 = e % 16; nn = e / 16; }
      const int gn = n0 + nn, gk2 = k0 + k2;
      Bs[k2][nn] = (gn < s.N && gk2 < s.K) ? ld(Bb, gk2 * s.bk + gn * s.bn) : C(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      C a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
  T* Cb = Cm + bz * (long long)s.M * s.N;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= s.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < s.N) Cb[(long long)gm * s.N + gn] = narrow<T, C>(acc[i][j]);
    }
  }
}

template <typename U> __global__ void k_gather_rows(const U* x, const long long* idx, U* out, long long n, long long rowlen, long long R) {
  GRID_STRIDE(i, n) {
    long long r = idx[i / rowlen];
    r = r < 0 ? 0 : (r > R - 1 ? R - 1 : r);
    out[i] = x[r * rowlen + i % rowlen];
  }
}

template <typename U> __global__ void k_gather2(const U* x, const long long* idx, U* out, long long n, long long R, long long Cn) {
  GRID_STRIDE(i, n) {
    long long r = idx[2 * i], c = idx[2 * i + 1];
    r = r < 0 ? 0 : (r > R - 1 ? R - 1 : r);
    c = c < 0 ? 0 : (c > Cn - 1 ? Cn - 1 : c);
    out[i] = x[r * Cn + c];
  }
}

template <typename T> __device__ __forceinline__ void atomic_add_t(T* p, T v) { atomicAdd(p, v); }

// scatter-add of the gradient rows (the result was zeroed before): sums arrive in any order
template <typename T> __global__ void k_scatter_rows(const T* g, const long long* idx, T* out, long long n, long long rowlen, long long R) {
  GRID_STRIDE(i, n) {
    long long r = idx[i / rowlen];
    r = r < 0 ? 0 : (r > R - 1 ? R - 1 : r);
    atomic_add_t(out + r * rowlen + i % rowlen, g[i]);
  }
}

template <typename T> __global__ void k_scatter2(const T* g, const long long* idx, T* out, long long n, long long R, long long Cn) {
  GRID_STRIDE(i, n) {
    const long long r = idx[2 * i], c = idx[2 * i + 1];
    if (r < 0 || r >= R || c < 0 || c >= Cn) continue;
    atomic_add_t(out + r * Cn + c, g[i]);
  }
}

// ------------------------------------------------------------------------------------------------
// launch helpers
// ------------------------------------------------------------------------------------------------
int blocks_for(long long n) {
  long long b = (n + TPB - 1) / TPB;
  if (b < 1) b = 1;
  if (b > 148 * 32) b = 148 * 32;
  return (int)b;
}

// merges neighbouring dimensions of a gather walk that the source also holds like one dimension, drops extents of 1
void collapse_walk(NdDesc* d) {
  NdDesc r;
  r.rank = 0; r.offset = d->offset;
  for (int k = 0; k < d->rank; ++k) {
    if (d->dim[k] == 1) continue;
    if (r.rank > 0 && r.stride[r.rank - 1] == d->stride[k] * d->dim[k]) { r.dim[r.rank - 1] *= d->dim[k]; r.stride[r.rank - 1] = d->stride[k]; continue; }
    r.dim[r.rank] = d->dim[k]; r.stride[r.rank] = d->stride[k]; r.rank += 1;
  }
  if (r.rank == 0) { r.rank = 1; r.dim[0] = 1; r.stride[0] = 0; }
  *d = r;
}

std::vector<long long> row_major_strides(const std::vector<int64_t>& shape) {
  std::vector<long long> s(shape.size(), 1);
  for (int i = (int)shape.size() - 2; i >= 0; --i) s[i] = s[i + 1] * shape[i + 1];
  return s;
}

#define BY_SIZE(es, ...)                                   \
  switch (es) {                                             \
    case 1: { typedef uint8_t U; __VA_ARGS__; break; }             \
    case 2: { typedef uint16_t U; __VA_ARGS__; break; }            \
    case 4: { typedef uint32_t U; __VA_ARGS__; break; }            \
    default: { typedef unsigned long long U; __VA_ARGS__; break; } \
  }

#define BY_TYPE(dt, ...)                                   \
  switch (dt) {                                             \
    case DT_F32: { typedef float T; __VA_ARGS__; break; }          \
    case DT_BF16: { typedef bf16 T; __VA_ARGS__; break; }          \
    case DT_F64: { typedef double T; __VA_ARGS__; break; }         \
    case DT_I64: { typedef long long T; __VA_ARGS__; break; }      \
    case DT_I32: { typedef int T; __VA_ARGS__; break; }            \
    default: { typedef uint8_t T; __VA_ARGS__; break; }            \
  }

#define BY_FLOAT(dt, ...)                                  \
  switch (dt) {                                             \
    case DT_F32: { typedef float T; __VA_ARGS__; break; }          \
    case DT_BF16: { typedef bf16 T; __VA_ARGS__; break; }          \
    default: { typedef double T; __VA_ARGS__; break; }             \
  }

bool is_fp(int dt) { return dt == DT_F32 || dt == DT_BF16 || dt == DT_F64; }
bool known(int dt) { return is_fp(dt) || dt == DT_I64 || dt == DT_I32 || dt == DT_BOOL; }

template <typename TI> void convert_from(cudaStream_t st, const void* in, void* out, int dto, long long n) {
  const int nb = blocks_for(n);
  switch (dto) {
    case DT_F32: k_convert<TI, float><<<nb, TPB, 0, st>>>((const TI*)in, (float*)out, n); break;
    case DT_BF16: k_convert<TI, bf16><<<nb, TPB, 0, st>>>((const TI*)in, (bf16*)out, n); break;
    case DT_F64: k_convert<TI, double><<<nb, TPB, 0, st>>>((const TI*)in, (double*)out, n); break;
    case DT_I64: k_convert<TI, long long><<<nb, TPB, 0, st>>>((const TI*)in, (long long*)out, n); break;
    case DT_I32: k_convert<TI, int><<<nb, TPB, 0, st>>>((const TI*)in, (int*)out, n); break;
    default: k_convert<TI, uint8_t><<<nb, TPB, 0, st>>>((const TI*)in, (uint8_t*)out, n); break;
  }
}

void convert(cudaStream_t st, const void* in, int dti, void* out, int dto, long long n) {
  BY_TYPE(dti, convert_from<T>(st, in, out, dto, n));
}

// a group of dimensions (in the given order) of a row-major tensor as ONE strided dimension; false if they do not
// lie in memory like one
bool collapse(const std::vector<int64_t>& shape, const std::vector<long long>& strides, const std::vector<int64_t>& dims,
              long long* size, long long* stride) {
  long long n = 1, st = 1;
  bool have = false;
  for (int i = (int)dims.size() - 1; i >= 0; --i) {
    const int64_t d = dims[i];
    if (shape[d] == 1) continue;
    if (!have) { st = strides[d]; n = shape[d]; have = true; continue; }
    if (strides[d] != st * n) return false;
    n *= shape[d];
  }
  *size = n; *stride = have ? st : 1;
  return true;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// plan
// ------------------------------------------------------------------------------------------------
struct GraphExec {
  Graph g;
  int n_params = 0;
  std::vector<int64_t> param_offsets;
  std::vector<int> root;                 // value -> the value whose storage it shares
  std::vector<char> where;               // per root: 0 external (argument), 1 constant arena, 2 step arena
  std::vector<long long> off;            // per root: byte offset in its arena
  std::vector<char> need_fwd, need_all;  // per op
  std::vector<char> is_const_op;
  struct OperandSrc { int mode = 0; unsigned inner = 1; int src = -1; double imm = 0.0; long long iimm = 0; };
  std::vector<OperandSrc> opnd;          // per op, two entries: how a binary op reads its operands (O_* modes)
  std::vector<char> absorbed;            // per op: a broadcast_in_dim that its only reader takes as a strided operand
  std::vector<char> skip;                // per op: a guard + clamp that runs inside its producer
  std::vector<int> post_of;              // per op: the guard + clamp op fused into it, -1 if none
  char *const_arena = nullptr, *arena = nullptr;
  char* red_scratch = nullptr;           // per-chunk partials of the column reductions
  size_t red_scratch_bytes = 0;
  char* scat_scratch = nullptr;          // sort buffers (and an f32 result for bf16) of the ordered row scatter
  size_t scat_scratch_bytes = 0;
  size_t const_bytes = 0, arena_bytes = 0;
  std::vector<const void*> ext;          // per value: pointer of an external value (set per run)
  std::vector<long long> placed_at, freed_after;   // per root in the step arena: the op that defines it, the op after which its space is free (-1: never)
  // CUDA graphs of whole runs, keyed by the bindings (pointers, seed, direction); a binding seen for the second time is
  // captured, so one-off buffers never pay for an instantiation
  struct Captured { cudaGraphExec_t exec; long long launches; };
  std::map<std::vector<unsigned long long>, Captured> captured;
  std::map<std::vector<unsigned long long>, int> seen;
};

namespace {

enum { W_EXT = 0, W_CONST = 1, W_STEP = 2 };

size_t round256(size_t x) { return (x + 255) & ~(size_t)255; }

unsigned int float_bits(float f) { unsigned int u; memcpy(&u, &f, 4); return u; }

struct FreeList {
  std::map<size_t, size_t> free_;        // offset -> size
  size_t end = 0;
  size_t alloc(size_t n) {
    // best fit
    auto best = free_.end();
    for (auto it = free_.begin(); it != free_.end(); ++it)
      if (it->second >= n && (best == free_.end() || it->second < best->second)) best = it;
    if (best != free_.end()) {
      const size_t o = best->first, sz = best->second;
      free_.erase(best);
      if (sz > n) free_[o + n] = sz - n;
      return o;
    }
    // grow; a free block touching the end is extended
    if (!free_.empty()) {
      auto last = std::prev(free_.end());
      if (last->first + last->second == end) {
        const size_t o = last->first;
        free_.erase(last);
        end = o + n;
        return o;
      }
    }
    const size_t o = end;
    end += n;
    return o;
  }
  void release(size_t o, size_t n) {
    auto it = free_.emplace(o, n).first;
    auto nx = std::next(it);
    if (nx != free_.end() && it->first + it->second == nx->first) { it->second += nx->second; free_.erase(nx); }
    if (it != free_.begin()) {
      auto pv = std::prev(it);
      if (pv->first + pv->second == it->first) { pv->second += it->second; free_.erase(it); }
    }
  }
};

void* ptr_of(const GraphExec& e, int v) {
  const int r = e.root[v];
  if (e.where[r] == W_EXT) return const_cast<void*>(e.ext[r]);
  return (e.where[r] == W_CONST ? e.const_arena : e.arena) + e.off[r];
}

#define LAUNCH_CHECK() do { cudaError_t le__ = cudaGetLastError(); if (le__ != cudaSuccess) return std::string("kernel launch failed: ") + cudaGetErrorString(le__); } while (0)

// how operand k of op i is read (binary, compare: operands 0 and 1; select: its value operands 1 and 2), null for the rest
const GraphExec::OperandSrc* operand_src(const GraphExec& e, int i, int k) {
  const int kind = e.g.ops[i].kind;
  if ((kind == G_BINARY || kind == G_COMPARE) && k < 2) return &e.opnd[2 * (size_t)i + k];
  if (kind == G_SELECT && (k == 1 || k == 2)) return &e.opnd[2 * (size_t)i + k - 1];
  return nullptr;
}

// the column-reduction form of a reduce: reduced dimensions all in front of the kept ones, enough rows to be worth it
bool cols_form(const GValue& x, const std::vector<int64_t>& dims, long long* n_red, long long* n_out) {
  long long nr = 1, no = 1;
  int64_t last_red = -1, first_kept = (int64_t)x.shape.size();
  for (size_t i = 0; i < x.shape.size(); ++i) {
    bool red = false;
    for (int64_t r : dims) red |= (r == (int64_t)i);
    if (x.shape[i] == 1) continue;
    if (red) { nr *= x.shape[i]; last_red = (int64_t)i; } else { no *= x.shape[i]; if (first_kept > (int64_t)i) first_kept = (int64_t)i; }
  }
  *n_red = nr; *n_out = no;
  return last_red < first_kept && no >= 32 && nr >= 16;
}
int cols_chunks(long long n_red) { const long long c = (n_red + 255) / 256; return (int)(c < 1 ? 1 : (c > 64 ? 64 : c)); }

// Runs one op (dry = true: only checks that it is supported).  fused_clamp: the adjoint guard that runs inside this
// element-wise op; osrc: the two operand sources of a binary / compare / select op (operand_src).
std::string run_op(GraphExec& e, const GOp& op, cudaStream_t st, bool dry, const std::function<int(int, const GemmArgs&)>* dot2d,
                   long long* launches, const GOp* fused_clamp = nullptr, const GraphExec::OperandSrc* osrc = nullptr) {
  Post post = {0, 0, 0.f, 0.f};
  if (fused_clamp) { post.on = 1; post.clamp = fused_clamp->sub; post.lo = fused_clamp->lo; post.hi = fused_clamp->hi; }
  const Graph& g = e.g;
  const GValue& o = g.vals[op.out];
  const long long n = o.numel;
  if (!known(o.dt)) return "unsupported element type";
  if (o.shape.size() > MAX_RANK) return "rank above 8";
  for (int i : op.in) if (!known(g.vals[i].dt) || g.vals[i].shape.size() > MAX_RANK) return "unsupported operand type";
  void* out = dry ? nullptr : ptr_of(e, op.out);
  auto in = [&](int k) -> const void* { return dry ? nullptr : ptr_of(e, op.in[k]); };
  auto count = [&](int k) { if (launches) *launches += k; };
  const int nb = blocks_for(n);
  const size_t es = dtype_size(o.dt);
  switch (op.kind) {
    case G_CONST_SPLAT:
    case G_SEED:
      if (dry) return "";
      BY_TYPE(o.dt, k_fill<T><<<nb, TPB, 0, st>>>((T*)out, n, op.fval, op.ival));
      count(1);
      break;
    case G_CONST_DATA:
      if ((long long)op.data.size() != n * (long long)es) return "constant payload of the wrong size";
      if (dry) return "";
      if (cudaMemcpyAsync(out, op.data.data(), op.data.size(), cudaMemcpyHostToDevice, st) != cudaSuccess) return "constant upload failed";
      break;
    case G_IOTA: {
      if (!(o.dt == DT_I64 || o.dt == DT_I32)) return "iota of this element type";
      if (op.a.size() != 1 || op.a[0] < 0 || op.a[0] >= (int64_t)o.shape.size()) return "iota: bad dimension";
      if (dry) return "";
      long long inner = 1;
      for (size_t i = op.a[0] + 1; i < o.shape.size(); ++i) inner *= o.shape[i];
      if (o.dt == DT_I64) k_iota<long long><<<nb, TPB, 0, st>>>((long long*)out, n, inner, o.shape[op.a[0]]);
      else k_iota<int><<<nb, TPB, 0, st>>>((int*)out, n, inner, o.shape[op.a[0]]);
      count(1);
      break;
    }
    case G_UNARY:
      if (!is_fp(o.dt) && !(op.sub == U_NEG || op.sub == U_ABS)) return "unary op on an integer type";
      if (o.dt == DT_BOOL) return "unary op on i1";
      if (dry) return "";
      BY_TYPE(o.dt, k_unary<T><<<nb, TPB, 0, st>>>(op.sub, (const T*)in(0), (T*)out, n, post));
      count(1);
      break;
    case G_BINARY:
      if (is_fp(o.dt) && (op.sub == B_AND || op.sub == B_OR)) return "logical op on a float type";
      if (!is_fp(o.dt) && op.sub == B_POW) return "power on an integer type";
      if (dry) return "";
      {
        Opnd od[2];
        const void* ptr[2];
        for (int k = 0; k < 2; ++k) {
          od[k].mode = O_DIRECT; od[k].inner = 1; od[k].imm = 0.0; od[k].iimm = 0;
          ptr[k] = nullptr;
          if (osrc && osrc[k].mode != O_DIRECT) {
            od[k].mode = osrc[k].mode; od[k].inner = osrc[k].inner; od[k].imm = osrc[k].imm; od[k].iimm = osrc[k].iimm;
            if (osrc[k].mode != O_IMM) ptr[k] = ptr_of(e, osrc[k].src);
          } else ptr[k] = in(k);
        }
        BY_TYPE(o.dt, k_binary<T><<<nb, TPB, 0, st>>>(op.sub, (const T*)ptr[0], (const T*)ptr[1], (T*)out, n, post, od[0], od[1]));
      }
      count(1);
      break;
    case G_COMPARE: {
      const int dt = g.vals[op.in[0]].dt;
      if (dt != g.vals[op.in[1]].dt || o.dt != DT_BOOL) return "compare: operand types";
      if (dry) return "";
      {
        Opnd od[2];
        const void* ptr[2];
        for (int k = 0; k < 2; ++k) {
          od[k].mode = O_DIRECT; od[k].inner = 1; od[k].imm = 0.0; od[k].iimm = 0;
          if (osrc && osrc[k].mode == O_IMM) { od[k].mode = O_IMM; od[k].imm = osrc[k].imm; od[k].iimm = osrc[k].iimm; ptr[k] = nullptr; }
          else ptr[k] = in(k);
        }
        BY_TYPE(dt, k_compare<T><<<nb, TPB, 0, st>>>(op.sub, (const T*)ptr[0], (const T*)ptr[1], (uint8_t*)out, n, od[0], od[1]));
      }
      count(1);
      break;
    }
    case G_SELECT:
      if (g.vals[op.in[0]].dt != DT_BOOL || g.vals[op.in[0]].numel != n) return "select: the predicate must be i1 of the result's shape";
      if (dry) return "";
      {
        unsigned long long bits[2] = {0, 0};
        int imm[2] = {0, 0};
        const void* ptr[2];
        for (int k = 0; k < 2; ++k) {
          if (osrc && osrc[k].mode == O_IMM) {
            imm[k] = 1; ptr[k] = nullptr;
            switch (o.dt) {
              case DT_F32: { const float f = (float)osrc[k].imm; unsigned u; memcpy(&u, &f, 4); bits[k] = u; break; }
              case DT_BF16: { const bf16 h = __float2bfloat16_rn((float)osrc[k].imm); unsigned short u; memcpy(&u, &h, 2); bits[k] = u; break; }
              case DT_F64: { memcpy(&bits[k], &osrc[k].imm, 8); break; }
              case DT_I32: bits[k] = (unsigned)(int)osrc[k].iimm; break;
              case DT_BOOL: bits[k] = osrc[k].iimm != 0; break;
              default: bits[k] = (unsigned long long)osrc[k].iimm; break;
            }
          } else ptr[k] = in(k + 1);
        }
        BY_SIZE(es, k_select<U><<<nb, TPB, 0, st>>>((const uint8_t*)in(0), (const U*)ptr[0], (const U*)ptr[1], (U*)out, n, imm[0], imm[1], (U)bits[0], (U)bits[1]));
      }
      count(1);
      break;
    case G_CONVERT:
      if (dry) return "";
      if (g.vals[op.in[0]].dt == o.dt) break;                 // shares its operand's storage
      convert(st, in(0), g.vals[op.in[0]].dt, out, o.dt, n);
      count(1);
      break;
    case G_RESHAPE:
      break;                                                   // shares its operand's storage
    case G_GUARD_CLAMP:
      if (!is_fp(o.dt)) return "adjoint of an integer type";
      if (dry) return "";
      BY_FLOAT(o.dt, k_guard_clamp<T><<<nb, TPB, 0, st>>>((const T*)in(0), (T*)out, n, op.sub, op.lo, op.hi));
      count(1);
      break;
    case G_TRANSPOSE:
    case G_BCAST:
    case G_SLICE: {
      const GValue& x = g.vals[op.in[0]];
      const std::vector<long long> xs = row_major_strides(x.shape);
      NdDesc d;
      d.rank = (int)o.shape.size(); d.offset = 0;
      for (int k = 0; k < d.rank; ++k) { d.dim[k] = o.shape[k]; d.stride[k] = 0; }
      if (op.kind == G_TRANSPOSE) {
        if (op.a.size() != o.shape.size()) return "transpose: rank mismatch";
        for (int k = 0; k < d.rank; ++k) {
          if (op.a[k] < 0 || op.a[k] >= d.rank || x.shape[op.a[k]] != o.shape[k]) return "transpose: bad permutation";
          d.stride[k] = xs[op.a[k]];
        }
      } else if (op.kind == G_BCAST) {
        if (op.a.size() != x.shape.size()) return "broadcast_in_dim: rank mismatch";
        for (size_t s = 0; s < op.a.size(); ++s) {
          const int64_t dst = op.a[s];
          if (dst < 0 || dst >= d.rank || (x.shape[s] != 1 && x.shape[s] != o.shape[dst])) return "broadcast_in_dim: bad dims";
          d.stride[dst] = (x.shape[s] == 1) ? 0 : xs[s];
        }
      } else {
        if (op.a.size() != x.shape.size() || x.shape.size() != o.shape.size()) return "slice: rank mismatch";
        for (int k = 0; k < d.rank; ++k) {
          if (op.c[k] < 1 || op.a[k] < 0 || op.b[k] > x.shape[k] || (op.b[k] - op.a[k] + op.c[k] - 1) / op.c[k] != o.shape[k]) return "slice: bad range";
          d.stride[k] = xs[k] * op.c[k];
          d.offset += op.a[k] * xs[k];
        }
      }
      if (dry) return "";
      collapse_walk(&d);
      const long long inner = d.dim[d.rank - 1];
      if (inner >= 32 && n < 0x7FFFFFFFLL) {
        const unsigned n_rows = (unsigned)(n / inner);
        const int rb = (int)std::min<long long>(((long long)n_rows * 32 + TPB - 1) / TPB, 148 * 32);
        BY_SIZE(es, k_gather_rows_nd<U><<<rb, TPB, 0, st>>>((const U*)in(0), (U*)out, n_rows, (unsigned)inner, d));
      } else {
        BY_SIZE(es, k_gather_nd<U><<<nb, TPB, 0, st>>>((const U*)in(0), (U*)out, n, d));
      }
      count(1);
      break;
    }
    case G_PAD: {
      const GValue& x = g.vals[op.in[0]];
      const std::vector<long long> os = row_major_strides(o.shape);
      if (op.a.size() != o.shape.size() || x.shape.size() != o.shape.size()) return "pad: rank mismatch";
      NdDesc d;
      d.rank = (int)x.shape.size(); d.offset = 0;
      for (int k = 0; k < d.rank; ++k) {
        if ((op.b[k] - op.a[k] + op.c[k] - 1) / op.c[k] != x.shape[k] || op.b[k] > o.shape[k]) return "pad: bad range";
        d.dim[k] = x.shape[k]; d.stride[k] = os[k] * op.c[k]; d.offset += op.a[k] * os[k];
      }
      if (dry) return "";
      if (cudaMemsetAsync(out, 0, (size_t)n * es, st) != cudaSuccess) return "memset failed";
      BY_SIZE(es, k_scatter_nd<U><<<blocks_for(x.numel), TPB, 0, st>>>((const U*)in(0), (U*)out, x.numel, d));
      count(1);
      break;
    }
    case G_CONCAT: {
      const std::vector<long long> os = row_major_strides(o.shape);
      const int64_t dim = op.a[0];
      if (dim < 0 || dim >= (int64_t)o.shape.size()) return "concatenate: bad dimension";
      long long at = 0;
      for (size_t i = 0; i < op.in.size(); ++i) {
        const GValue& x = g.vals[op.in[i]];
        if (x.shape.size() != o.shape.size() || x.dt != o.dt) return "concatenate: operand types";
        NdDesc d;
        d.rank = (int)x.shape.size(); d.offset = at * os[dim];
        for (int k = 0; k < d.rank; ++k) {
          if (k != dim && x.shape[k] != o.shape[k]) return "concatenate: operand shapes";
          d.dim[k] = x.shape[k]; d.stride[k] = os[k];
        }
        at += x.shape[dim];
        if (dry) continue;
        BY_SIZE(es, k_scatter_nd<U><<<blocks_for(x.numel), TPB, 0, st>>>((const U*)in((int)i), (U*)out, x.numel, d));
        count(1);
      }
      if (at != o.shape[dim]) return "concatenate: sizes do not add up";
      break;
    }
    case G_REDUCE: {
      const GValue& x = g.vals[op.in[0]];
      if (x.dt != o.dt || g.vals[op.in[1]].dt != o.dt || g.vals[op.in[1]].numel != 1) return "reduce: operand types";
      if (o.dt == DT_BOOL) return "reduce over i1";
      const std::vector<long long> xs = row_major_strides(x.shape);
      RedDesc d;
      d.krank = d.rrank = 0; d.n_out = 1; d.n_red = 1;
      for (size_t i = 0; i < x.shape.size(); ++i) {
        bool red = false;
        for (int64_t r : op.a) red |= (r == (int64_t)i);
        if (red) { d.rdim[d.rrank] = x.shape[i]; d.rstr[d.rrank++] = xs[i]; d.n_red *= x.shape[i]; }
        else { d.kdim[d.krank] = x.shape[i]; d.kstr[d.krank++] = xs[i]; d.n_out *= x.shape[i]; }
      }
      if (d.n_out != n) return "reduce: result shape mismatch";
      if (dry) return "";
      long long cr, co;
      if (cols_form(x, op.a, &cr, &co) && e.red_scratch) {
        const int chunks = cols_chunks(cr);
        if ((size_t)chunks * co * 8 <= e.red_scratch_bytes) {
          const long long rpc = (cr + chunks - 1) / chunks;
          const dim3 grid((unsigned)((co + 31) / 32), (unsigned)chunks);
#define REDC(T, KIND)                                                                                                  \
  do {                                                                                                                 \
    k_reduce_cols<T, KIND><<<grid, 256, 0, st>>>((const T*)in(0), (TT<T>::C*)e.red_scratch, cr, co, rpc);              \
    k_reduce_cols_finish<T, KIND><<<blocks_for(co), TPB, 0, st>>>((const TT<T>::C*)e.red_scratch, (const T*)in(1), (T*)out, chunks, co); \
  } while (0)
#define REDC2(T) do { if (op.sub == R_ADD) REDC(T, R_ADD); else REDC(T, R_MAX); } while (0)
          switch (o.dt) {
            case DT_F32: REDC2(float); break;
            case DT_BF16: REDC2(bf16); break;
            case DT_F64: REDC2(double); break;
            case DT_I64: REDC2(long long); break;
            default: REDC2(int); break;
          }
#undef REDC2
#undef REDC
          count(2);
          break;
        }
      }
      const bool wide = d.n_red >= 64;
      const long long threads = d.n_out * (wide ? 32 : 1);
      const int blocks = (int)((threads + TPB - 1) / TPB);
#define RED(T)                                                                                                        \
  do {                                                                                                                \
    if (op.sub == R_ADD) { if (wide) k_reduce<T, R_ADD, 32><<<blocks, TPB, 0, st>>>((const T*)in(0), (const T*)in(1), (T*)out, d); \
                           else k_reduce<T, R_ADD, 1><<<blocks, TPB, 0, st>>>((const T*)in(0), (const T*)in(1), (T*)out, d); }     \
    else { if (wide) k_reduce<T, R_MAX, 32><<<blocks, TPB, 0, st>>>((const T*)in(0), (const T*)in(1), (T*)out, d);              \
           else k_reduce<T, R_MAX, 1><<<blocks, TPB, 0, st>>>((const T*)in(0), (const T*)in(1), (T*)out, d); }                  \
  } while (0)
      switch (o.dt) {
        case DT_F32: RED(float); break;
        case DT_BF16: RED(bf16); break;
        case DT_F64: RED(double); break;
        case DT_I64: RED(long long); break;
        default: RED(int); break;
      }
#undef RED
      count(1);
      break;
    }
    case G_DOT: {
      const GValue &x = g.vals[op.in[0]], &y = g.vals[op.in[1]];
      if (!is_fp(o.dt) || x.dt != o.dt || y.dt != o.dt) return "dot_general: operand types";
      const std::vector<long long> xs = row_major_strides(x.shape), ys = row_major_strides(y.shape);
      auto inl = [](const std::vector<int64_t>& v, int64_t i) { for (int64_t q : v) if (q == i) return true; return false; };
      std::vector<int64_t> xf, yf;
      for (size_t i = 0; i < x.shape.size(); ++i) if (!inl(op.a, i) && !inl(op.c, i)) xf.push_back((int64_t)i);
      for (size_t i = 0; i < y.shape.size(); ++i) if (!inl(op.b, i) && !inl(op.d, i)) yf.push_back((int64_t)i);
      long long nbx, nby, M, N, K, K2;
      DotDesc d;
      if (!collapse(x.shape, xs, op.a, &nbx, &d.ab) || !collapse(y.shape, ys, op.b, &nby, &d.bb) ||
          !collapse(x.shape, xs, xf, &M, &d.am) || !collapse(y.shape, ys, yf, &N, &d.bn) ||
          !collapse(x.shape, xs, op.c, &K, &d.ak) || !collapse(y.shape, ys, op.d, &K2, &d.bk))
        return "dot_general: the dimension groups of an operand do not lie in memory like one dimension each";
      if (nbx != nby || K != K2 || nbx * M * N != n) return "dot_general: shape mismatch";
      if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF || nbx > 65535 || (M + 63) / 64 > 65535) return "dot_general: too large for the general kernel";
      d.M = (int)M; d.N = (int)N; d.K = (int)K;
      if (dry) return "";
      if (nbx == 1 && dot2d && *dot2d && (o.dt == DT_F32 || o.dt == DT_BF16)) {
        GemmArgs ga;
        ga.A = in(0); ga.sam = d.am; ga.sak = d.ak; ga.B = in(1); ga.sbk = d.bk; ga.sbn = d.bn; ga.C = out; ga.ldc = N;
        ga.R = nullptr; ga.C2 = nullptr; ga.M = d.M; ga.N = d.N; ga.K = d.K; ga.epi = EPI_STORE; ga.clip = 0.f;
        const int hr = (*dot2d)(o.dt, ga);
        if (hr == 0) break;
        if (hr != 1) return "dot_general: the GEMM dispatch failed";
      }
      const dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64), (unsigned)nbx);
      BY_FLOAT(o.dt, k_dot<T><<<grid, 256, 0, st>>>((const T*)in(0), (const T*)in(1), (T*)out, d));
      count(1);
      break;
    }
    case G_GATHER_ROWS: {
      const GValue& x = g.vals[op.in[0]];
      if (g.vals[op.in[1]].dt != DT_I64 || x.shape.empty() || x.dt != o.dt) return "gather: operand types";
      const long long rowlen = x.numel / x.shape[0];
      if (g.vals[op.in[1]].numel * rowlen != n) return "gather: shape mismatch";
      if (dry) return "";
      BY_SIZE(es, k_gather_rows<U><<<nb, TPB, 0, st>>>((const U*)in(0), (const long long*)in(1), (U*)out, n, rowlen, x.shape[0]));
      count(1);
      break;
    }
    case G_GATHER2: {
      const GValue& x = g.vals[op.in[0]];
      if (g.vals[op.in[1]].dt != DT_I64 || x.shape.size() != 2 || x.dt != o.dt || g.vals[op.in[1]].numel != 2 * n) return "gather: operand types";
      if (dry) return "";
      BY_SIZE(es, k_gather2<U><<<nb, TPB, 0, st>>>((const U*)in(0), (const long long*)in(1), (U*)out, n, x.shape[0], x.shape[1]));
      count(1);
      break;
    }
    case G_SCATTER_ROWS:
    case G_SCATTER2: {
      const GValue& gr = g.vals[op.in[0]];
      if (!is_fp(o.dt) || gr.dt != o.dt || g.vals[op.in[1]].dt != DT_I64 || o.shape.empty()) return "scatter: operand types";
      const long long rowlen = n / o.shape[0];
      if (op.kind == G_SCATTER_ROWS ? (g.vals[op.in[1]].numel * rowlen != gr.numel) : (o.shape.size() != 2 || g.vals[op.in[1]].numel != 2 * gr.numel))
        return "scatter: shape mismatch";
      if (dry) return "";
      if (op.kind == G_SCATTER_ROWS && e.scat_scratch && (o.dt == DT_F32 || o.dt == DT_BF16)) {
        // the embedding-gradient form: rows sorted by index (stable), summed in position order in f32 — no float
        // atomics, the same bits every run (embed_scatter.cu); indices are clamped like the gather's
        const int M = (int)g.vals[op.in[1]].numel, d = (int)rowlen, V = (int)o.shape[0];
        const size_t sorted_bytes = embed_scatter_scratch_bytes(M, d);
        const size_t tmp_bytes = o.dt == DT_BF16 ? (size_t)n * 4 : 0;
        if (sorted_bytes + tmp_bytes <= e.scat_scratch_bytes) {
          float* acc = o.dt == DT_F32 ? (float*)out : (float*)(e.scat_scratch + sorted_bytes);
          if (cudaMemsetAsync(acc, 0, (size_t)n * 4, st) != cudaSuccess) return "memset failed";
          if (launch_embed_scatter_sorted(st, o.dt, (const long long*)in(1), M, d, V, in(0), e.scat_scratch, sorted_bytes, acc) != cudaSuccess)
            return "the ordered row scatter failed";
          count(6);
          if (o.dt == DT_BF16) { convert(st, acc, DT_F32, out, DT_BF16, n); count(1); }
          break;
        }
      }
      if (cudaMemsetAsync(out, 0, (size_t)n * es, st) != cudaSuccess) return "memset failed";
      const int gb = blocks_for(gr.numel);
      if (op.kind == G_SCATTER_ROWS) {
        BY_FLOAT(o.dt, k_scatter_rows<T><<<gb, TPB, 0, st>>>((const T*)in(0), (const long long*)in(1), (T*)out, gr.numel, rowlen, o.shape[0]));
      } else {
        BY_FLOAT(o.dt, k_scatter2<T><<<gb, TPB, 0, st>>>((const T*)in(0), (const long long*)in(1), (T*)out, gr.numel, o.shape[0], o.shape[1]));
      }
      count(1);
      break;
    }
    default:
      return "unknown op kind";
  }
  if (!dry) LAUNCH_CHECK();
  return "";
}

}  // namespace

std::string graph_exec_create(const Graph& g, int n_params, const std::vector<int64_t>& param_offsets, cudaStream_t st,
                              GraphExec** out, bool plan_only) {
  *out = nullptr;
  GraphExec* e = new GraphExec();
  e->g = g;
  e->n_params = n_params;
  e->param_offsets = param_offsets;
  const int nv = (int)g.vals.size(), nops = (int)g.ops.size();
  auto failed = [&](const std::string& why) { graph_exec_destroy(e); return why; };
  // constants: produced without reading an argument or the seed
  std::vector<char> cval(nv, 0);
  e->is_const_op.assign(nops, 0);
  for (int i = 0; i < nops; ++i) {
    const GOp& op = g.ops[i];
    bool c = op.kind != G_SEED;
    for (int x : op.in) c = c && cval[x];
    e->is_const_op[i] = c;
    cval[op.out] = c;
  }
  // needed ops: those the result (forward) or the result and the gradients (all) depend on
  auto mark = [&](std::vector<char>& need, const std::vector<int>& outs, int upto) {
    std::vector<char> nval(nv, 0);
    for (int v : outs) if (v >= 0) nval[v] = 1;
    need.assign(nops, 0);
    for (int i = upto - 1; i >= 0; --i) {
      const GOp& op = g.ops[i];
      if (!nval[op.out]) continue;
      need[i] = 1;
      for (int x : op.in) nval[x] = 1;
    }
  };
  std::vector<int> outs = {g.ret};
  mark(e->need_fwd, outs, g.n_forward_ops);
  for (int v : g.grad_of_arg) outs.push_back(v);
  mark(e->need_all, outs, nops);
  // an adjoint-edge guard whose operand is an element-wise float result of the gradient program with no other reader
  // runs inside the producing kernel (PCPB_GRAPH_FUSE=0 keeps them apart)
  e->skip.assign(nops, 0);
  e->post_of.assign(nops, -1);
  // A guard + clamp of a value that is known to be finite and inside the bounds already is the identity and shares its
  // operand's storage: the operand is itself a guarded value, or pure data movement (reshape, transpose, slice,
  // broadcast, pad, concatenate, gather, select) of guarded values and in-range constants.  The AD rules produce many:
  // add, reshape, transpose, slice, broadcast and select hand an already guarded adjoint on.
  {
    const char* fe = getenv("PCPB_GRAPH_FUSE");
    const GOp* first = nullptr;
    for (int i = g.n_forward_ops; i < nops && !first; ++i) if (g.ops[i].kind == G_GUARD_CLAMP) first = &g.ops[i];
    std::vector<char> guarded(nv, 0);
    for (int i = 0; i < nops && first && !(fe && fe[0] == '0'); ++i) {
      const GOp& op = g.ops[i];
      auto in_ok = [&](size_t k) { return k < op.in.size() && guarded[op.in[k]]; };
      bool ok = false;
      switch (op.kind) {
        case G_GUARD_CLAMP:
          if (op.sub == first->sub && op.lo == first->lo && op.hi == first->hi) {
            if (in_ok(0) && e->need_all[i] && !e->is_const_op[i]) e->skip[i] = 1;
            ok = true;
          }
          break;
        case G_CONST_SPLAT: ok = is_fp(g.vals[op.out].dt) && std::isfinite(op.fval) && (!first->sub || (op.fval >= first->lo && op.fval <= first->hi)); break;
        case G_RESHAPE: case G_TRANSPOSE: case G_SLICE: case G_BCAST: case G_PAD: case G_GATHER_ROWS: case G_GATHER2: ok = in_ok(0); break;
        case G_CONVERT: ok = in_ok(0) && g.vals[op.in[0]].dt == g.vals[op.out].dt; break;
        case G_SELECT: ok = in_ok(1) && in_ok(2); break;
        case G_CONCAT: ok = true; for (size_t k = 0; k < op.in.size(); ++k) ok = ok && in_ok(k); break;
        case G_UNARY: ok = op.sub == U_NEG && in_ok(0) && (!first->sub || first->lo == -first->hi); break;
        default: break;
      }
      guarded[op.out] = ok;
    }
  }
  {
    const char* fe = getenv("PCPB_GRAPH_FUSE");
    std::vector<int> readers(nv, 0);
    for (int i = 0; i < nops; ++i)
      if (e->need_all[i]) for (int x : g.ops[i].in) readers[x] += 1;
    for (int v : outs) if (v >= 0) readers[v] += 1;
    for (int i = g.n_forward_ops; i < nops && !(fe && fe[0] == '0'); ++i) {
      const GOp& op = g.ops[i];
      if (!e->need_all[i] || op.kind != G_GUARD_CLAMP || e->is_const_op[i] || e->skip[i]) continue;
      const int v = op.in[0], j = g.vals[v].op;
      if (j < g.n_forward_ops || !e->need_all[j] || e->is_const_op[j] || readers[v] != 1 || e->post_of[j] >= 0) continue;
      if (!(g.ops[j].kind == G_UNARY || g.ops[j].kind == G_BINARY) || !is_fp(g.vals[v].dt)) continue;
      e->post_of[j] = i;
      e->skip[i] = 1;
    }
  }
  // storage sharing: reshape, same-type convert and a fused guard are views of their operand
  e->root.resize(nv);
  for (int v = 0; v < nv; ++v) e->root[v] = v;
  for (int i = 0; i < nops; ++i) {
    const GOp& op = g.ops[i];
    if (op.kind == G_RESHAPE || (op.kind == G_CONVERT && g.vals[op.in[0]].dt == g.vals[op.out].dt) || e->skip[i]) e->root[op.out] = e->root[op.in[0]];
  }
  // Operands of binary ops that need no tensor of their own: a broadcast_in_dim read by this op alone, of the forms
  // [rows, 1] -> [rows, inner], [inner] -> [rows, inner] or scalar -> anything, is read from its source with the index
  // arithmetic done in the kernel, and a constant that is a splat (through broadcasts and reshapes) is an immediate.
  // PCPB_GRAPH_FUSE=0 keeps every operand a tensor.
  e->opnd.assign(2 * (size_t)nops, GraphExec::OperandSrc());
  e->absorbed.assign(nops, 0);
  {
    const char* fe = getenv("PCPB_GRAPH_FUSE");
    const bool on = !(fe && fe[0] == '0');
    auto is_view = [&](int i) {
      const GOp& op = g.ops[i];
      return op.kind == G_RESHAPE || (op.kind == G_CONVERT && g.vals[op.in[0]].dt == g.vals[op.out].dt) || e->skip[i];
    };
    std::vector<std::vector<std::pair<int, int>>> kreaders(nv);
    std::vector<char> is_out(nv, 0);
    for (int i = 0; i < nops; ++i)
      if (e->need_all[i] && !is_view(i))
        for (size_t k = 0; k < g.ops[i].in.size(); ++k) kreaders[e->root[g.ops[i].in[k]]].push_back({i, (int)k});
    for (int v : outs) if (v >= 0) is_out[e->root[v]] = 1;
    for (int j = 0; j < nops && on; ++j) {
      const GOp& op = g.ops[j];
      if (!e->need_all[j] || e->is_const_op[j] || op.kind != G_BCAST || e->root[op.out] != op.out || is_out[op.out]) continue;
      const auto& rd = kreaders[op.out];
      if (rd.size() != 1) continue;
      const int i = rd[0].first, k = rd[0].second;
      const GValue &x = g.vals[op.in[0]], &o = g.vals[op.out];
      if (g.ops[i].kind != G_BINARY || e->is_const_op[i] || o.numel >= 0x7FFFFFFFLL || op.a.size() != x.shape.size()) continue;
      const std::vector<long long> xs = row_major_strides(x.shape);
      NdDesc d;
      d.rank = (int)o.shape.size(); d.offset = 0;
      bool ok = d.rank <= MAX_RANK;
      for (int q = 0; q < d.rank && ok; ++q) { d.dim[q] = o.shape[q]; d.stride[q] = 0; }
      for (size_t q = 0; q < op.a.size() && ok; ++q) {
        const int64_t dst = op.a[q];
        if (dst < 0 || dst >= d.rank || (x.shape[q] != 1 && x.shape[q] != o.shape[dst])) { ok = false; break; }
        d.stride[dst] = (x.shape[q] == 1) ? 0 : xs[q];
      }
      if (!ok) continue;
      collapse_walk(&d);
      GraphExec::OperandSrc os;
      os.src = op.in[0];
      if (d.rank == 1 && d.stride[0] == 0) os.mode = O_SCALAR;
      else if (d.rank == 2 && d.stride[0] == 1 && d.stride[1] == 0) { os.mode = O_PER_RUN; os.inner = (unsigned)d.dim[1]; }
      else if (d.rank == 2 && d.stride[0] == 0 && d.stride[1] == 1) { os.mode = O_IN_RUN; os.inner = (unsigned)d.dim[1]; }
      else continue;
      e->opnd[2 * (size_t)i + k] = os;
      e->absorbed[j] = 1;
    }
    // splat constants as immediates
    auto splat_of = [&](int v, double* f, long long* iv) {
      for (int hops = 0; hops < 8; ++hops) {
        const int pi = g.vals[v].op;
        if (pi < 0 || !e->is_const_op[pi]) return false;
        const GOp& po = g.ops[pi];
        if (po.kind == G_CONST_SPLAT) {
          const int dt = g.vals[po.out].dt;
          *f = dt == DT_F64 ? po.fval : (double)(dt == DT_BF16 ? __bfloat162float(__float2bfloat16_rn((float)po.fval)) : (float)po.fval);
          *iv = dt == DT_BOOL ? (po.ival != 0) : (dt == DT_I32 ? (long long)(int)po.ival : po.ival);
          return true;
        }
        if (po.kind == G_BCAST || po.kind == G_RESHAPE) { v = po.in[0]; continue; }
        return false;
      }
      return false;
    };
    for (int i = 0; i < nops && on; ++i) {
      const GOp& op = g.ops[i];
      if (!e->need_all[i] || e->is_const_op[i] || !(op.kind == G_BINARY || op.kind == G_COMPARE || op.kind == G_SELECT)) continue;
      const int first = op.kind == G_SELECT ? 1 : 0;           // select: the two value operands
      for (int k = 0; k < 2; ++k) {
        GraphExec::OperandSrc& os = e->opnd[2 * (size_t)i + k];
        if (os.mode != O_DIRECT) continue;
        double f; long long iv;
        if (splat_of(op.in[first + k], &f, &iv)) { os.mode = O_IMM; os.imm = f; os.iimm = iv; }
      }
    }
    // constants that nothing reads as a tensor any more (every reader takes an immediate) are neither evaluated nor stored
    std::vector<char> read(nv, 0);
    for (int v : outs) if (v >= 0) read[v] = 1;
    for (int i = nops - 1; i >= 0 && on; --i) {
      const GOp& op = g.ops[i];
      if (!e->need_all[i] || e->absorbed[i]) continue;
      if (e->is_const_op[i] && !read[op.out]) { e->need_all[i] = 0; e->need_fwd[i] = 0; continue; }
      for (size_t k = 0; k < op.in.size(); ++k) {
        int x = op.in[k];
        const GraphExec::OperandSrc* os = operand_src(*e, i, (int)k);
        if (os && os->mode == O_IMM) continue;
        if (os && os->mode != O_DIRECT) x = os->src;
        read[x] = 1;
      }
    }
  }
  // every needed op must have a kernel
  for (int i = 0; i < nops; ++i) {
    if (!e->need_all[i]) continue;
    const std::string why = run_op(*e, g.ops[i], st, true, nullptr, nullptr);
    if (!why.empty()) {
      const GValue& o = g.vals[g.ops[i].out];
      return failed(why + (o.name.empty() ? std::string(" (in the gradient program)") : " (%" + o.name + ")"));
    }
  }
  // placement
  e->where.assign(nv, W_STEP);
  e->off.assign(nv, 0);
  for (int a : g.args) e->where[a] = W_EXT;
  std::vector<long long> last(nv, -1);            // per root: index of the last needed step op that touches it
  const long long FOREVER = (long long)nops + 1;
  for (int i = 0; i < nops; ++i) {
    if (!e->need_all[i]) continue;
    const GOp& op = g.ops[i];
    if (e->is_const_op[i]) { e->where[e->root[op.out]] = W_CONST; continue; }
    if (e->absorbed[i]) continue;                        // never materialised: its reader takes the source
    last[e->root[op.out]] = std::max<long long>(last[e->root[op.out]], i);
    for (size_t k = 0; k < op.in.size(); ++k) {
      int x = op.in[k];
      const GraphExec::OperandSrc* os = operand_src(*e, i, (int)k);
      if (os && os->mode == O_IMM) continue;
      if (os && os->mode != O_DIRECT) x = os->src;
      last[e->root[x]] = std::max<long long>(last[e->root[x]], i);
    }
  }
  for (int v : outs) if (v >= 0) last[e->root[v]] = FOREVER;
  size_t cbytes = 0;
  FreeList fl;
  e->placed_at.assign(nv, -1);
  e->freed_after.assign(nv, -1);
  std::vector<char> placed(nv, 0);
  std::map<long long, std::vector<int>> dies;     // op index -> roots to release after it
  for (int i = 0; i < nops; ++i) {
    if (!e->need_all[i] || e->absorbed[i]) continue;
    const GOp& op = g.ops[i];
    const int r = e->root[op.out];
    const size_t bytes = round256((size_t)g.vals[r].numel * dtype_size(g.vals[r].dt));
    if (e->is_const_op[i]) {
      if (r == op.out && !placed[r]) { e->off[r] = (long long)cbytes; cbytes += bytes; placed[r] = 1; }
      continue;
    }
    if (e->where[r] == W_STEP && !placed[r] && !(g.vals[r].op >= 0 && e->absorbed[g.vals[r].op])) {   // an absorbed broadcast has no storage, nor have its views
      e->off[r] = (long long)fl.alloc(bytes);
      placed[r] = 1;
      e->placed_at[r] = i;
      if (last[r] != FOREVER) { dies[last[r]].push_back(r); e->freed_after[r] = last[r]; }
    }
    auto d = dies.find(i);
    if (d != dies.end())
      for (int dead : d->second) fl.release((size_t)e->off[dead], round256((size_t)g.vals[dead].numel * dtype_size(g.vals[dead].dt)));
  }
  e->const_bytes = cbytes;
  e->arena_bytes = fl.end;
  if (plan_only) { *out = e; return ""; }
  if (cudaMalloc(&e->const_arena, cbytes ? cbytes : 256) != cudaSuccess) { e->const_arena = nullptr; return failed("cudaMalloc of the constant arena failed"); }
  if (cudaMalloc(&e->arena, e->arena_bytes ? e->arena_bytes : 256) != cudaSuccess) {
    e->arena = nullptr;
    char m[128];
    snprintf(m, sizeof m, "cudaMalloc of the %zu-byte arena failed", e->arena_bytes);
    return failed(m);
  }
  e->ext.assign(nv, nullptr);
  // PCPB_POISON=1 (as for the workspace of the fused families): NaN patterns in the arenas, so that an op reading a
  // value nothing wrote shows up in the parity tests
  {
    const char* pe = getenv("PCPB_POISON");
    if (pe && pe[0] == '1') {
      cudaMemset(e->arena, 0xFF, e->arena_bytes ? e->arena_bytes : 256);
      cudaMemset(e->const_arena, 0xFF, cbytes ? cbytes : 256);
    }
  }
  // scratch of the column reductions: [chunks][n_out] partials of the widest one
  {
    size_t want = 0;
    for (int i = 0; i < nops; ++i) {
      if (!e->need_all[i] || g.ops[i].kind != G_REDUCE) continue;
      long long cr, co;
      if (cols_form(g.vals[g.ops[i].in[0]], g.ops[i].a, &cr, &co)) want = std::max<size_t>(want, (size_t)cols_chunks(cr) * (size_t)co * 8);
    }
    if (want) {
      if (cudaMalloc(&e->red_scratch, want) != cudaSuccess) { e->red_scratch = nullptr; return failed("cudaMalloc of the reduction scratch failed"); }
      e->red_scratch_bytes = want;
    }
  }
  // scratch of the ordered row scatter (PCPB_EMBED_ATOMIC=1: float atomics instead, as for the fused families)
  {
    const char* ae = getenv("PCPB_EMBED_ATOMIC");
    size_t want = 0;
    for (int i = 0; i < nops && !(ae && ae[0] == '1'); ++i) {
      const GOp& op = g.ops[i];
      if (!e->need_all[i] || op.kind != G_SCATTER_ROWS) continue;
      const GValue& o = g.vals[op.out];
      const long long M = g.vals[op.in[1]].numel, V = o.shape.empty() ? 0 : o.shape[0];
      if (!(o.dt == DT_F32 || o.dt == DT_BF16) || V <= 0 || M <= 0 || M >= 0x7FFFFFFFLL || V >= 0x7FFFFFFFLL || o.numel / V >= 0x7FFFFFFFLL) continue;
      const size_t need = round256(embed_scatter_scratch_bytes((int)M, (int)(o.numel / V))) + (o.dt == DT_BF16 ? (size_t)o.numel * 4 : 0);
      want = std::max(want, need);
    }
    if (want) {
      if (cudaMalloc(&e->scat_scratch, want) != cudaSuccess) { e->scat_scratch = nullptr; return failed("cudaMalloc of the scatter scratch failed"); }
      e->scat_scratch_bytes = want;
    }
  }
  // the constant part, once
  for (int i = 0; i < nops; ++i) {
    if (!e->need_all[i] || !e->is_const_op[i]) continue;
    const std::string why = run_op(*e, g.ops[i], st, false, nullptr, nullptr);
    if (!why.empty()) return failed(why);
  }
  if (cudaStreamSynchronize(st) != cudaSuccess) return failed("evaluating the constants of the graph failed");
  *out = e;
  return "";
}

void graph_exec_destroy(GraphExec* e) {
  if (!e) return;
  for (auto& c : e->captured) cudaGraphExecDestroy(c.second.exec);
  if (e->const_arena) cudaFree(e->const_arena);
  if (e->arena) cudaFree(e->arena);
  if (e->red_scratch) cudaFree(e->red_scratch);
  if (e->scat_scratch) cudaFree(e->scat_scratch);
  delete e;
}

size_t graph_exec_arena_bytes(const GraphExec* e) { return e ? e->arena_bytes + e->const_bytes : 0; }

namespace {

// the ops of one run, in order, as launches on st
std::string enqueue_run(GraphExec* e, cudaStream_t st, const GraphBind& bind, const std::function<int(int, const GemmArgs&)>& dot2d,
                        long long* launches) {
  const Graph& g = e->g;
  const int upto = bind.backward ? (int)g.ops.size() : g.n_forward_ops;
  const std::vector<char>& need = bind.backward ? e->need_all : e->need_fwd;
  for (int i = 0; i < upto; ++i) {
    if (!need[i] || e->is_const_op[i] || e->skip[i] || e->absorbed[i]) continue;
    GOp seed_op;
    const GOp* op = &g.ops[i];
    if (op->kind == G_SEED) { seed_op = *op; seed_op.fval = (double)bind.seed; seed_op.ival = (long long)bind.seed; op = &seed_op; }
    const std::string why = run_op(*e, *op, st, false, &dot2d, launches, e->post_of[i] >= 0 ? &g.ops[e->post_of[i]] : nullptr,
                                   &e->opnd[2 * (size_t)i]);
    if (!why.empty()) return why;
  }
  const GValue& r = g.vals[g.ret];
  if (bind.loss_out) {
    convert(st, ptr_of(*e, g.ret), r.dt, bind.loss_out, DT_F32, 1);
    if (launches) *launches += 1;
  }
  if (bind.backward && bind.grads) {
    for (int i = 0; i < e->n_params; ++i) {
      const GValue& p = g.vals[g.args[i]];
      float* dst = bind.grads + e->param_offsets[i];
      const int gv = g.grad_of_arg[i];
      if (gv < 0) { if (cudaMemsetAsync(dst, 0, (size_t)p.numel * 4, st) != cudaSuccess) return "memset failed"; continue; }
      convert(st, ptr_of(*e, gv), g.vals[gv].dt, dst, DT_F32, p.numel);
      if (launches) *launches += 1;
    }
  }
  LAUNCH_CHECK();
  return "";
}

}  // namespace

std::string graph_exec_run(GraphExec* e, cudaStream_t st, const GraphBind& bind,
                           const std::function<int(int, const GemmArgs&)>& dot2d, long long* launches) {
  const Graph& g = e->g;
  const int n_args = (int)g.args.size();
  if ((int)bind.data.size() != n_args - e->n_params) return "wrong number of data inputs";
  for (int i = 0; i < n_args; ++i) {
    const int v = g.args[i];
    if (i < e->n_params) e->ext[v] = (const char*)bind.params + (size_t)e->param_offsets[i] * dtype_size(g.vals[v].dt);
    else e->ext[v] = bind.data[i - e->n_params];
  }
  // Replay: the program is a fixed list of launches on fixed addresses once the bindings are known, and its kernels are
  // small, so a run is launch-bound; from the second run with the same bindings on it is one CUDA graph launch.
  // PCPB_GRAPH_CAPTURE=0 keeps plain launches.
  static const bool allow = [] { const char* v = getenv("PCPB_GRAPH_CAPTURE"); return !(v && v[0] == '0'); }();
  std::vector<unsigned long long> key = {(unsigned long long)(uintptr_t)bind.params, (unsigned long long)(uintptr_t)bind.grads,
                                         (unsigned long long)(uintptr_t)bind.loss_out, (unsigned long long)float_bits(bind.seed),
                                         bind.backward ? 1ull : 0ull};
  for (const void* d : bind.data) key.push_back((unsigned long long)(uintptr_t)d);
  if (allow) {
    auto hit = e->captured.find(key);
    if (hit != e->captured.end()) {
      if (cudaGraphLaunch(hit->second.exec, st) != cudaSuccess) return "launch of the captured program failed";
      if (launches) *launches += hit->second.launches;
      return "";
    }
  }
  bool capture = false;
  if (allow) {
    if (e->seen.size() > 64) e->seen.clear();
    capture = (e->seen[key]++ >= 1);
    if (capture && cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); capture = false; }
  }
  long long n_launch = 0;
  const std::string why = enqueue_run(e, st, bind, dot2d, &n_launch);
  if (launches) *launches += n_launch;
  if (!capture) return why;
  cudaGraph_t graph = nullptr;
  const cudaError_t ce = cudaStreamEndCapture(st, &graph);
  if (!why.empty() || ce != cudaSuccess || !graph) {
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    if (!why.empty()) return why;
    // the capture did not work out: run this time with plain launches and stop trying for these bindings
    e->seen[key] = -1000000;
    return enqueue_run(e, st, bind, dot2d, nullptr);
  }
  cudaGraphExec_t exec = nullptr;
  const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (ie != cudaSuccess || !exec) {
    cudaGetLastError();
    e->seen[key] = -1000000;
    return enqueue_run(e, st, bind, dot2d, nullptr);
  }
  if (e->captured.size() >= 4) {
    for (auto& c : e->captured) cudaGraphExecDestroy(c.second.exec);
    e->captured.clear();
  }
  e->captured[key] = GraphExec::Captured{exec, n_launch};
  if (cudaGraphLaunch(exec, st) != cudaSuccess) return "launch of the captured program failed";
  return "";
}

std::string graph_exec_plan_text(const Graph& g, int n_params, const std::vector<int64_t>& param_offsets, std::string* text) {
  GraphExec* e = nullptr;
  const std::string why = graph_exec_create(g, n_params, param_offsets, nullptr, &e, true);
  if (!why.empty()) return why;
  char buf[256];
  std::string s;
  snprintf(buf, sizeof buf, "plan arena=%zu const=%zu\n", e->arena_bytes, e->const_bytes);
  s += buf;
  for (size_t v = 0; v < g.vals.size(); ++v) {
    snprintf(buf, sizeof buf, "pv %zu root=%d where=%d off=%lld bytes=%zu placed_at=%lld freed_after=%lld\n", v, e->root[v], (int)e->where[e->root[v]],
             e->off[e->root[v]], round256((size_t)g.vals[e->root[v]].numel * dtype_size(g.vals[e->root[v]].dt)), e->placed_at[e->root[v]],
             e->freed_after[e->root[v]]);
    s += buf;
  }
  for (size_t i = 0; i < g.ops.size(); ++i) {
    const GraphExec::OperandSrc &a = e->opnd[2 * i], &b = e->opnd[2 * i + 1];
    snprintf(buf, sizeof buf, "po %zu need=%d fwd=%d const=%d skip=%d absorbed=%d post=%d oa=%d:%d ob=%d:%d\n", i, (int)e->need_all[i],
             i < e->need_fwd.size() ? (int)e->need_fwd[i] : 0, (int)e->is_const_op[i], (int)e->skip[i], (int)e->absorbed[i], e->post_of[i], a.mode, a.src,
             b.mode, b.src);
    s += buf;
  }
  graph_exec_destroy(e);
  *text = s;
  return "";
}

}  // namespace pcpb
