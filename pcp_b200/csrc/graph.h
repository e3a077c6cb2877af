// General StableHLO front end: an op-by-op program for graphs the family recogniser does not know.
//
// The reference trains ANY exported forward graph: its AD engine walks the StableHLO ops in reverse and emits a gradient
// graph from per-op VJP rules (src/autodiff/engine.zig:196-348, rules src/autodiff/vjp_rules.zig), which IREE then
// compiles.  This is the same idea without a compiler: graph_parse reads the "pretty" StableHLO text of @main into a
// small tensor program, graph_add_gradients appends the gradient program (same traversal, same rules incl. the +1e-4
// terms, and the finite guard + clamp on every adjoint edge, engine.zig:604-702), and graph_exec.cu runs the program
// with one CUDA kernel per op out of a statically planned arena.  The fused kernels of the two recognised families stay
// the fast path; this is what keeps other graphs trainable.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

namespace pcpb {

enum GKind : int {
  G_CONST_SPLAT = 0,   // fval / ival, element type of the result
  G_CONST_DATA,        // data: the elements, little endian
  G_IOTA,              // a = {dim}
  G_UNARY,             // sub: GUnary
  G_BINARY,            // sub: GBinary
  G_COMPARE,           // sub: GCmp; result i1
  G_SELECT,            // in = pred, on_true, on_false
  G_CONVERT,
  G_RESHAPE,
  G_TRANSPOSE,         // a = permutation (result dim k = operand dim a[k])
  G_BCAST,             // a = dims (operand dim i -> result dim a[i])
  G_SLICE,             // a = start, b = limit, c = stride
  G_CONCAT,            // a = {dim}
  G_REDUCE,            // sub: GRed, a = dims; in = operand, init
  G_DOT,               // a, b = batching dims (lhs, rhs); c, d = contracting dims (lhs, rhs)
  G_GATHER_ROWS,       // in = operand [R, ...], indices; result row r = operand[clamp(indices[r])]
  G_GATHER2,           // in = operand [R, C], indices [..., 2]; result i = operand[clamp(i0), clamp(i1)]
  // produced by the gradient rules only
  G_PAD,               // VJP of slice: zeros of the result shape with the operand at a : b : c
  G_SCATTER_ROWS,      // VJP of G_GATHER_ROWS: in = g, indices; zeros of the result shape, rows of g added at the indices
  G_SCATTER2,          // VJP of G_GATHER2
  G_GUARD_CLAMP,       // adjoint edge: non-finite -> 0, then (sub = 1) clamp to [lo, hi] in f32
  G_SEED,              // d(result): bound when the program runs
};
enum GUnary : int { U_RSQRT = 0, U_SQRT, U_EXP, U_LOG, U_TANH, U_LOGISTIC, U_NEG, U_CEIL, U_FLOOR, U_SIN, U_COS, U_ABS };
enum GBinary : int { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_POW, B_MAX, B_MIN, B_AND, B_OR };
enum GCmp : int { C_EQ = 0, C_NE, C_GE, C_GT, C_LE, C_LT };
enum GRed : int { R_ADD = 0, R_MAX };

struct GValue {
  std::vector<int64_t> shape;
  int dt = 0;                       // DT_* of common.cuh
  int64_t numel = 1;
  int op = -1;                      // producing op, -1 for a function argument
  std::string name;                 // SSA name in the text (arguments and forward values), "" for gradient values
};

struct GOp {
  int kind = 0, sub = 0;
  std::vector<int> in;
  int out = -1;
  std::vector<int64_t> a, b, c, d;
  double fval = 0.0;
  long long ival = 0;
  float lo = 0.f, hi = 0.f;
  std::vector<uint8_t> data;
};

struct Graph {
  std::vector<GValue> vals;
  std::vector<GOp> ops;
  std::vector<int> args;            // values of the @main arguments, in order
  int ret = -1;                     // the returned value
  int n_forward_ops = 0;            // ops [0, n_forward_ops) are the forward graph
  int seed = -1;                    // G_SEED value (after graph_add_gradients)
  std::vector<int> grad_of_arg;     // per argument: the value of its adjoint, -1 if it has none
};

// Both return "" on success, else what was not understood.  sanitize: apply the reference's stability patches to the
// forward graph as DiLoCo.init does before compiling (src/algorithms/diloco.zig:158-177, src/compiler/sanitizer.zig).
std::string graph_parse(const char* text, size_t n, bool sanitize, Graph* g);
// Appends the gradient program for the first n_params arguments (float tensors).  clamp = 0 leaves the clamp out.
std::string graph_add_gradients(Graph* g, int n_params, int clamp, float lo, float hi);
// One line per value and op (the format tests/graph_program.py reads).
std::string graph_dump(const Graph& g);

}  // namespace pcpb
