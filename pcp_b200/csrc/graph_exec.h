// Runs a tensor program of the general StableHLO front end (graph.h) on the GPU: one kernel per op, all intermediate
// values in one arena whose layout is planned when the artefact is loaded (no allocation while a step runs).
#pragma once
#include <cuda_runtime.h>

#include <functional>
#include <string>
#include <vector>

#include "graph.h"
#include "kernels.h"

namespace pcpb {

struct GraphExec;

struct GraphBind {
  const void* params = nullptr;            // flat parameter buffer in the model dtype; argument i at param_offsets[i] elements
  std::vector<const void*> data;           // the remaining @main arguments (ids, targets), device pointers
  float seed = 1.f;                        // d(result)
  float* grads = nullptr;                  // f32, flat, same offsets (written when backward)
  float* loss_out = nullptr;               // f32 scalar
  bool backward = true;
};

// Plans the program (constant folding, dead-op elimination, liveness, arena offsets), checks that every op has a
// kernel, allocates the arenas and evaluates the constant part once.  Returns "" or the reason.
// plan_only: stop after the planning (no device is touched): for graph_exec_plan_text.
std::string graph_exec_create(const Graph& g, int n_params, const std::vector<int64_t>& param_offsets, cudaStream_t st,
                              GraphExec** out, bool plan_only = false);
// The plan as text, without a device: one line per value (its storage: which value's buffer it shares, arena, offset,
// bytes, the ops that define and release it) and per op (needed, constant, dropped guard, absorbed broadcast, fused
// guard, operand modes).  The CPU tests check the plan's invariants from it.
std::string graph_exec_plan_text(const Graph& g, int n_params, const std::vector<int64_t>& param_offsets, std::string* text);
void graph_exec_destroy(GraphExec* e);
size_t graph_exec_arena_bytes(const GraphExec* e);
// dot2d(element type, product): hook for un-batched f32 / bf16 products (the caller's GEMM dispatch, tensor cores when
// the shape qualifies); returns 0 when it launched the product, 1 to leave it to the general kernel, anything else on
// failure.  launches: incremented per kernel launch.  Returns "" or the reason.
std::string graph_exec_run(GraphExec* e, cudaStream_t st, const GraphBind& bind,
                           const std::function<int(int, const GemmArgs&)>& dot2d, long long* launches);

}  // namespace pcpb
