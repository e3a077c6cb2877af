"""CPU oracle for the PCP training hot path.  TEST INFRASTRUCTURE ONLY.

A torch-CPU restatement of the reference's algorithm for the path
forward -> reverse-AD backward -> AdamW inner step -> DiLoCo/Nesterov outer
step.  It is the checker that the CUDA library's results are compared with;
nothing in the shipped package imports it.  Only the test-suite, the smoke
entry point and the benchmark's cpu-baseline leg may import this package.

Parity status: the reference executes this path through IREE v3.9.0 (compiler
+ runtime, not part of the reference tree and not installable offline), so the
oracle cannot be compared with an execution of the reference itself: "parity
unpinned" at the IREE boundary.  It IS pinned against every closed-form
known-answer test the reference's own test executables hold for the path
(src/examples/isolated_vjp_tests.zig, src/examples/mlir_optimizer_test.zig,
src/examples/cpu_pipeline_test.zig) and against the forward-loss value recorded
in test/nanochat/test_generate_nanochat_mlir_forward_loss.py where inputs are
reproducible.

Modules
  stablehlo.py  parser + evaluator for the StableHLO text subset the reference's
                model exports use (models/*.mlir)
  sanitizer.py  src/compiler/sanitizer.zig restated (text patches)
  autodiff.py   src/autodiff/engine.zig + vjp_rules.zig restated (eager tape)
  optim.py      src/optimizers/adam_mlir.zig, src/optimizers/nesterov.zig
  loader.py     src/data/loader.zig batchers (FIFO: exact; random: unpinned PRNG)
  worker.py     src/nodes/workers/worker.zig inner loop +
                src/algorithms/diloco.zig outer step
"""
