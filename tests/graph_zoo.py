"""A hand-written forward graph that uses the ops and op forms the model exporters do not: sine / cosine, logistic,
sqrt / abs / floor / minimum (no gradient rule: they stop the gradient), strided slices, a three-way concatenate, a
rank-3 transpose, a batched dot_general, a maximum-reduction over a middle dimension, an add-reduction over two leading
dimensions, a broadcast into non-adjacent dimensions, i32 and f32 converts of the integer inputs, compare + select,
power, divide, rsqrt, tanh.  Test infrastructure for the general front end (CPU and GPU tests)."""

ZOO_PARAM_SHAPES = [(8, 6), (6, 6), (6,)]
ZOO_BATCH, ZOO_BLOCK, ZOO_VOCAB = 2, 4, 8

ZOO_MLIR = """module {
  func.func @main(%arg0: tensor<8x6xf32>, %arg1: tensor<6x6xf32>, %arg2: tensor<6xf32>, %arg3: tensor<2x4xi64>, %arg4: tensor<2x4xi64>) -> tensor<f32> {
    %cst = stablehlo.constant dense<0xFF800000> : tensor<f32>
    %cst_0 = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %cst_1 = stablehlo.constant dense<2.000000e+00> : tensor<2x4xf32>
    %cst_2 = stablehlo.constant dense<5.000000e-01> : tensor<2x4xf32>
    %cst_3 = stablehlo.constant dense<1.000000e+00> : tensor<2x4xf32>
    %0 = "stablehlo.gather"(%arg0, %arg3) <{dimension_numbers = #stablehlo.gather<offset_dims = [2], collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, slice_sizes = array<i64: 1, 6>}> : (tensor<8x6xf32>, tensor<2x4xi64>) -> tensor<2x4x6xf32>
    %1 = stablehlo.sine %0 : tensor<2x4x6xf32>
    %2 = stablehlo.cosine %0 : tensor<2x4x6xf32>
    %3 = stablehlo.multiply %1, %2 : tensor<2x4x6xf32>
    %4 = stablehlo.reshape %3 : (tensor<2x4x6xf32>) -> tensor<8x6xf32>
    %5 = stablehlo.transpose %arg1, dims = [1, 0] : (tensor<6x6xf32>) -> tensor<6x6xf32>
    %6 = stablehlo.dot_general %4, %5, contracting_dims = [1] x [0] : (tensor<8x6xf32>, tensor<6x6xf32>) -> tensor<8x6xf32>
    %7 = stablehlo.broadcast_in_dim %arg2, dims = [1] : (tensor<6xf32>) -> tensor<8x6xf32>
    %8 = stablehlo.add %6, %7 : tensor<8x6xf32>
    %9 = stablehlo.logistic %8 : tensor<8x6xf32>
    %10 = stablehlo.reshape %9 : (tensor<8x6xf32>) -> tensor<2x4x6xf32>
    %11 = stablehlo.slice %10 [0:2, 0:4, 0:6:2] : (tensor<2x4x6xf32>) -> tensor<2x4x3xf32>
    %12 = stablehlo.slice %10 [0:2, 0:4, 1:6:2] : (tensor<2x4x6xf32>) -> tensor<2x4x3xf32>
    %13 = stablehlo.negate %12 : tensor<2x4x3xf32>
    %14 = stablehlo.concatenate %13, %11, %12, dim = 2 : (tensor<2x4x3xf32>, tensor<2x4x3xf32>, tensor<2x4x3xf32>) -> tensor<2x4x9xf32>
    %15 = stablehlo.transpose %14, dims = [0, 2, 1] : (tensor<2x4x9xf32>) -> tensor<2x9x4xf32>
    %16 = stablehlo.dot_general %14, %15, batching_dims = [0] x [0], contracting_dims = [2] x [1] : (tensor<2x4x9xf32>, tensor<2x9x4xf32>) -> tensor<2x4x4xf32>
    %17 = stablehlo.reduce(%16 init: %cst) applies stablehlo.maximum across dimensions = [1] : (tensor<2x4x4xf32>, tensor<f32>) -> tensor<2x4xf32>
    %18 = stablehlo.broadcast_in_dim %17, dims = [0, 2] : (tensor<2x4xf32>) -> tensor<2x4x4xf32>
    %19 = stablehlo.subtract %16, %18 : tensor<2x4x4xf32>
    %20 = stablehlo.exponential %19 : tensor<2x4x4xf32>
    %21 = stablehlo.reduce(%20 init: %cst_0) applies stablehlo.add across dimensions = [1] : (tensor<2x4x4xf32>, tensor<f32>) -> tensor<2x4xf32>
    %22 = stablehlo.log %21 : tensor<2x4xf32>
    %23 = stablehlo.convert %arg4 : (tensor<2x4xi64>) -> tensor<2x4xi32>
    %24 = stablehlo.convert %23 : (tensor<2x4xi32>) -> tensor<2x4xf32>
    %25 = stablehlo.multiply %24, %cst_2 : tensor<2x4xf32>
    %26 = stablehlo.floor %25 : tensor<2x4xf32>
    %27 = stablehlo.add %26, %cst_3 : tensor<2x4xf32>
    %28 = stablehlo.divide %22, %27 : tensor<2x4xf32>
    %29 = stablehlo.power %28, %cst_1 : tensor<2x4xf32>
    %30 = stablehlo.add %29, %cst_3 : tensor<2x4xf32>
    %31 = stablehlo.rsqrt %30 : tensor<2x4xf32>
    %32 = stablehlo.tanh %17 : tensor<2x4xf32>
    %33 = stablehlo.compare  GT, %32, %31,  FLOAT : (tensor<2x4xf32>, tensor<2x4xf32>) -> tensor<2x4xi1>
    %34 = stablehlo.select %33, %32, %31 : tensor<2x4xi1>, tensor<2x4xf32>
    %35 = stablehlo.sqrt %21 : tensor<2x4xf32>
    %36 = stablehlo.abs %22 : tensor<2x4xf32>
    %37 = stablehlo.minimum %35, %36 : tensor<2x4xf32>
    %38 = stablehlo.maximum %28, %cst_2 : tensor<2x4xf32>
    %39 = stablehlo.add %34, %37 : tensor<2x4xf32>
    %40 = stablehlo.add %39, %38 : tensor<2x4xf32>
    %41 = stablehlo.reduce(%40 init: %cst_0) applies stablehlo.add across dimensions = [0, 1] : (tensor<2x4xf32>, tensor<f32>) -> tensor<f32>
    return %41 : tensor<f32>
  }
}
"""
