// Inputs written for this repository's boundary tests (shapes follow the kind of IR the reference's matcher sees).
func.func @gemv(%act: tensor<1x4096xf16>,
                %weight: tensor<4096x4096xi8>)
                -> tensor<1x4096xf16> {
  %cst = arith.constant 0.0 : f16
  %init = tensor.empty() : tensor<1x4096xf16>
  %filled = linalg.fill ins(%cst : f16) outs(%init : tensor<1x4096xf16>) -> tensor<1x4096xf16>
  %result = linalg.matmul {qf.scale = dense<5.000000e-01> : tensor<f16>,
                           qf.zp    = dense<8>   : tensor<i8>}
                          ins(%act, %weight : tensor<1x4096xf16>, tensor<4096x4096xi8>)
                          outs(%filled : tensor<1x4096xf16>) -> tensor<1x4096xf16>
  return %result : tensor<1x4096xf16>
}

func.func @fp16_untouched(%act: tensor<4x8xf16>, %weight: tensor<8x16xf16>) -> tensor<4x16xf16> {
  %cst = arith.constant 0.0 : f16
  %init = tensor.empty() : tensor<4x16xf16>
  %filled = linalg.fill ins(%cst : f16) outs(%init : tensor<4x16xf16>) -> tensor<4x16xf16>
  %result = linalg.matmul ins(%act, %weight : tensor<4x8xf16>, tensor<8x16xf16>)
                          outs(%filled : tensor<4x16xf16>) -> tensor<4x16xf16>
  return %result : tensor<4x16xf16>
}

func.func @int8_lhs(%act: tensor<2x256xi8>, %weight: tensor<256x512xi8>) -> tensor<2x512xf16> {
  %cst = arith.constant 0.0 : f16
  %init = tensor.empty() : tensor<2x512xf16>
  %filled = linalg.fill ins(%cst : f16) outs(%init : tensor<2x512xf16>) -> tensor<2x512xf16>
  %result = linalg.matmul ins(%act, %weight : tensor<2x256xi8>, tensor<256x512xi8>)
                          outs(%filled : tensor<2x512xf16>) -> tensor<2x512xf16>
  return %result : tensor<2x512xf16>
}
