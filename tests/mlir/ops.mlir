func.func @unpack_only(%arg0: tensor<4096x2048xi8>) -> tensor<4096x4096xi8> {
  %0 = qf.unpack %arg0 : tensor<4096x2048xi8> -> tensor<4096x4096xi8>
  return %0 : tensor<4096x4096xi8>
}

func.func @dequant_symmetric(%input: tensor<64x64xi8>, %scale: tensor<f16>) -> tensor<64x64xf16> {
  %zp = arith.constant dense<0> : tensor<i8>
  %output = qf.dequant %input, %scale, %zp :
      tensor<64x64xi8>, tensor<f16>, tensor<i8> -> tensor<64x64xf16>
  return %output : tensor<64x64xf16>
}

func.func @dequant_asymmetric(%input: tensor<64x64xi8>, %scale: tensor<f16>) -> tensor<64x64xf16> {
  %zp = arith.constant dense<8> : tensor<i8>
  %output = qf.dequant %input, %scale, %zp {group_size = 128 : i64} :
      tensor<64x64xi8>, tensor<f16>, tensor<i8> -> tensor<64x64xf16>
  return %output : tensor<64x64xf16>
}
