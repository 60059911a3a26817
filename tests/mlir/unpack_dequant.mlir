func.func @unpack_only(%arg0: tensor<4096x2048xi8>) -> tensor<4096x4096xi8> {
  %0 = qf.unpack %arg0 : tensor<4096x2048xi8> -> tensor<4096x4096xi8>
  return %0 : tensor<4096x4096xi8>
}

func.func @unpack_dequant(%w: tensor<256x64xi8>, %scale: tensor<f16>, %zp: tensor<i8>) -> tensor<256x128xf16> {
  %u = qf.unpack %w : tensor<256x64xi8> -> tensor<256x128xi8>
  %d = qf.dequant %u, %scale, %zp {group_size = 128 : i64} : tensor<256x128xi8>, tensor<f16>, tensor<i8> -> tensor<256x128xf16>
  return %d : tensor<256x128xf16>
}

func.func @fold_subf_zero(%x: f16) -> f16 {
  %zero = arith.constant 0.0 : f16
  %result = arith.subf %x, %zero : f16
  return %result : f16
}
