module {
  func.func @decode_splitk_bf16(%q: memref<64x32x128xbf16>, %k: memref<64x8x32768x128xbf16>, %v: memref<64x8x32768x128xbf16>, %partials: memref<64x32x16x130xf32>, %out: memref<64x32x128xbf16>) attributes {htile.operator = "decode_splitk", n_splits = 16 : i64, scale = 0.0883883461356163 : f32} {
    return
  }
}
