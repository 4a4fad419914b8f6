module {
  func.func @selective_scan_bf16(%u: memref<8x4096x4096xbf16>, %delta: memref<8x4096x4096xbf16>, %A: memref<4096x16xf32>, %B: memref<8x16x4096xbf16>, %C: memref<8x16x4096xbf16>, %D: memref<4096xf32>, %z: memref<8x4096x4096xbf16>, %out: memref<8x4096x4096xbf16>) attributes {htile.operator = "selective_scan"} {
    return
  }
}
