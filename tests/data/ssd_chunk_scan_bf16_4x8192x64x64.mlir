module {
  func.func @ssd_chunk_scan_bf16(%x: memref<4x8192x64x64xbf16>, %dt: memref<4x8192x64xf32>, %A: memref<64xf32>, %B: memref<4x8192x1x128xbf16>, %C: memref<4x8192x1x128xbf16>, %workspace: memref<25169152xi8>, %y: memref<4x8192x64x64xbf16>) attributes {htile.operator = "ssd_chunk_scan", chunk = 256 : i64} {
    return
  }
}
