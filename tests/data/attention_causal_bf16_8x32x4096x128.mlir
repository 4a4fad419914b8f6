#shared = #htile.encoding<placement = shared>
#local = #htile.encoding<placement = local>

module {
  func.func @attention_causal_bf16(%q: memref<8x32x4096x128xbf16>, %k: memref<8x32x4096x128xbf16>, %v: memref<8x32x4096x128xbf16>, %out: memref<8x32x4096x128xbf16>) {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %grid_m = arith.constant 32 : index
    %heads = arith.constant 32 : index
    %batch = arith.constant 8 : index
    %kv_steps = arith.constant 64 : index
    %bm = arith.constant 128 : index
    %bn = arith.constant 64 : index
    %zero = arith.constant 0.0 : f32
    %lowest = arith.constant -3.40282347E+38 : f32
    %c = arith.constant 0.127517431974411 : f32
    gpu.launch blocks(%bx, %by, %bz) in (%gx = %grid_m, %gy = %heads, %gz = %batch)
               threads(%tx, %ty, %tz) in (%sx = %bm, %sy = %c1, %sz = %c1) {
      %i0 = arith.muli %bx, %bm : index
      %q_tile = htile.load %q[%bz, %by, %i0, %c0] : memref<8x32x4096x128xbf16> -> tensor<128x128xbf16, #shared>
      %m_init = htile.full %lowest : f32 -> tensor<128xf32, #local>
      %l_init = htile.full %zero : f32 -> tensor<128xf32, #local>
      %acc_init = htile.full %zero : f32 -> tensor<128x128xf32, #local>
      %i1 = arith.addi %i0, %bm : index
      %rows = htile.arange %i0 to %i1 : tensor<128xindex, #local>
      %rows_e = tensor.empty() : tensor<128x64xindex, #local>
      %rows_b = linalg.broadcast ins(%rows : tensor<128xindex, #local>) outs(%rows_e : tensor<128x64xindex, #local>) dimensions = [1]
      %fill = htile.full %lowest : f32 -> tensor<128x64xf32, #local>
      %l_out, %acc_out, %m_out = scf.for %j = %c0 to %kv_steps step %c1
          iter_args(%l = %l_init, %acc = %acc_init, %m = %m_init)
          -> (tensor<128xf32, #local>, tensor<128x128xf32, #local>, tensor<128xf32, #local>) {
        %j0 = arith.muli %j, %bn : index
        %k_tile = htile.load %k[%bz, %by, %j0, %c0] : memref<8x32x4096x128xbf16> -> tensor<64x128xbf16, #shared>
        %qk = htile.dot %q_tile, %k_tile {transpose_b, warp_policy = "full_row"} : tensor<128x128xbf16, #shared>, tensor<64x128xbf16, #shared> -> tensor<128x64xf32, #local>
        %c_tile = htile.full %c : f32 -> tensor<128x64xf32, #local>
        %s_raw = arith.mulf %qk, %c_tile : tensor<128x64xf32, #local>
        %j1 = arith.addi %j0, %bn : index
        %cols = htile.arange %j0 to %j1 : tensor<64xindex, #local>
        %cols_e = tensor.empty() : tensor<128x64xindex, #local>
        %cols_b = linalg.broadcast ins(%cols : tensor<64xindex, #local>) outs(%cols_e : tensor<128x64xindex, #local>) dimensions = [0]
        %visible = arith.cmpi sge, %rows_b, %cols_b : tensor<128x64xindex, #local>
        %s = arith.select %visible, %s_raw, %fill : tensor<128x64xi1, #local>, tensor<128x64xf32, #local>
        %s_max = htile.reduce %s axis 1 kind "max" : tensor<128x64xf32, #local> -> tensor<128xf32, #local>
        %m_new = arith.maximumf %m, %s_max : tensor<128xf32, #local>
        %m_new_e = tensor.empty() : tensor<128x64xf32, #local>
        %m_new_b = linalg.broadcast ins(%m_new : tensor<128xf32, #local>) outs(%m_new_e : tensor<128x64xf32, #local>) dimensions = [1]
        %shifted = arith.subf %s, %m_new_b : tensor<128x64xf32, #local>
        %p = math.exp2 %shifted : tensor<128x64xf32, #local>
        %p_sum = htile.reduce %p axis 1 kind "sum" : tensor<128x64xf32, #local> -> tensor<128xf32, #local>
        %dm = arith.subf %m, %m_new : tensor<128xf32, #local>
        %alpha = math.exp2 %dm : tensor<128xf32, #local>
        %l_scaled = arith.mulf %l, %alpha : tensor<128xf32, #local>
        %l_new = arith.addf %l_scaled, %p_sum : tensor<128xf32, #local>
        %p_lo = arith.truncf %p : tensor<128x64xf32, #local> to tensor<128x64xbf16, #local>
        %v_tile = htile.load %v[%bz, %by, %j0, %c0] : memref<8x32x4096x128xbf16> -> tensor<64x128xbf16, #shared>
        %pv = htile.dot %p_lo, %v_tile {warp_policy = "full_row"} : tensor<128x64xbf16, #local>, tensor<64x128xbf16, #shared> -> tensor<128x128xf32, #local>
        %alpha_e = tensor.empty() : tensor<128x128xf32, #local>
        %alpha_b = linalg.broadcast ins(%alpha : tensor<128xf32, #local>) outs(%alpha_e : tensor<128x128xf32, #local>) dimensions = [1]
        %acc_scaled = arith.mulf %acc, %alpha_b : tensor<128x128xf32, #local>
        %acc_new = arith.addf %acc_scaled, %pv : tensor<128x128xf32, #local>
        scf.yield %l_new, %acc_new, %m_new : tensor<128xf32, #local>, tensor<128x128xf32, #local>, tensor<128xf32, #local>
      } {htile.pipeline_stages = 2 : i32}
      %l_e = tensor.empty() : tensor<128x128xf32, #local>
      %l_b = linalg.broadcast ins(%l_out : tensor<128xf32, #local>) outs(%l_e : tensor<128x128xf32, #local>) dimensions = [1]
      %o = arith.divf %acc_out, %l_b : tensor<128x128xf32, #local>
      %o_lo = arith.truncf %o : tensor<128x128xf32, #local> to tensor<128x128xbf16, #local>
      htile.store %o_lo, %out[%bz, %by, %i0, %c0] : tensor<128x128xbf16, #local>, memref<8x32x4096x128xbf16>
      gpu.terminator
    }
    return
  }
}
