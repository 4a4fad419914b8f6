#shared = #htile.encoding<placement = shared>
#local = #htile.encoding<placement = local>

module {
  func.func @decode_splitk_htile_bf16(%q: memref<64x32x128xbf16>, %k: memref<64x8x32768x128xbf16>, %v: memref<64x8x32768x128xbf16>, %partials: memref<64x32x16x130xf32>, %out: memref<64x32x128xbf16>) {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %splits = arith.constant 16 : index
    %kv_heads = arith.constant 8 : index
    %q_heads = arith.constant 32 : index
    %batch = arith.constant 64 : index
    %group = arith.constant 4 : index
    %split_rows = arith.constant 2048 : index
    %kv_steps = arith.constant 32 : index
    %bn = arith.constant 64 : index
    %col_m = arith.constant 128 : index
    %col_l = arith.constant 129 : index
    %threads = arith.constant 256 : index
    %zero = arith.constant 0.0 : f32
    %lowest = arith.constant -3.40282347E+38 : f32
    %c = arith.constant 0.127517431974411 : f32
    gpu.launch blocks(%bx, %by, %bz) in (%gx = %splits, %gy = %kv_heads, %gz = %batch)
               threads(%tx, %ty, %tz) in (%sx = %threads, %sy = %c1, %sz = %c1) {
      %h0 = arith.muli %by, %group : index
      %t0 = arith.muli %bx, %split_rows : index
      %q_tile = htile.load %q[%bz, %h0, %c0] : memref<64x32x128xbf16> -> tensor<4x128xbf16, #shared>
      %m_init = htile.full %lowest : f32 -> tensor<4xf32, #local>
      %l_init = htile.full %zero : f32 -> tensor<4xf32, #local>
      %acc_init = htile.full %zero : f32 -> tensor<4x128xf32, #local>
      %l_out, %acc_out, %m_out = scf.for %j = %c0 to %kv_steps step %c1
          iter_args(%l = %l_init, %acc = %acc_init, %m = %m_init)
          -> (tensor<4xf32, #local>, tensor<4x128xf32, #local>, tensor<4xf32, #local>) {
        %j0 = arith.muli %j, %bn : index
        %r0 = arith.addi %t0, %j0 : index
        %k_tile = htile.load %k[%bz, %by, %r0, %c0] : memref<64x8x32768x128xbf16> -> tensor<64x128xbf16, #shared>
        %qk = htile.dot %q_tile, %k_tile {transpose_b, warp_policy = "full_row"} : tensor<4x128xbf16, #shared>, tensor<64x128xbf16, #shared> -> tensor<4x64xf32, #local>
        %c_tile = htile.full %c : f32 -> tensor<4x64xf32, #local>
        %s = arith.mulf %qk, %c_tile : tensor<4x64xf32, #local>
        %s_max = htile.reduce %s axis 1 kind "max" : tensor<4x64xf32, #local> -> tensor<4xf32, #local>
        %m_new = arith.maximumf %m, %s_max : tensor<4xf32, #local>
        %m_new_e = tensor.empty() : tensor<4x64xf32, #local>
        %m_new_b = linalg.broadcast ins(%m_new : tensor<4xf32, #local>) outs(%m_new_e : tensor<4x64xf32, #local>) dimensions = [1]
        %shifted = arith.subf %s, %m_new_b : tensor<4x64xf32, #local>
        %p = math.exp2 %shifted : tensor<4x64xf32, #local>
        %p_sum = htile.reduce %p axis 1 kind "sum" : tensor<4x64xf32, #local> -> tensor<4xf32, #local>
        %dm = arith.subf %m, %m_new : tensor<4xf32, #local>
        %alpha = math.exp2 %dm : tensor<4xf32, #local>
        %l_scaled = arith.mulf %l, %alpha : tensor<4xf32, #local>
        %l_new = arith.addf %l_scaled, %p_sum : tensor<4xf32, #local>
        %v_tile = htile.load %v[%bz, %by, %r0, %c0] : memref<64x8x32768x128xbf16> -> tensor<64x128xbf16, #shared>
        %v_f = arith.extf %v_tile : tensor<64x128xbf16, #shared> to tensor<64x128xf32, #local>
        %pv = htile.dot %p, %v_f {warp_policy = "full_row"} : tensor<4x64xf32, #local>, tensor<64x128xf32, #local> -> tensor<4x128xf32, #local>
        %alpha_e = tensor.empty() : tensor<4x128xf32, #local>
        %alpha_b = linalg.broadcast ins(%alpha : tensor<4xf32, #local>) outs(%alpha_e : tensor<4x128xf32, #local>) dimensions = [1]
        %acc_scaled = arith.mulf %acc, %alpha_b : tensor<4x128xf32, #local>
        %acc_new = arith.addf %acc_scaled, %pv : tensor<4x128xf32, #local>
        scf.yield %l_new, %acc_new, %m_new : tensor<4xf32, #local>, tensor<4x128xf32, #local>, tensor<4xf32, #local>
      }
      %o3 = htile.unsqueeze %acc_out mask [false, true, false] : tensor<4x128xf32, #local> -> tensor<4x1x128xf32, #local>
      htile.store %o3, %partials[%bz, %h0, %bx, %c0] : tensor<4x1x128xf32, #local>, memref<64x32x16x130xf32>
      %m3 = htile.unsqueeze %m_out mask [false, true, true] : tensor<4xf32, #local> -> tensor<4x1x1xf32, #local>
      htile.store %m3, %partials[%bz, %h0, %bx, %col_m] : tensor<4x1x1xf32, #local>, memref<64x32x16x130xf32>
      %l3 = htile.unsqueeze %l_out mask [false, true, true] : tensor<4xf32, #local> -> tensor<4x1x1xf32, #local>
      htile.store %l3, %partials[%bz, %h0, %bx, %col_l] : tensor<4x1x1xf32, #local>, memref<64x32x16x130xf32>
      gpu.terminator
    }
    gpu.launch blocks(%cx, %cy, %cz) in (%hx = %q_heads, %hy = %batch, %hz = %c1)
               threads(%ux, %uy, %uz) in (%wx = %threads, %wy = %c1, %wz = %c1) {
      %o_sh = htile.load %partials[%cy, %cx, %c0, %c0] : memref<64x32x16x130xf32> -> tensor<16x128xf32, #shared>
      %ms_sh = htile.load %partials[%cy, %cx, %c0, %col_m] : memref<64x32x16x130xf32> -> tensor<16x1xf32, #shared>
      %ls_sh = htile.load %partials[%cy, %cx, %c0, %col_l] : memref<64x32x16x130xf32> -> tensor<16x1xf32, #shared>
      %o = htile.copy %o_sh : tensor<16x128xf32, #shared> -> tensor<16x128xf32, #local>
      %ms = htile.copy %ms_sh : tensor<16x1xf32, #shared> -> tensor<16x1xf32, #local>
      %ls = htile.copy %ls_sh : tensor<16x1xf32, #shared> -> tensor<16x1xf32, #local>
      %big = htile.reduce %ms axis 0 kind "max" : tensor<16x1xf32, #local> -> tensor<1xf32, #local>
      %big_e = tensor.empty() : tensor<16x1xf32, #local>
      %big_b = linalg.broadcast ins(%big : tensor<1xf32, #local>) outs(%big_e : tensor<16x1xf32, #local>) dimensions = [0]
      %dms = arith.subf %ms, %big_b : tensor<16x1xf32, #local>
      %w = math.exp2 %dms : tensor<16x1xf32, #local>
      %wl = arith.mulf %w, %ls : tensor<16x1xf32, #local>
      %den = htile.reduce %wl axis 0 kind "sum" : tensor<16x1xf32, #local> -> tensor<1xf32, #local>
      %w1 = htile.reduce %w axis 1 kind "sum" : tensor<16x1xf32, #local> -> tensor<16xf32, #local>
      %w_e = tensor.empty() : tensor<16x128xf32, #local>
      %w_b = linalg.broadcast ins(%w1 : tensor<16xf32, #local>) outs(%w_e : tensor<16x128xf32, #local>) dimensions = [1]
      %wo = arith.mulf %o, %w_b : tensor<16x128xf32, #local>
      %num = htile.reduce %wo axis 0 kind "sum" : tensor<16x128xf32, #local> -> tensor<128xf32, #local>
      %num2 = htile.unsqueeze %num mask [true, false] : tensor<128xf32, #local> -> tensor<1x128xf32, #local>
      %den_e = tensor.empty() : tensor<1x128xf32, #local>
      %den_b = linalg.broadcast ins(%den : tensor<1xf32, #local>) outs(%den_e : tensor<1x128xf32, #local>) dimensions = [1]
      %res = arith.divf %num2, %den_b : tensor<1x128xf32, #local>
      %res_lo = arith.truncf %res : tensor<1x128xf32, #local> to tensor<1x128xbf16, #local>
      htile.store %res_lo, %out[%cy, %cx, %c0] : tensor<1x128xbf16, #local>, memref<64x32x128xbf16>
      gpu.terminator
    }
    return
  }
}
