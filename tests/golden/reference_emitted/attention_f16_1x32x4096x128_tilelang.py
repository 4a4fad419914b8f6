# Emitted by the reference project's tilelang translator (imported unmodified from the reference tree)
# for tests/data/attention_f16_1x32x4096x128.mlir; written by tests/golden/make_reference_translations.py.
# Not product code: the benchmark launches it as the reference's own GPU path.
import tilelang.language as T

@T.prim_func
def attention_f16(buf_0: T.Buffer((1, 32, 4096, 128), 'float16'), buf_1: T.Buffer((1, 32, 4096, 128), 'float16'), buf_2: T.Buffer((1, 32, 4096, 128), 'float16'), buf_3: T.Buffer((1, 32, 4096, 128), 'float16')):
    c_4 = 0
    c_5 = 1
    c_6 = 32
    c_7 = 32
    c_8 = 1
    c_9 = 64
    c_10 = 128
    c_11 = 64
    c_12 = 0.0
    c_13 = -3.4028234663852886e+38
    c_14 = 0.127517431974411
    with T.Kernel(c_6, c_7, c_8, threads=c_10) as (bx, by, bz):
        shared_15 = T.alloc_shared([128, 128], 'float16')
        frag_16 = T.alloc_fragment([128], 'float32')
        frag_17 = T.alloc_fragment([128], 'float32')
        frag_18 = T.alloc_fragment([128, 128], 'float32')
        shared_19 = T.alloc_shared([64, 128], 'float16')
        dot_20 = T.alloc_fragment([128, 64], 'float32')
        frag_21 = T.alloc_fragment([128, 64], 'float32')
        frag_22 = T.alloc_fragment([128, 64], 'float32')
        red_23 = T.alloc_fragment([128], 'float32')
        frag_24 = T.alloc_fragment([128], 'float32')
        frag_25 = T.alloc_fragment([128, 64], 'float32')
        exp_26 = T.alloc_fragment([128, 64], 'float32')
        red_27 = T.alloc_fragment([128], 'float32')
        frag_28 = T.alloc_fragment([128], 'float32')
        exp_29 = T.alloc_fragment([128], 'float32')
        frag_30 = T.alloc_fragment([128], 'float32')
        frag_31 = T.alloc_fragment([128], 'float32')
        cast_32 = T.alloc_fragment([128, 64], 'float16')
        shared_33 = T.alloc_shared([64, 128], 'float16')
        dot_34 = T.alloc_fragment([128, 128], 'float32')
        frag_35 = T.alloc_fragment([128, 128], 'float32')
        frag_36 = T.alloc_fragment([128, 128], 'float32')
        frag_37 = T.alloc_fragment([128, 128], 'float32')
        cast_38 = T.alloc_fragment([128, 128], 'float16')
        v_39 = bx * c_10
        T.copy(buf_0[c_4, by, v_39:v_39 + 128, c_4:c_4 + 128], shared_15)
        T.fill(frag_16, c_13)
        T.fill(frag_17, c_12)
        T.fill(frag_18, c_12)
        for j_40 in T.Pipelined(c_4, c_9, num_stages=2):
            v_41 = j_40 * c_11
            T.copy(buf_1[c_4, by, v_41:v_41 + 64, c_4:c_4 + 128], shared_19)
            T.gemm(shared_15, shared_19, dot_20, clear_accum=True, transpose_B=True, policy=T.GemmWarpPolicy.FullRow)
            T.fill(frag_21, c_14)
            for i0_42, i1_43 in T.Parallel(128, 64):
                frag_22[i0_42, i1_43] = dot_20[i0_42, i1_43] * frag_21[i0_42, i1_43]
            T.reduce_max(frag_22, red_23, dim=1)
            for i0_44 in T.Parallel(128):
                frag_24[i0_44] = T.max(frag_16[i0_44], red_23[i0_44])
            for i0_45, i1_46 in T.Parallel(128, 64):
                frag_25[i0_45, i1_46] = frag_22[i0_45, i1_46] - frag_24[i0_45]
            for i0_47, i1_48 in T.Parallel(128, 64):
                exp_26[i0_47, i1_48] = T.exp2(frag_25[i0_47, i1_48])
            T.reduce_sum(exp_26, red_27, dim=1)
            for i0_49 in T.Parallel(128):
                frag_28[i0_49] = frag_16[i0_49] - frag_24[i0_49]
            for i0_50 in T.Parallel(128):
                exp_29[i0_50] = T.exp2(frag_28[i0_50])
            for i0_51 in T.Parallel(128):
                frag_30[i0_51] = frag_17[i0_51] * exp_29[i0_51]
            for i0_52 in T.Parallel(128):
                frag_31[i0_52] = frag_30[i0_52] + red_27[i0_52]
            for i0_53, i1_54 in T.Parallel(128, 64):
                cast_32[i0_53, i1_54] = T.cast(exp_26[i0_53, i1_54], 'float16')
            T.copy(buf_2[c_4, by, v_41:v_41 + 64, c_4:c_4 + 128], shared_33)
            T.gemm(cast_32, shared_33, dot_34, clear_accum=True, policy=T.GemmWarpPolicy.FullRow)
            for i0_55, i1_56 in T.Parallel(128, 128):
                frag_35[i0_55, i1_56] = frag_18[i0_55, i1_56] * exp_29[i0_55]
            for i0_57, i1_58 in T.Parallel(128, 128):
                frag_36[i0_57, i1_58] = frag_35[i0_57, i1_58] + dot_34[i0_57, i1_58]
            T.copy(frag_31, frag_17)
            T.copy(frag_36, frag_18)
            T.copy(frag_24, frag_16)
        for i0_59, i1_60 in T.Parallel(128, 128):
            frag_37[i0_59, i1_60] = frag_18[i0_59, i1_60] / frag_17[i0_59]
        for i0_61, i1_62 in T.Parallel(128, 128):
            cast_38[i0_61, i1_62] = T.cast(frag_37[i0_61, i1_62], 'float16')
        T.copy(cast_38, buf_3[c_4, by, v_39:v_39 + 128, c_4:c_4 + 128])
