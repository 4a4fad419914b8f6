# Emitted by the reference project's triton translator (imported unmodified from the reference tree)
# for tests/data/attention_f16_1x32x4096x128.mlir; written by tests/golden/make_reference_translations.py.
# Not product code: the benchmark launches it as the reference's own GPU path.
import triton
from triton import language as tl

@triton.jit
def attention_f16(ptr_0, ptr_1, ptr_2, ptr_3):
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
    pid_m = tl.program_id(0)
    pid_h = tl.program_id(1)
    pid_b = tl.program_id(2)
    v_15 = pid_m * c_10
    ptr_16 = ptr_0 + (0 + c_4 * 16777216 + pid_h * 524288)
    bp_17 = tl.make_block_ptr(base=ptr_16, shape=[4096, 128], strides=[128, 1], offsets=[v_15, c_4], block_shape=[128, 128], order=[1, 0])
    tile_18 = tl.load(bp_17, boundary_check=[0, 1])
    tile_19 = tl.full([128], c_13, tl.float32)
    tile_20 = tl.full([128], c_12, tl.float32)
    tile_21 = tl.full([128, 128], c_12, tl.float32)
    acc_22 = tile_20
    acc_23 = tile_21
    acc_24 = tile_19
    for j_25 in range(c_4, c_9, c_5):
        v_26 = j_25 * c_11
        ptr_27 = ptr_1 + (0 + c_4 * 16777216 + pid_h * 524288)
        bp_28 = tl.make_block_ptr(base=ptr_27, shape=[128, 4096], strides=[1, 128], offsets=[c_4, v_26], block_shape=[128, 64], order=[0, 1])
        tile_29 = tl.load(bp_28, boundary_check=[0, 1])
        tile_30 = tl.dot(tile_18, tile_29)
        tile_31 = tl.full([128, 64], c_14, tl.float32)
        v_32 = tile_30 * tile_31
        red_33 = tl.max(v_32, 1, keep_dims=False)
        v_34 = tl.maximum(acc_24, red_33)
        bcast_35 = v_34[:, None]
        v_36 = v_32 - bcast_35
        v_37 = tl.exp2(v_36)
        red_38 = tl.sum(v_37, 1, keep_dims=False)
        v_39 = acc_24 - v_34
        v_40 = tl.exp2(v_39)
        v_41 = acc_22 * v_40
        v_42 = v_41 + red_38
        v_43 = tl.cast(v_37, tl.float16)
        ptr_44 = ptr_2 + (0 + c_4 * 16777216 + pid_h * 524288)
        bp_45 = tl.make_block_ptr(base=ptr_44, shape=[4096, 128], strides=[128, 1], offsets=[v_26, c_4], block_shape=[64, 128], order=[1, 0])
        tile_46 = tl.load(bp_45, boundary_check=[0, 1])
        tile_47 = tl.dot(v_43, tile_46)
        bcast_48 = v_40[:, None]
        v_49 = acc_23 * bcast_48
        v_50 = v_49 + tile_47
        acc_22 = v_42
        acc_23 = v_50
        acc_24 = v_34
    bcast_51 = acc_22[:, None]
    v_52 = acc_23 / bcast_51
    v_53 = tl.cast(v_52, tl.float16)
    ptr_54 = ptr_3 + (0 + c_4 * 16777216 + pid_h * 524288)
    bp_55 = tl.make_block_ptr(base=ptr_54, shape=[4096, 128], strides=[128, 1], offsets=[v_15, c_4], block_shape=[128, 128], order=[1, 0])
    tl.store(bp_55, v_53, boundary_check=[0, 1])
