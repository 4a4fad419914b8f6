# Emitted by the reference project's cutile translator (imported unmodified from the reference tree)
# for tests/data/attention_f16_1x32x4096x128.mlir; written by tests/golden/make_reference_translations.py.
# Not product code: the benchmark launches it as the reference's own GPU path.
import cuda.tile as ct

@ct.kernel
def attention_f16(arr_0, arr_1, arr_2, arr_3):
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
    bid_m = ct.bid(0)
    bid_h = ct.bid(1)
    bid_b = ct.bid(2)
    v_15 = bid_m * c_10
    load_16 = ct.load(arr_0, (c_4, bid_h, v_15 // 128, c_4 // 128), (1, 1, 128, 128), order=(0, 1, 2, 3))
    tile_17 = ct.reshape(load_16, (128, 128))
    tile_18 = ct.full((128,), c_13, dtype=ct.float32)
    tile_19 = ct.full((128,), c_12, dtype=ct.float32)
    tile_20 = ct.full((128, 128), c_12, dtype=ct.float32)
    acc_21 = tile_19
    acc_22 = tile_20
    acc_23 = tile_18
    for j_24 in range(c_4, c_9, c_5):
        v_25 = j_24 * c_11
        load_26 = ct.load(arr_1, (c_4, bid_h, c_4 // 128, v_25 // 64), (1, 1, 128, 64), order=(0, 1, 3, 2))
        tile_27 = ct.reshape(load_26, (128, 64))
        tile_28 = ct.mma(tile_17, tile_27, ct.full((128, 64), 0, dtype=ct.float32))
        tile_29 = ct.full((128, 64), c_14, dtype=ct.float32)
        v_30 = tile_28 * tile_29
        red_31 = ct.max(v_30, 1, keepdims=False)
        v_32 = ct.maximum(acc_23, red_31)
        bcast_33 = ct.broadcast_to(ct.expand_dims(v_32, axis=1), (128, 64))
        v_34 = v_30 - bcast_33
        v_35 = ct.exp2(v_34)
        red_36 = ct.sum(v_35, 1, keepdims=False)
        v_37 = acc_23 - v_32
        v_38 = ct.exp2(v_37)
        v_39 = acc_21 * v_38
        v_40 = v_39 + red_36
        v_41 = ct.astype(v_35, ct.float16)
        load_42 = ct.load(arr_2, (c_4, bid_h, v_25 // 64, c_4 // 128), (1, 1, 64, 128), order=(0, 1, 2, 3))
        tile_43 = ct.reshape(load_42, (64, 128))
        tile_44 = ct.mma(v_41, tile_43, ct.full((128, 128), 0, dtype=ct.float32))
        bcast_45 = ct.broadcast_to(ct.expand_dims(v_38, axis=1), (128, 128))
        v_46 = acc_22 * bcast_45
        v_47 = v_46 + tile_44
        acc_21 = v_40
        acc_22 = v_47
        acc_23 = v_32
    bcast_48 = ct.broadcast_to(ct.expand_dims(acc_21, axis=1), (128, 128))
    v_49 = acc_22 / bcast_48
    v_50 = ct.astype(v_49, ct.float16)
    ct.store(arr_3, (c_4, bid_h, v_15 // 128, c_4 // 128), ct.reshape(v_50, (1, 1, 128, 128)))
