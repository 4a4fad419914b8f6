from neptune_mlir import runtime as nb200

def decode_splitk_htile_bf16(ptr_0, ptr_1, ptr_2, ptr_3, ptr_4):
    nb200.decode_splitk(ptr_0, ptr_1, ptr_2, ptr_3, ptr_4, B=64, Hq=32, Hkv=8, L=32768, D=128, n_splits=16, dtype='bf16', scale_log2=0.127517431974411)
