from neptune_mlir import runtime as nb200

def attention_f16(ptr_0, ptr_1, ptr_2, ptr_3):
    nb200.attn_fwd(ptr_0, ptr_1, ptr_2, ptr_3, shape=(1, 32, 4096, 128), kv_len=4096, dtype='f16', scale_log2=0.127517431974411, causal=False)
