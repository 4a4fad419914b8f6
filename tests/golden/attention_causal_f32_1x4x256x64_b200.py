from neptune_mlir import runtime as nb200

def attention_causal_f32(ptr_0, ptr_1, ptr_2, ptr_3):
    nb200.attn_fwd(ptr_0, ptr_1, ptr_2, ptr_3, shape=(1, 4, 256, 64), kv_len=256, dtype='f32', scale_log2=0.1803368777036667, causal=True)
