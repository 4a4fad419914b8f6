from neptune_mlir import runtime as nb200

def selective_scan_bf16(ptr_0, ptr_1, ptr_2, ptr_3, ptr_4, ptr_5, ptr_6, ptr_7):
    nb200.selective_scan(ptr_0, ptr_1, ptr_2, ptr_3, ptr_4, ptr_5, ptr_6, ptr_7, B=8, Dm=4096, L=4096, N=16, dtype='bf16')
