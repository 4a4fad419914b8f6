from neptune_mlir import runtime as nb200

def ssd_chunk_scan_bf16(ptr_0, ptr_1, ptr_2, ptr_3, ptr_4, ptr_5, ptr_6):
    nb200.ssd_chunk_scan(ptr_0, ptr_1, ptr_2, ptr_3, ptr_4, ptr_5, ptr_6, B=4, L=8192, H=64, P=64, N=128, G=1, chunk=256, dtype='bf16')
