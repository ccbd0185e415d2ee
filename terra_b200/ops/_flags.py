"""Epilogue flag bits of the tcgen05 GEMM kernel (mirrors csrc/gemm_sm100.cuh)."""
EPI_BIAS = 1 << 0
EPI_GELU = 1 << 1
EPI_SAVE_PRE = 1 << 2
EPI_RESIDUAL = 1 << 3
EPI_MUL_DGELU = 1 << 4
EPI_OUT_F32 = 1 << 5
EPI_ATOMIC = 1 << 6
EPI_ROW_CONV = 1 << 7
EPI_ROW_SHUFFLE = 1 << 8
EPI_BIAS_F32 = 1 << 9
