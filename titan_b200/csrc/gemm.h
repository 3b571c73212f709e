// Epilogues shared by the matrix-product kernels (see gemm_simt.cu for their meaning).
#pragma once
#define TB_EPI_STORE 0
#define TB_EPI_F32 1
#define TB_EPI_ADD 2
#define TB_EPI_SWIGLU 3
