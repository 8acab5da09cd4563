// dense_mma.cu -- bfloat16 tensor-core tiles for the dense matmul (dense_mm.cu picks this path first and falls back on PIB_ERR_UNSUPP).
#include "hybrid.cuh"

int pib_dense_mm_tc(const pib_mm & a, cudaStream_t st) {
    (void) a; (void) st;
    return PIB_ERR_UNSUPP;
}
