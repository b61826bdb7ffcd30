// Optional: stand-ins for the three cuBLAS symbols the reference's model code still calls
// (cublasCreate / cublasSetMathMode / cublasDestroy at llama2-mistral/src/model.cpp:11,372,
// 404-405,709) so that its `train` binary links and runs with no libcublas at all.  The
// handle they hand out is a token; the GEMM overloads ignore it.
#include <cstdlib>

struct cublasContext { int token; };
typedef struct cublasContext* cublasHandle_t;

extern "C" {
int cublasCreate_v2(cublasHandle_t* handle) {
    if (!handle) return 7;  // CUBLAS_STATUS_INVALID_VALUE
    *handle = static_cast<cublasHandle_t>(malloc(sizeof(cublasContext)));
    if (!*handle) return 3;  // CUBLAS_STATUS_ALLOC_FAILED
    (*handle)->token = 0xB200;
    return 0;
}
int cublasDestroy_v2(cublasHandle_t handle) {
    free(handle);
    return 0;
}
int cublasSetMathMode(cublasHandle_t, int) { return 0; }
}
