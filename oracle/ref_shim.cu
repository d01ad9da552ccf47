// Re-exports the reference's two host launchers with C linkage so that the
// test-suite can call the reference's own CUDA kernels through ctypes.
// TEST INFRASTRUCTURE ONLY.  The reference translation unit is compiled from
// where it lies (include path given by oracle/Makefile); no reference source
// is copied.  wrapper(): kernel.cu:3009; dequantize_wrapper(): kernel.cu:3243.
#include "kernel.cu"

extern "C" void tuna_ref_matmul(void *q, void *x, void *code, void *absmax, void *o,
                                int m, int n, int k, cudaStream_t stream)
{
    wrapper(q, x, code, absmax, o, m, n, k, stream);
}

extern "C" void tuna_ref_dequant(void *q, void *absmax, void *code, void *o,
                                 int m, int k, cudaStream_t stream)
{
    dequantize_wrapper(q, absmax, code, o, m, k, stream);
}
