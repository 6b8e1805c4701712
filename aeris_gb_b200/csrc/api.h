// C ABI of libaeris_b200.so. Every function returns 0 on success and a negative code on a host-side argument or
// launch error. Kernels report device-side problems (bounded waits that ran out, failed bounds checks) through
// the `status` word, which the caller owns and reads after synchronising.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

int aeris_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                    int a_mn, int b_mn, int epi, const void* resid, int ldr, const float* gate,
                    int rows_per_gate, void* aux, int ld_aux, int swiglu_f, int k_splits, int bn, int* status,
                    void* stream);

#ifdef __cplusplus
}
#endif
