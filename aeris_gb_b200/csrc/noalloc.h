// Allocation-free entry point of the attention backward pass. This function has no counterpart in the reference
// implementation; it exists for one class of callers of this library.
//
// Who needs it: a host program that is not allowed to create device memory when it calls us. Typical cases are an
// inference or training server that sizes all of its GPU memory at start-up and forbids allocation afterwards (so
// that a request can never fail with out-of-memory or stall on the allocator's implicit device synchronisation),
// and code that runs where an allocation call is simply illegal or would dead-lock, for example while another
// library holds the device in a state in which cudaMalloc must not be called. Such a caller can hand us its inputs
// and outputs, but it has nowhere to get the backward pass's scratch buffer from.
//
// What it does: exactly aeris_attn_bwd (see api.h), except that the `delta` scratch (one float for every
// (window, head, token), written by the first kernel and read by the second) is a fixed device array that is part of
// the library image. The function calls no cudaMalloc / cudaFree and no allocating library routine; the caller still
// passes every input and output.
//
// Limits and rules:
//   * n_win * H * N must not exceed AERIS_NOALLOC_MAX_SCRATCH_FLOATS (4 Mi floats = 16 MiB); larger problems are
//     refused with AERIS_NOALLOC_ERR_TOO_LARGE and nothing is launched. Split the windows over several calls.
//   * Every GPU that loads the library holds those 16 MiB until the process exits.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current) and remembers it; make that first call outside of any stream capture.
//   * All calls on a device share the one array, and it keeps the previous call's contents. Nothing in it has to
//     start at zero: each call overwrites every entry it later reads. Two calls whose kernels can overlap on the GPU
//     (different streams, or different host threads) race on the array: serialise them on one stream.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define AERIS_NOALLOC_MAX_SCRATCH_FLOATS (1 << 22)
#define AERIS_NOALLOC_MAX_DEVICES 64
#define AERIS_NOALLOC_ERR_BAD_SHAPE (-40)
#define AERIS_NOALLOC_ERR_TOO_LARGE (-41)
#define AERIS_NOALLOC_ERR_DEVICE (-42)
#define AERIS_NOALLOC_ERR_SYMBOL (-43)

// Returns 0 on success, one of the codes above, or the error code of aeris_attn_bwd. Arguments as aeris_attn_bwd
// without `delta`.
int aeris_attn_bwd_noalloc(const void* qkv, int ldq, int q_col0, int k_col0, int v_col0, const void* o, const void* d_o,
                           int ldo, const float* lse, void* dqkv, int ldg, int n_win, int N, int H, int head_dim,
                           float scale, int* status, void* stream);

#ifdef __cplusplus
}
#endif
