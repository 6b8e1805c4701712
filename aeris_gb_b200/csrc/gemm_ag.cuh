// All-gather of the A operand fused into the GEMM kernels (see GemmParams::ag_*): device helpers shared by the one-CTA
// and the two-CTA kernel.
#pragma once
#include "gemm_epilogue.cuh"

namespace aeris {

// Four copier warps behind the six GEMM warps: 128 threads x 8 vectors keep 16 KB of posted peer stores in flight per
// SM, which the link needs at 8 ranks (two warps reached 360 GB/s of egress there).
constexpr int AG_COPY_THREADS = 128;
constexpr int AG_UNROLL = 8;          // 16-byte vectors in flight per copier thread (local loads, posted peer stores)

__device__ __forceinline__ uint32_t ld_acquire_sys(const unsigned* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits (bounded) until every CTA of rank `c` has pushed its slice of chunk `c` into this rank's buffer.
__device__ __forceinline__ bool ag_wait_chunk(const GemmParams& p, int c) {
  auto ready = [&] { return static_cast<int>(ld_acquire_sys(p.ag_count + c) - p.ag_expect) >= 0; };
  if (ready()) return true;
  const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (ready()) return true;
      __nanosleep(64);
    }
    if (globaltimer_ns() - t0 > AERIS_WAIT_TIMEOUT_NS) {
      if (p.status) atomicCAS(p.status, 0, ERR_TIMEOUT_SIGNAL);
      return false;
    }
    if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) return false;
  }
}
// Before the TMA loads of A rows [row0, row1): every chunk they touch has arrived. `ready` caches what was seen.
__device__ __forceinline__ bool ag_wait_rows(const GemmParams& p, int row0, int row1, uint32_t& ready) {
  const int c_lo = row0 / p.ag_rows, c_hi = (min(p.M, row1) - 1) / p.ag_rows;
  for (int c = c_lo; c <= c_hi; ++c) {
    if (c == p.ag_rank || (ready >> c) & 1u) continue;
    if (!ag_wait_chunk(p, c)) return false;
    ready |= 1u << c;
    asm volatile("fence.proxy.async;" ::: "memory");   // the rows were written through the generic proxy
  }
  return true;
}
// Copier warps: push this CTA's slice of this rank's chunk into every peer's buffer, nearest consumer first, and add one
// to this rank's arrival word on that peer. `cid` = thread index among the AG_COPY_THREADS copier threads.
__device__ __forceinline__ void ag_push_chunk(const GemmParams& p, int cid) {
  const long long vecs = static_cast<long long>(p.ag_rows) * p.K / 8;   // 16-byte vectors of this rank's chunk
  const long long per = (vecs + gridDim.x - 1) / gridDim.x;
  const long long v0 = per * blockIdx.x, v1 = min(vecs, v0 + per);
  const size_t off = static_cast<size_t>(p.ag_rank) * p.ag_rows * p.K * 2;
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.ag_local) + off);
  for (int j = 1; j < p.ag_world; ++j) {
    const int dst_rank = (p.ag_rank - j + p.ag_world) % p.ag_world;     // the rank that needs this chunk soonest
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.ag_peers[dst_rank]) + off);
    long long i = v0 + cid;
    for (; i + (AG_UNROLL - 1) * AG_COPY_THREADS < v1; i += AG_UNROLL * AG_COPY_THREADS) {
      uint4 t[AG_UNROLL];
#pragma unroll
      for (int u = 0; u < AG_UNROLL; ++u) t[u] = src[i + u * AG_COPY_THREADS];
#pragma unroll
      for (int u = 0; u < AG_UNROLL; ++u) dst[i + u * AG_COPY_THREADS] = t[u];
    }
    for (; i < v1; i += AG_COPY_THREADS) dst[i] = src[i];
    __threadfence_system();
    asm volatile("bar.sync 1, %0;" ::"n"(AG_COPY_THREADS) : "memory");
    if (cid == 0)
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.ag_count_peers[dst_rank] + p.ag_rank) : "memory");
  }
}

}  // namespace aeris
