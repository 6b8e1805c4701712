// All-gather of the A operand fused into the GEMM kernels (see GemmParams::ag_*): device helpers shared by the one-CTA
// and the two-CTA kernel.
#pragma once
#include "gemm_epilogue.cuh"

namespace aeris {

// One copier warp (6) behind the GEMM warps; its elected lane drives the TMA unit: 16 KB pieces of this CTA's slice go
// local memory -> shared memory ring (two buffers) -> the peer's buffer as bulk copies, so the transfer needs neither
// registers nor issue slots and keeps two 16 KB stores in flight per SM. (Copier warps that moved the data through
// registers with posted 16-byte stores reached about 360 GB/s of egress, whether two or four of them.)
constexpr int AG_COPY_THREADS = 32;
constexpr uint32_t AG_PIECE = 16384;

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
__device__ __forceinline__ void bulk_load_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
// Copier (one elected thread): push this CTA's slice of this rank's chunk into every peer's buffer, nearest consumer
// first, and add one to this rank's arrival word on that peer. `ring`: 2 * AG_PIECE bytes of shared memory (16-byte
// aligned), `bars`: two mbarriers initialised with count 1. Slices start and end on 16-byte boundaries.
__device__ __forceinline__ void ag_push_chunk(const GemmParams& p, uint8_t* ring, uint64_t* bars) {
  const long long bytes_total = static_cast<long long>(p.ag_rows) * p.K * 2;
  const long long per = ((bytes_total / 16 + gridDim.x - 1) / gridDim.x) * 16;
  const long long b0 = per * blockIdx.x, b1 = min(bytes_total, b0 + per);
  const size_t off = static_cast<size_t>(p.ag_rank) * p.ag_rows * p.K * 2;
  const uint8_t* src = reinterpret_cast<const uint8_t*>(p.ag_local) + off;
  uint32_t phase[2] = {0u, 0u};
  int buf = 0;
  bool ok = true;
  for (int j = 1; j < p.ag_world; ++j) {
    const int dst_rank = (p.ag_rank - j + p.ag_world) % p.ag_world;     // the rank that needs this chunk soonest
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.ag_peers[dst_rank]) + off;
    for (long long pos = b0; pos < b1 && ok; pos += AG_PIECE) {
      const uint32_t n = static_cast<uint32_t>(min(static_cast<long long>(AG_PIECE), b1 - pos));
      // the store that last read this buffer (two pieces ago) has left shared memory
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      mbar_expect_tx(&bars[buf], n);
      bulk_load_g2s(ring + buf * AG_PIECE, src + pos, n, &bars[buf]);
      if (!mbar_wait_poll(&bars[buf], phase[buf], p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
      phase[buf] ^= 1u;
      bulk_store_s2g(dst + pos, ring + buf * AG_PIECE, n);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      buf ^= 1;
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");            // every store of this chunk has completed
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence_system();
    if (ok)
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.ag_count_peers[dst_rank] + p.ag_rank) : "memory");
  }
}

}  // namespace aeris
