// Two-CTA variant of the persistent tcgen05 GEMM: a thread-block cluster of two CTAs (one SM pair) computes one
// 256 x 256 output tile with `tcgen05.mma.cta_group::2`. Each CTA stages its own 128 rows of A and only HALF of the
// B tile (128 of the 256 columns), so the shared-memory operand traffic per FLOP is a third lower than in the
// one-CTA 128 x 256 kernel, which is bound by exactly that traffic (73 % tensor-pipe utilisation).
//
// Every CTA issues its own plain TMA loads (no load is shared between the two CTAs). Cross-CTA signalling:
//   * stage filled : both CTAs' TMA loads credit their bytes to ONE barrier in the leader CTA (loads issued with
//                    cta_group::2, barrier addressed through the cluster window), on which the MMA thread waits;
//   * stage free   : one `tcgen05.commit` arrives on the same barrier in both CTAs (commit with a CTA mask);
//   * accumulator ready: same two-CTA commit; accumulator drained: both CTAs' epilogue warps arrive on the leader.
// Every wait is bounded and every role falls through to one final cluster barrier, so a time-out in one CTA can not
// leave its peer waiting forever.
#include "common.cuh"
#include "api.h"
#include "host.h"
#include "gemm_epilogue.cuh"
#include "gemm_ag.cuh"

#include <stdio.h>
#include <stdlib.h>

namespace aeris {

constexpr int G2_BM = 128;       // rows per CTA (256 per pair)
constexpr int G2_BN = 256;
constexpr int G2_BK = 64;
constexpr int G2_THREADS = 192;
constexpr int G2_STAGES = 6;
constexpr int G2_A_BYTES = G2_BM * G2_BK * 2;         // 16 KB
constexpr int G2_B_BYTES = (G2_BN / 2) * G2_BK * 2;   // 16 KB: this CTA's half of B
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_PUSH_OFF = G2_STAGES * G2_STAGE_BYTES + 512;     // staging of the peer-push epilogues, 8 KB per warp
constexpr int G2_SMEM = G2_PUSH_OFF + 4 * PUSH_STAGE_BYTES + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled TMA load for a CTA pair: the data lands in THIS CTA's shared memory, the byte count is credited to the
// barrier at `bar_cluster_addr`, which may live in the other CTA of the pair (the leader's "stage full" barrier).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive on the barrier at the same shared-memory offset in every CTA named by `mask` once all prior tcgen05 ops of
// this thread have completed.
__device__ __forceinline__ void tc_commit2_mc(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}
__device__ __forceinline__ void umma2_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// AG = true: the A operand is all-gathered over peer memory inside the kernel (GemmParams::ag_*): m-tiles are visited
// starting with this rank's own row chunk while two extra warps (6, 7) of every CTA push that chunk into the peers'
// buffers; the producer of each CTA waits for the chunks its 128 rows come from. The grid is then always the full
// number of CTA pairs, so that every call adds the same amount to the arrival counters.
template <int A_MN, int B_MN, bool AG = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(AG ? G2_THREADS + AG_COPY_THREADS : G2_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
             const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + G2_STAGES * G2_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + G2_STAGES;
  uint64_t* tfull_bar = empty_bar + G2_STAGES;       // [2]
  uint64_t* tempty_bar = tfull_bar + 2;              // [2], leader only: 8 arrivals (4 epilogue warps x 2 CTAs)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  // AG: the last operand stage is the copier's ring (two 16 KB bulk-copy buffers), with its barriers behind tmem_slot
  // (the reduce-scatter epilogue gives up the same stage: its fourth warp stages its rows there)
  const int STAGES = (AG || p.epi == EPI_RS_PUSH) ? G2_STAGES - 1 : G2_STAGES;
  [[maybe_unused]] uint8_t* ag_ring = smem + (G2_STAGES - 1) * G2_STAGE_BYTES;
  [[maybe_unused]] uint64_t* ag_bars = reinterpret_cast<uint64_t*>(smem + G2_STAGES * G2_STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();          // 0 = leader (issues the MMAs)
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  const int m_tiles = (p.M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int n_tiles = p.N / G2_BN;
  const int kb_total = (p.K + G2_BK - 1) / G2_BK;
  const int kb_per_split = (kb_total + p.k_splits - 1) / p.k_splits;
  const int total_tiles = m_tiles * n_tiles * p.k_splits;
  const int tm_rot = AG ? (p.ag_rank * p.ag_rows) / (2 * G2_BM) : p.tm_rot;
  auto phys_tm = [&](int tm) { return (tm + tm_rot) % m_tiles; };

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);
      if constexpr (AG) mbar_init(&ag_bars[a], 1);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 2 * G2_BN);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // both CTAs' barriers are initialised and TMEM is allocated before anyone signals
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (each CTA loads its own operands)
    if (elect_one_sync()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      [[maybe_unused]] uint32_t ag_ready = 0;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
        const int split = tile / (m_tiles * n_tiles);
        const int mn = tile - split * (m_tiles * n_tiles);
        const int tm = phys_tm(mn / n_tiles), tn = mn - (mn / n_tiles) * n_tiles;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb_total, kb0 + kb_per_split);
        const int m0 = tm * 2 * G2_BM + crank * G2_BM;
        if constexpr (AG) {
          if (m0 < p.M && !ag_wait_rows(p, m0, m0 + G2_BM, ag_ready)) { ok = false; break; }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_poll(&empty_bar[stage], phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * G2_STAGE_BYTES;
          uint8_t* sb = sa + G2_A_BYTES;
          // one "stage full" barrier per pair, in the leader: it expects the bytes of both CTAs' copies
          if (crank == 0) mbar_expect_tx(&full_bar[stage], 2 * G2_STAGE_BYTES);
          const uint32_t fb = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (A_MN == 0) {
            tma_load_2d_pair(sa, &tmap_a, fb, kb * G2_BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < G2_BM / 64; ++j)
              tma_load_2d_pair(sa + j * 8192, &tmap_a, fb, m0 + j * 64, kb * G2_BK);
          }
          if (B_MN == 0) {
            // rows of B for this CTA's half: plain tiles take 128 consecutive rows; the SwiGLU layouts pair the
            // leader with the gate rows and the peer with the up rows of the same features
            const int r0 = tn * p.b_tile_stride + (crank ? p.b_half_off : 0);
            tma_load_2d_pair(sb, &tmap_b, fb, kb * G2_BK, r0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_2d_pair(sb + j * 8192, &tmap_b, fb, tn * G2_BN + (crank * 2 + j) * 64, kb * G2_BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (crank == 0) {
        // -------------------------------------------------------- leader: MMA issuer for the CTA pair
        constexpr uint32_t idesc = make_idesc_bf16(2 * G2_BM, G2_BN, A_MN, B_MN);
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
          const int split = tile / (m_tiles * n_tiles);
          const int kb0 = split * kb_per_split;
          const int kb1 = min(kb_total, kb0 + kb_per_split);
          if (!mbar_wait_poll(&tempty_bar[acc], acc_phase ^ 1, p.status, ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tmem_acc = tmem_base + acc * G2_BN;
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait_poll(&full_bar[stage], phase, p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * G2_STAGE_BYTES);
            const uint32_t sb = sa + G2_A_BYTES;
#pragma unroll
            for (int kk = 0; kk < G2_BK / 16; ++kk) {
              const uint64_t adesc = A_MN ? make_smem_desc(sa + kk * 2048, 8192, 1024)
                                          : make_smem_desc(sa + kk * 32, 0, 1024);
              const uint64_t bdesc = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024)
                                          : make_smem_desc(sb + kk * 32, 0, 1024);
              umma2_ss(tmem_acc, adesc, bdesc, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
            }
            tc_commit2_mc(&empty_bar[stage], 0x3);     // frees the stage in both CTAs
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          tc_commit2_mc(&tfull_bar[acc], 0x3);         // accumulator ready in both CTAs
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
  } else if (AG && warp >= 6) {
    // ------------------------------------------------------------ all-gather copier (warp 6 of both CTAs)
    if constexpr (AG) {
      if (elect_one_sync()) ag_push_chunk(p, ag_ring, ag_bars);
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t leader_tempty0 = map_to_cta(smem_u32(&tempty_bar[0]), 0);
    for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
      const int split = tile / (m_tiles * n_tiles);
      const int mn = tile - split * (m_tiles * n_tiles);
      const int tm = phys_tm(mn / n_tiles), tn = mn - (mn / n_tiles) * n_tiles;
      if (!mbar_wait_poll(&tfull_bar[acc], acc_phase, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * 2 * G2_BM + crank * G2_BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * G2_BN + (static_cast<uint32_t>(q * 32) << 16);
      const bool kempty = (split * kb_per_split) >= kb_total;
      uint8_t* stg = smem + G2_PUSH_OFF + q * PUSH_STAGE_BYTES;
      if (p.epi == EPI_RS_PUSH)     // 8704-byte linear stages: three in the push area, the fourth in the freed operand stage
        stg = (q < 3) ? smem + G2_PUSH_OFF + q * RS_STAGE_BYTES : smem + (G2_STAGES - 1) * G2_STAGE_BYTES;
      gemm_epilogue_row<G2_BN>(p, taddr, row, row < p.M, tn, kempty, stg);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(leader_tempty0 + acc * 8);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    // the bulk copies of the reduce-scatter push have been performed before this thread leaves (the owners read
    // their slots after a rank barrier that follows this kernel in the stream)
    if (p.epi == EPI_RS_PUSH) rs_stage_drain();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // nobody leaves while the pair may still touch its shared memory or TMEM
  tc_fence_after();
  if (warp == 1) tmem_dealloc2(tmem_base, 2 * G2_BN);
}

template <int A_MN, int B_MN, bool AG = false>
static int launch_gemm2(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p_in, cudaStream_t stream) {
  static bool configured = false;
  GemmParams p = p_in;
  constexpr int THREADS = AG ? G2_THREADS + AG_COPY_THREADS : G2_THREADS;
  auto kern = gemm2_kernel<A_MN, B_MN, AG>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM) != cudaSuccess) return -20;
    configured = true;
  }
  const int m_tiles = (p.M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int tiles = m_tiles * (p.N / G2_BN) * p.k_splits;
  // persistent grid = the number of CTA pairs the device can actually hold at once
  static int max_clusters = 0;
  if (max_clusters == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms(), 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = G2_SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = num_sms() / 2;
    max_clusters = n;
    if (getenv("AERIS_DEBUG")) fprintf(stderr, "gemm2: max active clusters %d\n", n);
  }
  int clusters = max_clusters;
  if (tiles < clusters && !AG) clusters = tiles;
  if (AG) p.ag_expect *= static_cast<unsigned>(2 * clusters);   // came in as the call index
  kern<<<2 * clusters, THREADS, G2_SMEM, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace aeris

using namespace aeris;

// Same contract as aeris_gemm_bf16 (api.h); N must be a multiple of 256.
extern "C" int aeris_gemm_bf16_2cta(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                    int ldc, int a_mn, int b_mn, int epi, const void* resid, int ldr,
                                    const float* gate, int rows_per_gate, void* aux, int ld_aux, int swiglu_f,
                                    int k_splits, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (N % G2_BN != 0) return -2;
  const bool swiglu_fwd = (epi == EPI_SWIGLU || epi == EPI_SWIGLU_BOTH);
  if (swiglu_fwd && b_mn) return -3;
  if (k_splits < 1) k_splits = 1;
  if (k_splits > 1 && epi != EPI_ACC_F32) return -4;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.epi = epi; p.C = C; p.ldc = ldc;
  p.resid = reinterpret_cast<const __nv_bfloat16*>(resid); p.ldr = ldr;
  p.gate = gate; p.rows_per_gate = rows_per_gate > 0 ? rows_per_gate : M;
  p.aux = reinterpret_cast<__nv_bfloat16*>(aux); p.ld_aux = ld_aux;
  p.k_splits = k_splits; p.status = status; p.swiglu_f = swiglu_f;
  {
    // bf16-output epilogues write through the shared-memory stage as 256-byte row segments (measured 1-13 % faster
    // than one 16-byte piece per row and instruction); AERIS_GEMM_STAGED_OUT=0 selects the direct stores
    static const int staged = [] { const char* e = getenv("AERIS_GEMM_STAGED_OUT"); return e ? atoi(e) : 1; }();
    p.staged_out = staged;
    static const int staged_red = [] { const char* e = getenv("AERIS_GEMM_STAGED_RED"); return e ? atoi(e) : 0; }();
    p.staged_red = staged_red;
  }
  if (swiglu_fwd) { p.b_tile_stride = G2_BN / 2; p.b_half_off = swiglu_f; }
  else            { p.b_tile_stride = G2_BN;     p.b_half_off = G2_BN / 2; }
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d_bf16(&ta, A, K, M, lda, G2_BK, G2_BM);
  else       r = make_tmap_2d_bf16(&ta, A, M, K, lda, 64, G2_BK);
  if (r) return r;
  if (!b_mn) {
    const uint64_t brows = swiglu_fwd ? static_cast<uint64_t>(2) * swiglu_f : static_cast<uint64_t>(N);
    r = make_tmap_2d_bf16(&tb, B, K, brows, ldb, G2_BK, G2_BN / 2);
  } else {
    r = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, G2_BK);
  }
  if (r) return r - 100;
  if (!a_mn && !b_mn) return launch_gemm2<0, 0>(ta, tb, p, stream);
  if (!a_mn && b_mn) return launch_gemm2<0, 1>(ta, tb, p, stream);
  if (a_mn && !b_mn) return launch_gemm2<1, 0>(ta, tb, p, stream);
  return launch_gemm2<1, 1>(ta, tb, p, stream);
}

// QKV (or dO) projection whose epilogue performs the Ulysses head<->sequence exchange: C is not written locally;
// every head's tile goes straight into the symmetric buffer of the rank that owns the head (`peers[owner]`).
// A: [M, K] row-major tokens (M = windows * n_local), B: [N, K] weights (or stored [K, N] with b_mn).
extern "C" int aeris_gemm_scatter_heads(const void* A, const void* B, int M, int N, int K, int lda, int ldb,
                                        int b_mn, const void* const* peers, int sp, int sp_rank, int n_local, int L,
                                        int sec_w, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N % G2_BN != 0 || K <= 0 || sp < 1 || sp > 8) return -1;
  if (sec_w % sp != 0 || (sec_w / sp) % 32 != 0 || N % sec_w != 0 || M % n_local != 0) return -2;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.epi = EPI_SCATTER_HEADS; p.C = nullptr; p.ldc = 0;
  p.rows_per_gate = M; p.k_splits = 1; p.status = status;
  p.b_tile_stride = G2_BN; p.b_half_off = G2_BN / 2;
  for (int i = 0; i < sp; ++i) p.scat_peers[i] = const_cast<void*>(peers[i]);
  p.scat_rank = sp_rank; p.scat_n_local = n_local; p.scat_L = L; p.scat_sec_w = sec_w; p.scat_own_w = sec_w / sp;
  p.scat_ld = (N / sec_w) * (sec_w / sp);
  CUtensorMap ta, tb;
  int r = make_tmap_2d_bf16(&ta, A, K, M, lda, G2_BK, G2_BM);
  if (r) return r;
  r = b_mn ? make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, G2_BK) : make_tmap_2d_bf16(&tb, B, K, N, ldb, G2_BK, G2_BN / 2);
  if (r) return r - 100;
  return b_mn ? launch_gemm2<0, 1>(ta, tb, p, stream) : launch_gemm2<0, 0>(ta, tb, p, stream);
}

// GEMM -> reduce-scatter by rows in one kernel: rank `rank` computes its partial product for all `world *
// rows_per_rank` rows (A: [M, K] with K this rank's slice of the reduction dimension) and the epilogue stores each bf16
// tile into slot `rank` of the owner's [world * rows_per_rank, N] buffer `peers[owner]` (peer memory), so the
// transfer rides along tile by tile. The owner sums its `world` slots afterwards (aeris_rs_finalize).
extern "C" int aeris_gemm_rs_push(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int b_mn,
                                  const void* const* peers, int world, int rank, int rows_per_rank, int ld_dst,
                                  int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N % G2_BN != 0 || K <= 0 || world < 1 || world > 8 || rank < 0 || rank >= world) return -1;
  if (M != world * rows_per_rank || ld_dst % 8 != 0 || ld_dst < N) return -2;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.epi = EPI_RS_PUSH; p.C = nullptr; p.ldc = 0;
  p.rows_per_gate = M; p.k_splits = 1; p.status = status;
  p.b_tile_stride = G2_BN; p.b_half_off = G2_BN / 2;
  for (int i = 0; i < world; ++i) p.scat_peers[i] = const_cast<void*>(peers[i]);
  p.scat_rank = rank; p.scat_n_local = rows_per_rank; p.scat_ld = ld_dst;
  p.tm_rot = static_cast<int>((static_cast<long long>((rank + 1) % world) * rows_per_rank) / (2 * G2_BM));
  CUtensorMap ta, tb;
  int r = make_tmap_2d_bf16(&ta, A, K, M, lda, G2_BK, G2_BM);
  if (r) return r;
  r = b_mn ? make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, G2_BK) : make_tmap_2d_bf16(&tb, B, K, N, ldb, G2_BK, G2_BN / 2);
  if (r) return r - 100;
  return b_mn ? launch_gemm2<0, 1>(ta, tb, p, stream) : launch_gemm2<0, 0>(ta, tb, p, stream);
}

// All-gather -> GEMM in one kernel (two-CTA tiles). `A` is this rank's [world * rows_per_rank, K] buffer (row pitch K)
// whose chunk `rank` is filled; `peers[p]` is rank p's buffer of the same layout and `counter_peers[p]` its array of 8
// arrival words (peer memory; zero before the first call, never reset). `call_index` counts the calls made on this
// exchange (1, 2, ...; the same on every rank). On return of the kernel the whole gathered A is resident in `A` (the
// weight-gradient product reuses it). The caller synchronises the ranks before the call (every rank is done with the
// previous contents of the buffers). Epilogues: EPI_STORE, EPI_SWIGLU, EPI_SWIGLU_BOTH, EPI_SWIGLU_BWD.
extern "C" int aeris_gemm_allgather_a(void* A, const void* const* peers, const void* const* counter_peers, int world,
                                      int rank, int rows_per_rank, unsigned call_index, const void* B, void* C, int N,
                                      int K, int ldb, int ldc, int b_mn, int epi, const void* resid, int ldr, void* aux,
                                      int ld_aux, int swiglu_f, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (world < 1 || world > 8 || rank < 0 || rank >= world || rows_per_rank <= 0 || N <= 0 || K <= 0) return -1;
  if (N % G2_BN != 0 || K % 8 != 0 || (static_cast<long long>(rows_per_rank) * K) % 8 != 0) return -2;
  const bool swiglu_fwd = (epi == EPI_SWIGLU || epi == EPI_SWIGLU_BOTH);
  if (swiglu_fwd && b_mn) return -3;
  if (epi != EPI_STORE && !swiglu_fwd && epi != EPI_SWIGLU_BWD) return -4;
  const int M = world * rows_per_rank;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.epi = epi; p.C = C; p.ldc = ldc;
  p.resid = reinterpret_cast<const __nv_bfloat16*>(resid); p.ldr = ldr;
  p.rows_per_gate = M; p.aux = reinterpret_cast<__nv_bfloat16*>(aux); p.ld_aux = ld_aux;
  p.k_splits = 1; p.status = status; p.swiglu_f = swiglu_f;
  if (swiglu_fwd) { p.b_tile_stride = G2_BN / 2; p.b_half_off = swiglu_f; }
  else            { p.b_tile_stride = G2_BN;     p.b_half_off = G2_BN / 2; }
  for (int i = 0; i < world; ++i) {
    p.ag_peers[i] = const_cast<void*>(peers[i]);
    p.ag_count_peers[i] = reinterpret_cast<unsigned*>(const_cast<void*>(counter_peers[i]));
  }
  p.ag_local = A; p.ag_count = p.ag_count_peers[rank]; p.ag_world = world; p.ag_rank = rank; p.ag_rows = rows_per_rank;
  p.ag_expect = call_index;     // multiplied by the grid size at launch
  CUtensorMap ta, tb;
  int r = make_tmap_2d_bf16(&ta, A, K, M, K, G2_BK, G2_BM);
  if (r) return r;
  if (!b_mn) {
    const uint64_t brows = swiglu_fwd ? static_cast<uint64_t>(2) * swiglu_f : static_cast<uint64_t>(N);
    r = make_tmap_2d_bf16(&tb, B, K, brows, ldb, G2_BK, G2_BN / 2);
  } else {
    r = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, G2_BK);
  }
  if (r) return r - 100;
  return b_mn ? launch_gemm2<0, 1, true>(ta, tb, p, stream) : launch_gemm2<0, 0, true>(ta, tb, p, stream);
}
