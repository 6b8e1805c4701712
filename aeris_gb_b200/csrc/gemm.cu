// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128B swizzle) -> tcgen05.mma with
// fp32 accumulators in TMEM (double buffered) -> tcgen05.ld epilogue with fused element-wise tails.
//
//   C[M,N] (op)= A[M,K] * B[N,K]^T
//
// Either operand may be given "MN-major" (stored transposed, reduction dimension strided), which is what the
// weight-gradient (dW = dY^T X) and data-gradient (dX = dY W) products need, so no transposed copies of
// activations or weights are ever made.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue.
// Covers the linear layers of the Swin block (reference: src/aeris/models/parallel_swin.py:92-100,236-237,
// to_qkv / wo / w1 / w2) with the SwiGLU and gated-residual tails of parallel_swin.py:99-100,460-461 fused in.
#include "common.cuh"
#include "api.h"
#include "host.h"
#include "gemm_epilogue.cuh"

#include <mutex>
#include <stdio.h>

namespace aeris {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = TILE_BYTES + BAR_BYTES + 1024;  // + alignment slack
};

template <int BN, int A_MN, int B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::TILE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  {  // an earlier kernel already failed: leave before touching TMEM (decision made once per CTA)
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    __syncthreads();
    if (s_abort) return;
  }

  const int m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = p.N / BN;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_per_split = (kb_total + p.k_splits - 1) / p.k_splits;
  const int total_tiles = m_tiles * n_tiles * p.k_splits;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);  // 2 accumulators of BN fp32 columns (256 or 512 columns)
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one_sync()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int split = tile / (m_tiles * n_tiles);
        const int mn = tile - split * (m_tiles * n_tiles);
        const int tm = mn / n_tiles, tn = mn - tm * n_tiles;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb_total, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          if (A_MN == 0) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, tm * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[stage], tm * BM + j * 64, kb * BK);
          }
          if (B_MN == 0) {
            const int r0 = tn * p.b_tile_stride;
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, r0);
            tma_load_2d(sb + (BN / 2) * 128, &tmap_b, &full_bar[stage], kb * BK, r0 + p.b_half_off);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], tn * BN + j * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (ok) {
        // Drain: wait until the MMA warp has released every stage we filled, so no copy is in flight at exit.
        for (int s = 0; s < STAGES; ++s) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) break;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one_sync()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int split = tile / (m_tiles * n_tiles);
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb_total, kb0 + kb_per_split);
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status, ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t adesc = A_MN ? make_smem_desc(sa + kk * 2048, 8192, 1024)
                                        : make_smem_desc(sa + kk * 32, 0, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024)
                                        : make_smem_desc(sb + kk * 32, 0, 1024);
            umma_ss(tmem_acc, adesc, bdesc, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int split = tile / (m_tiles * n_tiles);
      const int mn = tile - split * (m_tiles * n_tiles);
      const int tm = mn / n_tiles, tn = mn - tm * n_tiles;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const bool kempty = (split * kb_per_split) >= kb_total;  // split with no k-blocks: accumulator undefined
      gemm_epilogue_row<BN>(p, taddr, row, row < p.M, tn, kempty);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(ptr);
  });
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `rows` rows, row pitch `ld` elements.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t ld,
                      uint32_t box_inner, uint32_t box_rows) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return -10;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -11;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                      uint64_t pitch2, uint32_t b0, uint32_t b1) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return -10;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((pitch1 * 2) & 15) || ((pitch2 * 2) & 15)) return -11;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1 * 2, pitch2 * 2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

static int g_num_sms = 0;
int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <int BN, int A_MN, int B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using S = GemmSmem<BN>;
  static bool configured = false;
  auto kern = gemm_kernel<BN, A_MN, B_MN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return -20;
    configured = true;
  }
  const int m_tiles = (p.M + BM - 1) / BM;
  const int tiles = m_tiles * (p.N / BN) * p.k_splits;
  const int grid = tiles < num_sms() ? tiles : num_sms();
  kern<<<grid, GEMM_THREADS, S::TOTAL, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace aeris

using namespace aeris;

int aeris_num_sms() { return aeris::num_sms(); }

extern "C" int aeris_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                               int ldc, int a_mn, int b_mn, int epi, const void* resid, int ldr,
                               const float* gate, int rows_per_gate, void* aux, int ld_aux, int swiglu_f,
                               int k_splits, int bn, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (bn != 128 && bn != 256) bn = (N % 256 == 0) ? 256 : 128;
  if (N % bn != 0) return -2;
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
  if (swiglu_fwd) {
    // N counts gate+up columns (2F); a tile holds bn/2 gate columns and the matching bn/2 up columns.
    p.b_tile_stride = bn / 2;
    p.b_half_off = swiglu_f;
  } else {
    p.b_tile_stride = bn;
    p.b_half_off = bn / 2;
  }
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  else       r = make_tmap_2d_bf16(&ta, A, M, K, lda, 64, BK);
  if (r) return r;
  if (!b_mn) {
    const uint64_t brows = swiglu_fwd ? static_cast<uint64_t>(2) * swiglu_f : static_cast<uint64_t>(N);
    r = make_tmap_2d_bf16(&tb, B, K, brows, ldb, BK, bn / 2);
  } else {
    r = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, BK);
  }
  if (r) return r - 100;
#define AERIS_DISPATCH(BN_)                                                                   \
  if (!a_mn && !b_mn) return launch_gemm<BN_, 0, 0>(ta, tb, p, stream);                       \
  if (!a_mn && b_mn) return launch_gemm<BN_, 0, 1>(ta, tb, p, stream);                        \
  if (a_mn && !b_mn) return launch_gemm<BN_, 1, 0>(ta, tb, p, stream);                        \
  return launch_gemm<BN_, 1, 1>(ta, tb, p, stream);
  if (bn == 256) { AERIS_DISPATCH(256) } else { AERIS_DISPATCH(128) }
#undef AERIS_DISPATCH
}

