// Windowed multi-head attention for sm_100a: softmax(Q K^T * scale) V per (window, head), non-causal and unmasked,
// forward and backward, flash-style (no N x N matrix in memory), on tcgen05 tensor cores with TMEM accumulators.
//
// Reference semantics: src/aeris/models/parallel_swin.py:257-258 (F.scaled_dot_product_attention, is_causal=False)
// and src/aeris_wp_inference/model.py:289-309 (naive softmax(QK^T)V over each window's tokens).
//
// Data layout: tokens are window-major, rows [w*N, (w+1)*N) belong to window w; Q, K, V are column slices of a
// row-major [T, ld] bf16 tensor (the fused qkv projection output, columns ordered (q|k|v, head, d)).
//
// Every kernel has the same skeleton (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..5 = one thread per tile row doing the softmax-side math straight out of TMEM.
#include "common.cuh"
#include "api.h"
#include "host.h"

namespace aeris {

constexpr int ATT_THREADS = 192;
constexpr int TILE = 128;

struct AttnFwdParams {
  __nv_bfloat16* O;
  int ldo;
  float* lse;  // [n_win * H * N], log2 domain: m + log2(l)
  int N, H, n_win;
  int q_col0, k_col0, v_col0;
  float scale_log2;
  int* status;
  // Ulysses output push (all null / 0 when unused): row `grow` of window `win` belongs to rank grow / push_n_local and
  // is stored at row win * push_n_local + grow % push_n_local, column push_col0 + head * d of that rank's buffer.
  void* o_peers[8];
  int push_n_local, push_ld, push_col0;
};

// Byte offset of 16-byte vector `v` (0..7) of row `r` inside a [rows x 64] bf16 tile stored with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz128(int r, int v) { return r * 128 + (((v ^ (r & 7)) & 7) << 4); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed two-wide fp32 arithmetic (sm_100 f32x2 instructions): one issue slot per two scores.
__device__ __forceinline__ float mufu_exp2(float x) {   // not volatile: the scheduler may interleave it freely
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for a pair of exponents on the FMA pipe instead of the exp unit (which limits attention at head_dim 64):
// x = r + f with r = round(x), f in [-0.5, 0.5]; 2^f by a cubic (relative error 7.5e-5, far below bf16 resolution),
// 2^r by adding r to the exponent field. x is clamped at -125 so the exponent field cannot wrap; callers keep x <= 8.
__device__ __forceinline__ void poly_exp2_pair(uint64_t t2, float& p0, float& p1) {
  float t0, t1;
  f2_unpack(t2, t0, t1);
  t2 = f2_pack(fmaxf(t0, -125.f), fmaxf(t1, -125.f));
  const uint64_t magic = f2_pack(12582912.f, 12582912.f);     // 1.5 * 2^23: the sum's low mantissa bits hold round(x)
  const uint64_t tm = f2_add(t2, magic);
  const uint64_t f = f2_sub(t2, f2_sub(tm, magic));
  uint64_t q = f2_fma(f2_pack(0.0551716574f, 0.0551716574f), f, f2_pack(0.2426111251f, 0.2426111251f));
  q = f2_fma(q, f, f2_pack(0.6932609677f, 0.6932609677f));
  q = f2_fma(q, f, f2_pack(0.9999280572f, 0.9999280572f));
  float q0, q1, m0, m1;
  f2_unpack(q, q0, q1);
  f2_unpack(tm, m0, m1);
  p0 = __uint_as_float(__float_as_uint(m0) * 0x00800000u + __float_as_uint(q0));
  p1 = __uint_as_float(__float_as_uint(m1) * 0x00800000u + __float_as_uint(q1));
}

// Probabilities of one 64-score row segment (raw scores in v0 | v1) against the reference maximum m_ref: bf16 pairs
// into pk, their sum returned. POLY of every eight pairs take the polynomial path, the rest the exp unit, interleaved
// so that both pipes stay busy.
template <int POLY>
__device__ __forceinline__ float softmax_row64(const uint32_t (&v0)[32], const uint32_t (&v1)[32], float sl2,
                                               float m_ref, uint32_t (&pk)[32]) {
  const uint64_t sl = f2_pack(sl2, sl2), nm = f2_pack(-m_ref, -m_ref);
  uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};      // bit pattern of (0.f, 0.f)
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint32_t a = (i < 16) ? v0[2 * i] : v1[2 * i - 32], b = (i < 16) ? v0[2 * i + 1] : v1[2 * i - 31];
    const uint64_t t = f2_fma(f2_pack(__uint_as_float(a), __uint_as_float(b)), sl, nm);
    float p0, p1;
    if ((i & 7) < POLY) {
      poly_exp2_pair(t, p0, p1);
    } else {
      float t0, t1;
      f2_unpack(t, t0, t1);
      p0 = mufu_exp2(t0);
      p1 = mufu_exp2(t1);
    }
    acc[i & 3] = f2_add(acc[i & 3], f2_pack(p0, p1));
    pk[i] = pack_bf16x2(p0, p1);
  }
  float s0, s1;
  f2_unpack(f2_add(f2_add(acc[0], acc[1]), f2_add(acc[2], acc[3])), s0, s1);
  return s0 + s1;
}

// -------------------------------------------------------------------------------------------------------- forward
// grid = (q_tiles, H, n_win). One CTA owns a 128-row Q tile and streams the window's K/V in 64-row tiles through a
// two-stage TMA ring. Per tile: S = Q K^T lands in TMEM, the four softmax warps (one thread per query row) read its 64
// scores once into registers and release the buffer at once, so the tensor core computes the next tile's scores under
// the exponentials; the bf16 probabilities go to shared memory as the A operand of P V, which ACCUMULATES in one TMEM
// buffer over all tiles. The running output is therefore never read back per tile: the exponentials use a reference
// maximum that is only raised (and the TMEM accumulator and row sum rescaled) when a row's maximum grows by more than
// 2^8, which bounds the probabilities by 256 and is exact after the final division by the row sum. The small footprint
// (64 KB shared memory, 128 TMEM columns, no register-resident output) lets three CTAs share an SM at head_dim 64.
constexpr int KVT = 64;
constexpr float RESCALE_LOG2 = 8.0f;

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// acc[lane row, 0..cols) *= alpha in TMEM, eight columns at a time: it runs only when a row maximum jumps and must not add
// to the register pressure of the caller, whose 64 scores are live.
__device__ __forceinline__ void rescale_tmem_rows(uint32_t taddr, int cols, float alpha) {
#pragma unroll 1
  for (int c = 0; c < cols; c += 8) {
    uint32_t v[8];
    tmem_ld8(taddr + c, v);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
    tmem_st8(taddr + c, v);
  }
  tmem_wait_st();
}

// Depth of the K and V rings of the forward kernel: at head_dim 64 three CTAs of 72 KB share an SM, at 128 two of 112 KB.
#ifdef AERIS_ATTN_TRACE
// Measurement build only: warp 2, lane 0 of CTA (0, 0, 0) stamps clock64 at the phase boundaries of every tile.
__device__ long long* g_attn_trace = nullptr;
#define ATTN_STAMP(slot) do { if (trace_on) g_attn_trace[(j) * 8 + (slot)] = clock64(); } while (0)
#else
#define ATTN_STAMP(slot) do { } while (0)
#endif

// Forward kernel modes. 0: probabilities through shared memory, three CTAs per SM at head_dim 64. 1: probabilities in
// tensor memory, over the score columns they came from (P V takes its A operand from TMEM). 2: as 1 with four lighter
// CTAs per SM. (A variant with two score buffers, which computes the scores of tile j + 1 under the softmax of tile j
// without the shared-memory round trip, fits only two CTAs per SM and measured no faster.)
template <int DCH, int MODE> struct AttnFwdRing {
  static constexpr int NSK = (DCH == 1 && MODE != 2) ? 3 : 2;
  static constexpr int NSV = 2;
  static constexpr int MIN_CTAS = (DCH == 2) ? 2 : (MODE == 2 ? 4 : 3);
};

// POLY < 0: scalar softmax arithmetic, every exponential on the exp unit; POLY >= 0: two-wide fp32 arithmetic with POLY of
// every eight score pairs exponentiated by the polynomial.
// PTMEM: the probabilities never touch shared memory. Each softmax thread writes its row of bf16 pairs back into the
// TMEM columns it has just read the scores from, and P V takes its A operand from tensor memory. An M128 x N64 x K16
// product with both operands in shared memory reads 6 KB for 32 cycles of math, more than the 128 B/cycle the shared
// memory delivers, so the kernel with P in shared memory (16 KB written and 16 KB read back per tile, on top of
// Q, K and V) is bound by shared-memory bandwidth rather than by the tensor or the exp unit.
template <int DCH, int POLY, int MODE>
__global__ void __launch_bounds__(ATT_THREADS, AttnFwdRing<DCH, MODE>::MIN_CTAS)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnFwdParams p) {
  constexpr int HD = 64 * DCH;
  constexpr int Q_BYTES = DCH * 16384;
  constexpr int T_BYTES = DCH * 8192;       // one K tile or one V tile (64 rows)
  // K and V travel in rings of their own: a K tile is free as soon as its Q K^T has completed, a whole softmax before
  // the V tile of the same step, so its successor is requested that much earlier and the load latency hides behind
  // the softmax of the tiles in between.
  constexpr bool PTMEM = MODE != 0;
  constexpr int NSK = AttnFwdRing<DCH, MODE>::NSK, NSV = AttnFwdRing<DCH, MODE>::NSV;
  constexpr int P_BYTES = PTMEM ? 0 : 16384;   // [128 x 64] bf16
  constexpr int TMEM_COLS = (DCH == 1) ? 128 : 256;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sKr = sQ + Q_BYTES;
  uint8_t* sVr = sKr + NSK * T_BYTES;
  uint8_t* sP = sVr + NSV * T_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;     // [NSK <= 4]
  uint64_t* k_empty = bars + 5;    // [NSK <= 4]
  uint64_t* v_full = bars + 9;     // [NSV <= 4]
  uint64_t* v_empty = bars + 13;   // [NSV <= 4]
  uint64_t* s_full = bars + 17;    // scores of tile j are in TMEM
  uint64_t* s_free = bars + 18;    // every softmax warp has read them into registers
  uint64_t* p_full = bars + 19;    // probabilities of tile j are in shared memory
  uint64_t* pv_done = bars + 20;   // P V of tile j has completed (P buffer reusable, accumulator up to date)
  static_assert(NSK <= 4 && NSV <= 4, "barrier slots");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, head = blockIdx.y, win = blockIdx.z;
  const int N = p.N;
  const int nfull = N / KVT, rem = N - nfull * KVT;
  const int nkv = nfull + (rem ? 1 : 0);
  const int n_last = rem ? ((rem + 15) & ~15) : KVT;  // MMA N of the last K/V tile

  if (threadIdx.x == 0) {
    int ab = (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    if ((smem_u32(smem) & 1023u) != 0) {
      ab = 1;
      if (p.status) atomicCAS(p.status, 0, ERR_BOUNDS);
    }
    *s_abort = ab;
  }
  __syncthreads();
  if (*s_abort) return;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < NSK; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < NSV; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    // only the softmax warps that own at least one real query row take part in the hand-shakes: a warp without rows
    // would run a tile ahead of the others and its arrivals would complete a phase that belongs to the slower warps
    const int n_valid_warps = min(4, (N - qt * TILE + 31) / 32);
    mbar_init(s_full, 1); mbar_init(s_free, n_valid_warps); mbar_init(p_full, n_valid_warps); mbar_init(pv_done, 1);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;          // S : 64 columns
  const uint32_t tO = tmem_base + 64;     // O : HD columns, accumulated over all tiles

  if (warp == 0) {
    if (elect_one_sync()) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int c = 0; c < DCH; ++c)
        tma_load_3d(sQ + c * 16384, &tm_q, q_full, p.q_col0 + head * HD + c * 64, qt * TILE, win);
      // K_i, then V_{i-1}: the order in which their slots come free (K_i after Q K^T of tile i - NSK, V_{i-1} after P V
      // of tile i - 1 - NSV, which completes later), so no wait holds up a load whose slot is already free
      for (int i = 0; i <= nkv; ++i) {
        if (i < nkv) {
          const int st = i % NSK;
          if (!mbar_wait(&k_empty[st], ((i / NSK) & 1) ^ 1, p.status, ERR_TIMEOUT_ATTN)) break;
          mbar_expect_tx(&k_full[st], T_BYTES);
#pragma unroll
          for (int c = 0; c < DCH; ++c)
            tma_load_3d(sKr + st * T_BYTES + c * 8192, &tm_k, &k_full[st], p.k_col0 + head * HD + c * 64, i * KVT, win);
        }
        if (i >= 1) {
          const int j = i - 1, st = j % NSV;
          if (!mbar_wait(&v_empty[st], ((j / NSV) & 1) ^ 1, p.status, ERR_TIMEOUT_ATTN)) break;
          mbar_expect_tx(&v_full[st], T_BYTES);
#pragma unroll
          for (int c = 0; c < DCH; ++c)
            tma_load_3d(sVr + st * T_BYTES + c * 8192, &tm_v, &v_full[st], p.v_col0 + head * HD + c * 64, j * KVT, win);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      bool ok = mbar_wait(q_full, 0, p.status, ERR_TIMEOUT_ATTN);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP), aKr = smem_u32(sKr), aVr = smem_u32(sVr);
      // S = Q K_j^T  (A = Q K-major, B = K K-major, reduction over d)
      auto issue_qk = [&](int j) -> bool {
        const int st = j % NSK;
        if (!mbar_wait(&k_full[st], (j / NSK) & 1, p.status, ERR_TIMEOUT_ATTN)) return false;
        tc_fence_after();
        const int ncur = (j == nkv - 1) ? n_last : KVT;
        const uint32_t aK = aKr + st * T_BYTES;
        const uint32_t idesc_qk = make_idesc_bf16(TILE, ncur, 0, 0);
#pragma unroll
        for (int kk = 0; kk < 4 * DCH; ++kk) {
          const uint32_t qoff = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t koff = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_ss(tS, make_smem_desc(aQ + qoff, 0, 1024), make_smem_desc(aK + koff, 0, 1024), idesc_qk, kk > 0);
        }
        tc_commit(s_full);
        tc_commit(&k_empty[st]);       // the K tile is free once these products have completed
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < nkv && ok; ++j) {
        const int st = j % NSV;
        const int ncur = (j == nkv - 1) ? n_last : KVT;
        if constexpr (!PTMEM) {
          if (j + 1 < nkv) {     // the next tile's scores, as soon as this tile's have been read out of TMEM
            if (!mbar_wait(s_free, j & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
            tc_fence_after();
            if (!issue_qk(j + 1)) { ok = false; break; }
          }
        }
        if (!mbar_wait(&v_full[st], (j / NSV) & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
        if (!mbar_wait(p_full, j & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
        tc_fence_after();
        // O += P_j V_j  (A = P K-major over kv, B = V MN-major: d contiguous, kv rows strided)
        const uint32_t aV = aVr + st * T_BYTES;
        const uint32_t idesc_pv = make_idesc_bf16(TILE, HD, 0, 1);
        for (int kk = 0; kk < ncur / 16; ++kk) {
          const uint32_t acc = (j > 0 || kk > 0) ? 1u : 0u;
          if constexpr (PTMEM)      // A = P in the score columns: 16 bf16 = 8 columns per K step
            umma_ts(tO, tS + kk * 8, make_smem_desc(aV + kk * 2048, 8192, 1024), idesc_pv, acc);
          else
            umma_ss(tO, make_smem_desc(aP + kk * 32, 0, 1024), make_smem_desc(aV + kk * 2048, 8192, 1024), idesc_pv, acc);
        }
        tc_commit(pv_done);
        tc_commit(&v_empty[st]);
        if constexpr (PTMEM) {
          // the tensor core executes in issue order: these scores overwrite P_j only after P_j V_j has consumed it
          if (j + 1 < nkv && !issue_qk(j + 1)) { ok = false; break; }
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;            // row inside the Q tile == TMEM lane
    const int grow = qt * TILE + row;         // row inside the window
    const bool warp_valid = (qt * TILE + q * 32) < N;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const float sl2 = p.scale_log2;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // Raises the reference maximum to m_new: rescales the TMEM accumulator (once P V of the previous tile is done) and l.
    auto rescale = [&](int j, float m_new, bool& waited) -> bool {
      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1, p.status, ERR_TIMEOUT_ATTN)) return false;
        waited = true;
        tc_fence_after();
        const float alpha = fast_exp2(m_ref - m_new);
        rescale_tmem_rows(tO + lane_addr, HD, alpha);
        tc_fence_before();
        l *= alpha;
      }
      m_ref = m_new;
      return true;
    };
#ifdef AERIS_ATTN_TRACE
    const bool trace_on = g_attn_trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 &&
                          warp == 2 && lane == 0;
#endif
    for (int j = 0; j < nkv && ok && warp_valid; ++j) {
      const bool last = (j == nkv - 1);
      ATTN_STAMP(0);
      const uint32_t tSj = tS;
      if (!mbar_wait(s_full, j & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
      tc_fence_after();
      ATTN_STAMP(1);
      bool waited = false;
      if (!last || rem == 0) {
        // full 64-column tile: one TMEM read, scores stay in registers, the TMEM buffer is released at once
        uint32_t v0[32], v1[32];
        if (warp_valid) {
          tmem_ld32(tSj + lane_addr, v0);
          tmem_ld32(tSj + lane_addr + 32, v1);
          tmem_wait_ld();
        }
        ATTN_STAMP(2);
        if constexpr (!PTMEM) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_free);
        }
        if (warp_valid) {
          // four independent chains of eight 3-input maxima instead of one chain of thirty-two
          float mxc[4];
#pragma unroll
          for (int c = 0; c < 4; ++c)
            mxc[c] = fmaxf(__uint_as_float(v0[c]), __uint_as_float(v1[c]));
#pragma unroll
          for (int i = 1; i < 8; ++i) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
              mxc[c] = max3(mxc[c], __uint_as_float(v0[4 * i + c]), __uint_as_float(v1[4 * i + c]));
          }
          const float mx = fmaxf(max3(mxc[0], mxc[1], mxc[2]), mxc[3]);
          const float m_new = fmaxf(m_ref, mx * sl2);
          if (__any_sync(0xffffffffu, m_new - m_ref > RESCALE_LOG2)) {
            if (!rescale(j, m_new, waited)) { ok = false; break; }
          }
          ATTN_STAMP(3);
          uint32_t pk[32];
          if constexpr (POLY >= 0) {
            l += softmax_row64<POLY>(v0, v1, sl2, m_ref, pk);
          } else {
            float rs[4] = {0.f, 0.f, 0.f, 0.f};
  #pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float p0 = fast_exp2(fmaf(__uint_as_float(v0[2 * i]), sl2, -m_ref));
              const float p1 = fast_exp2(fmaf(__uint_as_float(v0[2 * i + 1]), sl2, -m_ref));
              rs[(2 * i) & 3] += p0; rs[(2 * i + 1) & 3] += p1;
              pk[i] = pack_bf16x2(p0, p1);
            }
  #pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float p0 = fast_exp2(fmaf(__uint_as_float(v1[2 * i]), sl2, -m_ref));
              const float p1 = fast_exp2(fmaf(__uint_as_float(v1[2 * i + 1]), sl2, -m_ref));
              rs[(2 * i) & 3] += p0; rs[(2 * i + 1) & 3] += p1;
              pk[16 + i] = pack_bf16x2(p0, p1);
            }
            l += (rs[0] + rs[1]) + (rs[2] + rs[3]);
          }
          ATTN_STAMP(4);
          if constexpr (PTMEM) {
            // scores of tile j exist, so P V of tile j - 1 (issued before them) is done: the columns are this thread's
            tmem_st32(tSj + lane_addr, pk);
            tmem_wait_st();
          } else {
            if (j > 0 && !waited && !mbar_wait(pv_done, (j - 1) & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
#pragma unroll
            for (int g = 0; g < 8; ++g)
              *reinterpret_cast<uint4*>(sP + swz128(row, g)) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
          }
        }
      } else {
        // last, partial tile: n_last (multiple of 16) columns computed, `rem` of them valid; no tile follows
        if (warp_valid) {
          float mx = -INFINITY;
#pragma unroll 1
          for (int c = 0; c < n_last; c += 16) {
            uint32_t v[16];
            tmem_ld16(tSj + lane_addr + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (c + i < rem) mx = fmaxf(mx, __uint_as_float(v[i]));
          }
          const float m_new = fmaxf(m_ref, mx * sl2);
          if (__any_sync(0xffffffffu, m_new - m_ref > RESCALE_LOG2)) {
            if (!rescale(j, m_new, waited)) { ok = false; break; }
          }
          if constexpr (!PTMEM) {
            if (j > 0 && !waited && !mbar_wait(pv_done, (j - 1) & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
          }
          float rs = 0.f;
#pragma unroll 1
          for (int c = 0; c < n_last; c += 16) {
            uint32_t v[16], pk[8];
            tmem_ld16(tSj + lane_addr + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float p0 = fast_exp2(fmaf(__uint_as_float(v[2 * i]), sl2, -m_ref));
              float p1 = fast_exp2(fmaf(__uint_as_float(v[2 * i + 1]), sl2, -m_ref));
              if (c + 2 * i >= rem) p0 = 0.f;
              if (c + 2 * i + 1 >= rem) p1 = 0.f;
              rs += p0 + p1;
              pk[i] = pack_bf16x2(p0, p1);
            }
            if constexpr (PTMEM) {
              // 16 scores become 8 columns of bf16 pairs at column c / 2 <= c: only scores already consumed are overwritten
              tmem_st8(tSj + lane_addr + (c >> 1), pk);
            } else {
#pragma unroll
              for (int g = 0; g < 2; ++g)
                *reinterpret_cast<uint4*>(sP + swz128(row, (c >> 3) + g)) =
                    make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
            }
          }
          if constexpr (PTMEM) tmem_wait_st();
          l += rs;
        }
        if constexpr (!PTMEM) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_free);
        }
      }
      ATTN_STAMP(5);
      if constexpr (!PTMEM) fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      ATTN_STAMP(6);
    }
    if (ok && warp_valid && mbar_wait(pv_done, (nkv - 1) & 1, p.status, ERR_TIMEOUT_ATTN)) {
      tc_fence_after();
      {
        const float inv = 1.f / l;
        const size_t trow = static_cast<size_t>(win) * N + grow;
        __nv_bfloat16* dst = (p.O && grow < N) ? p.O + trow * p.ldo + head * HD : nullptr;
        __nv_bfloat16* pdst = nullptr;
        if (p.push_n_local > 0 && grow < N) {
          const int owner = grow / p.push_n_local;
          pdst = reinterpret_cast<__nv_bfloat16*>(p.o_peers[owner]) +
                 (static_cast<size_t>(win) * p.push_n_local + (grow - owner * p.push_n_local)) * p.push_ld +
                 p.push_col0 + head * HD;
        }
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t v[32];
          tmem_ld32(tO + lane_addr + c, v);
          tmem_wait_ld();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(v[8 * g]) * inv, __uint_as_float(v[8 * g + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv);
            if (dst) *reinterpret_cast<uint4*>(dst + c + 8 * g) = u;
            if (pdst) *reinterpret_cast<uint4*>(pdst + c + 8 * g) = u;
          }
        }
        if (p.lse && grow < N) p.lse[(static_cast<size_t>(win) * p.H + head) * N + grow] = m_ref + log2f(l);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

static int g_fwd_smem_pad = 0;   // extra dynamic shared memory per CTA: lowers the number of CTAs per SM (measurements)

template <int DCH, int POLY, int MODE>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const AttnFwdParams& p, cudaStream_t stream) {
  constexpr int SMEM = DCH * 16384 + (AttnFwdRing<DCH, MODE>::NSK + AttnFwdRing<DCH, MODE>::NSV) * DCH * 8192 +
                       (MODE != 0 ? 0 : 16384) + 256;
  static int configured = -1;
  auto kern = attn_fwd_kernel<DCH, POLY, MODE>;
  const int smem = SMEM + g_fwd_smem_pad;
  if (configured != smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
    configured = smem;
  }
  dim3 grid((p.N + TILE - 1) / TILE, p.H, p.n_win);
  kern<<<grid, ATT_THREADS, smem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}


// -------------------------------------------------------------------------------------------------------- backward
// Two kernels, neither needs atomics:
//   attn_bwd_dq : one CTA per 128-row Q tile, streams K/V in 64-row tiles.  S = Q K^T, dP = dO V^T,
//                 dS = P * (dP - delta) * scale, dQ += dS K.   Also writes delta = rowsum(dO * O).
//   attn_bwd_dkv: one CTA per 128-row K/V tile, streams Q/dO in 64-row tiles. S^T = K Q^T, dP^T = V dO^T,
//                 dV += P^T dO, dK += dS^T Q.
struct AttnBwdParams {
  const __nv_bfloat16* O;   // forward output, [T, ldo]
  const __nv_bfloat16* dO;  // [T, ldo]
  int ldo;
  const float* lse;         // [n_win*H*N] log2 domain
  float* delta;             // [n_win*H*N]
  __nv_bfloat16* dQKV;      // [T, ldg] gradient of the fused qkv tensor
  int ldg;
  int N, H, n_win;
  int q_col0, k_col0, v_col0;
  float scale_log2, scale;
  int* status;
  // Ulysses gradient push (null / 0 when unused): the gradient row of token `grow` goes to rank grow / push_n_local,
  // row win * push_n_local + grow % push_n_local, column section * push_sec_w + push_col0 + head * d.
  void* dq_peers[8];
  int push_n_local, push_ld, push_sec_w, push_col0;
};
constexpr int BT = 64;

template <int HD>
__device__ __forceinline__ __nv_bfloat16* bwd_dst(const AttnBwdParams& p, int win, int grow, int head, int section,
                                                  int local_col0) {
  if (p.push_n_local > 0) {
    const int owner = grow / p.push_n_local;
    return reinterpret_cast<__nv_bfloat16*>(p.dq_peers[owner]) +
           (static_cast<size_t>(win) * p.push_n_local + (grow - owner * p.push_n_local)) * p.push_ld +
           section * p.push_sec_w + p.push_col0 + head * HD;
  }
  return p.dQKV + (static_cast<size_t>(win) * p.N + grow) * p.ldg + local_col0 + head * HD;
}  // streamed tile rows in the backward kernels

// Both backward kernels stream 64-row tiles but run the tensor core and the math warps at a granularity of 32 score
// columns ("halves"), double buffered in TMEM: while the math warps turn half g into dS (and P), the tensor core is
// already computing the scores of half g+1, and the accumulating products of half g are issued as soon as its
// operands are in shared memory. Half g uses buffer g & 1; only the last streamed tile can have a single half.
__device__ __forceinline__ int half_cols(int g, int n_tiles, int n_last) {
  const int j = g >> 1, h = g & 1;
  return (j == n_tiles - 1) ? min(32, n_last - 32 * h) : 32;
}

template <int DCH>
__global__ void __launch_bounds__(ATT_THREADS, (DCH == 1) ? 2 : 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                   const AttnBwdParams p) {
  constexpr int HD = 64 * DCH;
  constexpr int QB = DCH * 16384;       // Q tile, dO tile (128 rows)
  constexpr int KB = DCH * 8192;        // K tile, V tile (64 rows)
  constexpr int STAGE = 2 * KB;
  constexpr int NST = 3;
  constexpr int TMEM_COLS = 256;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + QB;
  uint8_t* sKV = sdO + QB;
  uint8_t* sdS = sKV + NST * STAGE;  // [128 x 64] bf16
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 16384);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [3]
  uint64_t* kv_empty = bars + 4;   // [3]
  uint64_t* sp_full = bars + 7;    // [2]
  uint64_t* ds_full = bars + 9;    // [2]
  uint64_t* dq_full = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, head = blockIdx.y, win = blockIdx.z;
  const int N = p.N;
  const int nfull = N / BT, rem = N - nfull * BT;
  const int nkv = nfull + (rem ? 1 : 0);
  const int n_last = rem ? ((rem + 15) & ~15) : BT;
  const int G = 2 * (nkv - 1) + (n_last > 32 ? 2 : 1);   // number of halves

  if (threadIdx.x == 0) {
    int ab = (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    if ((smem_u32(smem) & 1023u) != 0) { ab = 1; if (p.status) atomicCAS(p.status, 0, ERR_BOUNDS); }
    *s_abort = ab;
  }
  __syncthreads();
  if (*s_abort) return;
  if (threadIdx.x == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_do);
    mbar_init(q_full, 1);
    for (int i = 0; i < NST; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sp_full[i], 1); mbar_init(&ds_full[i], 4); }
    mbar_init(dq_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tdQ = tmem_base + 128;   // S[2] and dP[2]: 32 columns each

  if (warp == 0) {
    if (elect_one_sync()) {
      mbar_expect_tx(q_full, 2 * QB);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_3d(sQ + c * 16384, &tm_q, q_full, p.q_col0 + head * HD + c * 64, qt * TILE, win);
        tma_load_3d(sdO + c * 16384, &tm_do, q_full, head * HD + c * 64, qt * TILE, win);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < nkv; ++j) {
        if (!mbar_wait(&kv_empty[st], ph ^ 1, p.status, ERR_TIMEOUT_ATTN)) break;
        uint8_t* sK = sKV + st * STAGE;
        uint8_t* sV = sK + KB;
        mbar_expect_tx(&kv_full[st], STAGE);
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          tma_load_3d(sK + c * 8192, &tm_k, &kv_full[st], p.k_col0 + head * HD + c * 64, j * BT, win);
          tma_load_3d(sV + c * 8192, &tm_v, &kv_full[st], p.v_col0 + head * HD + c * 64, j * BT, win);
        }
        if (++st == NST) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      bool ok = mbar_wait(q_full, 0, p.status, ERR_TIMEOUT_ATTN);
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), adS = smem_u32(sdS), aKV = smem_u32(sKV);
      // S[h] = Q K[32h..]^T and dP[h] = dO V[32h..]^T for half g
      auto issue_sp = [&](int g) -> bool {
        const int j = g >> 1, h = g & 1, st = j % NST;
        if (h == 0 && !mbar_wait(&kv_full[st], (j / NST) & 1, p.status, ERR_TIMEOUT_ATTN)) return false;
        tc_fence_after();
        const int nc = half_cols(g, nkv, n_last);
        const uint32_t aK = aKV + st * STAGE + h * 4096, aV = aK + KB;
        const uint32_t idesc_s = make_idesc_bf16(TILE, nc, 0, 0);
#pragma unroll
        for (int kk = 0; kk < 4 * DCH; ++kk) {
          const uint32_t qoff = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t koff = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_ss(tS + h * 32, make_smem_desc(aQ + qoff, 0, 1024), make_smem_desc(aK + koff, 0, 1024), idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < 4 * DCH; ++kk) {
          const uint32_t qoff = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t koff = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_ss(tdP + h * 32, make_smem_desc(adO + qoff, 0, 1024), make_smem_desc(aV + koff, 0, 1024), idesc_s, kk > 0);
        }
        tc_commit(&sp_full[h]);
        return true;
      };
      if (ok) ok = issue_sp(0);
      if (ok && G > 1) ok = issue_sp(1);
      for (int g = 0; g < G && ok; ++g) {
        const int j = g >> 1, h = g & 1, st = j % NST;
        const int nc = half_cols(g, nkv, n_last);
        if (!mbar_wait(&ds_full[h], (g >> 1) & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
        tc_fence_after();
        // dQ += dS[:, half] K[half rows] : A = dS (K-major over kv), B = K MN-major (d contiguous, kv rows strided)
        const uint32_t aK = aKV + st * STAGE;
        const uint32_t idesc_dq = make_idesc_bf16(TILE, HD, 0, 1);
        for (int kk = 0; kk < nc / 16; ++kk) {
          const int k16 = 2 * h + kk;   // 16-column group inside the 64-column tile
          umma_ss(tdQ, make_smem_desc(adS + k16 * 32, 0, 1024), make_smem_desc(aK + k16 * 2048, 8192, 1024), idesc_dq,
                  (g > 0 || kk > 0) ? 1u : 0u);
        }
        const bool tile_done = (h == 1) || (g == G - 1);
        if (tile_done) tc_commit(&kv_empty[st]);
        if (g + 2 < G) ok = issue_sp(g + 2);
      }
      if (ok) tc_commit(dq_full);
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int grow = qt * TILE + row;
    const bool row_ok = grow < N;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const size_t trow = static_cast<size_t>(win) * N + (row_ok ? grow : 0);
    const size_t sidx = (static_cast<size_t>(win) * p.H + head) * N + (row_ok ? grow : 0);
    float lse = 0.f, delta = 0.f;
    if (row_ok) {
      lse = p.lse[sidx];
      const __nv_bfloat16* o = p.O + trow * p.ldo + head * HD;
      const __nv_bfloat16* go = p.dO + trow * p.ldo + head * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        const uint4 a = *reinterpret_cast<const uint4*>(o + c), b = *reinterpret_cast<const uint4*>(go + c);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 x = unpack_bf16x2(aw[i]), y = unpack_bf16x2(bw[i]);
          delta = fmaf(x.x, y.x, delta);
          delta = fmaf(x.y, y.y, delta);
        }
      }
      p.delta[sidx] = delta;
    }
    const float sl2 = p.scale_log2, sc = p.scale;
    bool ok = true;
    for (int g = 0; g < G && ok; ++g) {
      const int j = g >> 1, h = g & 1;
      const bool last = (j == nkv - 1);
      const int nc = half_cols(g, nkv, n_last);
      const int valid = (last && rem) ? rem - 32 * h : 32;     // valid columns inside this half
      if (!mbar_wait(&sp_full[h], (g >> 1) & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
      tc_fence_after();
      if (nc == 32 && valid >= 32) {
        uint32_t sv[32], dv[32];
        tmem_ld32(tS + h * 32 + lane_addr, sv);
        tmem_ld32(tdP + h * 32 + lane_addr, dv);
        tmem_wait_ld();
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
          uint32_t pk[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int e = 8 * gq + 2 * i;
            const float p0 = fast_exp2(fmaf(__uint_as_float(sv[e]), sl2, -lse));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sv[e + 1]), sl2, -lse));
            float d0 = p0 * (__uint_as_float(dv[e]) - delta) * sc;
            float d1 = p1 * (__uint_as_float(dv[e + 1]) - delta) * sc;
            if (!row_ok) { d0 = 0.f; d1 = 0.f; }
            pk[i] = pack_bf16x2(d0, d1);
          }
          *reinterpret_cast<uint4*>(sdS + swz128(row, 4 * h + gq)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < nc; c += 16) {
          uint32_t sv[16], dv[16], pk[8];
          tmem_ld16(tS + h * 32 + lane_addr + c, sv);
          tmem_ld16(tdP + h * 32 + lane_addr + c, dv);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sv[2 * i]), sl2, -lse));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sv[2 * i + 1]), sl2, -lse));
            float d0 = p0 * (__uint_as_float(dv[2 * i]) - delta) * sc;
            float d1 = p1 * (__uint_as_float(dv[2 * i + 1]) - delta) * sc;
            if (c + 2 * i >= valid || !row_ok) d0 = 0.f;
            if (c + 2 * i + 1 >= valid || !row_ok) d1 = 0.f;
            pk[i] = pack_bf16x2(d0, d1);
          }
#pragma unroll
          for (int gq = 0; gq < 2; ++gq)
            *reinterpret_cast<uint4*>(sdS + swz128(row, 4 * h + (c >> 3) + gq)) =
                make_uint4(pk[4 * gq], pk[4 * gq + 1], pk[4 * gq + 2], pk[4 * gq + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[h]);
    }
    if (ok && mbar_wait(dq_full, 0, p.status, ERR_TIMEOUT_ATTN)) {
      tc_fence_after();
      __nv_bfloat16* dst = bwd_dst<HD>(p, win, row_ok ? grow : 0, head, 0, p.q_col0);
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t v[32];
        tmem_ld32(tdQ + lane_addr + c, v);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int gq = 0; gq < 4; ++gq)
            *reinterpret_cast<uint4*>(dst + c + gq * 8) = make_uint4(
                pack_bf16x2(__uint_as_float(v[8 * gq]), __uint_as_float(v[8 * gq + 1])),
                pack_bf16x2(__uint_as_float(v[8 * gq + 2]), __uint_as_float(v[8 * gq + 3])),
                pack_bf16x2(__uint_as_float(v[8 * gq + 4]), __uint_as_float(v[8 * gq + 5])),
                pack_bf16x2(__uint_as_float(v[8 * gq + 6]), __uint_as_float(v[8 * gq + 7])));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int DCH>
__global__ void __launch_bounds__(ATT_THREADS, (DCH == 1) ? 2 : 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                    const AttnBwdParams p, const int stat_floats) {
  constexpr int HD = 64 * DCH;
  constexpr int KB = DCH * 16384;  // K tile, V tile (128 rows)
  constexpr int QB = DCH * 8192;   // Q tile, dO tile (64 rows)
  constexpr int STAGE = 2 * QB;
  constexpr int NST = 2;
  constexpr int TMEM_COLS = (DCH == 1) ? 256 : 512;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = sK + KB;
  uint8_t* sQD = sV + KB;
  uint8_t* sPT = sQD + NST * STAGE;  // [128 x 64] bf16
  uint8_t* sdST = sPT + 16384;       // [128 x 64] bf16
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdST + 16384);
  uint64_t* k_full = bars;
  uint64_t* qd_full = bars + 1;    // [2]
  uint64_t* qd_empty = bars + 3;   // [2]
  uint64_t* sp_full = bars + 5;    // [2]
  uint64_t* pd_full = bars + 7;    // [2]
  uint64_t* acc_full = bars + 9;
  uint64_t* stat_bar = bars + 10;  // lse/delta of the whole window staged in shared memory (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
  float* s_lse = reinterpret_cast<float*>(bars + 16);   // [stat_floats] then delta [stat_floats]
  float* s_delta = s_lse + stat_floats;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, head = blockIdx.y, win = blockIdx.z;
  const int N = p.N;
  const int nfull = N / BT, rem = N - nfull * BT;
  const int nq = nfull + (rem ? 1 : 0);
  const int n_last = rem ? ((rem + 15) & ~15) : BT;
  const int G = 2 * (nq - 1) + (n_last > 32 ? 2 : 1);

  if (threadIdx.x == 0) {
    int ab = (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    if ((smem_u32(smem) & 1023u) != 0) { ab = 1; if (p.status) atomicCAS(p.status, 0, ERR_BOUNDS); }
    *s_abort = ab;
  }
  __syncthreads();
  if (*s_abort) return;
  if (threadIdx.x == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_do);
    mbar_init(k_full, 1);
    for (int i = 0; i < NST; ++i) { mbar_init(&qd_full[i], 1); mbar_init(&qd_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sp_full[i], 1); mbar_init(&pd_full[i], 4); }
    mbar_init(acc_full, 1); mbar_init(stat_bar, 128);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tdK = tmem_base + 128, tdV = tmem_base + 128 + HD;

  if (warp == 0) {
    if (elect_one_sync()) {
      mbar_expect_tx(k_full, 2 * KB);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_3d(sK + c * 16384, &tm_k, k_full, p.k_col0 + head * HD + c * 64, kt * TILE, win);
        tma_load_3d(sV + c * 16384, &tm_v, k_full, p.v_col0 + head * HD + c * 64, kt * TILE, win);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int i = 0; i < nq; ++i) {
        if (!mbar_wait(&qd_empty[st], ph ^ 1, p.status, ERR_TIMEOUT_ATTN)) break;
        uint8_t* sQ = sQD + st * STAGE;
        uint8_t* sdO = sQ + QB;
        mbar_expect_tx(&qd_full[st], STAGE);
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          tma_load_3d(sQ + c * 8192, &tm_q, &qd_full[st], p.q_col0 + head * HD + c * 64, i * BT, win);
          tma_load_3d(sdO + c * 8192, &tm_do, &qd_full[st], head * HD + c * 64, i * BT, win);
        }
        if (++st == NST) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      bool ok = mbar_wait(k_full, 0, p.status, ERR_TIMEOUT_ATTN);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aPT = smem_u32(sPT), adST = smem_u32(sdST);
      const uint32_t aQD = smem_u32(sQD);
      auto issue_sp = [&](int g) -> bool {
        const int i = g >> 1, h = g & 1, st = i % NST;
        if (h == 0 && !mbar_wait(&qd_full[st], (i / NST) & 1, p.status, ERR_TIMEOUT_ATTN)) return false;
        tc_fence_after();
        const int nc = half_cols(g, nq, n_last);
        const uint32_t aQ = aQD + st * STAGE + h * 4096, adO = aQ + QB;
        const uint32_t idesc_s = make_idesc_bf16(TILE, nc, 0, 0);
#pragma unroll
        for (int kk = 0; kk < 4 * DCH; ++kk) {
          const uint32_t koff = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t qoff = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_ss(tS + h * 32, make_smem_desc(aK + koff, 0, 1024), make_smem_desc(aQ + qoff, 0, 1024), idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < 4 * DCH; ++kk) {
          const uint32_t koff = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t qoff = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_ss(tdP + h * 32, make_smem_desc(aV + koff, 0, 1024), make_smem_desc(adO + qoff, 0, 1024), idesc_s, kk > 0);
        }
        tc_commit(&sp_full[h]);
        return true;
      };
      if (ok) ok = issue_sp(0);
      if (ok && G > 1) ok = issue_sp(1);
      for (int g = 0; g < G && ok; ++g) {
        const int i = g >> 1, h = g & 1, st = i % NST;
        const int nc = half_cols(g, nq, n_last);
        if (!mbar_wait(&pd_full[h], (g >> 1) & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aQ = aQD + st * STAGE, adO = aQ + QB;
        const uint32_t idesc_acc = make_idesc_bf16(TILE, HD, 0, 1);
        for (int kk = 0; kk < nc / 16; ++kk) {
          const int k16 = 2 * h + kk;
          const uint32_t acc = (g > 0 || kk > 0) ? 1u : 0u;
          umma_ss(tdV, make_smem_desc(aPT + k16 * 32, 0, 1024), make_smem_desc(adO + k16 * 2048, 8192, 1024),
                  idesc_acc, acc);
          umma_ss(tdK, make_smem_desc(adST + k16 * 32, 0, 1024), make_smem_desc(aQ + k16 * 2048, 8192, 1024),
                  idesc_acc, acc);
        }
        const bool tile_done = (h == 1) || (g == G - 1);
        if (tile_done) tc_commit(&qd_empty[st]);
        if (g + 2 < G) ok = issue_sp(g + 2);
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;  // kv row within the tile
    const int grow = kt * TILE + row;
    const bool row_ok = grow < N;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const int t128 = threadIdx.x - 64;  // 0..127 among the four math warps
    const size_t sbase = (static_cast<size_t>(win) * p.H + head) * N;
    // stage lse and delta of every query row of this (window, head) once
    for (int i = t128; i < stat_floats; i += 128) {
      s_lse[i] = (i < N) ? p.lse[sbase + i] : 0.f;
      s_delta[i] = (i < N) ? p.delta[sbase + i] : 0.f;
    }
    mbar_arrive(stat_bar);
    bool ok = mbar_wait(stat_bar, 0, p.status, ERR_TIMEOUT_ATTN);
    const float sl2 = p.scale_log2, sc = p.scale;
    for (int g = 0; g < G && ok; ++g) {
      const int i = g >> 1, h = g & 1;
      const bool last = (i == nq - 1);
      const int nc = half_cols(g, nq, n_last);
      const int valid = (last && rem) ? rem - 32 * h : 32;
      const float* ls = s_lse + i * BT + 32 * h;
      const float* de = s_delta + i * BT + 32 * h;
      if (!mbar_wait(&sp_full[h], (g >> 1) & 1, p.status, ERR_TIMEOUT_ATTN)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < nc; c += 16) {
        uint32_t sv[16], dv[16], pp[8], dd[8];
        tmem_ld16(tS + h * 32 + lane_addr + c, sv);
        tmem_ld16(tdP + h * 32 + lane_addr + c, dv);
        float lq[16], dq[16];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float4 a = *reinterpret_cast<const float4*>(ls + c + 4 * k);
          const float4 b = *reinterpret_cast<const float4*>(de + c + 4 * k);
          lq[4 * k] = a.x; lq[4 * k + 1] = a.y; lq[4 * k + 2] = a.z; lq[4 * k + 3] = a.w;
          dq[4 * k] = b.x; dq[4 * k + 1] = b.y; dq[4 * k + 2] = b.z; dq[4 * k + 3] = b.w;
        }
        tmem_wait_ld();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float p0 = fast_exp2(fmaf(__uint_as_float(sv[2 * k]), sl2, -lq[2 * k]));
          float p1 = fast_exp2(fmaf(__uint_as_float(sv[2 * k + 1]), sl2, -lq[2 * k + 1]));
          if (c + 2 * k >= valid || !row_ok) p0 = 0.f;
          if (c + 2 * k + 1 >= valid || !row_ok) p1 = 0.f;
          const float d0 = p0 * (__uint_as_float(dv[2 * k]) - dq[2 * k]) * sc;
          const float d1 = p1 * (__uint_as_float(dv[2 * k + 1]) - dq[2 * k + 1]) * sc;
          pp[k] = pack_bf16x2(p0, p1);
          dd[k] = pack_bf16x2(d0, d1);
        }
#pragma unroll
        for (int gq = 0; gq < 2; ++gq) {
          const uint32_t off = swz128(row, 4 * h + (c >> 3) + gq);
          *reinterpret_cast<uint4*>(sPT + off) = make_uint4(pp[4 * gq], pp[4 * gq + 1], pp[4 * gq + 2], pp[4 * gq + 3]);
          *reinterpret_cast<uint4*>(sdST + off) = make_uint4(dd[4 * gq], dd[4 * gq + 1], dd[4 * gq + 2], dd[4 * gq + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pd_full[h]);
    }
    if (ok && mbar_wait(acc_full, 0, p.status, ERR_TIMEOUT_ATTN)) {
      tc_fence_after();
      const size_t trow = static_cast<size_t>(win) * N + (row_ok ? grow : 0);
      __nv_bfloat16* dk = bwd_dst<HD>(p, win, row_ok ? grow : 0, head, 1, p.k_col0);
      __nv_bfloat16* dv = bwd_dst<HD>(p, win, row_ok ? grow : 0, head, 2, p.v_col0);
      (void)trow;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t t = which ? tdV : tdK;
        __nv_bfloat16* dst = which ? dv : dk;
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t v[32];
          tmem_ld32(t + lane_addr + c, v);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int gq = 0; gq < 4; ++gq)
              *reinterpret_cast<uint4*>(dst + c + gq * 8) = make_uint4(
                  pack_bf16x2(__uint_as_float(v[8 * gq]), __uint_as_float(v[8 * gq + 1])),
                  pack_bf16x2(__uint_as_float(v[8 * gq + 2]), __uint_as_float(v[8 * gq + 3])),
                  pack_bf16x2(__uint_as_float(v[8 * gq + 4]), __uint_as_float(v[8 * gq + 5])),
                  pack_bf16x2(__uint_as_float(v[8 * gq + 6]), __uint_as_float(v[8 * gq + 7])));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int DCH>
static int launch_attn_bwd(const CUtensorMap& tq128, const CUtensorMap& tk64, const CUtensorMap& tv64,
                           const CUtensorMap& tdo128, const CUtensorMap& tq64, const CUtensorMap& tk128,
                           const CUtensorMap& tv128, const CUtensorMap& tdo64, const AttnBwdParams& p,
                           cudaStream_t stream) {
  const int stat_floats = ((p.N + BT - 1) / BT) * BT;      // lse and delta of one window, padded to whole tiles
  const int SMEM_DQ = 2 * DCH * 16384 + 3 * 2 * DCH * 8192 + 16384 + 128;
  const int SMEM_DKV = 2 * DCH * 16384 + 2 * 2 * DCH * 8192 + 2 * 16384 + 128 + 2 * stat_floats * 4;
  if (SMEM_DKV > 227 * 1024) return -23;
  auto k1 = attn_bwd_dq_kernel<DCH>;
  auto k2 = attn_bwd_dkv_kernel<DCH>;
  static int configured_dkv = 0;
  static bool configured_dq = false;
  if (!configured_dq) {
    if (cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DQ) != cudaSuccess) return -20;
    configured_dq = true;
  }
  if (configured_dkv < SMEM_DKV) {
    if (cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DKV) != cudaSuccess) return -20;
    configured_dkv = SMEM_DKV;
  }
  dim3 grid((p.N + TILE - 1) / TILE, p.H, p.n_win);
  k1<<<grid, ATT_THREADS, SMEM_DQ, stream>>>(tq128, tk64, tv64, tdo128, p);
  if (cudaGetLastError() != cudaSuccess) return -21;
  k2<<<grid, ATT_THREADS, SMEM_DKV, stream>>>(tq64, tk128, tv128, tdo64, p, stat_floats);
  return cudaGetLastError() == cudaSuccess ? 0 : -22;
}

}  // namespace aeris

using namespace aeris;

// Variant of the forward kernel. poly (head_dim 64 only): -1 = scalar softmax arithmetic, exp unit only; 0 = two-wide
// fp32 arithmetic; 2 = two-wide with two of every eight score pairs on the polynomial exp2. mode: see AttnFwdRing
// (0 probabilities through shared memory; 1 in tensor memory; 2 in tensor memory, four CTAs per SM).
static int g_fwd_poly = -1;
static int g_fwd_mode = 0;
extern "C" int aeris_attn_set_fwd_variant(int poly, int mode) {
  if ((poly != -1 && poly != 0 && poly != 2) || mode < 0 || mode > 2) return -1;
  g_fwd_poly = poly;
  g_fwd_mode = mode;
  return 0;
}
#ifdef AERIS_ATTN_TRACE
extern "C" int aeris_attn_set_trace(long long* buf) {
  return cudaMemcpyToSymbol(aeris::g_attn_trace, &buf, sizeof(buf)) == cudaSuccess ? 0 : -1;
}
#endif
extern "C" int aeris_attn_set_fwd_smem_pad(int bytes) {
  if (bytes < 0 || bytes > 160 * 1024) return -1;
  g_fwd_smem_pad = bytes;
  return 0;
}

// q, k, v: base pointers of row-major [n_win * N, ld*] bf16 tensors; *_col0 = column of head 0.
static int attn_fwd_impl(const void* q, int ldq, int q_col0, const void* k, int ldk, int k_col0, const void* v,
                         int ldv, int v_col0, void* o, int ldo, float* lse, int n_win, int N, int H, int head_dim,
                         float scale, int* status, void* stream_, const void* const* o_peers, int sp,
                         int push_n_local, int push_ld, int push_col0);

extern "C" int aeris_attn_fwd(const void* q, int ldq, int q_col0, const void* k, int ldk, int k_col0, const void* v,
                              int ldv, int v_col0, void* o, int ldo, float* lse, int n_win, int N, int H,
                              int head_dim, float scale, int* status, void* stream_) {
  return attn_fwd_impl(q, ldq, q_col0, k, ldk, k_col0, v, ldv, v_col0, o, ldo, lse, n_win, N, H, head_dim, scale, status,
                       stream_, nullptr, 0, 0, 0, 0);
}

// Forward whose output rows are (also) pushed to the ranks that own the tokens (Ulysses return exchange fused into the
// attention epilogue). `o` may be null when only the pushed copy is wanted.
extern "C" int aeris_attn_fwd_push(const void* qkv, int ld, int H_local, void* o, int ldo, float* lse, int n_win, int N,
                                   int head_dim, float scale, const void* const* o_peers, int sp, int n_local,
                                   int push_ld, int push_col0, int* status, void* stream_) {
  const int hd = H_local * head_dim;
  return attn_fwd_impl(qkv, ld, 0, qkv, ld, hd, qkv, ld, 2 * hd, o, ldo, lse, n_win, N, H_local, head_dim, scale,
                       status, stream_, o_peers, sp, n_local, push_ld, push_col0);
}

static int attn_fwd_impl(const void* q, int ldq, int q_col0, const void* k, int ldk, int k_col0, const void* v,
                         int ldv, int v_col0, void* o, int ldo, float* lse, int n_win, int N, int H, int head_dim,
                         float scale, int* status, void* stream_, const void* const* o_peers, int sp,
                         int push_n_local, int push_ld, int push_col0) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (head_dim != 64 && head_dim != 128) return -1;
  if (n_win <= 0 || N <= 0 || H <= 0 || n_win > 65535 || H > 65535) return -2;
  if (sp < 0 || sp > 8 || (!o && !o_peers)) return -3;
  AttnFwdParams p{};
  for (int i = 0; i < sp; ++i) p.o_peers[i] = const_cast<void*>(o_peers[i]);
  p.push_n_local = o_peers ? push_n_local : 0; p.push_ld = push_ld; p.push_col0 = push_col0;
  p.O = reinterpret_cast<__nv_bfloat16*>(o); p.ldo = ldo; p.lse = lse; p.N = N; p.H = H; p.n_win = n_win;
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_tmap_3d_bf16(&tq, q, ldq, N, n_win, ldq, static_cast<uint64_t>(N) * ldq, 64, TILE))) return r;
  if ((r = make_tmap_3d_bf16(&tk, k, ldk, N, n_win, ldk, static_cast<uint64_t>(N) * ldk, 64, KVT))) return r;
  if ((r = make_tmap_3d_bf16(&tv, v, ldv, N, n_win, ldv, static_cast<uint64_t>(N) * ldv, 64, KVT))) return r;
  if (head_dim == 128) {
    switch (g_fwd_mode) {
      case 1: return launch_attn_fwd<2, -1, 1>(tq, tk, tv, p, stream);
      default: return launch_attn_fwd<2, -1, 0>(tq, tk, tv, p, stream);
    }
  }
  const bool poly = g_fwd_poly == 2;
  switch (g_fwd_mode) {
    case 1: return poly ? launch_attn_fwd<1, 2, 1>(tq, tk, tv, p, stream) : launch_attn_fwd<1, -1, 1>(tq, tk, tv, p, stream);
    case 2: return launch_attn_fwd<1, -1, 2>(tq, tk, tv, p, stream);
    default: break;
  }
  if (g_fwd_poly == 0) return launch_attn_fwd<1, 0, 0>(tq, tk, tv, p, stream);
  return poly ? launch_attn_fwd<1, 2, 0>(tq, tk, tv, p, stream) : launch_attn_fwd<1, -1, 0>(tq, tk, tv, p, stream);
}

// Backward. qkv: fused [T, ldq] tensor (q/k/v column blocks at *_col0); o, d_o: [T, ldo]; dqkv: [T, ldg] (same
// column layout as qkv); lse from the forward; delta: scratch [n_win*H*N] fp32 written by the first kernel.
static int attn_bwd_impl(const void* qkv, int ldq, int q_col0, int k_col0, int v_col0, const void* o, const void* d_o,
                         int ldo, const float* lse, float* delta, void* dqkv, int ldg, int n_win, int N, int H,
                         int head_dim, float scale, int* status, void* stream_, const void* const* dq_peers, int sp,
                         int push_n_local, int push_ld, int push_sec_w, int push_col0);

extern "C" int aeris_attn_bwd(const void* qkv, int ldq, int q_col0, int k_col0, int v_col0, const void* o,
                              const void* d_o, int ldo, const float* lse, float* delta, void* dqkv, int ldg,
                              int n_win, int N, int H, int head_dim, float scale, int* status, void* stream_) {
  return attn_bwd_impl(qkv, ldq, q_col0, k_col0, v_col0, o, d_o, ldo, lse, delta, dqkv, ldg, n_win, N, H, head_dim,
                       scale, status, stream_, nullptr, 0, 0, 0, 0, 0);
}

// Backward whose dQ / dK / dV rows are pushed to the ranks that own the tokens (layout [tokens_local, 3 * heads * d]).
extern "C" int aeris_attn_bwd_push(const void* qkv, int ld, int H_local, const void* o, const void* d_o, int ldo,
                                   const float* lse, float* delta, int n_win, int N, int head_dim, float scale,
                                   const void* const* dq_peers, int sp, int n_local, int push_ld, int push_sec_w,
                                   int push_col0, int* status, void* stream_) {
  const int hd = H_local * head_dim;
  return attn_bwd_impl(qkv, ld, 0, hd, 2 * hd, o, d_o, ldo, lse, delta, nullptr, 0, n_win, N, H_local, head_dim, scale,
                       status, stream_, dq_peers, sp, n_local, push_ld, push_sec_w, push_col0);
}

static int attn_bwd_impl(const void* qkv, int ldq, int q_col0, int k_col0, int v_col0, const void* o, const void* d_o,
                         int ldo, const float* lse, float* delta, void* dqkv, int ldg, int n_win, int N, int H,
                         int head_dim, float scale, int* status, void* stream_, const void* const* dq_peers, int sp,
                         int push_n_local, int push_ld, int push_sec_w, int push_col0) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (head_dim != 64 && head_dim != 128) return -1;
  if (n_win <= 0 || N <= 0 || H <= 0 || n_win > 65535 || H > 65535) return -2;
  if (sp < 0 || sp > 8 || (!dqkv && !dq_peers)) return -3;
  AttnBwdParams p{};
  for (int i = 0; i < sp; ++i) p.dq_peers[i] = const_cast<void*>(dq_peers[i]);
  p.push_n_local = dq_peers ? push_n_local : 0; p.push_ld = push_ld; p.push_sec_w = push_sec_w; p.push_col0 = push_col0;
  p.O = reinterpret_cast<const __nv_bfloat16*>(o); p.dO = reinterpret_cast<const __nv_bfloat16*>(d_o); p.ldo = ldo;
  p.lse = lse; p.delta = delta; p.dQKV = reinterpret_cast<__nv_bfloat16*>(dqkv); p.ldg = ldg;
  p.N = N; p.H = H; p.n_win = n_win; p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  CUtensorMap t128, t64, d128, d64;
  int r;
  const uint64_t wq = static_cast<uint64_t>(N) * ldq, wo = static_cast<uint64_t>(N) * ldo;
  if ((r = make_tmap_3d_bf16(&t128, qkv, ldq, N, n_win, ldq, wq, 64, TILE))) return r;
  if ((r = make_tmap_3d_bf16(&t64, qkv, ldq, N, n_win, ldq, wq, 64, BT))) return r;
  if ((r = make_tmap_3d_bf16(&d128, d_o, ldo, N, n_win, ldo, wo, 64, TILE))) return r;
  if ((r = make_tmap_3d_bf16(&d64, d_o, ldo, N, n_win, ldo, wo, 64, BT))) return r;
  return head_dim == 64 ? launch_attn_bwd<1>(t128, t64, t64, d128, t64, t128, t128, d64, p, stream)
                        : launch_attn_bwd<2>(t128, t64, t64, d128, t64, t128, t128, d64, p, stream);
}

// ------------------------------------------------------------------------------------------ allocation-free variant
// Same computation as aeris_attn_bwd, for hosts that must not allocate device memory at call time (declared and
// described in noalloc.h). The `delta` scratch (one float per (window, head, token)) lives in this file-scope device
// array instead of a caller-provided buffer. The array name is only a host-side handle: its device address is
// looked up once per device with cudaGetSymbolAddress and that address is what the kernels receive.
#include "noalloc.h"

static __device__ __align__(256) float g_attn_delta_scratch[AERIS_NOALLOC_MAX_SCRATCH_FLOATS];
static float* g_attn_delta_ptr[AERIS_NOALLOC_MAX_DEVICES] = {};

extern "C" int aeris_attn_bwd_noalloc(const void* qkv, int ldq, int q_col0, int k_col0, int v_col0, const void* o,
                                      const void* d_o, int ldo, const float* lse, void* dqkv, int ldg, int n_win,
                                      int N, int H, int head_dim, float scale, int* status, void* stream_) {
  if (n_win <= 0 || N <= 0 || H <= 0) return AERIS_NOALLOC_ERR_BAD_SHAPE;
  const long long need = static_cast<long long>(n_win) * H * N;
  if (need > AERIS_NOALLOC_MAX_SCRATCH_FLOATS) return AERIS_NOALLOC_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= AERIS_NOALLOC_MAX_DEVICES)
    return AERIS_NOALLOC_ERR_DEVICE;
  if (g_attn_delta_ptr[dev] == nullptr) {
    // one-time set-up for this device (which is current): resolve the device address of the scratch array
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_attn_delta_scratch);
    if (e != cudaSuccess || ptr == nullptr) return AERIS_NOALLOC_ERR_SYMBOL;
    g_attn_delta_ptr[dev] = ptr;
  }
  return aeris_attn_bwd(qkv, ldq, q_col0, k_col0, v_col0, o, d_o, ldo, lse, g_attn_delta_ptr[dev], dqkv, ldg, n_win,
                        N, H, head_dim, scale, status, stream_);
}
