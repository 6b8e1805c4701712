// Memory-bound kernels of the Swin block and the optimizer:
//   * AdaLN modulate + RMSNorm, both orderings, forward and backward, with an optional row gather that pulls
//     rows from this GPU or from a peer GPU's buffer (window re-partition / halo exchange for the shifted
//     layers: reference src/aeris_wp_inference/model.py:18-119 does this with blocking send/recv + roll)
//   * SwiGLU forward / backward, gate-weight scaling and gate-gradient finalisation
//   * row gather (re-partition of gradients), sum of squares, fused AdamW (+clip, NaN guard, bf16 cast, EMA)
// Reference math: src/aeris/models/parallel_swin.py:55-59 (modulate), :454-472 (block orderings), :99-100 (SwiGLU);
// optimizer semantics: src/aeris/parallelism/parallel_engine.py:709-738, 832, 862-884.
#include "common.cuh"
#include "api.h"

namespace aeris {

struct PeerPtrs {
  const __nv_bfloat16* p[16];
#ifdef AERIS_BOUNDS_CHECK
  // checking build: every gather code (source rank, source row) is validated before the access; a bad one records
  // ERR_BOUNDS in the status word and the row is read as zeros (never a trap, never the access)
  int n;               // number of valid entries of p
  unsigned src_rows;   // rows of every source buffer (0: unknown, only the rank is checked)
  int* status;
#endif
};

#ifdef AERIS_BOUNDS_CHECK
static unsigned g_chk_src_rows = 0;
static int* g_chk_status = nullptr;
__device__ __forceinline__ bool gather_code_ok(const PeerPtrs& pp, uint32_t code) {
  const unsigned rank = code >> 28, row = code & 0x0fffffffu;
  const bool ok = rank < static_cast<unsigned>(pp.n) && pp.p[rank] != nullptr && (pp.src_rows == 0 || row < pp.src_rows);
  if (!ok && pp.status) atomicCAS(pp.status, 0, ERR_BOUNDS);
  return ok;
}
#define AERIS_GATHER_OK(pp, code) gather_code_ok(pp, code)
#define AERIS_FILL_CHECK(pp, n_peers) do { (pp).n = (n_peers); (pp).src_rows = g_chk_src_rows; (pp).status = g_chk_status; } while (0)
#else
#define AERIS_GATHER_OK(pp, code) true
#define AERIS_FILL_CHECK(pp, n_peers) do { } while (0)
#endif

// Checking build only (no effect otherwise): the status word and the number of rows of the source buffers of the
// gathers launched next. Returns 1 when the library was built with the checks, else 0.
extern "C" int aeris_debug_set_gather_bounds(int* status, unsigned src_rows) {
#ifdef AERIS_BOUNDS_CHECK
  g_chk_status = status;
  g_chk_src_rows = src_rows;
  return 1;
#else
  (void)status; (void)src_rows;
  return 0;
#endif
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void loadf8(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// Block-wide sum of NRED values per thread. `red` holds 2 * NRED * 32 floats (double buffered by `parity`, so one
// __syncthreads per call is enough when calls alternate parity).
template <int NRED>
__device__ __forceinline__ void block_sum(float (&v)[NRED], float* red, int parity) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int k = 0; k < NRED; ++k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[k] += __shfl_xor_sync(0xffffffffu, v[k], o);
  }
  float* slot = red + parity * NRED * 32;
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < NRED; ++k) slot[k * 32 + warp] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < NRED; ++k) {
    float s = 0.f;
    for (int w = 0; w < nwarps; ++w) s += slot[k * 32 + w];
    v[k] = s;
  }
}

// Block-wide sums of FOUR values per thread for CTAs of at most eight warps, built for few instructions: inside a warp
// the four values are folded by halving (lanes that differ in bit 4 split the values two and two, lanes that differ in
// bit 3 one and one: 6 shuffles instead of 20), the four lane groups write value k of warp w to slot k * 8 + w, and
// after one __syncthreads every lane sums one slot row with three more shuffles and fetches the four totals.
// `red`: [2][32] floats zeroed at kernel start (slots of absent warps stay zero), double buffered by `parity`.
__device__ __forceinline__ void block_sum4_shfl(float (&s)[4], float (*red)[32], int parity, int lane, int warp) {
  const bool b4 = lane & 16, b3 = lane & 8;
  float a0 = b4 ? s[2] : s[0], a1 = b4 ? s[3] : s[1];
  const float g0 = b4 ? s[0] : s[2], g1 = b4 ? s[1] : s[3];
  a0 += __shfl_xor_sync(0xffffffffu, g0, 16);
  a1 += __shfl_xor_sync(0xffffffffu, g1, 16);
  float c = b3 ? a1 : a0;
  const float d = b3 ? a0 : a1;
  c += __shfl_xor_sync(0xffffffffu, d, 8);
  c += __shfl_xor_sync(0xffffffffu, c, 4);
  c += __shfl_xor_sync(0xffffffffu, c, 2);
  c += __shfl_xor_sync(0xffffffffu, c, 1);
  if ((lane & 7) == 0) red[parity][(lane >> 3) * 8 + warp] = c;      // value index = 2 * bit4 + bit3 = lane >> 3
  __syncthreads();
  float t = red[parity][lane];
  t += __shfl_xor_sync(0xffffffffu, t, 4);
  t += __shfl_xor_sync(0xffffffffu, t, 2);
  t += __shfl_xor_sync(0xffffffffu, t, 1);
#pragma unroll
  for (int j = 0; j < 4; ++j) s[j] = __shfl_sync(0xffffffffu, t, j * 8);
}

// ------------------------------------------------------------------------------------------------ modulate + RMSNorm
// One CTA streams over rows; thread t owns columns [8t, 8t+8). mode 0: h = RMSNorm(x*(1+scale)+shift)*w
// (modulate -> norm); mode 1: h = (RMSNorm(x)*w)*(1+scale)+shift (norm -> modulate). scale/shift may be null
// (plain RMSNorm). With `gidx`, source row r comes from peers.p[gidx[r] >> 28] at row (gidx[r] & 0x0fffffff), and
// the gathered row is also written to x_out.
constexpr int FWD_RPI = 4;  // rows per iteration of one CTA: one block-wide reduction serves four rows
__global__ void modnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ gidx,
                                   PeerPtrs peers, __nv_bfloat16* __restrict__ x_out,
                                   const float* __restrict__ scale, const float* __restrict__ shift,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h, int rows,
                                   int D, int mode, float eps, int rows_per_cta, const float* __restrict__ wf,
                                   __nv_bfloat16* __restrict__ h_lo) {
  __shared__ float red[2 * FWD_RPI * 32];
  const int c0 = threadIdx.x * 8;
  const bool active = c0 < D;
  float sc[8], sh[8], wv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { sc[i] = 0.f; sh[i] = 0.f; wv[i] = 0.f; }
  if (active) {
    if (scale) loadf8(scale + c0, sc);
    if (shift) loadf8(shift + c0, sh);
    if (wf) loadf8(wf + c0, wv); else load8(w + c0, wv);
  }
  // CTAs sweep the rows together (CTA b takes row groups b, b + grid, ...). The rows of the next group are requested
  // before the current group is reduced, so every thread keeps up to eight 16-byte loads in flight across the
  // block-wide reduction.
  (void)rows_per_cta;
  const int r1 = rows;
  const int stride = gridDim.x * FWD_RPI;
  uint4 nxt[FWD_RPI];
  auto fetch = [&](int r) {
#pragma unroll
    for (int k = 0; k < FWD_RPI; ++k) {
      const int rr = r + k;
      nxt[k] = make_uint4(0u, 0u, 0u, 0u);
      if (active && rr < r1) {
        const __nv_bfloat16* src;
        bool ok = true;
        if (gidx) {
          const uint32_t code = gidx[rr];
          ok = AERIS_GATHER_OK(peers, code);
          src = peers.p[code >> 28] + static_cast<size_t>(code & 0x0fffffffu) * D + c0;
        } else {
          src = x + static_cast<size_t>(rr) * D + c0;
        }
        if (ok) nxt[k] = *reinterpret_cast<const uint4*>(src);
      }
    }
  };
  int parity = 0;
  int r = blockIdx.x * FWD_RPI;
  if (r < r1) fetch(r);
  for (; r < r1; r += stride, parity ^= 1) {
    float y[FWD_RPI][8];
    float ss[FWD_RPI];
    uint4 cur[FWD_RPI];
#pragma unroll
    for (int k = 0; k < FWD_RPI; ++k) cur[k] = nxt[k];
    if (r + stride < r1) fetch(r + stride);
#pragma unroll
    for (int k = 0; k < FWD_RPI; ++k) {
      float v[8];
      {
        const uint32_t w4[4] = {cur[k].x, cur[k].y, cur[k].z, cur[k].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t = unpack_bf16x2(w4[i]);
          v[2 * i] = t.x;
          v[2 * i + 1] = t.y;
        }
      }
      const int rr = r + k;
      if (active && rr < r1 && x_out) *reinterpret_cast<uint4*>(x_out + static_cast<size_t>(rr) * D + c0) = cur[k];
      ss[k] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        y[k][i] = (mode == 0) ? fmaf(v[i], sc[i], v[i]) + sh[i] : v[i];
        ss[k] += y[k][i] * y[k][i];
      }
      if (!active || rr >= r1) ss[k] = 0.f;
    }
    block_sum<FWD_RPI>(ss, red, parity);
#pragma unroll
    for (int k = 0; k < FWD_RPI; ++k) {
      const int rr = r + k;
      if (active && rr < r1) {
        const float rinv = rsqrtf(ss[k] / D + eps);
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float n = y[k][i] * rinv * wv[i];
          o[i] = (mode == 0) ? n : fmaf(n, sc[i], n) + sh[i];
        }
        store8(h + static_cast<size_t>(rr) * D + c0, o);
        if (h_lo) {
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] -= __bfloat162float(__float2bfloat16_rn(o[i]));
          store8(h_lo + static_cast<size_t>(rr) * D + c0, o);
        }
      }
    }
  }
}

// The same forward for rows of up to 1536 columns (at most six warps), written for the instruction issue rate: the kernel
// above executes 20.6 warp instructions per element and keeps the schedulers 64 % busy with no memory stall to speak
// of. Here every per-element operation works on a column pair (`*.f32x2`), 1 + scale is formed once, the row mean uses
// a multiplication, and the four rows' sums go through block_sum4_shfl.
__global__ void __launch_bounds__(192, 3)
modnorm_fwd_pair_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ gidx, PeerPtrs peers,
                        __nv_bfloat16* __restrict__ x_out, const float* __restrict__ scale,
                        const float* __restrict__ shift, const __nv_bfloat16* __restrict__ w,
                        __nv_bfloat16* __restrict__ h, int rows, int D, int mode, float eps,
                        const float* __restrict__ wf, __nv_bfloat16* __restrict__ h_lo) {
  static_assert(FWD_RPI == 4, "block_sum4_shfl reduces four values");
  __shared__ float red[2][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 64; i += blockDim.x) (&red[0][0])[i] = 0.f;
  const int c0 = threadIdx.x * 8;
  const bool active = c0 < D;
  uint64_t sc1[4], sh[4], wv[4];
  {
    float t_sc[8], t_sh[8], t_w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { t_sc[i] = 0.f; t_sh[i] = 0.f; t_w[i] = 0.f; }
    if (active) {
      if (scale) loadf8(scale + c0, t_sc);
      if (shift) loadf8(shift + c0, t_sh);
      if (wf) loadf8(wf + c0, t_w); else load8(w + c0, t_w);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sc1[i] = f2_pack(1.f + t_sc[2 * i], 1.f + t_sc[2 * i + 1]);
      sh[i] = f2_pack(t_sh[2 * i], t_sh[2 * i + 1]);
      wv[i] = f2_pack(t_w[2 * i], t_w[2 * i + 1]);
    }
  }
  __syncthreads();
  const int r1 = rows;
  const int stride = gridDim.x * FWD_RPI;
  const float inv_d = 1.f / D;
  uint4 nxt[FWD_RPI];
  auto fetch = [&](int r) {
#pragma unroll
    for (int k = 0; k < FWD_RPI; ++k) {
      const int rr = r + k;
      nxt[k] = make_uint4(0u, 0u, 0u, 0u);
      if (active && rr < r1) {
        const __nv_bfloat16* src;
        bool ok = true;
        if (gidx) {
          const uint32_t code = gidx[rr];
          ok = AERIS_GATHER_OK(peers, code);
          src = peers.p[code >> 28] + static_cast<size_t>(code & 0x0fffffffu) * D + c0;
        } else {
          src = x + static_cast<size_t>(rr) * D + c0;
        }
        if (ok) nxt[k] = *reinterpret_cast<const uint4*>(src);
      }
    }
  };
  int parity = 0;
  int r = blockIdx.x * FWD_RPI;
  if (r < r1) fetch(r);
  for (; r < r1; r += stride, parity ^= 1) {
    uint64_t y[FWD_RPI][4];
    float ss[FWD_RPI];
    uint4 cur[FWD_RPI];
#pragma unroll
    for (int k = 0; k < FWD_RPI; ++k) cur[k] = nxt[k];
    if (r + stride < r1) fetch(r + stride);
#pragma unroll
    for (int k = 0; k < FWD_RPI; ++k) {
      const int rr = r + k;
      const bool live = active && rr < r1;
      if (live && x_out) *reinterpret_cast<uint4*>(x_out + static_cast<size_t>(rr) * D + c0) = cur[k];
      const uint32_t w4[4] = {cur[k].x, cur[k].y, cur[k].z, cur[k].w};
      uint64_t p = 0ull;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint64_t v = f2_from_bf16x2(w4[i]);
        y[k][i] = (mode == 0) ? f2_fma(v, sc1[i], sh[i]) : v;
        p = f2_fma(y[k][i], y[k][i], p);
      }
      float p0, p1;
      f2_unpack(p, p0, p1);
      ss[k] = live ? p0 + p1 : 0.f;
    }
    block_sum4_shfl(ss, red, parity, lane, warp);
#pragma unroll
    for (int k = 0; k < FWD_RPI; ++k) {
      const int rr = r + k;
      if (!active || rr >= r1) continue;
      const float rinv = rsqrtf(ss[k] * inv_d + eps);
      const uint64_t rinv2 = f2_pack(rinv, rinv);
      uint64_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint64_t n = f2_mul(f2_mul(y[k][i], rinv2), wv[i]);
        o[i] = (mode == 0) ? n : f2_fma(n, sc1[i], sh[i]);
      }
      uint32_t hw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) hw[i] = f2_to_bf16x2(o[i]);
      *reinterpret_cast<uint4*>(h + static_cast<size_t>(rr) * D + c0) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
      if (h_lo) {          // the part of the fp32 value that the bf16 value above does not hold
        uint32_t lw[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) lw[i] = f2_to_bf16x2(f2_sub(o[i], f2_from_bf16x2(hw[i])));
        *reinterpret_cast<uint4*>(h_lo + static_cast<size_t>(rr) * D + c0) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
      }
    }
  }
}

// Backward of the above. dx = dres + d(norm path). Column sums are kept in registers over the CTA's rows and
// flushed with atomics at the end: dscale, dshift (fp32 [D], one modulation vector per launch) and dw (fp32 [D]).
// MAXT / MINB: launch bounds by row width: up to 1536 columns 192 threads and two CTAs per SM (three were measured slower: spills), up to 5120 columns
// 640 threads, wider rows 1024 threads (register cap 64: spills, but it launches).
template <int MAXT, int MINB, int RPI>
__global__ void __launch_bounds__(MAXT, MINB)
modnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dh,
                                   const __nv_bfloat16* __restrict__ dres, const float* __restrict__ scale,
                                   const float* __restrict__ shift, const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dscale,
                                   float* __restrict__ dshift, float* __restrict__ dw, int rows, int D, int mode,
                                   float eps, int rows_per_cta, const float* __restrict__ wf) {
  // RPI rows per iteration share one block-wide reduction, and the next RPI rows are requested before it: with
  // RPI = 2 every thread keeps 12 sixteen-byte loads in flight (one row at a time left the memory system idle
  // during the reduction)
  __shared__ float red[2 * 2 * RPI * 32];
  const int c0 = threadIdx.x * 8;
  const bool active = c0 < D;
  float sc[8], sh[8], wv[8], a_sc[8], a_sh[8], a_w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { sc[i] = 0.f; sh[i] = 0.f; wv[i] = 0.f; a_sc[i] = 0.f; a_sh[i] = 0.f; a_w[i] = 0.f; }
  if (active) {
    if (scale) loadf8(scale + c0, sc);
    if (shift) loadf8(shift + c0, sh);
    if (wf) loadf8(wf + c0, wv); else load8(w + c0, wv);
  }
  (void)rows_per_cta;
  const int r1 = rows;
  const int stride = gridDim.x * RPI;
  int parity = 0;
  uint4 nx[RPI], ng[RPI], nr[RPI];
#pragma unroll
  for (int k = 0; k < RPI; ++k) nx[k] = ng[k] = nr[k] = make_uint4(0u, 0u, 0u, 0u);
  // iteration `it` of this CTA covers rows it * stride + blockIdx.x + k * gridDim.x, k < RPI (interleaved with the others)
  auto fetch = [&](int base) {
#pragma unroll
    for (int k = 0; k < RPI; ++k) {
      const int r = base + k * static_cast<int>(gridDim.x);
      if (active && r < r1) {
        const size_t off = static_cast<size_t>(r) * D + c0;
        nx[k] = *reinterpret_cast<const uint4*>(x + off);
        ng[k] = *reinterpret_cast<const uint4*>(dh + off);
        if (dres) nr[k] = *reinterpret_cast<const uint4*>(dres + off);
      }
    }
  };
  auto unpack8 = [](const uint4& u, float (&f)[8]) {
    const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = unpack_bf16x2(w4[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  };
  fetch(blockIdx.x);
  for (int base = blockIdx.x; base < r1; base += stride, parity ^= 1) {
    float v[RPI][8], g[RPI][8], dr[RPI][8];
#pragma unroll
    for (int k = 0; k < RPI; ++k) {
      unpack8(nx[k], v[k]);
      unpack8(ng[k], g[k]);
      unpack8(nr[k], dr[k]);
    }
    if (base + stride < r1) fetch(base + stride);
    float s[2 * RPI];
    if (mode == 0) {
      // y = x(1+sc)+sh ; h = y * rinv * w       (v <- y, g stays, gy recomputed after the reduction)
#pragma unroll
      for (int k = 0; k < RPI; ++k) {
        s[2 * k] = 0.f; s[2 * k + 1] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float y = fmaf(v[k][i], sc[i], v[k][i]) + sh[i];
          s[2 * k] += y * y;
          s[2 * k + 1] += y * (g[k][i] * wv[i]);
        }
        if (!active || base + k * static_cast<int>(gridDim.x) >= r1) { s[2 * k] = 0.f; s[2 * k + 1] = 0.f; }
      }
    } else {
      // n = x * rinv ; hn = n * w ; h = hn(1+sc)+sh
#pragma unroll
      for (int k = 0; k < RPI; ++k) {
        s[2 * k] = 0.f; s[2 * k + 1] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float gn = fmaf(g[k][i], sc[i], g[k][i]) * wv[i];
          s[2 * k] += v[k][i] * v[k][i];
          s[2 * k + 1] += v[k][i] * gn;
        }
        if (!active || base + k * static_cast<int>(gridDim.x) >= r1) { s[2 * k] = 0.f; s[2 * k + 1] = 0.f; }
      }
    }
    block_sum<2 * RPI>(s, red, parity);
#pragma unroll
    for (int k = 0; k < RPI; ++k) {
      const int r = base + k * static_cast<int>(gridDim.x);
      if (!active || r >= r1) continue;
      const float rinv = rsqrtf(s[2 * k] / D + eps);
      const float coef = rinv * rinv * rinv * (s[2 * k + 1] / D);
      float o[8];
      if (mode == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float y = fmaf(v[k][i], sc[i], v[k][i]) + sh[i];
          const float dy = rinv * (g[k][i] * wv[i]) - y * coef;
          a_w[i] += g[k][i] * y * rinv;
          a_sc[i] += dy * v[k][i];
          a_sh[i] += dy;
          o[i] = dr[k][i] + fmaf(dy, sc[i], dy);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float n = v[k][i] * rinv;
          const float dhn = fmaf(g[k][i], sc[i], g[k][i]);
          a_sc[i] += g[k][i] * n * wv[i];
          a_sh[i] += g[k][i];
          a_w[i] += dhn * n;
          o[i] = dr[k][i] + rinv * (dhn * wv[i]) - v[k][i] * coef;
        }
      }
      store8(dx + static_cast<size_t>(r) * D + c0, o);
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (dscale) atomicAdd(dscale + c0 + i, a_sc[i]);
      if (dshift) atomicAdd(dshift + c0 + i, a_sh[i]);
      if (dw) atomicAdd(dw + c0 + i, a_w[i]);
    }
  }
}

// The same backward for rows of up to 1536 columns (at most six warps per row), cut down to what the instruction
// issue rate allows: the one-row-at-a-time kernel above executed about 42 warp instructions per element and kept the
// schedulers 53 % busy with three resident warps each, i.e. it was bound by instruction issue, not by memory.
//   * every per-element operation works on a pair of columns (`*.f32x2`, half the issue slots);
//   * two rows share one block-wide reduction, whose cross-warp part is one shared-memory load and seven shuffles per
//     thread (lane k * 8 + w holds value k of warp w) instead of 24 loads and adds;
//   * 1 + scale is formed once per thread.
template <int RPI, int MINB>
__global__ void __launch_bounds__(192, MINB)
modnorm_bwd_pair_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dh,
                        const __nv_bfloat16* __restrict__ dres, const float* __restrict__ scale,
                        const float* __restrict__ shift, const __nv_bfloat16* __restrict__ w,
                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dscale, float* __restrict__ dshift,
                        float* __restrict__ dw, int rows, int D, int mode, float eps, const float* __restrict__ wf) {
  constexpr int NV = 2 * RPI;                    // values to reduce per iteration
  constexpr int NL = (NV * 8 + 31) / 32;         // slot k * 8 + w holds value k of warp w; a lane sums NL of them
  __shared__ float red[2][NL * 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 2 * NL * 32; i += blockDim.x) (&red[0][0])[i] = 0.f;   // slots of absent warps stay zero
  const int c0 = threadIdx.x * 8;
  const bool active = c0 < D;
  uint64_t sc1[4], sh[4], wv[4], a_sc[4], a_sh[4], a_w[4];
  {
    float t_sc[8], t_sh[8], t_w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { t_sc[i] = 0.f; t_sh[i] = 0.f; t_w[i] = 0.f; }
    if (active) {
      if (scale) loadf8(scale + c0, t_sc);
      if (shift) loadf8(shift + c0, t_sh);
      if (wf) loadf8(wf + c0, t_w); else load8(w + c0, t_w);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sc1[i] = f2_pack(1.f + t_sc[2 * i], 1.f + t_sc[2 * i + 1]);
      sh[i] = f2_pack(t_sh[2 * i], t_sh[2 * i + 1]);
      wv[i] = f2_pack(t_w[2 * i], t_w[2 * i + 1]);
      a_sc[i] = a_sh[i] = a_w[i] = 0ull;
    }
  }
  __syncthreads();
  const int r1 = rows;
  const int gstep = gridDim.x;
  const int stride = gstep * RPI;
  const float inv_d = 1.f / D;
  int parity = 0;
  uint4 nx[RPI], ng[RPI], nr[RPI];
#pragma unroll
  for (int k = 0; k < RPI; ++k) nx[k] = ng[k] = nr[k] = make_uint4(0u, 0u, 0u, 0u);
  auto fetch = [&](int base) {
#pragma unroll
    for (int k = 0; k < RPI; ++k) {
      const int r = base + k * gstep;
      if (active && r < r1) {
        const size_t off = static_cast<size_t>(r) * D + c0;
        nx[k] = *reinterpret_cast<const uint4*>(x + off);
        ng[k] = *reinterpret_cast<const uint4*>(dh + off);
        if (dres) nr[k] = *reinterpret_cast<const uint4*>(dres + off);
      }
    }
  };
  fetch(blockIdx.x);
  for (int base = blockIdx.x; base < r1; base += stride, parity ^= 1) {
    uint64_t v[RPI][4], g[RPI][4];
    uint4 dr[RPI];
#pragma unroll
    for (int k = 0; k < RPI; ++k) {
      const uint32_t xw[4] = {nx[k].x, nx[k].y, nx[k].z, nx[k].w}, gw[4] = {ng[k].x, ng[k].y, ng[k].z, ng[k].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[k][i] = f2_from_bf16x2(xw[i]);
        g[k][i] = f2_from_bf16x2(gw[i]);
      }
      dr[k] = nr[k];
    }
    if (base + stride < r1) fetch(base + stride);
    // ---- the two row sums of each row: mode 0  sum y^2, sum y (g w);  mode 1  sum x^2, sum x (g (1 + sc) w)
    float s[2 * RPI];
#pragma unroll
    for (int k = 0; k < RPI; ++k) {
      uint64_t p0 = 0ull, p1 = 0ull;
      if (mode == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint64_t y = f2_fma(v[k][i], sc1[i], sh[i]);
          p0 = f2_fma(y, y, p0);
          p1 = f2_fma(y, f2_mul(g[k][i], wv[i]), p1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          p0 = f2_fma(v[k][i], v[k][i], p0);
          p1 = f2_fma(v[k][i], f2_mul(f2_mul(g[k][i], sc1[i]), wv[i]), p1);
        }
      }
      float a0, a1, b0, b1;
      f2_unpack(p0, a0, a1);
      f2_unpack(p1, b0, b1);
      const bool live = active && base + k * gstep < r1;
      s[2 * k] = live ? a0 + a1 : 0.f;
      s[2 * k + 1] = live ? b0 + b1 : 0.f;
    }
    // ---- block-wide sums
    if constexpr (RPI == 2) {
      block_sum4_shfl(s, red, parity, lane, warp);
    } else {
#pragma unroll
      for (int j = 0; j < 2 * RPI; ++j) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s[j] += __shfl_xor_sync(0xffffffffu, s[j], o);
      }
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < 2 * RPI; ++j) red[parity][j * 8 + warp] = s[j];
      }
      __syncthreads();
      float t[NL];
#pragma unroll
      for (int q = 0; q < NL; ++q) {
        t[q] = red[parity][q * 32 + lane];
        t[q] += __shfl_xor_sync(0xffffffffu, t[q], 4);
        t[q] += __shfl_xor_sync(0xffffffffu, t[q], 2);
        t[q] += __shfl_xor_sync(0xffffffffu, t[q], 1);
      }
#pragma unroll
      for (int j = 0; j < NV; ++j) s[j] = __shfl_sync(0xffffffffu, t[j / 4], (j % 4) * 8);
    }
    // ---- gradients
#pragma unroll
    for (int k = 0; k < RPI; ++k) {
      const int r = base + k * gstep;
      if (!active || r >= r1) continue;
      const float rinv = rsqrtf(s[2 * k] * inv_d + eps);
      const float ncoef = -rinv * rinv * rinv * (s[2 * k + 1] * inv_d);
      const uint64_t rinv2 = f2_pack(rinv, rinv), ncoef2 = f2_pack(ncoef, ncoef);
      const uint32_t dw4[4] = {dr[k].x, dr[k].y, dr[k].z, dr[k].w};
      uint32_t ow[4];
      if (mode == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint64_t y = f2_fma(v[k][i], sc1[i], sh[i]);
          const uint64_t dy = f2_fma(ncoef2, y, f2_mul(rinv2, f2_mul(g[k][i], wv[i])));
          a_w[i] = f2_fma(f2_mul(g[k][i], y), rinv2, a_w[i]);
          a_sc[i] = f2_fma(dy, v[k][i], a_sc[i]);
          a_sh[i] = f2_add(a_sh[i], dy);
          ow[i] = f2_to_bf16x2(f2_fma(dy, sc1[i], f2_from_bf16x2(dw4[i])));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint64_t n = f2_mul(v[k][i], rinv2);
          const uint64_t dhn = f2_mul(g[k][i], sc1[i]);
          a_sc[i] = f2_fma(f2_mul(g[k][i], n), wv[i], a_sc[i]);
          a_sh[i] = f2_add(a_sh[i], g[k][i]);
          a_w[i] = f2_fma(dhn, n, a_w[i]);
          const uint64_t t2 = f2_fma(rinv2, f2_mul(dhn, wv[i]), f2_from_bf16x2(dw4[i]));
          ow[i] = f2_to_bf16x2(f2_fma(ncoef2, v[k][i], t2));
        }
      }
      *reinterpret_cast<uint4*>(dx + static_cast<size_t>(r) * D + c0) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float lo, hi;
      if (dscale) { f2_unpack(a_sc[i], lo, hi); atomicAdd(dscale + c0 + 2 * i, lo); atomicAdd(dscale + c0 + 2 * i + 1, hi); }
      if (dshift) { f2_unpack(a_sh[i], lo, hi); atomicAdd(dshift + c0 + 2 * i, lo); atomicAdd(dshift + c0 + 2 * i + 1, hi); }
      if (dw) { f2_unpack(a_w[i], lo, hi); atomicAdd(dw + c0 + 2 * i, lo); atomicAdd(dw + c0 + 2 * i + 1, hi); }
    }
  }
}

// ------------------------------------------------------------------------------------------------ row gather
__global__ void gather_rows_kernel(const uint32_t* __restrict__ gidx, PeerPtrs peers,
                                   __nv_bfloat16* __restrict__ out, long long rows, int D) {
  const int vec_per_row = D / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int v = static_cast<int>(i - r * vec_per_row);
    const uint32_t code = gidx[r];
    if (!AERIS_GATHER_OK(peers, code)) {
      reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * D)[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(peers.p[code >> 28] +
                                                      static_cast<size_t>(code & 0x0fffffffu) * D) + v;
    reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * D)[v] = *src;
  }
}

// ------------------------------------------------------------------------------------------------ SwiGLU
// u = [gate | up] of width 2F per row. act = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ act,
                                  long long rows, int F) {
  const int vec = F / 8;
  const long long total = rows * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec;
    const int c = static_cast<int>(i - r * vec) * 8;
    float g[8], up[8], o[8];
    load8(u + r * 2 * F + c, g);
    load8(u + r * 2 * F + F + c, up);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * up[k];
    store8(act + r * F + c, o);
  }
}
// du = [dact * up * dsilu(gate) | dact * silu(gate)]
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ du, long long rows, int F) {
  const int vec = F / 8;
  const long long total = rows * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec;
    const int c = static_cast<int>(i - r * vec) * 8;
    float g[8], up[8], d[8], dg[8], dup[8];
    load8(u + r * 2 * F + c, g);
    load8(u + r * 2 * F + F + c, up);
    load8(dact + r * F + c, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = 1.f / (1.f + __expf(-g[k]));
      const float silu = g[k] * s;
      dup[k] = d[k] * silu;
      dg[k] = d[k] * up[k] * (s + silu * (1.f - s));
    }
    store8(du + r * 2 * F + c, dg);
    store8(du + r * 2 * F + F + c, dup);
  }
}

// ------------------------------------------------------------------------------------------------ rotary embedding
// In-place axial 2-D rotary embedding of the q and k sections of a fused qkv tensor [rows, 3 * heads * d] (columns
// q | k | v, head, d): the (2i, 2i + 1) channel pairs of every head rotate by the angle of (token, pair i), with the
// token = row mod L and cos / sin tables [L, d / 2] (fp32). `inverse` rotates by the negative angles (what the backward
// pass applies to the gradients of the rotated q and k). One thread: eight channels = four pairs.
__global__ void rope_qk_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cs, const float* __restrict__ sn,
                               long long rows, int L, int heads, int d, int inverse) {
  const int HD = heads * d;
  const int vec_per_row = 2 * HD / 8;              // q and k sections only
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;       // column inside q | k
    const int within = c % d;                                      // channel inside the head
    const int tok = static_cast<int>(r % L);
    __nv_bfloat16* ptr = qkv + static_cast<size_t>(r) * 3 * HD + c;
    float v[8];
    load8(ptr, v);
    const float4 c4 = *reinterpret_cast<const float4*>(cs + static_cast<size_t>(tok) * (d / 2) + within / 2);
    float4 s4 = *reinterpret_cast<const float4*>(sn + static_cast<size_t>(tok) * (d / 2) + within / 2);
    if (inverse) { s4.x = -s4.x; s4.y = -s4.y; s4.z = -s4.z; s4.w = -s4.w; }
    const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
    float o[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      o[2 * k] = v[2 * k] * cc[k] - v[2 * k + 1] * ss[k];
      o[2 * k + 1] = v[2 * k + 1] * cc[k] + v[2 * k] * ss[k];
    }
    store8(ptr, o);
  }
}

// ------------------------------------------------------------------------------------------------ gate helpers
// Wg[r, :] = g[r] * W[r, :]  (bf16), used as the B operand of the gated data-gradient GEMMs.
__global__ void scale_rows_kernel(const __nv_bfloat16* __restrict__ W, const float* __restrict__ g,
                                  __nv_bfloat16* __restrict__ Wg, int R, int C) {
  const int vec = C / 8;
  const long long total = static_cast<long long>(R) * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / vec);
    const int c = static_cast<int>(i - static_cast<long long>(r) * vec) * 8;
    float v[8];
    load8(W + static_cast<size_t>(r) * C + c, v);
    const float s = g[r];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] *= s;
    store8(Wg + static_cast<size_t>(r) * C + c, v);
  }
}
// G = dY^T A (ungated weight gradient of out = resid + g * (A W^T)). Then
//   dW[r, :] += g[r] * G[r, :]   and   dg[r] += sum_c W[r, c] * G[r, c];   G is zeroed for the next sample.
__global__ void gate_grad_finalize_kernel(float* __restrict__ G, const __nv_bfloat16* __restrict__ W,
                                          const float* __restrict__ g, float* __restrict__ dW,
                                          float* __restrict__ dg, int R, int C) {
  __shared__ float red[2 * 1 * 32];
  const int r = blockIdx.x;
  const float s = g[r];
  float acc[1] = {0.f};
  for (int c = threadIdx.x * 4; c < C; c += blockDim.x * 4) {
    const size_t off = static_cast<size_t>(r) * C + c;
    const float4 gv = *reinterpret_cast<const float4*>(G + off);
    const uint2 wu = *reinterpret_cast<const uint2*>(W + off);
    const float2 w01 = unpack_bf16x2(wu.x), w23 = unpack_bf16x2(wu.y);
    acc[0] += gv.x * w01.x + gv.y * w01.y + gv.z * w23.x + gv.w * w23.y;
    float4 d = *reinterpret_cast<float4*>(dW + off);
    d.x = fmaf(s, gv.x, d.x); d.y = fmaf(s, gv.y, d.y); d.z = fmaf(s, gv.z, d.z); d.w = fmaf(s, gv.w, d.w);
    *reinterpret_cast<float4*>(dW + off) = d;
    *reinterpret_cast<float4*>(G + off) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  block_sum<1>(acc, red, 0);
  if (threadIdx.x == 0) dg[r] += acc[0];
}

// ------------------------------------------------------------------------------------------------ optimizer
// Sum of squares of a flat fp32 buffer into out[0] (double), |x| finite check folded in by the caller.
__global__ void sumsq_kernel(const float* __restrict__ x, long long n, double* __restrict__ out) {
  __shared__ float red[2 * 1 * 32];
  float acc[1] = {0.f};
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    acc[0] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = n4 * 4; i < n; ++i) acc[0] += x[i] * x[i];
  block_sum<1>(acc, red, 0);
  if (threadIdx.x == 0) atomicAdd(out, static_cast<double>(acc[0]));
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias1, bias2;       // 1 - beta^t
  float grad_scale;         // multiplies the raw accumulated gradient (1 / (DP * GAS))
  float max_norm;           // <= 0: no clipping
  float ema_beta;           // < 0: no EMA
  float nan_clamp;          // +-inf replacement magnitude, NaN -> 0
};
// One fused pass over a flat shard: g = nan_to_num(grad * grad_scale * clip); AdamW on the fp32 master; bf16 copy of
// the new weight; EMA lerp; gradient buffer zeroed. `norm_sq` is the global sum of squares of (grad * grad_scale).
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ grad, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ wbf16, float* __restrict__ ema,
                             const double* __restrict__ norm_sq, long long n, AdamArgs a) {
  float clip = 1.f;
  if (a.max_norm > 0.f && norm_sq) {
    const float total = static_cast<float>(sqrt(*norm_sq));
    const float c = a.max_norm / (total + 1.0e-6f);
    if (c < 1.f) clip = c;
  }
  const float gs = a.grad_scale * clip;
  const bool do_ema = ema && a.ema_beta >= 0.f;
  auto update = [&](float g, float& p, float& mi, float& vi, float& e) {
    g *= gs;
    if (g != g) g = 0.f;
    else if (g > 3.0e38f) g = a.nan_clamp;
    else if (g < -3.0e38f) g = -a.nan_clamp;
    mi = a.beta1 * mi + (1.f - a.beta1) * g;
    vi = a.beta2 * vi + (1.f - a.beta2) * g * g;
    p *= (1.f - a.lr * a.weight_decay);
    p -= a.lr * (mi / a.bias1) / (sqrtf(vi / a.bias2) + a.eps);
    if (do_ema) e = p + a.ema_beta * (e - p);  // lerp(p, ema, beta)
  };
  // main part: four elements per thread and iteration through 16-byte vectors (buffers are 16-byte aligned)
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float4 p4 = reinterpret_cast<const float4*>(master)[i];
    float4 m4 = reinterpret_cast<const float4*>(m)[i];
    float4 v4 = reinterpret_cast<const float4*>(v)[i];
    float4 e4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (do_ema) e4 = reinterpret_cast<const float4*>(ema)[i];
    update(g4.x, p4.x, m4.x, v4.x, e4.x);
    update(g4.y, p4.y, m4.y, v4.y, e4.y);
    update(g4.z, p4.z, m4.z, v4.z, e4.z);
    update(g4.w, p4.w, m4.w, v4.w, e4.w);
    reinterpret_cast<float4*>(master)[i] = p4;
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    if (do_ema) reinterpret_cast<float4*>(ema)[i] = e4;
    if (wbf16) {
      uint2 u;
      u.x = pack_bf16x2(p4.x, p4.y);
      u.y = pack_bf16x2(p4.z, p4.w);
      reinterpret_cast<uint2*>(wbf16)[i] = u;
    }
    reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long i = n4 * 4; i < n; ++i) {
      float p = master[i], mi = m[i], vi = v[i], e = do_ema ? ema[i] : 0.f;
      update(grad[i], p, mi, vi, e);
      master[i] = p; m[i] = mi; v[i] = vi;
      if (do_ema) ema[i] = e;
      if (wbf16) wbf16[i] = __float2bfloat16_rn(p);
      grad[i] = 0.f;
    }
  }
}

// Owner side of the row reduce-scatter: out = resid + gate[col] * sum_s slots[s * rows + r] (bf16 slots, fp32 sum).
__global__ void rs_finalize_kernel(const __nv_bfloat16* __restrict__ slots, int world, long long rows, int D,
                                   const __nv_bfloat16* __restrict__ resid, const float* __restrict__ gate,
                                   __nv_bfloat16* __restrict__ out) {
  const int vec = D / 8;
  const long long total = rows * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec;
    const int c = static_cast<int>(i - r * vec) * 8;
    float acc[8];
    load8(slots + r * D + c, acc);
    for (int s = 1; s < world; ++s) {
      float t[8];
      load8(slots + (static_cast<long long>(s) * rows + r) * D + c, t);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += t[k];
    }
    if (gate) {
      float g[8];
      loadf8(gate + c, g);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] *= g[k];
    }
    if (resid) {
      float t[8];
      load8(resid + r * D + c, t);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += t[k];
    }
    store8(out + r * D + c, acc);
  }
}

static inline int grid_for(long long work, int threads, int max_blocks) {
  long long b = (work + threads - 1) / threads;
  if (b > max_blocks) b = max_blocks;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}
static inline int row_threads(int D) {
  int t = (D / 8 + 31) / 32 * 32;
  return t < 32 ? 32 : t;
}

}  // namespace aeris

using namespace aeris;
extern int aeris_num_sms();

static int pick_rows_per_cta(int rows) {
  const int target_ctas = aeris_num_sms() * 8;
  int rpc = (rows + target_ctas - 1) / target_ctas;
  if (rpc < 1) rpc = 1;
  return rpc;
}

extern "C" int aeris_modnorm_fwd(const void* x, const void* gidx, const void* const* peer_ptrs, int n_peers,
                                 void* x_out, const float* scale, const float* shift, const void* w, void* h,
                                 int rows, int D, int mode, float eps, const float* w_f32, void* h_lo,
                                 void* stream) {
  if (D % 8 || D > 8192 || rows <= 0 || (!w && !w_f32)) return -1;
  PeerPtrs pp{};
  for (int i = 0; i < n_peers && i < 16; ++i) pp.p[i] = reinterpret_cast<const __nv_bfloat16*>(peer_ptrs[i]);
  if (gidx && n_peers <= 0) return -2;
  AERIS_FILL_CHECK(pp, n_peers);
  const int rpc = pick_rows_per_cta(rows);
  int grid = (rows + FWD_RPI - 1) / FWD_RPI;
  if (grid > aeris_num_sms() * 8) grid = aeris_num_sms() * 8;
  if (row_threads(D) <= 192) {
    modnorm_fwd_pair_kernel<<<grid, row_threads(D), 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const uint32_t*>(gidx), pp,
        reinterpret_cast<__nv_bfloat16*>(x_out), scale, shift, reinterpret_cast<const __nv_bfloat16*>(w),
        reinterpret_cast<__nv_bfloat16*>(h), rows, D, mode, eps, w_f32, reinterpret_cast<__nv_bfloat16*>(h_lo));
    return cudaGetLastError() == cudaSuccess ? 0 : -21;
  }
  modnorm_fwd_kernel<<<grid, row_threads(D), 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const uint32_t*>(gidx), pp,
      reinterpret_cast<__nv_bfloat16*>(x_out), scale, shift, reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<__nv_bfloat16*>(h), rows, D, mode, eps, rpc, w_f32, reinterpret_cast<__nv_bfloat16*>(h_lo));
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_modnorm_bwd(const void* x, const void* dh, const void* dres, const float* scale,
                                 const float* shift, const void* w, void* dx, float* dscale, float* dshift,
                                 float* dw, int rows, int D, int mode, float eps, const float* w_f32, void* stream) {
  if (D % 8 || D > 8192 || rows <= 0 || (!w && !w_f32)) return -1;
  int rpc = pick_rows_per_cta(rows);
  if (rpc < 16) rpc = rows < 16 ? rows : 16;  // amortise the atomic flush of the column sums
  const int grid = (rows + rpc - 1) / rpc;    // every CTA takes about rpc rows, interleaved with the others
  const int nt = row_threads(D);
  if (nt <= 192) {
    // two rows per reduction and two CTAs per SM measured best (0.381 ms for 129600 x 1536; one row and three CTAs
    // 0.430 ms, four rows and one CTA 0.398 ms, two rows under a 112-register cap spill: 0.822 ms)
    modnorm_bwd_pair_kernel<2, 2><<<grid, nt, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(dh),
        reinterpret_cast<const __nv_bfloat16*>(dres), scale, shift, reinterpret_cast<const __nv_bfloat16*>(w),
        reinterpret_cast<__nv_bfloat16*>(dx), dscale, dshift, dw, rows, D, mode, eps, w_f32);
    return cudaGetLastError() == cudaSuccess ? 0 : -21;
  }
  auto kern = (nt <= 640) ? modnorm_bwd_kernel<640, 1, 1> : modnorm_bwd_kernel<1024, 1, 1>;
  kern<<<grid, row_threads(D), 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(dh),
      reinterpret_cast<const __nv_bfloat16*>(dres), scale, shift, reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<__nv_bfloat16*>(dx), dscale, dshift, dw, rows, D, mode, eps, rpc, w_f32);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_gather_rows(const void* gidx, const void* const* peer_ptrs, int n_peers, void* out,
                                 long long rows, int D, void* stream) {
  if (D % 8 || rows <= 0 || n_peers <= 0) return -1;
  PeerPtrs pp{};
  for (int i = 0; i < n_peers && i < 16; ++i) pp.p[i] = reinterpret_cast<const __nv_bfloat16*>(peer_ptrs[i]);
  AERIS_FILL_CHECK(pp, n_peers);
  const int grid = grid_for(rows * (D / 8), 256, aeris_num_sms() * 16);
  gather_rows_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(gidx), pp, reinterpret_cast<__nv_bfloat16*>(out), rows, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_swiglu_fwd(const void* u, void* act, long long rows, int F, void* stream) {
  if (F % 8 || rows <= 0) return -1;
  const int grid = grid_for(rows * (F / 8), 256, aeris_num_sms() * 16);
  swiglu_fwd_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(u), reinterpret_cast<__nv_bfloat16*>(act), rows, F);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_swiglu_bwd(const void* u, const void* dact, void* du, long long rows, int F, void* stream) {
  if (F % 8 || rows <= 0) return -1;
  const int grid = grid_for(rows * (F / 8), 256, aeris_num_sms() * 16);
  swiglu_bwd_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(u), reinterpret_cast<const __nv_bfloat16*>(dact),
      reinterpret_cast<__nv_bfloat16*>(du), rows, F);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_scale_rows(const void* W, const float* g, void* Wg, int R, int C, void* stream) {
  if (C % 8) return -1;
  const int grid = grid_for(static_cast<long long>(R) * (C / 8), 256, aeris_num_sms() * 8);
  scale_rows_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(W), g, reinterpret_cast<__nv_bfloat16*>(Wg), R, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_rope_qk(void* qkv, const float* cos_t, const float* sin_t, long long rows, int L, int heads,
                             int d, int inverse, void* stream) {
  if (rows <= 0 || L <= 0 || d % 8 != 0 || heads <= 0) return -1;
  if ((reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t)) & 15) return -3;
  const int grid = grid_for(rows * (2 * heads * d / 8), 256, aeris_num_sms() * 16);
  rope_qk_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(qkv), cos_t, sin_t, rows, L, heads, d, inverse);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_gate_grad_finalize(float* G, const void* W, const float* g, float* dW, float* dg, int R,
                                        int C, void* stream) {
  if (C % 4) return -1;
  gate_grad_finalize_kernel<<<R, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      G, reinterpret_cast<const __nv_bfloat16*>(W), g, dW, dg, R, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_sumsq(const float* x, long long n, double* out, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for(n / 4 + 1, 256, aeris_num_sms() * 8);
  sumsq_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, n, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_adamw(float* master, float* grad, float* m, float* v, void* wbf16, float* ema,
                           const double* norm_sq, long long n, float lr, float beta1, float beta2, float eps,
                           float weight_decay, int step, float grad_scale, float max_norm, float ema_beta,
                           void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(ema)) & 15) return -3;
  if (reinterpret_cast<uintptr_t>(wbf16) & 7) return -3;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f - powf(beta1, static_cast<float>(step));
  a.bias2 = 1.f - powf(beta2, static_cast<float>(step));
  a.grad_scale = grad_scale; a.max_norm = max_norm; a.ema_beta = ema_beta; a.nan_clamp = 1.0e5f;
  const int grid = grid_for(n / 4 + 1, 256, aeris_num_sms() * 16);
  adamw_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      master, grad, m, v, reinterpret_cast<__nv_bfloat16*>(wbf16), ema, norm_sq, n, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_rs_finalize(const void* slots, int world, long long rows, int D, const void* resid,
                                 const float* gate, void* out, void* stream) {
  if (D % 8 || rows <= 0 || world < 1) return -1;
  const int grid = grid_for(rows * (D / 8), 256, aeris_num_sms() * 16);
  rs_finalize_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(slots), world, rows, D, reinterpret_cast<const __nv_bfloat16*>(resid), gate,
      reinterpret_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
