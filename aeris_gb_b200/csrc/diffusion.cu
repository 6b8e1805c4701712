// Diffusion-side kernels around the transformer: everything between the image-layout fields on the device and the
// window-major token stream.
//   * embed_pack: TrigFlow noising with counter-based (Philox4x32-10) Gaussian noise, additive 2-D sinusoidal
//     position encoding, window partition by index arithmetic, and the split of the fp32 model input into bf16
//     (hi, lo) parts so that the K = 144 input projection runs on the tensor cores at fp32-level accuracy
//     (reference: src/aeris/parallelism/parallel_engine.py:21-33,673-678; src/aeris/models/parallel_swin.py:120-155,
//     383-386)
//   * trigflow_loss: weighted v-prediction loss and its gradient in one pass, the noise regenerated from the counter
//     (parallel_engine.py:990-997); the loss stays on the device
//   * sampler_update / noise_mix / affine_channels: Euler and Heun updates, churn and initial noise, and the
//     (un)standardisation + residual add of the rollout, all on the device (src/aeris/pp_generate.py:228-241,
//     298-333, which round-trips through host numpy)
//   * gemv_bias_act: the M <= 8 modulation MLP layers (parallel_swin.py:321-325)
// The noise of pixel (sample, Y, X), channel c depends only on the seed and on those global coordinates, so it does not
// change with the window-parallel or sequence-parallel layout of the run.
#include "common.cuh"
#include "api.h"

namespace aeris {

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  return c;
}

__device__ __forceinline__ float u01(uint32_t r) { return (static_cast<float>(r >> 8) + 0.5f) * (1.0f / 16777216.0f); }

// Four independent N(0,1) draws for channels [4 * group, 4 * group + 4) of global pixel `pix`.
__device__ __forceinline__ float4 normal4(unsigned long long seed, unsigned long long pix, uint32_t group) {
  const uint4 r = philox4x32_10(make_uint4(static_cast<uint32_t>(pix), static_cast<uint32_t>(pix >> 32), group, 0x41455249u),
                                make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)));
  const float r0 = sqrtf(-2.0f * logf(u01(r.x))), r1 = sqrtf(-2.0f * logf(u01(r.z)));
  float s0, c0, s1, c1;
  sincosf(6.283185307179586f * u01(r.y), &s0, &c0);
  sincosf(6.283185307179586f * u01(r.w), &s1, &c1);
  return make_float4(r0 * c0, r0 * s0, r1 * c1, r1 * s1);
}

struct Pixel {
  int b, y, x;
};
__device__ __forceinline__ int geom_rows_per_sample(const TokGeom& g) { return g.nwy_loc * g.nwx_loc * g.n_local; }
// Row of this rank's token stream (unshifted window layout, this rank's slice of every window's sequence) -> pixel
// of this rank's image block.
__device__ __forceinline__ Pixel row_to_pixel(const TokGeom& g, long long row) {
  const int rps = geom_rows_per_sample(g);
  Pixel p;
  p.b = static_cast<int>(row / rps);
  const int r = static_cast<int>(row - static_cast<long long>(p.b) * rps);
  const int w = r / g.n_local, tok = r - w * g.n_local;
  const int seq = g.sp_rank * g.n_local + tok;
  const int iy = seq / g.ws_x, ix = seq - iy * g.ws_x;
  const int wy = w / g.nwx_loc, wx = w - wy * g.nwx_loc;
  p.y = wy * g.ws_y + iy;
  p.x = wx * g.ws_x + ix;
  return p;
}
__device__ __forceinline__ unsigned long long global_pixel(const TokGeom& g, const Pixel& p) {
  return (static_cast<unsigned long long>(g.sample0 + p.b) * g.H + (g.y0 + p.y)) * g.W + (g.x0 + p.x);
}
__device__ __forceinline__ size_t block_pixel(const TokGeom& g, const Pixel& p) {
  return (static_cast<size_t>(p.b) * (g.nwy_loc * g.ws_y) + p.y) * (g.nwx_loc * g.ws_x) + p.x;
}

constexpr int EMBED_MAX_C = 256;
constexpr int EMBED_WARPS = 8;

// One warp per token row. Output row: [hi(v) | lo(v) | hi(v) | 1 | 1 | 0...] of width KP (bf16), v the fp32 model
// input cat[x_t / sigma_d, cond] + ape. Multiplied by [hi(W) | hi(W) | lo(W) | hi(b) | lo(b) | 0...] this gives
// v W^T + b up to the dropped lo*lo term.
__global__ void __launch_bounds__(EMBED_WARPS * 32)
embed_pack_kernel(const float* __restrict__ x_img, const float* __restrict__ c_img, const float* __restrict__ cs,
                  TokGeom g, int Cx, int Cc, const float* __restrict__ ape_y, const float* __restrict__ ape_x,
                  int ape_ch, unsigned long long seed, float sd, int noise, __nv_bfloat16* __restrict__ out, int KP,
                  long long row0, long long rows) {
  __shared__ float vbuf[EMBED_WARPS][EMBED_MAX_C];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* v = vbuf[warp];
  const int Cin = Cx + Cc;
  const float inv_sd = 1.0f / sd;
  for (long long i = static_cast<long long>(blockIdx.x) * EMBED_WARPS + warp; i < rows;
       i += static_cast<long long>(gridDim.x) * EMBED_WARPS) {
    const Pixel p = row_to_pixel(g, row0 + i);
    const size_t bp = block_pixel(g, p);
    const unsigned long long gp = global_pixel(g, p);
    const float ct = cs[2 * p.b], st = cs[2 * p.b + 1];
    for (int grp = lane; grp * 4 < Cx; grp += 32) {
      float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      if (noise) z = normal4(seed, gp, grp);
      const float zz[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = grp * 4 + k;
        if (c < Cx) v[c] = (ct * x_img[bp * Cx + c] + st * sd * zz[k]) * inv_sd;
      }
    }
    for (int c = lane; c < Cc; c += 32) v[Cx + c] = c_img[bp * Cc + c];
    __syncwarp();
    if (ape_y) {
      const float* ay = ape_y + static_cast<size_t>(g.y0 + p.y) * ape_ch;
      const float* ax = ape_x + static_cast<size_t>(g.x0 + p.x) * ape_ch;
      for (int c = lane; c < Cin; c += 32) {
        if (c < ape_ch) v[c] += ay[c];
        else if (c < 2 * ape_ch) v[c] += ax[c - ape_ch];
      }
      __syncwarp();
    }
    uint32_t* orow = reinterpret_cast<uint32_t*>(out + static_cast<size_t>(i) * KP);
    for (int j2 = lane; j2 < KP / 2; j2 += 32) {
      float o[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = 2 * j2 + h;
        float val = 0.f;
        if (j < 3 * Cin) {
          const int sec = j / Cin, c = j - sec * Cin;
          const float f = v[c];
          const float hi = __bfloat162float(__float2bfloat16_rn(f));
          val = (sec == 1) ? (f - hi) : hi;
        } else if (j < 3 * Cin + 2) {
          val = 1.0f;
        }
        o[h] = val;
      }
      orow[j2] = pack_bf16x2(o[0], o[1]);
    }
    __syncwarp();
  }
}

// Loss and its gradient. pred: fp32 [rows, ldp] (network output F in token order); the target is
// v = cos(t) z sigma_d - sin(t) x. loss += sum_rows sum_c w_var[c] w_lat[Y] (sigma_d F - v)^2 * inv_rows;
// dpred (bf16 [rows, ldd], columns >= Cx zero) = d loss / d F * gscale.
__global__ void __launch_bounds__(EMBED_WARPS * 32)
trigflow_loss_kernel(const float* __restrict__ pred, int ldp, const float* __restrict__ x_img,
                     const float* __restrict__ cs, TokGeom g, int Cx, unsigned long long seed, float sd,
                     const float* __restrict__ w_var, const float* __restrict__ w_lat, float inv_rows, float gscale,
                     __nv_bfloat16* __restrict__ dpred, int ldd, double* __restrict__ loss, long long row0,
                     long long rows) {
  __shared__ float part[EMBED_WARPS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float acc = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * EMBED_WARPS + warp; i < rows;
       i += static_cast<long long>(gridDim.x) * EMBED_WARPS) {
    const Pixel p = row_to_pixel(g, row0 + i);
    const size_t bp = block_pixel(g, p);
    const unsigned long long gp = global_pixel(g, p);
    const float ct = cs[2 * p.b], st = cs[2 * p.b + 1];
    const float wl = w_lat ? w_lat[g.y0 + p.y] : 1.0f;
    const float* prow = pred + static_cast<size_t>(i) * ldp;
    for (int grp = lane; grp * 4 < ldd; grp += 32) {
      float d[4] = {0.f, 0.f, 0.f, 0.f};
      if (grp * 4 < Cx) {
        const float4 z = normal4(seed, gp, grp);
        const float zz[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = grp * 4 + k;
          if (c < Cx) {
            const float vt = ct * sd * zz[k] - st * x_img[bp * Cx + c];
            const float e = sd * prow[c] - vt;
            const float wgt = (w_var ? w_var[c] : 1.0f) * wl;
            acc += wgt * e * e;
            d[k] = 2.0f * sd * wgt * e * inv_rows * gscale;
          }
        }
      }
      if (dpred) {
        uint2 u;
        u.x = pack_bf16x2(d[0], d[1]);
        u.y = pack_bf16x2(d[2], d[3]);
        *reinterpret_cast<uint2*>(dpred + static_cast<size_t>(i) * ldd + grp * 4) = u;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) part[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < EMBED_WARPS; ++w) s += part[w];
    atomicAdd(loss, static_cast<double>(s) * inv_rows);
  }
}

// x_out[pixel, c] = x_base[pixel, c] + ca * pa[row, c] + cb * pb[row, c]   (pa, pb in token order, x in image order)
__global__ void sampler_update_kernel(float* __restrict__ x_out, const float* __restrict__ x_base,
                                      const float* __restrict__ pa, const float* __restrict__ pb, int ldp, float ca,
                                      float cb, TokGeom g, int Cx, long long rows) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (long long i = static_cast<long long>(blockIdx.x) * nw + warp; i < rows;
       i += static_cast<long long>(gridDim.x) * nw) {
    const Pixel p = row_to_pixel(g, i);
    const size_t bp = block_pixel(g, p);
    for (int c = lane; c < Cx; c += 32) {
      float v = x_base[bp * Cx + c] + ca * pa[static_cast<size_t>(i) * ldp + c];
      if (pb) v += cb * pb[static_cast<size_t>(i) * ldp + c];
      x_out[bp * Cx + c] = v;
    }
  }
}

// x[pixel, c] = a * x[pixel, c] + b * z(pixel, c): initial noise (a = 0) and churn rotations of the sampler.
__global__ void noise_mix_kernel(float* __restrict__ x, float a, float b, unsigned long long seed, TokGeom g, int Cx,
                                 long long n_pix) {
  const int groups = (Cx + 3) / 4;
  const long long total = n_pix * groups;
  const int hb = g.nwy_loc * g.ws_y, wb = g.nwx_loc * g.ws_x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long pix = i / groups;
    const int grp = static_cast<int>(i - pix * groups);
    Pixel p;
    p.b = static_cast<int>(pix / (static_cast<long long>(hb) * wb));
    const int rem = static_cast<int>(pix - static_cast<long long>(p.b) * hb * wb);
    p.y = rem / wb;
    p.x = rem - p.y * wb;
    const float4 z = normal4(seed, global_pixel(g, p), grp);
    const float zz[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = grp * 4 + k;
      if (c < Cx) {
        float* q = x + pix * Cx + c;
        *q = (a != 0.f ? a * *q : 0.f) + b * zz[k];
      }
    }
  }
}

// out[i] = in[i] * a[c] + b[c] (+ add[i]), c = i mod C: standardise, un-standardise, residual add of the rollout.
__global__ void affine_channels_kernel(float* __restrict__ out, const float* __restrict__ in,
                                       const float* __restrict__ a, const float* __restrict__ b,
                                       const float* __restrict__ add, long long n, int C) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % C);
    float v = in[i] * a[c] + b[c];
    if (add) v += add[i];
    out[i] = v;
  }
}

// y[b, n] = act(sum_k W[n, k] x[b, k] + bias[n]) for B <= 8 rows: one warp per output feature streams one weight
// row. act: 0 none, 1 SiLU. W bf16 or fp32 (w_f32).
template <typename WT>
__global__ void gemv_bias_act_kernel(const WT* __restrict__ W, const float* __restrict__ bias,
                                     const float* __restrict__ x, float* __restrict__ y, int N, int K, int B, int act,
                                     int silu_in) {
  extern __shared__ float xs[];  // [B, K]
  for (int i = threadIdx.x; i < B * K; i += blockDim.x) {
    const float t = x[i];
    xs[i] = silu_in ? t / (1.f + __expf(-t)) : t;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int n = blockIdx.x * nw + warp; n < N; n += gridDim.x * nw) {
    float acc[8];
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[b] = 0.f;
    const WT* wr = W + static_cast<size_t>(n) * K;
    for (int k = lane; k < K; k += 32) {
      float w;
      if constexpr (sizeof(WT) == 2) w = __bfloat162float(wr[k]); else w = wr[k];
#pragma unroll
      for (int b = 0; b < 8; ++b)
        if (b < B) acc[b] = fmaf(w, xs[b * K + k], acc[b]);
    }
#pragma unroll
    for (int b = 0; b < 8; ++b) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[b] += __shfl_xor_sync(0xffffffffu, acc[b], o);
    }
    if (lane == 0) {
      const float bv = bias ? bias[n] : 0.f;
      for (int b = 0; b < B; ++b) {
        float v = acc[b] + bv;
        if (act == 1) v = v / (1.f + __expf(-v));
        y[static_cast<size_t>(b) * N + n] = v;
      }
    }
  }
}

}  // namespace aeris

using namespace aeris;
extern int aeris_num_sms();

static inline int warp_grid(long long rows, int warps_per_cta) {
  long long b = (rows + warps_per_cta - 1) / warps_per_cta;
  const long long cap = static_cast<long long>(aeris_num_sms()) * 16;
  if (b > cap) b = cap;
  return static_cast<int>(b < 1 ? 1 : b);
}
static inline bool geom_ok(const TokGeom* g) {
  return g && g->B > 0 && g->nwy_loc > 0 && g->nwx_loc > 0 && g->ws_y > 0 && g->ws_x > 0 && g->n_local > 0 &&
         g->sp_rank >= 0 && (g->sp_rank + 1) * g->n_local <= g->ws_y * g->ws_x;
}

extern "C" int aeris_embed_pack(const float* x_img, const float* c_img, const float* cs, const TokGeom* g, int Cx,
                                int Cc, const float* ape_y, const float* ape_x, int ape_ch,
                                unsigned long long seed, float sd, int noise, void* out, int KP, long long row0,
                                long long rows, void* stream) {
  if (!geom_ok(g) || Cx <= 0 || Cc < 0 || Cx + Cc > EMBED_MAX_C || KP % 8 || KP < 3 * (Cx + Cc) + 2 || rows <= 0)
    return -1;
  if (row0 < 0 || row0 + rows > static_cast<long long>(g->B) * g->nwy_loc * g->nwx_loc * g->n_local) return -2;
  embed_pack_kernel<<<warp_grid(rows, EMBED_WARPS), EMBED_WARPS * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      x_img, c_img, cs, *g, Cx, Cc, ape_y, ape_x, ape_ch, seed, sd, noise, reinterpret_cast<__nv_bfloat16*>(out), KP,
      row0, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_trigflow_loss(const float* pred, int ldp, const float* x_img, const float* cs, const TokGeom* g,
                                   int Cx, unsigned long long seed, float sd, const float* w_var, const float* w_lat,
                                   float inv_rows, float gscale, void* dpred, int ldd, double* loss, long long row0,
                                   long long rows, void* stream) {
  if (!geom_ok(g) || Cx <= 0 || Cx > ldp || ldd % 4 || (dpred && Cx > ldd) || rows <= 0) return -1;
  if (row0 < 0 || row0 + rows > static_cast<long long>(g->B) * g->nwy_loc * g->nwx_loc * g->n_local) return -2;
  trigflow_loss_kernel<<<warp_grid(rows, EMBED_WARPS), EMBED_WARPS * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pred, ldp, x_img, cs, *g, Cx, seed, sd, w_var, w_lat, inv_rows, gscale, reinterpret_cast<__nv_bfloat16*>(dpred),
      ldd, loss, row0, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_sampler_update(float* x_out, const float* x_base, const float* pa, const float* pb, int ldp,
                                    float ca, float cb, const TokGeom* g, int Cx, void* stream) {
  if (!geom_ok(g) || Cx <= 0 || Cx > ldp) return -1;
  const long long rows = static_cast<long long>(g->B) * g->nwy_loc * g->nwx_loc * g->n_local;
  sampler_update_kernel<<<warp_grid(rows, 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      x_out, x_base, pa, pb, ldp, ca, cb, *g, Cx, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_noise_mix(float* x, float a, float b, unsigned long long seed, const TokGeom* g, int Cx,
                               void* stream) {
  if (!geom_ok(g) || Cx <= 0) return -1;
  const long long n_pix = static_cast<long long>(g->B) * g->nwy_loc * g->ws_y * g->nwx_loc * g->ws_x;
  const long long work = n_pix * ((Cx + 3) / 4);
  long long blocks = (work + 255) / 256;
  const long long cap = static_cast<long long>(aeris_num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  noise_mix_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, a, b, seed, *g,
                                                                                                 Cx, n_pix);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_affine_channels(float* out, const float* in, const float* a, const float* b, const float* add,
                                     long long n, int C, void* stream) {
  if (n <= 0 || C <= 0) return -1;
  long long blocks = (n + 255) / 256;
  const long long cap = static_cast<long long>(aeris_num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  affine_channels_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(out, in, a, b,
                                                                                                       add, n, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_gemv_bias_act(const void* W, int w_f32, const float* bias, const float* x, float* y, int N, int K,
                                   int B, int act, int silu_in, void* stream) {
  if (N <= 0 || K <= 0 || B <= 0 || B > 8) return -1;
  const size_t smem = static_cast<size_t>(B) * K * sizeof(float);
  if (smem > 48 * 1024) return -2;
  const int warps = 8;
  int grid = (N + warps - 1) / warps;
  const int cap = aeris_num_sms() * 8;
  if (grid > cap) grid = cap;
  auto st = reinterpret_cast<cudaStream_t>(stream);
  if (w_f32)
    gemv_bias_act_kernel<float><<<grid, warps * 32, smem, st>>>(reinterpret_cast<const float*>(W), bias, x, y, N, K, B,
                                                               act, silu_in);
  else
    gemv_bias_act_kernel<__nv_bfloat16><<<grid, warps * 32, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(W),
                                                                       bias, x, y, N, K, B, act, silu_in);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
