// Collectives written as kernels over peer memory (NVLink P2P mappings of symmetric buffers, optionally the NVSwitch
// multicast address of the same buffers), fused with the arithmetic that surrounds them:
//
//   * signal barrier between the ranks of one node: release-stores of an epoch into every peer's flag word, bounded
//     acquire-spin on the own flags
//   * gradient reduce-scatter + scale + sum of squares in one pass: every rank pulls its shard of the flat fp32
//     gradient from all peers (plain P2P loads, or one multimem.ld_reduce per vector through the switch)
//   * AdamW on the fp32 master shard (+ clip, NaN guard, EMA) whose bf16 result is written straight into every
//     peer's parameter buffer (P2P stores, or one multimem.st per vector): the all-gather is the store
//
// Reference behaviour replaced: flat-buffer all-reduce / reduce-scatter, scaling, clipping, optimizer step and
// all-gather as separate framework calls (src/aeris/parallelism/parallel_engine.py:709-724, 751-787, 832-859).
//
// Every wait is bounded; a time-out sets the status word and the kernel returns. No TMA, no cluster multicast here.
#include "common.cuh"
#include "api.h"

namespace aeris {

struct PeerList {
  void* p[16];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// flags[r][q] (uint32, one row of 32 words per rank): rank q's arrival epoch as seen by rank r.
// One CTA; thread q < world handles peer q.
__global__ void signal_barrier_kernel(PeerList flags, int rank, int world, uint32_t epoch, int* status,
                                      unsigned long long timeout_ns) {
  const int q = threadIdx.x;
  if (q < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[q]) + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + q;
    const uint64_t t0 = globaltimer_ns();
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (status) atomicCAS(status, 0, ERR_TIMEOUT_SIGNAL);
        break;
      }
      __nanosleep(200);
    }
  }
}

// Waits (bounded) until *flag >= expected. Used by the tests of the time-out path: a flag that nothing sets.
__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t expected, int* status, unsigned long long timeout_ns) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();
    while (static_cast<int32_t>(ld_acquire_sys(flag) - expected) < 0) {
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (status) atomicCAS(status, 0, ERR_TIMEOUT_SIGNAL);
        break;
      }
      __nanosleep(500);
    }
  }
}

__device__ __forceinline__ float4 ld_cg_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b128(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// Reduce-scatter of this rank's shard [lo, lo + n) of the flat fp32 gradient: out[i] = scale * sum_r grad_r[lo + i];
// sumsq += sum out[i]^2 (double). n is a multiple of 4. With `mc` (multicast address of the gradient buffer) the sum is
// done by the switch; otherwise by `world` peer loads.
__global__ void grad_reduce_scatter_kernel(PeerList grads, const float* mc, int world, long long lo, long long n,
                                           float scale, float* __restrict__ out, double* __restrict__ sumsq) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 s;
    if (mc) {
      s = multimem_ld_reduce_f4(mc + lo + 4 * i);
    } else {
      s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const float4 v = ld_cg_f4(reinterpret_cast<const float*>(grads.p[r]) + lo + 4 * i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += red[w];
    atomicAdd(sumsq, static_cast<double>(t));
  }
}

struct ShardAdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2, max_norm, ema_beta, nan_clamp;
};
// AdamW on the shard; the bf16 result is written into every rank's parameter buffer at [lo, lo + n). Eight elements
// per thread iteration so that each peer store is one 16-byte vector. `grad` is the already reduced and scaled shard.
__global__ void shard_adamw_allgather_kernel(float* __restrict__ master, const float* __restrict__ grad,
                                             float* __restrict__ m, float* __restrict__ v, float* __restrict__ ema,
                                             PeerList params, void* mc_params, int world, long long lo, long long n,
                                             const double* __restrict__ norm_sq, ShardAdamArgs a) {
  float clip = 1.f;
  if (a.max_norm > 0.f && norm_sq) {
    const float c = a.max_norm / (static_cast<float>(sqrt(*norm_sq)) + 1.0e-6f);
    if (c < 1.f) clip = c;
  }
  const long long n8 = n / 8;
  const bool do_ema = ema && a.ema_beta >= 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    // 16-byte vector loads: two per array and thread, all issued before the first use
    float4 g4[2], p4[2], m4[2], v4[2], e4[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long j = 2 * i + h;
      g4[h] = reinterpret_cast<const float4*>(grad)[j];
      p4[h] = reinterpret_cast<const float4*>(master)[j];
      m4[h] = reinterpret_cast<const float4*>(m)[j];
      v4[h] = reinterpret_cast<const float4*>(v)[j];
      if (do_ema) e4[h] = reinterpret_cast<const float4*>(ema)[j];
    }
    float pw[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float* gg = reinterpret_cast<float*>(&g4[h]);
      float* pp = reinterpret_cast<float*>(&p4[h]);
      float* mm = reinterpret_cast<float*>(&m4[h]);
      float* vv = reinterpret_cast<float*>(&v4[h]);
      float* ee = reinterpret_cast<float*>(&e4[h]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float g = gg[k] * clip;
        if (g != g) g = 0.f;
        else if (g > 3.0e38f) g = a.nan_clamp;
        else if (g < -3.0e38f) g = -a.nan_clamp;
        float p = pp[k];
        const float mi = a.beta1 * mm[k] + (1.f - a.beta1) * g;
        const float vi = a.beta2 * vv[k] + (1.f - a.beta2) * g * g;
        mm[k] = mi;
        vv[k] = vi;
        p *= (1.f - a.lr * a.weight_decay);
        p -= a.lr * (mi / a.bias1) / (sqrtf(vi / a.bias2) + a.eps);
        pp[k] = p;
        if (do_ema) ee[k] = p + a.ema_beta * (ee[k] - p);
        pw[4 * h + k] = p;
      }
      const long long j = 2 * i + h;
      reinterpret_cast<float4*>(master)[j] = p4[h];
      reinterpret_cast<float4*>(m)[j] = m4[h];
      reinterpret_cast<float4*>(v)[j] = v4[h];
      if (do_ema) reinterpret_cast<float4*>(ema)[j] = e4[h];
    }
    uint4 u;
    u.x = pack_bf16x2(pw[0], pw[1]);
    u.y = pack_bf16x2(pw[2], pw[3]);
    u.z = pack_bf16x2(pw[4], pw[5]);
    u.w = pack_bf16x2(pw[6], pw[7]);
    if (mc_params) {
      multimem_st_b128(reinterpret_cast<__nv_bfloat16*>(mc_params) + lo + 8 * i, u);
    } else {
      for (int r = 0; r < world; ++r)
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + lo + 8 * i) = u;
    }
  }
}

}  // namespace aeris

using namespace aeris;
extern int aeris_num_sms();

static PeerList make_list(const void* const* ptrs, int n) {
  PeerList l{};
  for (int i = 0; i < n && i < 16; ++i) l.p[i] = const_cast<void*>(ptrs[i]);
  return l;
}

extern "C" int aeris_signal_barrier(const void* const* flag_ptrs, int rank, int world, unsigned epoch, int* status,
                                    double timeout_s, void* stream) {
  if (world < 1 || world > 16 || rank < 0 || rank >= world) return -1;
  signal_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_list(flag_ptrs, world), rank, world, epoch, status, static_cast<unsigned long long>(timeout_s * 1e9));
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_wait_flag(const void* flag, unsigned expected, int* status, double timeout_s, void* stream) {
  wait_flag_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(flag), expected, status, static_cast<unsigned long long>(timeout_s * 1e9));
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_grad_reduce_scatter(const void* const* grad_ptrs, const void* mc_grad, int world, long long lo,
                                         long long n, float scale, float* out, double* sumsq, void* stream) {
  if (world < 1 || world > 16 || n <= 0 || (n & 3) || (lo & 3)) return -1;
  long long blocks = (n / 4 + 255) / 256;
  const long long cap = static_cast<long long>(aeris_num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  grad_reduce_scatter_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_list(grad_ptrs, world), reinterpret_cast<const float*>(mc_grad), world, lo, n, scale, out, sumsq);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int aeris_shard_adamw_allgather(float* master, const float* grad, float* m, float* v, float* ema,
                                           const void* const* param_ptrs, void* mc_params, int world, long long lo,
                                           long long n, const double* norm_sq, float lr, float beta1, float beta2,
                                           float eps, float weight_decay, int step, float max_norm, float ema_beta,
                                           void* stream) {
  if (world < 1 || world > 16 || n <= 0 || (n & 7) || (lo & 7)) return -1;
  ShardAdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f - powf(beta1, static_cast<float>(step));
  a.bias2 = 1.f - powf(beta2, static_cast<float>(step));
  a.max_norm = max_norm; a.ema_beta = ema_beta; a.nan_clamp = 1.0e5f;
  long long blocks = (n / 8 + 255) / 256;
  const long long cap = static_cast<long long>(aeris_num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  shard_adamw_allgather_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      master, grad, m, v, ema, make_list(param_ptrs, world), mc_params, world, lo, n, norm_sq, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
