// Shared by the one-CTA and the two-CTA GEMM kernels: parameters and the TMEM -> registers -> global epilogue.
#pragma once
#include "common.cuh"

namespace aeris {

enum : int { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_GATE_RESID = 2, EPI_ACC_F32 = 3, EPI_STORE_F32 = 4,
              EPI_SWIGLU_BOTH = 5,   // EPI_SWIGLU that also stores the raw [gate | up] product to aux [M, 2F]
              EPI_SWIGLU_BWD = 6,    // acc = d(act); reads u = [gate | up] from resid [M, 2F], writes d(u) to C [M, 2F]
              EPI_SCATTER_HEADS = 7,    // Ulysses: every head's columns are stored into the buffer of the rank that
                                        // owns the head (peer memory), rows re-indexed to whole-window order
              EPI_RS_PUSH = 8 };        // reduce-scatter by rows: the bf16 partial tile of row block `o` is stored into
                                        // slot `rank` of owner o's [world * rows_per_rank, N] buffer (peer memory)

struct GemmParams {
  int M, N, K;
  int epi;
  void* C;
  int ldc;
  const __nv_bfloat16* resid;  // EPI_GATE_RESID: out = resid + gate[col] * acc
  int ldr;
  const float* gate;           // [M / rows_per_gate][N]
  int rows_per_gate;
  __nv_bfloat16* aux;          // optional raw copy of acc (bf16) in EPI_GATE_RESID
  int ld_aux;
  int b_tile_stride;           // rows of B advanced per n-tile (BN, or BN/2 for SwiGLU)
  int b_half_off;              // row offset of the second half-box of B (BN/2, or F for SwiGLU)
  int k_splits;
  int swiglu_f;                // F for the SwiGLU epilogues
  // EPI_SCATTER_HEADS: source columns are `n_sec` sections of width sec_w (q | k | v, or one section); inside a section
  // the columns of rank r's heads are [r * own_w, (r + 1) * own_w). Source row (window w, local token i) goes to row
  // w * L + rank * n_local + i of the owner's [*, n_sec * own_w] buffer.
  // EPI_RS_PUSH reuses scat_peers / scat_rank / scat_ld with scat_n_local = rows owned by one rank.
  void* scat_peers[8];
  int scat_rank, scat_n_local, scat_L, scat_sec_w, scat_own_w, scat_ld;
  // All-gather fused into the A operand (two-CTA kernel): A's rows are `ag_world` chunks of `ag_rows` rows. Chunk
  // ag_rank is this rank's own and already in place in `ag_local`; a copier thread PUSHES it into every peer's buffer
  // `ag_peers[p]` (same layout on every rank; bulk copies, nearest consumer first) and then adds 1 to word `ag_rank` of
  // that peer's counter array `ag_count_peers[p]`. Tiles of chunk c wait until the local word `ag_count[c]` reaches
  // `ag_expect` (counters only ever grow: expect = calls so far x CTAs per call).
  void* ag_peers[8];
  unsigned* ag_count_peers[8];
  const void* ag_local;
  const unsigned* ag_count;
  unsigned ag_expect;
  int ag_world, ag_rank, ag_rows;
  int tm_rot;       // first m-tile (of 256 rows) visited by the two-CTA kernel; the others follow cyclically. The
                    // reduce-scatter GEMM starts at the rows of rank + 1 and ends with its own, so that at any moment
                    // every rank pushes to a different owner and no GPU's ingress carries all the traffic
  int staged_out;   // bf16-output epilogues: move rows through the warp's shared-memory stage (coalesced global stores)
  int staged_red;   // split-K fp32 accumulation: stage 32 rows x 64 columns and issue the reductions row-contiguously
  int* status;
};


// Peer-memory pushes: a thread that owns one accumulator row would write 16-byte pieces of 32 different rows per store
// instruction, which crosses NVLink as 32 small packets. The push epilogues therefore stage 32 rows x 128 bf16 columns
// per warp in shared memory (`stage`, 8 KB, 16-byte chunks XOR-swizzled by row) and write them out as 256-byte row
// segments, two rows per store instruction.
constexpr int PUSH_STAGE_BYTES = 8192;
__device__ __forceinline__ void push_stage_put(uint8_t* stage, int lane, int col, const uint32_t (&o)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint4*>(stage + lane * 256 + (((col / 8 + i) ^ (lane & 15)) << 4)) =
        make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
}
// `dst_row`: where this lane's row stores its 128 staged columns (null: row not written).
__device__ __forceinline__ void push_stage_flush(uint8_t* stage, int lane, __nv_bfloat16* dst_row) {
  __syncwarp();
  const unsigned long long mine = reinterpret_cast<unsigned long long>(dst_row);
  const int ch = lane & 15;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int r = 2 * i + (lane >> 4);
    const unsigned long long d = __shfl_sync(0xffffffffu, mine, r);
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((ch ^ (r & 15)) << 4));
    if (d) *reinterpret_cast<uint4*>(d + ch * 16) = v;
  }
  __syncwarp();
}

// Same, but the staged 128 columns are two 64-column halves with different destinations (two 128-byte segments per row).
__device__ __forceinline__ void push_stage_flush2(uint8_t* stage, int lane, __nv_bfloat16* dst_a, __nv_bfloat16* dst_b) {
  __syncwarp();
  const unsigned long long ma = reinterpret_cast<unsigned long long>(dst_a);
  const unsigned long long mb = reinterpret_cast<unsigned long long>(dst_b);
  const int ch = lane & 15;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int r = 2 * i + (lane >> 4);
    const unsigned long long da = __shfl_sync(0xffffffffu, ma, r), db = __shfl_sync(0xffffffffu, mb, r);
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((ch ^ (r & 15)) << 4));
    const unsigned long long d = (ch < 8) ? da + ch * 16 : db + (ch - 8) * 16;
    if (da) *reinterpret_cast<uint4*>(d) = v;
  }
  __syncwarp();
}

// Reduce-scatter push: the same 32 rows x 128 columns per warp, but laid out linearly (row pitch 272 bytes: 16-byte
// accesses of the 8 lanes of a quarter warp fall into different banks), because every lane then hands its own 256-byte
// row segment to the TMA unit as one bulk copy into the owner's slot buffer. The epilogue warp neither issues the 16
// store instructions per group nor waits on posted peer stores; the copy engine keeps the link busy.
constexpr int RS_PITCH = 272;
constexpr int RS_STAGE_BYTES = 32 * RS_PITCH;   // 8704
__device__ __forceinline__ void rs_stage_put(uint8_t* stage, int lane, int col, const uint32_t (&o)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint4*>(stage + lane * RS_PITCH + (col / 8 + i) * 16) =
        make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
}
__device__ __forceinline__ void rs_stage_flush_bulk(uint8_t* stage, int lane, __nv_bfloat16* dst_row) {
  // this lane wrote its row through the generic proxy; the bulk copy reads it through the async proxy
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (dst_row)
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 256;" ::"l"(dst_row),
                 "r"(smem_u32(stage + lane * RS_PITCH))
                 : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// before this lane overwrites its staged row: the copy that read it has left shared memory
__device__ __forceinline__ void rs_stage_reuse_wait() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// before the kernel signals completion / exits: this lane's copies have been performed
__device__ __forceinline__ void rs_stage_drain() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// fp32 variant for the split-K reduction: the stage holds 32 rows x 64 fp32 columns; every flush instruction adds two
// 256-byte row segments to global memory (red.add), so the atomics of one instruction fall into 16 sectors, not 32.
__device__ __forceinline__ void push_stage_put_f32(uint8_t* stage, int lane, int col, const uint32_t (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 8; ++i)
    *reinterpret_cast<uint4*>(stage + lane * 256 + (((col / 4 + i) ^ (lane & 15)) << 4)) =
        make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}
__device__ __forceinline__ void push_stage_flush_red(uint8_t* stage, int lane, float* dst_row) {
  __syncwarp();
  const unsigned long long mine = reinterpret_cast<unsigned long long>(dst_row);
  const int ch = lane & 15;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int r = 2 * i + (lane >> 4);
    const unsigned long long d = __shfl_sync(0xffffffffu, mine, r);
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((ch ^ (r & 15)) << 4));
    if (d)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d + ch * 16), "f"(__uint_as_float(v.x)),
                   "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                   : "memory");
  }
  __syncwarp();
}

// One thread = one accumulator row (TMEM lane) of a BN-column tile whose first accumulator column is `taddr`.
// `row` is the global output row, `tn` the tile's index along N, `kempty` marks a split-K slice without work.
// `stage`: this warp's PUSH_STAGE_BYTES of shared memory for the push epilogues, or null (direct stores).
template <int BN>
__device__ __forceinline__ void gemm_epilogue_row(const GemmParams& p, uint32_t taddr, int row, bool row_ok, int tn,
                                                  bool kempty, uint8_t* stage = nullptr) {
  const int lane = threadIdx.x & 31;

  if (p.epi == EPI_SCATTER_HEADS) {
    const int w = row / p.scat_n_local;
    const size_t drow = static_cast<size_t>(w) * p.scat_L + p.scat_rank * p.scat_n_local + (row - w * p.scat_n_local);
    const bool staged = stage != nullptr && (p.scat_own_w % 128) == 0;   // a 128-column group has one owner
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c, v);
      tmem_wait_ld();
      const int c0 = tn * BN + (staged ? (c & ~127) : c);
      const int sec = c0 / p.scat_sec_w;
      const int hc = c0 - sec * p.scat_sec_w;
      const int owner = hc / p.scat_own_w;
#ifdef AERIS_BOUNDS_CHECK
      // checking build: the owner must be one of the (at most 8) ranks with a buffer; otherwise record and skip
      if (owner < 0 || owner >= 8 || p.scat_peers[owner] == nullptr) {
        if (p.status) atomicCAS(p.status, 0, ERR_BOUNDS);
        continue;
      }
#endif
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.scat_peers[owner]) + drow * p.scat_ld +
                           sec * p.scat_own_w + (hc - owner * p.scat_own_w);
      uint32_t o[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) o[i] = pack_bf16x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
      if (staged) {
        push_stage_put(stage, lane, c & 127, o);
        if ((c & 127) == 96) push_stage_flush(stage, lane, row_ok ? dst : nullptr);
      } else if (row_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(dst + 8 * i) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
      }
    }
  } else if (p.epi == EPI_RS_PUSH) {
    const int owner = row_ok ? row / p.scat_n_local : 0;
    const size_t drow = static_cast<size_t>(p.scat_rank) * p.scat_n_local + (row - owner * p.scat_n_local);
#ifdef AERIS_BOUNDS_CHECK
    // checking build: a row whose owner is not one of the (at most 8) ranks with a buffer is recorded and not stored
    // (the lane stays in the warp-wide staging below, as rows past the end of the matrix do)
    if (row_ok && (owner < 0 || owner >= 8 || p.scat_peers[owner < 8 ? owner : 0] == nullptr)) {
      if (p.status) atomicCAS(p.status, 0, ERR_BOUNDS);
      row_ok = false;
    }
#endif
    __nv_bfloat16* rowdst = reinterpret_cast<__nv_bfloat16*>(p.scat_peers[owner]) + drow * p.scat_ld + tn * BN;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c, v);
      tmem_wait_ld();
      uint32_t o[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) o[i] = pack_bf16x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
      if (stage) {
        if ((c & 127) == 0) rs_stage_reuse_wait();
        rs_stage_put(stage, lane, c & 127, o);
        if ((c & 127) == 96) rs_stage_flush_bulk(stage, lane, row_ok ? rowdst + (c - 96) : nullptr);
      } else if (row_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(rowdst + c + 8 * i) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
      }
    }
  } else if (p.epi == EPI_SWIGLU_BWD) {
    // d(gate) = d(act) * up * dsilu(gate), d(up) = d(act) * silu(gate); u is read and d(u) written in place
    const __nv_bfloat16* usrc = p.resid + static_cast<size_t>(row) * p.ldr + tn * BN;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + tn * BN;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c, v);
      tmem_wait_ld();
      if (row_ok) {
        uint32_t og[16], ou[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 g4 = *reinterpret_cast<const uint4*>(usrc + c + 8 * i);
          const uint4 u4 = *reinterpret_cast<const uint4*>(usrc + p.swiglu_f + c + 8 * i);
          const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 g2 = unpack_bf16x2(gw[j]), u2 = unpack_bf16x2(uw[j]);
            const float d0 = __uint_as_float(v[8 * i + 2 * j]), d1 = __uint_as_float(v[8 * i + 2 * j + 1]);
            const float s0 = 1.f / (1.f + __expf(-g2.x)), s1 = 1.f / (1.f + __expf(-g2.y));
            const float si0 = g2.x * s0, si1 = g2.y * s1;
            og[4 * i + j] = pack_bf16x2(d0 * u2.x * (s0 + si0 * (1.f - s0)), d1 * u2.y * (s1 + si1 * (1.f - s1)));
            ou[4 * i + j] = pack_bf16x2(d0 * si0, d1 * si1);
          }
        }
        if (stage != nullptr && p.staged_out) {
          // 64 d(gate) columns and the matching 64 d(up) columns share one stage group
          push_stage_put(stage, lane, (c & 32), og);
          push_stage_put(stage, lane, 64 + (c & 32), ou);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            *reinterpret_cast<uint4*>(dst + c + 8 * i) = make_uint4(og[4 * i], og[4 * i + 1], og[4 * i + 2], og[4 * i + 3]);
            *reinterpret_cast<uint4*>(dst + p.swiglu_f + c + 8 * i) =
                make_uint4(ou[4 * i], ou[4 * i + 1], ou[4 * i + 2], ou[4 * i + 3]);
          }
        }
      }
      if (stage != nullptr && p.staged_out && (c & 32))
        push_stage_flush2(stage, lane, row_ok ? dst + (c - 32) : nullptr, row_ok ? dst + p.swiglu_f + (c - 32) : nullptr);
    }
  } else if ((p.epi == EPI_SWIGLU || p.epi == EPI_SWIGLU_BOTH) && stage != nullptr && p.staged_out && BN == 256) {
    // staged stores: the 128 activation columns of the tile are one stage group; with EPI_SWIGLU_BOTH the raw gate
    // and up columns follow as two more groups (second pass over the accumulator in TMEM)
    constexpr int H = BN / 2;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + tn * H;
#pragma unroll 1
    for (int c = 0; c < H; c += 32) {
      uint32_t g[32], u[32];
      tmem_ld32(taddr + c, g);
      tmem_ld32(taddr + H + c, u);
      tmem_wait_ld();
      uint32_t o[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
        const float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
        const float s0 = g0 / (1.f + __expf(-g0)), s1 = g1 / (1.f + __expf(-g1));
        o[i] = pack_bf16x2(s0 * u0, s1 * u1);
      }
      push_stage_put(stage, lane, c, o);
    }
    push_stage_flush(stage, lane, row_ok ? out : nullptr);
    if (p.epi == EPI_SWIGLU_BOTH) {
      __nv_bfloat16* raw = p.aux + static_cast<size_t>(row) * p.ld_aux + tn * H;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
#pragma unroll 1
        for (int c = 0; c < H; c += 32) {
          uint32_t v[32], o[16];
          tmem_ld32(taddr + half * H + c, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = pack_bf16x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
          push_stage_put(stage, lane, c, o);
        }
        push_stage_flush(stage, lane, row_ok ? raw + half * p.swiglu_f : nullptr);
      }
    }
  } else if (p.epi == EPI_SWIGLU || p.epi == EPI_SWIGLU_BOTH) {
    constexpr int H = BN / 2;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + tn * H;
    __nv_bfloat16* raw = (p.epi == EPI_SWIGLU_BOTH) ? p.aux + static_cast<size_t>(row) * p.ld_aux + tn * H : nullptr;
#pragma unroll 1
    for (int c = 0; c < H; c += 32) {
      uint32_t g[32], u[32];
      tmem_ld32(taddr + c, g);
      tmem_ld32(taddr + H + c, u);
      tmem_wait_ld();
      if (row_ok) {
        if (raw) {
          uint32_t rg[16], ru[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            rg[i] = pack_bf16x2(__uint_as_float(g[2 * i]), __uint_as_float(g[2 * i + 1]));
            ru[i] = pack_bf16x2(__uint_as_float(u[2 * i]), __uint_as_float(u[2 * i + 1]));
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            *reinterpret_cast<uint4*>(raw + c + 8 * i) = make_uint4(rg[4 * i], rg[4 * i + 1], rg[4 * i + 2], rg[4 * i + 3]);
            *reinterpret_cast<uint4*>(raw + p.swiglu_f + c + 8 * i) =
                make_uint4(ru[4 * i], ru[4 * i + 1], ru[4 * i + 2], ru[4 * i + 3]);
          }
        }
        uint32_t o[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
          const float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
          const float s0 = g0 / (1.f + __expf(-g0)), s1 = g1 / (1.f + __expf(-g1));
          o[i] = pack_bf16x2(s0 * u0, s1 * u1);
        }
        uint4* dst = reinterpret_cast<uint4*>(out + c);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
      }
    }
  } else if (p.epi == EPI_ACC_F32 && p.k_splits > 1 && stage != nullptr && p.staged_red) {
    float* out = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + tn * BN;
    const bool live = row_ok && !kempty;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c, v);
      tmem_wait_ld();
      push_stage_put_f32(stage, lane, c & 32, v);
      if (c & 32) push_stage_flush_red(stage, lane, live ? out + (c - 32) : nullptr);
    }
  } else if (p.epi == EPI_ACC_F32 || p.epi == EPI_STORE_F32) {
    float* out = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + tn * BN;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c, v);
      tmem_wait_ld();
      if (row_ok && !kempty) {
        if (p.epi == EPI_STORE_F32) {
          float4* dst = reinterpret_cast<float4*>(out + c);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                 __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
        } else if (p.k_splits > 1) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + c + 4 * i),
                         "f"(__uint_as_float(v[4 * i])), "f"(__uint_as_float(v[4 * i + 1])),
                         "f"(__uint_as_float(v[4 * i + 2])), "f"(__uint_as_float(v[4 * i + 3]))
                         : "memory");
          }
        } else {
          float4* dst = reinterpret_cast<float4*>(out + c);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float4 o = dst[i];
            o.x += __uint_as_float(v[4 * i]);
            o.y += __uint_as_float(v[4 * i + 1]);
            o.z += __uint_as_float(v[4 * i + 2]);
            o.w += __uint_as_float(v[4 * i + 3]);
            dst[i] = o;
          }
        }
      }
    }
  } else if (stage != nullptr && p.staged_out && p.aux == nullptr) {
    // EPI_STORE / EPI_GATE_RESID with coalesced stores: every lane combines its own row (the residual is read
    // directly: staging it too was measured slower), the packed results of a 128-column group go through the warp's
    // stage and leave as 256-byte row segments.
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + tn * BN;
    const bool gated = (p.epi == EPI_GATE_RESID) && row_ok;
    const __nv_bfloat16* res = p.resid ? p.resid + static_cast<size_t>(row) * p.ldr + tn * BN : nullptr;
    const float* gate = nullptr;
    if (gated) gate = p.gate + static_cast<size_t>(row / p.rows_per_gate) * p.N + tn * BN;
    uint4 r4[4], r4n[4];       // residual of this and of the next 32 columns (requested one step ahead)
    if (gated) {
#pragma unroll
      for (int i = 0; i < 4; ++i) r4n[i] = reinterpret_cast<const uint4*>(res)[i];
    }
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c, v);
      if (gated) {
#pragma unroll
        for (int i = 0; i < 4; ++i) r4[i] = r4n[i];
        if (c + 32 < BN) {
#pragma unroll
          for (int i = 0; i < 4; ++i) r4n[i] = reinterpret_cast<const uint4*>(res + c + 32)[i];
        }
      }
      tmem_wait_ld();
      uint32_t o[16];
      if (gated) {
        const float4* gsrc = reinterpret_cast<const float4*>(gate + c);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t rr[4] = {r4[i].x, r4[i].y, r4[i].z, r4[i].w};
          const float4 ga = gsrc[2 * i], gb = gsrc[2 * i + 1];
          const float gg[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 r2 = unpack_bf16x2(rr[j]);
            const float a0 = __uint_as_float(v[8 * i + 2 * j]), a1 = __uint_as_float(v[8 * i + 2 * j + 1]);
            o[4 * i + j] = pack_bf16x2(fmaf(gg[2 * j], a0, r2.x), fmaf(gg[2 * j + 1], a1, r2.y));
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = pack_bf16x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
      }
      push_stage_put(stage, lane, c & 127, o);
      if ((c & 127) == 96) push_stage_flush(stage, lane, row_ok ? out + (c - 96) : nullptr);
    }
  } else {
    // EPI_STORE / EPI_GATE_RESID : bf16 output
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + tn * BN;
    const __nv_bfloat16* res =
        p.resid ? p.resid + static_cast<size_t>(row) * p.ldr + tn * BN : nullptr;
    const float* gate = nullptr;
    if (p.epi == EPI_GATE_RESID && row_ok)
      gate = p.gate + static_cast<size_t>(row / p.rows_per_gate) * p.N + tn * BN;
    __nv_bfloat16* aux = p.aux ? p.aux + static_cast<size_t>(row) * p.ld_aux + tn * BN : nullptr;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c, v);
      tmem_wait_ld();
      if (row_ok) {
        uint32_t o[16];
        if (p.epi == EPI_GATE_RESID) {
          if (aux) {
            uint32_t a[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
              a[i] = pack_bf16x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            uint4* adst = reinterpret_cast<uint4*>(aux + c);
#pragma unroll
            for (int i = 0; i < 4; ++i) adst[i] = make_uint4(a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
          }
          const uint4* rsrc = reinterpret_cast<const uint4*>(res + c);
          const float4* gsrc = reinterpret_cast<const float4*>(gate + c);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 r4 = rsrc[i];
            const uint32_t rr[4] = {r4.x, r4.y, r4.z, r4.w};
            const float4 ga = gsrc[2 * i], gb = gsrc[2 * i + 1];
            const float gg[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 r2 = unpack_bf16x2(rr[j]);
              const float a0 = __uint_as_float(v[8 * i + 2 * j]), a1 = __uint_as_float(v[8 * i + 2 * j + 1]);
              o[4 * i + j] = pack_bf16x2(fmaf(gg[2 * j], a0, r2.x), fmaf(gg[2 * j + 1], a1, r2.y));
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            o[i] = pack_bf16x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
        }
        uint4* dst = reinterpret_cast<uint4*>(out + c);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
      }
    }
  }
}

}  // namespace aeris
