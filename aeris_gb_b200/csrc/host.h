// Host-side helpers shared by the .cu files (defined in gemm.cu).
#pragma once
#include <cuda.h>
#include <stdint.h>
namespace aeris {
// 2-D bf16 map with 128-byte swizzle: `inner` contiguous elements, `rows` rows of pitch `ld` elements.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t ld,
                      uint32_t box_inner, uint32_t box_rows);
// 3-D bf16 map with 128-byte swizzle: dims {d0 (contiguous), d1, d2}, pitches in elements, box {b0, b1, 1}.
int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                      uint64_t pitch2, uint32_t b0, uint32_t b1);
int num_sms();
}  // namespace aeris
