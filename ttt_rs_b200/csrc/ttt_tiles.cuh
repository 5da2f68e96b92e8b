// Shared-memory tile formats per element type, and the per-thread "slab" (register tile) helpers.
//
// bf16 I/O: a tile is one swizzled bf16 plane written directly by TMA; tensor-core operands are read from it
// with ldmatrix and element-wise code reads the same bytes.
// f32 I/O: TMA lands the raw float tile (two swizzled 128-byte-row halves); all threads then split it into
// three bf16 planes (see Pk<3>) that ldmatrix reads, while element-wise code reads the raw floats.
#pragma once

#include <type_traits>

#include "ttt_common.cuh"

namespace ttt {

template <typename T>
struct TileFmt;

template <>
struct TileFmt<__nv_bfloat16> {
  static constexpr int NP = 1;
  static constexpr uint32_t RAW_BYTES = TILE_BF16_BYTES;
  static constexpr uint32_t PLANE_OFF = 0;              // plane 0 is the raw tile
  static constexpr uint32_t BYTES = TILE_BF16_BYTES;    // per tile, multiple of 1024
  static constexpr uint32_t ELT = 2;
  static constexpr int TMA_BOXES = 1;                   // one [16 x 64] box
  static constexpr int TMA_BOX_COLS = 64;
};
template <>
struct TileFmt<float> {
  static constexpr int NP = 3;
  static constexpr uint32_t RAW_BYTES = TILE_F32_BYTES;
  static constexpr uint32_t PLANE_OFF = TILE_F32_BYTES;
  static constexpr uint32_t BYTES = TILE_F32_BYTES + 3 * TILE_BF16_BYTES;  // 10240
  static constexpr uint32_t ELT = 4;
  static constexpr int TMA_BOXES = 2;                   // two [16 x 32] boxes
  static constexpr int TMA_BOX_COLS = 32;
};

// element pair (row, col..col+1), col even, from the raw tile
template <typename T>
__device__ __forceinline__ float2 ld_pair(uint32_t tile, int row, int col);
template <>
__device__ __forceinline__ float2 ld_pair<__nv_bfloat16>(uint32_t tile, int row, int col) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(tile + off_bf16(row, col)));
  return make_float2(bf16_lo(v), bf16_hi(v));
}
template <>
__device__ __forceinline__ float2 ld_pair<float>(uint32_t tile, int row, int col) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(tile + off_f32(row, col)));
  return v;
}
template <typename T>
__device__ __forceinline__ void st_pair(uint32_t tile, int row, int col, float x, float y);
template <>
__device__ __forceinline__ void st_pair<__nv_bfloat16>(uint32_t tile, int row, int col, float x, float y) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile + off_bf16(row, col)), "r"(pack_bf16(x, y)) : "memory");
}
template <>
__device__ __forceinline__ void st_pair<float>(uint32_t tile, int row, int col, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(tile + off_f32(row, col)), "f"(x), "f"(y) : "memory");
}

// Write an element pair into operand planes (bf16 planes at `planes`, plane stride 2048).
template <int NP>
__device__ __forceinline__ void st_pair_planes(uint32_t planes, int row, int col, float x, float y) {
  const Pk<NP> v = split_pack<NP>(x, y);
  const uint32_t a = planes + off_bf16(row, col);
#pragma unroll
  for (int p = 0; p < NP; ++p) asm volatile("st.shared.b32 [%0], %1;" ::"r"(a + p * TILE_BF16_BYTES), "r"(v.p[p]) : "memory");
}

// f32 only: split a raw float tile into its three bf16 operand planes. All 128 threads take part.
__device__ __forceinline__ void split_tile_f32(uint32_t tile, int tid) {
  const int row = tid >> 3, c0 = (tid & 7) << 3;
  float v[8];
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3])
               : "r"(tile + off_f32(row, c0)));
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
               : "r"(tile + off_f32(row, c0 + 4)));
  uint32_t pl[3][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const Pk<3> s = split_pack<3>(v[2 * i], v[2 * i + 1]);
    pl[0][i] = s.p[0];
    pl[1][i] = s.p[1];
    pl[2][i] = s.p[2];
  }
  const uint32_t dst = tile + TileFmt<float>::PLANE_OFF + off_bf16(row, c0);
#pragma unroll
  for (int p = 0; p < 3; ++p)
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst + p * TILE_BF16_BYTES), "r"(pl[p][0]),
                 "r"(pl[p][1]), "r"(pl[p][2]), "r"(pl[p][3])
                 : "memory");
}

// Issue the TMA load(s) of one [16 x 64] tile whose first row is `row0` of the 2-D view [rows, 64].
template <typename T>
__device__ __forceinline__ void tma_load_tile(uint32_t tile, const CUtensorMap* tm, int row0, uint32_t bar) {
  if constexpr (TileFmt<T>::TMA_BOXES == 1) {
    tma_load_2d(tile, tm, 0, row0, bar);
  } else {
    tma_load_2d(tile, tm, 0, row0, bar);
    tma_load_2d(tile + 2048, tm, 32, row0, bar);
  }
}
template <typename T>
__device__ __forceinline__ void tma_store_tile(const CUtensorMap* tm, int row0, uint32_t tile) {
  if constexpr (TileFmt<T>::TMA_BOXES == 1) {
    tma_store_2d(tm, 0, row0, tile);
  } else {
    tma_store_2d(tm, 0, row0, tile);
    tma_store_2d(tm, 32, row0, tile + 2048);
  }
}

// Tile of a PAIR of 32-wide heads (head_dim 32): the two heads' 16 x 32 blocks side by side in one 16 x 64 tile, so
// that the 64-wide kernels serve two such streams at once.  `pair` = index of the head pair (packed stream), `t0` =
// first token, `seq` = tokens per sequence; the caller's tensor is [B*H, seq, 32], heads 2 pair and 2 pair + 1.
//
// float32: a half tile is 16 rows of 128 bytes, exactly one 128-byte-swizzled TMA box of the 2-D view [B*H*seq, 32].
// bf16: a half tile is only 64 bytes wide, and a swizzled TMA box row narrower than the swizzle span still occupies a
// whole 128-byte row of shared memory, so TMA cannot put the two halves side by side.  The tile is gathered instead:
// 128 chunks of 16 bytes, one cp.async per thread, written at the swizzled position TMA would have used; results leave
// the same way (ld.shared + st.global per thread).
// How a kernel is handed one of the caller's [B,H,T,F] tensors: a TMA descriptor, or a plain pointer where the tiles
// are gathered (the kernel's parameter list is unchanged for every other instantiation).
struct alignas(64) RawTensor {
  void* ptr;
};
template <typename T, int SEG>
struct PairIo {
  static constexpr bool GATHER = (SEG == 32 && sizeof(T) == 2);
  using Ref = std::conditional_t<GATHER, RawTensor, CUtensorMap>;
};
template <int ROWS = 16>  // rows of the tile that exist (a mini-batch of 8 fills the first 8)
__device__ __forceinline__ void gather_pair_tile_bf16(uint32_t tile, const void* base, int pair, int t0, int seq, int tid) {
  const int row = tid >> 3, c = tid & 7;  // chunk c of the 128-byte row: head c >> 2, features 8 (c & 3) ..
  if (ROWS < 16 && row >= ROWS) return;
  const uint8_t* src = static_cast<const uint8_t*>(base) +
                       (((size_t)(2 * pair + (c >> 2)) * seq + t0 + row) * 32 + (c & 3) * 8) * 2;
  cp_async_16(tile + row * 128 + ((c ^ (row & 7)) << 4), src);
}
template <int ROWS = 16>
__device__ __forceinline__ void scatter_pair_tile_bf16(void* base, int pair, int t0, int seq, uint32_t tile, int tid) {
  const int row = tid >> 3, c = tid & 7;
  if (ROWS < 16 && row >= ROWS) return;
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(tile + row * 128 + ((c ^ (row & 7)) << 4)));
  uint8_t* dst = static_cast<uint8_t*>(base) + (((size_t)(2 * pair + (c >> 2)) * seq + t0 + row) * 32 + (c & 3) * 8) * 2;
  *reinterpret_cast<uint4*>(dst) = v;
}
// float32 pair tile by TMA: two boxes of the [B*H*seq, 32] view, one per head.
template <typename T>
__device__ __forceinline__ void tma_load_pair(uint32_t tile, const CUtensorMap* tm, int pair, int t0, int seq, uint32_t bar) {
  static_assert(sizeof(T) == 4, "bf16 pair tiles are gathered, not loaded by TMA");
  tma_load_2d(tile, tm, 0, (2 * pair) * seq + t0, bar);
  tma_load_2d(tile + 2048, tm, 0, (2 * pair + 1) * seq + t0, bar);
}
template <typename T>
__device__ __forceinline__ void tma_store_pair(const CUtensorMap* tm, int pair, int t0, int seq, uint32_t tile) {
  static_assert(sizeof(T) == 4, "bf16 pair tiles are scattered, not stored by TMA");
  tma_store_2d(tm, 0, (2 * pair) * seq + t0, tile);
  tma_store_2d(tm, 0, (2 * pair + 1) * seq + t0, tile + 2048);
}

}  // namespace ttt
