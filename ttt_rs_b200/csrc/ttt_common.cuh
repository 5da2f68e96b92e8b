// Device-side building blocks shared by the fused TTT inner-loop kernels (sm_100a).
//
// Role: what the reference's tile library provides to its fused kernels (shared-memory tiles with an XOR
// swizzle, per-thread register tiles, cooperative loads/stores, "mma", row/column reductions:
// rust/thundercube/src/tiles/st.rs:9-47, tiles/mma.rs:71-187, cube/reduce.rs:131-259) is provided here by
//   * TMA tile loads/stores (cp.async.bulk.tensor, 128-byte swizzle) completed on mbarriers,
//   * ldmatrix / movmatrix fragment moves,
//   * warp-level tensor-core products mma.sync.m16n8k16 (bf16 operands, f32 accumulate),
//   * warp-shuffle row reductions plus a tiny shared-memory exchange across the four warps of a CTA.
//
// Data layout convention used by every kernel: a "tile" is 16 tokens (rows) x 64 features (columns).
// Warp w of the CTA owns columns [16w, 16w+16).  Inside a warp, lane = 4*g + t holds, of its 16x16 slab,
// rows {g, g+8} and columns {8*nt + 2t, 8*nt + 2t + 1 : nt = 0,1}: this is the accumulator layout of
// mma.m16n8k16, so products chain without moving data.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ttt {

constexpr int CS = 16;        // mini-batch length (tokens per stage)
constexpr int HD = 64;        // head dim
constexpr int NTHREADS = 128; // 4 warps per (batch, head) stream
constexpr uint32_t TILE_BF16_BYTES = CS * HD * 2;  // 2048
constexpr uint32_t TILE_F32_BYTES = CS * HD * 4;   // 4096
constexpr uint32_t SPIN_LIMIT = 1u << 22;          // bounded mbarrier wait (iterations of try_wait)

// status words written by kernels: [0] error code, [1] where, [2] block, [3] stage
enum : uint32_t { KST_OK = 0, KST_TIMEOUT = 6 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------------------------------
// mbarrier + TMA
// ----------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Returns false if the phase did not complete within SPIN_LIMIT polls (caller reports and leaves).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 2-D tiled TMA load into this CTA's shared memory, completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tm), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// 2-D tiled TMA store from shared memory (bulk async-group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tm), "r"(x),
               "r"(y), "r"(src)
               : "memory");
}
// 16-byte asynchronous copy global -> shared by the executing thread (not the bulk / TMA path), and the arrival that
// makes an mbarrier wait for all such copies the thread has issued so far.  `.noinc`: the arrival is one of the
// arrivals the barrier was initialised to expect.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory");
}

// ----------------------------------------------------------------------------------------------------
// Swizzled tile addressing (matches CU_TENSOR_MAP_SWIZZLE_128B; tile bases are 1024-byte aligned)
// ----------------------------------------------------------------------------------------------------
// bf16 tile [16][64]: 128 bytes per row.
__device__ __forceinline__ uint32_t off_bf16(int row, int col) {
  return static_cast<uint32_t>(row * 128 + ((((col >> 3) ^ row) & 7) << 4) + ((col & 7) << 1));
}
// f32 tile [16][64] stored as two half tiles [16][32] of 128-byte rows (2048 bytes each).
__device__ __forceinline__ uint32_t off_f32(int row, int col) {
  return static_cast<uint32_t>(((col >> 5) << 11) + row * 128 + (((((col & 31) >> 2) ^ row) & 7) << 4) +
                               ((col & 3) << 2));
}

// ----------------------------------------------------------------------------------------------------
// Fragment moves
// ----------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// Transpose an 8x8 matrix of 16-bit values held one register per lane across the warp.
__device__ __forceinline__ uint32_t movm_t(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t a0, const uint32_t a1, const uint32_t a2,
                                         const uint32_t a3, const uint32_t b0, const uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// pack two floats into bf16x2 (lo = first element)
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// ----------------------------------------------------------------------------------------------------
// Operand planes.  NP = 1: operands are bf16.  NP = 3: a float is carried as three bf16 planes
// (x = p0 + p1 + p2, 24 mantissa bits) and a product uses the six plane pairs whose weight is >= 2^-16,
// which reproduces float32 operand precision on the bf16 tensor-core path.
// ----------------------------------------------------------------------------------------------------
template <int NP>
struct Pk {  // one 32-bit fragment register position (a pair of elements), NP planes
  uint32_t p[NP];
};

template <int NP>
__device__ __forceinline__ Pk<NP> split_pack(float x, float y);
template <>
__device__ __forceinline__ Pk<1> split_pack<1>(float x, float y) {
  Pk<1> r;
  r.p[0] = pack_bf16(x, y);
  return r;
}
template <>
__device__ __forceinline__ Pk<3> split_pack<3>(float x, float y) {
  Pk<3> r;
  r.p[0] = pack_bf16(x, y);
  float rx = x - bf16_lo(r.p[0]), ry = y - bf16_hi(r.p[0]);
  r.p[1] = pack_bf16(rx, ry);
  rx -= bf16_lo(r.p[1]);
  ry -= bf16_hi(r.p[1]);
  r.p[2] = pack_bf16(rx, ry);
  return r;
}

template <int NP>
__device__ __forceinline__ void mma_np(float (&c)[4], const Pk<NP> (&a)[4], const Pk<NP> (&b)[2]) {
  if constexpr (NP == 1) {
    mma_bf16(c, a[0].p[0], a[1].p[0], a[2].p[0], a[3].p[0], b[0].p[0], b[1].p[0]);
  } else {
    // The tensor core adds products to its accumulator with truncation, which biases long chained sums.
    // So each k-step is summed from zero (small cross terms and the leading term apart) and joined to the
    // running float32 accumulator with ordinary round-to-nearest adds.
    float lo[4] = {0.f, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
    constexpr int PA[5] = {1, 2, 0, 1, 0};
    constexpr int PB[5] = {1, 0, 2, 0, 1};
#pragma unroll
    for (int i = 0; i < 5; ++i)
      mma_bf16(lo, a[0].p[PA[i]], a[1].p[PA[i]], a[2].p[PA[i]], a[3].p[PA[i]], b[0].p[PB[i]], b[1].p[PB[i]]);
    mma_bf16(hi, a[0].p[0], a[1].p[0], a[2].p[0], a[3].p[0], b[0].p[0], b[1].p[0]);
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] += hi[i] + lo[i];
  }
}

template <int NP>
__device__ __forceinline__ Pk<NP> movm_t_np(const Pk<NP>& a) {
  Pk<NP> r;
#pragma unroll
  for (int i = 0; i < NP; ++i) r.p[i] = movm_t(a.p[i]);
  return r;
}

// ldmatrix x4 over NP planes (plane stride in bytes)
template <int NP>
__device__ __forceinline__ void ldsm_np(Pk<NP> (&r)[4], uint32_t addr, uint32_t plane_stride, bool trans) {
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    uint32_t v[4];
    if (trans)
      ldsm_x4_t(v, addr + p * plane_stride);
    else
      ldsm_x4(v, addr + p * plane_stride);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i].p[p] = v[i];
  }
}

// Lane address helpers for ldmatrix.x4 on a swizzled bf16 tile [16][64].
//  A operand (16 rows x 16 k-columns starting at kc): regs = {rows0-7/k-lo, rows8-15/k-lo, rows0-7/k-hi, rows8-15/k-hi}
__device__ __forceinline__ uint32_t lane_off_A(int lane, int kc) {
  const int m = lane >> 3, r = lane & 7;
  return off_bf16(r + ((m & 1) << 3), kc + ((m >> 1) << 3));
}
//  B operand read from a tile stored [n][k] (rows index the product's N, columns its K), both 8-row n-tiles,
//  16 k-columns starting at kc: regs = {n0-7/k-lo, n0-7/k-hi, n8-15/k-lo, n8-15/k-hi}
__device__ __forceinline__ uint32_t lane_off_B_nk(int lane, int kc) {
  const int m = lane >> 3, r = lane & 7;
  return off_bf16(r + ((m >> 1) << 3), kc + ((m & 1) << 3));
}
//  B operand read (with .trans) from a tile stored [k][n] (rows index the product's K = 16 tokens, columns
//  its N): two adjacent 8-column n-tiles starting at nc: regs = {k0-7/n-tile0, k8-15/n-tile0, k0-7/n-tile1, k8-15/n-tile1}
__device__ __forceinline__ uint32_t lane_off_B_kn(int lane, int nc) {
  const int m = lane >> 3, r = lane & 7;
  return off_bf16(r + ((m & 1) << 3), nc + ((m >> 1) << 3));
}

// ----------------------------------------------------------------------------------------------------
// Packed float32x2 arithmetic (one instruction per column pair on sm_100).
// ----------------------------------------------------------------------------------------------------
typedef float2 F2;
__device__ __forceinline__ F2 f2(float a) { return make_float2(a, a); }
__device__ __forceinline__ F2 f2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ F2 f2fma(F2 a, F2 b, F2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ F2 f2mul(F2 a, F2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ F2 f2add(F2 a, F2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ F2 f2sub(F2 a, F2 b) { return __ffma2_rn(b, make_float2(-1.f, -1.f), a); }
__device__ __forceinline__ F2 f2neg(F2 a) { return make_float2(-a.x, -a.y); }
__device__ __forceinline__ float f2hsum(F2 a) { return a.x + a.y; }
// accumulator quad {r0e0, r0e1, r1e0, r1e1} viewed as the column pair of row r
__device__ __forceinline__ F2 pr(const float (&c)[4], int r) { return make_float2(c[2 * r], c[2 * r + 1]); }

// ----------------------------------------------------------------------------------------------------
// Reductions
// ----------------------------------------------------------------------------------------------------
// sum over the 4 lanes that share a row (lane bits 0,1)
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}
// sum over the 8 lanes that share a column pair (lane bits 2,3,4)
__device__ __forceinline__ float col_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  return v;
}

template <typename T>
__device__ __forceinline__ float ld_as_float(const void* base, size_t idx);
template <>
__device__ __forceinline__ float ld_as_float<float>(const void* base, size_t idx) {
  return static_cast<const float*>(base)[idx];
}
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const void* base, size_t idx) {
  return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
}
template <typename T>
__device__ __forceinline__ void st_from_float(void* base, size_t idx, float v);
template <>
__device__ __forceinline__ void st_from_float<float>(void* base, size_t idx, float v) {
  static_cast<float*>(base)[idx] = v;
}
template <>
__device__ __forceinline__ void st_from_float<__nv_bfloat16>(void* base, size_t idx, float v) {
  static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
}


// ---- tensor memory as a per-thread scratchpad (no tensor-core instruction touches it) ---------------------------
// A warp can address the 32 tensor-memory lanes of its quarter (warp index % 4) only, and with the 32x32b shape lane l
// of the warp gets lane 32 (warp % 4) + l: N consecutive columns of that lane are N private 32-bit words of the
// thread.  A kernel whose per-thread float32 state crowds its registers keeps it there between the places that use
// it: a load + store round trip of 32 columns costs about 100 cycles (measured by probe_chain_latency.cu).
// taddr = allocation base + (first lane of the quarter << 16) + column.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, int columns) {  // one whole warp; a power of 2 >= 32
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, int columns) {  // the warp that allocated
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 columns <-> an [8][4] register array (the accumulator fragments of eight 16 x 8 tiles).  The load waits for its
// data; the store does not wait: tmem_wait_st() before the next load of the same columns.
__device__ __forceinline__ void tmem_ld_8x4(uint32_t taddr, float (&r)[8][4]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=f"(r[0][0]), "=f"(r[0][1]), "=f"(r[0][2]), "=f"(r[0][3]), "=f"(r[1][0]), "=f"(r[1][1]), "=f"(r[1][2]), "=f"(r[1][3]), "=f"(r[2][0]), "=f"(r[2][1]), "=f"(r[2][2]), "=f"(r[2][3]), "=f"(r[3][0]), "=f"(r[3][1]), "=f"(r[3][2]), "=f"(r[3][3]), "=f"(r[4][0]), "=f"(r[4][1]), "=f"(r[4][2]), "=f"(r[4][3]), "=f"(r[5][0]), "=f"(r[5][1]), "=f"(r[5][2]), "=f"(r[5][3]), "=f"(r[6][0]), "=f"(r[6][1]), "=f"(r[6][2]), "=f"(r[6][3]), "=f"(r[7][0]), "=f"(r[7][1]), "=f"(r[7][2]), "=f"(r[7][3])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_8x4(uint32_t taddr, const float (&r)[8][4]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
      ::"f"(r[0][0]), "f"(r[0][1]), "f"(r[0][2]), "f"(r[0][3]), "f"(r[1][0]), "f"(r[1][1]), "f"(r[1][2]), "f"(r[1][3]), "f"(r[2][0]), "f"(r[2][1]), "f"(r[2][2]), "f"(r[2][3]), "f"(r[3][0]), "f"(r[3][1]), "f"(r[3][2]), "f"(r[3][3]), "f"(r[4][0]), "f"(r[4][1]), "f"(r[4][2]), "f"(r[4][3]), "f"(r[5][0]), "f"(r[5][1]), "f"(r[5][2]), "f"(r[5][3]), "f"(r[6][0]), "f"(r[6][1]), "f"(r[6][2]), "f"(r[6][3]), "f"(r[7][0]), "f"(r[7][1]), "f"(r[7][2]), "f"(r[7][3]), "r"(taddr)
      : "memory");
}

}  // namespace ttt
