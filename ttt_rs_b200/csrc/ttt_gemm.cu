// bf16 GEMM for the outer layer's projections on the 5th-generation tensor cores (sm_100a):
//     C[M, N] = A[M, K] . B[N, K]^T      (A = hidden states, rows = tokens; B = a weight matrix as the layer stores
//                                          it, rows = output features; float32 accumulation, bf16 result)
// This is the product behind the reference layer's `Linear` projections q/k/v/g, the per-head learning-rate weights
// and o_proj (rust/layer/src/ttt.rs:152-227,289-299), which it gets from Burn's matmul.
//
// Persistent CTAs (one per SM) walk the 128 x 256 tiles of C, n fastest (the CTAs running at one time share a few
// row blocks of A through L2; B stays L2-resident).  The tile is 256 wide because a tcgen05.mma reads both operands
// from shared memory for every instruction: at M = 128, N = 128, K = 16 that is 8 KB per 64 tensor-pipe cycles, the
// whole 128 bytes per cycle of an SM's shared memory, which the TMA fill of the next stages needs as well -- such
// tiles measured 39-47 % tensor-pipe activity whatever the pipeline depth; at N = 256 the same bytes of A serve twice
// the columns (12 KB per 128 cycles).
//   * warp 0 (one lane) is the TMA producer: an A tile of 128 rows x 64 k and a B tile of 256 rows x 64 k (128-byte
//     rows, 128-byte swizzle) per stage into a ring of shared-memory stages that never drains between tiles,
//     completion counted in bytes on the stage's `full` mbarrier;
//   * warp 1 (one lane) issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = 256 -- less in the last tile column,
//     any multiple of 16 -- K = 16): operands by shared-memory descriptor, accumulators in tensor memory -- TWO buffers
//     of 128 lanes x 256 float32 columns (all 512 columns of the SM), used alternately; after the four k-steps of a
//     stage a tcgen05.commit on the stage's `empty` mbarrier hands the stage back to the producer, and after a tile's
//     last stage a commit on `acc_full[buffer]` releases the epilogue;
//   * warps 2-5 are the epilogue: each reads its quarter of the tensor-memory lanes (one row per thread) with
//     tcgen05.ld, 64 columns at a time, converts to bf16, writes a swizzled staging tile (two, used alternately) and
//     one thread stores it with TMA (rows / columns beyond M / N are clipped by the tensor map); after the last read
//     `acc_empty[buffer]` gives the accumulator back.  So the epilogue of tile i runs under the main loop of tile i + 1.
// In this form every CTA is on its own: no thread-block cluster, each CTA loads its own operands.
//
// Pair form (PAIR = true; tcgen05 cta_group::2): two CTAs of a cluster, on neighbouring SMs, share one 256 x 256 tile.
// CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and rows [128 r, ...) of the B tile into its own
// shared memory only (TMA loads whose bytes are counted on the LEADER's `full` barrier, cta_group::2 form:
// half the B bytes per CTA and per FLOP of the single form, and what a tcgen05.mma reads per cycle drops from 96 to 64
// bytes per SM); the CTA of rank 0 issues tcgen05.mma.cta_group::2 (M = 256: 128 rows in each CTA's tensor memory;
// N = 256: 128 rows of B from each CTA's shared memory at the same offset) once the stage is full in both CTAs, and
// commits every hand-back twice, to its own barrier and to the peer's (mapa address).  Each CTA's epilogue drains its own 128 accumulator rows; the leader
// reuses an accumulator when both epilogues have arrived on its `acc_empty` (count 2, the peer's arrival remote).
// Before leaving, each producer waits for the last hand-backs of its stages and the leader for the last accumulator
// releases, so that no remote arrival can land in the shared memory of a CTA that has exited; a cluster barrier then
// precedes the release of tensor memory.
//
// Fused form (ttt_layer_projections): the same main loop over the layer's stacked q | k | v | (g) | lr weights, with
// the step that follows the projections in the layer folded into the epilogue -- what `get_qkv` / `get_lr` do with the
// projection output (rust/layer/src/ttt.rs:152-227): every 64-column quarter of a tile is one head of q, k, v or the
// gate, or the block of learning-rate logits.  q and k quarters are rotated (rotary pairs are adjacent columns, so a
// pair sits in one thread's registers, still in float32) and stored as XQ / XK [B,H,T,F]; v quarters go to XV, gate
// quarters to a [B*T, H*F] buffer, logits become ttt_lr_eta[b,h,t] = base_lr / F * sigmoid(logit + bias).  The
// [B*T, N] projection output is never written.  Needs seq_len % 128 == 0 (a tile's 128 tokens then belong to one
// batch element and land in 128 consecutive rows of [B*H*T, F]).
//
// Every mbarrier wait is bounded: on expiry the role sets a flag, everybody falls through to the common exit, tensor
// memory is freed and the status words get {TTT_ERR_TIMEOUT, where, block, k-block}.
#include <cstdio>
#include <cstdlib>

#include "ttt_kernels.h"
#include "ttt_stage.cuh"

namespace ttt {

constexpr int GEMM_BM = 128, GEMM_BN = 256, GEMM_BK = 64;
constexpr uint32_t GEMM_A_BYTES = GEMM_BM * GEMM_BK * 2;  // 16 KB: the A tile of a stage
constexpr uint32_t GEMM_B_BYTES = GEMM_BN * GEMM_BK * 2;  // 32 KB: the B tile of a stage
constexpr uint32_t GEMM_STAGE_BYTES = GEMM_A_BYTES + GEMM_B_BYTES;
constexpr uint32_t GEMM_STG_BYTES = GEMM_BM * 64 * 2;     // 16 KB: one [128][64] bf16 staging tile of the epilogue
constexpr int GEMM_THREADS = 192;

template <bool FUSED, bool PAIR>
struct GemmSmem {
  // a stage: the A tile, then this CTA's rows of the B tile (all 256, or 128 of them in the pair form); the fused
  // form keeps a rotary table in shared memory and gives up one stage for it
  static constexpr uint32_t B_BYTES = PAIR ? GEMM_B_BYTES / 2 : GEMM_B_BYTES;
  static constexpr uint32_t STAGE_BYTES = GEMM_A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? (FUSED ? 5 : 6) : (FUSED ? 3 : 4);
  static constexpr uint32_t OFF_STG = STAGES * STAGE_BYTES;         // epilogue staging: two [128][64] bf16 tiles
  // full[S], empty[S], acc_full[2], acc_empty[2]
  static constexpr uint32_t OFF_BAR = OFF_STG + 2 * GEMM_STG_BYTES;
  static constexpr int NBAR = 2 * STAGES + 4;
  static constexpr uint32_t OFF_TMEM = OFF_BAR + NBAR * 8;
  // fused epilogue: (cos, sin) for 16 positions x 32 pairs; rows padded to 33 entries so that the 16 rows the lanes
  // of a warp read (consecutive tokens = consecutive positions) fall in distinct banks
  static constexpr uint32_t OFF_ROPE = OFF_TMEM + 8;
  static constexpr uint32_t ROPE_ROW = 33;
  static constexpr uint32_t TOTAL = OFF_ROPE + (FUSED ? 16 * ROPE_ROW * 8 : 0);
  static constexpr uint32_t DYN_BYTES = TOTAL + 1024;
};

// shared-memory matrix descriptor for a K-major bf16 tile of 128-byte rows with 128-byte swizzle: start address >> 4,
// stride between 8-row groups = 1024 bytes, descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// instruction descriptor, kind::f16: D float32 (bit 4), A and B bf16 (bits 7, 10), both K-major, N >> 3 at bit 17,
// M >> 4 at bit 24
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N) {  // N: a multiple of 16, 16..256, at M = 128
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// cta_group::2 forms: issued by the leader CTA of a pair; `bar` of the commit may be a mapa address in the peer.
__device__ __forceinline__ void umma2_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// address of `addr` (a shared-memory address of this CTA) in the CTA of rank `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// bounded wait on a barrier of this CTA whose arrivals come from the other CTA of the cluster
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// 2-D tiled TMA load into this CTA's shared memory whose completion is counted on a barrier of the pair's leader
// (`bar` is a shared::cluster address; the bytes go to the issuing CTA only)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tm), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// FUSED: tm_c is unused; tm_o0..3 are the stores of XQ, XK, XV ([B*H*T, 64] views) and of the gate buffer.
// PAIR: launched as clusters of two CTAs (see the head of the file); tm_b then has a box of 128 rows.
template <bool FUSED, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    ttt_gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                            const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_o0,
                            const __grid_constant__ CUtensorMap tm_o1, const __grid_constant__ CUtensorMap tm_o2,
                            const __grid_constant__ CUtensorMap tm_o3, const GemmParams p) {
  using SM = GemmSmem<FUSED, PAIR>;
  constexpr int GEMM_STAGES = SM::STAGES;
  constexpr uint32_t STAGE_BYTES = SM::STAGE_BYTES;
  constexpr int TILE_M = PAIR ? 2 * GEMM_BM : GEMM_BM;  // rows of C per tile (128 per CTA)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw_u32);
  const uint32_t bar_full = base + SM::OFF_BAR, bar_empty = bar_full + 8 * GEMM_STAGES,
                 bar_acc_full = bar_empty + 8 * GEMM_STAGES, bar_acc_empty = bar_acc_full + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + SM::OFF_TMEM);
  __shared__ int s_fail;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // 0 = the CTA that issues the pair's products
  const int KB = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int tiles_n = (p.N + GEMM_BN - 1) / GEMM_BN, tiles_m = (p.M + TILE_M - 1) / TILE_M;
  const int ntiles = tiles_n * tiles_m;
  // this CTA's (pair's) tiles: first, stride
  const int tile0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tstep = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  // columns a tile really has, rounded up to the instruction's granule (the last tile column is narrower); in the
  // pair form each CTA supplies half of them, so the granule is 32
  auto n_eff_of = [&](int tile) {
    const int n_left = p.N - (tile % tiles_n) * GEMM_BN;
    return n_left >= GEMM_BN ? GEMM_BN : (PAIR ? ((n_left + 31) & ~31) : ((n_left + 15) & ~15));
  };

  if (tid == 0) {
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_b);
    if (FUSED) {
      prefetch_tmap(&tm_o0);
      prefetch_tmap(&tm_o1);
      prefetch_tmap(&tm_o2);
      prefetch_tmap(&tm_o3);
    } else {
      prefetch_tmap(&tm_c);
    }
    for (int i = 0; i < SM::NBAR; ++i) {
      // one arrival per phase, except (pair form) `acc_empty`: an accumulator is free when the epilogues of both CTAs
      // have arrived, the peer's from the other CTA
      const uint32_t b = bar_full + 8 * i;
      mbar_init(b, (PAIR && (b == bar_acc_empty || b == bar_acc_empty + 8)) ? 2 : 1);
    }
    fence_mbar_init();
    s_fail = 0;
  }
  if (warp == 1) {  // tensor memory: two accumulators of 256 float32 columns (the same warp frees them at the end)
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(base + SM::OFF_TMEM)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(base + SM::OFF_TMEM)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // both CTAs' barriers are initialised and both hold their tensor memory
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer: one ring over all the tiles of this CTA
    if (lane == 0) {
      uint32_t it = 0;  // k-blocks issued so far
      bool ok = true;
      const uint32_t leader_full = PAIR ? mapa_rank(bar_full, 0) : bar_full;
      for (int tile = tile0; tile < ntiles && ok; tile += tstep) {
        const int m0 = (tile / tiles_n) * TILE_M + GEMM_BM * (int)rank;
        // rows of B: all of the tile's, or this CTA's half of the columns the products will use
        const int n0 = (tile % tiles_n) * GEMM_BN + (PAIR ? (int)rank * (n_eff_of(tile) >> 1) : 0);
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t st = it % GEMM_STAGES;
          if (it >= GEMM_STAGES) {
            if (!(PAIR && rank == 1 ? mbar_wait_bounded_cluster(bar_empty + 8 * st, ((it / GEMM_STAGES) - 1) & 1)
                                    : mbar_wait_bounded(bar_empty + 8 * st, ((it / GEMM_STAGES) - 1) & 1))) {
              s_fail = 1;
              report_timeout(p.status, 31, kb);
              ok = false;
              break;
            }
          }
          if constexpr (PAIR) {
            // both CTAs' loads complete on the leader's barrier, which expects the bytes of both
            if (rank == 0) mbar_expect_tx(bar_full + 8 * st, 2 * STAGE_BYTES);
            tma_load_2d_pair(base + st * STAGE_BYTES, &tm_a, kb * GEMM_BK, m0, leader_full + 8 * st);
            tma_load_2d_pair(base + st * STAGE_BYTES + GEMM_A_BYTES, &tm_b, kb * GEMM_BK, n0, leader_full + 8 * st);
          } else {
            mbar_expect_tx(bar_full + 8 * st, STAGE_BYTES);  // (rows beyond M / N arrive as zeros and count)
            tma_load_2d(base + st * STAGE_BYTES, &tm_a, kb * GEMM_BK, m0, bar_full + 8 * st);
            tma_load_2d(base + st * STAGE_BYTES + GEMM_A_BYTES, &tm_b, kb * GEMM_BK, n0, bar_full + 8 * st);
          }
        }
      }
      if (PAIR && ok) {
        // the last hand-backs of the stages (the peer's arrive from the other CTA) must land before this CTA leaves
        const uint32_t last = it < (uint32_t)GEMM_STAGES ? it : (uint32_t)GEMM_STAGES;
        for (uint32_t j = 0; j < last; ++j) {
          const uint32_t i2 = it - 1 - j;  // the last k-block issued into stage i2 % GEMM_STAGES
          if (!(rank == 1 ? mbar_wait_bounded_cluster(bar_empty + 8 * (i2 % GEMM_STAGES), (i2 / GEMM_STAGES) & 1)
                          : mbar_wait_bounded(bar_empty + 8 * (i2 % GEMM_STAGES), (i2 / GEMM_STAGES) & 1))) {
            s_fail = 1;
            report_timeout(p.status, 35, j);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (the leader of a pair); the peer only reports its stages
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, tl = 0;  // k-blocks consumed, tiles started
      const uint32_t peer_empty = PAIR ? mapa_rank(bar_empty, 1) : 0u, peer_acc_full = PAIR ? mapa_rank(bar_acc_full, 1) : 0u;
      bool ok = true;
      for (int tile = tile0; tile < ntiles && ok; tile += tstep, ++tl) {
        const uint32_t buf = tl & 1;
        const uint32_t idesc = umma_idesc_bf16(TILE_M, n_eff_of(tile));
        // the epilogue(s) must have drained this accumulator (its previous use was two tiles ago)
        if (tl >= 2 && !(PAIR ? mbar_wait_bounded_cluster(bar_acc_empty + 8 * buf, ((tl >> 1) - 1) & 1)
                              : mbar_wait_bounded(bar_acc_empty + 8 * buf, ((tl >> 1) - 1) & 1))) {
          s_fail = 1;
          report_timeout(p.status, 34, tl);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t st = it % GEMM_STAGES;
          if (!(PAIR ? mbar_wait_bounded_cluster(bar_full + 8 * st, (it / GEMM_STAGES) & 1)
                     : mbar_wait_bounded(bar_full + 8 * st, (it / GEMM_STAGES) & 1))) {
            s_fail = 1;
            report_timeout(p.status, 32, kb);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = base + st * STAGE_BYTES, b_addr = a_addr + GEMM_A_BYTES;
#pragma unroll
          for (int ks = 0; ks < GEMM_BK / 16; ++ks) {  // 32 bytes per k-step inside the swizzled 128-byte rows
            if constexpr (PAIR)
              umma2_bf16(tmem + buf * GEMM_BN, umma_desc_sw128(a_addr + 32 * ks), umma_desc_sw128(b_addr + 32 * ks),
                         idesc, (kb | ks) != 0 ? 1u : 0u);
            else
              umma_bf16(tmem + buf * GEMM_BN, umma_desc_sw128(a_addr + 32 * ks), umma_desc_sw128(b_addr + 32 * ks),
                        idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          // the stage is free once these products have read it (in both CTAs)
          if constexpr (PAIR) {
            umma2_commit(bar_empty + 8 * st);
            umma2_commit(peer_empty + 8 * st);
          } else {
            umma_commit(bar_empty + 8 * st);
          }
        }
        if (!ok) break;
        // arrives when every product of this tile is complete
        if constexpr (PAIR) {
          umma2_commit(bar_acc_full + 8 * buf);
          umma2_commit(peer_acc_full + 8 * buf);
        } else {
          umma_commit(bar_acc_full + 8 * buf);
        }
      }
      if (PAIR && ok) {
        // the peer's last accumulator releases arrive from the other CTA: let them land before this CTA leaves
        for (uint32_t j = 0; j < 2 && j < tl; ++j) {
          const uint32_t t2 = tl - 1 - j;
          if (!mbar_wait_bounded_cluster(bar_acc_empty + 8 * (t2 & 1), (t2 >> 1) & 1)) {
            s_fail = 1;
            report_timeout(p.status, 36, t2);
            break;
          }
        }
      }
    }
  } else {
    // ---------------- epilogue: 4 warps, warp w reads the tensor-memory lanes of quarter w % 4
    const int q = warp & 3;
    const int row = 32 * q + lane;
    const float2* rope_tab = reinterpret_cast<const float2*>(gbase + SM::OFF_ROPE);
    if (FUSED && p.f.rope_mode == 1) {
      // (cos, sin) of position x pair, positions taken modulo the mini-batch length (at most 16 here)
      const float log2_theta = log2f(p.f.rope_theta);
      float2* tab = reinterpret_cast<float2*>(gbase + SM::OFF_ROPE);
      for (int e = tid - 64; e < p.f.pos_mod * 32; e += 128) {
        const int ps = e >> 5, i = e & 31;
        float sn, cs;
        sincosf(ps * exp2f(-(2.f * i / 64.f) * log2_theta), &sn, &cs);
        tab[ps * SM::ROPE_ROW + i] = make_float2(cs, sn);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    uint32_t tl = 0;
    // where this CTA reports an accumulator drained: its own barrier, or the pair leader's
    const uint32_t acc_empty_at = PAIR ? mapa_rank(bar_acc_empty, 0) : bar_acc_empty;
    for (int tile = tile0; tile < ntiles; tile += tstep, ++tl) {
      const int m0 = (tile / tiles_n) * TILE_M + GEMM_BM * (int)rank, n0 = (tile % tiles_n) * GEMM_BN;
      const uint32_t buf = tl & 1;
      // fused: what each 64-column group of this tile is (0 q, 1 k, 2 v, 3 gate, 4 learning-rate logits, -1 nothing)
      // (packed into two words, 8 bits per group, so that the group loop can index them without a local array)
      uint32_t kind_w = 0, head_w = 0;
      int pos = 0, tok = 0, bat = 0;
      if (FUSED) {
        const int C = p.f.H * 64;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col0 = n0 + 64 * j;
          int kd = -1, hd = 0;
          if (col0 >= p.f.q_col && col0 < p.f.q_col + C) {
            kd = 0; hd = (col0 - p.f.q_col) >> 6;
          } else if (col0 >= p.f.k_col && col0 < p.f.k_col + C) {
            kd = 1; hd = (col0 - p.f.k_col) >> 6;
          } else if (col0 >= p.f.v_col && col0 < p.f.v_col + C) {
            kd = 2; hd = (col0 - p.f.v_col) >> 6;
          } else if (p.f.g_col >= 0 && col0 >= p.f.g_col && col0 < p.f.g_col + C) {
            kd = 3; hd = (col0 - p.f.g_col) >> 6;
          } else if (col0 == p.f.lr_col) {
            kd = 4;
          }
          kind_w |= (uint32_t)(kd + 1) << (8 * j);
          head_w |= (uint32_t)hd << (8 * j);
        }
        tok = (m0 + row) % p.f.T;
        bat = (m0 + row) / p.f.T;
        pos = (p.f.start_idx + tok) % p.f.pos_mod;
      }
      bool ok = mbar_wait_bounded(bar_acc_full + 8 * buf, (tl >> 1) & 1);
      if (!ok) {
        s_fail = 1;
        if (lane == 0) report_timeout(p.status, 33, tl);
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      {
        // barrier of the four epilogue warps that also agrees on failure: every thread leaves with the same verdict
        const uint32_t mine = (!ok || s_fail != 0) ? 1u : 0u;
        uint32_t any;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(any)
            : "r"(mine)
            : "memory");
        ok = (any == 0);
      }
      const int t0 = FUSED ? m0 % p.f.T : 0, b0 = FUSED ? m0 / p.f.T : 0;
#pragma unroll 1
      for (int j = 0; j < 4; ++j) {  // 64 columns at a time through one of the two staging tiles
        const int kd = (int)((kind_w >> (8 * j)) & 0xff) - 1, hd = (int)((head_w >> (8 * j)) & 0xff);
        const bool live = ok && n0 + 64 * j < p.N && (!FUSED || kd >= 0);
        const uint32_t stg = base + SM::OFF_STG + (j & 1) * GEMM_STG_BYTES;
        // the store issued two groups ago must have read this staging tile before it is overwritten
        if (warp == 2 && lane == 0) bulk_wait_read<1>();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (live) {
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            const int c = 2 * j + hc;  // 32-column slice of the accumulator
            uint32_t r[32];
            tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + buf * GEMM_BN + 32 * c, r);
            if (FUSED) {
              if (kd == 4) {
                // learning-rate logits: column i of this group is head i
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  const int h = 32 * hc + i;
                  if (h < p.f.H && m0 + row < p.M) {
                    float z = __uint_as_float(r[i]);
                    if (p.f.lr_bias != nullptr) z += __bfloat162float(static_cast<const __nv_bfloat16*>(p.f.lr_bias)[h]);
                    static_cast<__nv_bfloat16*>(p.f.lr_out)[((size_t)bat * p.f.H + h) * p.f.T + tok] =
                        __float2bfloat16_rn(p.f.base_lr * (1.f / 64.f) / (1.f + expf(-z)));
                  }
                }
                continue;
              }
              if (kd <= 1 && p.f.rope_mode == 1) {
                const float2* cs = rope_tab + pos * SM::ROPE_ROW + 16 * hc;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  // (x0, x1) -> (x0 c - x1 s, x1 c + x0 s) as two packed float32x2 operations
                  const F2 x = f2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                  const float2 w = cs[i];
                  const F2 y = f2fma(f2(-x.y, x.x), f2(w.y), f2mul(x, f2(w.x)));
                  r[2 * i] = __float_as_uint(y.x);
                  r[2 * i + 1] = __float_as_uint(y.y);
                }
              }
            }
            // staging: [128 rows][64 columns] bf16 in the swizzled layout the TMA store expects
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int chunk = hc * 4 + i;  // 16-byte chunk of the 128-byte row
              const uint32_t v0 = pack_bf16(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
              const uint32_t v1 = pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
              const uint32_t v2 = pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
              const uint32_t v3 = pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
              asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(stg + row * 128 + ((chunk ^ (row & 7)) << 4)),
                           "r"(v0), "r"(v1), "r"(v2), "r"(v3)
                           : "memory");
            }
          }
          fence_proxy_async_smem();
        }
        if (j == 3) asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          // after the last group every tcgen05.ld of this accumulator has completed (wait::ld): hand it back
          if (j == 3) {
            if constexpr (PAIR) mbar_arrive_cluster(acc_empty_at + 8 * buf);
            else mbar_arrive(bar_acc_empty + 8 * buf);
          }
          if (live && !(FUSED && kd == 4)) {
            if (FUSED) {
              const int y = (b0 * p.f.H + hd) * p.f.T + t0;  // first of 128 consecutive rows of [B*H*T, 64]
              if (kd == 0) tma_store_2d(&tm_o0, 0, y, stg);
              if (kd == 1) tma_store_2d(&tm_o1, 0, y, stg);
              if (kd == 2) tma_store_2d(&tm_o2, 0, y, stg);
              if (kd == 3) tma_store_2d(&tm_o3, 64 * hd, m0, stg);
            } else {
              tma_store_2d(&tm_c, n0 + 64 * j, m0, stg);
            }
          }
          bulk_commit();  // (an empty group when nothing was stored: keeps the two-buffer count in step)
        }
      }
      if (!ok) break;
    }
    if (warp == 2 && lane == 0) bulk_wait_read<0>();  // the staging tiles must outlive the last stores' reads
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (PAIR) {
    cluster_sync_all();  // neither CTA releases tensor memory or leaves while the other may still use the pair's
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
  } else {
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
  }
}

template <bool FUSED>
static cudaError_t launch_gemm_t(const CUtensorMap* m, const GemmParams& p, cudaStream_t st) {
  using SM = GemmSmem<FUSED, false>;
  auto kfn = ttt_gemm_bf16_tn_kernel<FUSED, false>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::DYN_BYTES);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  const long ntiles = (long)((p.N + GEMM_BN - 1) / GEMM_BN) * ((p.M + GEMM_BM - 1) / GEMM_BM);
  const int grid = (int)(ntiles < sms ? ntiles : sms);  // persistent: one CTA per SM walks the tiles
  kfn<<<grid, GEMM_THREADS, SM::DYN_BYTES, st>>>(m[0], m[1], m[2], m[3], m[4], m[5], m[6], p);
  return cudaGetLastError();
}

// pair form: clusters of two CTAs, as many as can be resident (a cluster waits on nothing outside itself)
template <bool FUSED>
static cudaError_t launch_gemm_pair_t(const CUtensorMap* m, const GemmParams& p, cudaStream_t st) {
  using SM = GemmSmem<FUSED, true>;
  auto kfn = ttt_gemm_bf16_tn_kernel<FUSED, true>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::DYN_BYTES);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = SM::DYN_BYTES;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(2 * (sms / 2));
  int nclusters = 0;
  if ((e = cudaOccupancyMaxActiveClusters(&nclusters, kfn, &cfg)) != cudaSuccess) return e;
  if (nclusters < 1) return cudaErrorLaunchOutOfResources;
  const long ntiles = (long)((p.N + GEMM_BN - 1) / GEMM_BN) * ((p.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM));
  if (nclusters > sms / 2) nclusters = sms / 2;
  if (nclusters > ntiles) nclusters = (int)ntiles;
  cfg.gridDim = dim3(2 * nclusters);
  return cudaLaunchKernelEx(&cfg, kfn, m[0], m[1], m[2], m[3], m[4], m[5], m[6], p);
}

// maps: A, B, C (plain) or A, B, -, XQ, XK, XV, gate (fused: p.f filled in).  pair: the cluster form, whose B map has
// a box of 128 rows.
cudaError_t launch_gemm_bf16_tn(const CUtensorMap* maps, const GemmParams& p, bool fused, bool pair, cudaStream_t st) {
  if (pair) return fused ? launch_gemm_pair_t<true>(maps, p, st) : launch_gemm_pair_t<false>(maps, p, st);
  return fused ? launch_gemm_t<true>(maps, p, st) : launch_gemm_t<false>(maps, p, st);
}

}  // namespace ttt
