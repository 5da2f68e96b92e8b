// Latency of ONE dependent tensor-core step, measured two ways on sm_100a (stand-alone program, prints one JSON line).
//
// The fused TTT inner loop is a chain: every 16-token stage needs the state the previous stage produced, and inside
// a stage the products feed one another through element-wise math (K.W -> LayerNorm gradient -> state update).  What
// bounds such a chain is the round trip "issue product -> result in registers -> next operand ready", not tensor
// throughput.  This program times that round trip
//   (a) on the 5th-generation path: tcgen05.mma (operands by shared-memory descriptor, accumulator in tensor
//       memory) -> tcgen05.commit -> mbarrier wait -> tcgen05.ld into registers [-> convert to bf16, write the next
//       B operand to shared memory, fence.proxy.async, CTA barrier], for the transposed products a 16-token stage
//       would use (M = 64 or 128 state rows, N = 16 tokens, K = 64 in four k-steps) and for the rank-16 state update
//       (M = 64, N = 64, K = 16);
//   (b) on the warp-level path the kernels use: four dependent mma.sync.m16n8k16 k-steps whose accumulator is
//       packed to bf16 and fed back as the next A operand through registers [or through shared memory + ldmatrix].
//   (c) tensor memory used as a per-thread scratchpad, with no tcgen05.mma at all: tcgen05.ld of a thread's own 32
//       columns, an update (an add, or eight mma.sync accumulations), tcgen05.st back -- what a read-modify-write of
//       float32 state that does not fit the register budget costs there (the TTT-MLP backward keeps its float32
//       masters this way), alone and with three blocks per SM.
// Cycles per step come from clock64 over CHAIN dependent steps.  The first tcgen05 step is checked against a host
// product so that a mis-encoded descriptor cannot pass as a fast result.
//
// Every wait is bounded; on a timeout the kernel frees its tensor memory and reports instead of hanging.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

namespace {

constexpr int CHAIN = 128;
constexpr uint32_t SPIN = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major operand tile [rows][64] bf16, 128-byte rows, 128-byte swizzle (what a TMA load with SWIZZLE_128B leaves):
// 16-byte chunk c of row r sits at chunk (c ^ (r & 7)).
__host__ __device__ inline uint32_t off_sw128(int row, int col) {
  return (uint32_t)(row * 128 + ((((col >> 3) ^ row) & 7) << 4) + ((col & 7) << 1));
}
// MN-major operand without swizzle ("interleaved" core matrices of 8 k-rows x 8 n, 16 bytes per k-row):
// element (n, k) at (k % 8) * 16 + (n % 8) * 2 + (n / 8) * SBO + (k / 8) * LBO, with SBO = 128, LBO = 128 * (N / 8).
__host__ __device__ inline uint32_t off_mn(int n, int k, int N) {
  return (uint32_t)((k & 7) * 16 + (n & 7) * 2 + (n >> 3) * 128 + (k >> 3) * 128 * (N >> 3));
}

// shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets (all >> 4),
// version 1, layout type in bits 61..63 (0 = no swizzle, 2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)((lbo >> 4) & 0x3fff) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3fff) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}
// instruction descriptor, kind::f16: D = f32, A = B = bf16, A K-major, B K- or MN-major, N >> 3 at bit 17, M >> 4 at 24
__host__ __device__ inline uint32_t make_idesc(int M, int N, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < SPIN; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

struct Result {
  unsigned long long cycles;  // for CHAIN steps
  unsigned int error;         // 0 ok, 1 a wait ran out
  float first[16];            // row 1 of D after the first step (checked on the host)
};

// One CTA of 128 threads.  A: [M][64] K-major, 128-byte swizzle (the state, fixed).  B: N = 16 tokens x K = 64,
// MN-major without swizzle (rewritten every step from the result when WRITE_BACK).  D: [M][N] float32 in tensor memory.
// MODE 0: products M x 16 x 64 (four k-steps).  MODE 1: one product M x 64 x 16 (the rank-16 update shape).
template <int M, int MODE, bool WRITE_BACK>
__global__ void __launch_bounds__(128, 1) tc5_chain(Result* out) {
  constexpr int N = MODE == 0 ? 16 : 64;
  constexpr int KSTEPS = MODE == 0 ? 4 : 1;
  __shared__ __align__(1024) uint8_t sA[128 * 128];
  __shared__ __align__(1024) uint8_t sB[64 * 64 * 2];
  __shared__ __align__(8) uint64_t bar_mem;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_fail;
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t bar = smem_u32(&bar_mem);

  // A[m][k] = 1/8 on a band (m % 64 == k) plus a small ramp; B[n][k] = (n + 1) * (k % 5 - 2) / 64
  for (int i = tid; i < M * 64; i += 128) {
    const int m = i / 64, k = i % 64;
    const float v = ((m % 64) == k ? 0.125f : 0.f) + 0.001f * (float)((m + 2 * k) % 7 - 3);
    *reinterpret_cast<__nv_bfloat16*>(sA + off_sw128(m, k)) = __float2bfloat16_rn(v);
  }
  const int KB = MODE == 0 ? 64 : 16;
  for (int i = tid; i < N * KB; i += 128) {
    const int n = i / KB, k = i % KB;
    const float v = (float)(n % 16 + 1) * (float)(k % 5 - 2) * (1.f / 64.f);
    *reinterpret_cast<__nv_bfloat16*>(sB + off_mn(n, k, N)) = __float2bfloat16_rn(v);
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_fail = 0;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 64;" ::"r"(smem_u32(&tmem_base_s))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;
  const uint32_t idesc = make_idesc(M, N, 1);
  const uint32_t a_addr = smem_u32(sA), b_addr = smem_u32(sB);
  // this warp's quarter of the tensor-memory lanes; with M = 64 rows m sit in lanes (m % 16) + 32 * (m / 16)
  const uint32_t my_taddr = tmem + ((uint32_t)(32 * warp) << 16);

  bool failed = false;
  unsigned long long t0 = 0, t1 = 0;
  for (int it = 0; it < CHAIN + 1 && !failed; ++it) {
    if (it == 1) t0 = clock64();  // step 0 is the checked warm-up
    if (tid == 0) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        // A: advance 32 bytes per k-step inside the swizzled 128-byte rows; 8-row groups are 1024 bytes apart
        const uint64_t ad = make_desc(a_addr + 32 * ks, 16, 1024, 2);
        // B (MN-major, no swizzle): a k-step of 16 = two core-matrix rows of k, LBO apart
        const uint64_t bd = make_desc(b_addr + ks * 2 * 128 * (N >> 3), 128 * (N >> 3), 128, 0);
        mma_ss(tmem, ad, bd, idesc, ks > 0 ? 1u : 0u);
      }
      commit(bar);
    }
    int bad = wait_bar(bar, (uint32_t)(it & 1)) ? 0 : 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t r[16];
    ld16(my_taddr, r);
    if (it == 0 && tid == 1) {
      for (int i = 0; i < 16; ++i) out->first[i] = __uint_as_float(r[i]);
    }
    if (WRITE_BACK) {
      // next B operand from this result: thread (row k) writes B[n = 0..15][k] = D[k][n] / 4, bf16, two 16-byte stores
      const int m = (M == 128) ? tid : ((tid & 15) + 16 * warp);
      const bool owner = (M == 128) ? (tid < KB) : ((tid & 31) < 16 && m < KB);
      if (owner) {
        uint32_t v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          v[i] = pack_bf16(0.25f * __uint_as_float(r[2 * i]), 0.25f * __uint_as_float(r[2 * i + 1]));
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(b_addr + off_mn(0, m, N)), "r"(v[0]), "r"(v[1]),
                     "r"(v[2]), "r"(v[3])
                     : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(b_addr + off_mn(8, m, N)), "r"(v[4]), "r"(v[5]),
                     "r"(v[6]), "r"(v[7])
                     : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    bad = __syncthreads_or(bad);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (bad) failed = true;
  }
  t1 = clock64();
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 64;" ::"r"(tmem) : "memory");
  if (tid == 0) {
    out->cycles = t1 - t0;
    out->error = failed ? 1u : 0u;
  }
}

// Warp-level path: one warp, four dependent k-steps per step; the accumulator (16 x 8) is packed to bf16 and becomes
// part of the next step's A fragments.  THROUGH_SMEM routes the repacked operand through shared memory + ldmatrix.
template <bool THROUGH_SMEM>
__global__ void __launch_bounds__(32, 1) mma_sync_chain(Result* out) {
  __shared__ __align__(16) uint32_t tile[16 * 8];
  const int lane = threadIdx.x;
  uint32_t a[4] = {0x3c003c00u + lane, 0x3c003c01u, 0x3c003c02u + lane, 0x3c003c03u};
  const uint32_t b0 = 0x3a003a00u, b1 = 0x3a003b00u;
  unsigned long long t0 = 0;
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  for (int it = 0; it < CHAIN + 1; ++it) {
    if (it == 1) t0 = clock64();
    c[0] = c[1] = c[2] = c[3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                   : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                   : "r"(a[0] + ks), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    const uint32_t p0 = pack_bf16(c[0] * 0.01f, c[1] * 0.01f), p1 = pack_bf16(c[2] * 0.01f, c[3] * 0.01f);
    if (THROUGH_SMEM) {
      tile[lane] = p0;
      tile[32 + lane] = p1;
      __syncwarp();
      uint32_t r[4];
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                   : "r"(smem_u32(tile) + (lane & 15) * 16 + (lane >> 4) * 256));
      a[0] = r[0]; a[1] = r[1]; a[2] = r[2]; a[3] = r[3];
      __syncwarp();
    } else {
      a[0] = p0;
      a[1] = p1;
    }
  }
  const unsigned long long t1 = clock64();
  if (lane == 0) {
    out->cycles = t1 - t0;
    out->error = 0;
    out->first[0] = c[0];
  }
}

// Tensor memory as a per-thread scratchpad (no tcgen05.mma involved): a warp addresses the 32 lanes of its quarter, so
// with the 32x32b shape N columns are N private 32-bit words of a thread.  One step = load 32 columns, update them,
// store them back (a read-modify-write of float32 state that does not fit the register budget); MODE 1 updates them
// with eight mma.sync accumulations (the rank-16 state update of the TTT-MLP backward), MODE 2 is those eight
// mma.sync alone, for the difference.  Run with one block and with several blocks per SM (grid > 1).
#define TTT_L32 "%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31"
#define TTT_O8(r, b) "=f"(r[b]), "=f"(r[b + 1]), "=f"(r[b + 2]), "=f"(r[b + 3]), "=f"(r[b + 4]), "=f"(r[b + 5]), "=f"(r[b + 6]), "=f"(r[b + 7])
#define TTT_I8(r, b) "f"(r[b]), "f"(r[b + 1]), "f"(r[b + 2]), "f"(r[b + 3]), "f"(r[b + 4]), "f"(r[b + 5]), "f"(r[b + 6]), "f"(r[b + 7])
template <int MODE>
__global__ void __launch_bounds__(128) tmem_scratch(Result* out) {
  __shared__ uint32_t s_tmem;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 64;" ::"r"(smem_u32(&s_tmem)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t ta = s_tmem + ((32u * (uint32_t)warp) << 16);
  float r[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = (float)(threadIdx.x + i);
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {" TTT_L32 "};\n\ttcgen05.wait::st.sync.aligned;"
               ::TTT_I8(r, 0), TTT_I8(r, 8), TTT_I8(r, 16), TTT_I8(r, 24), "r"(ta) : "memory");
  __syncthreads();
  unsigned long long t0 = 0;
  for (int it = 0; it < CHAIN + 1; ++it) {
    if (it == 1) t0 = clock64();
    if (MODE != 2)
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {" TTT_L32 "}, [%32];\n\ttcgen05.wait::ld.sync.aligned;"
                   : TTT_O8(r, 0), TTT_O8(r, 8), TTT_O8(r, 16), TTT_O8(r, 24) : "r"(ta) : "memory");
    if (MODE == 0) {
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] += 1.f;
    } else {
      const uint32_t a0 = 0x3c003c00u + it, b0 = 0x3a003a00u;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(r[4 * u]), "+f"(r[4 * u + 1]), "+f"(r[4 * u + 2]), "+f"(r[4 * u + 3])
                     : "r"(a0), "r"(a0), "r"(a0), "r"(a0), "r"(b0), "r"(b0));
    }
    if (MODE != 2)
      asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {" TTT_L32 "};\n\ttcgen05.wait::st.sync.aligned;"
                   ::TTT_I8(r, 0), TTT_I8(r, 8), TTT_I8(r, 16), TTT_I8(r, 24), "r"(ta) : "memory");
  }
  const unsigned long long t1 = clock64();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    out->cycles = t1 - t0;
    out->error = 0;
    out->first[0] = r[0];
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 64;" ::"r"(s_tmem) : "memory");
}

template <typename K>
Result run(K kernel, int threads, int grid = 1) {
  Result* d;
  Result h{};
  cudaMalloc(&d, sizeof(Result));
  cudaMemset(d, 0, sizeof(Result));
  kernel<<<grid, threads>>>(d);
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    fprintf(stderr, "kernel failed: %s\n", cudaGetErrorString(e));
    exit(2);
  }
  cudaMemcpy(&h, d, sizeof(Result), cudaMemcpyDeviceToHost);
  cudaFree(d);
  return h;
}

float bf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// expected row 1 of D after the first step of MODE 0: D[m][n] = sum_k A[m][k] B[n][k]
double first_step_error(const Result& r) {
  double worst = 0;
  for (int n = 0; n < 16; ++n) {
    double acc = 0;
    for (int k = 0; k < 64; ++k) {
      const float a = bf((1 == k ? 0.125f : 0.f) + 0.001f * (float)((1 + 2 * k) % 7 - 3));
      const float b = bf((float)(n + 1) * (float)(k % 5 - 2) * (1.f / 64.f));
      acc += (double)a * b;
    }
    worst = fmax(worst, fabs(acc - r.first[n]));
  }
  return worst;
}

}  // namespace

int main() {
  struct Row {
    const char* name;
    Result r;
    bool checked;
  };
  std::vector<Row> rows;
  rows.push_back({"tcgen05 M=128 N=16 K=64: mma x4 -> commit -> mbarrier -> tcgen05.ld", run(tc5_chain<128, 0, false>, 128), true});
  rows.push_back({"tcgen05 M=128 N=16 K=64: ... -> cvt, st.shared next operand, fence.proxy.async, barrier", run(tc5_chain<128, 0, true>, 128), true});
  rows.push_back({"tcgen05 M=64 N=16 K=64: mma x4 -> commit -> mbarrier -> tcgen05.ld", run(tc5_chain<64, 0, false>, 128), true});
  rows.push_back({"tcgen05 M=64 N=16 K=64: ... -> cvt, st.shared next operand, fence.proxy.async, barrier", run(tc5_chain<64, 0, true>, 128), true});
  rows.push_back({"tcgen05 M=64 N=64 K=16 (state update shape): mma -> commit -> mbarrier -> tcgen05.ld", run(tc5_chain<64, 1, false>, 128), false});
  rows.push_back({"mma.sync m16n8k16 x4 dependent k-steps -> cvt -> next A fragment in registers", run(mma_sync_chain<false>, 32), false});
  rows.push_back({"mma.sync m16n8k16 x4 dependent k-steps -> cvt -> st.shared -> ldmatrix -> next A fragment", run(mma_sync_chain<true>, 32), false});
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  rows.push_back({"tensor-memory scratchpad: tcgen05.ld 32 columns -> add -> tcgen05.st (one block)", run(tmem_scratch<0>, 128), false});
  rows.push_back({"8 x mma.sync m16n8k16 into 32 accumulator registers (one block)", run(tmem_scratch<2>, 128), false});
  rows.push_back({"tcgen05.ld 32 columns -> 8 x mma.sync into them -> tcgen05.st (one block)", run(tmem_scratch<1>, 128), false});
  rows.push_back({"8 x mma.sync m16n8k16 into 32 accumulator registers (3 blocks per SM)", run(tmem_scratch<2>, 128, 3 * sms), false});
  rows.push_back({"tcgen05.ld 32 columns -> 8 x mma.sync into them -> tcgen05.st (3 blocks per SM)", run(tmem_scratch<1>, 128, 3 * sms), false});
  printf("{\"chain_steps\": %d, \"rows\": [", CHAIN);
  for (size_t i = 0; i < rows.size(); ++i) {
    const Row& w = rows[i];
    printf("%s{\"what\": \"%s\", \"cycles_per_step\": %.1f, \"timed_out\": %s", i ? ", " : "", w.name,
           (double)w.r.cycles / CHAIN, w.r.error ? "true" : "false");
    if (w.checked) printf(", \"first_step_max_abs_error\": %.3g", first_step_error(w.r));
    printf("}");
  }
  printf("]}\n");
  return 0;
}
