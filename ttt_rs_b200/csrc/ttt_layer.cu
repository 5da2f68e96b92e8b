// The steps of the outer TTT layer on either side of the inner loop, as two bandwidth-bound kernels (sm_100a).
//
// Reference semantics: rust/layer/src/ttt.rs:152-299 (`get_qkv`, `get_lr`, `conv_qk`, `forward`), rotary embedding
// rust/core/src/util.rs:284-392 (PyTorch twin reference/ttt.py:215-270,701-915).  There the projections' outputs
// are reshaped and permuted to [B,H,T,F] (one materialised copy per tensor), rotated by separate element-wise
// kernels, the learning-rate gate is a chain of small tensor ops, and after the inner loop the result is permuted
// back and normalised by further kernels.  Here:
//   * ttt_layer_prologue_kernel reads the projection output once in its native [B*T, columns] layout and writes
//     XQ, XK, XV in the inner loop's [B,H,T,F] layout with the shared-QK causal convolutions and the rotary
//     rotation applied on the way, plus ttt_lr_eta = base_lr * sigmoid(logit + bias) / F in [B,H,T];
//   * ttt_layer_epilogue_kernel reads the inner loop's [B,H,T,F] output once and writes [B,T,H*F] with the post
//     LayerNorm and the optional gelu(tanh) gate applied.
// Every global access is a full 128-byte (bf16) or 256-byte (f32) row segment per 8 / 32 lanes; no shared-memory
// staging is needed because a (token, head) row of F = 64 or 32 features is contiguous in both layouts.
#include "ttt_kernels.h"
#include "ttt_common.cuh"

namespace ttt {

template <typename T>
struct Vec8;  // eight consecutive elements
template <>
struct Vec8<__nv_bfloat16> {
  uint4 raw;
  __device__ __forceinline__ void load(const void* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(void* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = bf16_lo(w[i]);
      f[2 * i + 1] = bf16_hi(w[i]);
    }
  }
  __device__ __forceinline__ void pack(const float (&f)[8]) {
    raw.x = pack_bf16(f[0], f[1]);
    raw.y = pack_bf16(f[2], f[3]);
    raw.z = pack_bf16(f[4], f[5]);
    raw.w = pack_bf16(f[6], f[7]);
  }
};
template <>
struct Vec8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const void* p) {
    a = reinterpret_cast<const float4*>(p)[0];
    b = reinterpret_cast<const float4*>(p)[1];
  }
  __device__ __forceinline__ void store(void* p) const {
    reinterpret_cast<float4*>(p)[0] = a;
    reinterpret_cast<float4*>(p)[1] = b;
  }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  __device__ __forceinline__ void pack(const float (&f)[8]) {
    a = make_float4(f[0], f[1], f[2], f[3]);
    b = make_float4(f[4], f[5], f[6], f[7]);
  }
};

constexpr int PRO_THREADS = 256;
constexpr int PRO_TCHUNK = 32;   // tokens per warp task
constexpr int PRO_MAXK = 4;      // causal convolution taps supported
constexpr int PRO_MAXPOS = 64;   // rotary table rows (positions modulo the mini-batch length)

// One warp task = (batch b, group of HPW heads, chunk of PRO_TCHUNK tokens), HPW = 4 heads of 64 features or 8 heads of
// 32.  Lane = SUBS*hq + sub (SUBS = F/8) handles head HPW*hgroup + hq, features [8*sub, 8*sub+8) = rotary pairs
// 4*sub .. 4*sub+3, and walks the chunk's tokens in groups of PRO_TG whose loads are all issued before any of them is
// used (memory-level parallelism).
constexpr int PRO_TG = 4;

template <typename T, bool CONV, int FD>
__global__ void __launch_bounds__(PRO_THREADS, (CONV || sizeof(T) == 4) ? 1 : 3) ttt_layer_prologue_kernel(const LayerProParams p) {
  __shared__ float2 rope_tab[PRO_MAXPOS][32];  // (cos, sin) per position and pair (the first FD/2 pairs are used)
  constexpr int F = FD, SUBS = FD / 8, HPW = 32 / SUBS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = p.H, NT = p.T;
  const bool rope = p.rope_mode != 0;
  const bool rope_wrap = p.rope_mode == 1;
  const float log2_theta = log2f(p.rope_theta);
  if (rope && rope_wrap) {
    for (int e = tid; e < p.pos_mod * 32; e += PRO_THREADS) {
      const int pos = e >> 5, i = e & 31;
      const float inv_freq = exp2f(-(2.f * i / F) * log2_theta);
      float s, c;
      sincosf(pos * inv_freq, &s, &c);
      rope_tab[pos][i] = make_float2(c, s);
    }
  }
  __syncthreads();

  const int hq = lane / SUBS, sub = lane % SUBS;
  const int hgroups = (H + HPW - 1) / HPW, tchunks = (NT + PRO_TCHUNK - 1) / PRO_TCHUNK;
  const long ntasks = (long)p.B * hgroups * tchunks;
  const int KC = p.conv_k;

  for (long task = (long)blockIdx.x * (PRO_THREADS / 32) + warp; task < ntasks; task += (long)gridDim.x * (PRO_THREADS / 32)) {
    const int tc = (int)(task % tchunks);
    const int hg = (int)((task / tchunks) % hgroups);
    const int b = (int)(task / ((long)tchunks * hgroups));
    const int h = HPW * hg + hq;
    if (h >= H) continue;
    const int col = h * F + 8 * sub;  // first of this lane's 8 columns inside a projection block
    const int t0 = tc * PRO_TCHUNK, t1 = min(NT, t0 + PRO_TCHUNK);

    // convolution taps and biases of this lane's 8 channels (loop-invariant); window slot j holds token
    // t-(PRO_MAXK-1)+j and taps are right-aligned (the last tap multiplies token t), so slots older than the kernel
    // length get zero weights
    float wq[CONV ? PRO_MAXK : 1][8], wk[CONV ? PRO_MAXK : 1][8], bq[8], bk[8];
    float hist[CONV ? PRO_MAXK - 1 : 1][8];  // the previous PRO_MAXK-1 rows of the shared projection (oldest first)
    if constexpr (CONV) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        bq[c] = ld_as_float<T>(p.conv_q_b, (size_t)(col + c));
        bk[c] = ld_as_float<T>(p.conv_k_b, (size_t)(col + c));
#pragma unroll
        for (int j = 0; j < PRO_MAXK; ++j) {
          const int wj = j - (PRO_MAXK - KC);
          wq[j][c] = (wj >= 0) ? ld_as_float<T>(p.conv_q_w, (size_t)(col + c) * KC + wj) : 0.f;
          wk[j][c] = (wj >= 0) ? ld_as_float<T>(p.conv_k_w, (size_t)(col + c) * KC + wj) : 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < PRO_MAXK - 1; ++j) {
        const int tt = t0 - (PRO_MAXK - 1) + j;
        if (tt >= 0) {
          Vec8<T> v;
          v.load(static_cast<const T*>(p.q_src) + ((size_t)b * NT + tt) * p.ld_src + col);
          v.unpack(hist[j]);
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) hist[j][c] = 0.f;
        }
      }
    }

    for (int tb = t0; tb < t1; tb += PRO_TG) {
      Vec8<T> vq[PRO_TG], vk[PRO_TG], vv[PRO_TG];
#pragma unroll
      for (int u = 0; u < PRO_TG; ++u) {
        if (tb + u < t1) {
          const size_t srow = ((size_t)b * NT + tb + u) * p.ld_src + col;
          vq[u].load(static_cast<const T*>(p.q_src) + srow);
          if constexpr (!CONV) vk[u].load(static_cast<const T*>(p.k_src) + srow);
          vv[u].load(static_cast<const T*>(p.v_src) + srow);
        }
      }
#pragma unroll
      for (int u = 0; u < PRO_TG; ++u) {
        const int t = tb + u;
        if (t < t1) {
          float fq[8], fk[8];
          if constexpr (CONV) {
            float cur[8];
            vq[u].unpack(cur);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              float aq = bq[c], ak = bk[c];
#pragma unroll
              for (int j = 0; j < PRO_MAXK - 1; ++j) {
                aq = fmaf(wq[j][c], hist[j][c], aq);
                ak = fmaf(wk[j][c], hist[j][c], ak);
              }
              fq[c] = fmaf(wq[PRO_MAXK - 1][c], cur[c], aq);
              fk[c] = fmaf(wk[PRO_MAXK - 1][c], cur[c], ak);
            }
#pragma unroll
            for (int j = 0; j < PRO_MAXK - 2; ++j)
#pragma unroll
              for (int c = 0; c < 8; ++c) hist[j][c] = hist[j + 1][c];
#pragma unroll
            for (int c = 0; c < 8; ++c) hist[PRO_MAXK - 2][c] = cur[c];
          } else {
            vq[u].unpack(fq);
            vk[u].unpack(fk);
          }
          if (rope) {
            const int pos = p.start_idx + t;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float2 cs;
              if (rope_wrap) {
                cs = rope_tab[pos % p.pos_mod][4 * sub + j];
              } else {
                const float inv_freq = exp2f(-(2.f * (4 * sub + j) / F) * log2_theta);
                sincosf(pos * inv_freq, &cs.y, &cs.x);
              }
              const float q0 = fq[2 * j], q1 = fq[2 * j + 1], k0 = fk[2 * j], k1 = fk[2 * j + 1];
              fq[2 * j] = q0 * cs.x - q1 * cs.y;
              fq[2 * j + 1] = q1 * cs.x + q0 * cs.y;
              fk[2 * j] = k0 * cs.x - k1 * cs.y;
              fk[2 * j + 1] = k1 * cs.x + k0 * cs.y;
            }
          }
          if (CONV || rope) {
            vq[u].pack(fq);
            vk[u].pack(fk);
          }
          const size_t drow = (((size_t)b * H + h) * NT + t) * F + 8 * sub;
          vq[u].store(static_cast<T*>(p.xq) + drow);
          vk[u].store(static_cast<T*>(p.xk) + drow);
          vv[u].store(static_cast<T*>(p.xv) + drow);
        }
      }
    }
  }

  // ttt_lr_eta[b,h,t] = base_lr / F * sigmoid(logit[b*T+t][h] + bias[h])
  const long nlr = (long)p.B * H * NT;
  for (long e = (long)blockIdx.x * PRO_THREADS + tid; e < nlr; e += (long)gridDim.x * PRO_THREADS) {
    const int t = (int)(e % NT);
    const int h = (int)((e / NT) % H);
    const int b = (int)(e / ((long)NT * H));
    float z = ld_as_float<T>(p.lr_logits, ((size_t)b * NT + t) * p.ld_lr + h);
    if (p.lr_bias != nullptr) z += ld_as_float<T>(p.lr_bias, (size_t)h);
    st_from_float<T>(p.lr_out, (size_t)e, p.base_lr / F / (1.f + expf(-z)));
  }
}

constexpr int EPI_THREADS = 256;


// One CTA per tile of TT consecutive tokens of one batch element.  Load phase: for every head the tile's TT rows of
// F features are one contiguous segment of the [B,H,T,F] tensor; all threads fetch the segments with 16-byte loads
// (the whole tile is in flight at once) and scatter them into a [TT][H*F] tile in shared memory.  Row phase: each
// warp takes whole rows from shared memory (three sweeps: sum, squared deviations, output), applies the norm and the
// optional gate and writes the row to [B,T,H*F] with 16-byte stores.  Several CTAs per SM overlap the two phases.
// MAXCH: 16-byte chunks of one row per lane (rows of up to 32 * MAXCH chunks = 512 * MAXCH bytes); the tile holds
// TT = 64 / MAXCH tokens, so the [TT][H*F] staging tile stays at or below 32 KB and several CTAs share an SM.
template <typename T, int MAXCH, int FD>
__global__ void __launch_bounds__(EPI_THREADS, (MAXCH <= 4 ? 4 : 2)) ttt_layer_epilogue_kernel(const LayerEpiParams p) {
  constexpr int HD = FD;  // features per head in this instantiation
  constexpr int TT = 64 / MAXCH;
  constexpr int EPC = 16 / sizeof(T);  // elements per 16-byte chunk
  constexpr int NPAIR = EPC / 2;
  constexpr int CPR = HD / EPC;        // chunks per head row
  extern __shared__ __align__(16) uint8_t epi_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = p.H, NT = p.T, C = H * HD;
  const size_t tile_bytes = (size_t)TT * C * sizeof(T);
  float* gam = reinterpret_cast<float*>(epi_smem + 2 * tile_bytes);  // two tiles (double buffer), then gamma, beta
  float* bet = gam + C;
  for (int c = tid; c < C; c += EPI_THREADS) {
    gam[c] = ld_as_float<T>(p.ln_w, (size_t)c);
    bet[c] = ld_as_float<T>(p.ln_b, (size_t)c);
  }
  const int tiles_per_b = (NT + TT - 1) / TT;
  const long ntiles = (long)p.B * tiles_per_b;
  const int nch = C / EPC;          // chunks per output row
  constexpr int seg = TT * CPR;     // chunks per head segment of a full tile (a power of two)

  // asynchronous 16-byte copies global -> shared of one tile (no register staging); one commit group per tile
  auto fetch = [&](long tile_id, int buf) {
    if (tile_id < ntiles) {
      const int b = (int)(tile_id / tiles_per_b);
      const int t0 = (int)(tile_id % tiles_per_b) * TT;
      const int rows = min(TT, NT - t0);
      const uint32_t dst0 = smem_u32(epi_smem + buf * tile_bytes);
      for (int idx = tid; idx < H * seg; idx += EPI_THREADS) {
        const int h = idx / seg, i = idx - h * seg, r = i / CPR, cc = i - r * CPR;
        if (r < rows) {
          const T* src = static_cast<const T*>(p.inner_out) + (((size_t)b * H + h) * NT + t0) * HD + (size_t)i * EPC;
          const uint32_t dst = dst0 + (uint32_t)(((size_t)r * C + h * HD + cc * EPC) * sizeof(T));
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  int buf = 0;
  fetch(blockIdx.x, 0);
  for (long tile_id = blockIdx.x; tile_id < ntiles; tile_id += gridDim.x, buf ^= 1) {
    const int b = (int)(tile_id / tiles_per_b);
    const int t0 = (int)(tile_id % tiles_per_b) * TT;
    const int rows = min(TT, NT - t0);
    fetch(tile_id + gridDim.x, buf ^ 1);  // the other buffer was released by the barrier that ended the last tile
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();  // this tile has landed for every thread (and gam / bet are written, first time round)
    const T* tile = reinterpret_cast<const T*>(epi_smem + buf * tile_bytes);
    for (int r = warp; r < rows; r += EPI_THREADS / 32) {
      const T* row = tile + (size_t)r * C;
      F2 v[MAXCH][NPAIR];
      F2 acc = f2(0.f);
#pragma unroll
      for (int j = 0; j < MAXCH; ++j) {
        const int ch = j * 32 + lane;
        if (ch < nch) {
          const uint4 raw = *reinterpret_cast<const uint4*>(row + ch * EPC);
          if constexpr (sizeof(T) == 2) {
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) v[j][k] = f2(bf16_lo(w[k]), bf16_hi(w[k]));
          } else {
            v[j][0] = f2(__uint_as_float(raw.x), __uint_as_float(raw.y));
            v[j][1] = f2(__uint_as_float(raw.z), __uint_as_float(raw.w));
          }
#pragma unroll
          for (int k = 0; k < NPAIR; ++k) acc = f2add(acc, v[j][k]);
        }
      }
      float s = f2hsum(acc);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s / C;
      acc = f2(0.f);
#pragma unroll
      for (int j = 0; j < MAXCH; ++j) {
        if (j * 32 + lane < nch) {
#pragma unroll
          for (int k = 0; k < NPAIR; ++k) {
            v[j][k] = f2sub(v[j][k], f2(mean));
            acc = f2fma(v[j][k], v[j][k], acc);
          }
        }
      }
      float q = f2hsum(acc);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
      const float rstd = 1.f / sqrtf(q / C + p.eps);
      const size_t tok = (size_t)b * NT + t0 + r;
#pragma unroll
      for (int j = 0; j < MAXCH; ++j) {
        const int ch = j * 32 + lane;
        if (ch < nch) {
          const int c0 = ch * EPC;
          float y[EPC], gq[EPC], bq[EPC];
#pragma unroll
          for (int e = 0; e < EPC; e += 4) {
            const float4 g4 = *reinterpret_cast<const float4*>(gam + c0 + e), b4 = *reinterpret_cast<const float4*>(bet + c0 + e);
            gq[e] = g4.x; gq[e + 1] = g4.y; gq[e + 2] = g4.z; gq[e + 3] = g4.w;
            bq[e] = b4.x; bq[e + 1] = b4.y; bq[e + 2] = b4.z; bq[e + 3] = b4.w;
          }
#pragma unroll
          for (int k = 0; k < NPAIR; ++k) {
            const F2 o = f2fma(v[j][k], f2mul(f2(gq[2 * k], gq[2 * k + 1]), f2(rstd)), f2(bq[2 * k], bq[2 * k + 1]));
            y[2 * k] = o.x;
            y[2 * k + 1] = o.y;
          }
          if (p.gate != nullptr) {
            float gt[EPC];
            const T* gp = static_cast<const T*>(p.gate) + tok * p.ld_gate + c0;
            if constexpr (sizeof(T) == 2) {
              // gate rows are only 8-byte aligned: two 8-byte loads
              const uint2 g0 = reinterpret_cast<const uint2*>(gp)[0], g1 = reinterpret_cast<const uint2*>(gp)[1];
              gt[0] = bf16_lo(g0.x); gt[1] = bf16_hi(g0.x); gt[2] = bf16_lo(g0.y); gt[3] = bf16_hi(g0.y);
              gt[4] = bf16_lo(g1.x); gt[5] = bf16_hi(g1.x); gt[6] = bf16_lo(g1.y); gt[7] = bf16_hi(g1.y);
            } else {
              const float2 g0 = reinterpret_cast<const float2*>(gp)[0], g1 = reinterpret_cast<const float2*>(gp)[1];
              gt[0] = g0.x; gt[1] = g0.y; gt[2] = g1.x; gt[3] = g1.y;
            }
#pragma unroll
            for (int e = 0; e < EPC; ++e) {
              // gelu, tanh form (rust/layer/src/ttt.rs:290-293; constants thundercube/src/unary_ops.rs:136-137)
              const float g = gt[e], u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
              y[e] *= 0.5f * g * (1.f + tanhf(u));
            }
          }
          T* dst = static_cast<T*>(p.y) + tok * C + c0;
          if constexpr (sizeof(T) == 2) {
            uint4 o;
            o.x = pack_bf16(y[0], y[1]); o.y = pack_bf16(y[2], y[3]); o.z = pack_bf16(y[4], y[5]); o.w = pack_bf16(y[6], y[7]);
            *reinterpret_cast<uint4*>(dst) = o;
          } else {
            *reinterpret_cast<float4*>(dst) = make_float4(y[0], y[1], y[2], y[3]);
          }
        }
      }
    }
    __syncthreads();  // every warp is done with this buffer before the next iteration refills it
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

static int sm_count() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

// grid of the two prologue kernels: one warp per (batch, group of 256 / head_dim heads, token chunk), capped
static int prologue_grid(int B, int H, int T, int head_dim) {
  const int hpw = 256 / head_dim;
  const long ntasks = (long)B * ((H + hpw - 1) / hpw) * ((T + PRO_TCHUNK - 1) / PRO_TCHUNK);
  const long want = (ntasks + PRO_THREADS / 32 - 1) / (PRO_THREADS / 32);
  const long cap = (long)sm_count() * 8;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

template <typename T, int FD>
static void launch_pro_t(const LayerProParams& p, int grid, cudaStream_t st) {
  if (p.conv_q_w != nullptr)
    ttt_layer_prologue_kernel<T, true, FD><<<grid, PRO_THREADS, 0, st>>>(p);
  else
    ttt_layer_prologue_kernel<T, false, FD><<<grid, PRO_THREADS, 0, st>>>(p);
}

cudaError_t launch_layer_prologue(int dtype, int head_dim, const LayerProParams& p, cudaStream_t st) {
  const int grid = prologue_grid(p.B, p.H, p.T, head_dim);
  if (head_dim == 32) {
    if (dtype == 1) launch_pro_t<__nv_bfloat16, 32>(p, grid, st);
    else launch_pro_t<float, 32>(p, grid, st);
  } else {
    if (dtype == 1) launch_pro_t<__nv_bfloat16, 64>(p, grid, st);
    else launch_pro_t<float, 64>(p, grid, st);
  }
  return cudaGetLastError();
}

template <typename T, int MAXCH, int FD>
static cudaError_t launch_epi_t(const LayerEpiParams& p, cudaStream_t st) {
  const int C = p.H * FD;
  constexpr int TT = 64 / MAXCH;
  const size_t smem = 2 * (size_t)TT * C * sizeof(T) + 2 * (size_t)C * sizeof(float);
  auto kfn = ttt_layer_epilogue_kernel<T, MAXCH, FD>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const long ntiles = (long)p.B * ((p.T + TT - 1) / TT);
  int per_sm = 1;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kfn, EPI_THREADS, smem);
  if (e != cudaSuccess) return e;
  const long cap = (long)sm_count() * (per_sm < 1 ? 1 : per_sm);
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  kfn<<<grid < 1 ? 1 : grid, EPI_THREADS, smem, st>>>(p);
  return cudaGetLastError();
}

template <int FD>
static cudaError_t launch_epi_f(int dtype, const LayerEpiParams& p, cudaStream_t st) {
  // chunks of one row per lane: H*F elements / (elements per 16 bytes) / 32 lanes
  const int C = p.H * FD;
  if (dtype == 1) return C <= 1024 ? launch_epi_t<__nv_bfloat16, 4, FD>(p, st) : launch_epi_t<__nv_bfloat16, 8, FD>(p, st);
  if (C <= 512) return launch_epi_t<float, 4, FD>(p, st);
  return C <= 1024 ? launch_epi_t<float, 8, FD>(p, st) : launch_epi_t<float, 16, FD>(p, st);
}

cudaError_t launch_layer_epilogue(int dtype, int head_dim, const LayerEpiParams& p, cudaStream_t st) {
  return head_dim == 32 ? launch_epi_f<32>(dtype, p, st) : launch_epi_f<64>(dtype, p, st);
}

}  // namespace ttt

// =====================================================================================================
// Backward of the two layer steps (training).  Reference: Burn autodiff over the tensor ops of
// rust/layer/src/ttt.rs:152-299; here each step's gradient is one more bandwidth-bound pass.
// =====================================================================================================
namespace ttt {

// Prologue backward (configuration without the shared-QK convolutions): gradients of XQ, XK, XV [B,H,T,F] go back
// to the projection layout [B*T, ld] with the inverse rotation applied to q and k; the gradient of ttt_lr_eta goes
// back through the sigmoid to the logits' columns (lr = c sigma(z), c = base_lr / F  =>  dz = dlr * lr * (1 - lr/c));
// padding columns after the H logit columns are zeroed.
template <typename T, int FD>
__global__ void __launch_bounds__(PRO_THREADS, sizeof(T) == 2 ? 3 : 1) ttt_layer_prologue_bwd_kernel(const LayerProBwdParams p) {
  __shared__ float2 rope_tab[PRO_MAXPOS][32];
  constexpr int F = FD, SUBS = FD / 8, HPW = 32 / SUBS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = p.H, NT = p.T;
  const bool rope = p.rope_mode != 0, rope_wrap = p.rope_mode == 1;
  const float log2_theta = log2f(p.rope_theta);
  if (rope && rope_wrap) {
    for (int e = tid; e < p.pos_mod * 32; e += PRO_THREADS) {
      const int pos = e >> 5, i = e & 31;
      float s, c;
      sincosf(pos * exp2f(-(2.f * i / F) * log2_theta), &s, &c);
      rope_tab[pos][i] = make_float2(c, s);
    }
  }
  __syncthreads();
  const int hq = lane / SUBS, sub = lane % SUBS;
  const int hgroups = (H + HPW - 1) / HPW, tchunks = (NT + PRO_TCHUNK - 1) / PRO_TCHUNK;
  const long ntasks = (long)p.B * hgroups * tchunks;
  for (long task = (long)blockIdx.x * (PRO_THREADS / 32) + warp; task < ntasks; task += (long)gridDim.x * (PRO_THREADS / 32)) {
    const int tc = (int)(task % tchunks);
    const int hg = (int)((task / tchunks) % hgroups);
    const int b = (int)(task / ((long)tchunks * hgroups));
    const int h = HPW * hg + hq;
    if (h >= H) continue;
    const int col = h * F + 8 * sub;
    const int t0 = tc * PRO_TCHUNK, t1 = min(NT, t0 + PRO_TCHUNK);
    for (int tb = t0; tb < t1; tb += PRO_TG) {
      Vec8<T> vq[PRO_TG], vk[PRO_TG], vv[PRO_TG];
#pragma unroll
      for (int u = 0; u < PRO_TG; ++u) {
        if (tb + u < t1) {
          const size_t srow = (((size_t)b * H + h) * NT + tb + u) * F + 8 * sub;
          vq[u].load(static_cast<const T*>(p.dxq) + srow);
          vk[u].load(static_cast<const T*>(p.dxk) + srow);
          vv[u].load(static_cast<const T*>(p.dxv) + srow);
        }
      }
#pragma unroll
      for (int u = 0; u < PRO_TG; ++u) {
        const int t = tb + u;
        if (t < t1) {
          if (rope) {
            float fq[8], fk[8];
            vq[u].unpack(fq);
            vk[u].unpack(fk);
            const int pos = p.start_idx + t;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float2 cs;
              if (rope_wrap) {
                cs = rope_tab[pos % p.pos_mod][4 * sub + j];
              } else {
                sincosf(pos * exp2f(-(2.f * (4 * sub + j) / F) * log2_theta), &cs.y, &cs.x);
              }
              // transpose of the forward rotation
              const float q0 = fq[2 * j], q1 = fq[2 * j + 1], k0 = fk[2 * j], k1 = fk[2 * j + 1];
              fq[2 * j] = q0 * cs.x + q1 * cs.y;
              fq[2 * j + 1] = q1 * cs.x - q0 * cs.y;
              fk[2 * j] = k0 * cs.x + k1 * cs.y;
              fk[2 * j + 1] = k1 * cs.x - k0 * cs.y;
            }
            vq[u].pack(fq);
            vk[u].pack(fk);
          }
          const size_t drow = ((size_t)b * NT + t) * p.ld_dst + col;
          vq[u].store(static_cast<T*>(p.dq_dst) + drow);
          vk[u].store(static_cast<T*>(p.dk_dst) + drow);
          vv[u].store(static_cast<T*>(p.dv_dst) + drow);
        }
      }
    }
  }
  const float inv_c = (float)F / p.base_lr;
  const long nlr = (long)p.B * NT * p.lr_cols;
  for (long e = (long)blockIdx.x * PRO_THREADS + tid; e < nlr; e += (long)gridDim.x * PRO_THREADS) {
    const int h = (int)(e % p.lr_cols);
    const long row = e / p.lr_cols;  // b * T + t
    float dz = 0.f;
    if (h < H) {
      const int t = (int)(row % NT), b = (int)(row / NT);
      const size_t i = ((size_t)b * H + h) * NT + t;
      const float lr = ld_as_float<T>(p.lr, i);
      dz = ld_as_float<T>(p.dlr, i) * lr * (1.f - lr * inv_c);
    }
    st_from_float<T>(p.dlogits_dst, (size_t)row * p.ld_dlr + h, dz);
  }
}

// Epilogue backward.  Same tiling as the forward kernel: the inner-output tile is fetched into shared memory, each
// warp takes whole rows, recomputes the row statistics, forms
//   dn = dy * gelu(g),  dg = dy * n * gelu'(g)   (n = gamma x_hat + beta; without a gate dn = dy),
//   dz = rstd * (dx - mean(dx) - x_hat * mean(dx * x_hat)),  dx = dn * gamma,
// writes dz back into the tile (then scattered to [B,H,T,F] per head segment) and leaves (mean, rstd) of every row in
// `row_stats` for the parameter-gradient kernel below.
template <typename T, int MAXCH, int FD>
__global__ void __launch_bounds__(EPI_THREADS, (MAXCH <= 4 ? 2 : 1)) ttt_layer_epilogue_bwd_kernel(const LayerEpiBwdParams p) {
  constexpr int HD = FD;  // features per head in this instantiation
  constexpr int TT = 64 / MAXCH;
  constexpr int EPC = 16 / sizeof(T);
  constexpr int CPR = HD / EPC;
  extern __shared__ __align__(16) uint8_t epi_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = p.H, NT = p.T, C = H * HD;
  const size_t tile_bytes = (size_t)TT * C * sizeof(T);
  float* gam = reinterpret_cast<float*>(epi_smem + 2 * tile_bytes);
  float* bet = gam + C;
  for (int c = tid; c < C; c += EPI_THREADS) {
    gam[c] = ld_as_float<T>(p.ln_w, (size_t)c);
    bet[c] = ld_as_float<T>(p.ln_b, (size_t)c);
  }
  const int tiles_per_b = (NT + TT - 1) / TT;
  const long ntiles = (long)p.B * tiles_per_b;
  const int nch = C / EPC;
  constexpr int seg = TT * CPR;

  auto fetch = [&](long tile_id, int buf) {
    if (tile_id < ntiles) {
      const int b = (int)(tile_id / tiles_per_b);
      const int t0 = (int)(tile_id % tiles_per_b) * TT;
      const int rows = min(TT, NT - t0);
      const uint32_t dst0 = smem_u32(epi_smem + buf * tile_bytes);
      for (int idx = tid; idx < H * seg; idx += EPI_THREADS) {
        const int h = idx / seg, i = idx - h * seg, r = i / CPR, cc = i - r * CPR;
        if (r < rows) {
          const T* src = static_cast<const T*>(p.inner_out) + (((size_t)b * H + h) * NT + t0) * HD + (size_t)i * EPC;
          const uint32_t dst = dst0 + (uint32_t)(((size_t)r * C + h * HD + cc * EPC) * sizeof(T));
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  int buf = 0;
  fetch(blockIdx.x, 0);
  for (long tile_id = blockIdx.x; tile_id < ntiles; tile_id += gridDim.x, buf ^= 1) {
    const int b = (int)(tile_id / tiles_per_b);
    const int t0 = (int)(tile_id % tiles_per_b) * TT;
    const int rows = min(TT, NT - t0);
    fetch(tile_id + gridDim.x, buf ^ 1);
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    T* tile = reinterpret_cast<T*>(epi_smem + buf * tile_bytes);
    for (int r = warp; r < rows; r += EPI_THREADS / 32) {
      T* row = tile + (size_t)r * C;
      const size_t tok = (size_t)b * NT + t0 + r;
      float v[MAXCH][EPC];
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < MAXCH; ++j) {
        const int ch = j * 32 + lane;
        if (ch < nch) {
          if constexpr (sizeof(T) == 2) {
            Vec8<T> raw;
            raw.load(row + ch * EPC);
            raw.unpack(v[j]);
          } else {
            const float4 f = *reinterpret_cast<const float4*>(row + ch * EPC);
            v[j][0] = f.x; v[j][1] = f.y; v[j][2] = f.z; v[j][3] = f.w;
          }
#pragma unroll
          for (int e = 0; e < EPC; ++e) s += v[j][e];
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s / C;
      float q = 0.f;
#pragma unroll
      for (int j = 0; j < MAXCH; ++j)
        if (j * 32 + lane < nch) {
#pragma unroll
          for (int e = 0; e < EPC; ++e) {
            v[j][e] -= mean;
            q = fmaf(v[j][e], v[j][e], q);
          }
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
      const float rstd = 1.f / sqrtf(q / C + p.eps);
      if (lane == 0) p.row_stats[tok] = make_float2(mean, rstd);
      // pass 1: x_hat, dn (and dg), dx = dn * gamma and its two row sums
      float dxv[MAXCH][EPC];
      float m1 = 0.f, m2 = 0.f;
#pragma unroll
      for (int j = 0; j < MAXCH; ++j) {
        const int ch = j * 32 + lane;
        if (ch < nch) {
          const int c0 = ch * EPC;
          float dy[EPC];
          const T* dyp = static_cast<const T*>(p.dy) + tok * C + c0;
          if constexpr (sizeof(T) == 2) {
            Vec8<T> raw;
            raw.load(dyp);
            raw.unpack(dy);
          } else {
            const float4 f = *reinterpret_cast<const float4*>(dyp);
            dy[0] = f.x; dy[1] = f.y; dy[2] = f.z; dy[3] = f.w;
          }
          float gt[EPC], dg[EPC];
          if (p.gate != nullptr) {
            const T* gp = static_cast<const T*>(p.gate) + tok * p.ld_gate + c0;
            if constexpr (sizeof(T) == 2) {
              const uint2 g0 = reinterpret_cast<const uint2*>(gp)[0], g1 = reinterpret_cast<const uint2*>(gp)[1];
              gt[0] = bf16_lo(g0.x); gt[1] = bf16_hi(g0.x); gt[2] = bf16_lo(g0.y); gt[3] = bf16_hi(g0.y);
              gt[4] = bf16_lo(g1.x); gt[5] = bf16_hi(g1.x); gt[6] = bf16_lo(g1.y); gt[7] = bf16_hi(g1.y);
            } else {
              const float2 g0 = reinterpret_cast<const float2*>(gp)[0], g1 = reinterpret_cast<const float2*>(gp)[1];
              gt[0] = g0.x; gt[1] = g0.y; gt[2] = g1.x; gt[3] = g1.y;
            }
          }
#pragma unroll
          for (int e = 0; e < EPC; ++e) {
            const float xh = v[j][e] * rstd;
            float dn = dy[e];
            if (p.gate != nullptr) {
              const float g = gt[e], g2 = g * g;
              const float u = 0.7978845608028654f * (g + 0.044715f * g * g2);
              const float th = tanhf(u);
              const float gelu = 0.5f * g * (1.f + th);
              const float dgelu = 0.5f * (1.f + th) + 0.5f * g * (1.f - th * th) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * g2);
              dg[e] = dy[e] * (gam[c0 + e] * xh + bet[c0 + e]) * dgelu;
              dn = dy[e] * gelu;
            }
            const float dx = dn * gam[c0 + e];
            dxv[j][e] = dx;
            m1 += dx;
            m2 = fmaf(dx, xh, m2);
          }
          if (p.gate != nullptr) {
            T* dgp = static_cast<T*>(p.dgate) + tok * p.ld_dgate + c0;
            if constexpr (sizeof(T) == 2) {
              uint2 o0, o1;
              o0.x = pack_bf16(dg[0], dg[1]); o0.y = pack_bf16(dg[2], dg[3]);
              o1.x = pack_bf16(dg[4], dg[5]); o1.y = pack_bf16(dg[6], dg[7]);
              reinterpret_cast<uint2*>(dgp)[0] = o0;
              reinterpret_cast<uint2*>(dgp)[1] = o1;
            } else {
              reinterpret_cast<float2*>(dgp)[0] = make_float2(dg[0], dg[1]);
              reinterpret_cast<float2*>(dgp)[1] = make_float2(dg[2], dg[3]);
            }
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        m1 += __shfl_xor_sync(0xffffffffu, m1, o);
        m2 += __shfl_xor_sync(0xffffffffu, m2, o);
      }
      m1 /= C;
      m2 /= C;
      // pass 2: dz back into the tile, in place
#pragma unroll
      for (int j = 0; j < MAXCH; ++j) {
        const int ch = j * 32 + lane;
        if (ch < nch) {
          float dz[EPC];
#pragma unroll
          for (int e = 0; e < EPC; ++e) dz[e] = rstd * (dxv[j][e] - m1 - v[j][e] * rstd * m2);
          if constexpr (sizeof(T) == 2) {
            Vec8<T> o;
            o.pack(dz);
            o.store(row + ch * EPC);
          } else {
            *reinterpret_cast<float4*>(row + ch * EPC) = make_float4(dz[0], dz[1], dz[2], dz[3]);
          }
        }
      }
    }
    __syncthreads();  // the tile now holds dz for every row
    for (int idx = tid; idx < H * seg; idx += EPI_THREADS) {
      const int h = idx / seg, i = idx - h * seg, r = i / CPR, cc = i - r * CPR;
      if (r < rows) {
        T* dst = static_cast<T*>(p.d_inner) + (((size_t)b * H + h) * NT + t0) * HD + (size_t)i * EPC;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(tile + (size_t)r * C + h * HD + cc * EPC);
      }
    }
    __syncthreads();  // done with this buffer before the next iteration refills it
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

}

// Parameter gradients of the post norm: d weight[c] = sum over tokens of dn * x_hat, d bias[c] = sum of dn.  One CTA
// per slab of PARAM_SLAB tokens, one thread per column pair, rows walked in order; the slab's sums go to `partials`.
constexpr int PARAM_SLAB = 128;
template <typename T, int FD>
__global__ void ttt_layer_epilogue_bwd_param_kernel(const LayerEpiBwdParams p) {
  constexpr int HD = FD;  // features per head in this instantiation
  const int H = p.H, NT = p.T, C = H * HD;
  const int pair = threadIdx.x;          // columns 2*pair, 2*pair+1
  const int c = 2 * pair, h = c / HD, f = c % HD;
  const long ntok = (long)p.B * NT;
  const long row0 = (long)blockIdx.x * PARAM_SLAB;
  const long row1 = row0 + PARAM_SLAB < ntok ? row0 + PARAM_SLAB : ntok;
  auto ld2 = [](const void* base, size_t idx) -> float2 {
    if constexpr (sizeof(T) == 2) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(static_cast<const T*>(base) + idx);
      return make_float2(bf16_lo(w), bf16_hi(w));
    } else {
      return *reinterpret_cast<const float2*>(static_cast<const T*>(base) + idx);
    }
  };
  float2 ag = make_float2(0.f, 0.f), ab = make_float2(0.f, 0.f);
  int t = (int)(row0 % NT), b = (int)(row0 / NT);
  size_t zoff = (((size_t)b * H + h) * NT + t) * HD + f;  // advances by one row per token, re-based at a batch boundary
  size_t doff = (size_t)row0 * C + c, goff = (size_t)row0 * p.ld_gate + c;
#pragma unroll 4
  for (long tok = row0; tok < row1; ++tok) {
    const float2 st = p.row_stats[tok];
    const float2 z = ld2(p.inner_out, zoff);
    float2 dn = ld2(p.dy, doff);
    if (p.gate != nullptr) {
      const float2 g = ld2(p.gate, goff);
      const float u0 = 0.7978845608028654f * (g.x + 0.044715f * g.x * g.x * g.x);
      const float u1 = 0.7978845608028654f * (g.y + 0.044715f * g.y * g.y * g.y);
      dn.x *= 0.5f * g.x * (1.f + tanhf(u0));
      dn.y *= 0.5f * g.y * (1.f + tanhf(u1));
    }
    ag.x = fmaf(dn.x, (z.x - st.x) * st.y, ag.x);
    ag.y = fmaf(dn.y, (z.y - st.x) * st.y, ag.y);
    ab.x += dn.x;
    ab.y += dn.y;
    doff += C;
    goff += p.ld_gate;
    zoff += HD;
    if (++t == NT) {
      t = 0;
      ++b;
      zoff = ((size_t)b * H + h) * NT * HD + f;
    }
  }
  float* out = p.partials + (size_t)blockIdx.x * 2 * C;
  *reinterpret_cast<float2*>(out + c) = ag;
  *reinterpret_cast<float2*>(out + C + c) = ab;
}

// d post_norm_weight / d post_norm_bias: the slabs' partial rows added in a fixed order.  A CTA owns 32 columns;
// its 8 warps each add an interleaved eighth of the parts (lanes = columns, so every load is one coalesced 128-byte
// row segment), and the eight sums are combined in warp order through shared memory.
__global__ void __launch_bounds__(256) ttt_layer_epilogue_bwd_reduce_kernel(const float* partials, int nparts, int C,
                                                                            float* dw, float* db) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;  // column of the [2][C] row
  float s = 0.f;
  if (c < 2 * C)
    for (int i = warp; i < nparts; i += 8) s += partials[(size_t)i * 2 * C + c];
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < 2 * C) {
    float tot = red[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) tot += red[w][lane];
    if (c < C)
      dw[c] = tot;
    else
      db[c - C] = tot;
  }
}

cudaError_t launch_layer_prologue_bwd(int dtype, int head_dim, const LayerProBwdParams& p, cudaStream_t st) {
  const int grid = prologue_grid(p.B, p.H, p.T, head_dim);
  if (head_dim == 32) {
    if (dtype == 1) ttt_layer_prologue_bwd_kernel<__nv_bfloat16, 32><<<grid, PRO_THREADS, 0, st>>>(p);
    else ttt_layer_prologue_bwd_kernel<float, 32><<<grid, PRO_THREADS, 0, st>>>(p);
  } else {
    if (dtype == 1) ttt_layer_prologue_bwd_kernel<__nv_bfloat16, 64><<<grid, PRO_THREADS, 0, st>>>(p);
    else ttt_layer_prologue_bwd_kernel<float, 64><<<grid, PRO_THREADS, 0, st>>>(p);
  }
  return cudaGetLastError();
}

size_t layer_epilogue_bwd_workspace_bytes(int B, int H, int T, int head_dim) {
  const size_t ntok = (size_t)B * T, nslab = (ntok + PARAM_SLAB - 1) / PARAM_SLAB;
  return ntok * sizeof(float2) + nslab * 2 * (size_t)H * head_dim * sizeof(float);
}

template <typename T, int MAXCH, int FD>
static cudaError_t launch_epi_bwd_t(LayerEpiBwdParams p, cudaStream_t st) {
  const int C = p.H * FD;
  constexpr int TT = 64 / MAXCH;
  const size_t smem = 2 * (size_t)TT * C * sizeof(T) + 2 * (size_t)C * sizeof(float);
  auto kfn = ttt_layer_epilogue_bwd_kernel<T, MAXCH, FD>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const long ntiles = (long)p.B * ((p.T + TT - 1) / TT);
  int per_sm = 1;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kfn, EPI_THREADS, smem);
  if (e != cudaSuccess) return e;
  if (per_sm > 2) per_sm = 2;
  const long cap = (long)sm_count() * (per_sm < 1 ? 1 : per_sm);
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  kfn<<<grid < 1 ? 1 : grid, EPI_THREADS, smem, st>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const long ntok = (long)p.B * p.T;
  const int nslab = (int)((ntok + PARAM_SLAB - 1) / PARAM_SLAB);
  ttt_layer_epilogue_bwd_param_kernel<T, FD><<<nslab, C / 2, 0, st>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  ttt_layer_epilogue_bwd_reduce_kernel<<<(2 * C + 31) / 32, 256, 0, st>>>(p.partials, nslab, C, p.d_ln_w, p.d_ln_b);
  return cudaGetLastError();
}

template <int FD>
static cudaError_t launch_epi_bwd_f(int dtype, const LayerEpiBwdParams& p, cudaStream_t st) {
  const int C = p.H * FD;
  if (dtype == 1) return C <= 1024 ? launch_epi_bwd_t<__nv_bfloat16, 4, FD>(p, st) : launch_epi_bwd_t<__nv_bfloat16, 8, FD>(p, st);
  if (C <= 512) return launch_epi_bwd_t<float, 4, FD>(p, st);
  return C <= 1024 ? launch_epi_bwd_t<float, 8, FD>(p, st) : launch_epi_bwd_t<float, 16, FD>(p, st);
}

cudaError_t launch_layer_epilogue_bwd(int dtype, int head_dim, const LayerEpiBwdParams& p0, cudaStream_t st) {
  // workspace: (mean, rstd) per token, then the slabs' partial parameter gradients
  LayerEpiBwdParams p = p0;
  p.row_stats = reinterpret_cast<float2*>(p0.partials);
  p.partials = p0.partials + 2 * (size_t)p0.B * p0.T;
  return head_dim == 32 ? launch_epi_bwd_f<32>(dtype, p, st) : launch_epi_bwd_f<64>(dtype, p, st);
}

// ----------------------------------------------------------------------------------------------------
// Shared-QK convolutions as a differentiable step (training path of the shared-QK layout; inference applies them
// inside the prologue kernel).  A thread owns four adjacent channels and walks LAYER_CONV_CHUNK tokens of one batch
// row with a rolling window, so every global access of a warp is one contiguous row piece.
// ----------------------------------------------------------------------------------------------------
template <typename T>
struct Vec4;
template <>
struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const void* p, float (&f)[4]) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    f[0] = bf16_lo(r.x); f[1] = bf16_hi(r.x); f[2] = bf16_lo(r.y); f[3] = bf16_hi(r.y);
  }
  static __device__ __forceinline__ void store(void* p, const float (&f)[4]) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]));
  }
};
template <>
struct Vec4<float> {
  static __device__ __forceinline__ void load(const void* p, float (&f)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w;
  }
  static __device__ __forceinline__ void store(void* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

template <typename T>
__global__ void __launch_bounds__(256) ttt_layer_conv_kernel(const LayerConvParams p) {
  const int ncg = p.C / 4, nch = (p.T + LAYER_CONV_CHUNK - 1) / LAYER_CONV_CHUNK;
  const long total = (long)p.B * nch * ncg;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int cg = (int)(idx % ncg);
    const long rest = idx / ncg;
    const int ch = (int)(rest % nch), b = (int)(rest / nch);
    const int c0 = 4 * cg, t0 = ch * LAYER_CONV_CHUNK, t1 = min(t0 + LAYER_CONV_CHUNK, p.T);
    float wq[4][4], wk[4][4], bq[4], bk[4];  // [channel][tap]
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      Vec4<T>::load(static_cast<const T*>(p.wq) + (size_t)(c0 + c) * 4, wq[c]);
      Vec4<T>::load(static_cast<const T*>(p.wk) + (size_t)(c0 + c) * 4, wk[c]);
    }
    Vec4<T>::load(static_cast<const T*>(p.bq) + c0, bq);
    Vec4<T>::load(static_cast<const T*>(p.bk) + c0, bk);
    const T* xb = static_cast<const T*>(p.x) + (size_t)b * p.T * p.ld_x + c0;
    float win[3][4];  // x at t-3, t-2, t-1
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      const int t = t0 - 3 + d;
      if (t >= 0) {
        Vec4<T>::load(xb + (size_t)t * p.ld_x, win[d]);
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) win[d][c] = 0.f;
      }
    }
    for (int t = t0; t < t1; ++t) {
      float xv[4], q[4], k[4];
      Vec4<T>::load(xb + (size_t)t * p.ld_x, xv);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        q[c] = bq[c] + wq[c][0] * win[0][c] + wq[c][1] * win[1][c] + wq[c][2] * win[2][c] + wq[c][3] * xv[c];
        k[c] = bk[c] + wk[c][0] * win[0][c] + wk[c][1] * win[1][c] + wk[c][2] * win[2][c] + wk[c][3] * xv[c];
        win[0][c] = win[1][c];
        win[1][c] = win[2][c];
        win[2][c] = xv[c];
      }
      const size_t o = ((size_t)b * p.T + t) * p.C + c0;
      Vec4<T>::store(static_cast<T*>(p.q) + o, q);
      Vec4<T>::store(static_cast<T*>(p.k) + o, k);
    }
  }
}

// dx[t] = sum_j wq[j] dq[t + 3 - j] + wk[j] dk[t + 3 - j] (terms beyond the sequence end dropped); parameter
// gradients d w[j] = sum_t d out[t] x[t - 3 + j], d b = sum_t d out[t], as per-chunk partials (summed afterwards in a
// fixed order).  The chunk is walked from its last token to its first.
template <typename T>
__global__ void __launch_bounds__(256) ttt_layer_conv_bwd_kernel(const LayerConvBwdParams p) {
  const int ncg = p.C / 4, nch = (p.T + LAYER_CONV_CHUNK - 1) / LAYER_CONV_CHUNK;
  const long total = (long)p.B * nch * ncg;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int cg = (int)(idx % ncg);
    const long rest = idx / ncg;
    const int ch = (int)(rest % nch), b = (int)(rest / nch);
    const int c0 = 4 * cg, t0 = ch * LAYER_CONV_CHUNK, t1 = min(t0 + LAYER_CONV_CHUNK, p.T);
    float wq[4][4], wk[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      Vec4<T>::load(static_cast<const T*>(p.wq) + (size_t)(c0 + c) * 4, wq[c]);
      Vec4<T>::load(static_cast<const T*>(p.wk) + (size_t)(c0 + c) * 4, wk[c]);
    }
    const T* xb = static_cast<const T*>(p.x) + (size_t)b * p.T * p.ld_x + c0;
    const T* dqb = static_cast<const T*>(p.dq) + (size_t)b * p.T * p.C + c0;
    const T* dkb = static_cast<const T*>(p.dk) + (size_t)b * p.T * p.C + c0;
    float gq[3][4], gk[3][4];  // d out at t+1, t+2, t+3
    float xw[4][4];            // x at t, t-1, t-2, t-3
    float aq[5][4], ak[5][4];  // accumulators: taps 0..3, bias
#pragma unroll
    for (int j = 0; j < 5; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) aq[j][c] = ak[j][c] = 0.f;
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      const int t = t1 + d;
      if (t < p.T) {
        Vec4<T>::load(dqb + (size_t)t * p.C, gq[d]);
        Vec4<T>::load(dkb + (size_t)t * p.C, gk[d]);
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) gq[d][c] = gk[d][c] = 0.f;
      }
    }
#pragma unroll
    for (int d = 0; d < 4; ++d) {
      const int t = t1 - 1 - d;
      if (t >= 0) {
        Vec4<T>::load(xb + (size_t)t * p.ld_x, xw[d]);
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) xw[d][c] = 0.f;
      }
    }
    for (int t = t1 - 1; t >= t0; --t) {
      float dqv[4], dkv[4], dx[4];
      Vec4<T>::load(dqb + (size_t)t * p.C, dqv);
      Vec4<T>::load(dkb + (size_t)t * p.C, dkv);
      float xn[4];  // x at t-4, for the next step
      if (t - 4 >= 0) {
        Vec4<T>::load(xb + (size_t)(t - 4) * p.ld_x, xn);
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) xn[c] = 0.f;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        // tap j multiplies x[t - 3 + j]: its transpose sends d out[t + 3 - j] to x[t]
        dx[c] = wq[c][3] * dqv[c] + wq[c][2] * gq[0][c] + wq[c][1] * gq[1][c] + wq[c][0] * gq[2][c] +
                wk[c][3] * dkv[c] + wk[c][2] * gk[0][c] + wk[c][1] * gk[1][c] + wk[c][0] * gk[2][c];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          aq[j][c] += dqv[c] * xw[3 - j][c];
          ak[j][c] += dkv[c] * xw[3 - j][c];
        }
        aq[4][c] += dqv[c];
        ak[4][c] += dkv[c];
        gq[2][c] = gq[1][c]; gq[1][c] = gq[0][c]; gq[0][c] = dqv[c];
        gk[2][c] = gk[1][c]; gk[1][c] = gk[0][c]; gk[0][c] = dkv[c];
        xw[0][c] = xw[1][c]; xw[1][c] = xw[2][c]; xw[2][c] = xw[3][c]; xw[3][c] = xn[c];
      }
      Vec4<T>::store(static_cast<T*>(p.dx) + ((size_t)b * p.T + t) * p.C + c0, dx);
    }
    float* row = p.partials + ((size_t)b * nch + ch) * 10 * p.C;
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      *reinterpret_cast<float4*>(row + (size_t)j * p.C + c0) = make_float4(aq[j][0], aq[j][1], aq[j][2], aq[j][3]);
      *reinterpret_cast<float4*>(row + (size_t)(5 + j) * p.C + c0) = make_float4(ak[j][0], ak[j][1], ak[j][2], ak[j][3]);
    }
  }
}

static int conv_grid(const long total) {
  const long want = (total + 255) / 256, cap = (long)sm_count() * 8;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

cudaError_t launch_layer_conv(int dtype, const LayerConvParams& p, cudaStream_t st) {
  const long total = (long)p.B * ((p.T + LAYER_CONV_CHUNK - 1) / LAYER_CONV_CHUNK) * (p.C / 4);
  if (dtype == 1)
    ttt_layer_conv_kernel<__nv_bfloat16><<<conv_grid(total), 256, 0, st>>>(p);
  else
    ttt_layer_conv_kernel<float><<<conv_grid(total), 256, 0, st>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_layer_conv_bwd(int dtype, const LayerConvBwdParams& p, cudaStream_t st) {
  const int nch = (p.T + LAYER_CONV_CHUNK - 1) / LAYER_CONV_CHUNK;
  const long total = (long)p.B * nch * (p.C / 4);
  if (dtype == 1)
    ttt_layer_conv_bwd_kernel<__nv_bfloat16><<<conv_grid(total), 256, 0, st>>>(p);
  else
    ttt_layer_conv_bwd_kernel<float><<<conv_grid(total), 256, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // sum the chunks' partial rows [10 C] in a fixed order: first 5 C -> the q parameters, last 5 C -> the k parameters
  ttt_layer_epilogue_bwd_reduce_kernel<<<(10 * p.C + 31) / 32, 256, 0, st>>>(p.partials, p.B * nch, 5 * p.C,
                                                                            p.dparams_q, p.dparams_k);
  return cudaGetLastError();
}

}  // namespace ttt
