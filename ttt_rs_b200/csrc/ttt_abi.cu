// C ABI of the fused TTT inner loop: argument validation, TMA descriptor set-up and kernel launches.
// Signatures and their reference counterparts are documented in include/ttt_b200.h.
#include <cstdarg>
#include <cstdio>
#include <atomic>
#include <cstring>
#include <cstdlib>
#include <mutex>

#include "../../include/ttt_b200.h"
#include "ttt_kernels.h"

namespace {

thread_local char g_err[512] = "";

// Diagnostic knobs of the persistent backward (ttt_b200_debug_handoff): poll limit of the hand-off wait and an offset
// added to the work-item numbers.
constexpr uint32_t kHandoffPollsDefault = 1u << 24;
std::atomic<uint32_t> g_handoff_polls{kHandoffPollsDefault};
std::atomic<int32_t> g_item_base{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;  // benign race: every thread resolves the same pointer
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

// 2-D view [rows, 64] of a [B,H,T,64] tensor, box = one 16-token tile (or half of it for float32),
// 128-byte swizzle so that ldmatrix / element-wise shared-memory reads are bank-conflict free.
int make_tile_map(CUtensorMap* m, const void* base, int64_t rows, int dtype, int box_rows = 16) {
  EncodeFn enc = get_encode_fn();
  if (enc == nullptr) return fail(TTT_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const bool bf = dtype == TTT_BF16;
  const cuuint64_t dims[2] = {64, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)(64 * (bf ? 2 : 4))};
  const cuuint32_t box[2] = {(cuuint32_t)(bf ? 64 : 32), (cuuint32_t)box_rows};  // (8 rows: mini-batches of 8 tokens)
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, bf ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TTT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TTT_OK;
}

// 2-D bf16 view [rows, cols] with a row pitch of `ld` elements, box = 64 columns x `box_rows` rows (128: A operand
// and result tiles of the projection GEMM; 256: its B operand), 128-byte swizzle.
int make_gemm_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows = 128) {
  EncodeFn enc = get_encode_fn();
  if (enc == nullptr) return fail(TTT_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)(ld * 2)};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TTT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TTT_OK;
}

// View of a float32 [B,H,T,32] tensor for the kernels that take a PAIR of 32-wide heads per 64-wide tile: 2-D
// [B*H*T, 32], box = 16 tokens x 32 features = 16 rows of 128 bytes = one half tile.  (In bf16 a half tile is 64 bytes
// wide, narrower than the swizzle span; those tiles are gathered by the kernel from the plain pointer and the map is a
// placeholder over the same memory.)
int make_pair_map(CUtensorMap* m, const void* base, int64_t pairs, int64_t T, int dtype, int box_rows = 16) {
  EncodeFn enc = get_encode_fn();
  if (enc == nullptr) return fail(TTT_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const bool bf = dtype == TTT_BF16;
  const cuuint64_t dims[2] = {32, (cuuint64_t)(2 * pairs * T)};
  const cuuint64_t strides[1] = {(cuuint64_t)(32 * (bf ? 2 : 4))};
  const cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, bf ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   bf ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TTT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TTT_OK;
}

// How the problem looks to the 64-wide kernels: head_dim 64 as it is; head_dim 32 (TTT-Linear only) as H/2 streams per
// batch row, each a pair of heads side by side.
struct Packing {
  int seg;         // features per head: 64 or 32
  int nh;          // heads per tile: 1 or 2
  int heads;       // streams per batch row as the kernels count them
  int64_t streams; // batch * heads
  int64_t rows;    // streams * seq_len
};
Packing packing(const ttt_dims* d) {
  Packing k;
  k.seg = d->head_dim;
  k.nh = 64 / d->head_dim;
  k.heads = d->heads / k.nh;
  k.streams = (int64_t)d->batch * k.heads;
  k.rows = k.streams * d->seq_len;
  return k;
}
// map of one [B,H,T,F] input or output of the caller
int make_io_map(CUtensorMap* m, const void* base, const ttt_dims* d) {
  const Packing k = packing(d);
  if (k.seg == 64) return make_tile_map(m, base, k.rows, d->dtype, d->mini_batch);
  return make_pair_map(m, base, k.streams, d->seq_len, d->dtype, d->mini_batch);
}

// Which form of the projection GEMM runs: CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles) when the product has at
// least two such rows of tiles, single CTAs (128 x 256 tiles) below that (decode steps, short prefills).
// TTT_GEMM_PAIR=0 / 1 in the environment forces one form (measurements, tests).
bool gemm_pair_form(int64_t m) {
  static const int forced = [] {
    const char* e = std::getenv("TTT_GEMM_PAIR");
    return (e != nullptr && e[0] != '\0') ? (e[0] != '0' ? 1 : 0) : -1;
  }();
  return forced >= 0 ? forced != 0 : m >= 512;
}

int check_dims(const ttt_dims* d, bool linear_tiles = false) {
  if (d == nullptr) return fail(TTT_ERR_NULL, "dims is null");
  if (d->batch <= 0 || d->heads <= 0 || d->seq_len <= 0 || d->head_dim <= 0 || d->mini_batch <= 0)
    return fail(TTT_ERR_SHAPE, "batch, heads, seq_len, head_dim and mini_batch must be positive");
  if (d->checkpoint_interval < 1) return fail(TTT_ERR_SHAPE, "checkpoint_interval must be >= 1");
  if (d->dtype != TTT_F32 && d->dtype != TTT_BF16) return fail(TTT_ERR_UNSUPPORTED, "unknown dtype %d", d->dtype);
  // TTT-Linear forward / backward (`linear_tiles`): 16x64, 16x32, 8x64, 8x32; everything else: 16x64
  const bool mb_ok = d->mini_batch == 16 || (linear_tiles && d->mini_batch == 8);
  const bool hd_ok = d->head_dim == 64 || (linear_tiles && d->head_dim == 32);
  if (!mb_ok || !hd_ok)
    return fail(TTT_ERR_UNSUPPORTED, "Unsupported tile config: mini_batch_len=%d, head_dim=%d (supported: 16x64%s)",
                d->mini_batch, d->head_dim, linear_tiles ? ", 16x32, 8x64, 8x32" : "");
  if (d->head_dim == 32 && d->heads % 2 != 0)
    return fail(TTT_ERR_UNSUPPORTED, "head_dim 32 runs two heads per tile and needs an even number of heads (got %d)",
                d->heads);
  if (d->seq_len % d->mini_batch != 0)
    return fail(TTT_ERR_SHAPE, "seq_len (%d) must be divisible by mini_batch_len (%d)", d->seq_len, d->mini_batch);
  if ((int64_t)d->batch * d->heads * d->seq_len >= (int64_t)1 << 31)
    return fail(TTT_ERR_SHAPE, "batch*heads*seq_len must be below 2^31");
  if (!(d->epsilon >= 0.f)) return fail(TTT_ERR_SHAPE, "epsilon must be >= 0");
  return TTT_OK;
}

struct NamedPtr {
  const char* name;
  const void* p;
};

int check_ptrs(const NamedPtr* ptrs, int n) {
  for (int i = 0; i < n; ++i) {
    if (ptrs[i].p == nullptr) return fail(TTT_ERR_NULL, "%s is null", ptrs[i].name);
    if ((reinterpret_cast<uintptr_t>(ptrs[i].p) & 15u) != 0)
      return fail(TTT_ERR_ALIGN, "%s is not 16-byte aligned", ptrs[i].name);
  }
  return TTT_OK;
}

int64_t num_ckpt(const ttt_dims* d) {
  const int64_t ns = d->seq_len / d->mini_batch;
  return (ns + d->checkpoint_interval - 1) / d->checkpoint_interval;
}

// Layout of the second saved-state buffer ("aux"): the lr-scaled LN gradient tiles Gp [B*H*T, 64] of the I/O type,
// then two float4 of row statistics per token, then the float32 bias at the start of every stage (+ final).
struct AuxLayout {
  size_t off_gp, off_stats, off_bias, total_bytes;
};
AuxLayout aux_layout(const ttt_dims* d) {
  const Packing k = packing(d);
  const size_t rows = (size_t)k.rows;
  const size_t streams = (size_t)k.streams;
  const size_t ns = (size_t)d->seq_len / d->mini_batch;
  AuxLayout a;
  a.off_gp = 0;
  a.off_stats = a.off_gp + rows * 64 * (d->dtype == TTT_BF16 ? 2 : 4);
  a.off_bias = a.off_stats + rows * 32 * k.nh;  // one record of two float4 per (token, head)
  a.total_bytes = a.off_bias + streams * (ns + 1) * 64 * sizeof(float);
  return a;
}

// workspace layout of the backward (float32 words)
constexpr int kBwdChunkStages = 16;  // stages per work item of the persistent backward kernel
struct WsLayout {
  size_t off_ln, off_te, off_w, off_handoff, off_sched, total_bytes;
  int nch;
};
WsLayout ws_layout(const ttt_dims* d) {
  const Packing k = packing(d);
  const size_t streams = (size_t)k.streams;                    // as the kernel counts them
  const size_t heads_all = (size_t)d->batch * d->heads;        // as the caller counts them
  const size_t F = (size_t)d->head_dim;
  const int ns = d->seq_len / d->mini_batch;
  WsLayout w;
  w.nch = (ns + kBwdChunkStages - 1) / kBwdChunkStages;
  w.off_ln = 0;
  w.off_te = w.off_ln + streams * (size_t)w.nch * 2 * 64;
  w.off_w = w.off_te + heads_all * (size_t)d->seq_len;
  w.off_handoff = w.off_w + heads_all * (F * F + F);
  w.off_sched = w.off_handoff + streams * (2 * 64 * 64 + 64);
  const size_t words = w.off_sched + ((1 + streams + 3) & ~(size_t)3);
  w.total_bytes = words * sizeof(float);
  return w;
}

}  // namespace

// workspace of the TTT-MLP backward (which the forward can pre-fill)
namespace {
struct MlpWsLayout {
  size_t stride_floats, off_te, off_ln, off_sched, total_bytes;
};
MlpWsLayout mlp_ws_layout(const ttt_dims* d) {
  const size_t streams = (size_t)d->batch * d->heads;
  MlpWsLayout l;
  l.stride_floats = ttt::mlp_bwd_ws_stride_floats(d->seq_len);
  l.off_te = streams * l.stride_floats;
  l.off_ln = l.off_te + streams * (size_t)d->seq_len;
  l.off_sched = l.off_ln + streams * 2 * 64;
  l.total_bytes = (l.off_sched + ((1 + streams + 3) & ~(size_t)3)) * sizeof(float);
  return l;
}
}  // namespace

extern "C" {

int ttt_b200_abi_version(void) { return TTT_B200_ABI_VERSION; }

const char* ttt_b200_status_string(int s) {
  switch (s) {
    case TTT_OK: return "ok";
    case TTT_ERR_NULL: return "null pointer";
    case TTT_ERR_SHAPE: return "bad shape";
    case TTT_ERR_UNSUPPORTED: return "unsupported configuration";
    case TTT_ERR_ALIGN: return "misaligned pointer";
    case TTT_ERR_CUDA: return "CUDA error";
    case TTT_ERR_TIMEOUT: return "device-side wait timed out";
    case TTT_ERR_WORKSPACE: return "workspace too small";
    default: return "unknown status";
  }
}

const char* ttt_b200_last_error(void) { return g_err; }

int ttt_gemm_bf16_tn(int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, const void* b, int64_t ldb, void* c,
                     int64_t ldc, void* status, void* stream) {
  if (m <= 0 || n <= 0 || k <= 0 || m >= ((int64_t)1 << 31) || n >= ((int64_t)1 << 31) || k >= ((int64_t)1 << 31))
    return fail(TTT_ERR_SHAPE, "m, n, k must be positive and below 2^31");
  if (lda < k || ldb < k || ldc < n) return fail(TTT_ERR_SHAPE, "a row pitch is shorter than the row");
  if ((lda | ldb | ldc) % 8 != 0) return fail(TTT_ERR_ALIGN, "row pitches must be multiples of 8 elements (16 bytes)");
  const NamedPtr ptrs[] = {{"a", a}, {"b", b}, {"c", c}};
  int rc = check_ptrs(ptrs, 3);
  if (rc != TTT_OK) return rc;
  CUtensorMap maps[7];
  if ((rc = make_gemm_map(&maps[0], a, m, k, lda)) != TTT_OK) return rc;
  const bool pair = gemm_pair_form(m);
  if ((rc = make_gemm_map(&maps[1], b, n, k, ldb, pair ? 128 : 256)) != TTT_OK) return rc;
  if ((rc = make_gemm_map(&maps[2], c, m, n, ldc)) != TTT_OK) return rc;
  for (int i = 3; i < 7; ++i) maps[i] = maps[2];
  ttt::GemmParams p{};
  p.M = (int)m;
  p.N = (int)n;
  p.K = (int)k;
  p.status = static_cast<uint32_t*>(status);
  cudaError_t e = ttt::launch_gemm_bf16_tn(maps, p, false, pair, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "GEMM launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

int ttt_layer_projections(const ttt_dims* d, const void* x, int64_t x_ld, int64_t hidden, const void* weights,
                          int64_t w_ld, int64_t w_rows, int64_t q_col, int64_t k_col, int64_t v_col, int64_t g_col,
                          int64_t lr_col, const void* lr_bias, int start_idx, int rope_mode, float rope_theta,
                          float base_lr, void* xq, void* xk, void* xv, void* gate, void* ttt_lr_eta, void* status,
                          void* stream) {
  if (d == nullptr) return fail(TTT_ERR_NULL, "dims is null");
  if (d->batch <= 0 || d->heads <= 0 || d->seq_len <= 0) return fail(TTT_ERR_SHAPE, "batch, heads, seq_len must be positive");
  if (d->dtype != TTT_BF16 || d->head_dim != 64)
    return fail(TTT_ERR_UNSUPPORTED, "the fused projection is built for bf16 and head_dim 64");
  if (d->seq_len % 128 != 0)
    return fail(TTT_ERR_UNSUPPORTED, "the fused projection needs seq_len %% 128 == 0 (got %d): use ttt_gemm_bf16_tn + "
                                     "ttt_layer_prologue", d->seq_len);
  if (d->heads > 64) return fail(TTT_ERR_UNSUPPORTED, "at most 64 heads");
  if (rope_mode != 0 && rope_mode != 1)
    return fail(TTT_ERR_UNSUPPORTED, "the fused projection rotates with wrapped positions (rope_mode 1) or not at all");
  if (rope_mode == 1 && (d->mini_batch < 1 || d->mini_batch > 16))
    return fail(TTT_ERR_UNSUPPORTED, "wrapped rotary positions need 1 <= mini_batch <= 16 here (got %d)", d->mini_batch);
  if (rope_mode == 1 && !(rope_theta > 0.f)) return fail(TTT_ERR_SHAPE, "rope_theta must be positive");
  if (start_idx < 0) return fail(TTT_ERR_SHAPE, "start_idx must be >= 0");
  const int64_t C = (int64_t)d->heads * 64, M = (int64_t)d->batch * d->seq_len;
  if (hidden <= 0 || w_rows <= 0 || x_ld < hidden || w_ld < hidden || ((x_ld | w_ld) & 7) != 0)
    return fail(TTT_ERR_SHAPE, "hidden, pitches: x_ld and w_ld must be >= hidden and multiples of 8");
  const int64_t cols[5] = {q_col, k_col, v_col, g_col, lr_col};
  for (int i = 0; i < 5; ++i) {
    if (i == 3 && g_col < 0) continue;
    if (cols[i] < 0 || (cols[i] & 63) != 0 || cols[i] + (i == 4 ? d->heads : C) > w_rows)
      return fail(TTT_ERR_SHAPE, "column block %d starts at %lld: must be a multiple of 64 inside the %lld weight rows",
                  i, (long long)cols[i], (long long)w_rows);
  }
  if ((g_col >= 0) != (gate != nullptr)) return fail(TTT_ERR_NULL, "gate buffer and g_col must be given together");
  const NamedPtr ptrs[] = {{"x", x}, {"weights", weights}, {"xq", xq}, {"xk", xk}, {"xv", xv}, {"ttt_lr_eta", ttt_lr_eta}};
  int rc = check_ptrs(ptrs, 6);
  if (rc != TTT_OK) return rc;
  const int64_t rows = (int64_t)d->batch * d->heads * d->seq_len;
  if (rows >= ((int64_t)1 << 31) || M >= ((int64_t)1 << 31)) return fail(TTT_ERR_SHAPE, "batch*heads*seq_len must be below 2^31");
  CUtensorMap maps[7];
  if ((rc = make_gemm_map(&maps[0], x, M, hidden, x_ld)) != TTT_OK) return rc;
  const bool pair = gemm_pair_form(M);
  if ((rc = make_gemm_map(&maps[1], weights, w_rows, hidden, w_ld, pair ? 128 : 256)) != TTT_OK) return rc;
  if ((rc = make_gemm_map(&maps[3], xq, rows, 64, 64)) != TTT_OK) return rc;
  if ((rc = make_gemm_map(&maps[4], xk, rows, 64, 64)) != TTT_OK) return rc;
  if ((rc = make_gemm_map(&maps[5], xv, rows, 64, 64)) != TTT_OK) return rc;
  if (gate != nullptr) {
    if ((rc = make_gemm_map(&maps[6], gate, M, C, C)) != TTT_OK) return rc;
  } else {
    maps[6] = maps[5];
  }
  maps[2] = maps[3];
  ttt::GemmParams p{};
  p.M = (int)M;
  p.N = (int)w_rows;
  p.K = (int)hidden;
  p.status = static_cast<uint32_t*>(status);
  p.f.q_col = (int)q_col; p.f.k_col = (int)k_col; p.f.v_col = (int)v_col; p.f.g_col = (int)g_col; p.f.lr_col = (int)lr_col;
  p.f.H = d->heads; p.f.T = d->seq_len;
  p.f.start_idx = start_idx; p.f.pos_mod = rope_mode == 1 ? d->mini_batch : 1; p.f.rope_mode = rope_mode;
  p.f.rope_theta = rope_mode == 1 ? rope_theta : 1.f; p.f.base_lr = base_lr;
  p.f.lr_bias = lr_bias; p.f.lr_out = ttt_lr_eta;
  cudaError_t e = ttt::launch_gemm_bf16_tn(maps, p, true, pair, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "fused projection launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

void ttt_b200_debug_handoff(uint32_t poll_limit, int32_t first_item) {
  g_handoff_polls.store(poll_limit == 0 ? kHandoffPollsDefault : poll_limit);
  g_item_base.store(first_item < 0 ? 0 : first_item);
}

int64_t ttt_linear_num_checkpoints(const ttt_dims* d) {
  if (check_dims(d, true) != TTT_OK) return -1;
  return num_ckpt(d);
}
size_t ttt_linear_weight_ckpt_bytes(const ttt_dims* d) {
  if (check_dims(d, true) != TTT_OK) return 0;
  return (size_t)packing(d).streams * (num_ckpt(d) + 1) * 64 * 64 * sizeof(float);
}
size_t ttt_linear_bias_ckpt_bytes(const ttt_dims* d) {
  if (check_dims(d, true) != TTT_OK) return 0;
  return aux_layout(d).total_bytes;
}

int ttt_linear_forward(const ttt_dims* d, const void* xq, const void* xk, const void* xv, const void* weight,
                       const void* bias, const void* token_eta, const void* ttt_lr_eta, const void* ln_weight,
                       const void* ln_bias, void* output, void* weight_out, void* bias_out, void* weight_ckpt,
                       void* bias_ckpt, void* status, void* stream) {
  int rc = check_dims(d, true);
  if (rc != TTT_OK) return rc;
  const NamedPtr ptrs[] = {{"xq", xq},           {"xk", xk},
                           {"xv", xv},           {"weight", weight},
                           {"bias", bias},       {"token_eta", token_eta},
                           {"ttt_lr_eta", ttt_lr_eta}, {"ln_weight", ln_weight},
                           {"ln_bias", ln_bias}, {"output", output},
                           {"weight_out", weight_out}, {"bias_out", bias_out},
                           {"weight_ckpt", weight_ckpt}, {"bias_ckpt", bias_ckpt}};
  // inference: both saved-state buffers null = nothing is kept for a backward
  const bool save = weight_ckpt != nullptr || bias_ckpt != nullptr;
  rc = check_ptrs(ptrs, (int)(sizeof(ptrs) / sizeof(ptrs[0])) - (save ? 0 : 2));
  if (rc != TTT_OK) return rc;
  if (status != nullptr && (reinterpret_cast<uintptr_t>(status) & 3u) != 0)
    return fail(TTT_ERR_ALIGN, "status is not 4-byte aligned");

  const Packing pk = packing(d);
  const AuxLayout al = aux_layout(d);
  uint8_t* aux = static_cast<uint8_t*>(bias_ckpt);
  CUtensorMap maps[5];
  const void* bases[4] = {xq, xk, xv, output};
  for (int i = 0; i < 4; ++i) {
    rc = make_io_map(&maps[i], bases[i], d);
    if (rc != TTT_OK) return rc;
  }
  // the saved Gp tiles are always kept 64 wide; without saved state the map is never used, but must be a valid one
  rc = save ? make_tile_map(&maps[4], aux + al.off_gp, pk.rows, d->dtype, d->mini_batch) : make_io_map(&maps[4], output, d);
  if (rc != TTT_OK) return rc;
  ttt::LinFwdParams p;
  p.w0 = weight;
  p.b0 = bias;
  p.token_eta = token_eta;
  p.lr = ttt_lr_eta;
  p.ln_g = ln_weight;
  p.ln_b = ln_bias;
  p.w_out = weight_out;
  p.b_out = bias_out;
  p.w_ckpt = static_cast<float*>(weight_ckpt);
  p.stats = save ? reinterpret_cast<float4*>(aux + al.off_stats) : nullptr;
  p.b_stage = save ? reinterpret_cast<float*>(aux + al.off_bias) : nullptr;
  p.status = static_cast<uint32_t*>(status);
  p.H = pk.heads;
  p.T = d->seq_len;
  p.NS = d->seq_len / d->mini_batch;
  p.K = d->checkpoint_interval;
  p.NCK = (int)num_ckpt(d);
  p.eps = d->epsilon;
  cudaError_t e =
      ttt::launch_linear_fwd(d->dtype, pk.seg, d->mini_batch, maps, bases, p, (int)pk.streams,
                             static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "forward launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

size_t ttt_linear_backward_workspace_bytes(const ttt_dims* d) {
  if (check_dims(d, true) != TTT_OK) return 0;
  return ws_layout(d).total_bytes;
}

int ttt_linear_backward(const ttt_dims* d, const void* xq, const void* xk, const void* xv, const void* weight,
                        const void* bias, const void* token_eta, const void* ttt_lr_eta, const void* ln_weight,
                        const void* ln_bias, const void* weight_ckpt, const void* bias_ckpt,
                        const void* grad_output, void* grad_xq, void* grad_xk, void* grad_xv, void* grad_weight,
                        void* grad_bias, void* grad_ttt_lr_eta, float* grad_token_eta, float* grad_ln_weight,
                        float* grad_ln_bias, float* outer_grad_packed, void* workspace, size_t workspace_bytes,
                        void* status, void* stream) {
  return ttt_linear_backward_state_grads(d, xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias,
                                         weight_ckpt, bias_ckpt, grad_output, nullptr, nullptr, grad_xq, grad_xk,
                                         grad_xv, grad_weight, grad_bias, grad_ttt_lr_eta, grad_token_eta,
                                         grad_ln_weight, grad_ln_bias, outer_grad_packed, workspace, workspace_bytes,
                                         status, stream);
}

int ttt_linear_backward_state_grads(const ttt_dims* d, const void* xq, const void* xk, const void* xv,
                                    const void* weight, const void* bias, const void* token_eta,
                                    const void* ttt_lr_eta, const void* ln_weight, const void* ln_bias,
                                    const void* weight_ckpt, const void* bias_ckpt, const void* grad_output,
                                    const void* grad_weight_out, const void* grad_bias_out, void* grad_xq,
                                    void* grad_xk, void* grad_xv, void* grad_weight, void* grad_bias,
                                    void* grad_ttt_lr_eta, float* grad_token_eta, float* grad_ln_weight,
                                    float* grad_ln_bias, float* outer_grad_packed, void* workspace,
                                    size_t workspace_bytes, void* status, void* stream) {
  int rc = check_dims(d, true);
  if (rc != TTT_OK) return rc;
  const NamedPtr ptrs[] = {{"xq", xq},
                           {"xk", xk},
                           {"xv", xv},
                           {"weight", weight},
                           {"bias", bias},
                           {"token_eta", token_eta},
                           {"ttt_lr_eta", ttt_lr_eta},
                           {"ln_weight", ln_weight},
                           {"ln_bias", ln_bias},
                           {"weight_ckpt", weight_ckpt},
                           {"bias_ckpt", bias_ckpt},
                           {"grad_output", grad_output},
                           {"grad_xq", grad_xq},
                           {"grad_xk", grad_xk},
                           {"grad_xv", grad_xv},
                           {"grad_weight", grad_weight},
                           {"grad_bias", grad_bias},
                           {"grad_ttt_lr_eta", grad_ttt_lr_eta},
                           {"grad_token_eta", grad_token_eta},
                           {"grad_ln_weight", grad_ln_weight},
                           {"grad_ln_bias", grad_ln_bias},
                           {"workspace", workspace}};
  rc = check_ptrs(ptrs, sizeof(ptrs) / sizeof(ptrs[0]));
  if (rc != TTT_OK) return rc;
  if (outer_grad_packed != nullptr && (reinterpret_cast<uintptr_t>(outer_grad_packed) & 15u) != 0)
    return fail(TTT_ERR_ALIGN, "outer_grad_packed is not 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(grad_weight_out) & 15u) != 0 || (reinterpret_cast<uintptr_t>(grad_bias_out) & 15u) != 0)
    return fail(TTT_ERR_ALIGN, "grad_weight_out / grad_bias_out is not 16-byte aligned");
  const WsLayout wl = ws_layout(d);
  if (workspace_bytes < wl.total_bytes)
    return fail(TTT_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, wl.total_bytes);

  const Packing pk = packing(d);
  const AuxLayout al = aux_layout(d);
  const uint8_t* aux = static_cast<const uint8_t*>(bias_ckpt);
  CUtensorMap maps[8];
  const void* bases[7] = {xq, xk, xv, grad_output, grad_xq, grad_xk, grad_xv};
  for (int i = 0; i < 7; ++i) {
    rc = make_io_map(&maps[i], bases[i], d);
    if (rc != TTT_OK) return rc;
  }
  rc = make_tile_map(&maps[7], aux + al.off_gp, pk.rows, d->dtype, d->mini_batch);
  if (rc != TTT_OK) return rc;
  float* ws = static_cast<float*>(workspace);
  ttt::LinBwdParams p;
  p.w0 = weight;
  p.b0 = bias;
  p.token_eta = token_eta;
  p.lr = ttt_lr_eta;
  p.ln_g = ln_weight;
  p.ln_b = ln_bias;
  p.w_ckpt = static_cast<const float*>(weight_ckpt);
  p.stats = reinterpret_cast<const float4*>(aux + al.off_stats);
  p.b_stage = reinterpret_cast<const float*>(aux + al.off_bias);
  p.dw_in = grad_weight_out;
  p.db_in = grad_bias_out;
  p.d_w = grad_weight;
  p.d_b = grad_bias;
  p.d_lr = grad_ttt_lr_eta;
  p.part_ln = ws + wl.off_ln;
  p.part_te = ws + wl.off_te;
  p.part_w = (outer_grad_packed != nullptr) ? ws + wl.off_w : nullptr;
  p.handoff = ws + wl.off_handoff;
  p.sched = reinterpret_cast<int*>(ws + wl.off_sched);
  p.CH = kBwdChunkStages;
  p.NCH = wl.nch;
  p.nstreams = (int)pk.streams;
  p.handoff_polls = g_handoff_polls.load();
  p.item_base = g_item_base.load();
  p.status = static_cast<uint32_t*>(status);
  p.H = pk.heads;
  p.T = d->seq_len;
  p.NS = d->seq_len / d->mini_batch;
  p.K = d->checkpoint_interval;
  p.NCK = (int)num_ckpt(d);
  p.eps = d->epsilon;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = ttt::launch_linear_bwd(d->dtype, pk.seg, d->mini_batch, maps, bases, p, (int)pk.streams, st);
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "backward launch failed: %s", cudaGetErrorString(e));
  ttt::ReduceParams r;
  r.part_ln = p.part_ln;
  r.part_te = p.part_te;
  r.part_w = p.part_w;
  r.d_token_eta = grad_token_eta;
  r.d_ln_g = grad_ln_weight;
  r.d_ln_b = grad_ln_bias;
  r.packed = outer_grad_packed;
  r.B = d->batch;
  r.H = d->heads;
  r.F = d->head_dim;
  r.mb = d->mini_batch;
  r.T = d->seq_len;
  r.NCH = wl.nch;
  e = ttt::launch_linear_bwd_reduce(r, st);
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "backward reduction launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

int ttt_mlp_forward(const ttt_dims* d, const void* xq, const void* xk, const void* xv, const void* w1, const void* b1,
                    const void* w2, const void* b2, const void* token_eta, const void* ttt_lr_eta,
                    const void* ln_weight, const void* ln_bias, void* output, void* w1_out, void* b1_out, void* w2_out,
                    void* b2_out, void* backward_workspace, size_t backward_workspace_bytes, void* status,
                    void* stream) {
  int rc = check_dims(d);
  if (rc != TTT_OK) return rc;
  if (d->dtype != TTT_BF16) return fail(TTT_ERR_UNSUPPORTED, "the TTT-MLP kernel is built for bf16 only");
  const MlpWsLayout wl = mlp_ws_layout(d);
  if (backward_workspace != nullptr) {
    if (backward_workspace_bytes < wl.total_bytes)
      return fail(TTT_ERR_WORKSPACE, "backward workspace of %zu bytes needed, %zu given", wl.total_bytes,
                  backward_workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(backward_workspace) & 15u) != 0)
      return fail(TTT_ERR_ALIGN, "backward workspace is not 16-byte aligned");
  }
  const NamedPtr ptrs[] = {{"xq", xq}, {"xk", xk}, {"xv", xv}, {"w1", w1}, {"b1", b1}, {"w2", w2}, {"b2", b2},
                           {"token_eta", token_eta}, {"ttt_lr_eta", ttt_lr_eta}, {"ln_weight", ln_weight},
                           {"ln_bias", ln_bias}, {"output", output}, {"w1_out", w1_out}, {"b1_out", b1_out},
                           {"w2_out", w2_out}, {"b2_out", b2_out}};
  rc = check_ptrs(ptrs, sizeof(ptrs) / sizeof(ptrs[0]));
  if (rc != TTT_OK) return rc;
  const int64_t rows = (int64_t)d->batch * d->heads * d->seq_len;
  CUtensorMap maps[4];
  const void* bases[4] = {xq, xk, xv, output};
  for (int i = 0; i < 4; ++i) {
    rc = make_tile_map(&maps[i], bases[i], rows, d->dtype);
    if (rc != TTT_OK) return rc;
  }
  ttt::MlpFwdParams p;
  p.w1 = w1; p.b1 = b1; p.w2 = w2; p.b2 = b2;
  p.token_eta = token_eta; p.lr = ttt_lr_eta; p.ln_g = ln_weight; p.ln_b = ln_bias;
  p.w1_out = w1_out; p.b1_out = b1_out; p.w2_out = w2_out; p.b2_out = b2_out;
  p.status = static_cast<uint32_t*>(status);
  p.bwd_ws = static_cast<float*>(backward_workspace);
  p.bwd_ws_stride = wl.stride_floats;
  // with a workspace the launch is persistent and uses the workspace's scheduler words (the backward re-zeroes them)
  p.sched = backward_workspace != nullptr ? reinterpret_cast<int*>(static_cast<float*>(backward_workspace) + wl.off_sched)
                                          : nullptr;
  p.nstreams = d->batch * d->heads;
  p.CH = p.NCH = 0;
  p.handoff_polls = g_handoff_polls.load();
  p.H = d->heads; p.T = d->seq_len; p.NS = d->seq_len / d->mini_batch; p.eps = d->epsilon;
  cudaError_t e = ttt::launch_mlp_fwd(maps, p, d->batch * d->heads, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "MLP forward launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

}  // extern "C"

// ----------------------------------------------------------------------------------------------------
// Backward for callers that cannot hand over a workspace.
//
// Some hosts of this operator have no way to obtain device memory at the point where the backward runs: a
// custom-operator hook that is given only the input and output buffers of the op, a runtime whose memory pool
// already owns the whole device so that a side allocation would fail or fragment it, or a latency-sensitive
// training loop that forbids cudaMalloc on the hot path because it synchronises the device.  For them the
// per-stream partial sums live in the array below instead of a caller-supplied workspace.
//
// The array is part of the library image: every GPU on which the library is used keeps these bytes resident
// until the process exits.  Its name is only a host-side handle; the device address is looked up once per
// device with cudaGetSymbolAddress (with that device current) and it is that address the kernels receive.
// ----------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_noalloc_scratch[TTT_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kMaxDevices] = {};

int noalloc_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(TTT_ERR_CUDA, "device ordinal %d outside [0, %d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(TTT_ERR_CUDA, "cudaGetSymbolAddress(built-in scratch) failed on device %d: %s", dev,
                  cudaGetErrorString(e));
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return TTT_OK;
}
}  // namespace

extern "C" int ttt_linear_backward_noalloc(const ttt_dims* d, const void* xq, const void* xk, const void* xv,
                                           const void* weight, const void* bias, const void* token_eta,
                                           const void* ttt_lr_eta, const void* ln_weight, const void* ln_bias,
                                           const void* weight_ckpt, const void* bias_ckpt, const void* grad_output,
                                           void* grad_xq, void* grad_xk, void* grad_xv, void* grad_weight,
                                           void* grad_bias, void* grad_ttt_lr_eta, float* grad_token_eta,
                                           float* grad_ln_weight, float* grad_ln_bias, float* outer_grad_packed,
                                           void* status, void* stream) {
  int rc = check_dims(d, true);
  if (rc != TTT_OK) return rc;
  const size_t need = ws_layout(d).total_bytes;
  if (need > (size_t)TTT_NOALLOC_SCRATCH_BYTES)
    return fail(TTT_ERR_WORKSPACE,
                "this problem needs %zu bytes of scratch but the built-in scratch holds %zu "
                "(about batch*heads*(1.5*seq_len + 12420)*4 bytes are needed): call ttt_linear_backward with a workspace",
                need, (size_t)TTT_NOALLOC_SCRATCH_BYTES);
  void* scratch = nullptr;
  rc = noalloc_scratch(&scratch);
  if (rc != TTT_OK) return rc;
  // Nothing in the scratch has to start at zero: the backward kernel overwrites every partial it later reads.
  return ttt_linear_backward(d, xq, xk, xv, weight, bias, token_eta, ttt_lr_eta, ln_weight, ln_bias, weight_ckpt,
                             bias_ckpt, grad_output, grad_xq, grad_xk, grad_xv, grad_weight, grad_bias,
                             grad_ttt_lr_eta, grad_token_eta, grad_ln_weight, grad_ln_bias, outer_grad_packed,
                             scratch, (size_t)TTT_NOALLOC_SCRATCH_BYTES, status, stream);
}

namespace {
int check_layer_dims(const ttt_dims* d) {
  if (d == nullptr) return fail(TTT_ERR_NULL, "dims is null");
  if (d->batch <= 0 || d->heads <= 0 || d->seq_len <= 0) return fail(TTT_ERR_SHAPE, "batch, heads and seq_len must be positive");
  if (d->dtype != TTT_F32 && d->dtype != TTT_BF16) return fail(TTT_ERR_UNSUPPORTED, "unknown dtype %d", d->dtype);
  if (d->head_dim != 64 && d->head_dim != 32)
    return fail(TTT_ERR_UNSUPPORTED, "Unsupported head_dim=%d (supported: 64, 32)", d->head_dim);
  if ((int64_t)d->batch * d->heads * d->seq_len >= (int64_t)1 << 31)
    return fail(TTT_ERR_SHAPE, "batch*heads*seq_len must be below 2^31");
  return TTT_OK;
}
}  // namespace

extern "C" int ttt_layer_prologue(const ttt_dims* d, const void* q_src, const void* k_src, const void* v_src,
                                  int64_t src_ld, const void* lr_logits, int64_t lr_ld, const void* lr_bias,
                                  const void* conv_q_weight, const void* conv_q_bias, const void* conv_k_weight,
                                  const void* conv_k_bias, int conv_kernel, int start_idx, int rope_mode,
                                  float rope_theta, float base_lr, void* xq, void* xk, void* xv, void* ttt_lr_eta,
                                  void* stream) {
  int rc = check_layer_dims(d);
  if (rc != TTT_OK) return rc;
  const bool conv = conv_q_weight != nullptr;
  if (conv != (conv_k_weight != nullptr) || conv != (conv_q_bias != nullptr) || conv != (conv_k_bias != nullptr))
    return fail(TTT_ERR_NULL, "conv_q_weight, conv_q_bias, conv_k_weight and conv_k_bias must be given together");
  if (conv && (conv_kernel < 1 || conv_kernel > 4))
    return fail(TTT_ERR_UNSUPPORTED, "conv_kernel=%d (supported: 1..4)", conv_kernel);
  if (rope_mode < 0 || rope_mode > 2) return fail(TTT_ERR_UNSUPPORTED, "rope_mode=%d (0 none, 1 wrapped, 2 global)", rope_mode);
  if (rope_mode == 1 && (d->mini_batch < 1 || d->mini_batch > 64))
    return fail(TTT_ERR_UNSUPPORTED, "wrapped rotary positions need 1 <= mini_batch <= 64 (got %d)", d->mini_batch);
  if (rope_mode != 0 && !(rope_theta > 0.f)) return fail(TTT_ERR_SHAPE, "rope_theta must be positive");
  if (start_idx < 0) return fail(TTT_ERR_SHAPE, "start_idx must be >= 0");
  const int64_t cols = (int64_t)d->heads * d->head_dim;
  if (src_ld < cols || (src_ld & 7) != 0)
    return fail(TTT_ERR_SHAPE, "src_ld (%lld) must be >= heads*head_dim and a multiple of 8", (long long)src_ld);
  if (lr_ld < d->heads) return fail(TTT_ERR_SHAPE, "lr_ld (%lld) must be >= heads", (long long)lr_ld);
  const NamedPtr ptrs[] = {{"q_src", q_src}, {"k_src", conv ? q_src : k_src}, {"v_src", v_src}, {"xq", xq},
                           {"xk", xk},       {"xv", xv}};
  rc = check_ptrs(ptrs, 6);
  if (rc != TTT_OK) return rc;
  if (lr_logits == nullptr || ttt_lr_eta == nullptr) return fail(TTT_ERR_NULL, "lr_logits / ttt_lr_eta is null");
  ttt::LayerProParams p;
  p.q_src = q_src;
  p.k_src = conv ? q_src : k_src;
  p.v_src = v_src;
  p.ld_src = (long)src_ld;
  p.lr_logits = lr_logits;
  p.ld_lr = (long)lr_ld;
  p.lr_bias = lr_bias;
  p.conv_q_w = conv_q_weight;
  p.conv_q_b = conv_q_bias;
  p.conv_k_w = conv_k_weight;
  p.conv_k_b = conv_k_bias;
  p.conv_k = conv ? conv_kernel : 0;
  p.xq = xq;
  p.xk = xk;
  p.xv = xv;
  p.lr_out = ttt_lr_eta;
  p.B = d->batch;
  p.H = d->heads;
  p.T = d->seq_len;
  p.start_idx = start_idx;
  p.pos_mod = rope_mode == 1 ? d->mini_batch : 1;
  p.rope_mode = rope_mode;
  p.rope_theta = rope_mode != 0 ? rope_theta : 1.f;
  p.base_lr = base_lr;
  cudaError_t e = ttt::launch_layer_prologue(d->dtype, d->head_dim, p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "layer prologue launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

extern "C" int ttt_layer_epilogue(const ttt_dims* d, const void* inner_out, const void* gate, int64_t gate_ld,
                                  const void* post_norm_weight, const void* post_norm_bias, float eps, void* y,
                                  void* stream) {
  int rc = check_layer_dims(d);
  if (rc != TTT_OK) return rc;
  if (d->heads * d->head_dim > 2048)
    return fail(TTT_ERR_UNSUPPORTED, "heads*head_dim=%d (supported: up to 2048)", d->heads * d->head_dim);
  if (!(eps >= 0.f)) return fail(TTT_ERR_SHAPE, "eps must be >= 0");
  const NamedPtr ptrs[] = {{"inner_out", inner_out}, {"y", y}};
  rc = check_ptrs(ptrs, 2);
  if (rc != TTT_OK) return rc;
  if (post_norm_weight == nullptr || post_norm_bias == nullptr) return fail(TTT_ERR_NULL, "post_norm_weight / post_norm_bias is null");
  if (gate != nullptr) {
    if (gate_ld < (int64_t)d->heads * d->head_dim || (gate_ld & 3) != 0)
      return fail(TTT_ERR_SHAPE, "gate_ld (%lld) must be >= heads*head_dim and a multiple of 4", (long long)gate_ld);
    if ((reinterpret_cast<uintptr_t>(gate) & 7u) != 0) return fail(TTT_ERR_ALIGN, "gate is not 8-byte aligned");
  }
  ttt::LayerEpiParams p;
  p.inner_out = inner_out;
  p.gate = gate;
  p.ld_gate = (long)gate_ld;
  p.ln_w = post_norm_weight;
  p.ln_b = post_norm_bias;
  p.y = y;
  p.B = d->batch;
  p.H = d->heads;
  p.T = d->seq_len;
  p.eps = eps;
  cudaError_t e = ttt::launch_layer_epilogue(d->dtype, d->head_dim, p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "layer epilogue launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

extern "C" int ttt_linear_forward_partial(const ttt_dims* d, const void* xq, const void* xk, const void* xv,
                                          const void* weight, const void* bias, const void* token_eta,
                                          const void* ttt_lr_eta, const void* ln_weight, const void* ln_bias,
                                          void* output, void* weight_out, void* bias_out, void* stream) {
  if (d == nullptr) return fail(TTT_ERR_NULL, "dims is null");
  if (d->batch <= 0 || d->heads <= 0) return fail(TTT_ERR_SHAPE, "batch and heads must be positive");
  if (d->dtype != TTT_F32 && d->dtype != TTT_BF16) return fail(TTT_ERR_UNSUPPORTED, "unknown dtype %d", d->dtype);
  if (d->head_dim != 64 && d->head_dim != 32)
    return fail(TTT_ERR_UNSUPPORTED, "Unsupported head_dim=%d (supported: 64, 32)", d->head_dim);
  if (d->seq_len < 1 || d->seq_len > 16)
    return fail(TTT_ERR_SHAPE, "a partial mini-batch has 1..16 tokens (got seq_len=%d)", d->seq_len);
  if (!(d->epsilon >= 0.f)) return fail(TTT_ERR_SHAPE, "epsilon must be >= 0");
  const NamedPtr ptrs[] = {{"xq", xq},         {"xk", xk},         {"xv", xv},
                           {"weight", weight}, {"bias", bias},     {"token_eta", token_eta},
                           {"ttt_lr_eta", ttt_lr_eta}, {"ln_weight", ln_weight}, {"ln_bias", ln_bias},
                           {"output", output}, {"weight_out", weight_out}, {"bias_out", bias_out}};
  for (const NamedPtr& np : ptrs)
    if (np.p == nullptr) return fail(TTT_ERR_NULL, "%s is null", np.name);
  ttt::LinPartialParams p;
  p.xq = xq;
  p.xk = xk;
  p.xv = xv;
  p.w0 = weight;
  p.b0 = bias;
  p.token_eta = token_eta;
  p.lr = ttt_lr_eta;
  p.ln_g = ln_weight;
  p.ln_b = ln_bias;
  p.out = output;
  p.w_out = weight_out;
  p.b_out = bias_out;
  p.H = d->heads;
  p.R = d->seq_len;
  p.eps = d->epsilon;
  cudaError_t e = ttt::launch_linear_partial(d->dtype, d->head_dim, p, d->batch * d->heads, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "partial forward launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

extern "C" int ttt_layer_prologue_backward(const ttt_dims* d, const void* grad_xq, const void* grad_xk,
                                           const void* grad_xv, const void* grad_ttt_lr_eta, const void* ttt_lr_eta,
                                           int start_idx, int rope_mode, float rope_theta, float base_lr,
                                           void* grad_q_dst, void* grad_k_dst, void* grad_v_dst, int64_t dst_ld,
                                           void* grad_lr_logits, int64_t lr_ld, int lr_cols, void* stream) {
  int rc = check_layer_dims(d);
  if (rc != TTT_OK) return rc;
  if (rope_mode < 0 || rope_mode > 2) return fail(TTT_ERR_UNSUPPORTED, "rope_mode=%d (0 none, 1 wrapped, 2 global)", rope_mode);
  if (rope_mode == 1 && (d->mini_batch < 1 || d->mini_batch > 64))
    return fail(TTT_ERR_UNSUPPORTED, "wrapped rotary positions need 1 <= mini_batch <= 64 (got %d)", d->mini_batch);
  if (rope_mode != 0 && !(rope_theta > 0.f)) return fail(TTT_ERR_SHAPE, "rope_theta must be positive");
  if (start_idx < 0) return fail(TTT_ERR_SHAPE, "start_idx must be >= 0");
  if (!(base_lr != 0.f)) return fail(TTT_ERR_SHAPE, "base_lr must be non-zero");
  if (dst_ld < (int64_t)d->heads * d->head_dim || (dst_ld & 7) != 0)
    return fail(TTT_ERR_SHAPE, "dst_ld (%lld) must be >= heads*head_dim and a multiple of 8", (long long)dst_ld);
  if (lr_cols < d->heads || lr_ld < lr_cols)
    return fail(TTT_ERR_SHAPE, "need heads <= lr_cols <= lr_ld (got lr_cols=%d, lr_ld=%lld)", lr_cols, (long long)lr_ld);
  const NamedPtr ptrs[] = {{"grad_xq", grad_xq},       {"grad_xk", grad_xk},       {"grad_xv", grad_xv},
                           {"grad_q_dst", grad_q_dst}, {"grad_k_dst", grad_k_dst}, {"grad_v_dst", grad_v_dst}};
  rc = check_ptrs(ptrs, 6);
  if (rc != TTT_OK) return rc;
  if (grad_ttt_lr_eta == nullptr || ttt_lr_eta == nullptr || grad_lr_logits == nullptr)
    return fail(TTT_ERR_NULL, "grad_ttt_lr_eta / ttt_lr_eta / grad_lr_logits is null");
  ttt::LayerProBwdParams p;
  p.dxq = grad_xq;
  p.dxk = grad_xk;
  p.dxv = grad_xv;
  p.dlr = grad_ttt_lr_eta;
  p.lr = ttt_lr_eta;
  p.dq_dst = grad_q_dst;
  p.dk_dst = grad_k_dst;
  p.dv_dst = grad_v_dst;
  p.ld_dst = (long)dst_ld;
  p.dlogits_dst = grad_lr_logits;
  p.ld_dlr = (long)lr_ld;
  p.lr_cols = lr_cols;
  p.B = d->batch;
  p.H = d->heads;
  p.T = d->seq_len;
  p.start_idx = start_idx;
  p.pos_mod = rope_mode == 1 ? d->mini_batch : 1;
  p.rope_mode = rope_mode;
  p.rope_theta = rope_mode != 0 ? rope_theta : 1.f;
  p.base_lr = base_lr;
  cudaError_t e = ttt::launch_layer_prologue_bwd(d->dtype, d->head_dim, p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "layer prologue backward launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

extern "C" int ttt_layer_qk_conv(const ttt_dims* d, const void* x, int64_t x_ld, const void* conv_q_weight,
                                 const void* conv_q_bias, const void* conv_k_weight, const void* conv_k_bias, void* q,
                                 void* k, void* stream) {
  int rc = check_layer_dims(d);
  if (rc != TTT_OK) return rc;
  const int64_t C = (int64_t)d->heads * d->head_dim;
  if (x_ld < C || (x_ld & 7) != 0)
    return fail(TTT_ERR_SHAPE, "x_ld (%lld) must be >= heads*head_dim and a multiple of 8", (long long)x_ld);
  const NamedPtr ptrs[] = {{"x", x}, {"q", q}, {"k", k}};
  rc = check_ptrs(ptrs, 3);
  if (rc != TTT_OK) return rc;
  if (conv_q_weight == nullptr || conv_q_bias == nullptr || conv_k_weight == nullptr || conv_k_bias == nullptr)
    return fail(TTT_ERR_NULL, "a convolution weight or bias is null");
  ttt::LayerConvParams p;
  p.x = x; p.ld_x = (long)x_ld; p.wq = conv_q_weight; p.bq = conv_q_bias; p.wk = conv_k_weight; p.bk = conv_k_bias;
  p.q = q; p.k = k; p.B = d->batch; p.T = d->seq_len; p.C = (int)C;
  cudaError_t e = ttt::launch_layer_conv(d->dtype, p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "shared-QK convolution launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

extern "C" size_t ttt_layer_qk_conv_backward_workspace_bytes(const ttt_dims* d) {
  if (check_layer_dims(d) != TTT_OK) return 0;
  const size_t nch = ((size_t)d->seq_len + ttt::LAYER_CONV_CHUNK - 1) / ttt::LAYER_CONV_CHUNK;
  return (size_t)d->batch * nch * 10 * (size_t)d->heads * d->head_dim * sizeof(float);
}

extern "C" int ttt_layer_qk_conv_backward(const ttt_dims* d, const void* grad_q, const void* grad_k, const void* x,
                                          int64_t x_ld, const void* conv_q_weight, const void* conv_k_weight,
                                          void* grad_x, float* grad_q_params, float* grad_k_params, void* workspace,
                                          size_t workspace_bytes, void* stream) {
  int rc = check_layer_dims(d);
  if (rc != TTT_OK) return rc;
  const int64_t C = (int64_t)d->heads * d->head_dim;
  if (x_ld < C || (x_ld & 7) != 0)
    return fail(TTT_ERR_SHAPE, "x_ld (%lld) must be >= heads*head_dim and a multiple of 8", (long long)x_ld);
  const NamedPtr ptrs[] = {{"grad_q", grad_q}, {"grad_k", grad_k}, {"x", x}, {"grad_x", grad_x}};
  rc = check_ptrs(ptrs, 4);
  if (rc != TTT_OK) return rc;
  if (conv_q_weight == nullptr || conv_k_weight == nullptr || grad_q_params == nullptr || grad_k_params == nullptr)
    return fail(TTT_ERR_NULL, "a convolution weight or parameter-gradient buffer is null");
  const size_t need = ttt_layer_qk_conv_backward_workspace_bytes(d);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TTT_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return fail(TTT_ERR_ALIGN, "workspace is not 16-byte aligned");
  ttt::LayerConvBwdParams p;
  p.dq = grad_q; p.dk = grad_k; p.x = x; p.ld_x = (long)x_ld; p.wq = conv_q_weight; p.wk = conv_k_weight;
  p.dx = grad_x; p.partials = static_cast<float*>(workspace); p.dparams_q = grad_q_params; p.dparams_k = grad_k_params;
  p.B = d->batch; p.T = d->seq_len; p.C = (int)C;
  cudaError_t e = ttt::launch_layer_conv_bwd(d->dtype, p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "shared-QK convolution backward launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}

extern "C" size_t ttt_layer_epilogue_backward_workspace_bytes(const ttt_dims* d) {
  if (check_layer_dims(d) != TTT_OK || d->heads * d->head_dim > 2048) return 0;
  return ttt::layer_epilogue_bwd_workspace_bytes(d->batch, d->heads, d->seq_len, d->head_dim);
}

extern "C" int ttt_layer_epilogue_backward(const ttt_dims* d, const void* grad_y, const void* inner_out,
                                           const void* gate, int64_t gate_ld, const void* post_norm_weight,
                                           const void* post_norm_bias, float eps, void* grad_inner_out,
                                           void* grad_gate, int64_t grad_gate_ld, float* grad_post_norm_weight,
                                           float* grad_post_norm_bias, void* workspace, size_t workspace_bytes,
                                           void* stream) {
  int rc = check_layer_dims(d);
  if (rc != TTT_OK) return rc;
  if (d->heads * d->head_dim > 2048)
    return fail(TTT_ERR_UNSUPPORTED, "heads*head_dim=%d (supported: up to 2048)", d->heads * d->head_dim);
  if (!(eps >= 0.f)) return fail(TTT_ERR_SHAPE, "eps must be >= 0");
  const NamedPtr ptrs[] = {{"grad_y", grad_y}, {"inner_out", inner_out}, {"grad_inner_out", grad_inner_out}};
  rc = check_ptrs(ptrs, 3);
  if (rc != TTT_OK) return rc;
  if (post_norm_weight == nullptr || post_norm_bias == nullptr || grad_post_norm_weight == nullptr ||
      grad_post_norm_bias == nullptr)
    return fail(TTT_ERR_NULL, "post_norm_weight / post_norm_bias / their gradients must not be null");
  if (gate != nullptr) {
    if (grad_gate == nullptr) return fail(TTT_ERR_NULL, "grad_gate is null although a gate is given");
    const int64_t cols = (int64_t)d->heads * d->head_dim;
    if (gate_ld < cols || (gate_ld & 3) != 0 || grad_gate_ld < cols || (grad_gate_ld & 3) != 0)
      return fail(TTT_ERR_SHAPE, "gate_ld / grad_gate_ld must be >= heads*head_dim and multiples of 4");
    if ((reinterpret_cast<uintptr_t>(gate) & 7u) != 0 || (reinterpret_cast<uintptr_t>(grad_gate) & 7u) != 0)
      return fail(TTT_ERR_ALIGN, "gate / grad_gate is not 8-byte aligned");
  }
  const size_t need = ttt_layer_epilogue_backward_workspace_bytes(d);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TTT_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  ttt::LayerEpiBwdParams p;
  p.dy = grad_y;
  p.inner_out = inner_out;
  p.gate = gate;
  p.ld_gate = (long)gate_ld;
  p.ln_w = post_norm_weight;
  p.ln_b = post_norm_bias;
  p.d_inner = grad_inner_out;
  p.dgate = grad_gate;
  p.ld_dgate = (long)grad_gate_ld;
  p.d_ln_w = grad_post_norm_weight;
  p.d_ln_b = grad_post_norm_bias;
  p.partials = static_cast<float*>(workspace);
  p.row_stats = nullptr;
  p.B = d->batch;
  p.H = d->heads;
  p.T = d->seq_len;
  p.eps = eps;
  cudaError_t e = ttt::launch_layer_epilogue_bwd(d->dtype, d->head_dim, p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "layer epilogue backward launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}


extern "C" size_t ttt_mlp_backward_workspace_bytes(const ttt_dims* d) {
  if (check_dims(d) != TTT_OK || d->dtype != TTT_BF16) return 0;
  return mlp_ws_layout(d).total_bytes;
}

extern "C" int ttt_mlp_backward(const ttt_dims* d, const void* xq, const void* xk, const void* xv, const void* w1,
                                const void* b1, const void* w2, const void* b2, const void* token_eta,
                                const void* ttt_lr_eta, const void* ln_weight, const void* ln_bias,
                                const void* grad_output, void* grad_xq, void* grad_xk, void* grad_xv, void* grad_w1,
                                void* grad_b1, void* grad_w2, void* grad_b2, void* grad_ttt_lr_eta,
                                float* grad_token_eta, float* grad_ln_weight, float* grad_ln_bias, void* workspace,
                                size_t workspace_bytes, int workspace_from_forward, void* status, void* stream) {
  int rc = check_dims(d);
  if (rc != TTT_OK) return rc;
  if (d->dtype != TTT_BF16) return fail(TTT_ERR_UNSUPPORTED, "the TTT-MLP kernels are built for bf16 only");
  const NamedPtr ptrs[] = {{"xq", xq}, {"xk", xk}, {"xv", xv}, {"w1", w1}, {"b1", b1}, {"w2", w2}, {"b2", b2},
                           {"token_eta", token_eta}, {"ttt_lr_eta", ttt_lr_eta}, {"ln_weight", ln_weight},
                           {"ln_bias", ln_bias}, {"grad_output", grad_output}, {"grad_xq", grad_xq},
                           {"grad_xk", grad_xk}, {"grad_xv", grad_xv}, {"grad_w1", grad_w1}, {"grad_b1", grad_b1},
                           {"grad_w2", grad_w2}, {"grad_b2", grad_b2}, {"grad_ttt_lr_eta", grad_ttt_lr_eta},
                           {"grad_token_eta", grad_token_eta}, {"grad_ln_weight", grad_ln_weight},
                           {"grad_ln_bias", grad_ln_bias}};
  for (const NamedPtr& np : ptrs)
    if (np.p == nullptr) return fail(TTT_ERR_NULL, "%s is null", np.name);
  const MlpWsLayout l = mlp_ws_layout(d);
  if (workspace == nullptr || workspace_bytes < l.total_bytes)
    return fail(TTT_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", l.total_bytes, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return fail(TTT_ERR_ALIGN, "workspace is not 16-byte aligned");
  float* ws = static_cast<float*>(workspace);
  ttt::MlpBwdParams p;
  p.xq = xq; p.xk = xk; p.xv = xv; p.w1 = w1; p.b1 = b1; p.w2 = w2; p.b2 = b2;
  p.token_eta = token_eta; p.lr = ttt_lr_eta; p.ln_g = ln_weight; p.ln_b = ln_bias; p.d_out = grad_output;
  p.d_q = grad_xq; p.d_k = grad_xk; p.d_v = grad_xv; p.d_w1 = grad_w1; p.d_b1 = grad_b1; p.d_w2 = grad_w2;
  p.d_b2 = grad_b2; p.d_lr = grad_ttt_lr_eta; p.d_token_eta = grad_token_eta; p.d_ln_g = grad_ln_weight;
  p.d_ln_b = grad_ln_bias;
  p.workspace = ws;
  p.ws_stride = l.stride_floats;
  p.part_te = ws + l.off_te;
  p.part_ln = ws + l.off_ln;
  p.sched = reinterpret_cast<int*>(ws + l.off_sched);
  p.pass1_done = workspace_from_forward != 0;
  p.status = static_cast<uint32_t*>(status);
  p.trace = static_cast<unsigned int*>(status);  // instrumented builds write 16 words of cycle counts here instead
  p.H = d->heads; p.T = d->seq_len; p.NS = d->seq_len / d->mini_batch; p.eps = d->epsilon;
  cudaError_t e = ttt::launch_mlp_bwd(p, d->batch, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TTT_ERR_CUDA, "MLP backward launch failed: %s", cudaGetErrorString(e));
  return TTT_OK;
}
