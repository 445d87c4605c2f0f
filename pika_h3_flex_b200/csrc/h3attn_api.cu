// C-ABI entry points of libh3attn.so: argument validation, TMA tensor maps, kernel launches and the
// host-side block-index builder.  Declarations and per-function contracts live in include/h3attn.h.
#include "../../include/h3attn.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "attn_fwd.cuh"
#include "attn_fwd_pair.cuh"
#include "qk_prep.cuh"
#include "qkv_proj.cuh"
#include "adaln.cuh"

namespace {

using h3a::AttnArgs;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// x[l*stride_l + h*stride_h + c]: dims (128, L, H); box = (box_inner, box_rows, 1 head), 128-byte swizzle.
int32_t make_map(CUtensorMap* m, const void* ptr, bool fp8, int64_t L, int64_t H, int64_t stride_l, int64_t stride_h,
                 uint32_t box_rows = 128) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return H3A_ERR_DRIVER;
  const int64_t es = fp8 ? 1 : 2;
  if (!aligned16(ptr) || (stride_l * es) % 16 != 0 || (stride_h * es) % 16 != 0) return H3A_ERR_ALIGN;
  if (stride_l <= 0 || stride_h <= 0) return H3A_ERR_ARG;
  cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(L), static_cast<cuuint64_t>(H)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(stride_l * es), static_cast<cuuint64_t>(stride_h * es)};
  cuuint32_t box[3] = {fp8 ? 128u : 64u, box_rows, 1u};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? H3A_OK : H3A_ERR_LAUNCH;
}

// m[r * stride + c], c < inner (contiguous), r < rows: box = 64 columns x 128 rows of bf16, 128-byte swizzle.
int32_t make_map2d(CUtensorMap* m, const void* ptr, int64_t inner, int64_t rows, int64_t stride) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return H3A_ERR_DRIVER;
  if (!aligned16(ptr) || (stride * 2) % 16 != 0) return H3A_ERR_ALIGN;
  if (stride < inner || inner <= 0 || rows <= 0) return H3A_ERR_ARG;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(stride * 2)};
  cuuint32_t box[2] = {64u, 128u};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? H3A_OK : H3A_ERR_LAUNCH;
}

int32_t check_arch() {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return H3A_ERR_LAUNCH;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return H3A_ERR_LAUNCH;
  return major == 10 ? H3A_OK : H3A_ERR_ARCH;
}

int32_t validate_attn(const h3a_attn_params* p) {
  if (!p || !p->q || !p->k || !p->v || !p->o) return H3A_ERR_ARG;
  if (p->d != 128 || p->B != 1) return H3A_ERR_SHAPE;
  if (p->Lq <= 0 || p->Lk <= 0 || p->H <= 0) return H3A_ERR_SHAPE;
  if (p->mode < H3A_MODE_DENSE_BF16 || p->mode > H3A_MODE_BLOCK_SPARSE) return H3A_ERR_ARG;
  if (p->mode == H3A_MODE_FP8_QK && (!p->q_scale || !p->k_scale)) return H3A_ERR_ARG;
  if (p->mode == H3A_MODE_BLOCK_SPARSE && (!p->row_ptr || !p->col_idx || p->nnz < 0)) return H3A_ERR_ARG;
  if (!aligned16(p->o) || (p->o_stride_l % 8) != 0 || (p->o_stride_h % 8) != 0) return H3A_ERR_ALIGN;
  if (p->o_stride_l <= 0 || p->o_stride_h <= 0) return H3A_ERR_ARG;
  if (p->o_n_ranks < 0 || p->o_n_ranks > H3A_MAX_RANKS) return H3A_ERR_ARG;
  if (p->o_n_ranks > 1) {
    if (p->o_rank_rows <= 0 || static_cast<int64_t>(p->o_rank_rows) * p->o_n_ranks < p->Lq) return H3A_ERR_SHAPE;
    for (int r = 0; r < p->o_n_ranks; ++r) {
      if (!p->o_rank_base[r]) return H3A_ERR_ARG;
      if (!aligned16(p->o_rank_base[r])) return H3A_ERR_ALIGN;
    }
  }
  return H3A_OK;
}

size_t sparse_workspace_bytes(const h3a_attn_params* p) {
  const size_t n_qpairs = (static_cast<size_t>(p->Lq) + 255) / 256;
  // plan entries (one per kept tile at most) followed by one count per query-tile pair
  return (static_cast<size_t>(p->nnz) + n_qpairs) * sizeof(int32_t);
}

constexpr int kMaxDevices = 64;

int sm_count_of_current_device();
// Persistent CTAs for the single-CTA kernel with a fixed softmax reference: one CTA per SM walks the (head, query
// tile pair) items, so that barriers, TMEM and the K/V ring are set up once per SM and the loads and S MMAs of the
// next item run under the epilogue of the current one.  It pays where an item is short (cross-attention to 512 text
// tokens: 4 key tiles per item).  H3A_PERSIST in the environment, read once: 0 = one CTA per item everywhere,
// 1 = persistent also for block-sparse launches, unset = dense launches only (block-sparse items differ in length
// by up to 30 x, which the hardware's CTA scheduler balances better than a fixed stride does).
int persist_mode() {
  static const int mode = [] {
    const char* e = std::getenv("H3A_PERSIST");
    if (e == nullptr || e[0] == '\0') return 2;
    return e[0] == '0' ? 0 : 1;
  }();
  return mode;
}

template <bool kFp8, bool kSparse, bool kFixed = false>
int32_t launch_attn(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& a, cudaStream_t st) {
  // function attributes belong to a device's context: set them once per device this process launches on
  static std::once_flag once[kMaxDevices];
  static cudaError_t attr_err[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return H3A_ERR_LAUNCH;
  std::call_once(once[dev], [dev] {
    cudaError_t e = cudaFuncSetAttribute(h3a::attn_fwd_kernel<kFp8, kSparse, kFixed>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         h3a::kAttnSmemBytes);
    // the in-kernel register re-allocation would block forever if the launch allocation were smaller
    cudaFuncAttributes fa;
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, h3a::attn_fwd_kernel<kFp8, kSparse, kFixed>);
    if (e == cudaSuccess && fa.numRegs < h3a::AttnLayout<kFixed>::kLaunchRegs) e = cudaErrorLaunchOutOfResources;
    attr_err[dev] = e;
  });
  if (attr_err[dev] != cudaSuccess) return H3A_ERR_LAUNCH;
  unsigned grid = static_cast<unsigned>(a.n_qpairs) * static_cast<unsigned>(a.H);
  if (kFixed) {  // the running-maximum kernel handles one item per CTA
    const int mode = persist_mode();
    const unsigned sms = static_cast<unsigned>(sm_count_of_current_device());
    if (sms > 0 && grid > sms && (mode == 1 || (mode == 2 && !kSparse))) grid = sms;
  }
  h3a::attn_fwd_kernel<kFp8, kSparse, kFixed><<<grid, h3a::AttnLayout<kFixed>::kThreads, h3a::kAttnSmemBytes, st>>>(mq, mk, mv, a);
  return cudaGetLastError() == cudaSuccess ? H3A_OK : H3A_ERR_LAUNCH;
}

// Dense attention with a fixed softmax reference runs on CTA pairs (attn_fwd_pair.cuh).  H3A_PAIR=0 in the
// environment (read once) keeps every launch on the single-CTA kernel, for side-by-side measurements.
// Pairs pay a cluster set-up per CTA; with very few key tiles (cross-attention to 512 text tokens = 4 tiles:
// 0.93 ms on pairs against 0.80 ms) the single-CTA kernel is the faster one.
constexpr int kPairMinKeyTiles = 16;
constexpr double kPairMinDensity = 0.12;

// Fixed softmax reference for a stated logit bound B (logits in [-B, B]).  Every term is 2^((s - ref) log2 e) in fp32
// (bf16 for P: the same exponent range); a row is exact as long as its LARGEST logit satisfies -64 <= s_max - ref <= 74
// (74: room for the row sum and the P V products below 2^127; -64: the row's own terms stay far above the flush-to-zero
// threshold and above the floor 2^-125 at which the polynomial exponential clamps).
//   B <= 30        ref = B        terms <= 1 (the original rule)
//   30 < B <= 60   ref = 60 - B   slides down to 0
//   60 < B <= 74   ref = 0
//   74 < B <= 110  ref = B - 74
// No data within the bound can overflow.  Every row is served while B <= 64 (its largest logit is at least -B); beyond
// that, every row whose largest logit is at least ref - 64 (-28 at B = 110); a row below that line shows in its row sum
// and is REPORTED (H3A_ERR_BOUND), never returned silently.
// Above 110 the line would cross the logits ordinary rows have: the online (running maximum) kernels are used.
constexpr float kMaxLogitBound = 110.f;
bool fixed_reference_ok(float bound) { return bound > 0.f && bound <= kMaxLogitBound; }
float fixed_reference(float bound) {
  if (bound <= 30.f) return bound;
  if (bound <= 60.f) return 60.f - bound;
  if (bound <= 74.f) return 0.f;
  return bound - 74.f;
}

// H3A_SCATTER_BULK=0 in the environment (read once) makes h3a_qk_prep_scatter store rows with ordinary 16-byte
// stores instead of one bulk copy per 128-row tile, for side-by-side measurements.
bool scatter_bulk_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("H3A_SCATTER_BULK");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

// Column tiles per band of the projection's tile order: the band's rows of W (256 x (K + R) bf16 per column tile)
// should stay resident in L2 next to the X and output streams: up to 28 MB (two bands at N = K = 5,120: measured best of 1, 2, 3, 5 and 10 bands).  H3A_PROJ_BAND in the environment (read
// once) overrides the choice, for measurements.
int proj_band_tiles(int n_tiles_n, int k_total) {
  static const int forced = [] {
    const char* e = std::getenv("H3A_PROJ_BAND");
    return e ? std::atoi(e) : 0;
  }();
  if (forced > 0) return std::min(forced, n_tiles_n);
  const long long per_tile = 256ll * k_total * 2;
  const int fit = static_cast<int>(std::max(1ll, (28ll << 20) / std::max(1ll, per_tile)));
  const int n_bands = (n_tiles_n + fit - 1) / fit;
  return (n_tiles_n + n_bands - 1) / n_bands;
}

// Scratch of the two-launch online softmax: a counter (padded to 16 bytes) and one entry per CTA pair.
size_t redo_list_bytes(int64_t Lq, int64_t H) { return (4 + static_cast<size_t>((Lq + 511) / 512 * H)) * sizeof(int); }
// H3A_ONLINE_TWO_LAUNCH=0 in the environment (read once) keeps launches without a logit bound on the running-maximum
// kernel alone, for side-by-side measurements.
bool two_launch_online_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("H3A_ONLINE_TWO_LAUNCH");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

bool pair_kernel_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("H3A_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

// ---- dense launches on CTA pairs: the last, partly filled wave --------------------------------------------
// One pair of CTAs runs per pair of SMs.  When the number of pairs is not a multiple of that, the pairs of the
// last wave are each replaced by S pairs that walk 1/S of the key tiles and leave partial sums in the caller's
// workspace (see AttnArgs::split_begin); a small kernel adds them up.  S minimises the length of that tail.
struct SplitPlan {
  int split_begin = 0, kv_splits = 1, groups = 0;
  size_t bytes = 0;
};

int sm_count_of_current_device() {
  static int cached[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) cached[dev] = n;
  }
  return cached[dev];
}

SplitPlan plan_split(int64_t Lq, int64_t Lk, int64_t H) {
  SplitPlan sp;
  const int sms = sm_count_of_current_device();
  const int64_t wave = sms / 2, total = (Lq + 511) / 512 * H, n_kv = (Lk + 127) / 128;
  sp.split_begin = static_cast<int>(total);
  if (wave <= 0 || total > (1 << 28)) return sp;
  const int64_t rest = total % wave;
  if (rest == 0) return sp;
  const double eps = 4.5 / static_cast<double>(n_kv);  // set-up, partial store and combine, relative to a full pair
  double best = 1.0 + eps;
  int best_s = 1;
  for (int64_t s = 2; s <= 16 && s * 4 <= n_kv && rest * s <= 4 * wave; ++s) {
    const double t = static_cast<double>((rest * s + wave - 1) / wave) * (1.0 / static_cast<double>(s) + eps);
    if (t < best - 0.02) {
      best = t;
      best_s = static_cast<int>(s);
    }
  }
  if (best_s > 1) {
    sp.split_begin = static_cast<int>(total - rest);
    sp.kv_splits = best_s;
    sp.groups = static_cast<int>(rest);
    sp.bytes = static_cast<size_t>(rest) * best_s * (4 * 128 * 128 + 4 * 128) * sizeof(float);
  }
  return sp;
}

// Dense bf16 launches with a logit bound and at most kPairStages / 2 key tiles (cross-attention to a few hundred text
// tokens) keep a head's K / V in the shared memory of a persistent CTA pair (attn_fwd_pair.cuh, kResident), once there
// are at least as many groups of four query tiles as CTA pairs fit the device.  H3A_RESIDENT=0 in the environment
// (read once) sends them to the single-CTA kernel instead, for side-by-side measurements.
bool resident_kernel_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("H3A_RESIDENT");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}
bool resident_kernel_applies(int32_t mode, bool fixed, int64_t Lq, int64_t Lk, int64_t H) {
  if (mode != H3A_MODE_DENSE_BF16 || !fixed || !pair_kernel_enabled() || !resident_kernel_enabled()) return false;
  const int64_t n_kv = (Lk + 127) / 128, items = (Lq + 511) / 512 * H;
  const int sms = sm_count_of_current_device();
  return n_kv >= 1 && n_kv <= h3a::kPairStages / 2 && sms >= 2 && items >= sms / 2;
}

// `mo`: tensor map of the output for the kernels that store through the copy engine (kResident); the others ignore it
template <bool kFp8, bool kSparse = false, bool kFixed = true, bool kRowRef = false, bool kResident = false>
int32_t launch_attn_pair(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& a, cudaStream_t st,
                         const CUtensorMap* mo = nullptr) {
  constexpr int kSmem = kResident ? h3a::kPairResidentSmemBytes : h3a::kPairSmemBytes;
  static std::once_flag once[kMaxDevices];
  static cudaError_t attr_err[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return H3A_ERR_LAUNCH;
  std::call_once(once[dev], [dev] {
    cudaError_t e = cudaFuncSetAttribute(h3a::attn_fwd_pair_kernel<kFp8, kSparse, kFixed, kRowRef, kResident>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmem);
    cudaFuncAttributes fa;
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, h3a::attn_fwd_pair_kernel<kFp8, kSparse, kFixed, kRowRef, kResident>);
    if (e == cudaSuccess && fa.numRegs < h3a::AttnLayout<kFixed>::kLaunchRegs) e = cudaErrorLaunchOutOfResources;
    attr_err[dev] = e;
  });
  if (attr_err[dev] != cudaSuccess) return H3A_ERR_LAUNCH;
  const unsigned n_clusters = static_cast<unsigned>((a.Lq + 511) / 512);
  unsigned pairs = n_clusters * static_cast<unsigned>(a.H);
  const bool split = !kSparse && !kResident && a.kv_splits > 1;
  if (kResident) pairs = std::min(pairs, static_cast<unsigned>(sm_count_of_current_device() / 2));  // persistent: one pair per two SMs
  if (split) pairs = static_cast<unsigned>(a.split_begin) + (pairs - static_cast<unsigned>(a.split_begin)) * static_cast<unsigned>(a.kv_splits);
  h3a::attn_fwd_pair_kernel<kFp8, kSparse, kFixed, kRowRef, kResident><<<2u * pairs, h3a::AttnLayout<kFixed>::kThreads, kSmem, st>>>(mq, mk, mv, mo ? *mo : mq, a);  // cluster shape (2,1,1) is the kernel's
  if (cudaGetLastError() != cudaSuccess) return H3A_ERR_LAUNCH;
  if (split) {
    const unsigned groups = n_clusters * static_cast<unsigned>(a.H) - static_cast<unsigned>(a.split_begin);
    h3a::combine_partials_kernel<<<4u * groups, 256, 0, st>>>(a, static_cast<int>(n_clusters));
    if (cudaGetLastError() != cudaSuccess) return H3A_ERR_LAUNCH;
  }
  return H3A_OK;
}

// ---- static scratch for h3a_attn_fwd_sparse_static -------------------------------------------------------
// One plan entry per kept tile plus one count per query-tile pair, all int32.  1 MiB covers the 768p-like
// sequence (985 x 985 tiles) up to about 27 % density.  Every GPU that loads this library holds the array
// until the process exits.
constexpr size_t kStaticScratchInts = 262144;
static __device__ __align__(256) int32_t g_static_scratch[kStaticScratchInts];

std::mutex g_scratch_mutex;
int32_t* g_scratch_addr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// In host code the name g_static_scratch is only a handle for the runtime, not a device pointer: the address
// a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
int32_t static_scratch_for_current_device(int32_t** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return H3A_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return H3A_ERR_LAUNCH;
    g_scratch_addr[dev] = static_cast<int32_t*>(ptr);
  }
  *out = g_scratch_addr[dev];
  return H3A_OK;
}

// The launch behind h3a_attn_fwd and h3a_attn_fwd_sparse_static: the two differ only in where the scratch comes from.
int32_t attn_fwd_impl(const h3a_attn_params* p, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  int32_t rc = H3A_OK;
  const bool fp8 = p->mode == H3A_MODE_FP8_QK;
  const bool sparse = p->mode == H3A_MODE_BLOCK_SPARSE;

  CUtensorMap mq, mk, mv;
  if ((rc = make_map(&mq, p->q, fp8, p->Lq, p->H, p->q_stride_l, p->q_stride_h)) != H3A_OK) return rc;
  if ((rc = make_map(&mk, p->k, fp8, p->Lk, p->H, p->k_stride_l, p->k_stride_h)) != H3A_OK) return rc;
  if ((rc = make_map(&mv, p->v, false, p->Lk, p->H, p->v_stride_l, p->v_stride_h)) != H3A_OK) return rc;

  AttnArgs a;
  std::memset(&a, 0, sizeof(a));
  a.Lq = p->Lq; a.Lk = p->Lk; a.H = p->H;
  a.nqb = (p->Lq + 127) / 128;
  a.nkb = (p->Lk + 127) / 128;
  a.n_kv_tiles = a.nkb;
  a.n_qpairs = (p->Lq + 255) / 256;
  const float scale = p->softmax_scale > 0.f ? p->softmax_scale : 1.0f / std::sqrt(static_cast<float>(p->d));
  a.scale_log2 = scale * 1.4426950408889634f;
  a.q_scale = p->q_scale; a.k_scale = p->k_scale;
  a.o = static_cast<__nv_bfloat16*>(p->o);
  a.o_stride_l = p->o_stride_l; a.o_stride_h = p->o_stride_h;
  a.lse = p->lse;
  a.status = p->status_word;
  a.wait_ns = p->wait_limit_ns > 0 ? p->wait_limit_ns : 2000000000ll;
  if (p->o_n_ranks > 1) {
    a.o_n_ranks = p->o_n_ranks;
    a.o_rank_rows = p->o_rank_rows;
    for (int r = 0; r < p->o_n_ranks; ++r) a.o_rank[r] = static_cast<__nv_bfloat16*>(p->o_rank_base[r]);
  }
  // fixed softmax reference in log2 units (x softmax_scale is already in the bound): see fixed_reference()
  const bool fixed = fixed_reference_ok(p->logit_bound);
  a.fixed_m = fixed ? fixed_reference(p->logit_bound) * 1.4426950408889634f : 0.f;

  if (sparse) {
    const size_t need = sparse_workspace_bytes(p);
    if (!workspace || workspace_bytes < need) return H3A_ERR_WORKSPACE;
    if (!aligned16(workspace)) return H3A_ERR_ALIGN;
    int32_t* plan = static_cast<int32_t*>(workspace);
    int32_t* plan_cnt = plan + p->nnz;
    const int threads = 128;
    a.row_ptr = p->row_ptr; a.plan = plan; a.plan_cnt = plan_cnt; a.nnz = p->nnz;
    a.heavy_pairs = (p->sparse_heavy_pairs > 0 && p->sparse_heavy_pairs < a.n_qpairs) ? p->sparse_heavy_pairs : 0;
    // A CTA pair computes a key tile for two adjacent query tiles whenever either lists it.  With very sparse
    // neighbourhood masks that duplicated work outweighs what the pair saves (measured: 7 % density, 7 % extra
    // tiles, 3 % slower; 23 % density, 0.4 % extra, 7 % faster), so sparse launches go to pairs from 12 % up.
    const double density = static_cast<double>(p->nnz) / (static_cast<double>(a.nqb) * static_cast<double>(a.nkb));
    if (fixed && pair_kernel_enabled() && density >= kPairMinDensity && a.n_kv_tiles >= kPairMinKeyTiles) {
      // CTA pairs: one merged plan per four query tiles (never longer than the four lists together, and there
      // are no more groups of four than pairs of two, so the same workspace holds it)
      const int n_clusters = (p->Lq + 511) / 512;
      h3a::build_cluster_plan_kernel<<<(n_clusters + threads - 1) / threads, threads, 0, st>>>(p->row_ptr, p->col_idx, a.nqb,
                                                                                              n_clusters, p->nnz, a.nkb, plan, plan_cnt, p->status_word);
      if (cudaGetLastError() != cudaSuccess) return H3A_ERR_LAUNCH;
      if ((rc = make_map(&mk, p->k, false, p->Lk, p->H, p->k_stride_l, p->k_stride_h, h3a::kPairKBoxRows)) != H3A_OK) return rc;
      return launch_attn_pair<false, true>(mq, mk, mv, a, st);
    }
    h3a::build_pair_plan_kernel<<<(a.n_qpairs + threads - 1) / threads, threads, 0, st>>>(p->row_ptr, p->col_idx, a.nqb,
                                                                                         a.n_qpairs, p->nnz, a.nkb, plan, plan_cnt, p->status_word);
    if (cudaGetLastError() != cudaSuccess) return H3A_ERR_LAUNCH;
    return fixed ? launch_attn<false, true, true>(mq, mk, mv, a, st) : launch_attn<false, true, false>(mq, mk, mv, a, st);
  }
  if (resident_kernel_applies(p->mode, fixed, p->Lq, p->Lk, p->H)) {
    a.split_begin = static_cast<int>((p->Lq + 511) / 512 * p->H);
    a.kv_splits = 1;
    if ((rc = make_map(&mk, p->k, false, p->Lk, p->H, p->k_stride_l, p->k_stride_h, h3a::kPairKBoxRows)) != H3A_OK) return rc;
    CUtensorMap mo;  // output rows leave as tile stores of 8 rows x 64 columns (not used when they go to several ranks)
    if ((rc = make_map(&mo, p->o, false, p->Lq, p->H, p->o_stride_l, p->o_stride_h, 8)) != H3A_OK) return rc;
    return launch_attn_pair<false, false, true, false, true>(mq, mk, mv, a, st, &mo);
  }
  if (fixed && pair_kernel_enabled() && a.n_kv_tiles >= kPairMinKeyTiles) {
    a.split_begin = static_cast<int>((p->Lq + 511) / 512 * p->H);
    a.kv_splits = 1;
    if (workspace && aligned16(workspace)) {
      const SplitPlan sp = plan_split(p->Lq, p->Lk, p->H);
      if (sp.kv_splits > 1 && workspace_bytes >= sp.bytes) {
        a.split_begin = sp.split_begin;
        a.kv_splits = sp.kv_splits;
        a.part = static_cast<float*>(workspace);
      }
    }
    // CTA pairs: each CTA stages 32-key boxes of K (its share of every 64-key MMA group) and 64 columns of V
    if ((rc = make_map(&mk, p->k, fp8, p->Lk, p->H, p->k_stride_l, p->k_stride_h, h3a::kPairKBoxRows)) != H3A_OK) return rc;
    return fp8 ? launch_attn_pair<true>(mq, mk, mv, a, st) : launch_attn_pair<false>(mq, mk, mv, a, st);
  }
  if (!fixed && pair_kernel_enabled() && a.n_kv_tiles >= kPairMinKeyTiles) {
    // no usable logit bound: the online softmax, also on CTA pairs; no split of the last wave (partial rows of
    // different references are not directly addable)
    a.split_begin = static_cast<int>((p->Lq + 511) / 512 * p->H);
    a.kv_splits = 1;
    if ((rc = make_map(&mk, p->k, fp8, p->Lk, p->H, p->k_stride_l, p->k_stride_h, h3a::kPairKBoxRows)) != H3A_OK) return rc;
    if (two_launch_online_enabled() && workspace && aligned16(workspace) && workspace_bytes >= redo_list_bytes(p->Lq, p->H)) {
      // Two launches.  (1) The fixed-reference kernel with a per-row reference taken from the row's first key tile:
      // four MMA -> softmax -> MMA chains per CTA and no maximum pass after the first tile; a pair in which a later
      // logit outgrows what that reference can represent puts itself on the list.  (2) The running-maximum kernel
      // over the listed pairs only (all others leave at once), which overwrites their rows.  The result is the exact
      // online softmax for any input.
      a.redo_count = static_cast<int*>(workspace);
      a.redo_list = a.redo_count + 4;
      if (cudaMemsetAsync(a.redo_count, 0, sizeof(int), st) != cudaSuccess) return H3A_ERR_LAUNCH;
      rc = fp8 ? launch_attn_pair<true, false, true, true>(mq, mk, mv, a, st) : launch_attn_pair<false, false, true, true>(mq, mk, mv, a, st);
      if (rc != H3A_OK) return rc;
    }
    return fp8 ? launch_attn_pair<true, false, false>(mq, mk, mv, a, st) : launch_attn_pair<false, false, false>(mq, mk, mv, a, st);
  }
  if (fp8) return fixed ? launch_attn<true, false, true>(mq, mk, mv, a, st) : launch_attn<true, false, false>(mq, mk, mv, a, st);
  return fixed ? launch_attn<false, false, true>(mq, mk, mv, a, st) : launch_attn<false, false, false>(mq, mk, mv, a, st);
}


// The launch behind h3a_qk_prep and h3a_qk_prep_scatter (`scatter`: rows go to the head's owning rank).
int32_t prep_impl(const h3a_prep_params* p, const h3a_head_scatter* q_to, const h3a_head_scatter* k_to, bool scatter, void* stream) {
  if (!p) return H3A_ERR_ARG;
  if (p->d != 128 || p->H <= 0) return H3A_ERR_SHAPE;
  if (p->rope_mode != H3A_ROPE_INTERLEAVED && p->rope_mode != H3A_ROPE_HALF) return H3A_ERR_ARG;
  if (p->flags & ~(H3A_PREP_FP8 | H3A_PREP_NO_NORM)) return H3A_ERR_ARG;
  const bool fp8 = (p->flags & H3A_PREP_FP8) != 0;
  if (scatter && fp8) return H3A_ERR_ARG;  // block scales need whole blocks of the full sequence: quantise at the owner
  int32_t rc = check_arch();
  if (rc != H3A_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int which = 0; which < 2; ++which) {
    h3a::PrepArgs a;
    std::memset(&a, 0, sizeof(a));
    a.in = static_cast<const __nv_bfloat16*>(which ? p->k_in : p->q_in);
    const h3a_head_scatter* to = which ? k_to : q_to;
    if (!a.in) {
      if (to) return H3A_ERR_ARG;
      continue;
    }
    a.out = which ? p->k_out : p->q_out;
    a.scale = which ? p->k_scale : p->q_scale;
    a.stride_l = which ? p->k_stride_l : p->q_stride_l;
    a.stride_h = which ? p->k_stride_h : p->q_stride_h;
    a.L = which ? p->Lk : p->Lq;
    a.H = p->H;
    a.rope = which ? p->k_rope : p->q_rope;
    a.weight = which ? p->k_weight : p->q_weight;
    a.eps = p->eps > 0.f ? p->eps : 1e-6f;
    a.rope_half = p->rope_mode == H3A_ROPE_HALF;
    a.no_norm = (p->flags & H3A_PREP_NO_NORM) != 0;
    if (a.L <= 0) return H3A_ERR_SHAPE;
    if (scatter) {
      if (!to) return H3A_ERR_ARG;
      if (to->n_ranks < 1 || to->n_ranks > H3A_MAX_RANKS || to->heads_per_rank < 1 || to->head0 < 0 || to->row_offset < 0) return H3A_ERR_ARG;
      if (static_cast<int64_t>(to->row_offset) + a.L > to->L_total) return H3A_ERR_SHAPE;
      if (static_cast<int64_t>(to->head0) + a.H > static_cast<int64_t>(to->heads_per_rank) * to->n_ranks) return H3A_ERR_SHAPE;
      for (int r = 0; r < to->n_ranks; ++r) {
        if (!to->base[r]) return H3A_ERR_ARG;
        if (!aligned16(to->base[r])) return H3A_ERR_ALIGN;
        a.rank_out[r] = to->base[r];
      }
      a.n_ranks = to->n_ranks; a.heads_per_rank = to->heads_per_rank; a.round_robin = to->round_robin != 0;
      a.head0 = to->head0; a.row_offset = to->row_offset; a.L_total = to->L_total;
      a.head_rot = to->start_head > 0 ? to->start_head % a.H : 0;
      a.out = to->base[0];
    }
    if (!a.out || (fp8 && !a.scale)) return H3A_ERR_ARG;
    if (!aligned16(a.in) || !aligned16(a.out) || (a.stride_l % 8) || (a.stride_h % 8)) return H3A_ERR_ALIGN;
    if (a.rope && !aligned16(a.rope)) return H3A_ERR_ALIGN;
    a.nblk = (a.L + 127) / 128;
    dim3 grid(a.nblk, a.H);
    if (fp8) h3a::qk_prep_kernel<true><<<grid, h3a::kPrepThreads, 0, st>>>(a);
    else if (scatter && scatter_bulk_enabled()) h3a::qk_prep_kernel<false, true><<<grid, h3a::kPrepThreads, 0, st>>>(a);
    else h3a::qk_prep_kernel<false><<<grid, h3a::kPrepThreads, 0, st>>>(a);
    if (cudaGetLastError() != cudaSuccess) return H3A_ERR_LAUNCH;
  }
  return H3A_OK;
}

}  // namespace

extern "C" {

int32_t h3a_version(int32_t* major, int32_t* minor) {
  if (major) *major = H3A_VERSION_MAJOR;
  if (minor) *minor = H3A_VERSION_MINOR;
  return H3A_OK;
}

const char* h3a_status_string(int32_t s) {
  switch (s) {
    case H3A_OK: return "ok";
    case H3A_ERR_ARG: return "invalid argument (null pointer, bad enum or flag)";
    case H3A_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
    case H3A_ERR_SHAPE: return "unsupported shape (head dim must be 128, batch 1, extents > 0)";
    case H3A_ERR_ARCH: return "device is not compute capability 10.x (B200)";
    case H3A_ERR_LAUNCH: return "CUDA runtime or driver call failed";
    case H3A_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case H3A_ERR_WORKSPACE: return "workspace missing or too small";
    case H3A_ERR_DRIVER: return "driver entry point cuTensorMapEncodeTiled not available";
    case H3A_ERR_STATIC_SCRATCH: return "block index too large for the static scratch array (kept tiles + query-tile pairs > 262144)";
    case H3A_ERR_BOUND: return "logit_bound does not hold for the data: a softmax row sum under- or overflowed (pass a larger bound, or 0)";
    case H3A_ERR_INDEX: return "malformed block index (row pointers must not decrease and stay within nnz; columns in range, ascending)";
    default: return "unknown status";
  }
}

int32_t h3a_attn_workspace_bytes(const h3a_attn_params* p, size_t* bytes) {
  if (!p || !bytes) return H3A_ERR_ARG;
  if (p->mode == H3A_MODE_BLOCK_SPARSE) {
    *bytes = sparse_workspace_bytes(p);
  } else {
    // optional: partial sums of the split last wave (dense launches with a logit bound); without it the launch
    // simply does not split
    const bool fixed = fixed_reference_ok(p->logit_bound);
    const bool pairs = pair_kernel_enabled() && p->Lq > 0 && p->H > 0 && (p->Lk + 127) / 128 >= kPairMinKeyTiles;
    if (pairs && fixed) *bytes = plan_split(p->Lq, p->Lk, p->H).bytes;
    else if (pairs && two_launch_online_enabled()) *bytes = redo_list_bytes(p->Lq, p->H);  // no bound: list of pairs to redo
    else *bytes = 0;
  }
  return H3A_OK;
}

int32_t h3a_attn_kernel_choice(const h3a_attn_params* p, int32_t* choice) {
  if (!p || !choice) return H3A_ERR_ARG;
  if (p->Lq <= 0 || p->Lk <= 0 || p->H <= 0) return H3A_ERR_SHAPE;
  const bool fixed = fixed_reference_ok(p->logit_bound);
  const int64_t nqb = (p->Lq + 127) / 128, nkb = (p->Lk + 127) / 128;
  const bool resident = resident_kernel_applies(p->mode, fixed, p->Lq, p->Lk, p->H);
  bool pairs = (pair_kernel_enabled() && nkb >= kPairMinKeyTiles) || resident;
  if (p->mode == H3A_MODE_BLOCK_SPARSE)
    pairs = pairs && fixed && static_cast<double>(p->nnz) / (static_cast<double>(nqb) * static_cast<double>(nkb)) >= kPairMinDensity;
  int32_t c = 0;
  if (pairs) c |= H3A_KERNEL_CTA_PAIRS;
  if (fixed) c |= H3A_KERNEL_FIXED_REFERENCE;
  if (pairs && fixed && !resident && p->mode != H3A_MODE_BLOCK_SPARSE && p->workspace && aligned16(p->workspace)) {
    const SplitPlan sp = plan_split(p->Lq, p->Lk, p->H);
    if (sp.kv_splits > 1 && p->workspace_bytes >= sp.bytes) c |= H3A_KERNEL_SPLIT_LAST_WAVE;
  }
  if (pairs && !fixed && p->mode != H3A_MODE_BLOCK_SPARSE && two_launch_online_enabled() && p->workspace && aligned16(p->workspace) &&
      p->workspace_bytes >= redo_list_bytes(p->Lq, p->H))
    c |= H3A_KERNEL_ONLINE_TWO_LAUNCH;
  // persistent blocks: the resident pairs, or one single-CTA block per SM (dense and FP8-QK launches with a bound and
  // more items than SMs; block-sparse launches only with H3A_PERSIST=1, which is not reported here)
  if (resident || (!pairs && fixed && p->mode != H3A_MODE_BLOCK_SPARSE && persist_mode() != 0 &&
                   ((p->Lq + 255) / 256) * p->H > sm_count_of_current_device()))
    c |= H3A_KERNEL_PERSISTENT;
  *choice = c;
  return H3A_OK;
}

int32_t h3a_attn_fwd(const h3a_attn_params* p, void* stream) {
  int32_t rc = validate_attn(p);
  if (rc != H3A_OK) return rc;
  rc = check_arch();
  if (rc != H3A_OK) return rc;
  return attn_fwd_impl(p, p->workspace, p->workspace_bytes, static_cast<cudaStream_t>(stream));
}

int32_t h3a_qk_prep(const h3a_prep_params* p, void* stream) { return prep_impl(p, nullptr, nullptr, false, stream); }

int32_t h3a_qk_prep_scatter(const h3a_prep_params* p, const h3a_head_scatter* q_to, const h3a_head_scatter* k_to, void* stream) {
  return prep_impl(p, q_to, k_to, true, stream);
}

int32_t h3a_peer_alloc(size_t bytes, void** ptr, uint8_t handle[H3A_PEER_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == H3A_PEER_HANDLE_BYTES, "handle size");
  if (!ptr || !handle || bytes == 0) return H3A_ERR_ARG;
  void* d = nullptr;
  if (cudaMalloc(&d, bytes) != cudaSuccess) return H3A_ERR_LAUNCH;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, d) != cudaSuccess) {
    cudaFree(d);
    return H3A_ERR_LAUNCH;
  }
  std::memcpy(handle, &h, sizeof(h));
  *ptr = d;
  return H3A_OK;
}

int32_t h3a_peer_open(const uint8_t handle[H3A_PEER_HANDLE_BYTES], void** ptr) {
  if (!ptr || !handle) return H3A_ERR_ARG;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* d = nullptr;
  if (cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return H3A_ERR_LAUNCH;
  *ptr = d;
  return H3A_OK;
}

int32_t h3a_peer_close(void* ptr) {
  if (!ptr) return H3A_ERR_ARG;
  return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? H3A_OK : H3A_ERR_LAUNCH;
}

int32_t h3a_peer_free(void* ptr) {
  if (!ptr) return H3A_ERR_ARG;
  return cudaFree(ptr) == cudaSuccess ? H3A_OK : H3A_ERR_LAUNCH;
}

int32_t h3a_rope_table(const float* pos, int32_t L, const int32_t split[3], float theta, float* table, void* stream) {
  if (!pos || !table || !split) return H3A_ERR_ARG;
  if (L <= 0) return H3A_ERR_SHAPE;
  if (split[0] + split[1] + split[2] != 128 || (split[0] | split[1] | split[2]) & 1 || split[0] <= 0 || split[1] < 0 || split[2] < 0)
    return H3A_ERR_SHAPE;
  if (!aligned16(table)) return H3A_ERR_ALIGN;
  int32_t rc = check_arch();
  if (rc != H3A_OK) return rc;
  const long long n = static_cast<long long>(L) * 64;
  const int threads = 256;
  h3a::rope_table_kernel<<<static_cast<unsigned>((n + threads - 1) / threads), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      pos, L, split[0], split[1], split[2], theta > 0.f ? theta : 10000.0f, table);
  return cudaGetLastError() == cudaSuccess ? H3A_OK : H3A_ERR_LAUNCH;
}

int32_t h3a_build_block_index(int32_t T, int32_t Hg, int32_t Wg, int32_t n_audio, int32_t wt, int32_t wh, int32_t ww,
                              int32_t* row_ptr, int32_t* col_idx, int64_t* nnz) {
  if (!nnz) return H3A_ERR_ARG;
  if (T <= 0 || Hg <= 0 || Wg <= 0 || n_audio < 0 || wt < 0 || wh < 0 || ww < 0) return H3A_ERR_SHAPE;
  const int64_t n_video = static_cast<int64_t>(T) * Hg * Wg;
  const int64_t L = n_audio + n_video;
  const int64_t nb = (L + 127) / 128;
  // column tiles that hold at least one audio key are always kept
  const int64_t n_audio_tiles = (n_audio + 127) / 128;
  std::vector<uint8_t> mark(static_cast<size_t>(nb));
  std::vector<int32_t> cols;
  int64_t total = 0;
  const bool fill = col_idx != nullptr;
  if (fill && !row_ptr) return H3A_ERR_ARG;
  const int64_t cap = fill ? *nnz : 0;
  if (fill) row_ptr[0] = 0;
  for (int64_t qb = 0; qb < nb; ++qb) {
    const int64_t lo = qb * 128, hi = std::min<int64_t>(L, lo + 128);
    if (lo < n_audio) {
      std::fill(mark.begin(), mark.end(), 1);  // the tile holds audio queries: dense row
    } else {
      std::fill(mark.begin(), mark.end(), 0);
      for (int64_t b = 0; b < n_audio_tiles; ++b) mark[b] = 1;
    }
    if (lo >= n_audio) {
      // video queries of this tile: each one sees a (2wt+1) x (2wh+1) set of row segments of width 2ww+1
      for (int64_t tok = lo; tok < hi; ++tok) {
        const int64_t n = tok - n_audio;
        const int t = static_cast<int>(n / (static_cast<int64_t>(Hg) * Wg));
        const int h = static_cast<int>((n / Wg) % Hg);
        const int w = static_cast<int>(n % Wg);
        const int w0 = std::max(0, w - ww), w1 = std::min(Wg - 1, w + ww);
        for (int tt = std::max(0, t - wt); tt <= std::min(T - 1, t + wt); ++tt)
          for (int hh = std::max(0, h - wh); hh <= std::min(Hg - 1, h + wh); ++hh) {
            const int64_t base = n_audio + (static_cast<int64_t>(tt) * Hg + hh) * Wg;
            const int64_t b0 = (base + w0) / 128, b1 = (base + w1) / 128;
            for (int64_t b = b0; b <= b1; ++b) mark[b] = 1;
          }
      }
    }
    for (int64_t b = 0; b < nb; ++b)
      if (mark[b]) {
        if (fill) {
          if (total >= cap) return H3A_ERR_WORKSPACE;
          col_idx[total] = static_cast<int32_t>(b);
        }
        ++total;
      }
    if (fill) row_ptr[qb + 1] = static_cast<int32_t>(total);
  }
  if (total > 0x7FFFFFFF) return H3A_ERR_SHAPE;
  *nnz = total;
  return H3A_OK;
}

int32_t h3a_memcpy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                           int32_t to_host, void* stream) {
  if (!dst || !src || width_bytes == 0 || rows == 0 || width_bytes > dst_pitch || width_bytes > src_pitch) return H3A_ERR_ARG;
  const cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows,
                                          to_host ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice,
                                          static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? H3A_OK : H3A_ERR_LAUNCH;
}

int32_t h3a_selftest_wait_timeout(int32_t* status_word, int64_t wait_limit_ns, void* stream) {
  if (!status_word || wait_limit_ns <= 0 || wait_limit_ns > 1000000000ll) return H3A_ERR_ARG;
  int32_t rc = check_arch();
  if (rc != H3A_OK) return rc;
  AttnArgs a;
  std::memset(&a, 0, sizeof(a));
  a.status = status_word;
  a.wait_ns = wait_limit_ns;
  h3a::wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? H3A_OK : H3A_ERR_LAUNCH;
}

int32_t h3a_static_scratch_capacity(size_t* plan_entries) {
  if (!plan_entries) return H3A_ERR_ARG;
  *plan_entries = kStaticScratchInts;
  return H3A_OK;
}

int32_t h3a_attn_fwd_sparse_static(const h3a_attn_params* p, void* stream) {
  int32_t rc = validate_attn(p);
  if (rc != H3A_OK) return rc;
  if (p->mode != H3A_MODE_BLOCK_SPARSE) return H3A_ERR_ARG;
  const size_t n_qpairs = (static_cast<size_t>(p->Lq) + 255) / 256;
  if (static_cast<size_t>(p->nnz) + n_qpairs > kStaticScratchInts) return H3A_ERR_STATIC_SCRATCH;
  rc = check_arch();
  if (rc != H3A_OK) return rc;
  int32_t* scratch = nullptr;
  if ((rc = static_scratch_for_current_device(&scratch)) != H3A_OK) return rc;
  // The plan kernel writes every count and every plan entry the attention kernel will read, so nothing in the
  // array has to start at zero and whatever the previous call left there is never looked at.  From here on the
  // launch is the one h3a_attn_fwd makes (same kernel choice from logit_bound and density, same scheduling hint),
  // so the two entry points give bit-identical results for the same arguments.
  return attn_fwd_impl(p, scratch, kStaticScratchInts * sizeof(int32_t), static_cast<cudaStream_t>(stream));
}

#ifdef H3A_TRACE
// debug builds only: point the timeline trace at a device buffer of 4*64*8 uint64
int32_t h3a_debug_set_trace(void* dev_buffer) {
  return cudaMemcpyToSymbol(h3a::g_trace, &dev_buffer, sizeof(void*)) == cudaSuccess ? H3A_OK : H3A_ERR_LAUNCH;
}
#endif

int32_t h3a_proj_fwd(const h3a_proj_params* p, void* stream) {
  if (!p || !p->x || !p->w || (!p->out && !p->out_to)) return H3A_ERR_ARG;
  if (p->L <= 0 || p->K <= 0 || p->N <= 0 || p->N % 128 != 0 || p->R < 0) return H3A_ERR_SHAPE;
  if (p->epilogue != H3A_PROJ_STORE && p->epilogue != H3A_PROJ_PREP && p->epilogue != H3A_PROJ_PREP_FP8) return H3A_ERR_ARG;
  if (p->epilogue == H3A_PROJ_PREP_FP8 && !p->out_scale) return H3A_ERR_ARG;
  if (p->rope_mode != H3A_ROPE_INTERLEAVED && p->rope_mode != H3A_ROPE_HALF) return H3A_ERR_ARG;
  const bool lora = p->R > 0;
  if (lora && (!p->lora_t || !p->lora_bs)) return H3A_ERR_ARG;
  const int64_t out_unit = p->epilogue == H3A_PROJ_PREP_FP8 ? 16 : 8;  // 16-byte stores
  if (!p->out_to && (!aligned16(p->out) || (p->out_stride_l % out_unit) || (p->out_stride_h % out_unit) || p->out_stride_l <= 0 || p->out_stride_h <= 0)) return H3A_ERR_ALIGN;
  if ((p->bias && !aligned16(p->bias)) || (p->rope && !aligned16(p->rope)) || (p->norm_weight && !aligned16(p->norm_weight))) return H3A_ERR_ALIGN;
  int32_t rc = check_arch();
  if (rc != H3A_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap mx, mw, mt, mb;
  if ((rc = make_map2d(&mx, p->x, p->K, p->L, p->x_stride_l)) != H3A_OK) return rc;
  if ((rc = make_map2d(&mw, p->w, p->K, p->N, p->w_stride_n)) != H3A_OK) return rc;
  if (lora) {
    if ((rc = make_map2d(&mt, p->lora_t, p->R, p->L, p->lora_t_stride_l)) != H3A_OK) return rc;
    if ((rc = make_map2d(&mb, p->lora_bs, p->R, p->N, p->lora_bs_stride_n)) != H3A_OK) return rc;
  } else {
    mt = mx;
    mb = mw;
  }
  h3a::ProjArgs a;
  std::memset(&a, 0, sizeof(a));
  a.wait.status = p->status_word;
  a.wait.wait_ns = p->wait_limit_ns > 0 ? p->wait_limit_ns : 2000000000ll;
  a.L = p->L; a.N = p->N;
  a.n_tiles_n = (p->N + 255) / 256;
  a.kb_main = (p->K + 63) / 64;
  a.kb_lora = lora ? (p->R + 63) / 64 : 0;
  a.epilogue = p->epilogue;
  a.bias = p->bias; a.rope = p->rope; a.norm_weight = p->norm_weight;
  a.eps = p->eps > 0.f ? p->eps : 1e-6f;
  a.rope_half = p->rope_mode == H3A_ROPE_HALF;
  a.out = p->out;
  a.out_stride_l = p->out_stride_l; a.out_stride_h = p->out_stride_h;
  if (p->out_to) {
    const h3a_head_scatter* to = p->out_to;
    if (p->epilogue == H3A_PROJ_PREP_FP8) return H3A_ERR_ARG;  // block scales need whole blocks of the full sequence
    if (to->n_ranks < 1 || to->n_ranks > H3A_MAX_RANKS || to->heads_per_rank < 1 || to->head0 < 0 || to->row_offset < 0) return H3A_ERR_ARG;
    if (static_cast<int64_t>(to->row_offset) + p->L > to->L_total) return H3A_ERR_SHAPE;
    if (static_cast<int64_t>(to->head0) + p->N / 128 > static_cast<int64_t>(to->heads_per_rank) * to->n_ranks) return H3A_ERR_SHAPE;
    for (int r = 0; r < to->n_ranks; ++r) {
      if (!to->base[r]) return H3A_ERR_ARG;
      if (!aligned16(to->base[r])) return H3A_ERR_ALIGN;
      a.rank_out[r] = to->base[r];
    }
    a.n_ranks = to->n_ranks; a.heads_per_rank = to->heads_per_rank; a.round_robin = to->round_robin != 0;
    a.head0 = to->head0; a.row_offset = to->row_offset; a.L_total = to->L_total;
    a.col_rot = to->start_head > 0 ? (to->start_head / 2) % ((p->N + 255) / 256) : 0;  // a column tile holds two heads
  }
  a.out_scale = p->out_scale;
  a.nblk = (p->L + 127) / 128;

  static std::once_flag once[kMaxDevices];
  static cudaError_t attr_err[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return H3A_ERR_LAUNCH;
  std::call_once(once[dev], [dev] {
    attr_err[dev] = cudaFuncSetAttribute(h3a::qkv_proj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, h3a::kProjSmemBytes);
  });
  if (attr_err[dev] != cudaSuccess) return H3A_ERR_LAUNCH;
  a.n_tiles_m = (p->L + 255) / 256;
  a.n_tiles = a.n_tiles_m * a.n_tiles_n;
  a.band_n = proj_band_tiles(a.n_tiles_n, p->K + p->R);
  const int sms = sm_count_of_current_device();
  const unsigned pairs = static_cast<unsigned>(std::min(a.n_tiles, std::max(1, sms / 2)));  // persistent: one pair per two SMs
  h3a::qkv_proj_kernel<<<2u * pairs, h3a::kProjThreads, h3a::kProjSmemBytes, st>>>(mx, mw, mt, mb, a);
  return cudaGetLastError() == cudaSuccess ? H3A_OK : H3A_ERR_LAUNCH;
}

int32_t h3a_adaln_norm(const h3a_adaln_params* p, void* stream) {
  if (!p || !p->x || !p->y || !p->scale || !p->shift) return H3A_ERR_ARG;
  if (p->L <= 0 || p->T <= 0 || p->D <= 0 || p->D % 8 != 0 || p->D > 8 * h3a::kAdaThreads * h3a::kAdaMaxChunks) return H3A_ERR_SHAPE;
  if (p->rms != 0 && p->rms != 1) return H3A_ERR_ARG;
  if (!aligned16(p->x) || !aligned16(p->y) || !aligned16(p->scale) || !aligned16(p->shift)) return H3A_ERR_ALIGN;
  if ((p->x_stride % 8) || (p->y_stride % 8) || (p->scale_stride % 8) || (p->shift_stride % 8)) return H3A_ERR_ALIGN;
  if (p->x_stride < p->D || p->y_stride < p->D || p->scale_stride < p->D || p->shift_stride < p->D) return H3A_ERR_ARG;
  h3a::AdaLnArgs a;
  a.x = static_cast<const __nv_bfloat16*>(p->x);
  a.y = static_cast<__nv_bfloat16*>(p->y);
  a.x_stride = p->x_stride; a.y_stride = p->y_stride;
  a.scale = static_cast<const __nv_bfloat16*>(p->scale);
  a.shift = static_cast<const __nv_bfloat16*>(p->shift);
  a.scale_stride = p->scale_stride; a.shift_stride = p->shift_stride;
  a.idx = reinterpret_cast<const long long*>(p->idx);
  a.weight = p->weight; a.bias = p->bias;
  a.L = p->L; a.D = p->D; a.T = p->T;
  a.eps = p->eps > 0.f ? p->eps : 1e-6f;
  a.rms = p->rms;
  const unsigned grid = static_cast<unsigned>(p->L);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch ((p->D / 8 + h3a::kAdaThreads - 1) / h3a::kAdaThreads) {  // 16-byte chunks per thread
    case 1: h3a::adaln_norm_kernel<1><<<grid, h3a::kAdaThreads, 0, st>>>(a); break;
    case 2: h3a::adaln_norm_kernel<2><<<grid, h3a::kAdaThreads, 0, st>>>(a); break;
    case 3: h3a::adaln_norm_kernel<3><<<grid, h3a::kAdaThreads, 0, st>>>(a); break;
    case 4: h3a::adaln_norm_kernel<4><<<grid, h3a::kAdaThreads, 0, st>>>(a); break;
    case 5: h3a::adaln_norm_kernel<5><<<grid, h3a::kAdaThreads, 0, st>>>(a); break;
    case 6: h3a::adaln_norm_kernel<6><<<grid, h3a::kAdaThreads, 0, st>>>(a); break;
    case 7: h3a::adaln_norm_kernel<7><<<grid, h3a::kAdaThreads, 0, st>>>(a); break;
    default: h3a::adaln_norm_kernel<8><<<grid, h3a::kAdaThreads, 0, st>>>(a); break;
  }
  return cudaGetLastError() == cudaSuccess ? H3A_OK : H3A_ERR_LAUNCH;
}

int32_t h3a_read_device_status(const int32_t* status_word, void* stream, int32_t* raw) {
  if (!status_word) return H3A_ERR_ARG;
  int32_t v = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&v, status_word, sizeof(v), cudaMemcpyDeviceToHost, st) != cudaSuccess) return H3A_ERR_LAUNCH;
  if (cudaStreamSynchronize(st) != cudaSuccess) return H3A_ERR_LAUNCH;
  if (raw) *raw = v;
  if (v == 0) return H3A_OK;
  if ((v & 0xFF) == h3a::kBadBlockIndex) return H3A_ERR_INDEX;
  return (v & 0xFF) == h3a::kBadLogitBound ? H3A_ERR_BOUND : H3A_ERR_TIMEOUT;
}

}  // extern "C"
