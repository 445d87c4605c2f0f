// Flash-style forward attention for sm_100a: tcgen05 MMAs with S/P/O accumulators in TMEM, K/V tiles
// staged by TMA through a multi-buffered shared-memory ring, warp-specialised roles.
//
// One CTA owns a PAIR of 128-row query tiles of one head (two "streams") and walks the key tiles:
//   warp 8   producer : TMA loads of Q (once) and of K_j, V_j (128 keys each) into a ring of 32 KB stages
//   warps 9,10 issuers: one warp per stream; its elected lane issues  S = Q_t K^T  (SS MMA, N = 64 keys)
//                       and  O_t += P V  (TS MMA, P read from TMEM, K = 64 keys); tcgen05.commit signals
//                       mbarriers.  Two issuers keep the tensor pipe fed while one of them polls a barrier.
//   warps 0-3 / 4-7   : softmax of stream 0 / 1, one query row per thread (TMEM lane == row): online
//                       max / exp2 / sum, P written back over S as packed bf16, lazy rescale of O
//                       (only when the running max grows by more than 2^8), final 1/l and store.
// Each 128-key tile is processed as two 64-key halves with their own S buffer, so each stream has two
// S/P buffers in flight: while the softmax warps work on one half, the tensor pipe already produces the
// next S into the other buffer (after the P V that frees it), and the two streams interleave on top.
// K_j and V_j are fetched once per 256 query rows.
//
// TMEM (512 columns x 128 lanes, fp32):
//   stream t: S/P buffer h at columns [128 t + 64 h, +64) (P = packed bf16 in its first 32 columns)
//   O_t at columns [256 + 128 t, +128)
//
// Every wait on an mbarrier is bounded: when the time limit runs out the CTA records a code in the
// caller's status word, raises a CTA-wide abort flag, lets copies in flight land, frees TMEM and returns.
#pragma once
#include "ptx.cuh"

namespace h3a {

constexpr int kTile = 128;
constexpr int kHeadDim = 128;
constexpr int kStages = 5;
constexpr int kStageBytes = 32768;
constexpr int kQTileBytes = 32768;
constexpr int kHalfBytes = 16384;  // one [128 rows][128 bytes] swizzled box
// Thread layout.  Running-maximum kernels: warpgroups 0,1 = softmax of stream 0,1 (a warp walks both halves of
// every tile, they share the row's running maximum); warpgroup 2 = producer, two issuers, one idle warp.
// Fixed-reference kernels have no per-row state besides the row sum, so every (stream, half) gets its own
// warpgroup: four softmax warps per SM sub-partition instead of two hide each other's TMEM-load, store and
// barrier latencies.
// Register re-allocation: setmaxnreg.inc BLOCKS until the registers exist, and they can only come from what the
// CTA owns at launch (registers per thread reported by the compiler x threads) minus what the helper warpgroup
// gives back.  kLaunchRegs is checked against the real kernel attribute before every first launch.
template <bool kFixed>
struct AttnLayout {
  static constexpr int kSoftmaxWarps = kFixed ? 16 : 8;
  static constexpr int kThreads = (kSoftmaxWarps + 4) * 32;
  static constexpr int kLaunchRegs = kFixed ? 96 : 168;
  static constexpr int kSoftmaxRegs = kFixed ? 104 : 208;
  static constexpr int kHelperRegs = kFixed ? 64 : 88;
  static_assert(kSoftmaxWarps * 32 * kSoftmaxRegs + 128 * kHelperRegs <= kLaunchRegs * kThreads,
                "setmaxnreg budget exceeds the launch allocation");
};
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// S production: 0 = one N=64 MMA group per half (each half's S is produced while softmax works on the other
// half, but these MMAs are shared-memory-bandwidth bound); 1 = one full-rate N=128 MMA group per key tile into
// both halves' buffers, issued after the P V of the previous tile's second half.
#ifndef H3A_FULL_S
#define H3A_FULL_S 0
#endif
constexpr bool kFullS = H3A_FULL_S != 0;
// Of every 4 element pairs, how many take the polynomial exp2 on the FMA pipe instead of the MUFU (0..4).  One in four
// is the fastest in CLOCK CYCLES (the MUFU is the busier pipe), but the polynomial's five FMAs cost more energy than one
// MUFU operation, and the long launches run under the board's power cap: with none the clock settles 4-5 % higher and
// the launch is shorter (dense config 1: 37.3 against 38.0 ms, block-sparse 20.2 against 20.8 ms, same box, alternating
// runs).  So the default is 0; kernels that are not power-limited ask for 1 (exp_half_tile's second argument).
#ifndef H3A_POLY_PAIRS
#define H3A_POLY_PAIRS 0
#endif
constexpr int kPolyPairsBf16 = H3A_POLY_PAIRS;
#ifndef H3A_POLY_FP8
#define H3A_POLY_FP8 0
#endif
constexpr int kPolyPairsFp8 = H3A_POLY_FP8;    // FP8 mode has its own share: its S MMAs are cheaper, the balance differs

// Of every 4 element pairs of an FP8-QK tile, how many take the packed-bf16 exponential (one MUFU operation for two
// elements, its row-sum share accumulated in bf16 over 8 pairs at a time).  FP8-QK is bound by the MUFU; its error
// budget (e4m3 operands) is an order of magnitude above what the bf16-rounded argument adds.
#ifndef H3A_BF16X2_FP8
#define H3A_BF16X2_FP8 0
#endif
#ifndef H3A_BF16X2_BF16
#define H3A_BF16X2_BF16 0
#endif
constexpr int kPackedExpFp8 = H3A_BF16X2_FP8, kPackedExpBf16 = H3A_BF16X2_BF16;

// P = 2^(s c - m) for the 64 logits in s[] (one half tile, one row per thread): the packed bf16 results replace
// s[0..31]; returns the row-sum share.  Pair i uses, by (i & 3): the packed-bf16 MUFU path, the FMA-pipe polynomial,
// or two fp32 MUFU operations.
template <bool kFp8, int kPolyShare = -1>
__device__ __forceinline__ float exp_half_tile(uint32_t (&s)[64], float c, float m_ref) {
  constexpr int kPacked = kFp8 ? kPackedExpFp8 : kPackedExpBf16;
  constexpr int kPoly = kPolyShare >= 0 ? kPolyShare : (kFp8 ? kPolyPairsFp8 : kPolyPairsBf16);
  uint64_t acc0 = 0, acc1 = 0;  // two packed accumulators = four partial row sums (bit pattern 0 == 0.0f)
  uint32_t accb[4] = {0u, 0u, 0u, 0u};
  const uint64_t c2 = pack2(c, c), nm2 = pack2(-m_ref, -m_ref);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint64_t x = fma2(pack2u(s[2 * i], s[2 * i + 1]), c2, nm2);
    if ((i & 3) < kPacked) {
      float x0, x1;
      unpack2(x, x0, x1);
      const uint32_t pb = ex2_bf16x2(pack_bf16x2(x0, x1));
      accb[i >> 3] = add_bf16x2(accb[i >> 3], pb);
      s[i] = pb;
      continue;
    }
    uint64_t pp;
    if ((i & 3) < kPacked + kPoly) {
      pp = exp2_poly2(x);
    } else {
      float x0, x1;
      unpack2(x, x0, x1);
      pp = pack2(ex2_approx(x0), ex2_approx(x1));
    }
    if (i & 1) acc1 = add2(acc1, pp);
    else acc0 = add2(acc0, pp);
    float p0, p1;
    unpack2(pp, p0, p1);
    s[i] = pack_bf16x2(p0, p1);  // slot i <= 2i: already consumed
  }
  float a0, a1, a2, a3;
  unpack2(acc0, a0, a1);
  unpack2(acc1, a2, a3);
  float l = (a0 + a1) + (a2 + a3);
  if constexpr (kPacked > 0) {
#pragma unroll
    for (int g = 0; g < 4; ++g) l += __uint_as_float(accb[g] << 16) + __uint_as_float(accb[g] & 0xFFFF0000u);
  }
  return l;
}

struct AttnBars {
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t q_full;
  uint64_t s_full[2][2];  // [stream][half]
  uint64_t p_full[2][2];
  uint64_t o_full[2][2];  // completion of the P V of (stream, half): one phase per key tile
  uint64_t q_empty;       // every S MMA of a group of query tiles has completed: the next group's Q may be loaded
  uint64_t o_free[2];     // the stream's softmax warps have read O of a group: its next group may overwrite it
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  uint32_t early_exit;
  volatile uint32_t stop[2];  // per stream: one thread's reading of abort_flag, so that both warpgroups leave together
};

constexpr int kRowSumBytes = 2 * 128 * 4;  // fixed-reference softmax: the row sums the two warpgroups of a stream exchange
constexpr int kAttnSmemBytes = 2 * kQTileBytes + kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/ + kRowSumBytes;
static_assert(sizeof(AttnBars) <= 256, "barrier block too large");
static_assert(kAttnSmemBytes <= 232448, "shared memory budget");

struct AttnArgs {
  int Lq, Lk, H;
  int n_kv_tiles;
  int n_qpairs;
  float scale_log2;        // softmax_scale * log2(e)
  const float* q_scale;    // fp8: [H, nqb]
  const float* k_scale;    // fp8: [H, nkb]
  int nqb, nkb;
  const int32_t* row_ptr;  // sparse: CSR row pointers (plan entries of pair p start at row_ptr[2p])
  const int32_t* plan;     // sparse: (tile << 2) | stream flags
  const int32_t* plan_cnt; // sparse: entries per pair
  __nv_bfloat16* o;
  long long o_stride_l, o_stride_h;
  float* lse;              // [H, Lq] or null
  int* status;             // device status word or null
  long long wait_ns;
  float fixed_m;           // fixed softmax reference in log2 units (kFixed kernels)
  int heavy_pairs;         // sparse: leading query-tile pairs whose CTAs (of every head) are scheduled first
  int nnz;                 // sparse: entries of col_idx = capacity of the plan; plan offsets are clamped to it
  // CTA pairs, dense: pairs numbered split_begin and up (the ones that would form a last, partly empty wave) are
  // each handled by kv_splits CTA pairs, every one over its share of the key tiles; they leave un-normalised
  // partial outputs and row sums in `part`, which combine_partials_kernel adds up (the fixed softmax reference
  // makes partial results of one row directly addable).  kv_splits <= 1: off.
  int split_begin;
  int kv_splits;
  float* part;             // [slot][4 query tiles][128 rows][128 + 1] fp32: O columns, then the row sum
  // Sequence parallelism: with o_n_ranks > 1 query row g is stored at row g % o_rank_rows of o_rank[g / o_rank_rows]
  // (the rank that holds token g: its own memory or a peer GPU's, stored to only) instead of in `o`.
  __nv_bfloat16* o_rank[8];
  int o_n_ranks, o_rank_rows;
  // Online softmax in two launches (CTA pairs, no logit bound).  First the fixed-reference kernel with a PER-ROW
  // reference taken from the row's first key tile; a pair in which some later logit outgrows what that reference can
  // represent appends its number to redo_list (redo_count counts).  Then the running-maximum kernel with the same two
  // pointers as redo_list / redo_count: pair i of its grid handles entry i of the list, pairs beyond the count leave at once.
  int* redo_count;
  int* redo_list;
};

// address of output row `q_row` of (local) head `head`
__device__ __forceinline__ __nv_bfloat16* out_row_ptr(const AttnArgs& a, int q_row, int head) {
  __nv_bfloat16* base = a.o;
  int r = q_row;
  if (a.o_n_ranks > 1) {
    const int t = min(q_row / a.o_rank_rows, a.o_n_ranks - 1);
    base = a.o_rank[t];
    r = q_row - t * a.o_rank_rows;
  }
  return base + static_cast<long long>(r) * a.o_stride_l + static_cast<long long>(head) * a.o_stride_h;
}

// status word layout: bits [0,8) code, bits [8,32) blockIdx.x (truncated)
enum : int {
  kWaitQFull = 1, kWaitKvEmpty = 2, kWaitKvFullK = 3, kWaitKvFullV = 4,
  kWaitSFull = 5, kWaitPFull = 6, kWaitOFull = 7,
  kWaitQEmpty = 12, kWaitOFree = 13  // persistent CTAs (8 = drain of a CTA pair, 9 = self-test, 10 / 11 = bad index / bound)
};

// Optional timeline trace (debug builds only, -DH3A_TRACE): CTA 0 stamps clock64() at phase boundaries.
#ifdef H3A_TRACE
__device__ unsigned long long* g_trace = nullptr;
#define H3A_STAMP(role, idx, k)                                                                   \
  do {                                                                                            \
    if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && g_trace != nullptr && (idx) < 64) g_trace[((role) * 64 + (idx)) * 8 + (k)] = clock64(); \
  } while (0)
#else
#define H3A_STAMP(role, idx, k) do {} while (0)
#endif

// The limits and the status word are read from the kernel's argument block when a wait runs out, so that a
// wait context costs two registers in the loops that carry it.
struct WaitCtx {
  uint32_t abort_smem;            // shared-memory address of this CTA's abort flag
  uint32_t peer_abort;            // shared::cluster address of the peer CTA's flag (CTA pairs), else 0
  const AttnArgs* args;           // status word and time limit
};
__device__ __forceinline__ uint32_t ld_shared_u32_volatile(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_u32_volatile(uint32_t addr, uint32_t v) {
  asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// H3A_WAIT_SLEEP_NS > 0: a waiting thread sleeps that long between polls (fewer issue slots and less power spent on
// polling, at the price of a later wake-up).
#ifndef H3A_WAIT_SLEEP_NS
#define H3A_WAIT_SLEEP_NS 0
#endif
__device__ __forceinline__ bool bounded_wait(const WaitCtx& c, uint32_t bar, uint32_t parity, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  uint32_t polls = 0;
  uint64_t t0 = 0;
  while (!mbar_try_wait(bar, parity)) {
#if H3A_WAIT_SLEEP_NS > 0
    __nanosleep(H3A_WAIT_SLEEP_NS);
#endif
    if ((++polls & 63u) == 0u) {
      if (ld_shared_u32_volatile(c.abort_smem)) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (static_cast<long long>(now - t0) > c.args->wait_ns) {
        st_shared_u32_volatile(c.abort_smem, 1u);
        if (c.peer_abort) st_shared_cluster_u32(c.peer_abort, 1u);  // the peer's waits give up at their next check
        if (c.args->status) atomicCAS(c.args->status, 0, code | (static_cast<int>(blockIdx.x & 0x7FFFFF) << 8));
        return false;
      }
    }
  }
  return true;
}

// Whole-warp wait.  Default: every lane polls and the verdicts are combined, which keeps control flow uniform.
// H3A_ONE_LANE_WAIT=1 lets lane 0 poll and broadcasts its verdict; measured 15 % slower (the divergent branch
// costs more than 32 lanes polling one barrier word).
#ifndef H3A_ONE_LANE_WAIT
#define H3A_ONE_LANE_WAIT 0
#endif
__device__ __forceinline__ bool warp_wait(const WaitCtx& c, uint32_t bar, uint32_t parity, int code) {
#if H3A_ONE_LANE_WAIT
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = bounded_wait(c, bar, parity, code) ? 1 : 0;
  __syncwarp();
  return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
#else
  return __all_sync(0xFFFFFFFFu, bounded_wait(c, bar, parity, code));
#endif
}

// Diagnostic: one warp waits, with the same bounded wait the attention kernel uses, on an mbarrier that nothing
// ever arrives on.  The wait must run out, record kWaitSelfTest in the status word and return.
constexpr int kWaitSelfTest = 9;
__global__ void wait_selftest_kernel(const AttnArgs args) {
  __shared__ AttnBars bars;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars.q_full), 1);
    bars.abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  WaitCtx wc{smem_u32(const_cast<const uint32_t*>(&bars.abort_flag)), 0u, &args};
  bounded_wait(wc, smem_u32(&bars.q_full), 0, kWaitSelfTest);
}

// The plan kernels do not trust the caller's block index.  Row pointers are clamped into [0, nnz] and must not
// decrease; column entries must lie in [0, nkb) and ascend strictly inside a row.  What breaks a rule is left out
// of the plan, never written past the plan's `nnz` entries and reported (once) through the status word as
// kBadBlockIndex | offending query tile << 8: the attention launch that follows then does nothing, exactly as
// after a wait that gave up.  Without a status word the launch runs on the entries that passed.
constexpr int kBadBlockIndex = 10;
// Fixed-reference kernels: a row whose exponentials overflowed, or whose largest term fell below the range the
// reference serves, shows in its row sum: inf / NaN, or less than 2^-100 (a served row's sum is at least its largest
// term, 2^-92 or more; a sum of nothing but flushed or clamped terms stays below 2^-109).  That happens when the
// caller's logit bound does not hold for the data, or (bounds above 69) for a row whose logits all lie far below
// the bound; it is reported through the status word (once) as kBadLogitBound | CTA << 8 and the launch's output is
// not to be used.  `zero_is_legal`: an exact zero is a block-sparse row that lists no key tile (or one share of a
// split row).
constexpr int kBadLogitBound = 11;
__device__ __forceinline__ void check_row_sum(const AttnArgs& a, float l, bool zero_is_legal) {
  const bool bad = !(l < 3.0e38f) || (!(l > 7.8e-31f) && !(zero_is_legal && l == 0.0f));  // NaN fails every comparison
  if (bad && a.status) atomicCAS(a.status, 0, kBadLogitBound | (static_cast<int>(blockIdx.x & 0x7FFFFF) << 8));
}
__device__ __forceinline__ int clamp_row_ptr(int v, int nnz) { return max(0, min(v, nnz)); }
__device__ __forceinline__ void report_bad_index(int* status, int q_tile) {
  if (status) atomicCAS(status, 0, kBadBlockIndex | ((q_tile & 0x7FFFFF) << 8));
}
// begin / end of the key-tile list of query tile r (empty beyond nqb); *bad is raised when row_ptr breaks a rule
__device__ __forceinline__ void row_range(const int32_t* __restrict__ row_ptr, int r, int nqb, int nnz, int& begin, int& end, bool& bad) {
  begin = end = 0;
  if (r >= nqb) return;
  const int a = row_ptr[r], b = row_ptr[r + 1];
  begin = clamp_row_ptr(a, nnz);
  end = clamp_row_ptr(b, nnz);
  if (a != begin || b != end || b < a) bad = true;
  if (end < begin) end = begin;
}

// Merge the sorted key-tile lists of query tiles 2p and 2p+1 into one list with stream flags.
__global__ void build_pair_plan_kernel(const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ col_idx,
                                       int nqb, int n_qpairs, int nnz, int nkb, int32_t* __restrict__ plan,
                                       int32_t* __restrict__ plan_cnt, int* __restrict__ status) {
  int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_qpairs) return;
  bool bad = false;
  int a, a_end, b, b_end;
  row_range(row_ptr, 2 * p, nqb, nnz, a, a_end, bad);
  row_range(row_ptr, 2 * p + 1, nqb, nnz, b, b_end, bad);
  int32_t* out = plan + a;
  const int cap = nnz - a;  // the merged list is never longer than the two lists together, which end at or before nnz
  int n = 0, prev = -1;
  while (a < a_end || b < b_end) {
    int ca = (a < a_end) ? col_idx[a] : 0x7FFFFFFF;
    int cb = (b < b_end) ? col_idx[b] : 0x7FFFFFFF;
    int c = min(ca, cb);
    int f = 0;
    if (ca == c) { f |= 1; ++a; }
    if (cb == c) { f |= 2; ++b; }
    if (c <= prev || c >= nkb || n >= cap) { bad = true; continue; }  // out of range, out of order or duplicate
    prev = c;
    out[n++] = (c << 2) | f;
  }
  plan_cnt[p] = n;
  if (bad) report_bad_index(status, 2 * p);
}

// kFixed: the caller supplied an upper bound of the logits; it is used as the softmax reference for every row, so
// there is no running maximum, no rescaling of O and no per-row state besides the row sum.
template <bool kFp8, bool kSparse, bool kFixed>
__global__ void __launch_bounds__(AttnLayout<kFixed>::kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // 128B-swizzled tiles want 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t q_smem = base;
  const uint32_t ring_smem = base + 2 * kQTileBytes;
  AttnBars* bars = reinterpret_cast<AttnBars*>(smem + 2 * kQTileBytes + kStages * kStageBytes);

  using LY = AttnLayout<kFixed>;
  constexpr int kProducerWarp = LY::kSoftmaxWarps;
  constexpr int kIssuerWarp = LY::kSoftmaxWarps + 1;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Work items: one per (head, pair of query tiles), head-major, so that the CTAs running at the same time share one
  // head's K/V in L2.  Block-sparse: the few pairs with long key lists (dense audio rows) of ALL heads come first,
  // otherwise the ones of the last heads would start late and run on alone at the end.
  // A CTA handles items blockIdx.x, blockIdx.x + gridDim.x, ...: with one CTA per item that is one item; with fewer
  // CTAs (fixed-reference kernels, one CTA per SM) the CTA is persistent: barriers, TMEM and the K/V ring are set up
  // once, and the Q load, S MMAs and K/V loads of the next item run under the epilogue of the current one.  Every
  // role walks the same item sequence on its own; no item number is passed between warps.
  const int n_items = args.n_qpairs * args.H;
  int head = 0, pair = 0, q0 = 0, n_it = 0, dense_flags = 3;
  const int32_t* plan = nullptr;
  auto set_item = [&](int item) {
    if (kSparse && args.heavy_pairs > 0) {
      const int n_heavy = args.heavy_pairs * args.H;
      if (item < n_heavy) {
        head = item / args.heavy_pairs;
        pair = item % args.heavy_pairs;
      } else {
        const int r = item - n_heavy, n_light = args.n_qpairs - args.heavy_pairs;
        head = r / n_light;
        pair = args.heavy_pairs + r % n_light;
      }
    } else {
      head = item / args.n_qpairs;
      pair = item % args.n_qpairs;
    }
    q0 = pair * 2 * kTile;
    // the plan: which key tiles, for which streams
    if constexpr (kSparse) {
      plan = args.plan + clamp_row_ptr(args.row_ptr[2 * pair], args.nnz);
      n_it = args.plan_cnt[pair];
    } else {
      n_it = args.n_kv_tiles;
      dense_flags = (q0 + kTile < args.Lq) ? 3 : 1;
    }
  };
  auto entry_at = [&](int it) -> int {
    if constexpr (kSparse) return plan[it];
    else return (it << 2) | dense_flags;
  };
  set_item(blockIdx.x);

  constexpr uint32_t kQBytes = kFp8 ? kHalfBytes : kQTileBytes;  // bytes per Q tile
  constexpr uint32_t kKBytes = kFp8 ? kHalfBytes : kStageBytes;  // bytes per K tile
  constexpr uint32_t kVBytes = kStageBytes;

  // ---- set-up
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&bars->kv_full[i]), 1);
      mbar_init(smem_u32(&bars->kv_empty[i]), 2);  // released by both issuer warps
    }
    mbar_init(smem_u32(&bars->q_full), 1);
    mbar_init(smem_u32(&bars->q_empty), 2);  // one commit from each issuer warp
    for (int t = 0; t < 2; ++t) {
      for (int hf = 0; hf < 2; ++hf) {
        mbar_init(smem_u32(&bars->s_full[t][hf]), 1);
        mbar_init(smem_u32(&bars->p_full[t][hf]), 128);
        mbar_init(smem_u32(&bars->o_full[t][hf]), 1);
      }
      mbar_init(smem_u32(&bars->o_free[t]), 8);  // one arrive per softmax warp of the stream (fixed reference: 8 warps)
      bars->stop[t] = 0;
    }
    bars->abort_flag = 0;
    bars->early_exit = (args.status != nullptr && *reinterpret_cast<volatile int*>(args.status) != 0) ? 1u : 0u;
    fence_mbar_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
  }
  __syncthreads();
  if (bars->early_exit) return;  // an earlier CTA of this launch already gave up: do nothing
  if (warp == kIssuerWarp) {
    tmem_alloc(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;

  WaitCtx wc{smem_u32(const_cast<const uint32_t*>(&bars->abort_flag)), 0u, &args};

  if (warp >= LY::kSoftmaxWarps) {
   setmaxnreg_dec<LY::kHelperRegs>();
   if (warp == kProducerWarp) {
    // =========================================================== producer
    // The whole warp walks the loop (uniform control flow, uniform operands); one elected lane issues.
    const uint32_t leader = elect_one();
    int cnt = 0;     // K / V tiles loaded so far: the ring runs on across items
    uint32_t g = 0;  // items with work so far: the phase of q_full / q_empty
    bool ok = true;
    for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
    set_item(item);
    if (n_it == 0) continue;
    // The Q tiles are free when every S MMA of the previous item has completed, which is late in that item; its K / V
    // ring slots free up earlier.  So the first two key tiles of an item are requested ahead of its Q tiles unless those
    // happen to be free already; the wait for them blocks only from the third key tile on (or the last, if sooner).
    const int q_at = g > 0 ? min(2, n_it - 1) : 0;
    bool q_loaded = false;
    for (int it = 0; ok && it < n_it; ++it) {
      if (!q_loaded) {
        bool q_free = g == 0;
        if (!q_free) q_free = __all_sync(0xFFFFFFFFu, mbar_test_wait(smem_u32(&bars->q_empty), (g - 1) & 1));
        if (!q_free && it >= q_at) {
          ok = warp_wait(wc, smem_u32(&bars->q_empty), (g - 1) & 1, kWaitQEmpty);
          if (!ok) break;
          q_free = true;
        }
        if (q_free) {
          const uint32_t qbar = smem_u32(&bars->q_full);
          mbar_arrive_expect_tx_if(leader, qbar, 2 * kQBytes);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            tma_load_3d_if(leader, q_smem + t * kQTileBytes, &tm_q, qbar, 0, q0 + t * kTile, head);
            if constexpr (!kFp8) tma_load_3d_if(leader, q_smem + t * kQTileBytes + kHalfBytes, &tm_q, qbar, 64, q0 + t * kTile, head);
          }
          q_loaded = true;
        }
      }
      const int tile = entry_at(it) >> 2;
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {  // K tile, then V tile
        const int s = cnt % kStages;
        const uint32_t ph = (cnt / kStages) & 1;
        ok = warp_wait(wc, smem_u32(&bars->kv_empty[s]), ph ^ 1u, kWaitKvEmpty);
        if (!ok) break;
        const uint32_t fb = smem_u32(&bars->kv_full[s]);
        const uint32_t dst = ring_smem + s * kStageBytes;
        if (kv == 0) {
          mbar_arrive_expect_tx_if(leader, fb, kKBytes);
          tma_load_3d_if(leader, dst, &tm_k, fb, 0, tile * kTile, head);
          if constexpr (!kFp8) tma_load_3d_if(leader, dst + kHalfBytes, &tm_k, fb, 64, tile * kTile, head);
        } else {
          mbar_arrive_expect_tx_if(leader, fb, kVBytes);
          tma_load_3d_if(leader, dst, &tm_v, fb, 0, tile * kTile, head);
          tma_load_3d_if(leader, dst + kHalfBytes, &tm_v, fb, 64, tile * kTile, head);
        }
        ++cnt;
      }
    }
    ++g;
    }  // items
    __syncwarp();
  } else if (warp == kIssuerWarp || warp == kIssuerWarp + 1) {
    // =========================================================== MMA issuers, one warp per stream
    // Uniform control flow for the whole warp; the elected lane issues every MMA and commit (a commit
    // tracks the MMAs of the thread that executes it, and the election is the same lane every time).
    // Each issuer walks every plan entry, also those that do not list its stream: a K/V stage is released
    // by one commit from each issuer, and waiting for the stage first keeps the two in step.
    {
      const int t = warp - kIssuerWarp;
      const uint32_t leader = elect_one();
      constexpr uint32_t kSN = kFullS ? 128 : 64;
      constexpr uint32_t idesc_s = kFp8 ? umma_idesc(UMMA_FMT_E4M3, UMMA_FMT_E4M3, 0, 0, 128, kSN)
                                        : umma_idesc(UMMA_FMT_BF16, UMMA_FMT_BF16, 0, 0, 128, kSN);
      constexpr uint32_t idesc_pv = umma_idesc(UMMA_FMT_BF16, UMMA_FMT_BF16, 0, 1, 128, 128);
      bool ok = true;
      uint32_t p_cnt[2] = {0, 0};  // P halves consumed so far (all items): the phase of p_full
      uint32_t pv_cnt = 0;         // P V groups issued for the current item: the first one overwrites O
      uint32_t g = 0;              // items with work so far: the phase of q_full / q_empty / o_free
      int c0 = 0;                  // K / V tiles of the ring consumed before the current item
      // the descriptor of the Q tile never changes; K/V descriptors are a per-stage base plus constants
      const uint64_t q_desc = umma_desc_sw128(q_smem + t * kQTileBytes, 16, 1024);
      const uint64_t k_desc0 = umma_desc_sw128(ring_smem, 16, 1024);
      const uint64_t v_desc0 = umma_desc_sw128(ring_smem, kHalfBytes, 1024);
      const uint32_t s_tmem = tmem + t * kTile;
      const uint32_t o_tmem = tmem + 256 + t * kTile;

      // S[t][hf] = Q_t K[hf]^T for keys [64 hf, 64 hf + 64) of ring stage `sk` (both operands K-major,
      // 128B swizzle, 8-row groups 1024 B apart; 64 key rows = 8192 B into each box)
      auto issue_s = [&](int hf, int sk) {
        const uint64_t kd = k_desc0 + static_cast<uint64_t>((sk * kStageBytes + hf * 8192) >> 4);
        const uint32_t d = s_tmem + hf * 64;
        if constexpr (kFp8) {
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 32 e4m3 = 32 bytes per step inside the 128-byte swizzle span
            umma_e4m3_ss_if(leader, d, q_desc + (k * 32 >> 4), kd + (k * 32 >> 4), idesc_s, k > 0);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {  // 16 bf16 = 32 bytes per step; dims 64..127 live in the second box
            const uint32_t off = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
            umma_bf16_ss_if(leader, d, q_desc + off, kd + off, idesc_s, k > 0);
          }
        }
        umma_commit_if(leader, smem_u32(&bars->s_full[t][hf]));
      };
      // O_t += P[t][hf] V[hf] for keys [64 hf, +64) of ring stage `sv`: A = P from TMEM (two bf16 per
      // column), B = V MN-major ([key][64 dims] boxes: 8-key groups 1024 B apart, the two 64-dim halves 16 KB apart)
      auto issue_pv = [&](int hf, int sv) {
        const uint64_t vd = v_desc0 + static_cast<uint64_t>((sv * kStageBytes + hf * 8192) >> 4);
        const uint32_t a = s_tmem + hf * 64;
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 16 keys per step = 16 rows of 128 B
          umma_bf16_ts_if(leader, o_tmem, a + k * 8, vd + (k * 2048 >> 4), idesc_pv, (pv_cnt > 0 || k > 0) ? 1u : 0u);
        ++pv_cnt;
        umma_commit_if(leader, smem_u32(&bars->o_full[t][hf]));
      };

      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
      set_item(item);
      if (n_it == 0) continue;
      ok = warp_wait(wc, smem_u32(&bars->q_full), g & 1, kWaitQFull);
      if (!ok) break;
      tc_fence_after_sync();
      pv_cnt = 0;
      {  // prologue: both S halves of entry 0 (in TMEM they follow the previous item's last P V: MMAs run in issue order)
        const int f0 = entry_at(0) & 3;
        const int s0 = c0 % kStages;
        ok = warp_wait(wc, smem_u32(&bars->kv_full[s0]), (c0 / kStages) & 1, kWaitKvFullK);
        if (ok) {
          tc_fence_after_sync();
          if ((f0 >> t) & 1) {
            issue_s(0, s0);
            if constexpr (!kFullS) issue_s(1, s0);
          }
          umma_commit_if(leader, smem_u32(&bars->kv_empty[s0]));
        }
      }
      for (int it = 0; ok && it < n_it; ++it) {
        const int f = entry_at(it) & 3;
        const bool has_next = (it + 1 < n_it);
        const int fn = has_next ? (entry_at(it + 1) & 3) : 0;
        const int cv = c0 + 2 * it + 1, ck = c0 + 2 * it + 2;
        const int sv = cv % kStages, sk = ck % kStages;
        const bool mine = (f >> t) & 1, mine_next = (fn >> t) & 1;
        // every S MMA of the item has been issued (the last one with the previous entry): when they complete, the Q
        // tiles may be reloaded for the next item
        if (!has_next) umma_commit_if(leader, smem_u32(&bars->q_empty));
        ok = warp_wait(wc, smem_u32(&bars->kv_full[sv]), (cv / kStages) & 1, kWaitKvFullV);
        if (!ok) break;
        bool k_ready = false;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          if (ok && mine) {
            H3A_STAMP(2 + t, 2 * it + hf, 0);
            ok = warp_wait(wc, smem_u32(&bars->p_full[t][hf]), p_cnt[hf] & 1, kWaitPFull);
            if (ok && pv_cnt == 0 && g > 0) {
              // the first P V of an item overwrites O: the stream's softmax warps must have read the previous item's.
              // They arrive once per item with work, and cannot pass this item before its MMAs are issued, so the
              // barrier is never more than one phase ahead of this wait.
              ok = warp_wait(wc, smem_u32(&bars->o_free[t]), (g - 1) & 1, kWaitOFree);
            }
            if (ok) {
              ++p_cnt[hf];
              tc_fence_after_sync();
              H3A_STAMP(2 + t, 2 * it + hf, 1);
              issue_pv(hf, sv);
              H3A_STAMP(2 + t, 2 * it + hf, 2);
            }
          }
          if (ok && has_next && !k_ready) {
            ok = warp_wait(wc, smem_u32(&bars->kv_full[sk]), (ck / kStages) & 1, kWaitKvFullK);
            if (ok) {
              k_ready = true;
              tc_fence_after_sync();
            }
          }
          if (ok && mine_next && (!kFullS || hf == 1)) {
            issue_s(kFullS ? 0 : hf, sk);  // with kFullS: both halves at once (hf offset 0, N = 128)
            H3A_STAMP(2 + t, 2 * it + hf, 3);
          }
        }
        if (!ok) break;
        umma_commit_if(leader, smem_u32(&bars->kv_empty[sv]));
        if (has_next) umma_commit_if(leader, smem_u32(&bars->kv_empty[sk]));
      }
      c0 += 2 * n_it;
      ++g;
      }  // items
    }
    __syncwarp();
   }
  } else {
    setmaxnreg_inc<LY::kSoftmaxRegs>();
    if constexpr (kFixed) {
    // =========================================================== softmax, fixed reference: one warpgroup per (stream, half)
    const int wg = warp >> 2;
    const int t = wg & 1;               // stream
    const int hf = wg >> 1;             // which 64-key half of every tile this warpgroup owns
    const int quarter = warp & 3;       // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t sb = tmem + lane_base + t * kTile + hf * 64;
    const uint32_t o_addr = tmem + lane_base + 256 + t * kTile + hf * 64;  // epilogue: this warpgroup's 64 O columns
    const int last_tile = args.n_kv_tiles - 1;
    const int tail = args.Lk - last_tile * kTile;
    const float m_ref = args.fixed_m;
    // row sums of the stream's two warpgroups meet here (one slot per row, used in turn by the two halves)
    float* lbuf = reinterpret_cast<float*>(smem + 2 * kQTileBytes + kStages * kStageBytes + 256) + t * 128;
    uint32_t j = 0;  // key tiles this warpgroup has processed, over all items: the phase of s_full / o_full
    bool ok = true;
    uint32_t s[64];
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    set_item(item);
    const int q_row = q0 + t * kTile + row;
    const bool row_valid = q_row < args.Lq;
    __nv_bfloat16* orow = out_row_ptr(args, q_row, head) + 64 * hf;
    if (n_it == 0) {  // (block-sparse) neither query tile lists a key tile: zero rows, and no other role does anything
      if (row_valid) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int x = 0; x < 64; x += 8) *reinterpret_cast<uint4*>(orow + x) = z;
        if (args.lse && hf == 0) args.lse[static_cast<long long>(head) * args.Lq + q_row] = -INFINITY;
      }
      continue;
    }
    float qs = 1.0f;
    if constexpr (kFp8) {
      const int qb = min(q0 / kTile + t, args.nqb - 1);
      qs = args.q_scale[head * args.nqb + qb];
    }
    float l_sum = 0.0f;
    const uint32_t j0 = j;
    for (int it = 0; ok && it < n_it; ++it) {
      const int e = entry_at(it);
      if (!((e >> t) & 1)) continue;
      const int tile = e >> 2;
      float c = args.scale_log2;
      if constexpr (kFp8) c *= qs * args.k_scale[head * args.nkb + tile];
      if (row == 0 && t == 0) H3A_STAMP(hf, j, 0);
      // with kFullS one N=128 MMA group fills both halves and signals s_full[t][0] for both warpgroups
      ok = warp_wait(wc, smem_u32(&bars->s_full[t][kFullS ? 0 : hf]), j & 1, kWaitSFull);
      if (!ok) break;
      tc_fence_after_sync();
      tmem_ld32(sb, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld32(sb + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_wait_ld();
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      if (row == 0 && t == 0) H3A_STAMP(hf, j, 2);
      if (tile == last_tile && tail < kTile) {
        const int valid = tail - hf * 64;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i >= valid) s[i] = 0xFF800000u;  // -inf
      }
      l_sum += exp_half_tile<kFp8>(s, c, m_ref);
      if (row == 0 && t == 0) H3A_STAMP(hf, j, 4);
      tmem_st32(sb, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars->p_full[t][hf]));
      if (row == 0 && t == 0) H3A_STAMP(hf, j, 5);
      ++j;
    }
    // ---- epilogue: the two warpgroups of a stream add their row sums through shared memory and each stores 64 of
    //      the 128 output columns.  A warpgroup may be up to a tile ahead of its partner, so it waits for its OWN
    //      last P V (never more than one phase away); two named barriers, which every thread of both warpgroups
    //      always reaches, carry the exchange: half 0 leaves its sum, half 1 swaps it for its own.  Between them ONE
    //      thread reads the abort flag for the stream, so that both warpgroups leave the item loop together (a
    //      warpgroup that went on alone would wait at the next item's named barrier for ever).
    bool have = ok && j > j0;
    if (have) {
      have = warp_wait(wc, smem_u32(&bars->o_full[t][hf]), (j - 1) & 1, kWaitOFull);
      if (have) tc_fence_after_sync();
    }
    if (hf == 0) lbuf[row] = l_sum;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "r"(256) : "memory");
    float l_other = 0.0f;
    if (hf == 1) {
      l_other = lbuf[row];
      lbuf[row] = l_sum;
    } else if (row == 0) {
      bars->stop[t] = bars->abort_flag;
    }
    asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "r"(256) : "memory");
    if (hf == 0) l_other = lbuf[row];
    const bool stop = bars->stop[t] != 0u;
    if (have) {
      // O leaves TMEM first: the next item's first P V may overwrite it while the rows are converted and stored
      tc_fence_after_sync();
      tmem_ld32(o_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld32(o_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_wait_ld();
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&s[32]));
    }
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bars->o_free[t]));  // once per item with work, whether or not the stream had tiles
    if (have) {
      const float l_tot = l_sum + l_other;
      if (hf == 0 && row_valid) check_row_sum(args, l_tot, false);
      const float inv = 1.0f / l_tot;
      if (row_valid) {
#pragma unroll
        for (int x = 0; x < 64; x += 8) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(s[x]) * inv, __uint_as_float(s[x + 1]) * inv);
          w.y = pack_bf16x2(__uint_as_float(s[x + 2]) * inv, __uint_as_float(s[x + 3]) * inv);
          w.z = pack_bf16x2(__uint_as_float(s[x + 4]) * inv, __uint_as_float(s[x + 5]) * inv);
          w.w = pack_bf16x2(__uint_as_float(s[x + 6]) * inv, __uint_as_float(s[x + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + x) = w;
        }
        if (args.lse && hf == 0)
          args.lse[static_cast<long long>(head) * args.Lq + q_row] = (m_ref + log2f(l_tot)) * 0.6931471805599453f;
      }
    } else if (ok && j == j0 && row_valid) {
      const uint4 z = make_uint4(0, 0, 0, 0);  // no key tile listed for this query tile: the output row is zero
#pragma unroll
      for (int x = 0; x < 64; x += 8) *reinterpret_cast<uint4*>(orow + x) = z;
      if (args.lse && hf == 0) args.lse[static_cast<long long>(head) * args.Lq + q_row] = -INFINITY;
    }
    if (stop) break;
    }  // items
    } else {
    // =========================================================== softmax / rescale / epilogue
    const int t = warp >> 2;            // stream
    const int quarter = warp & 3;       // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + t * kTile;
    const uint32_t o_addr = tmem + lane_base + 256 + t * kTile;
    const int q_row = q0 + t * kTile + row;
    const int last_tile = args.n_kv_tiles - 1;
    const int tail = args.Lk - last_tile * kTile;  // valid columns of the last key tile (1..128)

    float qs = 1.0f;
    if constexpr (kFp8) {
      const int qb = min(q0 / kTile + t, args.nqb - 1);
      qs = args.q_scale[head * args.nqb + qb];
    }
    float m_ref = kFixed ? args.fixed_m : 0.0f, l_sum = 0.0f;
    uint32_t j = 0;  // key tiles this stream has processed
    bool ok = true;
    uint32_t ra[64], rb[64];  // two register images of an S half: one being processed, one being prefetched

    auto next_entry = [&](int from) -> int {  // next plan entry that lists this stream, or n_it
      int x = from;
      while (x < n_it && !((entry_at(x) >> t) & 1)) ++x;
      return x;
    };
    // start the TMEM load of S[t][hf] into r (not waited for)
    auto load_s = [&](uint32_t (&r)[64], int hf) {
      tc_fence_after_sync();
      tmem_ld32(s_addr + hf * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
      tmem_ld32(s_addr + hf * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
    };
    // wait for S[t][hf] of the stream's tile number `jt`, then start its load
    auto fetch_s = [&](uint32_t (&r)[64], int hf, uint32_t jt) -> bool {
      const bool got = warp_wait(wc, smem_u32(&bars->s_full[t][hf]), jt & 1, kWaitSFull);
      if (got) load_s(r, hf);
      return got;
    };
    // if S[t][hf] of tile `jt` is already complete start its load now (its latency then hides behind the
    // P store); never block here: P of the current half must not be held back waiting for the tensor pipe
    auto try_fetch_s = [&](uint32_t (&r)[64], int hf, uint32_t jt) -> bool {
      const bool ready = __all_sync(0xFFFFFFFFu, mbar_test_wait(smem_u32(&bars->s_full[t][hf]), jt & 1));
      if (ready) load_s(r, hf);
      return ready;
    };
    // one half-step on the S image in s[]: online max, lazy rescale of O, P = 2^(s c - m) packed into s[0..31]
    auto softmax_half = [&](uint32_t (&s)[64], int hf, int tile, float c) -> bool {
      if (tile == last_tile && tail < kTile) {
        const int valid = tail - hf * 64;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i >= valid) s[i] = 0xFF800000u;  // -inf
      }
      if constexpr (!kFixed) {
      float mx0 = fmax3(__uint_as_float(s[0]), __uint_as_float(s[1]), __uint_as_float(s[2]));
      float mx1 = fmax3(__uint_as_float(s[3]), __uint_as_float(s[4]), __uint_as_float(s[5]));
      float mx2 = fmax3(__uint_as_float(s[6]), __uint_as_float(s[7]), __uint_as_float(s[8]));
      float mx3 = fmax3(__uint_as_float(s[9]), __uint_as_float(s[10]), __uint_as_float(s[11]));
#pragma unroll
      for (int i = 12; i < 60; i += 8) {
        mx0 = fmax3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        mx2 = fmax3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
        mx3 = fmax3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
      }
      mx0 = fmax3(mx0, __uint_as_float(s[60]), __uint_as_float(s[61]));
      mx1 = fmax3(mx1, __uint_as_float(s[62]), __uint_as_float(s[63]));
      const float m_tile = fmax3(fmaxf(mx0, mx1), mx2, mx3) * c;

      if (j == 0 && hf == 0) {
        m_ref = m_tile;
      } else {
        const bool grow = (m_tile - m_ref) > kRescaleThreshold;
        if (__any_sync(0xFFFFFFFFu, grow)) {
          const float m_new = fmaxf(m_ref, m_tile);
          const float alpha = ex2_approx(m_ref - m_new);
          m_ref = m_new;
          l_sum *= alpha;
          // O_t must be quiescent: the previous P V of this stream has to be complete (MMAs complete
          // in issue order, so it is the only one that can still be running).  Each (stream, half)
          // barrier advances one phase per key tile, so a parity wait is never two phases behind.
          if (!warp_wait(wc, smem_u32(&bars->o_full[t][hf ^ 1]), (hf ? j : j - 1) & 1, kWaitOFull))
            return false;
          tc_fence_after_sync();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t o[32];
            tmem_ld32(o_addr + 32 * i, o);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
            tmem_st32(o_addr + 32 * i, o);
          }
        }
      }
      }
      // p = 2^(s c - m): scale-and-subtract as packed FFMA2, exponentials spread over the MUFU and the FMA pipe
      l_sum += exp_half_tile<kFp8>(s, c, m_ref);
      return true;
    };
    // publish P[t][hf] (packed in s[0..31]) to TMEM and tell the issuer
    auto publish_p = [&](uint32_t (&s)[64], int hf) {
      tmem_st32(s_addr + hf * 64, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars->p_full[t][hf]));
    };

    int it = next_entry(0);
    if (it < n_it) {
      ok = fetch_s(ra, 0, 0);
      if (kFullS && ok) load_s(rb, 1);  // one barrier covers both halves
    }
    while (ok && it < n_it) {
      const int tile = entry_at(it) >> 2;
      const int it_next = next_entry(it + 1);
      float c = args.scale_log2;
      if constexpr (kFp8) c *= qs * args.k_scale[head * args.nkb + tile];

      // ---- half 0 from image A; the load of half 1 (image B) is started just before P is published when
      //      that S is already complete, so its latency overlaps the TMEM store and the barrier round trip
      if (row == 0) H3A_STAMP(t, 2 * j, 0);
      tmem_wait_ld();
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&ra[0]));
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&ra[32]));
      if (row == 0) H3A_STAMP(t, 2 * j, 2);
      ok = softmax_half(ra, 0, tile, c);
      if (!ok) break;
      if (row == 0) H3A_STAMP(t, 2 * j, 4);
      if constexpr (kFullS) {
        publish_p(ra, 0);
      } else {
        const bool early = try_fetch_s(rb, 1, j);
        publish_p(ra, 0);
        if (!early) ok = fetch_s(rb, 1, j);
        if (!ok) break;
      }
      if (row == 0) H3A_STAMP(t, 2 * j, 5);

      // ---- half 1 from image B; prefetch half 0 of the stream's next tile into image A
      if (row == 0) H3A_STAMP(t, 2 * j + 1, 0);
      tmem_wait_ld();
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&rb[0]));
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&rb[32]));
      if (row == 0) H3A_STAMP(t, 2 * j + 1, 2);
      ok = softmax_half(rb, 1, tile, c);
      if (!ok) break;
      if (row == 0) H3A_STAMP(t, 2 * j + 1, 4);
      if constexpr (kFullS) {
        publish_p(rb, 1);
        if (it_next < n_it) {
          ok = fetch_s(ra, 0, j + 1);
          if (!ok) break;
          load_s(rb, 1);
        }
      } else {
        const bool early = (it_next < n_it) && try_fetch_s(ra, 0, j + 1);
        publish_p(rb, 1);
        if (!early && it_next < n_it) ok = fetch_s(ra, 0, j + 1);
        if (!ok) break;
      }
      if (row == 0) H3A_STAMP(t, 2 * j + 1, 5);
      ++j;
      it = it_next;
    }

    // ---- epilogue: O / l -> bf16 -> global
    const bool row_valid = q_row < args.Lq;
    __nv_bfloat16* orow = out_row_ptr(args, q_row, head);
    if (ok && j > 0) {
      ok = warp_wait(wc, smem_u32(&bars->o_full[t][1]), (j - 1) & 1, kWaitOFull);
      if (ok) {
        tc_fence_after_sync();
        const float inv = 1.0f / l_sum;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t o[32];
          tmem_ld32(o_addr + 32 * i, o);
          tmem_wait_ld();
          if (row_valid) {
#pragma unroll
            for (int x = 0; x < 32; x += 8) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(o[x]) * inv, __uint_as_float(o[x + 1]) * inv);
              w.y = pack_bf16x2(__uint_as_float(o[x + 2]) * inv, __uint_as_float(o[x + 3]) * inv);
              w.z = pack_bf16x2(__uint_as_float(o[x + 4]) * inv, __uint_as_float(o[x + 5]) * inv);
              w.w = pack_bf16x2(__uint_as_float(o[x + 6]) * inv, __uint_as_float(o[x + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + 32 * i + x) = w;
            }
          }
        }
        if (row_valid && args.lse)
          args.lse[static_cast<long long>(head) * args.Lq + q_row] = (m_ref + log2f(l_sum)) * 0.6931471805599453f;
      }
    } else if (ok && row_valid) {
      // no key tile listed for this query tile: the output row is zero
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int x = 0; x < 128; x += 8) *reinterpret_cast<uint4*>(orow + x) = z;
      if (args.lse) args.lse[static_cast<long long>(head) * args.Lq + q_row] = -INFINITY;
    }
    }
  }

  // ---- tear-down
  if (args.o_n_ranks > 1) __threadfence_system();  // rows stored into other GPUs' memory
  tc_fence_before_sync();
  __syncthreads();
  if (bars->abort_flag) {
    // a wait gave up: give copies and MMAs in flight a bounded time to land before TMEM and smem go away
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == kIssuerWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace h3a
