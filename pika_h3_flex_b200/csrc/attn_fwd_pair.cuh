// Forward attention on CTA PAIRS (fixed softmax reference): two CTAs on neighbouring SMs (a cluster of two) run every MMA
// together (tcgen05 cta_group::2, M = 256 = 128 query rows in each CTA), so each CTA stages only HALF of every
// K and V tile in its shared memory and fetches half of the B operand per MMA.  The single-CTA kernel is bound by
// shared-memory bandwidth (operand fetch plus TMA writes); the pair moves 30 % fewer bytes through each SM's
// shared memory for the same math.
//
// A pair owns four consecutive 128-row query tiles of one head; stream t of CTA r (rank in the cluster) is tile
// 4 c + 2 t + r, so one M = 256 MMA covers two ADJACENT query tiles (in the block-sparse mode their key lists
// overlap most, and a key tile is computed for both when either lists it).  Per CTA, as in the single-CTA kernel:
//   warp 16  producer : TMA loads of its Q tiles (once) and of ITS HALF of K_j / V_j into a ring of 16 KB stages;
//                       the bytes of both CTAs are counted on the mbarriers of rank 0
//   warps 17,18       : rank 0 only - one issuer per stream; S = Q_t K^T (N = 64 keys per MMA group, 32 key rows
//                       from each CTA) and O_t += P V (P from TMEM, each CTA supplies 64 of V's 128 columns);
//                       every commit is sent to the barrier in both CTAs
//   warps 0-15        : softmax with the fixed reference, one warpgroup per (stream, 64-key half); P is published
//                       with one arrive per warp on rank 0's barrier (local or through the cluster)
// kFixed = true: the fixed-reference softmax (dense bf16, FP8-QK, block-sparse), 16 softmax warps as above.
// kFixed = false (dense bf16 and FP8-QK): the online softmax with a running row maximum and lazy rescaling of O in
// TMEM, for callers that cannot bound their logits: 8 softmax warps, one warpgroup per stream walking both halves of
// every tile exactly as in the single-CTA kernel; the issuers then also signal the completion of every P V
// (o_done), which a rescale has to wait for.
//
// Block-sparse: the four key-tile lists of a pair are merged into one plan, entry = (key tile << 4) | flags, flag
// bit 2 t + r set when query tile 4 c + 2 t + r lists the key tile.  Both CTAs load every listed tile; stream t
// computes an entry when either of its two query tiles lists it, and the CTA whose tile does not writes P = 0.
//
// Shared memory of a CTA:  Q tiles 2 x 32 KB | ring of 8 stages x 16 KB | barriers
//   K stage (bf16): [dim half][64-key half][32 keys][128 B]   - the 32 keys this CTA supplies to each N = 64 group
//   K stage (e4m3): [64-key half][32 keys][128 B]
//   V stage       : [128 keys][64 dims]                       - this CTA's half of the output columns
// TMEM: as in the single-CTA kernel, at the same addresses in both CTAs.
//
// Dense launches may split the key range for the pairs of the last, partly filled wave (AttnArgs::split_begin):
// those pairs store un-normalised partial rows and combine_partials_kernel adds the shares.
//
// Cluster protocol.  A cluster barrier after the mbarrier set-up (no remote arrive or TMA completion may reach
// an uninitialised barrier) and one before TMEM is freed (no CTA leaves while its peer may still signal its
// barriers or the pair's MMAs may still run).  Every thread reaches both on every path; all other waits are
// bounded as in the single-CTA kernel, and a CTA that gives up also raises its peer's abort flag.
#pragma once
#include "attn_fwd.cuh"

namespace h3a {

#ifndef H3A_PAIR_STAGES
#define H3A_PAIR_STAGES 8
#endif
constexpr int kPairStages = H3A_PAIR_STAGES;
constexpr int kPairStageBytes = 16384;
constexpr int kPairThreads = AttnLayout<true>::kThreads;  // fixed-reference kernels; the running-maximum ones use AttnLayout<false>

struct PairBars {
  uint64_t kv_full[kPairStages];   // waited on in rank 0: counts the bytes of both CTAs' halves
  uint64_t kv_empty[kPairStages];  // in both CTAs: one commit from each of rank 0's issuers
  uint64_t q_full;                 // rank 0
  uint64_t s_full[2][2];           // [stream][half], both CTAs
  uint64_t p_full[2][2];           // rank 0: one arrive per softmax warp of the (stream, half) warpgroup of BOTH CTAs
  uint64_t o_full[2];              // both CTAs: every MMA of stream t has completed (one phase, after the last tile)
  uint64_t o_done[2][2];           // both CTAs, running-maximum kernels: the P V of (stream, half) has completed, one phase per tile
  uint64_t drain[2];               // rank 0: last commit of issuer t
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  uint32_t early_exit;
  volatile uint32_t redo;          // kRowRef: a row of this pair outgrew its reference (rank 1 also raises rank 0's)
  // kResident (persistent pairs, K / V of a head kept in shared memory)
  uint64_t q_empty;                // both CTAs: every S MMA of an item has completed (one commit from each issuer)
  uint64_t o_free[2];              // rank 0: the softmax warps of stream t in BOTH CTAs have read O of an item (16 arrives)
  volatile uint32_t stop[2];       // per stream: one thread's reading of abort_flag, so that both warpgroups leave together
};
static_assert(sizeof(PairBars) <= 512, "barrier block too large");

constexpr int kPairRowRefBytes = 2 * 2 * 128 * 4;  // kRowRef: first-tile maxima, [stream][half][row] fp32
constexpr int kPairSmemBytes = 2 * kQTileBytes + kPairStages * kPairStageBytes + 1024 /*align slack*/ + 512 /*barriers*/ + kPairRowRefBytes;
static_assert(kPairSmemBytes <= 232448, "shared memory budget");
// kResident: between the ring and the barrier block, two 1 KB buffers per softmax warp (8 rows x 128 bytes each, in the
// 128-byte swizzle, hence 1024-byte aligned) through which the output rows leave as TMA tile stores
constexpr int kPairStoreStageBytes = 1024;
constexpr int kPairStoreStages = 2;
constexpr int kPairResidentStageBytes = 16 * kPairStoreStages * kPairStoreStageBytes;
constexpr int kPairResidentSmemBytes = kPairSmemBytes - kPairRowRefBytes / 2 + kPairResidentStageBytes;  // row sums need 1 KB
static_assert(kPairResidentSmemBytes <= 232448, "shared memory budget");

enum : int { kWaitDrain = 8 };
// S production: 0 = one N = 64 MMA group per 64-key half (32 key rows from each CTA); 1 = one N = 128 group per key
// tile (64 key rows from each CTA, 25 % less operand traffic, but both halves of a stream become available, and
// are needed back, together: two dependency chains per CTA instead of four; measured 11 % slower).  The host
// picks the matching K box (32 or 64 rows) from kPairKBoxRows.
#ifndef H3A_PAIR_FULL_S
#define H3A_PAIR_FULL_S 0
#endif
constexpr bool kPairFullS = H3A_PAIR_FULL_S != 0;
constexpr int kPairKBoxRows = kPairFullS ? 64 : 32;
#ifndef H3A_PAIR_SOFTMAX_REGS
#define H3A_PAIR_SOFTMAX_REGS 104
#endif
#ifndef H3A_PAIR_HELPER_REGS
#define H3A_PAIR_HELPER_REGS 64
#endif
constexpr int kPairSoftmaxRegs = H3A_PAIR_SOFTMAX_REGS, kPairHelperRegs = H3A_PAIR_HELPER_REGS;
static_assert(512 * kPairSoftmaxRegs + 128 * kPairHelperRegs <= AttnLayout<true>::kLaunchRegs * kPairThreads,
              "setmaxnreg budget exceeds the launch allocation");

// Merge the sorted key-tile lists of query tiles 4c .. 4c+3 into one list with a flag bit per query tile.
// The index is checked as in build_pair_plan_kernel.
__global__ void build_cluster_plan_kernel(const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ col_idx,
                                          int nqb, int n_clusters, int nnz, int nkb, int32_t* __restrict__ plan,
                                          int32_t* __restrict__ plan_cnt, int* __restrict__ status) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n_clusters) return;
  bool bad = false;
  int pos[4], end[4];
  for (int i = 0; i < 4; ++i) row_range(row_ptr, 4 * c + i, nqb, nnz, pos[i], end[i], bad);
  int32_t* out = plan + pos[0];  // the merged list is never longer than the four lists together
  const int cap = nnz - pos[0];
  int n = 0, prev = -1;
  for (;;) {
    int lo = 0x7FFFFFFF;
    for (int i = 0; i < 4; ++i)
      if (pos[i] < end[i]) lo = min(lo, col_idx[pos[i]]);
    if (lo == 0x7FFFFFFF) break;
    int f = 0;
    for (int i = 0; i < 4; ++i)
      if (pos[i] < end[i] && col_idx[pos[i]] == lo) {
        f |= 1 << i;
        ++pos[i];
      }
    if (lo <= prev || lo >= nkb || n >= cap) { bad = true; continue; }
    prev = lo;
    out[n++] = (lo << 4) | f;
  }
  plan_cnt[c] = n;
  if (bad) report_bad_index(status, 4 * c);
}

// Partial results of the split pairs: `part` holds [slot][4 query tiles][128 rows][128] un-normalised output sums,
// then [slot][4][128] row sums; slot = (pair - split_begin) * kv_splits + share.
__device__ __forceinline__ long long part_slots(const AttnArgs& a, int n_clusters) {
  return static_cast<long long>(n_clusters * a.H - a.split_begin) * a.kv_splits;
}
// Adds the shares up and writes the rows: one block per (split group of four query tiles, query tile), 16
// threads per row (8 columns each), 16 rows per pass.
__global__ void combine_partials_kernel(const AttnArgs args, int n_clusters) {
  // a wait gave up (now or in an earlier launch on this status word): the shares are incomplete, write nothing
  if (args.status != nullptr && *reinterpret_cast<volatile int*>(args.status) != 0) return;
  const int g = blockIdx.x >> 2, tile_in_group = blockIdx.x & 3;
  const int cidx = args.split_begin + g;
  const int head = cidx / n_clusters, cl = cidx % n_clusters;
  const int sub = threadIdx.x & 15, r0 = threadIdx.x >> 4;
  const float* part_l = args.part + part_slots(args, n_clusters) * 4 * 128 * 128;
  for (int row = r0; row < 128; row += 16) {
    const int q_row = (4 * cl + tile_in_group) * kTile + row;
    if (q_row >= args.Lq) break;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float l = 0.f;
    for (int s = 0; s < args.kv_splits; ++s) {
      const long long rix = (static_cast<long long>(g * args.kv_splits + s) * 4 + tile_in_group) * 128 + row;
      const float4 a = *reinterpret_cast<const float4*>(args.part + rix * 128 + 8 * sub);
      const float4 b = *reinterpret_cast<const float4*>(args.part + rix * 128 + 8 * sub + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      l += part_l[rix];
    }
    if (sub == 0) check_row_sum(args, l, false);
    const float inv = 1.0f / l;
    uint4 w;
    w.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
    w.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
    w.z = pack_bf16x2(acc[4] * inv, acc[5] * inv);
    w.w = pack_bf16x2(acc[6] * inv, acc[7] * inv);
    __nv_bfloat16* orow = out_row_ptr(args, q_row, head);
    *reinterpret_cast<uint4*>(orow + 8 * sub) = w;
    if (sub == 0 && args.lse) args.lse[static_cast<long long>(head) * args.Lq + q_row] = (args.fixed_m + log2f(l)) * 0.6931471805599453f;
  }
  if (args.o_n_ranks > 1) __threadfence_system();  // rows stored into other GPUs' memory
}

// kRowRef (with kFixed, dense): no caller-supplied bound.  The reference of a row is the maximum of ITS logits over the
// first key tile (the two warpgroups that share the row exchange their halves' maxima once, through shared memory), and
// stays fixed: every term is then at most 2^(growth of the row maximum after the first tile), exact in floating point
// until that growth passes about 60 in log2 units.  A half tile whose terms sum to more than 2^60 marks the pair for
// the second launch (AttnArgs::redo_list), which recomputes its four query tiles with the running-maximum kernel.
//
// kResident (with kFixed, dense bf16, at most kPairStages / 2 key tiles: cross-attention to a few hundred text tokens):
// the ring holds ALL of a head's K and V (each CTA its halves), loaded once per head, and the pair is persistent: the
// launch has one pair per two SMs, pair c walks the contiguous items [T c / C, T (c + 1) / C) of the head-major list
// of (head, group of four query tiles), so the head changes at most a few times per pair.  Per item only the Q tiles
// are loaded and the O rows stored; the Q load and the first S MMAs of the next item run under the epilogue of the
// current one (q_empty: the Q tiles are free; o_free: O has been read out of TMEM).
template <bool kFp8, bool kSparse, bool kFixed = true, bool kRowRef = false, bool kResident = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(AttnLayout<kFixed>::kThreads, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const AttnArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // the same offset in both CTAs: MMA descriptors are shared
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t q_smem = base;
  const uint32_t ring_smem = base + 2 * kQTileBytes;
  constexpr int kBarsOff = 2 * kQTileBytes + kPairStages * kPairStageBytes + (kResident ? kPairResidentStageBytes : 0);
  PairBars* bars = reinterpret_cast<PairBars*>(smem + kBarsOff);

  static_assert(kFixed || (!kSparse && !kPairFullS), "the running-maximum pair kernel is dense, with N = 64 S groups");
  static_assert(!kRowRef || (kFixed && !kSparse && !kPairFullS), "per-row references: dense, on the fixed-reference structure");
  static_assert(!kResident || (kFixed && !kSparse && !kRowRef && !kFp8 && !kPairFullS), "resident K / V: dense bf16, fixed reference");
  using LY = AttnLayout<kFixed>;
  constexpr int kHelperRegs = kFixed ? kPairHelperRegs : LY::kHelperRegs;
  constexpr int kSoftmaxRegs = kFixed ? kPairSoftmaxRegs : LY::kSoftmaxRegs;
  constexpr int kProducerWarp = LY::kSoftmaxWarps;
  constexpr int kIssuerWarp = LY::kSoftmaxWarps + 1;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int n_clusters = (args.Lq + 4 * kTile - 1) / (4 * kTile);
  int cid = blockIdx.x >> 1;
  int item_begin = 0, item_end = 0;  // kResident: this pair's share of the items
  if constexpr (kResident) {
    const long long total = static_cast<long long>(n_clusters) * args.H, n_pairs = gridDim.x >> 1;
    item_begin = static_cast<int>(total * cid / n_pairs);
    item_end = static_cast<int>(total * (cid + 1) / n_pairs);
    cid = item_begin;
  }
  if constexpr (!kFixed) {
    // second launch of the two-launch online softmax: only the listed pairs are redone.  Both CTAs of a pair read the
    // same count and leave together, before any cluster-wide state exists.
    if (args.redo_count != nullptr) {
      if (cid >= *args.redo_count) return;
      cid = args.redo_list[cid];
    }
  }
  // dense: the pairs from split_begin on share their group of query tiles with kv_splits - 1 others
  int split = 0, n_splits = 1, part_slot = -1;
  if constexpr (!kSparse) {
    if (args.kv_splits > 1 && cid >= args.split_begin) {
      const int x = cid - args.split_begin;
      n_splits = args.kv_splits;
      split = x % n_splits;
      cid = args.split_begin + x / n_splits;
      part_slot = x;
    }
  }
  // pair -> (head, group of four query tiles): head-major; block-sparse: the groups with long key lists (dense
  // audio rows) of ALL heads first, as in the single-CTA kernel
  int head = cid / n_clusters, cl = cid % n_clusters;
  if constexpr (kSparse) {
    const int heavy = (args.heavy_pairs + 1) / 2;
    if (heavy > 0 && heavy < n_clusters) {
      if (cid < heavy * args.H) {
        head = cid / heavy;
        cl = cid % heavy;
      } else {
        const int r = cid - heavy * args.H, n_light = n_clusters - heavy;
        head = r / n_light;
        cl = heavy + r % n_light;
      }
    }
  }
  auto q_tile = [&](int t) { return 4 * cl + 2 * t + static_cast<int>(rank); };  // query tile of this CTA's stream t

  // ---- plan: which key tiles, for which of the pair's four query tiles
  int n_it;
  const int32_t* plan = nullptr;
  if constexpr (kSparse) {
    plan = args.plan + clamp_row_ptr(args.row_ptr[min(4 * cl, args.nqb)], args.nnz);
    n_it = args.plan_cnt[cl];
  } else {
    n_it = args.n_kv_tiles;
  }
  int it0 = 0;  // first key tile of this pair's share
  if constexpr (!kSparse) {
    it0 = (args.n_kv_tiles * split) / n_splits;
    n_it = (args.n_kv_tiles * (split + 1)) / n_splits - it0;
  }
  auto entry_at = [&](int it) -> int {
    if constexpr (kSparse) return plan[it];
    else return ((it0 + it) << 4) | 15;
  };
  auto stream_needs = [](int e, int t) { return ((e >> (2 * t)) & 3) != 0; };

  constexpr uint32_t kQBytes = kFp8 ? kHalfBytes : kQTileBytes;  // bytes per Q tile
  constexpr uint32_t kKHalfBytes = kFp8 ? 8192 : 16384;          // this CTA's half of a K tile
  constexpr uint32_t kVHalfBytes = 16384;

  // ---- set-up
  if (threadIdx.x == 0) {
    for (int i = 0; i < kPairStages; ++i) {
      mbar_init(smem_u32(&bars->kv_full[i]), 1);
      mbar_init(smem_u32(&bars->kv_empty[i]), 2);
    }
    mbar_init(smem_u32(&bars->q_full), 1);
    for (int t = 0; t < 2; ++t) {
      for (int hf = 0; hf < 2; ++hf) {
        mbar_init(smem_u32(&bars->s_full[t][hf]), 1);
        mbar_init(smem_u32(&bars->p_full[t][hf]), 8);
      }
      mbar_init(smem_u32(&bars->o_full[t]), 1);
      mbar_init(smem_u32(&bars->o_done[t][0]), 1);
      mbar_init(smem_u32(&bars->o_done[t][1]), 1);
      mbar_init(smem_u32(&bars->drain[t]), 1);
      mbar_init(smem_u32(&bars->o_free[t]), 16);
      bars->stop[t] = 0;
    }
    mbar_init(smem_u32(&bars->q_empty), 2);
    bars->abort_flag = 0;
    bars->redo = 0;
    bars->early_exit = (args.status != nullptr && *reinterpret_cast<volatile int*>(args.status) != 0) ? 1u : 0u;
    fence_mbar_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
  }
  cluster_sync_all();  // barriers of both CTAs are initialised; rank 0's verdict below is visible
  // an earlier CTA of this launch already gave up: the pair does nothing (rank 0 decides for both)
  const bool run = ld_shared_cluster_u32(mapa_shared(smem_u32(&bars->early_exit), 0)) == 0u;
  uint32_t tmem = 0;
  const uint32_t bars0 = mapa_shared(smem_u32(bars), 0);         // rank 0's barrier block
  const uint32_t bars_peer = mapa_shared(smem_u32(bars), rank ^ 1u);
  auto at0 = [&](const void* local) { return bars0 + (smem_u32(local) - smem_u32(bars)); };
  auto at_peer = [&](const void* local) { return bars_peer + (smem_u32(local) - smem_u32(bars)); };
  WaitCtx wc{smem_u32(const_cast<const uint32_t*>(&bars->abort_flag)), at_peer(const_cast<const uint32_t*>(&bars->abort_flag)), &args};

  if (run) {
  if (warp == kIssuerWarp) {
    tmem_alloc_pair(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  tmem = bars->tmem_base;

  if (warp >= LY::kSoftmaxWarps) {
   setmaxnreg_dec<kHelperRegs>();
   if (warp == kProducerWarp) {
    // =========================================================== producer (both CTAs)
    const uint32_t leader = elect_one();
    if constexpr (kResident) {
      bool ok = true;
      uint32_t g = 0, hl = 0;  // items so far (phase of q_full / q_empty); heads loaded so far (phase of kv_full / kv_empty[0])
      int prev_head = -1;
      for (int item = item_begin; ok && item < item_end; ++item) {
        if (item > item_begin && ++cl == n_clusters) {  // (head, cl) = (item / n_clusters, item % n_clusters), without dividing
          cl = 0;
          ++head;
        }
        if (head != prev_head) {
          if (prev_head >= 0) {  // every MMA that reads the previous head's K / V has completed
            ok = warp_wait(wc, smem_u32(&bars->kv_empty[0]), (hl - 1) & 1, kWaitKvEmpty);
            if (!ok) break;
          }
          for (int it = 0; it < n_it; ++it) {  // key tile `it`: K halves in stage 2 it, V columns in stage 2 it + 1
            const int sk = 2 * it, sv = 2 * it + 1;
            if (rank == 0) mbar_arrive_expect_tx_if(leader, smem_u32(&bars->kv_full[sk]), 2 * kKHalfBytes);
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              const int key0 = it * kTile + 64 * hf + 32 * static_cast<int>(rank);
              tma_load_3d_pair_if(leader, ring_smem + sk * kPairStageBytes + hf * 4096, &tm_k, at0(&bars->kv_full[sk]), 0, key0, head);
              tma_load_3d_pair_if(leader, ring_smem + sk * kPairStageBytes + 8192 + hf * 4096, &tm_k, at0(&bars->kv_full[sk]), 64, key0, head);
            }
            if (rank == 0) mbar_arrive_expect_tx_if(leader, smem_u32(&bars->kv_full[sv]), 2 * kVHalfBytes);
            tma_load_3d_pair_if(leader, ring_smem + sv * kPairStageBytes, &tm_v, at0(&bars->kv_full[sv]), 64 * static_cast<int>(rank), it * kTile, head);
          }
          ++hl;
          prev_head = head;
        }
        if (g > 0) {  // the Q tiles are free when every S MMA of the previous item has completed
          ok = warp_wait(wc, smem_u32(&bars->q_empty), (g - 1) & 1, kWaitQEmpty);
          if (!ok) break;
        }
        if (rank == 0) mbar_arrive_expect_tx_if(leader, smem_u32(&bars->q_full), 2 * 2 * kQBytes);
        const uint32_t qbar = at0(&bars->q_full);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          tma_load_3d_pair_if(leader, q_smem + t * kQTileBytes, &tm_q, qbar, 0, q_tile(t) * kTile, head);
          tma_load_3d_pair_if(leader, q_smem + t * kQTileBytes + kHalfBytes, &tm_q, qbar, 64, q_tile(t) * kTile, head);
        }
        ++g;
      }
    } else {
    {
      if (rank == 0) mbar_arrive_expect_tx_if(leader, smem_u32(&bars->q_full), 2 * 2 * kQBytes);  // Q tiles of both CTAs
      const uint32_t qbar = at0(&bars->q_full);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        tma_load_3d_pair_if(leader, q_smem + t * kQTileBytes, &tm_q, qbar, 0, q_tile(t) * kTile, head);
        if constexpr (!kFp8) tma_load_3d_pair_if(leader, q_smem + t * kQTileBytes + kHalfBytes, &tm_q, qbar, 64, q_tile(t) * kTile, head);
      }
    }
    int cnt = 0;
    bool ok = true;
    for (int it = 0; ok && it < n_it; ++it) {
      const int tile = entry_at(it) >> 4;
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {  // K half-tile, then V half-tile
        const int s = cnt % kPairStages;
        const uint32_t ph = (cnt / kPairStages) & 1;
        ok = warp_wait(wc, smem_u32(&bars->kv_empty[s]), ph ^ 1u, kWaitKvEmpty);
        if (!ok) break;
        const uint32_t fb = at0(&bars->kv_full[s]);
        const uint32_t dst = ring_smem + s * kPairStageBytes;
        if (kv == 0) {
          if (rank == 0) mbar_arrive_expect_tx_if(leader, smem_u32(&bars->kv_full[s]), 2 * kKHalfBytes);
          if constexpr (kPairFullS) {  // the 64 keys this CTA supplies to the N = 128 group
            const int key0 = tile * kTile + 64 * static_cast<int>(rank);
            tma_load_3d_pair_if(leader, dst, &tm_k, fb, 0, key0, head);
            if constexpr (!kFp8) tma_load_3d_pair_if(leader, dst + 8192, &tm_k, fb, 64, key0, head);
          } else {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {  // the 32 keys this CTA supplies to the N = 64 group of half hf
              const int key0 = tile * kTile + 64 * hf + 32 * static_cast<int>(rank);
              tma_load_3d_pair_if(leader, dst + hf * 4096, &tm_k, fb, 0, key0, head);
              if constexpr (!kFp8) tma_load_3d_pair_if(leader, dst + 8192 + hf * 4096, &tm_k, fb, 64, key0, head);
            }
          }
        } else {
          if (rank == 0) mbar_arrive_expect_tx_if(leader, smem_u32(&bars->kv_full[s]), 2 * kVHalfBytes);
          tma_load_3d_pair_if(leader, dst, &tm_v, fb, 64 * static_cast<int>(rank), tile * kTile, head);
        }
        ++cnt;
      }
    }
    }  // !kResident
    __syncwarp();
  } else if ((warp == kIssuerWarp || warp == kIssuerWarp + 1) && rank == 0) {
    // =========================================================== MMA issuers of the pair (rank 0), one warp per stream
    if constexpr (kResident) {
      const int t = warp - kIssuerWarp;
      const uint32_t leader = elect_one();
      constexpr uint32_t idesc_s = umma_idesc(UMMA_FMT_BF16, UMMA_FMT_BF16, 0, 0, 256, 64);
      constexpr uint32_t idesc_pv = umma_idesc(UMMA_FMT_BF16, UMMA_FMT_BF16, 0, 1, 256, 128);
      const uint64_t q_desc = umma_desc_sw128(q_smem + t * kQTileBytes, 16, 1024);
      const uint64_t kv_desc0 = umma_desc_sw128(ring_smem, 16, 1024);
      const uint32_t s_tmem = tmem + t * kTile;
      const uint32_t o_tmem = tmem + 256 + t * kTile;
      uint32_t p_cnt[2] = {0, 0};  // P halves consumed so far (all items): the phase of p_full
      uint32_t pv_cnt = 0;         // P V groups of the current item: the first overwrites O
      uint32_t g = 0, hl = 0;
      int prev_head = -1;
      bool ok = true;
      auto commit_both = [&](const void* local) {
        umma_pair_commit_if(leader, smem_u32(local));
        umma_pair_commit_if(leader, at_peer(local));
      };
      auto issue_s = [&](int hf, int sk) {
        const uint64_t kd = kv_desc0 + static_cast<uint64_t>((sk * kPairStageBytes + hf * 4096) >> 4);
        const uint32_t d = s_tmem + hf * 64;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t offq = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
          const uint32_t offk = ((k >> 2) * 8192 + (k & 3) * 32) >> 4;
          umma_pair_bf16_ss_if(leader, d, q_desc + offq, kd + offk, idesc_s, k > 0);
        }
        commit_both(&bars->s_full[t][hf]);
      };
      auto issue_pv = [&](int hf, int sv) {
        const uint64_t vd = kv_desc0 + static_cast<uint64_t>((sv * kPairStageBytes + hf * 8192) >> 4);
        const uint32_t a = s_tmem + hf * 64;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_pair_bf16_ts_if(leader, o_tmem, a + k * 8, vd + (k * 2048 >> 4), idesc_pv, (pv_cnt > 0 || k > 0) ? 1u : 0u);
        ++pv_cnt;
      };
      for (int item = item_begin; ok && item < item_end; ++item) {
        if (item > item_begin && ++cl == n_clusters) {
          cl = 0;
          ++head;
        }
        const bool fresh = head != prev_head;  // this head's K / V is being loaded: wait for each stage at its first use
        if (fresh) {
          ++hl;
          prev_head = head;
        }
        const uint32_t kv_par = (hl - 1) & 1;
        const bool last_of_head = item + 1 < item_end && cl + 1 == n_clusters;
        H3A_STAMP(2 + t, g * n_it * 2, 4);
        ok = warp_wait(wc, smem_u32(&bars->q_full), g & 1, kWaitQFull);
        if (!ok) break;
        H3A_STAMP(2 + t, g * n_it * 2, 5);
        if (fresh) {
          ok = warp_wait(wc, smem_u32(&bars->kv_full[0]), kv_par, kWaitKvFullK);
          if (!ok) break;
        }
        tc_fence_after_sync();
        pv_cnt = 0;
        issue_s(0, 0);  // in TMEM these follow the previous item's last P V: MMAs run in issue order
        issue_s(1, 0);
        for (int it = 0; ok && it < n_it; ++it) {
          const bool has_next = (it + 1 < n_it);
          const int sv = 2 * it + 1, sk = 2 * it + 2;
          if (!has_next) commit_both(&bars->q_empty);  // every S MMA of the item has been issued
          if (fresh) {
            ok = warp_wait(wc, smem_u32(&bars->kv_full[sv]), kv_par, kWaitKvFullV);
            if (!ok) break;
            tc_fence_after_sync();
          }
          bool k_ready = !fresh;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            H3A_STAMP(2 + t, (g * n_it + it) * 2 + hf, 0);
            ok = warp_wait(wc, smem_u32(&bars->p_full[t][hf]), p_cnt[hf] & 1, kWaitPFull);
            if (!ok) break;
            H3A_STAMP(2 + t, (g * n_it + it) * 2 + hf, 1);
            ++p_cnt[hf];
            if (pv_cnt == 0 && g > 0) {
              // the first P V of an item overwrites O in both CTAs: their softmax warps must have read the previous item's
              ok = warp_wait(wc, smem_u32(&bars->o_free[t]), (g - 1) & 1, kWaitOFree);
              if (!ok) break;
            }
            tc_fence_after_sync();
            H3A_STAMP(2 + t, (g * n_it + it) * 2 + hf, 2);
            issue_pv(hf, sv);
            H3A_STAMP(2 + t, (g * n_it + it) * 2 + hf, 3);
            if (has_next && !k_ready) {
              ok = warp_wait(wc, smem_u32(&bars->kv_full[sk]), kv_par, kWaitKvFullK);
              if (!ok) break;
              k_ready = true;
              tc_fence_after_sync();
            }
            if (has_next) issue_s(hf, sk);
          }
        }
        if (!ok) break;
        commit_both(&bars->o_full[t]);  // one phase per item: every MMA of the stream's item has completed
        if (last_of_head) commit_both(&bars->kv_empty[0]);  // ... and with it every reader of this head's K / V
        ++g;
      }
      if (ok) {  // nothing of this issuer is still on its way to the peer CTA once this has arrived
        umma_pair_commit_if(leader, smem_u32(&bars->drain[t]));
        warp_wait(wc, smem_u32(&bars->drain[t]), 0, kWaitDrain);
      }
    } else
    if (n_it > 0) {
      const int t = warp - kIssuerWarp;
      const uint32_t leader = elect_one();
      constexpr uint32_t kSN = kPairFullS ? 128 : 64;
      constexpr uint32_t idesc_s = kFp8 ? umma_idesc(UMMA_FMT_E4M3, UMMA_FMT_E4M3, 0, 0, 256, kSN)
                                        : umma_idesc(UMMA_FMT_BF16, UMMA_FMT_BF16, 0, 0, 256, kSN);
      constexpr uint32_t idesc_pv = umma_idesc(UMMA_FMT_BF16, UMMA_FMT_BF16, 0, 1, 256, 128);
      bool ok = warp_wait(wc, smem_u32(&bars->q_full), 0, kWaitQFull);
      tc_fence_after_sync();
      uint32_t p_cnt[2] = {0, 0};
      uint32_t pv_cnt = 0;
      const uint64_t q_desc = umma_desc_sw128(q_smem + t * kQTileBytes, 16, 1024);
      const uint64_t k_desc0 = umma_desc_sw128(ring_smem, 16, 1024);
      const uint64_t v_desc0 = umma_desc_sw128(ring_smem, 16, 1024);
      const uint32_t s_tmem = tmem + t * kTile;
      const uint32_t o_tmem = tmem + 256 + t * kTile;
      // one commit for each CTA's copy of the barrier (a single instruction that signals both was measured
      // and is not faster)
      auto commit_both = [&](const void* local) {
        umma_pair_commit_if(leader, smem_u32(local));
        umma_pair_commit_if(leader, at_peer(local));
      };
      // S[t][hf] = Q_t K[hf]^T for keys [64 hf, +64) of ring stage `sk`: 32 key rows from each CTA
      auto issue_s = [&](int hf, int sk) {
        const uint64_t kd = k_desc0 + static_cast<uint64_t>((sk * kPairStageBytes + hf * 4096) >> 4);
        const uint32_t d = s_tmem + hf * 64;
        if constexpr (kFp8) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_pair_e4m3_ss_if(leader, d, q_desc + (k * 32 >> 4), kd + (k * 32 >> 4), idesc_s, k > 0);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {  // dims 64..127: second box of Q (16 KB on) and of this K half (8 KB on)
            const uint32_t offq = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
            const uint32_t offk = ((k >> 2) * 8192 + (k & 3) * 32) >> 4;
            umma_pair_bf16_ss_if(leader, d, q_desc + offq, kd + offk, idesc_s, k > 0);
          }
        }
        commit_both(&bars->s_full[t][hf]);
      };
      // O_t += P[t][hf] V[hf]: A = P from each CTA's TMEM, B = this CTA's 64 columns of V, MN-major
      auto issue_pv = [&](int hf, int sv) {
        const uint64_t vd = v_desc0 + static_cast<uint64_t>((sv * kPairStageBytes + hf * 8192) >> 4);
        const uint32_t a = s_tmem + hf * 64;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_pair_bf16_ts_if(leader, o_tmem, a + k * 8, vd + (k * 2048 >> 4), idesc_pv, (pv_cnt > 0 || k > 0) ? 1u : 0u);
        ++pv_cnt;
        if constexpr (!kFixed) commit_both(&bars->o_done[t][hf]);  // a rescale of O waits for this
      };

      // Each issuer walks every plan entry, also those its stream skips: a K/V stage is released by one commit
      // from each issuer, and waiting for the stage first keeps the two in step.
      if (ok) {  // prologue: both S halves of entry 0
        ok = warp_wait(wc, smem_u32(&bars->kv_full[0]), 0, kWaitKvFullK);
        if (ok) {
          tc_fence_after_sync();
          if (stream_needs(entry_at(0), t)) {
            issue_s(0, 0);
            if constexpr (!kPairFullS) issue_s(1, 0);
          }
          commit_both(&bars->kv_empty[0]);
        }
      }
      for (int it = 0; ok && it < n_it; ++it) {
        const bool has_next = (it + 1 < n_it);
        const bool mine = stream_needs(entry_at(it), t);
        const bool mine_next = has_next && stream_needs(entry_at(it + 1), t);
        const int cv = 2 * it + 1, ck = 2 * it + 2;
        const int sv = cv % kPairStages, sk = ck % kPairStages;
        ok = warp_wait(wc, smem_u32(&bars->kv_full[sv]), (cv / kPairStages) & 1, kWaitKvFullV);
        if (!ok) break;
        bool k_ready = false;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          if (mine) {
            H3A_STAMP(2 + t, 2 * it + hf, 0);
            ok = warp_wait(wc, smem_u32(&bars->p_full[t][hf]), p_cnt[hf] & 1, kWaitPFull);
            if (!ok) break;
            ++p_cnt[hf];
            tc_fence_after_sync();
            H3A_STAMP(2 + t, 2 * it + hf, 1);
            issue_pv(hf, sv);
            H3A_STAMP(2 + t, 2 * it + hf, 2);
          }
          if (has_next && !k_ready) {
            ok = warp_wait(wc, smem_u32(&bars->kv_full[sk]), (ck / kPairStages) & 1, kWaitKvFullK);
            if (!ok) break;
            k_ready = true;
            tc_fence_after_sync();
          }
          if (mine_next && (!kPairFullS || hf == 1)) issue_s(kPairFullS ? 0 : hf, sk);  // full: both halves at once
          H3A_STAMP(2 + t, 2 * it + hf, 3);
        }
        if (!ok) break;
        commit_both(&bars->kv_empty[sv]);
        if (has_next) commit_both(&bars->kv_empty[sk]);
      }
      // only the epilogue waits for O: one arrive per CTA once every MMA of the stream has completed
      if (ok) commit_both(&bars->o_full[t]);
      // the commits to the peer's barriers were issued before this one and complete in order: once it has
      // arrived nothing of this issuer is still on its way to the peer CTA
      if (ok) {
        umma_pair_commit_if(leader, smem_u32(&bars->drain[t]));
        warp_wait(wc, smem_u32(&bars->drain[t]), 0, kWaitDrain);
      }
    }
    __syncwarp();
   }
  } else {
    setmaxnreg_inc<kSoftmaxRegs>();
    if constexpr (kResident) {
    // =========================================================== softmax, fixed reference, persistent over items
    const int wg = warp >> 2;
    const int t = wg & 1;
    const int hf = wg >> 1;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t sb = tmem + lane_base + t * kTile + hf * 64;
    const uint32_t o_addr = tmem + lane_base + 256 + t * kTile + hf * 64;
    const int last_tile = args.n_kv_tiles - 1;
    const int tail = args.Lk - last_tile * kTile;
    const uint32_t p_bar = at0(&bars->p_full[t][hf]);
    const uint32_t free_bar = at0(&bars->o_free[t]);
    const float m_ref = args.fixed_m;
    const float c = args.scale_log2;
    // the row sums of the stream's two warpgroups meet here (the Q tiles are being reloaded at that time)
    float* lbuf = reinterpret_cast<float*>(smem + kBarsOff + 512) + t * 128;
    uint32_t j = 0;  // key tiles processed so far, all items: the phase of s_full
    uint32_t g = 0;  // items so far: the phase of o_full / o_free
    bool ok = true;
    uint32_t s[64];
    for (int item = item_begin; item < item_end; ++item) {
      if (item > item_begin && ++cl == n_clusters) {
        cl = 0;
        ++head;
      }
      const int q_row = q_tile(t) * kTile + row;
      const bool row_valid = q_row < args.Lq;
      __nv_bfloat16* orow = out_row_ptr(args, q_row, head) + 64 * hf;
      float l_sum = 0.0f;
      for (int it = 0; ok && it < n_it; ++it) {
        if (row == 0 && t == 0) H3A_STAMP(hf, j, 0);
        ok = warp_wait(wc, smem_u32(&bars->s_full[t][hf]), j & 1, kWaitSFull);
        if (!ok) break;
        if (row == 0 && t == 0) H3A_STAMP(hf, j, 1);
        tc_fence_after_sync();
        tmem_ld32(sb, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld32(sb + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_wait_ld();
        reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        if (it == last_tile && tail < kTile) {
          const int valid = tail - hf * 64;
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i >= valid) s[i] = 0xFF800000u;  // -inf
        }
        if (row == 0 && t == 0) H3A_STAMP(hf, j, 2);
        l_sum += exp_half_tile<false, 1>(s, c, m_ref);  // short launches at full clock: the cycle-optimal share
        if (row == 0 && t == 0) H3A_STAMP(hf, j, 3);
        tmem_st32(sb, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(p_bar);
        if (row == 0 && t == 0) H3A_STAMP(hf, j, 4);
        ++j;
      }
      // ---- epilogue of the item.  Two named barriers that every thread of the stream's two warpgroups always reaches
      //      carry the exchange of the row sums (half 0 leaves its sum, half 1 swaps it for its own); between them ONE
      //      thread reads the abort flag for the stream, so that both warpgroups leave the item loop together.
      bool have = ok;
      if (row == 0 && t == 0) H3A_STAMP(hf, 32 + g, 0);
      if (have) {
        have = warp_wait(wc, smem_u32(&bars->o_full[t]), g & 1, kWaitOFull);
        if (have) tc_fence_after_sync();
      }
      if (row == 0 && t == 0) H3A_STAMP(hf, 32 + g, 1);
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
      if (row == 0 && t == 0) H3A_STAMP(hf, 32 + g, 2);
      if (have) {
        // O leaves TMEM first: the next item's first P V may overwrite it while the rows are converted and stored
        tmem_ld32(o_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld32(o_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_wait_ld();
        reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      }
      if (row == 0 && t == 0) H3A_STAMP(hf, 32 + g, 3);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(free_bar);
      if (row == 0 && t == 0) H3A_STAMP(hf, 32 + g, 4);
      if (have) {
        const float l_tot = l_sum + l_other;
        if (hf == 0 && row_valid) check_row_sum(args, l_tot, false);
        const float inv = 1.0f / l_tot;
        if (row_valid && args.lse && hf == 0)
          args.lse[static_cast<long long>(head) * args.Lq + q_row] = (m_ref + log2f(l_tot)) * 0.6931471805599453f;
#pragma unroll
        for (int i = 0; i < 32; ++i)  // 64 columns of this row as 8 chunks of 16 bytes (slot i <= 2 i: already consumed)
          s[i] = pack_bf16x2(__uint_as_float(s[2 * i]) * inv, __uint_as_float(s[2 * i + 1]) * inv);
        if (row == 0 && t == 0) H3A_STAMP(hf, 32 + g, 5);
        // A thread owns a row, so a plain store instruction of the warp would touch 32 rows = 32 lines with 16 bytes
        // each, and the warps would sit in the store queue: an SM moves only about 18 bytes per cycle towards L2
        // (measured: 3,600 to 4,600 cycles per item for its 64 KB, however the stores are grouped).  So the rows leave
        // through the copy engine instead: 8 rows at a time the warp writes its 128-byte half rows into one of its two
        // 1 KB buffers (16-byte slots swizzled by the row, which is the tensor map's 128-byte swizzle and free of bank
        // conflicts), one lane issues a TMA tile store of 8 rows x 64 columns and goes on; a buffer is rewritten once
        // the copy engine has read it.  Rows beyond Lq are clipped by the tensor map.
        const uint32_t stg = smem_u32(smem + 2 * kQTileBytes + kPairStages * kPairStageBytes) + warp * (kPairStoreStages * kPairStoreStageBytes);
        const int tile_row0 = q_tile(t) * kTile + quarter * 32;
        if (args.o_n_ranks <= 1) {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const uint32_t buf = stg + (p & 1) * kPairStoreStageBytes;
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // the store that last used this buffer
            __syncwarp();
            if ((lane >> 3) == p) {
              const uint32_t r8 = lane & 7;
#pragma unroll
              for (uint32_t ch = 0; ch < 8; ++ch)
                st_shared_v4(buf + r8 * 128 + ((ch ^ r8) << 4), s[4 * ch], s[4 * ch + 1], s[4 * ch + 2], s[4 * ch + 3]);
              fence_proxy_async_smem();  // these rows are read by the copy engine
            }
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&tm_o, buf, 64 * hf, tile_row0 + p * 8, head);
              tma_store_commit();
            }
          }
        } else {
          // rows that go to other GPUs' memory (one base pointer per rank): plain stores, regrouped through the buffer
          // so that an instruction writes 4 whole half rows
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            if ((lane >> 3) == p) {
              const uint32_t r8 = lane & 7;
#pragma unroll
              for (uint32_t ch = 0; ch < 8; ++ch)
                st_shared_v4(stg + r8 * 128 + ((ch ^ r8) << 4), s[4 * ch], s[4 * ch + 1], s[4 * ch + 2], s[4 * ch + 3]);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const uint32_t r8 = (lane >> 3) + 4 * i, ch = lane & 7;
              uint4 w;
              ld_shared_v4(stg + r8 * 128 + ((ch ^ r8) << 4), w);
              const int rg = tile_row0 + p * 8 + static_cast<int>(r8);
              if (rg < args.Lq) *reinterpret_cast<uint4*>(out_row_ptr(args, rg, head) + 64 * hf + ch * 8) = w;
            }
            __syncwarp();
          }
        }
      }
      if (row == 0 && t == 0) H3A_STAMP(hf, 32 + g, 7);
      if (stop) break;
      ++g;
    }
    if (lane == 0) tma_store_wait_all();  // this lane's tile stores are complete before the CTA's shared memory goes away
    } else
    if constexpr (kFixed) {
    // =========================================================== softmax, fixed reference: one warpgroup per (stream, half)
    const int wg = warp >> 2;
    const int t = wg & 1;
    const int hf = wg >> 1;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t sb = tmem + lane_base + t * kTile + hf * 64;
    const uint32_t o_addr = tmem + lane_base + 256 + t * kTile + hf * 64;
    const int q_row = q_tile(t) * kTile + row;
    const int own_bit = 2 * t + static_cast<int>(rank);  // this CTA's query tile among the pair's four
    const int last_tile = args.n_kv_tiles - 1;
    const int tail = args.Lk - last_tile * kTile;
    const uint32_t p_bar = at0(&bars->p_full[t][hf]);
    float qs = 1.0f;
    if constexpr (kFp8) {
      const int qb = min(q_tile(t), args.nqb - 1);
      qs = args.q_scale[head * args.nqb + qb];
    }
    float m_ref = args.fixed_m;
    float l_sum = 0.0f;
    uint32_t j = 0;
    bool ok = true;
    bool met = false;   // kRowRef: this warp has been to the exchange of the first-tile maxima
    bool over = false;  // kRowRef: a half tile of this row summed past what its reference can represent
    float* rowref = reinterpret_cast<float*>(smem + kBarsOff + 512);
    uint32_t s[64];
    for (int it = 0; ok && it < n_it; ++it) {
      const int e = entry_at(it);
      if (!stream_needs(e, t)) continue;
      const int tile = e >> 4;
      float c = args.scale_log2;
      if constexpr (kFp8) c *= qs * args.k_scale[head * args.nkb + tile];
      if (row == 0 && t == 0) H3A_STAMP(hf, j, 0);
      ok = warp_wait(wc, smem_u32(&bars->s_full[t][kPairFullS ? 0 : hf]), j & 1, kWaitSFull);
      if (!ok) break;
      tc_fence_after_sync();
      if (kSparse && !((e >> own_bit) & 1)) {
        // the key tile is listed only for the peer's query tile: this CTA's rows contribute nothing (P = 0); the
        // S of the pair's MMA is complete, so its buffer may be overwritten
#pragma unroll
        for (int i = 0; i < 32; ++i) s[i] = 0u;
        tmem_st32(sb, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(p_bar);
        ++j;
        continue;
      }
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
      if constexpr (kRowRef) {
        if (j == 0) {
          // the row's reference: the maximum of its logits over the first key tile, both halves
          float mx0 = fmax3(__uint_as_float(s[0]), __uint_as_float(s[1]), __uint_as_float(s[2]));
          float mx1 = fmax3(__uint_as_float(s[3]), __uint_as_float(s[4]), __uint_as_float(s[5]));
#pragma unroll
          for (int i = 6; i < 60; i += 6) {
            mx0 = fmax3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
            mx1 = fmax3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
            mx0 = fmax3(mx0, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
          }
          mx0 = fmax3(mx0, __uint_as_float(s[60]), __uint_as_float(s[61]));
          mx1 = fmax3(mx1, __uint_as_float(s[62]), __uint_as_float(s[63]));
          const float hm = fmaxf(mx0, mx1) * c;
          rowref[(t * 2 + hf) * 128 + row] = hm;
          asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "r"(256) : "memory");  // the stream's two warpgroups
          met = true;
          m_ref = fmaxf(hm, rowref[(t * 2 + (hf ^ 1)) * 128 + row]);
        }
      }
      const float l_half = exp_half_tile<kFp8>(s, c, m_ref);
      l_sum += l_half;
      if constexpr (kRowRef) {
        over |= !(l_half < 1.0e18f);  // 2^60: a logit far above the row's reference (or inf / NaN): redo with the running maximum
      }
      if (row == 0 && t == 0) H3A_STAMP(hf, j, 4);
      tmem_st32(sb, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(p_bar);  // rank 0's barrier: its own CTA's or the peer's
      if (row == 0 && t == 0) H3A_STAMP(hf, j, 5);
      ++j;
    }
    if constexpr (kRowRef) {
      if (!met) asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "r"(256) : "memory");  // a wait gave up before the exchange: the partner must not block there
    }
    // ---- epilogue: as in the single-CTA kernel (own last P V, named barrier, row sums through the Q tile)
    bool have = ok && j > 0;
    if (have) {
      have = warp_wait(wc, smem_u32(&bars->o_full[t]), 0, kWaitOFull);  // its only phase: every MMA of the stream is done
      if (have) tc_fence_after_sync();
    }
    asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "r"(256) : "memory");
    float* lbuf = reinterpret_cast<float*>(smem + t * kQTileBytes);
    lbuf[hf * 128 + row] = l_sum;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "r"(256) : "memory");
    if (have) tc_fence_after_sync();
    const bool row_valid = q_row < args.Lq;
    __nv_bfloat16* orow = out_row_ptr(args, q_row, head) + 64 * hf;
    const float l_tot = l_sum + lbuf[(hf ^ 1) * 128 + row];
    // block-sparse: a row whose query tile lists nothing legitimately sums to zero; a share of a split row may too
    if constexpr (kRowRef) {
      over |= have && !(l_tot < 1.0e30f);
      if (__any_sync(0xFFFFFFFFu, over) && lane == 0) bars->redo = 1u;
    } else {
      if (have && hf == 0 && row_valid) check_row_sum(args, l_tot, kSparse || part_slot >= 0);
    }
    if (!kSparse && part_slot >= 0) {
      // a share of the key tiles: leave the un-normalised sums for the combining kernel
      if (have) {
        const long long rix = (static_cast<long long>(part_slot) * 4 + own_bit) * 128 + row;
        float* prow = args.part + rix * 128 + 64 * hf;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          uint32_t o[32];
          tmem_ld32(o_addr + 32 * i, o);
          tmem_wait_ld();
#pragma unroll
          for (int x = 0; x < 32; x += 4)
            *reinterpret_cast<uint4*>(prow + 32 * i + x) = make_uint4(o[x], o[x + 1], o[x + 2], o[x + 3]);
        }
        if (hf == 0) args.part[part_slots(args, n_clusters) * 4 * 128 * 128 + rix] = l_tot;
      }
    } else if (have) {
      // `have` is uniform over the warp, which the TMEM loads below require; whether a ROW has anything to divide by
      // is not (a row of a listed key tile can sum to zero, and after an overflow to NaN), so that is a select
      const bool live = l_tot > 0.0f;
      const float inv = live ? 1.0f / l_tot : 0.0f;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        uint32_t o[32];
        tmem_ld32(o_addr + 32 * i, o);
        tmem_wait_ld();
        if (row_valid) {
#pragma unroll
          for (int x = 0; x < 32; x += 8) {
            float f[8];
#pragma unroll
            for (int y = 0; y < 8; ++y) f[y] = live ? __uint_as_float(o[x + y]) * inv : 0.0f;
            uint4 w;
            w.x = pack_bf16x2(f[0], f[1]);
            w.y = pack_bf16x2(f[2], f[3]);
            w.z = pack_bf16x2(f[4], f[5]);
            w.w = pack_bf16x2(f[6], f[7]);
            *reinterpret_cast<uint4*>(orow + 32 * i + x) = w;
          }
        }
      }
      if (row_valid && args.lse && hf == 0)
        args.lse[static_cast<long long>(head) * args.Lq + q_row] = live ? (m_ref + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
    } else if (ok && row_valid && (j == 0 || have)) {
      // no key tile listed for this query tile (the stream may still have run for the peer's tile): zero rows
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int x = 0; x < 64; x += 8) *reinterpret_cast<uint4*>(orow + x) = z;
      if (args.lse && hf == 0) args.lse[static_cast<long long>(head) * args.Lq + q_row] = -INFINITY;
    }
    } else {
    // =========================================================== online softmax: running row maximum, lazy rescale of O
    // One warpgroup per stream walks both halves of every key tile (they share the row's maximum), as in the
    // single-CTA kernel.  What the pair changes: P is published with one arrive per warp on rank 0's barrier, and O
    // may be rescaled only when the pair's previous P V of the stream has completed in BOTH CTAs - o_done is
    // committed to each CTA's copy, and the next P V is not issued before all eight warps of the two CTAs have
    // published, which each does after its own rescale stores have completed.
    const int t = warp >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + t * kTile;
    const uint32_t o_addr = tmem + lane_base + 256 + t * kTile;
    const int q_row = q_tile(t) * kTile + row;
    const int last_tile = args.n_kv_tiles - 1;
    const int tail = args.Lk - last_tile * kTile;
    const uint32_t p_bar[2] = {at0(&bars->p_full[t][0]), at0(&bars->p_full[t][1])};
    float qs = 1.0f;
    if constexpr (kFp8) {
      const int qb = min(q_tile(t), args.nqb - 1);
      qs = args.q_scale[head * args.nqb + qb];
    }
    float m_ref = 0.0f, l_sum = 0.0f;
    uint32_t j = 0;
    bool ok = true;
    uint32_t ra[64], rb[64];  // two register images of an S half: one being processed, one being prefetched

    auto load_s = [&](uint32_t (&r)[64], int hf) {
      tc_fence_after_sync();
      tmem_ld32(s_addr + hf * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
      tmem_ld32(s_addr + hf * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
    };
    auto fetch_s = [&](uint32_t (&r)[64], int hf, uint32_t jt) -> bool {
      const bool got = warp_wait(wc, smem_u32(&bars->s_full[t][hf]), jt & 1, kWaitSFull);
      if (got) load_s(r, hf);
      return got;
    };
    auto try_fetch_s = [&](uint32_t (&r)[64], int hf, uint32_t jt) -> bool {
      const bool ready = __all_sync(0xFFFFFFFFu, mbar_test_wait(smem_u32(&bars->s_full[t][hf]), jt & 1));
      if (ready) load_s(r, hf);
      return ready;
    };
    auto softmax_half = [&](uint32_t (&s)[64], int hf, int tile, float c) -> bool {
      if (tile == last_tile && tail < kTile) {
        const int valid = tail - hf * 64;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i >= valid) s[i] = 0xFF800000u;  // -inf
      }
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
          // the stream's previous P V (the only one that can still be running: MMAs complete in issue order)
          if (!warp_wait(wc, smem_u32(&bars->o_done[t][hf ^ 1]), (hf ? j : j - 1) & 1, kWaitOFull)) return false;
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
      l_sum += exp_half_tile<kFp8>(s, c, m_ref);
      return true;
    };
    auto publish_p = [&](uint32_t (&s)[64], int hf) {
      tmem_st32(s_addr + hf * 64, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_wait_st();  // also covers the stores of a rescale of O just before
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(p_bar[hf]);
    };

    if (n_it > 0) ok = fetch_s(ra, 0, 0);
    for (int it = 0; ok && it < n_it; ++it) {
      const int tile = entry_at(it) >> 4;
      const bool has_next = it + 1 < n_it;
      float c = args.scale_log2;
      if constexpr (kFp8) c *= qs * args.k_scale[head * args.nkb + tile];
      // half 0 from image A; half 1 is loaded into image B as early as its S is complete
      tmem_wait_ld();
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&ra[0]));
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&ra[32]));
      ok = softmax_half(ra, 0, tile, c);
      if (!ok) break;
      {
        const bool early = try_fetch_s(rb, 1, j);
        publish_p(ra, 0);
        if (!early) ok = fetch_s(rb, 1, j);
        if (!ok) break;
      }
      tmem_wait_ld();
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&rb[0]));
      reg_fence32(*reinterpret_cast<uint32_t(*)[32]>(&rb[32]));
      ok = softmax_half(rb, 1, tile, c);
      if (!ok) break;
      {
        const bool early = has_next && try_fetch_s(ra, 0, j + 1);
        publish_p(rb, 1);
        if (!early && has_next) ok = fetch_s(ra, 0, j + 1);
        if (!ok) break;
      }
      ++j;
    }
    // ---- epilogue: O / l -> bf16 -> global (each thread owns its whole row)
    const bool row_valid = q_row < args.Lq;
    __nv_bfloat16* orow = out_row_ptr(args, q_row, head);
    if (ok && j > 0) {
      ok = warp_wait(wc, smem_u32(&bars->o_full[t]), 0, kWaitOFull);
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
    }
    }
  }
  }  // run

  // ---- tear-down
  if (args.o_n_ranks > 1) __threadfence_system();  // rows stored into other GPUs' memory
  tc_fence_before_sync();
  __syncthreads();
  if (bars->abort_flag) {
    // a wait gave up: give copies and MMAs in flight a bounded time to land before anything goes away
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if constexpr (kRowRef) {
    if (threadIdx.x == 0 && rank == 1 && bars->redo) st_shared_cluster_u32(mapa_shared(smem_u32(const_cast<const uint32_t*>(&bars->redo)), 0), 1u);
  }
  cluster_sync_all();  // neither CTA frees TMEM or leaves while the other may still use it or signal its barriers
  if constexpr (kRowRef) {
    if (threadIdx.x == 0 && rank == 0 && bars->redo && args.redo_count != nullptr) args.redo_list[atomicAdd(args.redo_count, 1)] = cid;
  }
  if (run && warp == kIssuerWarp) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem, 512);
  }
}

}  // namespace h3a
