// Q / K / V projection with the attention preparation fused into its epilogue, for sm_100a:
//   Y[l, n] = sum_k X[l, k] W[n, k]  (+ sum_r T[l, r] Bs[n, r])  (+ bias[n])
// X = hidden states [L, K] bf16, W = nn.Linear weight [N, K] bf16, N = heads x 128.  The optional second product is
// the LoRA update: T = X A^T [L, R] (computed by the caller, R = rank) and Bs = (alpha / rank) B [N, R]; it is just
// R more columns of the contraction.  Epilogue per head (128 output columns of one token, fp32):
//   kProjStore : bf16 store, head-major [head][token][128]                                    (V)
//   kProjPrep  : RMSNorm over the 128 columns (x weight), rotation by the (cos, sin) table, store   (Q, K)
//   kProjPrepFp8: the same, then e4m3 with one absmax / 448 scale per (head, 128-token block)       (Q, K of FP8-QK)
// so the projection output never makes a round trip through HBM before the preparation.
//
// One CTA PAIR (cluster of two, tcgen05 cta_group::2) computes tiles of 256 tokens x 256 output columns: each CTA
// stages its own 128 token rows of X and 128 rows of W (= one head) per 64-wide step of the contraction, the MMA is
// M = 256, N = 256, and each CTA ends up with its 128 tokens x both heads in TMEM (256 columns).  The kernel is
// persistent: one pair per two SMs walks the tiles pair, pair + pairs, ...; the accumulator is double-buffered in
// TMEM (2 x 256 columns) so the epilogue of one tile runs under the contraction of the next.
//   warp 8      producer : TMA loads into a ring of 6 stages x 32 KB; both CTAs' bytes count on rank 0's barrier
//   warp 9      issuer   : rank 0 only; 4 MMAs (K = 16 each) per stage, commits to both CTAs' barriers
//   warps 0-7   epilogue : warp w reads TMEM lane quarter w % 4 (one token per thread), head w / 4 of the tile;
//                          it frees the accumulator buffer (one arrive per warp on rank 0) before it stores
// The pair protocol (cluster barriers around set-up and tear-down, bounded waits, abort flag raised in the peer
// too) is the one of the attention kernel on CTA pairs.
#pragma once
#include <cuda_fp8.h>

#include "attn_fwd.cuh"

namespace h3a {

#ifndef H3A_PROJ_STAGES
#define H3A_PROJ_STAGES 6
#endif
constexpr int kProjStages = H3A_PROJ_STAGES;
constexpr int kProjStageBytes = 32768;  // 16 KB of X rows + 16 KB of W rows
constexpr int kProjThreads = 320;
constexpr int kProjStoreStageBytes = 2048;  // per epilogue warp: 32 rows x 64 bytes, to turn per-row stores into coalesced ones
constexpr int kProjSmemBytes = kProjStages * kProjStageBytes + 1024 + 256 + 8 * kProjStoreStageBytes;

enum : int { kProjStore = 0, kProjPrep = 1, kProjPrepFp8 = 2 };
enum : int { kWaitProjEmpty = 16, kWaitProjFull = 17, kWaitProjAcc = 18, kWaitProjDrain = 19, kWaitProjAccEmpty = 20, kWaitProjMax = 21 };

struct ProjBars {
  uint64_t full[kProjStages];   // rank 0: bytes of both CTAs
  uint64_t empty[kProjStages];  // both CTAs: one commit per use
  uint64_t acc_full[2];         // both CTAs: accumulator buffer b is complete
  uint64_t acc_empty[2];        // rank 0: all 16 epilogue warps of the pair have read buffer b
  uint64_t drain;               // rank 0
  uint64_t qmax[2];             // e4m3 epilogue: the 4 warps of warpgroup h have posted their maxima (one phase per tile)
  float wmax[2][2][4];          // [tile parity][warpgroup][warp]
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  uint32_t early_exit;
};
static_assert(sizeof(ProjBars) <= 256, "barrier block too large");

struct ProjArgs {
  AttnArgs wait;               // only .status and .wait_ns are used (bounded waits)
  int L, N, n_tiles_n, n_tiles; // tokens, output columns, 256-column tiles per token tile, all tiles
  int band_n, n_tiles_m;       // column tiles per band of the tile order (see tile_mn), 256-token tiles
  int kb_main, kb_lora;        // 64-wide steps of the two products
  int epilogue;
  const float* bias;           // [N] or null
  const float* rope;           // [L, 64, 2] or null
  const float* norm_weight;    // [128] or null
  float eps;
  int rope_half;
  void* out;                   // bf16 (or e4m3 bytes) [N / 128][L][128] by strides
  long long out_stride_l, out_stride_h;
  float* out_scale;            // kProjPrepFp8: [N / 128][nblk] absmax / 448 per (head, 128-token block)
  int nblk;
  // Sequence parallelism (n_ranks > 0, bf16 epilogues): the row of output head h goes to the rank that computes
  // head head0 + h, as in PrepArgs (qk_prep.cuh); col_rot rotates the column-tile order so that the ranks do not
  // all store to the same owner at the same time.
  void* rank_out[8];
  int n_ranks, heads_per_rank, round_robin, head0, row_offset, L_total, col_rot;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kProjThreads, 1)
qkv_proj_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_t, const __grid_constant__ CUtensorMap tm_b, const ProjArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t ring = base;
  ProjBars* bars = reinterpret_cast<ProjBars*>(smem + kProjStages * kProjStageBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  // Tile order: the output columns are cut into bands of band_n column tiles; a band is walked over ALL token tiles
  // (column tiles fastest inside the band) before the next band starts.  The pairs running together then share a few
  // token tiles of X and one band of W, and that band (band_n x 256 rows of W) is small enough to STAY in L2 from one
  // wave of tiles to the next; with a single band of all columns W (52 MB at N = K = 5,120) was evicted by the X and
  // output streams and re-read from DRAM by every wave.  X is read once per band instead of once.
  auto tile_mn = [&](int tile, int& mt, int& nt) {
    const int per_band = args.band_n * args.n_tiles_m;
    const int n_bands = (args.n_tiles_n + args.band_n - 1) / args.band_n;
    const int b = min(tile / per_band, n_bands - 1);
    const int r = tile - b * per_band;
    const int bw = (b == n_bands - 1) ? args.n_tiles_n - b * args.band_n : args.band_n;
    mt = r / bw;
    nt = b * args.band_n + r % bw;
    if (args.col_rot) nt = (nt + args.col_rot) % args.n_tiles_n;
  };
  auto tile_m0 = [&](int tile) { int mt, nt; tile_mn(tile, mt, nt); return mt * 256 + static_cast<int>(rank) * 128; };  // this CTA's first token
  auto tile_n0 = [&](int tile) { int mt, nt; tile_mn(tile, mt, nt); return nt * 256; };                                 // the pair's first column
  const int n_kb = args.kb_main + args.kb_lora;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kProjStages; ++i) {
      mbar_init(smem_u32(&bars->full[i]), 1);
      mbar_init(smem_u32(&bars->empty[i]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars->acc_full[b]), 1);
      mbar_init(smem_u32(&bars->acc_empty[b]), 16);
    }
    mbar_init(smem_u32(&bars->drain), 1);
    mbar_init(smem_u32(&bars->qmax[0]), 4);
    mbar_init(smem_u32(&bars->qmax[1]), 4);
    bars->abort_flag = 0;
    bars->early_exit = (args.wait.status != nullptr && *reinterpret_cast<volatile int*>(args.wait.status) != 0) ? 1u : 0u;
    fence_mbar_init();
  }
  if (warp == 8 && lane == 0) {
    prefetch_tmap(&tm_x);
    prefetch_tmap(&tm_w);
    if (args.kb_lora > 0) {
      prefetch_tmap(&tm_t);
      prefetch_tmap(&tm_b);
    }
  }
  cluster_sync_all();
  const bool run = ld_shared_cluster_u32(mapa_shared(smem_u32(&bars->early_exit), 0)) == 0u;
  const uint32_t bars0 = mapa_shared(smem_u32(bars), 0);
  const uint32_t bars_peer = mapa_shared(smem_u32(bars), rank ^ 1u);
  auto at0 = [&](const void* local) { return bars0 + (smem_u32(local) - smem_u32(bars)); };
  auto at_peer = [&](const void* local) { return bars_peer + (smem_u32(local) - smem_u32(bars)); };
  WaitCtx wc{smem_u32(const_cast<const uint32_t*>(&bars->abort_flag)), at_peer(const_cast<const uint32_t*>(&bars->abort_flag)), &args.wait};
  uint32_t tmem = 0;

  if (run) {
    if (warp == 9) {
      tmem_alloc_pair(smem_u32(&bars->tmem_base), 512);
      tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    tmem = bars->tmem_base;

    if (warp == 8) {
      // ======================================================= producer (both CTAs)
      const uint32_t leader = elect_one();
      bool ok = true;
      int kbg = 0;  // stage counter across tiles
      for (int tile = pair; ok && tile < args.n_tiles; tile += n_pairs) {
        const int m0 = tile_m0(tile), n0 = tile_n0(tile);
        for (int kb = 0; kb < n_kb; ++kb, ++kbg) {
          const int s = kbg % kProjStages;
          const uint32_t ph = (kbg / kProjStages) & 1;
          ok = warp_wait(wc, smem_u32(&bars->empty[s]), ph ^ 1u, kWaitProjEmpty);
          if (!ok) break;
          if (rank == 0) mbar_arrive_expect_tx_if(leader, smem_u32(&bars->full[s]), 2 * kProjStageBytes);
          const uint32_t fb = at0(&bars->full[s]);
          const uint32_t dst = ring + s * kProjStageBytes;
          const bool main = kb < args.kb_main;
          const int k0 = (main ? kb : kb - args.kb_main) * 64;
          // X (or T) rows of this CTA's 128 tokens; W (or Bs) rows of this CTA's head
          tma_load_2d_pair_if(leader, dst, main ? &tm_x : &tm_t, fb, k0, m0);
          tma_load_2d_pair_if(leader, dst + 16384, main ? &tm_w : &tm_b, fb, k0, n0 + 128 * static_cast<int>(rank));
        }
      }
      __syncwarp();
    } else if (warp == 9) {
      // ======================================================= MMA issuer (rank 0)
      if (rank == 0) {
        const uint32_t leader = elect_one();
        constexpr uint32_t idesc = umma_idesc(UMMA_FMT_BF16, UMMA_FMT_BF16, 0, 0, 256, 256);
        const uint64_t a_desc0 = umma_desc_sw128(ring, 16, 1024);
        const uint64_t b_desc0 = umma_desc_sw128(ring + 16384, 16, 1024);
        auto commit_both = [&](const void* local) {
          umma_pair_commit_if(leader, smem_u32(local));
          umma_pair_commit_if(leader, at_peer(local));
        };
        bool ok = true;
        int kbg = 0, it = 0;
        for (int tile = pair; ok && tile < args.n_tiles; tile += n_pairs, ++it) {
          const int buf = it & 1;
          // the epilogue warps of both CTAs must have read this buffer's previous tile (two tiles back)
          ok = warp_wait(wc, smem_u32(&bars->acc_empty[buf]), ((it >> 1) & 1) ^ 1u, kWaitProjAccEmpty);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem + 256 * buf;
          for (int kb = 0; kb < n_kb; ++kb, ++kbg) {
            const int s = kbg % kProjStages;
            ok = warp_wait(wc, smem_u32(&bars->full[s]), (kbg / kProjStages) & 1, kWaitProjFull);
            if (!ok) break;
            tc_fence_after_sync();
            const uint64_t so = static_cast<uint64_t>((s * kProjStageBytes) >> 4);
#pragma unroll
            for (int k = 0; k < 4; ++k)  // 16 bf16 = 32 bytes per step inside the 128-byte swizzle span
              umma_pair_bf16_ss_if(leader, d_tmem, a_desc0 + so + (k * 32 >> 4), b_desc0 + so + (k * 32 >> 4), idesc, (kb > 0 || k > 0) ? 1u : 0u);
            commit_both(&bars->empty[s]);
          }
          if (ok) commit_both(&bars->acc_full[buf]);
        }
        if (ok) {
          umma_pair_commit_if(leader, smem_u32(&bars->drain));
          warp_wait(wc, smem_u32(&bars->drain), 0, kWaitProjDrain);
        }
      }
      __syncwarp();
    } else {
      // ======================================================= epilogue: one token per thread, one head per warpgroup
      const int quarter = warp & 3, hsel = warp >> 2;
      const int row = quarter * 32 + lane;
      const uint32_t empty_bar0 = at0(&bars->acc_empty[0]);
      uint8_t* stg = smem + kProjStages * kProjStageBytes + 256 + warp * kProjStoreStageBytes;  // this warp's store staging
      const bool prep = args.epilogue != kProjStore;
      bool ok = true;
      int it = 0;
      for (int tile = pair; ok && tile < args.n_tiles; tile += n_pairs, ++it) {
        const int buf = it & 1;
        const int l = tile_m0(tile) + row;
        const int n_head0 = tile_n0(tile) + 128 * hsel;  // first output column of this thread's head
        const uint32_t t_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + 256 * buf + 128 * hsel;
        ok = warp_wait(wc, smem_u32(&bars->acc_full[buf]), (it >> 1) & 1, kWaitProjAcc);
        if (!ok) break;
        tc_fence_after_sync();
        const bool live = l < args.L && n_head0 < args.N;
        const float4* b4 = reinterpret_cast<const float4*>(args.bias + (args.bias ? n_head0 : 0));
        const float4* w4 = reinterpret_cast<const float4*>(args.norm_weight);
        const float4* t4 = reinterpret_cast<const float4*>(args.rope + (args.rope ? static_cast<long long>(min(l, args.L - 1)) * 128 : 0));
        // this warp has read all it needs of the accumulator buffer: hand it back (before the stores)
        auto release = [&]() {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(empty_bar0 + 8 * buf);
        };
        // pass 1 (with normalisation): the row's sum of squares; later passes read the accumulator again and keep
        // only 64 of the 128 columns in registers at a time
        float rinv = 1.0f;
        if (prep) {
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t r[32];
            tmem_ld32(t_addr + 32 * i, r);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
              if (args.bias && live) b = b4[(32 * i + c) >> 2];
              const float v0 = __uint_as_float(r[c]) + b.x, v1 = __uint_as_float(r[c + 1]) + b.y;
              const float v2 = __uint_as_float(r[c + 2]) + b.z, v3 = __uint_as_float(r[c + 3]) + b.w;
              ss += v0 * v0 + v1 * v1 + v2 * v2 + v3 * v3;
            }
          }
          rinv = rsqrtf(ss * (1.0f / 128.0f) + args.eps);
        }
        // columns [32 g, +32) -> lo and [64 + 32 g, +32) -> hi, finished (bias, norm, weight, rotation): both rotary
        // pair conventions stay inside one call
        auto prepare = [&](int g, float (&lo)[32], float (&hi)[32]) {
          uint32_t ra[32], rb[32];
          tmem_ld32(t_addr + 32 * g, ra);
          tmem_ld32(t_addr + 64 + 32 * g, rb);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            float4 ba = make_float4(0.f, 0.f, 0.f, 0.f), bb = ba;
            if (args.bias && live) {
              ba = b4[(32 * g + c) >> 2];
              bb = b4[(64 + 32 * g + c) >> 2];
            }
            float4 wa = make_float4(1.f, 1.f, 1.f, 1.f), wb = wa;
            if (prep && args.norm_weight) {
              wa = w4[(32 * g + c) >> 2];
              wb = w4[(64 + 32 * g + c) >> 2];
            }
            lo[c] = (__uint_as_float(ra[c]) + ba.x) * rinv * wa.x;
            lo[c + 1] = (__uint_as_float(ra[c + 1]) + ba.y) * rinv * wa.y;
            lo[c + 2] = (__uint_as_float(ra[c + 2]) + ba.z) * rinv * wa.z;
            lo[c + 3] = (__uint_as_float(ra[c + 3]) + ba.w) * rinv * wa.w;
            hi[c] = (__uint_as_float(rb[c]) + bb.x) * rinv * wb.x;
            hi[c + 1] = (__uint_as_float(rb[c + 1]) + bb.y) * rinv * wb.y;
            hi[c + 2] = (__uint_as_float(rb[c + 2]) + bb.z) * rinv * wb.z;
            hi[c + 3] = (__uint_as_float(rb[c + 3]) + bb.w) * rinv * wb.w;
          }
          if (prep && args.rope && live) {
            if (args.rope_half) {
              // pair e = (e, e + 64), e = 32 g + c: table entries 32 g .. 32 g + 31
#pragma unroll
              for (int c = 0; c < 32; c += 2) {
                const float4 cs = t4[(32 * g + c) >> 1];
                const float p0 = lo[c], q0 = hi[c], p1 = lo[c + 1], q1 = hi[c + 1];
                lo[c] = p0 * cs.x - q0 * cs.y;      hi[c] = p0 * cs.y + q0 * cs.x;
                lo[c + 1] = p1 * cs.z - q1 * cs.w;  hi[c + 1] = p1 * cs.w + q1 * cs.z;
              }
            } else {
              // pair j = (2 j, 2 j + 1): lo holds pairs 16 g .. 16 g + 15, hi holds pairs 32 + 16 g ..
#pragma unroll
              for (int c = 0; c < 32; c += 4) {
                const float4 cl = t4[(32 * g + c) >> 2], ch = t4[(64 + 32 * g + c) >> 2];
                float p, q;
                p = lo[c]; q = lo[c + 1]; lo[c] = p * cl.x - q * cl.y; lo[c + 1] = p * cl.y + q * cl.x;
                p = lo[c + 2]; q = lo[c + 3]; lo[c + 2] = p * cl.z - q * cl.w; lo[c + 3] = p * cl.w + q * cl.z;
                p = hi[c]; q = hi[c + 1]; hi[c] = p * ch.x - q * ch.y; hi[c + 1] = p * ch.y + q * ch.x;
                p = hi[c + 2]; q = hi[c + 3]; hi[c + 2] = p * ch.z - q * ch.w; hi[c + 3] = p * ch.w + q * ch.z;
              }
            }
          }
        };
        const long long out_off = static_cast<long long>(n_head0 / 128) * args.out_stride_h + static_cast<long long>(l) * args.out_stride_l;
        if (args.epilogue != kProjPrepFp8) {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(args.out) + out_off;
          if (args.n_ranks > 0) {  // the head's owning rank: its [heads_per_rank, L_total, 128] buffer, token row_offset + l
            const int h = args.head0 + n_head0 / 128;
            const int owner = args.round_robin ? h % args.n_ranks : min(h / args.heads_per_rank, args.n_ranks - 1);
            const int slot = args.round_robin ? h / args.n_ranks : h - owner * args.heads_per_rank;
            dst = static_cast<__nv_bfloat16*>(args.rank_out[owner]) + (static_cast<long long>(slot) * args.L_total + args.row_offset + l) * 128;
          }
          // A thread holds 64-byte pieces of ITS row; stored as they are, a warp instruction would write 32 separate
          // 16-byte chunks 256 bytes apart.  Each piece goes through 2 KB of shared memory (16-byte chunks XOR-swizzled
          // by the row so that neither side has bank conflicts) and leaves as 8 rows x 64 contiguous bytes per
          // instruction: fewer, larger transactions - what NVLink needs when the owner is another GPU, and kinder to
          // the local L2 as well.
          const int l_warp = tile_m0(tile) + quarter * 32;            // first token of this warp's 32 rows
          const long long row_step = args.n_ranks > 0 ? 128 : args.out_stride_l;
          __nv_bfloat16* dst_warp = dst - static_cast<long long>(lane) * row_step;  // row 0 of the warp (same head for all lanes)
          auto store_piece = [&](const float (&x)[32], int col0) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 w;
              w.x = pack_bf16x2(x[8 * c], x[8 * c + 1]); w.y = pack_bf16x2(x[8 * c + 2], x[8 * c + 3]);
              w.z = pack_bf16x2(x[8 * c + 4], x[8 * c + 5]); w.w = pack_bf16x2(x[8 * c + 6], x[8 * c + 7]);
              *reinterpret_cast<uint4*>(stg + lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4)) = w;
            }
            __syncwarp();
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int rr = (lane >> 2) + 8 * k, b = lane & 3;
              const uint4 w = *reinterpret_cast<const uint4*>(stg + rr * 64 + ((b ^ ((rr >> 1) & 3)) << 4));
              if (l_warp + rr < args.L && n_head0 < args.N)
                *reinterpret_cast<uint4*>(dst_warp + static_cast<long long>(rr) * row_step + col0 + 8 * b) = w;
            }
            __syncwarp();
          };
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            float lo[32], hi[32];
            prepare(g, lo, hi);
            if (g == 1) release();
            store_piece(lo, 32 * g);
            store_piece(hi, 64 + 32 * g);
          }
        } else {
          // e4m3 with one absmax scale per (head, 128-token block) = this warpgroup's 128 rows x 128 columns: a pass
          // for the block maximum (4 warps meet through shared memory and a bounded mbarrier), a pass to quantise
          float amax = 0.f;
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            float lo[32], hi[32];
            prepare(g, lo, hi);
            if (live) {
#pragma unroll
              for (int c = 0; c < 32; ++c) amax = fmaxf(amax, fmaxf(fabsf(lo[c]), fabsf(hi[c])));
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
          if (lane == 0) {
            bars->wmax[it & 1][hsel][quarter] = amax;
            mbar_arrive(smem_u32(&bars->qmax[hsel]));
          }
          ok = warp_wait(wc, smem_u32(&bars->qmax[hsel]), it & 1, kWaitProjMax);
          if (!ok) break;
          const float bm = fmaxf(fmaxf(bars->wmax[it & 1][hsel][0], bars->wmax[it & 1][hsel][1]),
                                 fmaxf(bars->wmax[it & 1][hsel][2], bars->wmax[it & 1][hsel][3]));
          const float scale = bm > 0.f ? bm / 448.0f : 1.0f;
          const float inv = 1.0f / scale;
          if (row == 0 && n_head0 < args.N && tile_m0(tile) < args.L)
            args.out_scale[static_cast<long long>(n_head0 / 128) * args.nblk + tile_m0(tile) / 128] = scale;
          uint8_t* dst = static_cast<uint8_t*>(args.out) + out_off;
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            float lo[32], hi[32];
            prepare(g, lo, hi);
            if (g == 1) release();
            if (live) {
#pragma unroll
              for (int c = 0; c < 32; c += 16) {
                uint32_t wl[4], wh[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                  const int e = c + 4 * x;
                  const auto q2 = [&](float a, float b) {
                    return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(
                        make_float2(fminf(fmaxf(a * inv, -448.f), 448.f), fminf(fmaxf(b * inv, -448.f), 448.f)), __NV_SATFINITE, __NV_E4M3));
                  };
                  wl[x] = q2(lo[e], lo[e + 1]) | (q2(lo[e + 2], lo[e + 3]) << 16);
                  wh[x] = q2(hi[e], hi[e + 1]) | (q2(hi[e + 2], hi[e + 3]) << 16);
                }
                *reinterpret_cast<uint4*>(dst + 32 * g + c) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                *reinterpret_cast<uint4*>(dst + 64 + 32 * g + c) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
              }
            }
          }
        }
      }  // tiles
    }
  }

  // ---- tear-down
  if (args.n_ranks > 1) __threadfence_system();  // rows stored into other GPUs' memory
  tc_fence_before_sync();
  __syncthreads();
  if (bars->abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  cluster_sync_all();
  if (run && warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem, 512);
  }
}

}  // namespace h3a
