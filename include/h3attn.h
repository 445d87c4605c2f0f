/*
 * h3attn — C ABI of the B200 (sm_100a) attention path for the Pika H3 Flex joint video+audio DiT.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, and returns an int32 status
 * (0 = H3A_OK, negative = error; h3a_status_string() names it).  Nothing throws or aborts across the
 * boundary.  Unless a comment says otherwise the library allocates nothing on the device, keeps no
 * pointer after it returns, and is stream-ordered and asynchronous: the caller owns every buffer,
 * the workspace and the status word, and may call from several host threads on different streams.
 *
 * What each entry point replaces in the reference project (Pika-Labs/Pika-H3-Flex): the reference
 * runs its DiT through `self.model(**model_inputs)` (src/pika_h3/core/wrapper.py:248) with the kwargs
 * assembled at src/pika_h3/core/wrapper.py:192-204; the per-block attention between the
 * `to_q/to_k/to_v` and `to_out.0` projections (module names fixed by src/pika_h3/core/loader.py:9)
 * lives in the un-vendored `diffusers` build pinned at pyproject.toml:12 (file
 * models/transformers/transformer_minimax_h3.py, identity pinned at src/pika_h3/runtime.py:9).
 * The functions below are what a binding for that per-block attention calls.
 */
#ifndef H3ATTN_H_
#define H3ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define H3A_VERSION_MAJOR 0
#define H3A_VERSION_MINOR 2

/* status codes */
enum {
  H3A_OK = 0,
  H3A_ERR_ARG = -1,     /* null pointer, bad enum, bad flag */
  H3A_ERR_ALIGN = -2,   /* pointer not 16-byte aligned, stride not a multiple of 16 bytes */
  H3A_ERR_SHAPE = -3,   /* head dim != 128, batch != 1, empty or oversized extent */
  H3A_ERR_ARCH = -4,    /* current device is not compute capability 10.x */
  H3A_ERR_LAUNCH = -5,  /* CUDA runtime / driver call failed */
  H3A_ERR_TIMEOUT = -6, /* a bounded device-side wait ran out (read back from the status word) */
  H3A_ERR_WORKSPACE = -7, /* workspace missing or too small */
  H3A_ERR_DRIVER = -8,  /* driver entry point for tensor-map encoding not found */
  H3A_ERR_STATIC_SCRATCH = -9, /* h3a_attn_fwd_sparse_static: block index larger than the built-in scratch */
  H3A_ERR_INDEX = -10,  /* the device-side check of a block index failed (read back from the status word) */
  H3A_ERR_BOUND = -11   /* logit_bound did not hold for the data: a row sum under- or overflowed (status word) */
};

#define H3A_MAX_RANKS 8 /* GPUs one sequence can be spread over (one NVSwitch domain) */

/* attention modes */
enum {
  H3A_MODE_DENSE_BF16 = 0,   /* Q, K, V bf16 */
  H3A_MODE_FP8_QK = 1,       /* Q, K e4m3 with per-(head, 128-token) fp32 scales; V bf16 */
  H3A_MODE_BLOCK_SPARSE = 2  /* bf16, only the 128x128 key tiles listed in the CSR block index */
};

/* rotary pair conventions */
enum {
  H3A_ROPE_INTERLEAVED = 0, /* pair j = dims (2j, 2j+1) */
  H3A_ROPE_HALF = 1         /* pair j = dims (j, j + 64) */
};

/* flags for h3a_prep_params.flags */
#define H3A_PREP_FP8 1u /* write e4m3 Q/K and per-(head, 128-token) scales instead of bf16 */
#define H3A_PREP_NO_NORM 2u /* skip the RMSNorm; with no rotation table either the call is a plain re-layout to
                               head-major (what V needs) or, with H3A_PREP_FP8, a quantisation of prepared rows */

/*
 * Forward attention  O = softmax(Q K^T * softmax_scale) V, non-causal, one document (batch 1, as the
 * reference: src/pika_h3/core/wrapper.py:231-232).
 * Tensors are addressed as x[l * stride_l + h * stride_h + c], c in [0,128) contiguous; strides are in
 * ELEMENTS of that tensor's type, so [L,H,128] and [H,L,128] (and Ulysses views of either) need no copy.
 * Lq may differ from Lk (cross-attention to a short text sequence).
 */
typedef struct h3a_attn_params {
  const void* q;          /* bf16, or e4m3 bytes in FP8_QK mode */
  const void* k;          /* bf16, or e4m3 bytes in FP8_QK mode */
  const void* v;          /* bf16 */
  void* o;                /* bf16 out */
  int64_t q_stride_l, q_stride_h;
  int64_t k_stride_l, k_stride_h;
  int64_t v_stride_l, v_stride_h;
  int64_t o_stride_l, o_stride_h;
  int32_t Lq, Lk, H, d;   /* d must be 128 */
  int32_t B;              /* must be 1 */
  int32_t mode;           /* H3A_MODE_* */
  float softmax_scale;    /* <= 0 selects 1/sqrt(d) */
  const float* q_scale;   /* FP8_QK: [H, ceil(Lq/128)] fp32, else NULL */
  const float* k_scale;   /* FP8_QK: [H, ceil(Lk/128)] fp32, else NULL */
  const int32_t* row_ptr; /* BLOCK_SPARSE: [ceil(Lq/128)+1] device int32, non-decreasing, 0 .. nnz, else NULL */
  const int32_t* col_idx; /* BLOCK_SPARSE: [nnz] device int32 in [0, ceil(Lk/128)), strictly ascending inside each row.
                             The index is checked on the device: entries that break a rule are left out, nothing is
                             written outside the workspace, and the status word (when given) receives code 10, after
                             which the attention launch does nothing (h3a_read_device_status: H3A_ERR_INDEX). */
  int32_t nnz;            /* BLOCK_SPARSE: number of kept tiles (host value of row_ptr[last]) */
  float* lse;             /* optional [H, Lq] fp32 natural-log-sum-exp out, or NULL */
  void* workspace;        /* device scratch of h3a_attn_workspace_bytes() bytes: required for BLOCK_SPARSE
                             (merged tile plan); optional for the dense modes (partial sums of a split last
                             wave of CTAs, or the redo list of the two-launch online softmax: without it, or when
                             it is too small, the launch simply does without) */
  size_t workspace_bytes;
  int32_t* status_word;   /* optional device int32; a kernel that gives up a bounded wait (or finds a malformed
                             block index) writes a non-zero code here and returns; while it is non-zero every
                             later launch given the same word does nothing, so one word can be shared by all the
                             calls of a forward pass and read once at its end; zero it before the first use */
  int64_t wait_limit_ns;  /* bound for each device-side wait; <= 0 selects 2 s */
  float logit_bound;      /* optional: a value B with |q.k| * softmax_scale <= B for every query/key pair (with
                             QK-RMSNorm: 128 * max|w_q| * max|w_k| * softmax_scale).  When 0 < B <= 110 the kernel
                             uses a fixed softmax reference instead of a running row maximum: the result is the same
                             softmax (any reference is exact while the terms stay inside fp32's range), without the max
                             pass and without rescaling.  The reference is B up to 30, slides to 0 at B = 60, stays 0 to
                             B = 74 and is B - 74 beyond.  Up to B = 64 every row of any data within the bound is served;
                             from there to 110 every row whose largest logit is at least ref - 64 (-64 up to B = 74, then
                             B - 138: at least one key not extremely anti-aligned with the query).  A row outside that, or data that violates the
                             bound far enough for a row sum to under- or overflow, is REPORTED through the status word
                             (code 11, H3A_ERR_BOUND; pass a status word) and that launch's output must not be used.
                             0, or a value above 110 = no usable bound: online softmax with a running row maximum. */
  int32_t sparse_heavy_pairs; /* BLOCK_SPARSE scheduling hint: the first this-many pairs of query tiles (256 rows
                             each) list far more key tiles than the rest (the dense audio rows of the joint
                             sequence); their CTAs of all heads are started first.  0 = no hint.  Never affects
                             results. */
  /* Sequence parallelism, return trip: when o_n_ranks > 1 the output rows are stored where their token lives instead
     of in `o`: query row g goes to o_rank_base[g / o_rank_rows] at row g % o_rank_rows, addressed with o_stride_l /
     o_stride_h like `o` (each base already points at this launch's first head).  The bases are device addresses of
     this process or of peer GPUs (see h3a_peer_open); they are only ever stored to.  `o` is then unused but must still
     be a valid aligned pointer (pass o_rank_base[own rank]). */
  void* o_rank_base[H3A_MAX_RANKS];
  int32_t o_n_ranks;      /* 0 or 1: everything goes to `o` */
  int32_t o_rank_rows;    /* tokens per rank */
} h3a_attn_params;

/*
 * Q/K preparation: per-head RMSNorm over d=128 (fp32 math), then rotation by a (cos,sin) table.
 * Replaces the norm + rotary step that the reference's DiT applies to to_q/to_k outputs before
 * attention (in the un-vendored model file; positions come from src/pika_h3/core/packing.py:126-133).
 * Input  x[l*in_stride_l + h*in_stride_h + c] bf16.
 * Output bf16 [H, L, 128] head-major contiguous, or with H3A_PREP_FP8 e4m3 [H, L, 128] bytes plus
 * scales [H, ceil(L/128)] fp32 (scale = absmax/448 of the block, 1 for an all-zero block).
 */
typedef struct h3a_prep_params {
  const void* q_in;  const void* k_in;     /* bf16; either may be NULL to skip that tensor */
  void* q_out;       void* k_out;
  float* q_scale;    float* k_scale;       /* H3A_PREP_FP8 only */
  int64_t q_stride_l, q_stride_h, k_stride_l, k_stride_h; /* elements */
  int32_t Lq, Lk, H, d;                    /* d must be 128 */
  const float* q_rope;  const float* k_rope; /* [L, 64, 2] fp32 (cos, sin) per token and pair, or NULL = no rotation */
  const float* q_weight; const float* k_weight; /* [128] fp32 RMSNorm weights, or NULL = ones */
  float eps;                               /* <= 0 selects 1e-6 */
  int32_t rope_mode;                       /* H3A_ROPE_* */
  uint32_t flags;                          /* H3A_PREP_* */
} h3a_prep_params;

/* Library version. */
int32_t h3a_version(int32_t* major, int32_t* minor);

/* Human-readable name of a status code (static storage). */
const char* h3a_status_string(int32_t status);

/* Bytes of device scratch for these params on the current device.  BLOCK_SPARSE: what h3a_attn_fwd needs.
 * Dense modes (optional scratch): with a logit bound, what lets the launch split its last wave of CTAs over the key
 * range (0 when that does not pay: short key range, or a CTA count that already fills whole waves); without a usable
 * bound, the redo list of the two-launch online softmax (without it the launch is the running-maximum kernel alone,
 * about 15 % slower).  Needs Lq, Lk, H, mode and logit_bound only. */
int32_t h3a_attn_workspace_bytes(const h3a_attn_params* p, size_t* bytes);

/* Which kernel h3a_attn_fwd would launch for these params on the current device (needs Lq, Lk, H, mode, logit_bound,
 * nnz for BLOCK_SPARSE, workspace / workspace_bytes for the split): an OR of the bits below.  For reports and tests. */
#define H3A_KERNEL_CTA_PAIRS 1        /* attn_fwd_pair_kernel (two CTAs per MMA) instead of attn_fwd_kernel */
#define H3A_KERNEL_FIXED_REFERENCE 2  /* fixed softmax reference from logit_bound instead of the running row maximum */
#define H3A_KERNEL_SPLIT_LAST_WAVE 4  /* the CTA pairs of the last wave split the key range (+ combine_partials_kernel) */
#define H3A_KERNEL_ONLINE_TWO_LAUNCH 8 /* online softmax as two launches: per-row fixed reference from the first key tile,
                                          then the running-maximum kernel over the few CTA pairs that outgrew it */
#define H3A_KERNEL_PERSISTENT 16       /* short key ranges with a logit bound: persistent blocks walk the query tiles (with
                                          CTA_PAIRS: a head's K / V stays in shared memory, up to 4 key tiles; without:
                                          one single-CTA block per SM).  H3A_RESIDENT=0 / H3A_PERSIST=0 in the environment,
                                          read once per process, switch these forms off; H3A_PAIR=0 all CTA-pair kernels */
int32_t h3a_attn_kernel_choice(const h3a_attn_params* p, int32_t* choice);

/* Launch the attention forward on `stream` (a cudaStream_t passed as void*). */
int32_t h3a_attn_fwd(const h3a_attn_params* p, void* stream);

/* Launch the Q/K preparation on `stream`. */
int32_t h3a_qk_prep(const h3a_prep_params* p, void* stream);

/*
 * Sequence parallelism, outbound trip.  (The reference runs one request on one GPU, README.md:115; this is the
 * multi-GPU path BASELINE's configuration 4 asks for.)  Each rank holds a token shard of every head and each head is
 * computed by one rank.  h3a_qk_prep_scatter runs the same preparation as h3a_qk_prep on this rank's tokens and
 * stores every prepared row straight where it is needed: head `h` (counted from `head0` for the first head of the
 * input) belongs to rank  h / heads_per_rank  (round_robin = 0) or  h % n_ranks  (round_robin = 1), in that rank's
 * head slot  h % heads_per_rank  or  h / n_ranks, and token l of this shard is row `row_offset + l` of the full
 * sequence: the row goes to  base[rank] + ((slot * L_total) + row_offset + l) * 128  elements (bf16).  base[p] is rank
 * p's [heads_per_rank, L_total, 128] buffer: this process's own memory or a peer GPU's, opened with h3a_peer_open;
 * peer memory is only ever stored to.  q_out / k_out / scales of `p` are ignored and H3A_PREP_FP8 is refused (block
 * scales need whole 128-token blocks of the FULL sequence: quantise on the owning rank after the exchange, with
 * H3A_PREP_NO_NORM | H3A_PREP_FP8).  Either of q_to / k_to may be NULL together with its input.  The values for V go
 * through the same call with H3A_PREP_NO_NORM and no rotation table.  The stores of one call are complete, for every
 * GPU, when the kernel has finished; the ranks still have to meet (a barrier) before the owners read.
 */
typedef struct h3a_head_scatter {
  void* base[H3A_MAX_RANKS];
  int32_t n_ranks;        /* 1 .. H3A_MAX_RANKS */
  int32_t heads_per_rank; /* head slots in every rank's buffer */
  int32_t round_robin;    /* 0: heads in blocks, 1: dealt round robin */
  int32_t head0;          /* global index of the input's first head */
  int32_t row_offset;     /* this shard's first token in the full sequence */
  int32_t L_total;        /* tokens of the full sequence */
  int32_t start_head;     /* the launch walks the input's heads in the order start_head, start_head + 1, ... (wrapping).
                             Results do not depend on it; give every rank a different start (the first head of the NEXT
                             rank's block, say): with the same order everywhere all ranks would store to the same owner
                             at the same time and share that one GPU's inbound NVLink bandwidth. */
} h3a_head_scatter;
int32_t h3a_qk_prep_scatter(const h3a_prep_params* p, const h3a_head_scatter* q_to, const h3a_head_scatter* k_to, void* stream);

/*
 * Device memory that other processes on the same machine can store to.  (No counterpart in the reference.)  These
 * four are the only entry points that allocate or map device memory; everything else works on caller-owned buffers.
 * h3a_peer_alloc: cudaMalloc of `bytes` on the current device plus the 64-byte inter-process handle of the
 * allocation, to be sent to the other ranks by any host channel.  h3a_peer_open: map another process's allocation
 * into this one (enables peer access between the two GPUs); the pointer is valid until h3a_peer_close.  The owner
 * frees with h3a_peer_free after every peer has closed.
 */
#define H3A_PEER_HANDLE_BYTES 64
int32_t h3a_peer_alloc(size_t bytes, void** ptr, uint8_t handle[H3A_PEER_HANDLE_BYTES]);
int32_t h3a_peer_open(const uint8_t handle[H3A_PEER_HANDLE_BYTES], void** ptr);
int32_t h3a_peer_close(void* ptr);
int32_t h3a_peer_free(void* ptr);

/*
 * Build the (cos, sin) table [L, 64, 2] fp32 on the device from a float position grid pos[L,3]
 * (device fp32; the reference builds this grid on the host in float64, src/pika_h3/core/packing.py:166,
 * and moves it to the device each forward, src/pika_h3/core/wrapper.py:164-166).
 * Head-dim split over (t,h,w) is split[0..2] (sum 128, each even); pair j of axis a turns by
 * pos[:,a] * theta^(-2j/split[a]).
 */
int32_t h3a_rope_table(const float* pos, int32_t L, const int32_t split[3], float theta, float* table, void* stream);

/*
 * Host-side block-index builder for the spatiotemporal-neighbourhood mask over 128x128 tiles.
 * Token order: n_audio audio tokens, then a (T,Hg,Wg) video grid frame-major / row-major
 * (src/pika_h3/core/packing.py:49-54).  A video-video tile is kept when some query token of the row
 * tile and some key token of the column tile differ by at most (wt,wh,ww) on the three axes; every
 * tile holding audio keys is kept; row tiles holding audio queries keep every column.
 * Two-call protocol: with col_idx == NULL only *nnz is written; otherwise row_ptr[nqb+1] and
 * col_idx[*nnz] (host memory, capacity passed in *nnz) are filled, columns ascending.
 */
int32_t h3a_build_block_index(int32_t T, int32_t Hg, int32_t Wg, int32_t n_audio,
                              int32_t wt, int32_t wh, int32_t ww,
                              int32_t* row_ptr, int32_t* col_idx, int64_t* nnz);

/*
 * Strided copy between pinned host memory and the device (to_host = 0: host -> device, 1: device -> host):
 * `rows` rows of `width_bytes`, row pitches in bytes.  Used by the host-buffer path to move the slice of a
 * group of heads of a token-major [L, H, 128] tensor (width = heads * 256 bytes, pitch = H * 256 bytes) while
 * another group is being computed; the reference moves whole tensors with `.to(device)` before the forward
 * (src/pika_h3/core/wrapper.py:164-166, src/pika_h3/pipeline.py:115,128).
 */
int32_t h3a_memcpy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                           int32_t to_host, void* stream);

/*
 * Block-sparse attention for callers that must not allocate device memory.  (No counterpart in the
 * reference project; it exists for hosts built around this library.)
 *
 * Who needs it: an embedding runtime that reserves the whole GPU for its own arena at start-up and forbids
 * cudaMalloc afterwards -- a serving process with a fixed memory plan, where a late allocation can fail,
 * fragment the arena or stall every stream while the driver synchronises the device -- has no buffer to pass
 * as `workspace`.  Here the scratch for the merged tile plan is a fixed array inside the library:
 * 262144 int32 (1 MiB) of device memory, held by every GPU that loads the library until the process exits.
 *
 * Same arguments, same kernel choice (logit_bound, density, sparse_heavy_pairs) and bit-identical results as
 * h3a_attn_fwd with mode == H3A_MODE_BLOCK_SPARSE (any other mode returns H3A_ERR_ARG); `workspace` and
 * `workspace_bytes` are ignored.  The caller still owns q, k, v, o, the block index, lse and the status word.
 *   - The 1 MiB is taken from the device when the library's code is loaded into that device's context, which
 *     with CUDA's default lazy loading is the first call into the library on that device, not dlopen(): an
 *     arena that claims "the rest of the GPU" must leave that much free.
 *   - Limit: nnz + ceil(Lq/256) must be <= 262144 (h3a_static_scratch_capacity reports it), otherwise
 *     H3A_ERR_STATIC_SCRATCH and nothing is launched.
 *   - It calls no cudaMalloc, cudaFree or other allocating routine.
 *   - The first call on each device looks up the array's device address (once per device, with that device
 *     current); make that first call before starting any stream capture on the device.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Nothing in it has
 *     to start at zero: each call rewrites every entry it later reads.  Two calls whose kernels can overlap on
 *     the GPU (different streams, no ordering between them) race on it: serialise them.
 */
int32_t h3a_attn_fwd_sparse_static(const h3a_attn_params* p, void* stream);

/* Capacity of that built-in scratch in plan entries (int32). */
int32_t h3a_static_scratch_capacity(size_t* plan_entries);

/*
 * Diagnostic for the bounded device-side waits (no counterpart in the reference): launches one warp that waits,
 * with the helper the attention kernels use, on a barrier that nothing ever signals.  After at most
 * wait_limit_ns (1 ns .. 1 s) the warp gives up, writes code 9 into *status_word and returns; the context stays
 * usable.  Lets a deployment check that a lost signal turns into H3A_ERR_TIMEOUT instead of a hung GPU.
 */
int32_t h3a_selftest_wait_timeout(int32_t* status_word, int64_t wait_limit_ns, void* stream);

/*
 * Projection with the attention preparation fused into its epilogue.  Replaces, for one of Q / K / V, the module
 * call `attn.to_q(hidden_states)` on a LoRA-wrapped Linear (reference: src/pika_h3/core/loader.py:9 names the
 * wrapped projections, :20-49 applies rank-128 LoRA with alpha = rank, src/pika_h3/pipeline.py:34) followed by
 * the per-head RMSNorm + rotation that h3a_qk_prep does as a separate pass:
 *   Y[l, n] = sum_k x[l, k] w[n, k]  +  sum_r lora_t[l, r] lora_bs[n, r]  +  bias[n]
 * x [L, K] and w [N, K] (nn.Linear layout) are bf16 with K contiguous; N = heads * 128.  The LoRA term is optional:
 * lora_t = x A^T [L, R] (the caller computes this thin product) and lora_bs = (alpha / rank) * B [N, R].
 * epilogue H3A_PROJ_STORE writes Y as bf16; H3A_PROJ_PREP applies RMSNorm over each head's 128 columns (times
 * norm_weight when given), then the rotation by `rope` ([L, 64, 2] fp32, optional), then writes bf16;
 * H3A_PROJ_PREP_FP8 additionally quantises to e4m3 exactly as h3a_qk_prep does with H3A_PREP_FP8.  Output
 * element (l, head, c) goes to out[l * out_stride_l + head * out_stride_h + c] (strides in elements).
 * Runs on CTA pairs (256 tokens x 256 columns per pair); needs compute capability 10.x.
 */
#define H3A_PROJ_STORE 0
#define H3A_PROJ_PREP 1
#define H3A_PROJ_PREP_FP8 2 /* as PREP, then e4m3 bytes + one absmax / 448 scale per (head, 128-token block) */
typedef struct h3a_proj_params {
  const void* x;          /* [L, K] bf16 */
  const void* w;          /* [N, K] bf16 */
  const void* lora_t;     /* [L, R] bf16 or NULL */
  const void* lora_bs;    /* [N, R] bf16 or NULL */
  const float* bias;      /* [N] fp32 or NULL */
  const float* rope;      /* H3A_PROJ_PREP: [L, 64, 2] fp32 (cos, sin) or NULL */
  const float* norm_weight; /* H3A_PROJ_PREP: [128] fp32 or NULL (unit weights) */
  void* out;              /* bf16; H3A_PROJ_PREP_FP8: e4m3 bytes (strides then count bytes) */
  float* out_scale;       /* H3A_PROJ_PREP_FP8: [N / 128, ceil(L / 128)] fp32, else NULL */
  int64_t x_stride_l, w_stride_n, lora_t_stride_l, lora_bs_stride_n; /* row strides in elements, multiples of 8 */
  int64_t out_stride_l, out_stride_h;
  int32_t L, K, N, R;
  int32_t epilogue;       /* H3A_PROJ_* */
  int32_t rope_mode;      /* H3A_ROPE_* */
  float eps;              /* <= 0 selects 1e-6 */
  int32_t* status_word;   /* as in h3a_attn_params */
  int64_t wait_limit_ns;
  const struct h3a_head_scatter* out_to; /* optional (H3A_PROJ_STORE / H3A_PROJ_PREP, head-major output): sequence parallelism,
                             the rows of output head h go straight to the rank that computes head out_to->head0 + h
                             (see h3a_qk_prep_scatter) instead of to `out`, which is then ignored; L is this rank's
                             token shard.  The projection's epilogue is then also the outbound trip of the reshard. */
} h3a_proj_params;
int32_t h3a_proj_fwd(const h3a_proj_params* p, void* stream);

/*
 * Pre-attention adaptive layer norm: y = norm(x) * (1 + scale[idx[l]]) + shift[idx[l]] per token row l.  Replaces the
 * reference's patched `self.norm(hidden_states)` followed by `hidden_states * (1.0 + scale.index_select(0,
 * timestep_indices)) + shift.index_select(0, timestep_indices)` (patches/0001-h3-adaln-fp32.patch:36-40; the
 * modulation tables come from the fp32-SiLU Linear of the same patch, :14-26).  x, y [L, D] bf16 (D a multiple of
 * 8, at most 8192), scale / shift [T, D] bf16 with their own row strides (they may be the two halves of one
 * [T, 2 D] tensor), idx [L] int64 or NULL (every token uses row 0).  norm is LayerNorm (rms = 0) or RMSNorm
 * (rms = 1) over D in fp32, with optional fp32 weight / bias [D].  HBM-bound: one read and one write of the rows.
 */
typedef struct h3a_adaln_params {
  const void* x;
  void* y;
  const void* scale;
  const void* shift;
  const int64_t* idx;
  const float* weight;
  const float* bias;
  int64_t x_stride, y_stride, scale_stride, shift_stride; /* row strides in elements, multiples of 8 */
  int32_t L, D, T;
  int32_t rms;
  float eps; /* <= 0 selects 1e-6 */
} h3a_adaln_params;
int32_t h3a_adaln_norm(const h3a_adaln_params* p, void* stream);

/* Copy the device status word to the host after synchronising `stream`.  Returns H3A_OK for 0, H3A_ERR_INDEX when a
 * block index failed its device-side check (low byte 10), H3A_ERR_BOUND when a logit bound did not hold (low byte
 * 11), H3A_ERR_TIMEOUT for every other non-zero value; *raw (optional)
 * receives the word: low byte = which wait or check, upper bits = the CTA (waits) or query tile (index check). */
int32_t h3a_read_device_status(const int32_t* status_word, void* stream, int32_t* raw);

#ifdef __cplusplus
}
#endif
#endif /* H3ATTN_H_ */
