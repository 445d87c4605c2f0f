// Q/K preparation kernels (HBM-bound): per-head RMSNorm over d=128 then rotation by a (cos,sin) table,
// written head-major as bf16 or as e4m3 with one absmax scale per (head, 128-token block); and the
// builder of that table from a float position grid.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace h3a {

constexpr int kPrepThreads = 256;

struct PrepArgs {
  const __nv_bfloat16* in;
  void* out;            // bf16 [H, L, 128] or e4m3 bytes [H, L, 128]
  float* scale;         // fp8: [H, nblk]
  long long stride_l, stride_h;
  int L, H, nblk;
  const float* rope;    // [L, 64, 2] or null
  const float* weight;  // [128] or null
  float eps;
  int rope_half;        // 0: pairs (2j,2j+1); 1: pairs (j, j+64)
  int no_norm;          // skip the RMSNorm (re-layout / quantisation of rows that are already prepared, or of V)
  // Sequence parallelism (n_ranks > 0, bf16 only): head h of the input is global head head0 + h, owned by rank
  // (head0 + h) / heads_per_rank [blocks] or (head0 + h) % n_ranks [round robin]; its rows go to that rank's
  // [heads_per_rank, L_total, 128] buffer (own memory or a peer GPU's), token l at row row_offset + l.
  void* rank_out[8];
  int n_ranks, heads_per_rank, round_robin, head0, row_offset, L_total;
  int head_rot;         // the grid's y index is rotated by this many heads (order of the stores, not their content)
};

// where row l of (local) head `head` is written: head-major in `out`, or at the head's owner
__device__ __forceinline__ __nv_bfloat16* prep_dst_bf16(const PrepArgs& a, int head, int l) {
  if (a.n_ranks > 0) {
    const int h = a.head0 + head;
    const int owner = a.round_robin ? h % a.n_ranks : h / a.heads_per_rank;
    const int slot = a.round_robin ? h / a.n_ranks : h % a.heads_per_rank;
    return static_cast<__nv_bfloat16*>(a.rank_out[owner]) + (static_cast<long long>(slot) * a.L_total + a.row_offset + l) * 128;
  }
  return static_cast<__nv_bfloat16*>(a.out) + (static_cast<long long>(head) * a.L + l) * 128;
}

// One CTA = one (128-token block, head).  Thread (r = tid/8, sub = tid%8) owns, in each of 4 passes,
// the two 8-element chunks [8*sub, 8*sub+8) and [64+8*sub, 64+8*sub+8) of row pass*32 + r, so that both
// rotary pair conventions stay inside a thread and a row's sum of squares is an 8-lane shuffle.
// kBulk (scatter mode, bf16): the CTA's 128 prepared rows are contiguous at their owner (32 KB), so they are staged in
// shared memory and leave as ONE bulk asynchronous copy (cp.async.bulk, shared -> global) instead of 16-byte stores:
// large transfers are what NVLink moves best when the owner is another GPU.  The destination is only written.
template <bool kFp8, bool kBulk = false>
__global__ void __launch_bounds__(kPrepThreads) qk_prep_kernel(const PrepArgs a) {
  const int blk = blockIdx.x;
  const int head = a.head_rot ? static_cast<int>((blockIdx.y + a.head_rot) % a.H) : static_cast<int>(blockIdx.y);
  const int tid = threadIdx.x;
  const int r = tid >> 3, sub = tid & 7;
  __shared__ float warp_max[kPrepThreads / 32];
  __shared__ __align__(128) __nv_bfloat16 stage[kBulk ? 128 * 128 : 8];

  float w_lo[8], w_hi[8];
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    w_lo[x] = a.weight ? a.weight[8 * sub + x] : 1.0f;
    w_hi[x] = a.weight ? a.weight[64 + 8 * sub + x] : 1.0f;
  }

  float v[4][16];
  float amax = 0.0f;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int l = blk * 128 + pass * 32 + r;
    const bool valid = l < a.L;
    float x_lo[8], x_hi[8];
    if (valid) {
      const __nv_bfloat16* src = a.in + static_cast<long long>(l) * a.stride_l + static_cast<long long>(head) * a.stride_h;
      const uint4 u0 = *reinterpret_cast<const uint4*>(src + 8 * sub);
      const uint4 u1 = *reinterpret_cast<const uint4*>(src + 64 + 8 * sub);
      const __nv_bfloat162* b0 = reinterpret_cast<const __nv_bfloat162*>(&u0);
      const __nv_bfloat162* b1 = reinterpret_cast<const __nv_bfloat162*>(&u1);
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float2 f0 = __bfloat1622float2(b0[x]);
        const float2 f1 = __bfloat1622float2(b1[x]);
        x_lo[2 * x] = f0.x; x_lo[2 * x + 1] = f0.y;
        x_hi[2 * x] = f1.x; x_hi[2 * x + 1] = f1.y;
      }
    } else {
#pragma unroll
      for (int x = 0; x < 8; ++x) { x_lo[x] = 0.f; x_hi[x] = 0.f; }
    }
    float ss = 0.f;
#pragma unroll
    for (int x = 0; x < 8; ++x) ss += x_lo[x] * x_lo[x] + x_hi[x] * x_hi[x];
    ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 1);
    ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 2);
    ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 4);
    const float rinv = a.no_norm ? 1.0f : rsqrtf(ss * (1.0f / 128.0f) + a.eps);
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      x_lo[x] = x_lo[x] * rinv * w_lo[x];
      x_hi[x] = x_hi[x] * rinv * w_hi[x];
    }
    if (a.rope && valid) {
      const float* tab = a.rope + static_cast<long long>(l) * 128;  // 64 pairs x (cos, sin)
      if (a.rope_half) {
        // pair e = (e, e+64), e = 8*sub + x
        float cs[16];
        const float4* t4 = reinterpret_cast<const float4*>(tab + 16 * sub);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float4 q = t4[x];
          cs[4 * x] = q.x; cs[4 * x + 1] = q.y; cs[4 * x + 2] = q.z; cs[4 * x + 3] = q.w;
        }
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          const float c = cs[2 * x], s = cs[2 * x + 1];
          const float p = x_lo[x], q = x_hi[x];
          x_lo[x] = p * c - q * s;
          x_hi[x] = p * s + q * c;
        }
      } else {
        // pair j = (2j, 2j+1): chunk lo holds pairs 4*sub..4*sub+3, chunk hi holds pairs 32+4*sub..
        const float4* t_lo = reinterpret_cast<const float4*>(tab + 8 * sub);
        const float4* t_hi = reinterpret_cast<const float4*>(tab + 64 + 8 * sub);
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const float4 cl = t_lo[x], ch = t_hi[x];
          float p, q;
          p = x_lo[4 * x]; q = x_lo[4 * x + 1];
          x_lo[4 * x] = p * cl.x - q * cl.y; x_lo[4 * x + 1] = p * cl.y + q * cl.x;
          p = x_lo[4 * x + 2]; q = x_lo[4 * x + 3];
          x_lo[4 * x + 2] = p * cl.z - q * cl.w; x_lo[4 * x + 3] = p * cl.w + q * cl.z;
          p = x_hi[4 * x]; q = x_hi[4 * x + 1];
          x_hi[4 * x] = p * ch.x - q * ch.y; x_hi[4 * x + 1] = p * ch.y + q * ch.x;
          p = x_hi[4 * x + 2]; q = x_hi[4 * x + 3];
          x_hi[4 * x + 2] = p * ch.z - q * ch.w; x_hi[4 * x + 3] = p * ch.w + q * ch.z;
        }
      }
    }
    if constexpr (kFp8) {
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        v[pass][x] = x_lo[x];
        v[pass][8 + x] = x_hi[x];
        amax = fmaxf(amax, fmaxf(fabsf(x_lo[x]), fabsf(x_hi[x])));
      }
    } else if (valid) {
      __nv_bfloat16* dst = kBulk ? stage + (pass * 32 + r) * 128 : prep_dst_bf16(a, head, l);
      uint4 o0, o1;
      __nv_bfloat162* p0 = reinterpret_cast<__nv_bfloat162*>(&o0);
      __nv_bfloat162* p1 = reinterpret_cast<__nv_bfloat162*>(&o1);
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        p0[x] = __floats2bfloat162_rn(x_lo[2 * x], x_lo[2 * x + 1]);
        p1[x] = __floats2bfloat162_rn(x_hi[2 * x], x_hi[2 * x + 1]);
      }
      *reinterpret_cast<uint4*>(dst + 8 * sub) = o0;
      *reinterpret_cast<uint4*>(dst + 64 + 8 * sub) = o1;
    }
  }

  if constexpr (kFp8) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if ((tid & 31) == 0) warp_max[tid >> 5] = amax;
    __syncthreads();
    float bm = warp_max[0];
#pragma unroll
    for (int w = 1; w < kPrepThreads / 32; ++w) bm = fmaxf(bm, warp_max[w]);
    const float scale = bm > 0.f ? bm / 448.0f : 1.0f;
    const float inv = 1.0f / scale;
    if (tid == 0) a.scale[static_cast<long long>(head) * a.nblk + blk] = scale;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int l = blk * 128 + pass * 32 + r;
      if (l < a.L) {
        uint8_t* dst = static_cast<uint8_t*>(a.out) + (static_cast<long long>(head) * a.L + l) * 128;
        uint32_t w[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float e0 = fminf(fmaxf(v[pass][4 * x] * inv, -448.f), 448.f);
          const float e1 = fminf(fmaxf(v[pass][4 * x + 1] * inv, -448.f), 448.f);
          const float e2 = fminf(fmaxf(v[pass][4 * x + 2] * inv, -448.f), 448.f);
          const float e3 = fminf(fmaxf(v[pass][4 * x + 3] * inv, -448.f), 448.f);
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(e0, e1), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(e2, e3), __NV_SATFINITE, __NV_E4M3);
          w[x] = lo | (hi << 16);
        }
        *reinterpret_cast<uint2*>(dst + 8 * sub) = make_uint2(w[0], w[1]);
        *reinterpret_cast<uint2*>(dst + 64 + 8 * sub) = make_uint2(w[2], w[3]);
      }
    }
  }
  if constexpr (kBulk) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the staged rows, written by ordinary stores, are read by the copy engine
    __syncthreads();
    if (tid == 0) {
      const int rows = min(128, a.L - blk * 128);
      const unsigned long long dst = reinterpret_cast<unsigned long long>(prep_dst_bf16(a, head, blk * 128));
      const uint32_t src = static_cast<uint32_t>(__cvta_generic_to_shared(stage));
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(rows * 256) : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // complete (not only read) before the CTA may leave
    }
  }
  if (a.n_ranks > 1) __threadfence_system();  // rows stored into other GPUs' memory: ordered before this kernel's completion is observed
}

// table[l][j] = (cos, sin)(pos[l][axis(j)] * theta^(-2 jj / d_axis)), computed in double like the host
// float64 grid it replaces, stored fp32.
__global__ void rope_table_kernel(const float* __restrict__ pos, int L, int d0, int d1, int d2, float theta, float* __restrict__ table) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(L) * 64) return;
  const int l = static_cast<int>(idx >> 6), j = static_cast<int>(idx & 63);
  int axis, jj, da;
  if (j < d0 / 2) { axis = 0; jj = j; da = d0; }
  else if (j < (d0 + d1) / 2) { axis = 1; jj = j - d0 / 2; da = d1; }
  else { axis = 2; jj = j - (d0 + d1) / 2; da = d2; }
  const double inv = pow(static_cast<double>(theta), -2.0 * jj / da);
  const double ang = static_cast<double>(pos[static_cast<long long>(l) * 3 + axis]) * inv;
  double s, c;
  sincos(ang, &s, &c);
  reinterpret_cast<float2*>(table)[idx] = make_float2(static_cast<float>(c), static_cast<float>(s));
}

}  // namespace h3a
