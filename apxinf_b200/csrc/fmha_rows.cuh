// Multi-query attention for a handful of query rows (the B=1 action expert: 10 tokens x 8
// heads = 80 rows over 532 cached keys). The work is tiny (43 MFLOP, 0.5 MB of K/V); what
// counts is the length of the dependent chain. One launch, no scratch in global memory:
//
//   * a thread-block CLUSTER of 8 CTAs serves one 16-row query tile (row = token * heads + head,
//     all heads share the K/V head); the CTAs split the keys;
//   * each CTA asks for its K slice, V slice and the query tile at once (cp.async, everything in
//     flight together), computes S = Q K^T on mma.sync m16n8k16 fragments, the slice's
//     probabilities, and an unnormalised partial output O = P V (V transposed on the fly by
//     ldmatrix.trans) with its row maxima and sums, all in its own shared memory;
//   * after one cluster barrier every CTA merges one eighth of the head dimension over the
//     eight partials through distributed shared memory (log-sum-exp weights) and writes bf16 /
//     e4m3 output rows.
//
// No cluster multicast and no remote TMA anywhere: plain ld.shared::cluster reads of the
// peers' partials. Same operands and output conventions as fmha_online_kernel; replaces, for
// launches with few query rows, the key-split kernel pair of fmha_split.cuh (two dependent
// launches through a global scratch) and with it the reference's three-launch cuBLAS MQA
// (crates/apxinf-cuda/adapters/cublas_adapter.cu:89-132).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "fmha.h"
#include "launch.cuh"

namespace pi05 {

constexpr int kRowsCluster = 8;    // CTAs per cluster = key slices per query tile
constexpr int kRowsThreads = 256;  // 8 warps
constexpr int kRowsWarps = kRowsThreads / 32;

struct FmhaRowsParams {
  const __nv_bfloat16* q;  // row r of sample b: q + b * q_sb1 + (r / heads) * q_ld + (r % heads) * q_sb0
  long long q_ld, q_sb0, q_sb1;
  const __nv_bfloat16* k;  // [keys, head_dim] per sample
  long long k_ld, k_sb1;
  const __nv_bfloat16* v;
  long long v_ld, v_sb1;
  void* out;
  long long out_ld, out_sb0, out_sb1;
  int rows;        // tokens * heads per sample
  int heads;
  int keys;
  int head_dim;    // multiple of 16, <= 256
  int slice_keys;  // keys per CTA (multiple of 16)
  int tiles;       // 16-row query tiles per sample
  float scale;
  int out_e4m3;
  float out_inv_scale;
};

__host__ __device__ constexpr int rows_q_stride(int hd) { return (hd * 2 + 127) / 128 * 128 + 64; }
__host__ __device__ constexpr int rows_v_stride(int hd) { return hd * 2 + 16; }
__host__ __device__ inline int fmha_rows_smem_bytes(int hd, int slice_keys) {
  return 16 * rows_q_stride(hd) + slice_keys * rows_q_stride(hd) + slice_keys * rows_v_stride(hd) +
         16 * (slice_keys + 8) * 2 + 16 * hd * 4 + (2 * kRowsWarps * 16 + 2 * 16) * 4 + 64;
}

namespace rows_detail {

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                   static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_row))));
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `local` (a shared-memory pointer of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t peer_address(const void* local, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(out)
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(local))), "r"(rank));
  return out;
}
__device__ __forceinline__ float ld_peer_f(uint32_t address) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(address));
  return v;
}
__device__ __forceinline__ float2 ld_peer_f2(uint32_t address) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(address));
  return v;
}

}  // namespace rows_detail

// The body has two callers. The stand-alone kernel runs it in clusters of 8 CTAs and merges the
// key slices through distributed shared memory (kCluster). The persistent denoise kernel
// (denoise_persistent.cuh) runs it as a stage on CTAs 0 .. 8 * tiles - 1 of a cooperative launch
// without clusters: the eight slices of a tile leave their partials in a global scratch, count
// themselves on the tile's flag, wait (bounded) for the other seven and merge from L2.
// `ctx`: cta (slice = cta % 8, tile = cta / 8), tid, sync(), wait() for the producer of Q and the
// cache rows; without clusters also scratch / flag / target of the tile exchange and the bounded
// wait `wait_flag(flag, target)`.
struct RowsLaunchCtx {
  int cta, tid;
  __device__ __forceinline__ void sync() const { __syncthreads(); }
  __device__ __forceinline__ void wait() const { pdl_wait(); }
  // unused by the cluster merge
  float* scratch = nullptr;
  unsigned* flags = nullptr;
  unsigned target = 0;
  __device__ __forceinline__ void wait_flag(const unsigned*, unsigned) const {}
};

// floats one slice leaves in the scratch: the partial output tile, then its row maxima and sums
__host__ __device__ constexpr int rows_partial_floats(int hd) { return 16 * hd + 32; }

template <bool kCluster, class Ctx>
__device__ __forceinline__ void fmha_rows_body(const FmhaRowsParams& p, uint8_t* rows_smem, const Ctx& ctx) {
  using namespace rows_detail;
  const int tid = ctx.tid;
  const int hd = p.head_dim;
  const int qs = rows_q_stride(hd), vs = rows_v_stride(hd);
  const int kc = p.slice_keys;
  uint8_t* q_tile = rows_smem;                    // [16][qs]   bf16, K-permutable layout
  uint8_t* k_tile = q_tile + 16 * qs;             // [kc][qs]
  uint8_t* v_tile = k_tile + kc * qs;             // [kc][vs]
  __nv_bfloat16* p_tile = reinterpret_cast<__nv_bfloat16*>(v_tile + kc * vs);  // [16][kc + 8]
  float* o_tile = reinterpret_cast<float*>(p_tile + 16 * (kc + 8));            // [16][hd]
  float* s_max = o_tile + 16 * hd;                // [warps][16]
  float* s_sum = s_max + kRowsWarps * 16;         // [warps][16]
  float* s_m = s_sum + kRowsWarps * 16;           // [16] slice maximum (unscaled scores)
  float* s_l = s_m + 16;                          // [16] slice sum relative to s_m

  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t rank = static_cast<uint32_t>(ctx.cta % kRowsCluster);  // = %cluster_ctarank in clusters of 8
  const int cluster_id = ctx.cta / kRowsCluster;
  const int tile = cluster_id % p.tiles;
  const int sample = cluster_id / p.tiles;
  const int row0 = tile * 16;
  const int key0 = static_cast<int>(rank) * kc;
  const int keys_here = max(0, min(kc, p.keys - key0));
  const int chunks = hd / 8;  // 16-byte chunks per row

  ctx.wait();

  // ---- everything this CTA reads, requested at once: Q tile + K slice, then V slice ----
  // (row, 16-byte chunk) items are walked with a fixed row step where the thread count is a
  // multiple of the chunks per row (every head dimension that is a power of two), so that no
  // item costs a division: these launches are bound by instructions per warp.
  {
    const int row_step = kRowsThreads / chunks;
    const bool regular = row_step * chunks == kRowsThreads;
    const int first_row = tid / chunks, my_chunk = tid - first_row * chunks;
    auto for_each_item = [&](int rows, auto&& body) {
      if (regular) {
        for (int r = first_row; r < rows; r += row_step) body(r, my_chunk);
      } else {
        for (int i = tid; i < rows * chunks; i += kRowsThreads) {
          const int r = i / chunks;
          body(r, i - r * chunks);
        }
      }
    };
    const __nv_bfloat16* qb = p.q + static_cast<long long>(sample) * p.q_sb1;
    for_each_item(16, [&](int r, int c) {
      const int row = row0 + r;
      uint8_t* dst = q_tile + r * qs + c * 16;
      if (row < p.rows) {
        cp_async16(dst, qb + static_cast<long long>(row / p.heads) * p.q_ld +
                            static_cast<long long>(row % p.heads) * p.q_sb0 + c * 8);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    });
    const __nv_bfloat16* kb = p.k + static_cast<long long>(sample) * p.k_sb1 + static_cast<long long>(key0) * p.k_ld;
    for_each_item(kc, [&](int r, int c) {
      uint8_t* dst = k_tile + r * qs + c * 16;
      if (r < keys_here) {
        cp_async16(dst, kb + static_cast<long long>(r) * p.k_ld + c * 8);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    });
    cp_async_commit();
    const __nv_bfloat16* vb = p.v + static_cast<long long>(sample) * p.v_sb1 + static_cast<long long>(key0) * p.v_ld;
    for_each_item(kc, [&](int r, int c) {
      uint8_t* dst = v_tile + r * vs + c * 16;
      if (r < keys_here) {
        cp_async16(dst, vb + static_cast<long long>(r) * p.v_ld + c * 8);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    });
    cp_async_commit();
  }
  cp_async_wait<1>();  // Q and K have landed (this thread's part)
  ctx.sync();

  // ---- S = Q K^T: warp w takes the 8-key tiles w, w + 8, ... of the slice ----
  const float scale_log2 = p.scale * 1.4426950408889634f;
  constexpr int kMaxTiles = 4;  // key tiles per warp: slices of up to 8 * 8 * 4 = 256 keys
  float s[kMaxTiles][4];
  const int key_tiles = kc / 8;
  const int steps = (hd * 2) / 64;  // 64-byte K steps of the head dimension
  float local_max[2] = {-3.0e38f, -3.0e38f};
#pragma unroll
  for (int i = 0; i < kMaxTiles; ++i) {
    const int kt = warp + i * kRowsWarps;
#pragma unroll
    for (int e = 0; e < 4; ++e) s[i][e] = 0.0f;
    if (kt < key_tiles) {
      const uint8_t* a_lo = q_tile + g * qs + t * 16;
      const uint8_t* a_hi = a_lo + 8 * qs;
      const uint8_t* b_row = k_tile + (kt * 8 + g) * qs + t * 16;
      for (int step = 0; step < steps; ++step) {
        const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + step * 64);
        const uint4 hi = *reinterpret_cast<const uint4*>(a_hi + step * 64);
        const uint4 b = *reinterpret_cast<const uint4*>(b_row + step * 64);
        mma_bf16(s[i], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
        mma_bf16(s[i], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
      }
      // columns 2t, 2t+1 of this tile; rows g (e = 0, 1) and g + 8 (e = 2, 3)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kt * 8 + 2 * t + (e & 1);
        if (key >= keys_here) s[i][e] = -3.0e38f;
        local_max[e >> 1] = fmaxf(local_max[e >> 1], s[i][e]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    local_max[h] = fmaxf(local_max[h], __shfl_xor_sync(0xffffffffu, local_max[h], 1));
    local_max[h] = fmaxf(local_max[h], __shfl_xor_sync(0xffffffffu, local_max[h], 2));
  }
  if (t == 0) {
    s_max[warp * 16 + g] = local_max[0];
    s_max[warp * 16 + g + 8] = local_max[1];
  }
  ctx.sync();
  float row_max[2] = {-3.0e38f, -3.0e38f};
#pragma unroll
  for (int w = 0; w < kRowsWarps; ++w) {
    row_max[0] = fmaxf(row_max[0], s_max[w * 16 + g]);
    row_max[1] = fmaxf(row_max[1], s_max[w * 16 + g + 8]);
  }
  // ---- probabilities (relative to the slice maximum) -> shared memory as bf16, row sums ----
  float local_sum[2] = {0.0f, 0.0f};
  const int p_stride = kc + 8;
#pragma unroll
  for (int i = 0; i < kMaxTiles; ++i) {
    const int kt = warp + i * kRowsWarps;
    if (kt < key_tiles) {
      float e[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int key = kt * 8 + 2 * t + (q & 1);
        const float m = row_max[q >> 1];
        e[q] = key < keys_here ? exp2f((s[i][q] - m) * scale_log2) : 0.0f;
        local_sum[q >> 1] += e[q];
      }
      *reinterpret_cast<__nv_bfloat162*>(p_tile + g * p_stride + kt * 8 + 2 * t) = __floats2bfloat162_rn(e[0], e[1]);
      *reinterpret_cast<__nv_bfloat162*>(p_tile + (g + 8) * p_stride + kt * 8 + 2 * t) =
          __floats2bfloat162_rn(e[2], e[3]);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    local_sum[h] += __shfl_xor_sync(0xffffffffu, local_sum[h], 1);
    local_sum[h] += __shfl_xor_sync(0xffffffffu, local_sum[h], 2);
  }
  if (t == 0) {
    s_sum[warp * 16 + g] = local_sum[0];
    s_sum[warp * 16 + g + 8] = local_sum[1];
  }
  cp_async_wait<0>();  // V has landed (this thread's part)
  ctx.sync();
  if (tid < 16) {
    float total = 0.0f, m = -3.0e38f;
    for (int w = 0; w < kRowsWarps; ++w) {
      total += s_sum[w * 16 + tid];
      m = fmaxf(m, s_max[w * 16 + tid]);
    }
    s_m[tid] = m;
    s_l[tid] = total;
  }

  // ---- O = P V: warp w takes the 16-dim pairs of tiles w, w + 8, ... ----
  {
    const int dim_pairs = hd / 16;  // two 8-dim tiles per ldmatrix.x4
    const int ksteps = kc / 16;
    for (int dp = warp; dp < dim_pairs; dp += kRowsWarps) {
      float acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
      for (int ks = 0; ks < ksteps; ++ks) {
        const __nv_bfloat16* pa = p_tile + g * p_stride + ks * 16 + 2 * t;
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(pa);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(pa + 8 * p_stride);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(pa + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(pa + 8 * p_stride + 8);
        // lanes 0-7: keys ks*16 + lane, dims dp*16; 8-15: keys + 8; 16-23 / 24-31: dims + 8
        const int key = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int dim = dp * 16 + (lane >> 4) * 8;
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_tile + key * vs + dim * 2);
        mma_bf16(acc[0], a0, a1, a2, a3, b[0], b[1]);
        mma_bf16(acc[1], a0, a1, a2, a3, b[2], b[3]);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int d = dp * 16 + j * 8 + 2 * t;
        *reinterpret_cast<float2*>(o_tile + g * hd + d) = make_float2(acc[j][0], acc[j][1]);
        *reinterpret_cast<float2*>(o_tile + (g + 8) * hd + d) = make_float2(acc[j][2], acc[j][3]);
      }
    }
  }

  // ---- merge the eight slices: this CTA finishes head dims [rank * hd / 8, (rank + 1) * hd / 8) ----
  const float* tile_scratch = nullptr;
  if constexpr (kCluster) {
    cluster_sync();
  } else {
    // partials to the scratch, one arrival per CTA on the tile's flag, bounded wait for all eight
    ctx.sync();
    float* mine = ctx.scratch + (static_cast<long long>(cluster_id) * kRowsCluster + rank) * rows_partial_floats(hd);
    for (int i = tid; i < 16 * hd / 4; i += kRowsThreads) {
      __stcg(reinterpret_cast<float4*>(mine) + i, reinterpret_cast<const float4*>(o_tile)[i]);
    }
    if (tid < 16) {
      __stcg(mine + 16 * hd + tid, s_m[tid]);
      __stcg(mine + 16 * hd + 16 + tid, s_l[tid]);
    }
    __threadfence();
    ctx.sync();
    if (tid == 0) {
      atomicAdd(ctx.flags + cluster_id, 1u);
      ctx.wait_flag(ctx.flags + cluster_id, ctx.target);
    }
    ctx.sync();
    tile_scratch = ctx.scratch + static_cast<long long>(cluster_id) * kRowsCluster * rows_partial_floats(hd);
  }
  {
    const int dims_here = hd / kRowsCluster;     // multiple of 2
    const int pairs = dims_here / 2;
    for (int item = tid; item < 16 * pairs; item += kRowsThreads) {
      const int r = item / pairs;
      const int d = static_cast<int>(rank) * dims_here + (item - r * pairs) * 2;
      const int row = row0 + r;
      if (row >= p.rows) continue;
      float m_s[kRowsCluster];
      float m_all = -3.0e38f;
#pragma unroll
      for (int c = 0; c < kRowsCluster; ++c) {
        if constexpr (kCluster) {
          m_s[c] = ld_peer_f(peer_address(s_m + r, c));
        } else {
          m_s[c] = __ldcg(tile_scratch + c * rows_partial_floats(hd) + 16 * hd + r);
        }
        m_all = fmaxf(m_all, m_s[c]);
      }
      float total = 0.0f, o0 = 0.0f, o1 = 0.0f;
#pragma unroll
      for (int c = 0; c < kRowsCluster; ++c) {
        float l;
        float2 o;
        if constexpr (kCluster) {
          l = ld_peer_f(peer_address(s_l + r, c));
          o = ld_peer_f2(peer_address(o_tile + r * hd + d, c));
        } else {
          const float* part = tile_scratch + c * rows_partial_floats(hd);
          l = __ldcg(part + 16 * hd + 16 + r);
          o = __ldcg(reinterpret_cast<const float2*>(part + r * hd + d));
        }
        const float w = exp2f((m_s[c] - m_all) * scale_log2);
        total = fmaf(w, l, total);
        o0 = fmaf(w, o.x, o0);
        o1 = fmaf(w, o.y, o1);
      }
      const float inv = total > 0.0f ? 1.0f / total : 0.0f;
      const long long at = static_cast<long long>(sample) * p.out_sb1 +
                           static_cast<long long>(row / p.heads) * p.out_ld +
                           static_cast<long long>(row % p.heads) * p.out_sb0 + d;
      const __nv_bfloat162 pair = __floats2bfloat162_rn(o0 * inv, o1 * inv);
      if (p.out_e4m3) {
        // the reference rounds the attention output to 16 bits before quantising it
        const float2 f = __bfloat1622float2(pair);
        const float c0 = fminf(448.0f, fmaxf(-448.0f, f.x * p.out_inv_scale));
        const float c1 = fminf(448.0f, fmaxf(-448.0f, f.y * p.out_inv_scale));
        uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + at;
        dst[0] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(c0, __NV_SATFINITE, __NV_E4M3));
        dst[1] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(c1, __NV_SATFINITE, __NV_E4M3));
      } else {
        *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.out) + at) = pair;
      }
    }
  }
  // nobody leaves while a peer may still read its partials
  if constexpr (kCluster) cluster_sync();
}

static __global__ void __launch_bounds__(kRowsThreads, 1) fmha_rows_cluster_kernel(const FmhaRowsParams p) {
  pdl_launch_dependents();
  extern __shared__ __align__(128) uint8_t rows_smem_base[];
  const RowsLaunchCtx ctx{static_cast<int>(blockIdx.x), static_cast<int>(threadIdx.x)};
  fmha_rows_body<true>(p, rows_smem_base, ctx);
}

}  // namespace pi05
