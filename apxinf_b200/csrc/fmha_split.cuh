// Key-split attention for launches with only a few query tiles (the B=1 action expert: one to
// four 128-row tiles over 532-572 keys). One CTA per (query tile, 64-key slice): everything it
// needs (Q tile, K slice, V slice) is requested from TMA at once, S = Q K^T is a single
// 128 x 64 accumulator, the slice's probabilities go through shared memory into O = P V, and
// the CTA leaves an unnormalised partial output with its row maxima and row sums in scratch.
// `fmha_combine_kernel` then merges the slices of a tile with the usual log-sum-exp weights.
// Two dependent launches of a few microseconds replace the QK^T GEMM -> softmax -> PV GEMM
// chain, and nine times as many SMs pull the K/V cache as the unsplit kernel would use.
// Same operands, tile packing (multi-query heads share a tile) and output conventions as
// fmha_online_kernel.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "fmha.h"
#include "fmha_common.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace pi05 {

constexpr int kSplitKeys = 64;                       // keys per CTA
constexpr int kSplitThreads = 64 + 128;              // TMA warp, MMA warp, 4 softmax warps
constexpr int kSplitQBytes = 4 * 16384;              // Q: up to 4 head-dim chunks of [128 x 128 B]
constexpr int kSplitKBytes = 4 * 8192;               // K slice: 4 chunks of [64 keys x 128 B]
constexpr int kSplitVBytes = 4 * 8192;               // V slice: 4 chunks of [64 keys x 64 dims]
constexpr int kSplitPBytes = 16384;                  // P: [128 rows x 64 keys] bf16
constexpr int kSplitSmemBytes = kSplitQBytes + kSplitKBytes + kSplitVBytes + kSplitPBytes + 1024 + 256;

// Scratch per work item: [128 rows][head_dim] fp32 partial output, then [128][2] (max, sum).
__host__ __device__ inline size_t fmha_split_item_floats(int head_dim) {
  return static_cast<size_t>(128) * (head_dim + 2);
}

__global__ void __launch_bounds__(kSplitThreads, 1)
fmha_split_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const FmhaParams p, float* scratch) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* k_smem = q_smem + kSplitQBytes;
  uint8_t* v_smem = k_smem + kSplitKBytes;
  uint8_t* p_smem = v_smem + kSplitVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + kSplitPBytes);
  uint64_t* qk_full = bars;      // Q tile and K slice landed
  uint64_t* v_full = bars + 1;   // V slice landed
  uint64_t* s_full = bars + 2;   // scores in TMEM
  uint64_t* p_full = bars + 3;   // probabilities in shared memory (128 arrivals)
  uint64_t* o_full = bars + 4;   // partial output in TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int pack = p.pack;
  const int tile_tokens = 128 / pack;
  const int q_tiles = (p.q_rows + tile_tokens - 1) / tile_tokens;
  const int heads_outer = pack > 1 ? 1 : p.nb0;
  const int splits = (p.keys + kSplitKeys - 1) / kSplitKeys;
  const int item = blockIdx.x;
  const int split = item % splits;
  const int tile = (item / splits) % q_tiles;
  const int batch = item / (splits * q_tiles);
  const int b0 = batch % heads_outer;
  const int b1 = batch / heads_outer;
  const int hd = p.head_dim;
  const int hd_chunks = (hd + 63) >> 6;
  const int n_pv = (hd + 15) & ~15;
  const int key0 = split * kSplitKeys;
  const int keys_here = min(kSplitKeys, p.keys - key0);

  if (threadIdx.x == 0) {
    ptx::mbar_init(qk_full, 1);
    ptx::mbar_init(v_full, 1);
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(p_full, 128);
    ptx::mbar_init(o_full, 1);
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_s = *tmem_slot;    // columns [0, 64): scores
  const uint32_t tmem_o = tmem_s + 256;  // columns [256, 256 + n_pv): partial output
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_q);
      ptx::prefetch_tensormap(&tmap_k);
      ptx::prefetch_tensormap(&tmap_v);
      ptx::mbar_arrive_expect_tx(qk_full, hd_chunks * (16384 + 8192));
      for (int c = 0; c < hd_chunks; ++c) {
        if (pack > 1) {
          ptx::tma_load_4d(q_smem + c * 16384, &tmap_q, qk_full, c * 64, 0, tile * tile_tokens, b1);
        } else {
          ptx::tma_load_4d(q_smem + c * 16384, &tmap_q, qk_full, c * 64, tile * 128, b0, b1);
        }
        ptx::tma_load_4d(k_smem + c * 8192, &tmap_k, qk_full, c * 64, key0, b0, b1);
      }
      ptx::mbar_arrive_expect_tx(v_full, hd_chunks * 8192);
      for (int c = 0; c < hd_chunks; ++c) {
        ptx::tma_load_4d(v_smem + c * 8192, &tmap_v, v_full, c * 64, key0, b0, b1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = ptx::make_idesc(1, 1, 1, 0, 0, 128, kSplitKeys);
      const uint32_t idesc_o = ptx::make_idesc(1, 1, 1, 0, 1, 128, static_cast<uint32_t>(n_pv));
      const uint32_t q_addr = ptx::smem_u32(q_smem);
      const uint32_t k_addr = ptx::smem_u32(k_smem);
      const uint32_t v_addr = ptx::smem_u32(v_smem);
      const uint32_t p_addr = ptx::smem_u32(p_smem);
      bool ok = ptx::mbar_wait(qk_full, 0);
      ptx::tc_fence_after();
      if (ok) {
        for (int c = 0; c < hd_chunks; ++c) {
          const int ksteps = min(4, (hd - c * 64 + 15) >> 4);
          for (int ks = 0; ks < ksteps; ++ks) {
            ptx::umma<ptx::MmaKind::kF16>(tmem_s, ptx::make_smem_desc(q_addr + c * 16384 + ks * 32, 16, 1024),
                                          ptx::make_smem_desc(k_addr + c * 8192 + ks * 32, 16, 1024), idesc_s,
                                          (c | ks) != 0 ? 1u : 0u);
          }
        }
      }
      // signalled even after a timeout so that nobody waits on a dead pipeline
      ptx::umma_commit(s_full);
      if (ok) ok = ptx::mbar_wait(p_full, 0);
      if (ok) ok = ptx::mbar_wait(v_full, 0);
      ptx::tc_fence_after();
      if (ok) {
        const int ksteps = (keys_here + 15) >> 4;  // rows of P beyond the slice are zero
        for (int ks = 0; ks < ksteps; ++ks) {
          ptx::umma<ptx::MmaKind::kF16>(tmem_o, ptx::make_smem_desc(p_addr + ks * 32, 16, 1024),
                                        ptx::make_smem_desc(v_addr + ks * 2048, 8192, 1024), idesc_o,
                                        ks != 0 ? 1u : 0u);
        }
      }
      ptx::umma_commit(o_full);
      if (!ok) atomicCAS(p.status, 0, kFmhaTimeout);
    }
  } else {
    // ---- softmax + partial epilogue: thread = query row ----
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int row = pack > 1 ? tile * tile_tokens + row_in_tile / pack : tile * 128 + row_in_tile;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    bool ok = ptx::mbar_wait(s_full, 0);
    ptx::tc_fence_after();
    uint32_t raw[4][16];
#pragma unroll
    for (int u = 0; u < 4; ++u) ptx::tmem_ld_16(tmem_s + lane_base + u * 16, raw[u]);
    ptx::tmem_ld_wait();
    float raw_max = -3.0e38f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        if (u * 16 + t < keys_here) raw_max = fmaxf(raw_max, __uint_as_float(raw[u][t]));
      }
    }
    const float max_log2 = raw_max * scale_log2;
    float row_sum = 0.0f;
    uint8_t* tile_base = p_smem + row_in_tile * 128;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t packed[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const int c = u * 16 + 2 * t;
        float e0 = exp2f(fmaf(__uint_as_float(raw[u][2 * t]), scale_log2, -max_log2));
        float e1 = exp2f(fmaf(__uint_as_float(raw[u][2 * t + 1]), scale_log2, -max_log2));
        e0 = c < keys_here ? e0 : 0.0f;
        e1 = c + 1 < keys_here ? e1 : 0.0f;
        row_sum += e0 + e1;
        const __nv_bfloat162 pair = __floats2bfloat162_rn(e0, e1);
        packed[t] = *reinterpret_cast<const uint32_t*>(&pair);
      }
      *reinterpret_cast<uint4*>(tile_base + (((2 * u) ^ (row_in_tile & 7)) << 4)) =
          make_uint4(packed[0], packed[1], packed[2], packed[3]);
      *reinterpret_cast<uint4*>(tile_base + (((2 * u + 1) ^ (row_in_tile & 7)) << 4)) =
          make_uint4(packed[4], packed[5], packed[6], packed[7]);
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before();
    ptx::mbar_arrive(p_full);

    float* part = scratch + static_cast<size_t>(item) * fmha_split_item_floats(hd);
    float* part_row = part + static_cast<size_t>(row_in_tile) * hd;
    float* stats = part + static_cast<size_t>(128) * hd;
    const bool row_ok = row < p.q_rows;
    if (row_ok) {
      stats[2 * row_in_tile] = raw_max;
      stats[2 * row_in_tile + 1] = row_sum;
    }
    if (ok) ok = ptx::mbar_wait(o_full, 0);
    ptx::tc_fence_after();
    if (!ok && lane == 0) atomicCAS(p.status, 0, kFmhaTimeout);
#pragma unroll 1
    for (int cc = 0; cc < n_pv / 16; cc += 2) {
      uint32_t o[2][16];
      ptx::tmem_ld_16(tmem_o + lane_base + cc * 16, o[0]);
      ptx::tmem_ld_16(tmem_o + lane_base + min(cc + 1, n_pv / 16 - 1) * 16, o[1]);
      ptx::tmem_ld_wait();
      if (!row_ok) continue;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int d0 = (cc + u) * 16;
        if (cc + u >= n_pv / 16) continue;
        const int valid = min(16, hd - d0);  // head_dim is a multiple of 8: 16 or 8
        float4* dst = reinterpret_cast<float4*>(part_row + d0);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          if (4 * q4 < valid) {
            dst[q4] = make_float4(__uint_as_float(o[u][4 * q4]), __uint_as_float(o[u][4 * q4 + 1]),
                                  __uint_as_float(o[u][4 * q4 + 2]), __uint_as_float(o[u][4 * q4 + 3]));
          }
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_s, 512);
  }
}

// out = sum_s w_s O_s / sum_s w_s l_s with w_s = 2^((m_s - max_s m_s) * scale * log2 e), over the
// slices' partials in scratch. One CTA per 8 rows of a query tile, one thread per (row, 8
// columns): the loads of all slices are in flight together, so the launch is about three
// L2 round trips long.
constexpr int kCombineRows = 8;

__global__ void __launch_bounds__(256)
fmha_combine_kernel(const FmhaParams p, const float* __restrict__ scratch) {
  pdl_launch_dependents();
  __shared__ float weight[kCombineRows][16];  // normalised slice weights of this CTA's rows
  const int pack = p.pack;
  const int tile_tokens = 128 / pack;
  const int q_tiles = (p.q_rows + tile_tokens - 1) / tile_tokens;
  const int heads_outer = pack > 1 ? 1 : p.nb0;
  const int splits = (p.keys + kSplitKeys - 1) / kSplitKeys;
  const int row_group = blockIdx.x % (128 / kCombineRows);
  const int tile_item = blockIdx.x / (128 / kCombineRows);
  const int tile = tile_item % q_tiles;
  const int batch = tile_item / q_tiles;
  const int b0 = batch % heads_outer;
  const int b1 = batch / heads_outer;
  const int hd = p.head_dim;
  const int groups = hd / 8;
  const size_t item_floats = fmha_split_item_floats(hd);
  const float* base = scratch + static_cast<size_t>(tile_item) * splits * item_floats;
  const float scale_log2 = p.scale * 1.4426950408889634f;
  auto row_of = [&](int r) { return pack > 1 ? tile * tile_tokens + r / pack : tile * 128 + r; };
  pdl_wait();
  if (row_of(row_group * kCombineRows) >= p.q_rows) return;  // rows only grow within a tile

  // one thread per (row, slice): the statistics of a row in one round trip, merged by shuffles
  {
    const int rl = threadIdx.x >> 4, s = threadIdx.x & 15;
    float m = -3.0e38f, l = 0.0f;
    if (rl < kCombineRows && s < splits) {
      const float* st = base + s * item_floats + 128 * hd + 2 * (row_group * kCombineRows + rl);
      m = __ldcg(st);
      l = __ldcg(st + 1);
    }
    float mx = m;
#pragma unroll
    for (int d = 8; d >= 1; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d, 16));
    const float w = s < splits ? exp2f((m - mx) * scale_log2) : 0.0f;
    float total = w * l;
#pragma unroll
    for (int d = 8; d >= 1; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d, 16);
    if (rl < kCombineRows) weight[rl][s] = total > 0.0f ? w / total : 0.0f;
  }
  __syncthreads();
  const int rl = threadIdx.x / groups;
  const int g = threadIdx.x % groups;
  const int r = row_group * kCombineRows + rl;
  const int row = row_of(r);
  if (rl >= kCombineRows || row >= p.q_rows) return;
  float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int s0 = 0; s0 < 16; s0 += 4) {
    if (s0 >= splits) break;
    float4 a[4], b[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {  // four slices' loads issued together
      const int s = min(s0 + u, splits - 1);
      const float4* src = reinterpret_cast<const float4*>(base + s * item_floats + r * hd + 8 * g);
      a[u] = __ldcg(src);
      b[u] = __ldcg(src + 1);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float w = s0 + u < splits ? weight[rl][s0 + u] : 0.0f;
      acc[0] = fmaf(w, a[u].x, acc[0]); acc[1] = fmaf(w, a[u].y, acc[1]);
      acc[2] = fmaf(w, a[u].z, acc[2]); acc[3] = fmaf(w, a[u].w, acc[3]);
      acc[4] = fmaf(w, b[u].x, acc[4]); acc[5] = fmaf(w, b[u].y, acc[5]);
      acc[6] = fmaf(w, b[u].z, acc[6]); acc[7] = fmaf(w, b[u].w, acc[7]);
    }
  }
  const int head = pack > 1 ? r % pack : b0;
  const long long at = (long long)head * p.out_sb0 + (long long)b1 * p.out_sb1 +
                       (long long)row * p.out_ld + 8 * g;
  uint32_t w16[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(acc[2 * t], acc[2 * t + 1]);
    w16[t] = *reinterpret_cast<const uint32_t*>(&pair);
  }
  if (p.out_e4m3) {
    // the reference rounds the attention output to 16 bits before quantising it
    uint32_t w8[2] = {0, 0};
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const uint32_t bits = (w16[t >> 1] >> (16 * (t & 1))) << 16;
      const float clamped = fminf(448.0f, fmaxf(-448.0f, __uint_as_float(bits) * p.out_inv_scale));
      const uint32_t byte = static_cast<uint8_t>(__nv_cvt_float_to_fp8(clamped, __NV_SATFINITE, __NV_E4M3));
      w8[t >> 2] |= byte << (8 * (t & 3));
    }
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + at;
    if ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
      *reinterpret_cast<uint2*>(dst) = make_uint2(w8[0], w8[1]);
    } else {
#pragma unroll
      for (int t = 0; t < 8; ++t) dst[t] = static_cast<uint8_t>(w8[t >> 2] >> (8 * (t & 3)));
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + at;
    if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(w16[0], w16[1], w16[2], w16[3]);
    } else {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        dst[t] = __ushort_as_bfloat16(static_cast<unsigned short>(w16[t >> 1] >> (16 * (t & 1))));
      }
    }
  }
}

}  // namespace pi05
