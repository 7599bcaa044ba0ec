// Fused attention for more than one 256-key block (prefix and batched action-expert MQA: 522 to
// 572 keys, head_dim 256): one pass over the keys with a running row maximum.
//
// Same tiles, operands, packing and warp roles as fmha_umma_kernel (which keeps the single-block
// case, where the scores stay in TMEM and nothing has to be rescaled). Per 256-key block j:
//   MMA warp      S_j = Q K_j^T into TMEM; S_{j+1} is issued as soon as the softmax warps have
//                 pulled S_j into registers, i.e. it runs under their exponentials
//   softmax warps block maximum (exchanged between the four column groups through shared
//                 memory), running maximum m, alpha = 2^((m_old - m) c); once PV_{j-1} is done:
//                 O *= alpha in TMEM (tcgen05.ld / st of this group's 64 output columns,
//                 skipped when no row of the warp moved its maximum), P_j = 2^(s c - m c) as
//                 bf16 into shared memory, row sums l = l alpha + sum P_j
//   MMA warp      O += P_j V_j with V MN-major from the [keys, head_dim] cache
// K and V are fetched once (the two-pass form fetched K twice and computed S twice); with a
// shared-memory ring of only two 32 KB stages beside the 64 KB query tile and the 64 KB
// probability tile, bytes through the ring are what bounds this kernel.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "fmha.h"
#include "fmha_umma.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace pi05 {

__global__ void __launch_bounds__(kFmhaThreads, 1)
fmha_online_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const FmhaParams p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* p_smem = q_smem + kFmhaQBytes + 2 * kFmhaStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + kFmhaPBytes);
  uint64_t* q_full = bars;          // Q tile landed
  uint64_t* ring_full = bars + 1;   // [kFmhaMaxStages]
  uint64_t* ring_empty = bars + 4;  // [kFmhaMaxStages]
  uint64_t* s_full = bars + 7;      // S block ready in TMEM
  uint64_t* s_free = bars + 8;      // softmax warps hold S in registers
  uint64_t* p_full = bars + 9;      // P block written and O rescaled
  uint64_t* p_free = bars + 10;     // PV MMAs done: P may be overwritten, O is up to date
  uint64_t* o_full = bars + 11;     // output accumulator complete
  uint64_t* q_free = bars + 12;     // every QK^T MMA of the tile has read Q
  uint64_t* o_free = bars + 13;     // epilogue has read the output accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  float* x_max = reinterpret_cast<float*>(p_smem + kFmhaPBytes + 256);  // [2][4][128] by block parity, then [4][128] row sums

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int pack = p.pack;
  const int tile_tokens = 128 / pack;
  const int q_tiles = (p.q_rows + tile_tokens - 1) / tile_tokens;
  const int heads_outer = pack > 1 ? 1 : p.nb0;
  const int total_items = q_tiles * heads_outer * p.nb1;
  auto decode = [&](int item, int* tile, int* b0, int* b1) {
    *tile = item % q_tiles;
    const int batch = item / q_tiles;
    *b0 = batch % heads_outer;
    *b1 = batch / heads_outer;
  };
  const int hd = p.head_dim;
  const int hd_chunks = (hd + 63) >> 6;
  const int n_blocks = (p.keys + kFmhaKeyBlock - 1) / kFmhaKeyBlock;
  const int stages = hd_chunks <= 2 ? 3 : 2;
  auto stage_ptr = [&](int s) -> uint8_t* {
    return s < 2 ? q_smem + kFmhaQBytes + s * kFmhaStageBytes : q_smem + 2 * 16384;
  };
  const int n_pv = (hd + 15) & ~15;  // UMMA N of the PV product
  auto keys_in_block = [&](int j) { return min(kFmhaKeyBlock, p.keys - j * kFmhaKeyBlock); };

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < kFmhaMaxStages; ++s) {
      ptx::mbar_init(&ring_full[s], 1);
      ptx::mbar_init(&ring_empty[s], 1);
    }
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(s_free, kFmhaSoftmaxThreads);
    ptx::mbar_init(p_full, kFmhaSoftmaxThreads);
    ptx::mbar_init(p_free, 1);
    ptx::mbar_init(o_full, 1);
    ptx::mbar_init(q_free, 1);
    ptx::mbar_init(o_free, kFmhaSoftmaxThreads);
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
  const uint32_t tmem_s = *tmem_slot;    // columns [0, 256): S block
  const uint32_t tmem_o = tmem_s + 256;  // columns [256, 512): output accumulator
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer: Q, K_0, then K_{j+1} before V_j ----------------
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_q);
      ptx::prefetch_tensormap(&tmap_k);
      ptx::prefetch_tensormap(&tmap_v);
      bool ok = true;
      int it = 0;
      int items_done = 0;
      auto acquire = [&]() -> uint8_t* {
        const int s = it % stages;
        const int round = it / stages;
        if (round > 0) ok = ok && ptx::mbar_wait(&ring_empty[s], (round - 1) & 1);
        return stage_ptr(s);
      };
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++items_done) {
        int tile, b0, b1;
        decode(item, &tile, &b0, &b1);
        if (items_done > 0) ok = ptx::mbar_wait(q_free, (items_done - 1) & 1);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(q_full, hd_chunks * 16384);
        for (int c = 0; c < hd_chunks; ++c) {
          if (pack > 1) {
            ptx::tma_load_4d(q_smem + c * 16384, &tmap_q, q_full, c * 64, 0, tile * tile_tokens, b1);
          } else {
            ptx::tma_load_4d(q_smem + c * 16384, &tmap_q, q_full, c * 64, tile * 128, b0, b1);
          }
        }
        auto load_k = [&](int j) {
          for (int c = 0; c < hd_chunks && ok; ++c, ++it) {  // K chunk: [256 keys x 64 dims]
            uint8_t* dst = acquire();
            if (!ok) break;
            ptx::mbar_arrive_expect_tx(&ring_full[it % stages], kFmhaStageBytes);
            ptx::tma_load_4d(dst, &tmap_k, &ring_full[it % stages], c * 64, j * kFmhaKeyBlock, b0, b1);
          }
        };
        load_k(0);
        for (int j = 0; j < n_blocks && ok; ++j) {
          if (j + 1 < n_blocks) load_k(j + 1);
          const int subs = (keys_in_block(j) + 63) >> 6;
          for (int v = 0; v < subs && ok; ++v, ++it) {  // V sub-block: [64 keys x head_dim]
            uint8_t* dst = acquire();
            if (!ok) break;
            ptx::mbar_arrive_expect_tx(&ring_full[it % stages], hd_chunks * 8192);
            for (int c = 0; c < hd_chunks; ++c) {
              ptx::tma_load_4d(dst + c * 8192, &tmap_v, &ring_full[it % stages], c * 64,
                               j * kFmhaKeyBlock + v * 64, b0, b1);
            }
          }
        }
      }
      if (!ok) atomicCAS(p.status, 0, kFmhaTimeout);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = true;
      const uint32_t idesc_s = ptx::make_idesc(1, 1, 1, 0, 0, 128, kFmhaKeyBlock);
      const uint32_t idesc_o = ptx::make_idesc(1, 1, 1, 0, 1, 128, static_cast<uint32_t>(n_pv));
      const uint32_t q_addr = ptx::smem_u32(q_smem);
      const uint32_t p_addr = ptx::smem_u32(p_smem);
      int it = 0;
      int s_blocks = 0;   // S blocks issued so far
      int pv_blocks = 0;  // PV blocks issued so far
      int items_done = 0;
      auto issue_s = [&]() {
        // S may be overwritten once the softmax warps hold the previous block in registers
        if (ok && s_blocks > 0) ok = ptx::mbar_wait(s_free, (s_blocks - 1) & 1);
        ptx::tc_fence_after();
        for (int c = 0; c < hd_chunks && ok; ++c, ++it) {
          const int s = it % stages;
          ok = ptx::mbar_wait(&ring_full[s], (it / stages) & 1);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t k_addr = ptx::smem_u32(stage_ptr(s));
          const int ksteps = min(4, (hd - c * 64 + 15) >> 4);
          for (int ks = 0; ks < ksteps; ++ks) {
            ptx::umma<ptx::MmaKind::kF16>(tmem_s, ptx::make_smem_desc(q_addr + c * 16384 + ks * 32, 16, 1024),
                                          ptx::make_smem_desc(k_addr + ks * 32, 16, 1024), idesc_s,
                                          (c | ks) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&ring_empty[s]);
        }
        // signalled even after a timeout so that nobody waits on a dead pipeline
        ptx::umma_commit(s_full);
        ++s_blocks;
      };
      for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++items_done) {
        if (ok) ok = ptx::mbar_wait(q_full, items_done & 1);
        issue_s();
        if (n_blocks == 1) ptx::umma_commit(q_free);
        for (int j = 0; j < n_blocks; ++j) {
          if (j + 1 < n_blocks) {
            issue_s();
            if (j + 2 == n_blocks) ptx::umma_commit(q_free);  // the last S product has read Q
          }
          if (ok) ok = ptx::mbar_wait(p_full, pv_blocks & 1);
          // the previous tile's epilogue must have drained the output accumulator
          if (ok && j == 0 && items_done > 0) ok = ptx::mbar_wait(o_free, (items_done - 1) & 1);
          ptx::tc_fence_after();
          const int subs = (keys_in_block(j) + 63) >> 6;
          for (int v = 0; v < subs && ok; ++v, ++it) {
            const int s = it % stages;
            ok = ptx::mbar_wait(&ring_full[s], (it / stages) & 1);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t v_addr = ptx::smem_u32(stage_ptr(s));
            for (int ks = 0; ks < 4; ++ks) {
              ptx::umma<ptx::MmaKind::kF16>(tmem_o, ptx::make_smem_desc(p_addr + v * 16384 + ks * 32, 16, 1024),
                                            ptx::make_smem_desc(v_addr + ks * 2048, 8192, 1024), idesc_o,
                                            (j | v | ks) != 0 ? 1u : 0u);
            }
            ptx::umma_commit(&ring_empty[s]);
          }
          ptx::umma_commit(p_free);
          ++pv_blocks;
        }
        ptx::umma_commit(o_full);
      }
      if (!ok) atomicCAS(p.status, 0, kFmhaTimeout);
    }
  } else {
    // ---------------- softmax + epilogue (warps 2..17) ----------------
    const int quarter = warp & 3;        // TMEM lane quarter this warp may read
    const int group = (warp - 2) >> 2;   // its 64-key column group and 64 output columns
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    bool ok = true;
    int s_blocks = 0, p_blocks = 0;
    int items_done = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++items_done) {
      int tile, b0, b1;
      decode(item, &tile, &b0, &b1);
      // query row (token) and head this thread owns
      const int row = pack > 1 ? tile * tile_tokens + row_in_tile / pack : tile * 128 + row_in_tile;
      const int head = pack > 1 ? row_in_tile % pack : b0;
      float run_max = -3.0e38f;  // running maximum of the unscaled scores of the whole row
      float row_sum = 0.0f;      // this column group's share of the row sum, relative to run_max
      for (int j = 0; j < n_blocks; ++j) {
        if (ok) ok = ptx::mbar_wait(s_full, s_blocks & 1);
        ptx::tc_fence_after();
        const int valid = keys_in_block(j) - group * 64;  // valid keys among this warp's 64 columns
        // 64 columns per TMEM round trip: four loads in flight, one wait (always issued: a
        // conditional TMEM load would push the array to local memory)
        uint32_t raw[4][16];
#pragma unroll
        for (int u = 0; u < 4; ++u) ptx::tmem_ld_16(tmem_s + lane_base + group * 64 + u * 16, raw[u]);
        ptx::tmem_ld_wait();
        ptx::tc_fence_before();
        ptx::mbar_arrive(s_free);  // S is in registers: the next S product may start
        ++s_blocks;
        float local = -3.0e38f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            if (u * 16 + t < valid) local = fmaxf(local, __uint_as_float(raw[u][t]));
          }
        }
        float* xm = x_max + (j & 1) * 512;
        xm[group * 128 + row_in_tile] = local;
        asm volatile("bar.sync 1, %0;" ::"n"(kFmhaSoftmaxThreads) : "memory");
        const float block_max = fmaxf(fmaxf(xm[row_in_tile], xm[128 + row_in_tile]),
                                      fmaxf(xm[256 + row_in_tile], xm[384 + row_in_tile]));
        const float new_max = fmaxf(run_max, block_max);
        // block 0 always has a valid key, so run_max is finite from block 1 on
        const float alpha = j == 0 ? 0.0f : exp2f((run_max - new_max) * scale_log2);
        run_max = new_max;
        const float max_log2 = new_max * scale_log2;
        // PV_{j-1} (of this tile or the last one of the previous tile) must be done before P is
        // overwritten and O is rescaled
        if (p_blocks > 0 && ok) ok = ptx::mbar_wait(p_free, (p_blocks - 1) & 1);
        ptx::tc_fence_after();
        if (j > 0 && !__all_sync(0xffffffffu, alpha == 1.0f)) {
#pragma unroll 1
          for (int cc = 4 * group; cc < min(4 * group + 4, n_pv / 16); cc += 2) {
            uint32_t o[2][16];
            const int c1 = min(cc + 1, n_pv / 16 - 1);
            ptx::tmem_ld_16(tmem_o + lane_base + cc * 16, o[0]);
            ptx::tmem_ld_16(tmem_o + lane_base + c1 * 16, o[1]);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              o[0][t] = __float_as_uint(__uint_as_float(o[0][t]) * alpha);
              o[1][t] = __float_as_uint(__uint_as_float(o[1][t]) * alpha);
            }
            ptx::tmem_st_16(tmem_o + lane_base + cc * 16, o[0]);
            if (c1 != cc) ptx::tmem_st_16(tmem_o + lane_base + c1 * 16, o[1]);
          }
          ptx::tmem_st_wait();
        }
        row_sum *= alpha;
        if (valid > 0) {
          // operand layout of P: one [128 rows x 128 B] tile per 64-key k-block (= this warp's
          // column group), 16-byte chunks XOR-swizzled by the row's position in its 8-row group
          uint8_t* tile_base = p_smem + group * 16384 + row_in_tile * 128;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t packed[8];
            float partial = 0.0f;
            const bool full = u * 16 + 16 <= valid;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              // p = exp(scale * s - max) = 2^(s * scale*log2(e) - max*log2(e)): one FMA + one EX2
              float e0 = exp2f(fmaf(__uint_as_float(raw[u][2 * t]), scale_log2, -max_log2));
              float e1 = exp2f(fmaf(__uint_as_float(raw[u][2 * t + 1]), scale_log2, -max_log2));
              if (!full) {
                const int c = u * 16 + 2 * t;
                e0 = c < valid ? e0 : 0.0f;
                e1 = c + 1 < valid ? e1 : 0.0f;
              }
              partial += e0 + e1;
              const __nv_bfloat162 pair = __floats2bfloat162_rn(e0, e1);
              packed[t] = *reinterpret_cast<const uint32_t*>(&pair);
            }
            row_sum += partial;
            *reinterpret_cast<uint4*>(tile_base + (((2 * u) ^ (row_in_tile & 7)) << 4)) =
                make_uint4(packed[0], packed[1], packed[2], packed[3]);
            *reinterpret_cast<uint4*>(tile_base + (((2 * u + 1) ^ (row_in_tile & 7)) << 4)) =
                make_uint4(packed[4], packed[5], packed[6], packed[7]);
          }
        }
        ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
        ptx::tc_fence_before();
        ptx::mbar_arrive(p_full);
        ++p_blocks;
      }
      // row sums of the four column groups (all of them relative to the final run_max)
      float* x_sum = x_max + 2 * 512;  // its own slot: the next tile's block 0 may already write x_max
      x_sum[group * 128 + row_in_tile] = row_sum;
      asm volatile("bar.sync 1, %0;" ::"n"(kFmhaSoftmaxThreads) : "memory");
      const float total = (x_sum[row_in_tile] + x_sum[128 + row_in_tile]) +
                          (x_sum[256 + row_in_tile] + x_sum[384 + row_in_tile]);
      if (ok) ok = ptx::mbar_wait(o_full, items_done & 1);
      ptx::tc_fence_after();
      if (!ok && lane == 0) atomicCAS(p.status, 0, kFmhaTimeout);
      const float inv = total > 0.0f ? 1.0f / total : 0.0f;
      const long long out_row =
          (long long)head * p.out_sb0 + (long long)b1 * p.out_sb1 + (long long)row * p.out_ld;
#pragma unroll 1
      for (int cc = group; cc < n_pv / 16; cc += 4) {
        uint32_t raw[16];
        ptx::tmem_ld_16(tmem_o + lane_base + cc * 16, raw);
        ptx::tmem_ld_wait();
        if (row >= p.q_rows) continue;
        fmha_store_chunk16(p, raw, inv, out_row, cc * 16, hd);
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(o_free);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_s, 512);
  }
}

}  // namespace pi05
