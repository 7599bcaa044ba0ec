// Fused attention for the PI0.5 forward on tcgen05 tensor cores: softmax(scale * Q K^T) V in one
// launch, for the three attention shapes of the model
//   SigLIP       per (image, head): 256 queries x 256 keys, head_dim 72
//   prefix MQA   per sample: (tokens x 8 heads) query rows share one K/V head, head_dim 256
//   action MQA   per sample: (horizon x 8 heads) rows over the prefix + action KV cache
// No mask; at most 1024 keys. Replaces the QK^T GEMM -> row softmax -> PV GEMM chain (and with it
// the logits round trip through HBM) that the reference runs through cuBLAS
// (crates/apxinf-cuda/adapters/cublas_adapter.cu:89-132) or its FMHA / FA2 kernels
// (crates/apxinf-cuda/kernels/cutlass/fmha_sm100.cu, fa2_bf16_sm80.cu).
//
// CTAs are persistent (one per SM) and walk 128-row query tiles; multi-query heads that share a
// K/V head are packed into one tile (row = token * heads + head). One pass over 128-key blocks
// with a running row maximum, the probabilities kept in TENSOR MEMORY. Warp roles: 0 = TMA
// producer, 1 = MMA issuer, 2..17 = softmax / epilogue: four warps per TMEM lane quarter
// (thread = query row), each owning 32 key columns of every block and 64 output columns.
// TMEM: two 128-column score buffers and the 256-column output accumulator. Per block j
// (buffer b = j & 1):
//   MMA warp      S_j = Q K_j^T (UMMA 128 x 128) into buffer b; S_{j+2} follows PV_j
//   softmax warps pull their 32 score columns into registers, exchange the block maximum
//                 through shared memory, p = 2^(s c - m c), write P_j as packed bf16 pairs over
//                 the first 64 columns of buffer b (tcgen05.st), then - once PV_{j-1} is done -
//                 rescale O by alpha = 2^((m_old - m) c) in TMEM (skipped when no row of the
//                 warp moved its maximum)
//   MMA warp      O += P_j V_j with the A operand read from TMEM and V MN-major from the
//                 [keys, head_dim] cache
// With no probability tile in shared memory the K/V ring has four 32 KB stages beside the 64 KB
// query tile: bytes in flight through TMA are what bounds this kernel. (Earlier forms: two
// passes with the probabilities staged in shared memory and a two-stage ring, then one pass
// with them still in shared memory.)
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "fmha.h"
#include "fmha_common.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace pi05 {

constexpr int kOnlineKeyBlock = 128;
constexpr int kOnlineStages = 4;
constexpr int kOnlineSmemBytes =
    kFmhaQBytes + kOnlineStages * kFmhaStageBytes + 1024 + 256 + kFmhaExchangeBytes;

__global__ void __launch_bounds__(kFmhaThreads, 1)
fmha_online_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const FmhaParams p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* ring = q_smem + kFmhaQBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + kOnlineStages * kFmhaStageBytes);
  uint64_t* q_full = bars;           // Q tile landed
  uint64_t* ring_full = bars + 1;    // [kOnlineStages]
  uint64_t* ring_empty = bars + 5;   // [kOnlineStages]
  uint64_t* s_full = bars + 9;       // [2] score buffer written
  uint64_t* p_full = bars + 11;      // P block in TMEM and O rescaled
  uint64_t* p_free = bars + 12;      // PV MMAs done: the score buffer may be reused, O is up to date
  uint64_t* o_full = bars + 13;      // output accumulator complete
  uint64_t* q_free = bars + 14;      // every QK^T MMA of the tile has read Q
  uint64_t* o_free = bars + 15;      // epilogue has read the output accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  float* x_max = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);  // [2][4][128] by block parity, then [4][128] row sums

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
  const int k_stages = (hd_chunks + 1) >> 1;  // ring stages per K block: two 64-dim chunks each
  const int n_blocks = (p.keys + kOnlineKeyBlock - 1) / kOnlineKeyBlock;
  auto stage_ptr = [&](int s) -> uint8_t* { return ring + s * kFmhaStageBytes; };
  const int n_pv = (hd + 15) & ~15;  // UMMA N of the PV product
  auto keys_in_block = [&](int j) { return min(kOnlineKeyBlock, p.keys - j * kOnlineKeyBlock); };

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < kOnlineStages; ++s) {
      ptx::mbar_init(&ring_full[s], 1);
      ptx::mbar_init(&ring_empty[s], 1);
    }
    ptx::mbar_init(&s_full[0], 1);
    ptx::mbar_init(&s_full[1], 1);
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
  const uint32_t tmem_s = *tmem_slot;    // columns [0, 128) and [128, 256): score / probability buffers
  const uint32_t tmem_o = tmem_s + 256;  // columns [256, 512): output accumulator
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer: Q, K_0, K_1, then V_j before K_{j+2} ----------------
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_q);
      ptx::prefetch_tensormap(&tmap_k);
      ptx::prefetch_tensormap(&tmap_v);
      bool ok = true;
      int it = 0;
      int items_done = 0;
      auto acquire = [&]() -> uint8_t* {
        const int s = it % kOnlineStages;
        const int round = it / kOnlineStages;
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
          for (int cp = 0; cp < k_stages && ok; ++cp, ++it) {  // two K chunks [128 keys x 64 dims] per stage
            uint8_t* dst = acquire();
            if (!ok) break;
            const int chunks = min(2, hd_chunks - 2 * cp);
            ptx::mbar_arrive_expect_tx(&ring_full[it % kOnlineStages], chunks * 16384);
            for (int c = 0; c < chunks; ++c) {
              ptx::tma_load_4d(dst + c * 16384, &tmap_k, &ring_full[it % kOnlineStages], (2 * cp + c) * 64,
                               j * kOnlineKeyBlock, b0, b1);
            }
          }
        };
        load_k(0);
        if (n_blocks > 1) load_k(1);
        for (int j = 0; j < n_blocks && ok; ++j) {
          const int subs = (keys_in_block(j) + 63) >> 6;
          for (int v = 0; v < subs && ok; ++v, ++it) {  // V sub-block: [64 keys x head_dim]
            uint8_t* dst = acquire();
            if (!ok) break;
            ptx::mbar_arrive_expect_tx(&ring_full[it % kOnlineStages], hd_chunks * 8192);
            for (int c = 0; c < hd_chunks; ++c) {
              ptx::tma_load_4d(dst + c * 8192, &tmap_v, &ring_full[it % kOnlineStages], c * 64,
                               j * kOnlineKeyBlock + v * 64, b0, b1);
            }
          }
          if (j + 2 < n_blocks) load_k(j + 2);
        }
      }
      if (!ok) atomicCAS(p.status, 0, kFmhaTimeout);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = true;
      const uint32_t idesc_s = ptx::make_idesc(1, 1, 1, 0, 0, 128, kOnlineKeyBlock);
      const uint32_t idesc_o = ptx::make_idesc(1, 1, 1, 0, 1, 128, static_cast<uint32_t>(n_pv));
      const uint32_t q_addr = ptx::smem_u32(q_smem);
      int it = 0;
      int pv_blocks = 0;  // PV blocks issued so far
      int items_done = 0;
      auto issue_s = [&](int j) {
        // the buffer's previous contents (P_{j-2}) were consumed by PV_{j-2}, which the caller
        // has waited for
        const int b = j & 1;
        for (int cp = 0; cp < k_stages && ok; ++cp, ++it) {
          const int s = it % kOnlineStages;
          ok = ptx::mbar_wait(&ring_full[s], (it / kOnlineStages) & 1);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t k_addr = ptx::smem_u32(stage_ptr(s));
          const int chunks = min(2, hd_chunks - 2 * cp);
          for (int c = 0; c < chunks; ++c) {
            const int chunk = 2 * cp + c;
            const int ksteps = min(4, (hd - chunk * 64 + 15) >> 4);
            for (int ks = 0; ks < ksteps; ++ks) {
              ptx::umma<ptx::MmaKind::kF16>(tmem_s + b * kOnlineKeyBlock,
                                            ptx::make_smem_desc(q_addr + chunk * 16384 + ks * 32, 16, 1024),
                                            ptx::make_smem_desc(k_addr + c * 16384 + ks * 32, 16, 1024), idesc_s,
                                            (chunk | ks) != 0 ? 1u : 0u);
            }
          }
          ptx::umma_commit(&ring_empty[s]);
        }
        // signalled even after a timeout so that nobody waits on a dead pipeline
        ptx::umma_commit(&s_full[b]);
        if (j == n_blocks - 1) ptx::umma_commit(q_free);  // the last S product has read Q
      };
      for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++items_done) {
        if (ok) ok = ptx::mbar_wait(q_full, items_done & 1);
        // both score buffers are free: every PV product of the previous tile was waited for below
        issue_s(0);
        if (n_blocks > 1) issue_s(1);
        for (int j = 0; j < n_blocks; ++j) {
          if (ok) ok = ptx::mbar_wait(p_full, pv_blocks & 1);
          // the previous tile's epilogue must have drained the output accumulator
          if (ok && j == 0 && items_done > 0) ok = ptx::mbar_wait(o_free, (items_done - 1) & 1);
          ptx::tc_fence_after();
          const int keys_here = keys_in_block(j);
          const int subs = (keys_here + 63) >> 6;
          const uint32_t p_tmem = tmem_s + (j & 1) * kOnlineKeyBlock;
          for (int v = 0; v < subs && ok; ++v, ++it) {
            const int s = it % kOnlineStages;
            ok = ptx::mbar_wait(&ring_full[s], (it / kOnlineStages) & 1);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t v_addr = ptx::smem_u32(stage_ptr(s));
            const int ksteps = min(4, (keys_here - v * 64 + 15) >> 4);
            for (int ks = 0; ks < ksteps; ++ks) {
              // A = P from TMEM: 8 columns (16 packed bf16 keys) per K step
              ptx::umma_f16_a_tmem(tmem_o, p_tmem + (v * 4 + ks) * 8,
                                   ptx::make_smem_desc(v_addr + ks * 2048, 8192, 1024), idesc_o,
                                   (j | v | ks) != 0 ? 1u : 0u);
            }
            ptx::umma_commit(&ring_empty[s]);
          }
          ptx::umma_commit(p_free);
          ++pv_blocks;
          // Every PV product is waited for before going on: S_{j+2} overwrites the buffer PV_j
          // reads its probabilities from, and the next tile's S_0 / S_1 overwrite the buffers of
          // this tile's last two products. Waiting on each phase in turn also keeps the parity
          // wait exact (a phase is never more than one behind the one asked for).
          if (ok) ok = ptx::mbar_wait(p_free, (pv_blocks - 1) & 1);
          ptx::tc_fence_after();
          if (j + 2 < n_blocks) issue_s(j + 2);
        }
        ptx::umma_commit(o_full);
      }
      if (!ok) atomicCAS(p.status, 0, kFmhaTimeout);
    }
  } else {
    // ---------------- softmax + epilogue (warps 2..17) ----------------
    const int quarter = warp & 3;        // TMEM lane quarter this warp may read
    const int group = (warp - 2) >> 2;   // its 32-key column group and 64 output columns
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    bool ok = true;
    int s_seen[2] = {0, 0};  // score blocks consumed per buffer
    int p_blocks = 0;
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
        const int b = j & 1;
        const uint32_t buf = tmem_s + lane_base + b * kOnlineKeyBlock;
        if (ok) ok = ptx::mbar_wait(&s_full[b], (b == 0 ? s_seen[0] : s_seen[1]) & 1);
        if (b == 0) ++s_seen[0]; else ++s_seen[1];
        ptx::tc_fence_after();
        const int valid = keys_in_block(j) - group * 32;  // valid keys among this warp's 32 columns
        uint32_t raw[2][16];
        ptx::tmem_ld_16(buf + group * 32, raw[0]);
        ptx::tmem_ld_16(buf + group * 32 + 16, raw[1]);
        ptx::tmem_ld_wait();
        float local = -3.0e38f;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            if (u * 16 + t < valid) local = fmaxf(local, __uint_as_float(raw[u][t]));
          }
        }
        float* xm = x_max + b * 512;
        xm[group * 128 + row_in_tile] = local;
        // also orders every group's score loads before the probability stores below, which
        // land on columns another group has just read
        ptx::tc_fence_before();
        asm volatile("bar.sync 1, %0;" ::"n"(kFmhaSoftmaxThreads) : "memory");
        ptx::tc_fence_after();
        const float block_max = fmaxf(fmaxf(xm[row_in_tile], xm[128 + row_in_tile]),
                                      fmaxf(xm[256 + row_in_tile], xm[384 + row_in_tile]));
        // The reference maximum only moves when the block maximum exceeds it by more than 2^8 in
        // the exponent (probabilities then stay below 256, well inside bf16 and fp32 range, and
        // the final division by the row sum cancels the choice exactly): most blocks need no
        // rescaling of O. Every column group of a row sees the same numbers and decides alike.
        // Block 0 always has a valid key, so run_max is finite from block 1 on.
        const bool keep = j > 0 && (block_max - run_max) * scale_log2 <= p.rescale_threshold;
        const float new_max = keep ? run_max : fmaxf(run_max, block_max);
        const float alpha = j == 0 ? 0.0f : exp2f((run_max - new_max) * scale_log2);
        run_max = new_max;
        const float max_log2 = new_max * scale_log2;
        // p = exp(scale * s - max) = 2^(s * scale*log2(e) - max*log2(e)): one FMA + one EX2;
        // packed bf16 pairs (key 2c low, 2c+1 high) = the A-operand layout in TMEM
        uint32_t packed[16];
        float partial = 0.0f;
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          const int c = 2 * t;
          float e0 = exp2f(fmaf(__uint_as_float(raw[t >> 3][(2 * t) & 15]), scale_log2, -max_log2));
          float e1 = exp2f(fmaf(__uint_as_float(raw[t >> 3][(2 * t + 1) & 15]), scale_log2, -max_log2));
          e0 = c < valid ? e0 : 0.0f;
          e1 = c + 1 < valid ? e1 : 0.0f;
          partial += e0 + e1;
          const __nv_bfloat162 pair = __floats2bfloat162_rn(e0, e1);
          packed[t] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        row_sum = row_sum * alpha + partial;
        ptx::tmem_st_16(buf + group * 16, packed);
        if (j > 0 && !__all_sync(0xffffffffu, alpha == 1.0f)) {
          // PV_{j-1} must be done before O is rescaled (no other reason to wait for it: P_j sits
          // in the other score buffer and PV products accumulate in issue order)
          if (ok) ok = ptx::mbar_wait(p_free, (p_blocks - 1) & 1);
          ptx::tc_fence_after();
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
        }
        ptx::tmem_st_wait();
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
