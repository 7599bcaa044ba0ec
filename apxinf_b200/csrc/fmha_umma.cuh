// Fused attention for the PI0.5 forward on tcgen05 tensor cores: softmax(scale * Q K^T) V
// in one launch, for the three attention shapes of the model
//   SigLIP       per (image, head): 256 queries x 256 keys, head_dim 72
//   prefix MQA   per sample: (tokens x 8 heads) query rows share one K/V head, head_dim 256
//   action MQA   per sample: (horizon x 8 heads) rows over the prefix + action KV cache
// No mask; at most 1024 keys. Replaces the QK^T GEMM -> row softmax -> PV GEMM chain (and
// with it the logits round trip through HBM) that the reference runs through cuBLAS
// (crates/apxinf-cuda/adapters/cublas_adapter.cu:89-132) or its FMHA / FA2 kernels
// (crates/apxinf-cuda/kernels/cutlass/fmha_sm100.cu, fa2_bf16_sm80.cu).
//
// CTAs are persistent (one per SM) and walk 128-row query tiles. Keys are processed in
// blocks of 256:
//   pass 1   S = Q K^T per block (UMMA 128 x 256, accumulator in TMEM), row maxima
//   pass 2   S again, p = exp(scale * s - max) in fp32 (one FMA + one EX2 per score),
//            P (bf16) written to shared memory in the 128-byte-swizzled operand layout,
//            O += P V with V consumed MN-major straight from the [keys, head_dim] cache
// Computing S twice costs a third more tensor work (tiny here) and removes the
// read-modify-write of the output accumulator that online rescaling needs.
// Warp roles: 0 = TMA producer, 1 = MMA issuer, 2..17 = softmax / epilogue: four warps per
// TMEM lane quarter (thread = query row), each owning one 64-key column group of every block.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "fmha.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace pi05 {

constexpr int kFmhaSoftmaxWarps = 16;  // 4 per TMEM lane quarter, one 64-key column group each
constexpr int kFmhaSoftmaxThreads = 32 * kFmhaSoftmaxWarps;
constexpr int kFmhaThreads = 64 + kFmhaSoftmaxThreads;
constexpr int kFmhaKeyBlock = 256;
constexpr int kFmhaQBytes = 4 * 16384;        // up to 4 head-dim chunks of [128 x 128 B]
constexpr int kFmhaStageBytes = 256 * 128;    // one K chunk [256 keys x 128 B] or one V sub-block
constexpr int kFmhaMaxStages = 3;  // two, plus one carved out of the query area when head_dim <= 128
constexpr int kFmhaPBytes = 4 * 16384;        // P: 4 k-blocks of [128 rows x 64 keys]
constexpr int kFmhaExchangeBytes = 3 * 4 * 128 * 4;  // per-row partial maxima (x2) and sums of the 4 column groups
constexpr int kFmhaSmemBytes =
    kFmhaQBytes + 2 * kFmhaStageBytes + kFmhaPBytes + 1024 + 256 + kFmhaExchangeBytes;

// One 16-column chunk of the output accumulator (fp32 bits in `raw`), normalised by `inv`, to
// global memory as bf16 or as e4m3(clamp(bf16(o) * out_inv_scale)); widest aligned stores.
__device__ __forceinline__ void fmha_store_chunk16(const FmhaParams& p, const uint32_t (&raw)[16],
                                                   float inv, long long out_row, int d0, int hd) {
  const int valid = min(16, hd - d0);
  if (p.out_e4m3) {
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + out_row + d0;
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      // the reference rounds the attention output to 16 bits before quantising it
      const float o = __bfloat162float(__float2bfloat16(__uint_as_float(raw[t]) * inv));
      const float clamped = fminf(448.0f, fmaxf(-448.0f, o * p.out_inv_scale));
      const uint32_t byte = static_cast<uint8_t>(__nv_cvt_float_to_fp8(clamped, __NV_SATFINITE, __NV_E4M3));
      w[t >> 2] |= byte << (8 * (t & 3));
    }
    // head_dim is a multiple of 8, so a row's chunk starts on an 8-byte boundary
    // whenever the head stride and leading dimension do: widest aligned store wins
    const uintptr_t addr = reinterpret_cast<uintptr_t>(dst);
    if (valid == 16 && (addr & 15u) == 0) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else if ((addr & 7u) == 0 && (valid & 7) == 0) {
      *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
      if (valid == 16) *reinterpret_cast<uint2*>(dst + 8) = make_uint2(w[2], w[3]);
    } else {
      for (int t = 0; t < valid; ++t) dst[t] = static_cast<uint8_t>(w[t >> 2] >> (8 * (t & 3)));
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + out_row + d0;
    uint32_t w[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(raw[2 * t]) * inv,
                                                       __uint_as_float(raw[2 * t + 1]) * inv);
      w[t] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    const uintptr_t addr = reinterpret_cast<uintptr_t>(dst);
    if ((addr & 15u) == 0 && (valid & 7) == 0) {
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      if (valid == 16) reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
      for (int t = 0; t < valid; ++t) {
        dst[t] = reinterpret_cast<const __nv_bfloat16*>(w)[t];
      }
    }
  }
}

__global__ void __launch_bounds__(kFmhaThreads, 1)
fmha_umma_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const FmhaParams p) {
  pdl_launch_dependents();
  const long long t_entry = clock64();
  const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
#define PI05_TRACE(slot) do { if (tracing && items_done == p.trace_item) p.trace[slot] = static_cast<unsigned int>(clock64() - t_entry); } while (0)
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
  uint64_t* s_free = bars + 8;      // softmax warps done reading S
  uint64_t* p_full = bars + 9;      // P block written
  uint64_t* p_free = bars + 10;     // PV MMAs done reading P
  uint64_t* o_full = bars + 11;     // output accumulator complete
  uint64_t* q_free = bars + 12;     // every QK^T MMA of the tile has read Q
  uint64_t* o_free = bars + 13;     // epilogue has read the output accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  float* x_max = reinterpret_cast<float*>(p_smem + kFmhaPBytes + 256);  // [4][128]
  float* x_sum = x_max + 4 * 128;                                       // [4][128]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // pack > 1: the nb0 query heads share one K/V head, so a 128-row tile holds 128 / pack
  // tokens x pack heads (row = token * pack + head) and K/V are fetched once for all of them
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
  // with a single key block the scores stay in TMEM between the two passes: no second S product
  const bool reuse_s = n_blocks == 1;
  // head_dim <= 128 leaves the upper half of the query area free: a third ring stage
  const int stages = hd_chunks <= 2 ? 3 : 2;
  auto stage_ptr = [&](int s) -> uint8_t* {
    return s < 2 ? q_smem + kFmhaQBytes + s * kFmhaStageBytes : q_smem + 2 * 16384;
  };
  const int n_pv = (hd + 15) & ~15;  // UMMA N of the PV product

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
  const uint32_t tmem_s = *tmem_slot;        // columns [0, 256): S block
  const uint32_t tmem_o = tmem_s + 256;      // columns [256, 512): output accumulator
  pdl_wait();

  auto keys_in_block = [&](int j) { return min(kFmhaKeyBlock, p.keys - j * kFmhaKeyBlock); };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
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
      PI05_TRACE(27);
      ptx::mbar_arrive_expect_tx(q_full, hd_chunks * 16384);
      for (int c = 0; c < hd_chunks; ++c) {
        if (pack > 1) {
          ptx::tma_load_4d(q_smem + c * 16384, &tmap_q, q_full, c * 64, 0, tile * tile_tokens, b1);
        } else {
          ptx::tma_load_4d(q_smem + c * 16384, &tmap_q, q_full, c * 64, tile * 128, b0, b1);
        }
      }
      for (int pass = 0; pass < 2 && ok; ++pass) {
        for (int j = 0; j < n_blocks && ok; ++j) {
          const bool need_s = pass == 0 || !reuse_s;
          for (int c = 0; c < hd_chunks && ok && need_s; ++c, ++it) {  // K chunk: [256 keys x 64 dims]
            uint8_t* dst = acquire();
            if (!ok) break;
            ptx::mbar_arrive_expect_tx(&ring_full[it % stages], kFmhaStageBytes);
            ptx::tma_load_4d(dst, &tmap_k, &ring_full[it % stages], c * 64, j * kFmhaKeyBlock, b0, b1);
          }
          if (pass == 1) {
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
      }
      }  // items
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
      for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++items_done) {
      if (ok) ok = ptx::mbar_wait(q_full, items_done & 1);
      PI05_TRACE(1);
      for (int pass = 0; pass < 2; ++pass) {
        for (int j = 0; j < n_blocks; ++j) {
          const bool need_s = pass == 0 || !reuse_s;
          // S may be overwritten once the softmax warps have read the previous block
          if (ok && need_s && s_blocks > 0) ok = ptx::mbar_wait(s_free, (s_blocks - 1) & 1);
          ptx::tc_fence_after();
          if (pass == 0 && j == 0) PI05_TRACE(26);
          for (int c = 0; c < hd_chunks && ok && need_s; ++c, ++it) {
            const int s = it % stages;
            ok = ptx::mbar_wait(&ring_full[s], (it / stages) & 1);
            if (!ok) break;
            ptx::tc_fence_after();
            if (pass == 0 && j == 0 && c == 0) PI05_TRACE(25);
            const uint32_t k_addr = ptx::smem_u32(stage_ptr(s));
            const int ksteps = min(4, (hd - c * 64 + 15) >> 4);
            for (int ks = 0; ks < ksteps; ++ks) {
              ptx::umma<ptx::MmaKind::kF16>(tmem_s, ptx::make_smem_desc(q_addr + c * 16384 + ks * 32, 16, 1024),
                                            ptx::make_smem_desc(k_addr + ks * 32, 16, 1024), idesc_s,
                                            (c | ks) != 0 ? 1u : 0u);
            }
            ptx::umma_commit(&ring_empty[s]);
          }
          if (need_s) {
            ptx::umma_commit(s_full);
            ++s_blocks;
          }
          if (pass == 0 && j == 0) PI05_TRACE(2);
          if (pass == 1 && j == n_blocks - 1) ptx::umma_commit(q_free);  // Q may be replaced
          if (pass == 1) {
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
        }
      }
      ptx::umma_commit(o_full);
      }  // items
      if (!ok) atomicCAS(p.status, 0, kFmhaTimeout);
    }
  } else {
    // ---------------- softmax + epilogue (warps 2..17) ----------------
    const int quarter = warp & 3;        // TMEM lane quarter this warp may read
    const int group = (warp - 2) >> 2;   // its 64-key column group
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    int s_blocks = 0, p_blocks = 0;
    int items_done = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++items_done) {
    int tile, b0, b1;
    decode(item, &tile, &b0, &b1);
    // query row (token) and head this thread owns
    const int row = pack > 1 ? tile * tile_tokens + row_in_tile / pack : tile * 128 + row_in_tile;
    const int head = pack > 1 ? row_in_tile % pack : b0;
    float raw_max = -3.0e38f;  // maximum of the unscaled scores of this thread's columns
    float row_max = 0.0f;      // scale * max over the whole row, known after pass 1
    float max_log2 = 0.0f;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    float row_sum = 0.0f;
    for (int pass = 0; pass < 2; ++pass) {
      if (pass == 1) {
        // combine the four column groups' maxima (the positive scale is applied afterwards)
        x_max[group * 128 + row_in_tile] = raw_max;
        asm volatile("bar.sync 1, %0;" ::"n"(kFmhaSoftmaxThreads) : "memory");
        const float m = fmaxf(fmaxf(x_max[row_in_tile], x_max[128 + row_in_tile]),
                              fmaxf(x_max[256 + row_in_tile], x_max[384 + row_in_tile]));
        row_max = m * p.scale;
        max_log2 = row_max * 1.4426950408889634f;
      }
      for (int j = 0; j < n_blocks; ++j) {
        if (ok && (pass == 0 || !reuse_s)) ok = ptx::mbar_wait(s_full, s_blocks & 1);
        ptx::tc_fence_after();
        if (threadIdx.x == 64) PI05_TRACE(3 + pass * n_blocks + j);
        const int valid = keys_in_block(j) - group * 64;  // valid keys among this warp's 64 columns
        if (pass == 1 && p_blocks > 0 && ok) ok = ptx::mbar_wait(p_free, (p_blocks - 1) & 1);
        if (valid > 0) {
          // 64 columns per TMEM round trip: four loads in flight, one wait
          uint32_t raw[4][16];
#pragma unroll
          for (int u = 0; u < 4; ++u) ptx::tmem_ld_16(tmem_s + lane_base + group * 64 + u * 16, raw[u]);
          ptx::tmem_ld_wait();
          if (threadIdx.x == 64 && pass == 1 && j == 0) PI05_TRACE(20);
          if (pass == 0) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (u * 16 + 16 <= valid) {
                float m0 = -3.0e38f, m1 = -3.0e38f;
#pragma unroll
                for (int t = 0; t < 16; t += 2) {
                  m0 = fmaxf(m0, __uint_as_float(raw[u][t]));
                  m1 = fmaxf(m1, __uint_as_float(raw[u][t + 1]));
                }
                raw_max = fmaxf(raw_max, fmaxf(m0, m1));
              } else if (u * 16 < valid) {
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                  if (u * 16 + t < valid) raw_max = fmaxf(raw_max, __uint_as_float(raw[u][t]));
                }
              }
            }
          } else {
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
        }
        if (pass == 1) {
          if (threadIdx.x == 64 && j == 0) PI05_TRACE(21);
          ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
          ptx::tc_fence_before();
          if (threadIdx.x == 64 && j == 0) PI05_TRACE(22);
          ptx::mbar_arrive(p_full);
          ++p_blocks;
        } else {
          ptx::tc_fence_before();
        }
        if (pass == 1 || !reuse_s) {
          ptx::mbar_arrive(s_free);
          ++s_blocks;
        }
        if (threadIdx.x == 64) PI05_TRACE(9 + pass * n_blocks + j);
      }
    }
    // row sums of the four column groups
    x_sum[group * 128 + row_in_tile] = row_sum;
    asm volatile("bar.sync 1, %0;" ::"n"(kFmhaSoftmaxThreads) : "memory");
    const float total = (x_sum[row_in_tile] + x_sum[128 + row_in_tile]) +
                        (x_sum[256 + row_in_tile] + x_sum[384 + row_in_tile]);
    if (ok) ok = ptx::mbar_wait(o_full, items_done & 1);
    ptx::tc_fence_after();
    if (threadIdx.x == 64) PI05_TRACE(15);
    if (!ok && lane == 0) atomicCAS(p.status, 0, kFmhaTimeout);
    const float inv = total > 0.0f ? 1.0f / total : 0.0f;
    if (threadIdx.x == 64) PI05_TRACE(24);
    const long long out_row = (long long)head * p.out_sb0 + (long long)b1 * p.out_sb1 + (long long)row * p.out_ld;
#pragma unroll 1
    for (int cc = group; cc < n_pv / 16; cc += 4) {
      uint32_t raw[16];
      ptx::tmem_ld_16(tmem_o + lane_base + cc * 16, raw);
      ptx::tmem_ld_wait();
      if (threadIdx.x == 64 && cc == 0) PI05_TRACE(23);
      if (row >= p.q_rows) continue;
      fmha_store_chunk16(p, raw, inv, out_row, cc * 16, hd);
    }
    if (threadIdx.x == 64) PI05_TRACE(16);
    ptx::tc_fence_before();
    ptx::mbar_arrive(o_free);
    }  // items
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_s, 512);
  }
}

}  // namespace pi05
