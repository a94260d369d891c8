// Fused epilogue: output LayerNorm + output projection + sigmoid output gate (+ residual).
//
//   y[pos, c] = z[pos, c] + sigmoid(x_hat[pos,:] Wg^T)[c] * (LN_out(t[pos,:]) Wo^T)[c]
//
// Both LayerNorms are folded around the GEMMs so the tensor cores consume the raw bf16 tiles:
//   LN(v) W^T = rstd * (v W'^T - mean * s) + d,   W' = bf16(0.5 * W * gamma), s = rowsum(W'), d = 0.5 * (W beta + bias)
// (the 0.5 turns sigmoid(g) * p into (tanh(g/2) + 1) * (p/2)).  mean / rstd are per position and come
// from the tiles already in shared memory; s, d are per output channel.
//
// One persistent CTA per SM walks tiles of 128 consecutive columns j of one pair row (b, i).  Per tile
//   P[pos, c] = t^T[pos, h] * Wo'[c, h]   (A = t tile as loaded from the row-plane layout: MN-major)
//   G[pos, c] = z[pos, c'] * Wg'[c, c']   (A = z tile, K-major)
// run on tcgen05 with TMEM lanes = positions, so each epilogue thread owns one position: its statistics
// live in registers, it adds the residual from the z tile in shared memory and writes y in place into
// that tile, which one thread then hands to a TMA store.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2-5 and 6-9 two
// epilogue groups that take alternate tiles (each owns one shared-memory stage and one TMEM buffer).
#pragma once

#include "ptx.cuh"

namespace trimul {

struct EpilogueParams {
  int tiles_per_row;  // ceil(N / 128)
  int num_tiles;      // B * rows * tiles_per_row
  const float4* c3;   // [128] {s_gate, d_gate, s_out, d_out}
  float eps_in;
  float eps_out;
  int residual;
  int* status;
};

constexpr int kEpilogueThreads = 320;
constexpr int kEpiWBytes = 2 * 32768;
constexpr int kEpiStageBytes = 65536;  // t tile (32 KiB) then z tile (32 KiB)
constexpr int kEpiSmemBytes = kEpiWBytes + 2 * kEpiStageBytes + 2048 + 128 + 1024;

__global__ void __launch_bounds__(kEpilogueThreads, 1)
epilogue_kernel(const __grid_constant__ CUtensorMap map_t, const __grid_constant__ CUtensorMap map_z,
                const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_w,
                const EpilogueParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t wo_base = smem_base;
  const uint32_t wg_base = smem_base + 32768;
  const uint32_t stage_base = smem_base + kEpiWBytes;
  const uint32_t const_base = stage_base + 2 * kEpiStageBytes;
  const uint32_t bar_base = const_base + 2048;
  float4* const_ptr = reinterpret_cast<float4*>(smem + kEpiWBytes + 2 * kEpiStageBytes);
  // barriers: w_full, tile_full[2], tile_empty[2], acc_full[2], acc_empty[2]
  const uint32_t w_full = bar_base;
  auto tile_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto tile_empty = [&](int s) { return bar_base + 8u * (3 + s); };
  auto acc_full = [&](int s) { return bar_base + 8u * (5 + s); };
  auto acc_empty = [&](int s) { return bar_base + 8u * (7 + s); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kEpiWBytes + 2 * kEpiStageBytes + 2048 + 8 * 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(tile_full(s), 1);
      mbar_init(tile_empty(s), 1);
      mbar_init(acc_full(s), 1);
      mbar_init(acc_empty(s), 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_t);
    prefetch_tmap(&map_z);
    prefetch_tmap(&map_y);
    prefetch_tmap(&map_w);
  }
  if (threadIdx.x >= 64 && threadIdx.x < 192) const_ptr[threadIdx.x - 64] = p.c3[threadIdx.x - 64];
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(w_full, kEpiWBytes);
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int kh = 0; kh < 2; ++kh)
          tma_load_2d(wo_base + m * 32768 + kh * 16384, &map_w, w_full, kh * 64, (4 + m) * 128);
      int it = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(tile_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) break;
        const int row = tile / p.tiles_per_row;
        const int j0 = (tile - row * p.tiles_per_row) * 128;
        const uint32_t ts = stage_base + s * kEpiStageBytes;
        const uint32_t zs = ts + 32768;
        mbar_arrive_expect_tx(tile_full(s), kEpiStageBytes);
        tma_load_3d(ts, &map_t, tile_full(s), j0, 0, row);
        tma_load_3d(ts + 16384, &map_t, tile_full(s), j0 + 64, 0, row);
        tma_load_3d(zs, &map_z, tile_full(s), 0, j0, row);
        tma_load_3d(zs + 16384, &map_z, tile_full(s), 64, j0, row);
      }
      // Drain every copy this thread started before the CTA may exit.
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(w_full, 0)) {
          if (clock64() - t0 > kWaitLimitCycles) {
            atomicCAS(p.status, 0, kDevTimeoutDrain);
            break;
          }
        }
      }
      for (int back = 1; back <= 2 && back <= it; ++back) {
        const int j = it - back;
        const long long t0 = clock64();
        while (!mbar_try_wait(tile_full(j & 1), (j >> 1) & 1)) {
          if (clock64() - t0 > kWaitLimitCycles) {
            atomicCAS(p.status, 0, kDevTimeoutDrain);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_p = umma_idesc(128, 128, true, false);
      constexpr uint32_t idesc_g = umma_idesc(128, 128, false, false);
      bool ok = mbar_wait(w_full, 0, abort_flag, p.status, kDevTimeoutMma);
      int it = 0;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(tile_full(s), ph, abort_flag, p.status, kDevTimeoutMma)) break;
        if (!mbar_wait(acc_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutMma)) break;
        tc_fence_after();
        const uint32_t ts = stage_base + s * kEpiStageBytes;
        const uint32_t zs = ts + 32768;
        const uint32_t d_p = tmem_base + s * 256;
        const uint32_t d_g = d_p + 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t da = umma_desc_mnmajor(ts + ks * 2048, 16384);
          const uint64_t db = umma_desc_kmajor(wo_base + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2);
          umma_bf16(d_p, da, db, idesc_p, ks != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t da = umma_desc_kmajor(zs + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2);
          const uint64_t db = umma_desc_kmajor(wg_base + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2);
          umma_bf16(d_g, da, db, idesc_g, ks != 0 ? 1u : 0u);
        }
        umma_commit(acc_full(s));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue groups
    const int grp = (warp - 2) >> 2;  // 0: even tiles, 1: odd tiles
    const int q = warp & 3;
    const int pos = q * 32 + lane;    // position inside the tile == TMEM lane
    const int bar_id = 2 + grp;
    const bool store_thread = (((warp - 2) & 3) == 0) && lane == 0;
    const uint32_t ts = stage_base + grp * kEpiStageBytes;
    const uint32_t zs = ts + 32768;
    const uint32_t t_p = tmem_base + grp * 256 + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t t_g = t_p + 128;
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      if ((it & 1) != grp) continue;
      const uint32_t ph = (it >> 1) & 1;
      const int row = tile / p.tiles_per_row;
      const int j0 = (tile - row * p.tiles_per_row) * 128;
      {
        const bool got = mbar_wait(tile_full(grp), ph, abort_flag, p.status, kDevTimeoutStats);
        if (!named_bar_and(bar_id, 128, got)) break;
      }
      // ---- input statistics from this position's z row (kept in registers for the residual)
      const uint32_t zrow = zs + pos * 128;
      uint4 zr[16];
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t addr = zrow + half * 16384 + ((c ^ (pos & 7)) << 4);
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(zr[half * 8 + c].x), "=r"(zr[half * 8 + c].y), "=r"(zr[half * 8 + c].z),
                         "=r"(zr[half * 8 + c].w)
                       : "r"(addr));
        }
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        sum += bf16_lo(zr[c].x) + bf16_hi(zr[c].x);
        sum += bf16_lo(zr[c].y) + bf16_hi(zr[c].y);
        sum += bf16_lo(zr[c].z) + bf16_hi(zr[c].z);
        sum += bf16_lo(zr[c].w) + bf16_hi(zr[c].w);
      }
      const float mean_in = sum * (1.0f / 128.0f);
      float ssq = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint32_t w4[4] = {zr[c].x, zr[c].y, zr[c].z, zr[c].w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float d0 = bf16_lo(w4[t]) - mean_in;
          const float d1 = bf16_hi(w4[t]) - mean_in;
          ssq = fmaf(d0, d0, ssq);
          ssq = fmaf(d1, d1, ssq);
        }
      }
      const float rs_in = rsqrtf(ssq * (1.0f / 128.0f) + p.eps_in);
      const float nmr_in = -mean_in * rs_in;

      // ---- output statistics from this position's column of the t tile (128 channels)
      float rs_out, nmr_out;
      {
        const uint32_t tcol = ts + (pos >> 6) * 16384 + ((pos & 7) << 1);
        const uint32_t chunk = (pos & 63) >> 3;
        float pivot = 0.f, s1 = 0.f, s2 = 0.f;
#pragma unroll 16
        for (int h = 0; h < 128; ++h) {
          uint16_t raw;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(raw) : "r"(tcol + h * 128 + ((chunk ^ (h & 7)) << 4)));
          const float x = __uint_as_float(static_cast<uint32_t>(raw) << 16);
          if (h == 0) pivot = x;
          const float d = x - pivot;
          s1 += d;
          s2 = fmaf(d, d, s2);
        }
        const float m1 = s1 * (1.0f / 128.0f);
        const float var = fmaxf(s2 * (1.0f / 128.0f) - m1 * m1, 0.f);
        rs_out = rsqrtf(var + p.eps_out);
        nmr_out = -(pivot + m1) * rs_out;
      }

      {
        const bool got = mbar_wait(acc_full(grp), ph, abort_flag, p.status, kDevTimeoutEpilogue);
        if (!named_bar_and(bar_id, 128, got)) break;
      }
      tc_fence_after();
#pragma unroll
      for (int c32 = 0; c32 < 4; ++c32) {  // fully unrolled so that zr[] stays in registers
        uint32_t vp[32], vg[32];
        tmem_ld32(t_p + c32 * 32, vp);
        tmem_ld32(t_g + c32 * 32, vg);
        tmem_ld_wait();
        if (c32 == 3) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty(grp));
        }
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          const int cc = c32 * 4 + c8;  // 16-byte chunk of the row: channels 8*cc .. 8*cc+7
          float r[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            float sg, dg, so, dout;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(sg), "=f"(dg), "=f"(so), "=f"(dout)
                         : "r"(const_base + (cc * 8 + t) * 16));
            const float g2 = fmaf(__uint_as_float(vg[c8 * 8 + t]), rs_in, fmaf(nmr_in, sg, dg));
            const float hp = fmaf(__uint_as_float(vp[c8 * 8 + t]), rs_out, fmaf(nmr_out, so, dout));
            const float th = tanh_approx(g2);
            r[t] = fmaf(th, hp, hp);
          }
          if (p.residual) {
            const uint4 zz = zr[cc];
            r[0] += bf16_lo(zz.x);
            r[1] += bf16_hi(zz.x);
            r[2] += bf16_lo(zz.y);
            r[3] += bf16_hi(zz.y);
            r[4] += bf16_lo(zz.z);
            r[5] += bf16_hi(zz.z);
            r[6] += bf16_lo(zz.w);
            r[7] += bf16_hi(zz.w);
          }
          const uint32_t addr = zrow + (cc >> 3) * 16384 + (((cc & 7) ^ (pos & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_bf16x2(r[0], r[1])),
                       "r"(pack_bf16x2(r[2], r[3])), "r"(pack_bf16x2(r[4], r[5])), "r"(pack_bf16x2(r[6], r[7]))
                       : "memory");
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(bar_id, 128);
      if (store_thread) {
        tma_store_3d(&map_y, zs, 0, j0, row);
        tma_store_3d(&map_y, zs + 16384, 64, j0, row);
        bulk_commit();
        bulk_wait_read<0>();
        mbar_arrive(tile_empty(grp));
      }
    }
    if (store_thread) bulk_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace trimul
