// Fused epilogue: output LayerNorm + output projection + sigmoid output gate (+ residual).
//
//   y[pos, c] = z[pos, c] + sigmoid(x_hat[pos,:] Wg^T)[c] * (LN_out(t[pos,:]) Wo^T)[c]
//
// Both LayerNorms are folded around the GEMMs so the tensor cores consume the raw bf16 tiles:
//   LN(v) W^T = rstd * (v W'^T - mean * s) + d,   W' = bf16(0.5 * W * gamma), s = rowsum(W'), d = 0.5 * (W beta + bias)
// (the 0.5 turns sigmoid(g) * p into (tanh(g/2) + 1) * (p/2)).  mean / rstd are per position and come
// from the tiles already in shared memory; s, d are per output channel.  Both operands of one MMA must
// share a 16-bit format (mixing bf16 with fp16 raises an illegal instruction), so the output projection
// is fp16 x fp16 (t arrives as fp16, scaled by 2^-4; eps_out is scaled by 2^-8 to match) and the gate is
// bf16 x bf16 (z is the module's bf16 input).
//
// One persistent CTA per SM walks tiles of 128 consecutive columns j of one pair row (b, i).  Per tile
//   P[pos, c] = t^T[pos, h] * Wo'[c, h]   (A = t tile as loaded from the row-plane layout: MN-major)
//   G[pos, c] = z[pos, c'] * Wg'[c, c']   (A = z tile, K-major)
// run on tcgen05 with TMEM lanes = positions.  An epilogue thread owns one position and 64 of the 128
// output channels: it adds the residual from the z tile in shared memory and writes y in place into that
// tile, which one thread then hands to a TMA store.
//
// Warp roles (576 threads): warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2-9 and 10-17 two
// epilogue groups of 256 threads that take alternate tiles (each owns one shared-memory stage and one
// TMEM buffer).  Inside a group the statistics are computed cooperatively (partial sums over channel
// slices, merged with the pairwise mean / M2 update) while the MMAs of the tile run.
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

constexpr int kEpilogueThreads = 576;
constexpr int kEpiWBytes = 2 * 32768;
constexpr int kEpiStageBytes = 65536;         // t tile (32 KiB) then z tile (32 KiB)
constexpr int kEpiConstBytes = 2048;          // per channel pair: {sg0,sg1,dg0,dg1} and {so0,so1,do0,do1}
constexpr int kEpiXchgBytes = 6144;           // per group: 2 x 128 input partials + 4 x 128 output partials (float2)
constexpr int kEpiSmemBytes = kEpiWBytes + 2 * kEpiStageBytes + kEpiConstBytes + 2 * kEpiXchgBytes + 128 + 1024;

// C = d_pair: the channels of z / y and the rows of both weight matrices (128, or 64 for the narrow pair stacks). The
// contracted width (channels of t, columns of Wo') is 128 in both cases. The shared-memory layout is that of C = 128;
// with C = 64 the z tile, the weights and the per-channel constants fill the first half of their regions.
template <int C = 128>
__global__ void __launch_bounds__(kEpilogueThreads, 1)
epilogue_kernel(const __grid_constant__ CUtensorMap map_t, const __grid_constant__ CUtensorMap map_z,
                const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_wo,
                const __grid_constant__ CUtensorMap map_wg, const EpilogueParams p) {
  static_assert(C == 128 || C == 64, "d_pair is 128 or 64");
  constexpr int kZHalves = C / 64;        // 64-channel (128-byte) halves of a z row
  constexpr int kWoHalf = C * 128;        // bytes of one 64-wide k half of a [C, *] weight matrix
  constexpr int CH = C / 2;               // output channels per epilogue thread
  constexpr int NCH = CH / 8;             // 16-byte chunks (8 channels) per epilogue thread
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t wo_base = smem_base;
  const uint32_t wg_base = smem_base + 32768;
  const uint32_t stage_base = smem_base + kEpiWBytes;
  const uint32_t const_base = stage_base + 2 * kEpiStageBytes;
  const uint32_t xchg_base = const_base + kEpiConstBytes;
  const uint32_t bar_base = xchg_base + 2 * kEpiXchgBytes;
  float4* const_ptr = reinterpret_cast<float4*>(smem + kEpiWBytes + 2 * kEpiStageBytes);
  // barriers: w_full, t_full[2], z_full[2], t_empty[2], z_empty[2], acc_full[2], acc_empty[2].
  // The t tile and the z tile of a stage are filled and released separately: t is dead as soon as the output
  // statistics and the P MMAs are done, so the next t tile streams in while the epilogue still works on z.
  const uint32_t w_full = bar_base;
  auto t_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto z_full = [&](int s) { return bar_base + 8u * (3 + s); };
  auto t_empty = [&](int s) { return bar_base + 8u * (5 + s); };
  auto z_empty = [&](int s) { return bar_base + 8u * (7 + s); };
  auto acc_full = [&](int s) { return bar_base + 8u * (9 + s); };
  auto acc_empty = [&](int s) { return bar_base + 8u * (11 + s); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kEpiWBytes + 2 * kEpiStageBytes + kEpiConstBytes +
                                                    2 * kEpiXchgBytes + 8 * 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(t_full(s), 1);
      mbar_init(z_full(s), 1);
      mbar_init(t_empty(s), 1);
      mbar_init(z_empty(s), 1);
      mbar_init(acc_full(s), 1);
      mbar_init(acc_empty(s), 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_t);
    prefetch_tmap(&map_z);
    prefetch_tmap(&map_y);
    prefetch_tmap(&map_wo);
    prefetch_tmap(&map_wg);
  }
  if (threadIdx.x >= 64 && threadIdx.x < 64 + C / 2) {
    // constants regrouped per channel pair so that one 16-byte load feeds a packed fp32x2 FMA
    const int cp = threadIdx.x - 64;
    const float4 a = p.c3[2 * cp];
    const float4 b = p.c3[2 * cp + 1];
    const_ptr[2 * cp] = make_float4(a.x, b.x, a.y, b.y);      // s_gate pair, d_gate pair
    const_ptr[2 * cp + 1] = make_float4(a.z, b.z, a.w, b.w);  // s_out pair,  d_out pair
  }
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
      // Wo' [C, 128] as two k halves, Wg' [C, C] as C / 64 k halves
      mbar_arrive_expect_tx(w_full, 2 * kWoHalf + kZHalves * kWoHalf);
#pragma unroll
      for (int kh = 0; kh < 2; ++kh) tma_load_2d(wo_base + kh * kWoHalf, &map_wo, w_full, kh * 64, 0);
#pragma unroll
      for (int kh = 0; kh < kZHalves; ++kh) tma_load_2d(wg_base + kh * kWoHalf, &map_wg, w_full, kh * 64, 0);
      int it = 0, t_issued = 0, z_issued = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int row = tile / p.tiles_per_row;
        const int j0 = (tile - row * p.tiles_per_row) * 128;
        const uint32_t ts = stage_base + s * kEpiStageBytes;
        const uint32_t zs = ts + 32768;
        if (!mbar_wait(t_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) break;
        mbar_arrive_expect_tx(t_full(s), 32768);
        // 4-d map (column, channel in group, channel group, row): one group of 128 channels on one GPU, 128/P
        // channels per group when the contraction was sharded by channels; the box covers every group
        tma_load_4d(ts, &map_t, t_full(s), j0, 0, 0, row);
        tma_load_4d(ts + 16384, &map_t, t_full(s), j0 + 64, 0, 0, row);
        ++t_issued;
        if (!mbar_wait(z_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) break;
        mbar_arrive_expect_tx(z_full(s), kZHalves * 16384);
#pragma unroll
        for (int kh = 0; kh < kZHalves; ++kh) tma_load_3d(zs + kh * 16384, &map_z, z_full(s), kh * 64, j0, row);
        ++z_issued;
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
      for (int which = 0; which < 2; ++which) {
        const int issued = which == 0 ? t_issued : z_issued;
        for (int back = 1; back <= 2 && back <= issued; ++back) {
          const int j = issued - back;
          const uint32_t bar = which == 0 ? t_full(j & 1) : z_full(j & 1);
          const long long t0 = clock64();
          while (!mbar_try_wait(bar, (j >> 1) & 1)) {
            if (clock64() - t0 > kWaitLimitCycles) {
              atomicCAS(p.status, 0, kDevTimeoutDrain);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_p = umma_idesc(128, C, true, false, kFmtF16, kFmtF16);
      constexpr uint32_t idesc_g = umma_idesc(128, C, false, false);
      bool ok = mbar_wait(w_full, 0, abort_flag, p.status, kDevTimeoutMma);
      int it = 0;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(t_full(s), ph, abort_flag, p.status, kDevTimeoutMma)) break;
        if (!mbar_wait(acc_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutMma)) break;
        tc_fence_after();
        const uint32_t ts = stage_base + s * kEpiStageBytes;
        const uint32_t zs = ts + 32768;
        const uint32_t d_p = tmem_base + s * 256;
        const uint32_t d_g = d_p + 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t da = umma_desc_mnmajor(ts + ks * 2048, 16384);
          const uint64_t db = umma_desc_kmajor(wo_base + (ks >> 2) * kWoHalf) + static_cast<uint64_t>((ks & 3) * 2);
          umma_bf16(d_p, da, db, idesc_p, ks != 0 ? 1u : 0u);
        }
        if (!mbar_wait(z_full(s), ph, abort_flag, p.status, kDevTimeoutMma)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < C / 16; ++ks) {
          const uint64_t da = umma_desc_kmajor(zs + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2);
          const uint64_t db = umma_desc_kmajor(wg_base + (ks >> 2) * kWoHalf) + static_cast<uint64_t>((ks & 3) * 2);
          umma_bf16(d_g, da, db, idesc_g, ks != 0 ? 1u : 0u);
        }
        umma_commit(acc_full(s));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue groups (256 threads each)
    const int grp = (warp - 2) >> 3;         // 0: even tiles, 1: odd tiles
    const int wg = (warp - 2) & 7;           // warp inside the group
    const int tg = wg * 32 + lane;           // thread inside the group
    const int half = wg >> 2;                // which C / 2 output channels this thread finishes
    const int q = warp & 3;                  // TMEM lane quarter this warp may read
    const int pos = q * 32 + lane;           // position inside the tile == TMEM lane
    const int bar_id = 2 + grp;
    const bool store_thread = tg == 0;
    const uint32_t ts = stage_base + grp * kEpiStageBytes;
    const uint32_t zs = ts + 32768;
    const uint32_t xin = xchg_base + grp * kEpiXchgBytes;   // float2 [2][128]: {mean, M2} over 64 channels of z
    const uint32_t xout = xin + 2048;                        // float2 [4][128]: {mean, M2} over 32 channels of t
    const uint32_t t_p = tmem_base + grp * 256 + half * CH + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t t_g = t_p + 128;
    // output statistics: this thread covers positions 2*pp, 2*pp+1 over channels 32*hq .. 32*hq+31
    const int pp = tg & 63;
    const int hq = tg >> 6;
    const uint32_t tcol = ts + ((2 * pp) >> 6) * 16384 + ((pp & 3) << 2);
    const uint32_t tchunk = ((2 * pp) & 63) >> 3;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      if ((it & 1) != grp) continue;
      const uint32_t ph = (it >> 1) & 1;
      const int row = tile / p.tiles_per_row;
      const int j0 = (tile - row * p.tiles_per_row) * 128;
      // (waits are per thread; a thread that gives up carries on and the group leaves at the tile's last barrier)
      ok &= mbar_wait_thread(t_full(grp), ph, abort_flag, p.status, kDevTimeoutStats);
      // ---- output partial statistics: two adjacent positions, 32 channels of the t tile
      {
        float2 pv = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
#pragma unroll 8
        for (int hh = 0; hh < 32; ++hh) {
          const int h = hq * 32 + hh;
          uint32_t raw;
          asm volatile("ld.shared.b32 %0, [%1];" : "=r"(raw) : "r"(tcol + h * 128 + ((tchunk ^ (h & 7)) << 4)));
          const float2 x = f16x2_to_float2(raw);
          if (hh == 0) pv = x;
          const float2 d = __fadd2_rn(x, make_float2(-pv.x, -pv.y));
          s1 = __fadd2_rn(s1, d);
          s2 = __ffma2_rn(d, d, s2);
        }
        const float mean0 = pv.x + s1.x * (1.0f / 32.0f), mean1 = pv.y + s1.y * (1.0f / 32.0f);
        const float m20 = fmaxf(s2.x - s1.x * s1.x * (1.0f / 32.0f), 0.f);
        const float m21 = fmaxf(s2.y - s1.y * s1.y * (1.0f / 32.0f), 0.f);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(xout + (hq * 128 + 2 * pp) * 8), "f"(mean0),
                     "f"(m20), "f"(mean1), "f"(m21)
                     : "memory");
      }
      ok &= mbar_wait_thread(z_full(grp), ph, abort_flag, p.status, kDevTimeoutStats);
      // ---- input partial statistics over this thread's C / 2 channels of its z row (kept for the residual)
      // C = 128: the thread's channels are one 64-channel half of the tile; C = 64: four of the eight 16-byte chunks of
      // the tile's only half
      const uint32_t zrow = zs + (C == 128 ? half * 16384 : 0) + pos * 128;
      constexpr int kChunk0 = C == 128 ? 0 : 1;  // chunk index of this thread's first chunk = half * 4 * kChunk0
      uint4 zr[NCH];
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(zr[c].x), "=r"(zr[c].y), "=r"(zr[c].z), "=r"(zr[c].w)
                     : "r"(zrow + (((half * 4 * kChunk0 + c) ^ (pos & 7)) << 4)));
      }
      {
        const float pv = bf16_lo(zr[0].x);
        const float2 npv = make_float2(-pv, -pv);
        float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const uint32_t w4[4] = {zr[c].x, zr[c].y, zr[c].z, zr[c].w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 d = __fadd2_rn(bf16x2_to_float2(w4[t]), npv);
            s1 = __fadd2_rn(s1, d);
            s2 = __ffma2_rn(d, d, s2);
          }
        }
        const float a1 = s1.x + s1.y, a2 = s2.x + s2.y;
        const float mean = pv + a1 * (1.0f / CH);
        const float m2 = fmaxf(a2 - a1 * a1 * (1.0f / CH), 0.f);
        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xin + (half * 128 + pos) * 8), "f"(mean), "f"(m2) : "memory");
      }
      named_bar_sync(bar_id, 256);
      // ---- merge the partials of this thread's position (equal-sized groups: mean of means, M2 + n * spread)
      float rs_in, nmr_in, rs_out, nmr_out;
      {
        float ma, qa, mb, qb;
        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(ma), "=f"(qa) : "r"(xin + pos * 8));
        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(mb), "=f"(qb) : "r"(xin + (128 + pos) * 8));
        const float mean = 0.5f * (ma + mb);
        const float dlt = ma - mb;
        const float m2 = qa + qb + dlt * dlt * (0.25f * C);  // n_a n_b / (n_a + n_b) = C / 4
        rs_in = rsqrtf(m2 * (1.0f / C) + p.eps_in);
        nmr_in = -mean * rs_in;
      }
      {
        float m[4], qv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(m[k]), "=f"(qv[k]) : "r"(xout + (k * 128 + pos) * 8));
        const float mean = 0.25f * (m[0] + m[1] + m[2] + m[3]);
        float m2 = qv[0] + qv[1] + qv[2] + qv[3];
#pragma unroll
        for (int k = 0; k < 4; ++k) m2 = fmaf(32.0f * (m[k] - mean), m[k] - mean, m2);
        rs_out = rsqrtf(m2 * (1.0f / 128.0f) + p.eps_out);
        nmr_out = -mean * rs_out;
      }
      const float2 rs_in2 = make_float2(rs_in, rs_in), nmr_in2 = make_float2(nmr_in, nmr_in);
      const float2 rs_out2 = make_float2(rs_out, rs_out), nmr_out2 = make_float2(nmr_out, nmr_out);

      ok &= mbar_wait_thread(acc_full(grp), ph, abort_flag, p.status, kDevTimeoutEpilogue);
      tc_fence_after();
      // every thread is past its output statistics (the exchange barrier above) and the P MMAs are complete: t is dead
      if (store_thread) mbar_arrive(t_empty(grp));
      // C / 16 chunks of 8 channels; the TMEM loads of chunk cc+1 are in flight while chunk cc is finished
      uint32_t vp[2][8], vg[2][8];
      tmem_ld8(t_p, vp[0]);
      tmem_ld8(t_g, vg[0]);
#pragma unroll
      for (int cc = 0; cc < NCH; ++cc) {  // fully unrolled so that zr[] and the two register sets stay in registers
        tmem_ld_wait();
        if (cc < NCH - 1) {
          tmem_ld8(t_p + (cc + 1) * 8, vp[(cc + 1) & 1]);
          tmem_ld8(t_g + (cc + 1) * 8, vg[(cc + 1) & 1]);
        } else {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty(grp));
        }
        uint32_t o[4];
        const uint32_t zz[4] = {zr[cc].x, zr[cc].y, zr[cc].z, zr[cc].w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int pair = half * (CH / 2) + cc * 4 + t;  // channel pair index 0 .. C / 2 - 1
          float4 cg, co;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(cg.x), "=f"(cg.y), "=f"(cg.z), "=f"(cg.w)
                       : "r"(const_base + pair * 32));
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(co.x), "=f"(co.y), "=f"(co.z), "=f"(co.w)
                       : "r"(const_base + pair * 32 + 16));
          const float2 accg = make_float2(__uint_as_float(vg[cc & 1][2 * t]), __uint_as_float(vg[cc & 1][2 * t + 1]));
          const float2 accp = make_float2(__uint_as_float(vp[cc & 1][2 * t]), __uint_as_float(vp[cc & 1][2 * t + 1]));
          const float2 g2 = __ffma2_rn(accg, rs_in2, __ffma2_rn(nmr_in2, make_float2(cg.x, cg.y), make_float2(cg.z, cg.w)));
          const float2 hp = __ffma2_rn(accp, rs_out2, __ffma2_rn(nmr_out2, make_float2(co.x, co.y), make_float2(co.z, co.w)));
          const float2 th = make_float2(tanh_approx(g2.x), tanh_approx(g2.y));
          float2 u = __ffma2_rn(th, hp, hp);
          if (p.residual) u = __fadd2_rn(u, bf16x2_to_float2(zz[t]));
          o[t] = pack_bf16x2(u);
        }
        const uint32_t addr = zrow + (((half * 4 * kChunk0 + cc) ^ (pos & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                     : "memory");
      }
      fence_proxy_async_smem();
      if (!named_bar_and(bar_id, 256, ok)) break;
      if (store_thread) {
#pragma unroll
        for (int kh = 0; kh < kZHalves; ++kh) tma_store_3d(&map_y, zs + kh * 16384, kh * 64, j0, row);
        bulk_commit();
        bulk_wait_read<0>();
        mbar_arrive(z_empty(grp));
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
