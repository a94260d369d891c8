// Fused epilogue for a contraction result of 64 * KCH channels held in KCH / 2 tensors of 128 channels each:
//
//   y[pos, c] = z[pos, c] + scale[pos, c] * sigmoid(x_hat[pos,:] Wg^T)[c] * (LN_out(t[pos,:]) Wo^T)[c]
//
// KCH = 4 is the bidirectional module: t = [t_outgoing (128), t_incoming (128)], one LayerNorm over the 256
// channels, Wo of shape [128, 256]. KCH = 2 is the unidirectional update again (used to check this kernel
// against epilogue_kernel). Same folding of both LayerNorms around the GEMMs as in epilogue.cuh:
//   LN(v) W^T = rstd * (v W'^T - mean * s) + d.
//
// The wider K does not fit the layout of epilogue_kernel (Wo' alone is 64 KiB), so the t operand streams
// through a ring of three 16 KiB chunks of [64 channels][128 positions] instead of one 32 KiB tile per stage:
// a chunk is released as soon as its four MMAs and the statistics over it are done. Per tile the producer loads
// the z tile and then the KCH chunks; the MMA thread accumulates P += chunk^T * Wo'[:, chunk] chunk by chunk and
// then issues G = z * Wg'^T; the tile's epilogue group keeps running shifted sums over the chunks for the output
// statistics. Everything after the statistics is as in epilogue_kernel.
//
// Warp roles (576 threads): warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2-9 and 10-17 two
// epilogue groups of 256 threads on alternate tiles (each owns one z stage and one TMEM half).
#pragma once

#include "epilogue.cuh"

namespace trimul {

struct EpilogueWideParams {
  int tiles_per_row;    // ceil(N / 128)
  int num_tiles;        // B * rows * tiles_per_row
  int rows_per_sample;  // pair rows per sample in this call (drop_scale lookup)
  int n;                // tokens N
  const float4* c3_a;   // [128] {s_gate, d_gate, s_out, d_out} of the first 128 contracted channels
  const float4* c3_b;   // the same for channels 128..255 (s_out, d_out are added; KCH = 4 only)
  const __nv_bfloat16* drop_scale;  // [B, N, 128] row-shared dropout scale (SCALED instantiations only)
  float eps_in;
  float eps_out;
  int residual;
  int* status;
};

constexpr int kWideRing = 3;
constexpr int kWideChunkBytes = 16384;  // [2 position halves][64 channels][64 positions] fp16
constexpr int kWideWBytes = 3 * 32768;  // Wo' (first 128 channels), Wg', Wo' (channels 128..255)
constexpr int kWideZBytes = 32768;
constexpr int kWideSmemBytes =
    kWideWBytes + kWideRing * kWideChunkBytes + 2 * kWideZBytes + kEpiConstBytes + 2 * kEpiXchgBytes + 256 + 1024;

template <int KCH, bool SCALED>
__global__ void __launch_bounds__(kEpilogueThreads, 1)
epilogue_wide_kernel(const __grid_constant__ CUtensorMap map_t0, const __grid_constant__ CUtensorMap map_t1,
                     const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_y,
                     const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                     const EpilogueWideParams p) {
  static_assert(KCH == 2 || KCH == 4, "two or four chunks of 64 contracted channels");
  constexpr int R = kWideRing;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t wo_base = smem_base;            // Wo' of tensor 0
  const uint32_t wg_base = smem_base + 32768;    // Wg'
  const uint32_t wo1_base = smem_base + 65536;   // Wo' of tensor 1
  const uint32_t ring_base = smem_base + kWideWBytes;
  const uint32_t z_base = ring_base + R * kWideChunkBytes;
  const uint32_t const_base = z_base + 2 * kWideZBytes;
  const uint32_t xchg_base = const_base + kEpiConstBytes;
  const uint32_t bar_base = xchg_base + 2 * kEpiXchgBytes;
  constexpr int kConstOff = kWideWBytes + R * kWideChunkBytes + 2 * kWideZBytes;
  float4* const_ptr = reinterpret_cast<float4*>(smem + kConstOff);
  // barriers: w_full, t_full[2][R], t_empty[R], z_full[2], z_empty[2], acc_full[2], acc_empty[2].
  // A ring slot is filled for tiles of either parity, but an epilogue group only looks at the chunks of its own
  // tiles. A waiter must see every phase of a barrier it waits on (a skipped phase makes the parity test pass
  // early), so "chunk landed" has one barrier per (group, slot): the producer signals the barrier of the group that
  // owns the tile, the group watches only its own, and the MMA thread, which handles every tile, watches both.
  // Each role keeps the parities of these six barriers in a bit mask that it flips per use.
  const uint32_t w_full = bar_base;
  auto t_full = [&](int g, int s) { return bar_base + 8u * (1 + g * R + s); };
  auto t_empty = [&](int s) { return bar_base + 8u * (1 + 2 * R + s); };
  auto z_full = [&](int s) { return bar_base + 8u * (1 + 3 * R + s); };
  auto z_empty = [&](int s) { return bar_base + 8u * (3 + 3 * R + s); };
  auto acc_full = [&](int s) { return bar_base + 8u * (5 + 3 * R + s); };
  auto acc_empty = [&](int s) { return bar_base + 8u * (7 + 3 * R + s); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kConstOff + kEpiConstBytes + 2 * kEpiXchgBytes + 8 * (9 + 3 * R));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int s = 0; s < R; ++s) {
      mbar_init(t_full(0, s), 1);
      mbar_init(t_full(1, s), 1);
      mbar_init(t_empty(s), 9);  // the eight warps of the tile's epilogue group and the MMA commit
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(z_full(s), 1);
      mbar_init(z_empty(s), 1);
      mbar_init(acc_full(s), 1);
      mbar_init(acc_empty(s), 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_t0);
    prefetch_tmap(&map_t1);
    prefetch_tmap(&map_z);
    prefetch_tmap(&map_y);
    prefetch_tmap(&map_w0);
    prefetch_tmap(&map_w1);
  }
  if (threadIdx.x >= 64 && threadIdx.x < 128) {
    // constants regrouped per channel pair so that one 16-byte load feeds a packed fp32x2 FMA
    const int cp = threadIdx.x - 64;
    float4 a = p.c3_a[2 * cp];
    float4 b = p.c3_a[2 * cp + 1];
    if constexpr (KCH == 4) {
      const float4 a1 = p.c3_b[2 * cp];
      const float4 b1 = p.c3_b[2 * cp + 1];
      a.z += a1.z, a.w += a1.w, b.z += b1.z, b.w += b1.w;
    }
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
      mbar_arrive_expect_tx(w_full, KCH == 4 ? kWideWBytes : 65536);
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int kh = 0; kh < 2; ++kh)
          tma_load_2d(wo_base + m * 32768 + kh * 16384, &map_w0, w_full, kh * 64, (4 + m) * 128);
      if constexpr (KCH == 4) {
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) tma_load_2d(wo1_base + kh * 16384, &map_w1, w_full, kh * 64, 4 * 128);
      }
      int it = 0, z_issued = 0;
      long long t_issued = 0;
      uint32_t full_par = 0;  // parity of the next use of t_full(g, slot), bit g * R + slot
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int row = tile / p.tiles_per_row;
        const int j0 = (tile - row * p.tiles_per_row) * 128;
        const uint32_t zs = z_base + s * kWideZBytes;
        if (!mbar_wait(z_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) break;
        mbar_arrive_expect_tx(z_full(s), 32768);
        tma_load_3d(zs, &map_z, z_full(s), 0, j0, row);
        tma_load_3d(zs + 16384, &map_z, z_full(s), 64, j0, row);
        ++z_issued;
#pragma unroll 1
        for (int c = 0; c < KCH; ++c) {
          const long long q = static_cast<long long>(it) * KCH + c;
          const int slot = static_cast<int>(q % R);
          const uint32_t tph = static_cast<uint32_t>((q / R) & 1);
          if (!mbar_wait(t_empty(slot), tph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) {
            ok = false;
            break;
          }
          const uint32_t cs = ring_base + slot * kWideChunkBytes;
          const CUtensorMap* mt = (c >> 1) == 0 ? &map_t0 : &map_t1;
          const int ch0 = (c & 1) * 64;
          mbar_arrive_expect_tx(t_full(s, slot), kWideChunkBytes);
          tma_load_3d(cs, mt, t_full(s, slot), j0, ch0, row);
          tma_load_3d(cs + 8192, mt, t_full(s, slot), j0 + 64, ch0, row);
          full_par ^= 1u << (s * R + slot);
          ++t_issued;
        }
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
      for (int back = 1; back <= 2 && back <= z_issued; ++back) {
        const int j = z_issued - back;
        const long long t0 = clock64();
        while (!mbar_try_wait(z_full(j & 1), (j >> 1) & 1)) {
          if (clock64() - t0 > kWaitLimitCycles) {
            atomicCAS(p.status, 0, kDevTimeoutDrain);
            break;
          }
        }
      }
      for (int back = 1; back <= R && back <= t_issued; ++back) {
        // the last R chunks sit in distinct slots, so each is the latest use of its (group, slot) barrier
        const long long q = t_issued - back;
        const int slot = static_cast<int>(q % R);
        const int g = static_cast<int>((q / KCH) & 1);
        const uint32_t par = ((full_par >> (g * R + slot)) & 1u) ^ 1u;
        const long long t0 = clock64();
        while (!mbar_try_wait(t_full(g, slot), par)) {
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
      constexpr uint32_t idesc_p = umma_idesc(128, 128, true, false, kFmtF16, kFmtF16);
      constexpr uint32_t idesc_g = umma_idesc(128, 128, false, false);
      bool ok = mbar_wait(w_full, 0, abort_flag, p.status, kDevTimeoutMma);
      int it = 0;
      uint32_t full_par = 0;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(acc_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutMma)) break;
        const uint32_t d_p = tmem_base + s * 256;
        const uint32_t d_g = d_p + 128;
#pragma unroll 1
        for (int c = 0; c < KCH; ++c) {
          const long long q = static_cast<long long>(it) * KCH + c;
          const int slot = static_cast<int>(q % R);
          const uint32_t tph = (full_par >> (s * R + slot)) & 1u;
          full_par ^= 1u << (s * R + slot);
          if (!mbar_wait(t_full(s, slot), tph, abort_flag, p.status, kDevTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t cs = ring_base + slot * kWideChunkBytes;
          const uint32_t wb = ((c >> 1) == 0 ? wo_base : wo1_base) + (c & 1) * 16384;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t da = umma_desc_mnmajor(cs + ks * 2048, 8192);
            const uint64_t db = umma_desc_kmajor(wb) + static_cast<uint64_t>(ks * 2);
            umma_bf16(d_p, da, db, idesc_p, (c | ks) != 0 ? 1u : 0u);
          }
          umma_commit(t_empty(slot));
        }
        if (!ok) break;
        if (!mbar_wait(z_full(s), ph, abort_flag, p.status, kDevTimeoutMma)) break;
        tc_fence_after();
        const uint32_t zs = z_base + s * kWideZBytes;
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
    // ------------------------------------------------------------ epilogue groups (256 threads each)
    const int grp = (warp - 2) >> 3;         // 0: even tiles, 1: odd tiles
    const int wg = (warp - 2) & 7;           // warp inside the group
    const int tg = wg * 32 + lane;           // thread inside the group
    const int half = wg >> 2;                // which 64 output channels this thread finishes
    const int q4 = warp & 3;                 // TMEM lane quarter this warp may read
    const int pos = q4 * 32 + lane;          // position inside the tile == TMEM lane
    const int bar_id = 2 + grp;
    const bool store_thread = tg == 0;
    const uint32_t zs = z_base + grp * kWideZBytes;
    const uint32_t xin = xchg_base + grp * kEpiXchgBytes;   // float2 [2][128]: {mean, M2} over 64 channels of z
    const uint32_t xout = xin + 2048;                        // float2 [4][128]: {mean, M2} over 16 * KCH channels of t
    const uint32_t t_p = tmem_base + grp * 256 + half * 64 + (static_cast<uint32_t>(q4 * 32) << 16);
    const uint32_t t_g = t_p + 128;
    // output statistics: this thread covers positions 2*pp, 2*pp+1 over channels 16*hq .. 16*hq+15 of every chunk
    const int pp = tg & 63;
    const int hq = tg >> 6;
    const uint32_t tcol_off = ((2 * pp) >> 6) * 8192 + ((pp & 3) << 2);
    const uint32_t tchunk = ((2 * pp) & 63) >> 3;
    constexpr float kInvPart = 1.0f / (16 * KCH);
    constexpr float kPartN = 16.0f * KCH;
    constexpr float kInvAll = 1.0f / (64 * KCH);
    uint32_t full_par = 0;  // parities of this group's t_full barriers, bit = slot
    int it = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      if ((it & 1) != grp) continue;
      const uint32_t ph = (it >> 1) & 1;
      const int row = tile / p.tiles_per_row;
      const int j0 = (tile - row * p.tiles_per_row) * 128;
      // ---- output partial statistics, chunk by chunk: shifted sums around the first value seen
      {
        float2 pv = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
        bool alive = true;
#pragma unroll 1
        for (int c = 0; c < KCH; ++c) {
          const long long q = static_cast<long long>(it) * KCH + c;
          const int slot = static_cast<int>(q % R);
          const uint32_t tph = (full_par >> slot) & 1u;
          full_par ^= 1u << slot;
          if (!mbar_wait_warp(t_full(grp, slot), tph, abort_flag, p.status, kDevTimeoutStats)) {
            alive = false;
            break;
          }
          const uint32_t tcol = ring_base + slot * kWideChunkBytes + tcol_off;
#pragma unroll 8
          for (int hh = 0; hh < 16; ++hh) {
            const int h = hq * 16 + hh;
            uint32_t raw;
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(raw) : "r"(tcol + h * 128 + ((tchunk ^ (h & 7)) << 4)));
            const float2 x = f16x2_to_float2(raw);
            if (c == 0 && hh == 0) pv = x;
            const float2 d = __fadd2_rn(x, make_float2(-pv.x, -pv.y));
            s1 = __fadd2_rn(s1, d);
            s2 = __ffma2_rn(d, d, s2);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(t_empty(slot));  // this warp's reads of the chunk are done
        }
        if (!named_bar_and(bar_id, 256, alive)) break;
        const float mean0 = pv.x + s1.x * kInvPart, mean1 = pv.y + s1.y * kInvPart;
        const float m20 = fmaxf(s2.x - s1.x * s1.x * kInvPart, 0.f);
        const float m21 = fmaxf(s2.y - s1.y * s1.y * kInvPart, 0.f);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(xout + (hq * 128 + 2 * pp) * 8), "f"(mean0),
                     "f"(m20), "f"(mean1), "f"(m21)
                     : "memory");
      }
      {
        const bool got = mbar_wait_warp(z_full(grp), ph, abort_flag, p.status, kDevTimeoutStats);
        if (!named_bar_and(bar_id, 256, got)) break;
      }
      // ---- input partial statistics over this thread's 64 channels of its z row (kept for the residual)
      const uint32_t zrow = zs + half * 16384 + pos * 128;
      uint4 zr[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(zr[c].x), "=r"(zr[c].y), "=r"(zr[c].z), "=r"(zr[c].w)
                     : "r"(zrow + ((c ^ (pos & 7)) << 4)));
      }
      {
        const float pv = bf16_lo(zr[0].x);
        const float2 npv = make_float2(-pv, -pv);
        float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t w4[4] = {zr[c].x, zr[c].y, zr[c].z, zr[c].w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 d = __fadd2_rn(bf16x2_to_float2(w4[t]), npv);
            s1 = __fadd2_rn(s1, d);
            s2 = __ffma2_rn(d, d, s2);
          }
        }
        const float a1 = s1.x + s1.y, a2 = s2.x + s2.y;
        const float mean = pv + a1 * (1.0f / 64.0f);
        const float m2 = fmaxf(a2 - a1 * a1 * (1.0f / 64.0f), 0.f);
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
        const float m2 = qa + qb + dlt * dlt * 32.0f;  // n_a n_b / (n_a + n_b) = 32
        rs_in = rsqrtf(m2 * (1.0f / 128.0f) + p.eps_in);
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
        for (int k = 0; k < 4; ++k) m2 = fmaf(kPartN * (m[k] - mean), m[k] - mean, m2);
        rs_out = rsqrtf(m2 * kInvAll + p.eps_out);
        nmr_out = -mean * rs_out;
      }
      const float2 rs_in2 = make_float2(rs_in, rs_in), nmr_in2 = make_float2(nmr_in, nmr_in);
      const float2 rs_out2 = make_float2(rs_out, rs_out), nmr_out2 = make_float2(nmr_out, nmr_out);
      // row-shared dropout scale of this thread's 64 channels (loaded before the accumulators are awaited)
      uint4 sc[SCALED ? 8 : 1];
      if constexpr (SCALED) {
        const int bb = row / p.rows_per_sample;
        const int j = j0 + pos < p.n ? j0 + pos : p.n - 1;
        const uint4* sp = reinterpret_cast<const uint4*>(p.drop_scale + (static_cast<size_t>(bb) * p.n + j) * 128 + half * 64);
#pragma unroll
        for (int c = 0; c < 8; ++c) sc[c] = __ldg(sp + c);
      }

      {
        const bool got = mbar_wait_warp(acc_full(grp), ph, abort_flag, p.status, kDevTimeoutEpilogue);
        if (!named_bar_and(bar_id, 256, got)) break;
      }
      tc_fence_after();
      // 8 chunks of 8 channels; the TMEM loads of chunk cc+1 are in flight while chunk cc is finished
      uint32_t vp[2][8], vg[2][8];
      tmem_ld8(t_p, vp[0]);
      tmem_ld8(t_g, vg[0]);
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {  // fully unrolled so that zr[] and the two register sets stay in registers
        tmem_ld_wait();
        if (cc < 7) {
          tmem_ld8(t_p + (cc + 1) * 8, vp[(cc + 1) & 1]);
          tmem_ld8(t_g + (cc + 1) * 8, vg[(cc + 1) & 1]);
        } else {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty(grp));
        }
        uint32_t o[4];
        const uint32_t zz[4] = {zr[cc].x, zr[cc].y, zr[cc].z, zr[cc].w};
        uint32_t ss[4] = {0u, 0u, 0u, 0u};
        if constexpr (SCALED) ss[0] = sc[cc].x, ss[1] = sc[cc].y, ss[2] = sc[cc].z, ss[3] = sc[cc].w;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int pair = half * 32 + cc * 4 + t;  // channel pair index 0..63
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
          if constexpr (SCALED) u = __fmul2_rn(u, bf16x2_to_float2(ss[t]));
          if (p.residual) u = __fadd2_rn(u, bf16x2_to_float2(zz[t]));
          o[t] = pack_bf16x2(u);
        }
        const uint32_t addr = zrow + ((cc ^ (pos & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                     : "memory");
      }
      fence_proxy_async_smem();
      named_bar_sync(bar_id, 256);
      if (store_thread) {
        tma_store_3d(&map_y, zs, 0, j0, row);
        tma_store_3d(&map_y, zs + 16384, 64, j0, row);
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
