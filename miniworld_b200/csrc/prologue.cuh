// Fused prologue: input LayerNorm + left/right gated projections + sigmoid gate + pair mask.
//
//   x_hat = LayerNorm_in(z)  (fp32 statistics, affine applied, rounded once to fp16 for the tensor cores:
//                             |x_hat| <= sqrt(127) |gamma| + |beta| fits easily and keeps three more
//                             mantissa bits than bf16; the packed weights are fp16 too)
//   left  = sigmoid(x_hat Wlg^T + blg) * (x_hat Wl^T + bl) * valid(i,k)      (biases optional)
//   right = likewise with Wrg, Wr
//
// Packed weights are fp16(0.5 * W) and d = 0.5 * bias, so that
// sigmoid(g) * p = (tanh(g/2) + 1) * (p/2) costs one MUFU op and one FMA per output.
//
// One persistent CTA per SM walks tiles of 128 consecutive columns j of one pair row (b, i).
// Per tile the four GEMMs are issued as D^T[h, pos] = W[h, c] * x_hat^T[c, pos] on tcgen05, so TMEM
// lanes are channels and columns are positions: each epilogue thread owns one channel and writes
// runs of consecutive positions, which is exactly the row-plane layout [B, rows, H, N] of the outputs
// (written as fp16; masked cells are exactly zero).
//
// Outputs leave through a swizzled shared-memory staging tile and TMA stores (full 128-byte rows);
// direct per-thread 16-byte stores to 128 different channel rows ran the store path at a third of this.
//
// Warp roles (832 threads):
//   warp 0        TMA producer (z tiles, weights once)
//   warp 1        MMA issuer / TMEM owner
//   warps 2-9     LayerNorm: 8 threads per position (16 channels each, their gamma/beta in registers),
//                 32 positions per pass, 4 passes per tile; normalises the tile in place in shared memory.
//                 The first four of these warps also build the tile's validity bitmap.
//   warps 10-17   epilogue for `left`  (64 positions at a time: TMEM -> tanh gate -> mask -> staging -> TMA store)
//   warps 18-25   epilogue for `right`
// The left and right accumulator pairs are separate TMEM buffers, so the MMAs of one overlap the
// epilogue of the other.
#pragma once

#include "ptx.cuh"

namespace trimul {

struct PrologueParams {
  int batch;           // B
  int rows;            // pair rows per sample handled by this call
  int n;               // tokens N (columns per row)
  int row_offset;      // global index of local row 0 (token-mask lookup)
  int tiles_per_row;   // ceil(N / 128)
  int num_tiles;       // B * rows * tiles_per_row
  const uint8_t* token_mask;  // [B, N] non-zero = valid, or null
  const uint8_t* pair_mask;   // [B, rows, N] non-zero = valid, or null
  const float* d1;            // [4][128] additive constants (0.5 * bias): left, left gate, right, right gate
  const float* ln_w;          // [128] LayerNorm gamma
  const float* ln_b;          // [128] LayerNorm beta
  float eps;
  int* status;
};

constexpr int kPrologueThreads = 832;
constexpr int kProStages = 2;
constexpr int kProRing = 5;            // mask ring entries (>= stages + 2)
constexpr int kProStageOutBytes = 2 * 16384;  // one [128 channels][64 positions] staging tile per output
constexpr int kProRingBytes = 272;     // 64 pair-mask words + 4 ballots
constexpr int kProWBytes = 4 * 32768;  // four 128x128 bf16 matrices
constexpr int kProZBytes = 32768;      // 128 positions x 128 channels bf16
constexpr int kProSmemBytes =
    kProWBytes + kProStages * kProZBytes + kProStageOutBytes + kProRing * kProRingBytes + 128 + 1024;

template <bool HAS_BIAS>
__global__ void __launch_bounds__(kPrologueThreads, 1)
prologue_kernel(const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ CUtensorMap map_l, const __grid_constant__ CUtensorMap map_r,
                const PrologueParams p) {
  constexpr int S = kProStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t w_base = smem_base;
  const uint32_t z_base = smem_base + kProWBytes;
  const uint32_t stage_out_base = z_base + S * kProZBytes;
  const uint32_t ring_base = stage_out_base + kProStageOutBytes;
  const uint32_t bar_base = ring_base + kProRing * kProRingBytes;
  uint32_t* ring_ptr = reinterpret_cast<uint32_t*>(smem + kProWBytes + S * kProZBytes + kProStageOutBytes);
  // barriers: w_full, z_full[S], xn_ready[S], z_empty[S], acc_full[2], acc_empty[2]
  const uint32_t w_full = bar_base;
  auto z_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto xn_ready = [&](int s) { return bar_base + 8u * (1 + S + s); };
  auto z_empty = [&](int s) { return bar_base + 8u * (1 + 2 * S + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (1 + 3 * S + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (1 + 3 * S + 2 + a); };
  uint32_t* tmem_slot =
      reinterpret_cast<uint32_t*>(smem + kProWBytes + S * kProZBytes + kProStageOutBytes + kProRing * kProRingBytes +
                                  8 * (1 + 3 * S + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int s = 0; s < S; ++s) {
      mbar_init(z_full(s), 1);
      mbar_init(xn_ready(s), 8);
      mbar_init(z_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full(a), 1);
      mbar_init(acc_empty(a), 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_z);
    prefetch_tmap(&map_w);
    prefetch_tmap(&map_l);
    prefetch_tmap(&map_r);
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
      mbar_arrive_expect_tx(w_full, kProWBytes);
#pragma unroll
      for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) tma_load_2d(w_base + m * 32768 + kh * 16384, &map_w, w_full, kh * 64, m * 128);
      int s = 0;
      uint32_t ph = 0;
      int issued = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
        if (!mbar_wait(z_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) break;
        const int row = tile / p.tiles_per_row;
        const int j0 = (tile - row * p.tiles_per_row) * 128;
        mbar_arrive_expect_tx(z_full(s), kProZBytes);
        tma_load_3d(z_base + s * kProZBytes, &map_z, z_full(s), 0, j0, row);
        tma_load_3d(z_base + s * kProZBytes + 16384, &map_z, z_full(s), 64, j0, row);
        ++issued;
        if (++s == S) {
          s = 0;
          ph ^= 1u;
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
      const int pending = issued < S ? issued : S;
      for (int q = 0; q < pending; ++q) {
        if (s == 0) {
          s = S;
          ph ^= 1u;
        }
        --s;
        const long long t0 = clock64();
        while (!mbar_try_wait(z_full(s), ph)) {
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
      constexpr uint32_t idesc = umma_idesc(128, 128, false, false, kFmtF16, kFmtF16);
      bool ok = mbar_wait(w_full, 0, abort_flag, p.status, kDevTimeoutMma);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
        if (!mbar_wait(xn_ready(s), ph, abort_flag, p.status, kDevTimeoutMma)) break;
        tc_fence_after();
        const uint32_t zs = z_base + s * kProZBytes;
        for (int set = 0; set < 2 && ok; ++set) {
          if (!mbar_wait(acc_empty(set), (it & 1) ^ 1u, abort_flag, p.status, kDevTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            const uint32_t d_tmem = tmem_base + set * 256 + m * 128;
            const uint32_t wm = w_base + (set * 2 + m) * 32768;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t da = umma_desc_kmajor(wm + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2);
              const uint64_t db = umma_desc_kmajor(zs + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2);
              umma_bf16(d_tmem, da, db, idesc, ks != 0 ? 1u : 0u);
            }
          }
          umma_commit(acc_full(set));
        }
        if (!ok) break;
        umma_commit(z_empty(s));
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------ LayerNorm (+ validity bitmap)
    const int ts = threadIdx.x - 64;  // 0 .. 255
    const int sub = ts & 7;           // 16-byte chunk: channels 8*sub .. 8*sub+7 of each 64-channel half
    const int slot = ts >> 3;         // position slot inside a pass
    float2 g[8], b[8];                // gamma / beta of this thread's 16 channels, as pairs
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int c = half * 64 + sub * 8 + 2 * t;
        g[half * 4 + t] = make_float2(p.ln_w[c], p.ln_w[c + 1]);
        b[half * 4 + t] = make_float2(p.ln_b[c], p.ln_b[c + 1]);
      }
    int s = 0;
    uint32_t ph = 0;
    int e = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
      const int row = tile / p.tiles_per_row;
      const int j0 = (tile - row * p.tiles_per_row) * 128;
      bool valid = false;
      if (ts < 128) {  // these four warps own one position each for the bitmap
        const int bb = row / p.rows;
        const int il = row - bb * p.rows;
        const int j = j0 + ts;
        const bool inside = j < p.n;
        const int jc = inside ? j : 0;  // clamped so that the three loads below can be issued together
        uint32_t mi = 1u, mj = 1u, mp = 1u;
        if (p.token_mask != nullptr) {
          const uint8_t* tm = p.token_mask + static_cast<size_t>(bb) * p.n;
          mi = tm[p.row_offset + il];
          mj = tm[jc];
        }
        if (p.pair_mask != nullptr) mp = p.pair_mask[static_cast<size_t>(row) * p.n + jc];
        valid = inside && mi != 0u && mj != 0u && mp != 0u;
      }

      const bool got = mbar_wait_warp(z_full(s), ph, abort_flag, p.status, kDevTimeoutStats);
      if (!named_bar_and(2, 256, got)) break;

      const uint32_t zs = z_base + s * kProZBytes;
#pragma unroll 2
      for (int pass = 0; pass < 4; ++pass) {
        const int pos = pass * 32 + slot;
        const uint32_t a0 = zs + pos * 128 + ((sub ^ (pos & 7)) << 4);
        const uint32_t a1 = a0 + 16384;
        uint32_t w[8];
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(a0));
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(a1));
        float2 v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) v[t] = bf16x2_to_float2(w[t]);
        float2 acc = v[0];
#pragma unroll
        for (int t = 1; t < 8; ++t) acc = __fadd2_rn(acc, v[t]);
        float sum = acc.x + acc.y;
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
        const float mean = sum * (1.0f / 128.0f);
        const float2 nmean = make_float2(-mean, -mean);
        float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          v[t] = __fadd2_rn(v[t], nmean);
          q2 = __ffma2_rn(v[t], v[t], q2);
        }
        float ssq = q2.x + q2.y;
        ssq += __shfl_xor_sync(0xFFFFFFFFu, ssq, 1);
        ssq += __shfl_xor_sync(0xFFFFFFFFu, ssq, 2);
        ssq += __shfl_xor_sync(0xFFFFFFFFu, ssq, 4);
        const float rstd = rsqrtf(ssq * (1.0f / 128.0f) + p.eps);
        const float2 rstd2 = make_float2(rstd, rstd);
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = pack_f16x2(__ffma2_rn(__fmul2_rn(v[t], rstd2), g[t], b[t]));
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a0), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a1), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
      }
      if (ts < 128) {
        // mask ring entry: 64 pair-mask words (one per two positions) and the four warp ballots
        const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, valid);
        uint32_t* ring = ring_ptr + e * (kProRingBytes / 4);
        if (lane < 16) {
          const uint32_t two = (ballot >> (2 * lane)) & 3u;
          ring[(warp - 2) * 16 + lane] = ((two & 1u) ? 0x0000FFFFu : 0u) | ((two & 2u) ? 0xFFFF0000u : 0u);
        }
        if (lane == 0) ring[64 + (warp - 2)] = ballot;
      }
      fence_proxy_async_smem();  // x_hat was written through the generic proxy; the MMA reads it through the async one
      __syncwarp();
      if (lane == 0) mbar_arrive(xn_ready(s));
      if (++s == S) {
        s = 0;
        ph ^= 1u;
      }
      if (++e == kProRing) e = 0;
    }
  } else {
    // ------------------------------------------------------------ epilogue: warps 10-17 left, 18-25 right
    // The 8 warps of a set work on 64 positions at a time: warp pair (same TMEM lane quarter) splits them
    // 32 + 32. Results go to a 16 KiB swizzled staging tile [128 channels][64 positions] that one thread
    // hands to a TMA store, so global memory sees full 128-byte rows.
    const int ew = warp - 10;
    const int set = ew >> 3;
    const int sub = (ew >> 2) & 1;  // which 32 of the 64 positions in flight
    const int q = warp & 3;         // TMEM lane quarter this warp may read
    const int h = q * 32 + lane;
    const int bar_id = 3 + set;
    const bool store_thread = ((ew & 7) == 0) && lane == 0;
    const CUtensorMap* map_o = set == 0 ? &map_l : &map_r;
    float dp = 0.f, dg = 0.f;
    if constexpr (HAS_BIAS) {
      dp = p.d1[(set * 2 + 0) * 128 + h];
      dg = p.d1[(set * 2 + 1) * 128 + h];
    }
    const uint32_t stg = stage_out_base + set * 16384;
    const uint32_t stg_row = stg + h * 128;
    const uint32_t t_p = tmem_base + set * 256 + sub * 32 + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t t_g = t_p + 128;
    int it = 0;
    int e = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int row = tile / p.tiles_per_row;
      const int j0 = (tile - row * p.tiles_per_row) * 128;
      const bool got = mbar_wait_warp(acc_full(set), it & 1, abort_flag, p.status, kDevTimeoutEpilogue);
      if (!named_bar_and(bar_id, 256, got)) break;
      tc_fence_after();
      const uint32_t ring = ring_base + e * kProRingBytes;
      uint32_t bal[4];
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(bal[0]), "=r"(bal[1]), "=r"(bal[2]), "=r"(bal[3])
                   : "r"(ring + 256));
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        // validity of this thread's 32 positions (selects, so that bal[] stays in registers)
        const uint32_t bits = half == 0 ? (sub == 0 ? bal[0] : bal[1]) : (sub == 0 ? bal[2] : bal[3]);
        uint32_t o[16];
        if (bits != 0u) {
#pragma unroll
          for (int c16 = 0; c16 < 2; ++c16) {
            uint32_t vp[16], vg[16];
            tmem_ld16(t_p + half * 64 + c16 * 16, vp);
            tmem_ld16(t_g + half * 64 + c16 * 16, vg);
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              float2 hp = make_float2(__uint_as_float(vp[2 * t]), __uint_as_float(vp[2 * t + 1]));
              float2 gg = make_float2(__uint_as_float(vg[2 * t]), __uint_as_float(vg[2 * t + 1]));
              if constexpr (HAS_BIAS) {
                hp = __fadd2_rn(hp, make_float2(dp, dp));
                gg = __fadd2_rn(gg, make_float2(dg, dg));
              }
              const float2 th = make_float2(tanh_approx(gg.x), tanh_approx(gg.y));
              o[c16 * 8 + t] = pack_f16x2(__ffma2_rn(th, hp, hp));
            }
          }
          if (bits != 0xFFFFFFFFu) {
            const uint32_t ma = ring + (half * 32 + sub * 16) * 4;
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              uint32_t m0, m1, m2, m3;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(m0), "=r"(m1), "=r"(m2), "=r"(m3) : "r"(ma + v4 * 16));
              o[v4 * 4 + 0] &= m0;
              o[v4 * 4 + 1] &= m1;
              o[v4 * 4 + 2] &= m2;
              o[v4 * 4 + 3] &= m3;
            }
          }
        } else {
#pragma unroll
          for (int t = 0; t < 16; ++t) o[t] = 0u;
        }
        if (half == 1) {
          // every TMEM read of this tile is done: hand the accumulators back to the MMA issuer
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty(set));
        }
        // the staging tile may be overwritten once the previous TMA store has read it
        if (store_thread) bulk_wait_read<0>();
        named_bar_sync(bar_id, 256);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t addr = stg_row + (((sub * 4 + c) ^ (h & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[4 * c]), "r"(o[4 * c + 1]),
                       "r"(o[4 * c + 2]), "r"(o[4 * c + 3])
                       : "memory");
        }
        fence_proxy_async_smem();
        named_bar_sync(bar_id, 256);
        if (store_thread) {
          const int col0 = j0 + half * 64;
          if (col0 < p.n) tma_store_3d(map_o, stg, col0, 0, row);
          bulk_commit();
        }
      }
      if (++e == kProRing) e = 0;
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
