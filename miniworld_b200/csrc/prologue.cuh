// Fused prologue: input LayerNorm + left/right gated projections + sigmoid gate + pair mask.
//
//   x_hat = (z - mean) * rstd                          (affine folded into the packed weights)
//   left  = sigmoid(x_hat Wlg'^T + dlg) * (x_hat Wl'^T + dl) * valid(i,k)
//   right = likewise with Wrg', Wr'
//
// Packed weights carry 0.5 * W * gamma (bf16) and d = 0.5 * (W beta + bias), so that
// sigmoid(g) * p = (tanh(g/2) + 1) * (p/2) costs one MUFU op and one FMA per output.
//
// One persistent CTA per SM walks tiles of 128 consecutive columns j of one pair row (b, i).
// Per tile the four GEMMs are issued as D^T[h, pos] = W'[h, c] * x_hat^T[c, pos] on tcgen05, so TMEM
// lanes are channels and columns are positions: each epilogue thread owns one channel and writes
// runs of consecutive positions, which is exactly the row-plane layout [B, rows, H, N] of the outputs.
//
// Warp roles (448 threads): warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2-5 LayerNorm
// (one thread per position, normalises the tile in place in shared memory and builds the mask),
// warps 6-9 epilogue for `left`, warps 10-13 epilogue for `right`.  The left and right accumulator
// pairs are separate TMEM buffers, so the MMAs of one overlap the epilogue of the other.
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
  const float* d1;            // [4][128] additive constants: left, left gate, right, right gate
  __nv_bfloat16* left_out;    // [B, rows, 128, N]
  __nv_bfloat16* right_out;   // [B, rows, 128, N]
  float eps;
  int* status;
};

constexpr int kPrologueThreads = 448;
constexpr int kProStages = 3;
constexpr int kProRing = 5;            // mask ring entries (>= stages + 2)
constexpr int kProRingBytes = 272;     // 64 pair-mask words + 4 ballots
constexpr int kProWBytes = 4 * 32768;  // four 128x128 bf16 matrices
constexpr int kProZBytes = 32768;      // 128 positions x 128 channels bf16
constexpr int kProSmemBytes = kProWBytes + kProStages * kProZBytes + kProRing * kProRingBytes + 128 + 1024;

__global__ void __launch_bounds__(kPrologueThreads, 1)
prologue_kernel(const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_w,
                const PrologueParams p) {
  constexpr int S = kProStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t w_base = smem_base;
  const uint32_t z_base = smem_base + kProWBytes;
  const uint32_t ring_base = z_base + S * kProZBytes;
  const uint32_t bar_base = ring_base + kProRing * kProRingBytes;
  uint32_t* ring_ptr = reinterpret_cast<uint32_t*>(smem + kProWBytes + S * kProZBytes);
  // barriers: w_full, z_full[S], xn_ready[S], z_empty[S], acc_full[2], acc_empty[2]
  const uint32_t w_full = bar_base;
  auto z_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto xn_ready = [&](int s) { return bar_base + 8u * (1 + S + s); };
  auto z_empty = [&](int s) { return bar_base + 8u * (1 + 2 * S + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (1 + 3 * S + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (1 + 3 * S + 2 + a); };
  uint32_t* tmem_slot =
      reinterpret_cast<uint32_t*>(smem + kProWBytes + S * kProZBytes + kProRing * kProRingBytes + 8 * (1 + 3 * S + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int s = 0; s < S; ++s) {
      mbar_init(z_full(s), 1);
      mbar_init(xn_ready(s), 4);
      mbar_init(z_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full(a), 1);
      mbar_init(acc_empty(a), 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_z);
    prefetch_tmap(&map_w);
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
      constexpr uint32_t idesc = umma_idesc(128, 128, false, false);
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
  } else if (warp < 6) {
    // ------------------------------------------------------------ LayerNorm + mask (one thread per position)
    const int pos = (warp - 2) * 32 + lane;
    int s = 0;
    uint32_t ph = 0;
    int e = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
      const int row = tile / p.tiles_per_row;
      const int j0 = (tile - row * p.tiles_per_row) * 128;
      const int bb = row / p.rows;
      const int il = row - bb * p.rows;
      const int j = j0 + pos;
      bool valid = j < p.n;
      if (valid && p.token_mask != nullptr) {
        const uint8_t* tm = p.token_mask + static_cast<size_t>(bb) * p.n;
        valid = (tm[p.row_offset + il] != 0) && (tm[j] != 0);
      }
      if (valid && p.pair_mask != nullptr) valid = p.pair_mask[static_cast<size_t>(row) * p.n + j] != 0;

      const bool got = mbar_wait(z_full(s), ph, abort_flag, p.status, kDevTimeoutStats);
      if (!named_bar_and(2, 128, got)) break;

      const uint32_t rowaddr = z_base + s * kProZBytes + pos * 128;
      uint4 v[16];
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t addr = rowaddr + half * 16384 + ((c ^ (pos & 7)) << 4);
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v[half * 8 + c].x), "=r"(v[half * 8 + c].y), "=r"(v[half * 8 + c].z),
                         "=r"(v[half * 8 + c].w)
                       : "r"(addr));
        }
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        sum += bf16_lo(v[c].x) + bf16_hi(v[c].x);
        sum += bf16_lo(v[c].y) + bf16_hi(v[c].y);
        sum += bf16_lo(v[c].z) + bf16_hi(v[c].z);
        sum += bf16_lo(v[c].w) + bf16_hi(v[c].w);
      }
      const float mean = sum * (1.0f / 128.0f);
      float ssq = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint32_t w4[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float d0 = bf16_lo(w4[t]) - mean;
          const float d1 = bf16_hi(w4[t]) - mean;
          ssq = fmaf(d0, d0, ssq);
          ssq = fmaf(d1, d1, ssq);
        }
      }
      const float rstd = rsqrtf(ssq * (1.0f / 128.0f) + p.eps);
      const float nmr = -mean * rstd;
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 in = v[half * 8 + c];
          uint4 o;
          o.x = pack_bf16x2(fmaf(bf16_lo(in.x), rstd, nmr), fmaf(bf16_hi(in.x), rstd, nmr));
          o.y = pack_bf16x2(fmaf(bf16_lo(in.y), rstd, nmr), fmaf(bf16_hi(in.y), rstd, nmr));
          o.z = pack_bf16x2(fmaf(bf16_lo(in.z), rstd, nmr), fmaf(bf16_hi(in.z), rstd, nmr));
          o.w = pack_bf16x2(fmaf(bf16_lo(in.w), rstd, nmr), fmaf(bf16_hi(in.w), rstd, nmr));
          const uint32_t addr = rowaddr + half * 16384 + ((c ^ (pos & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                       : "memory");
        }
      // mask ring entry: 64 pair-mask words (one per two positions) and the four warp ballots
      const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, valid);
      uint32_t* ring = ring_ptr + e * (kProRingBytes / 4);
      if (lane < 16) {
        const uint32_t two = (ballot >> (2 * lane)) & 3u;
        ring[(warp - 2) * 16 + lane] = ((two & 1u) ? 0x0000FFFFu : 0u) | ((two & 2u) ? 0xFFFF0000u : 0u);
      }
      if (lane == 0) ring[64 + (warp - 2)] = ballot;
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
    // ------------------------------------------------------------ epilogue: warps 6-9 left, 10-13 right
    const int set = (warp - 6) >> 2;
    const int q = warp & 3;
    const int h = q * 32 + lane;
    const float dp = p.d1[(set * 2 + 0) * 128 + h];
    const float dg = p.d1[(set * 2 + 1) * 128 + h];
    __nv_bfloat16* out_base = set == 0 ? p.left_out : p.right_out;
    const uint32_t t_p = tmem_base + set * 256 + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t t_g = t_p + 128;
    int it = 0;
    int e = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int row = tile / p.tiles_per_row;
      const int j0 = (tile - row * p.tiles_per_row) * 128;
      const bool got = mbar_wait(acc_full(set), it & 1, abort_flag, p.status, kDevTimeoutEpilogue);
      if (!named_bar_and(3 + set, 128, got)) break;
      tc_fence_after();
      const uint32_t ring = ring_base + e * kProRingBytes;
      uint32_t b0, b1, b2, b3;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(ring + 256));
      const bool all_valid = (b0 & b1 & b2 & b3) == 0xFFFFFFFFu;
      const bool none_valid = (b0 | b1 | b2 | b3) == 0u;
      __nv_bfloat16* dst = out_base + (static_cast<size_t>(row) * 128 + h) * p.n + j0;
#pragma unroll 1
      for (int c32 = 0; c32 < 4; ++c32) {
        uint32_t vp[32], vg[32];
        if (!none_valid) {
          tmem_ld32(t_p + c32 * 32, vp);
          tmem_ld32(t_g + c32 * 32, vg);
          tmem_ld_wait();
        }
        if (c32 == 3) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty(set));
        }
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          const int col = c32 * 32 + c8 * 8;
          uint4 o = make_uint4(0u, 0u, 0u, 0u);
          if (!none_valid) {
            float r[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              const float hp = __uint_as_float(vp[c8 * 8 + t]) + dp;
              const float th = tanh_approx(__uint_as_float(vg[c8 * 8 + t]) + dg);
              r[t] = fmaf(th, hp, hp);
            }
            o.x = pack_bf16x2(r[0], r[1]);
            o.y = pack_bf16x2(r[2], r[3]);
            o.z = pack_bf16x2(r[4], r[5]);
            o.w = pack_bf16x2(r[6], r[7]);
            if (!all_valid) {
              uint32_t m0, m1, m2, m3;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(m0), "=r"(m1), "=r"(m2), "=r"(m3)
                           : "r"(ring + (col >> 1) * 4));
              o.x &= m0;
              o.y &= m1;
              o.z &= m2;
              o.w &= m3;
            }
          }
          if (j0 + col < p.n) *reinterpret_cast<uint4*>(dst + col) = o;
        }
      }
      if (++e == kProRing) e = 0;
    }
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
