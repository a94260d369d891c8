// Backward of the triangle update around the contraction: the epilogue's gradients (output LayerNorm, output
// projection, output gate) and the prologue's gradients (input LayerNorm, the four gated projections, the mask).
//
// Both kernels walk tiles of 128 consecutive columns j of one pair row, one CTA per SM, 512 threads: four threads per
// position (its TMEM lane), each covering a quarter of the channels. A tile goes through a fixed sequence of phases
// separated by CTA-wide barriers; one thread issues the TMA copies and the MMAs. Per tile:
//   1. TMA loads of the tile's inputs; the LayerNorm inputs are normalised in place in shared memory (fp16),
//   2. the forward GEMMs are recomputed on the tensor cores (weights with the LayerNorm gamma folded in, fp16),
//   3. the threads turn the upstream gradient into the gradients of the GEMM outputs (fp16 tiles in shared memory),
//   4. the tensor cores compute, from those tiles, the gradients with respect to the normalised inputs (the same weight
//      tiles read MN-major) and accumulate the weight gradients M = dOut^T x_hat over all tiles of the CTA in TMEM,
//   5. the threads finish (LayerNorm backward) and the results leave through TMA stores.
// The four tile buffers of a CTA rotate their roles from tile to tile: the next tile's inputs are copied into the
// buffers the gradient GEMMs have finished with while the tile completes, and a store is only waited for when its
// buffer is needed again. Column sums of the dOut tiles (the bias-like terms) are accumulated per thread in
// registers. At the end every CTA writes its partial M and column sums; small kernels add the partials and form the
// parameter gradients. Both kernels are templates on the input width C (128, or 64 for the narrow pair stacks); the
// epilogue's backward also has a two-launch form for an output LayerNorm over 256 channels (the bidirectional module).
//
// Gradients travel in fp16 tiles, so the upstream gradient is multiplied by a power of two c (read from device
// memory, chosen from max |dy| by `bwd_amax_kernel` / `bwd_scale_kernel`); every output of these kernels carries that
// factor, and the final kernels divide it out in fp32.
#pragma once

#include "ptx.cuh"

namespace trimul {

#ifndef TRIMUL_BWD_PARTS
#define TRIMUL_BWD_PARTS 4
#endif
constexpr int kBwdParts = TRIMUL_BWD_PARTS;      // threads per position: each covers 128 / kBwdParts channels
constexpr int kBwdThreads = 128 * kBwdParts;
constexpr int kBwdCh = 128 / kBwdParts;          // channels per thread of a 128-channel tile
constexpr int kBwdChunks = kBwdCh / 8;           // 16-byte chunks (8 channels) per thread
constexpr int kBwdTile = 32768;  // one [128][128] 16-bit tile
constexpr int kBwdXchgHalf = kBwdParts * 128 * 8;  // float2 [kBwdParts][128]
constexpr int kBwdXchg = 2 * kBwdXchgHalf;         // two exchange buffers, used in turn (see normalise_tile)
constexpr int kBwdSmemBytes = 6 * kBwdTile + kBwdXchg + 1024 /* constants */ + 256 /* barriers */ + 1024;

// swizzled byte offset of element (r, e) in a [128 rows][128 elements] 16-bit tile stored as two halves of 64 elements,
// each [128 rows][128 bytes] with the 128-byte TMA swizzle
__device__ __forceinline__ uint32_t tile_off(int r, int e) {
  return static_cast<uint32_t>((e >> 6) * 16384 + r * 128 + ((((e & 63) >> 3) ^ (r & 7)) << 4) + (e & 7) * 2);
}
// offset of the 16-byte chunk holding elements 8*ch .. 8*ch+7 (ch = 0..15) of row r
__device__ __forceinline__ uint32_t tile_chunk(int r, int ch) {
  return static_cast<uint32_t>((ch >> 3) * 16384 + r * 128 + (((ch & 7) ^ (r & 7)) << 4));
}

__device__ __forceinline__ float ld_f16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ void st_f16_sat(uint32_t addr, float x) {
  uint16_t v;
  asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(v) : "f"(x));
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_chunk(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void st_chunk(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// 32 bytes per thread in one request (address 32-byte aligned): a warp whose lanes read different 128-byte lines pays
// per line and request, so half as many requests as with 16-byte loads
__device__ __forceinline__ void ldg_32B(const void* p, uint4& a, uint4& b) {
  asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
               : "l"(p));
}
// `chunks` 16-byte pieces (an even count) from p: 32-byte requests if the address allows, else 16-byte ones
template <int CHUNKS>
__device__ __forceinline__ void ldg_chunks(const uint4* p, bool wide, uint4 (&out)[CHUNKS]) {
  static_assert(CHUNKS % 2 == 0, "pairs of 16-byte chunks");
  if (wide) {
#pragma unroll
    for (int c = 0; c < CHUNKS; c += 2) ldg_32B(p + c, out[c], out[c + 1]);
  } else {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) out[c] = __ldg(p + c);
  }
}
__device__ __forceinline__ float sigmoid_fast(float x) { return fmaf(tanh_approx(0.5f * x), 0.5f, 0.5f); }

// (see mbar_wait_thread: a thread that gives up carries on and the CTA leaves together at the tile's closing barrier)
__device__ __forceinline__ bool thread_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  return mbar_wait_thread(bar, parity, abort_flag, status, code);
}
// CTA-wide bounded wait on an mbarrier: one lane per warp polls, the decision is shared by all 256 threads.
__device__ __forceinline__ bool cta_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  const bool got = mbar_wait_warp(bar, parity, abort_flag, status, code);
  return named_bar_and(1, kBwdThreads, got);
}

// Normalise the CT channels of every position of a tile in place (fp16 result), the thread covering CT / kBwdParts of them.
// ROWS_ARE_POSITIONS: element (pos, c) (a [pos][c] tile, input bf16 or fp16), else element (c, pos) (a [c][pos] tile,
// fp16). Returns rstd of the thread's position. `xchg` holds float2 [kBwdParts][128]; the caller must not pass the same
// buffer to two calls (or other uses) without a CTA-wide barrier between them.
template <bool ROWS_ARE_POSITIONS, bool IN_BF16, int CT = 128>
__device__ __forceinline__ float normalise_tile(uint32_t tile, uint32_t xchg, int pos, int part, float eps) {
  constexpr int kCh = CT / kBwdParts;  // channels per thread
  constexpr int kChunks = kCh / 8;
  float pv = 0.f, s1 = 0.f, s2 = 0.f;
  float xt[ROWS_ARE_POSITIONS ? 1 : kCh];  // the [c][pos] form keeps its values between the two passes
  if constexpr (ROWS_ARE_POSITIONS) {
#pragma unroll
    for (int ch = 0; ch < kChunks; ++ch) {
      const uint4 v = ld_chunk(tile + tile_chunk(pos, part * kChunks + ch));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 x = IN_BF16 ? bf16x2_to_float2(w[t]) : f16x2_to_float2(w[t]);
        if (ch == 0 && t == 0) pv = x.x;
        const float d0 = x.x - pv, d1 = x.y - pv;
        s1 += d0 + d1;
        s2 = fmaf(d0, d0, fmaf(d1, d1, s2));
      }
    }
  } else {
#pragma unroll
    for (int cc = 0; cc < kCh; ++cc) xt[cc] = ld_f16(tile + tile_off(part * kCh + cc, pos));
    pv = xt[0];
#pragma unroll
    for (int cc = 0; cc < kCh; ++cc) {
      const float d = xt[cc] - pv;
      s1 += d;
      s2 = fmaf(d, d, s2);
    }
  }
  const float mean_h = pv + s1 * (1.0f / kCh);
  const float m2_h = fmaxf(s2 - s1 * s1 * (1.0f / kCh), 0.f);
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xchg + (part * 128 + pos) * 8), "f"(mean_h), "f"(m2_h) : "memory");
  named_bar_sync(1, kBwdThreads);
  // merge the equal-sized partials of this position: mean of means, M2 = sum M2_k + n_k sum (mean_k - mean)^2
  float mk[kBwdParts], qk[kBwdParts];
  float mean = 0.f, m2 = 0.f;
#pragma unroll
  for (int k = 0; k < kBwdParts; ++k) {
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(mk[k]), "=f"(qk[k]) : "r"(xchg + (k * 128 + pos) * 8));
    mean += mk[k];
    m2 += qk[k];
  }
  mean *= 1.0f / kBwdParts;
#pragma unroll
  for (int k = 0; k < kBwdParts; ++k) m2 = fmaf(static_cast<float>(kCh) * (mk[k] - mean), mk[k] - mean, m2);
  const float rstd = rsqrtf(m2 * (1.0f / CT) + eps);
  const float nmr = -mean * rstd;
  if constexpr (ROWS_ARE_POSITIONS) {
#pragma unroll
    for (int ch = 0; ch < kChunks; ++ch) {
      const uint32_t addr = tile + tile_chunk(pos, part * kChunks + ch);
      const uint4 v = ld_chunk(addr);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t o[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 x = IN_BF16 ? bf16x2_to_float2(w[t]) : f16x2_to_float2(w[t]);
        o[t] = pack_f16x2_sat(make_float2(fmaf(x.x, rstd, nmr), fmaf(x.y, rstd, nmr)));
      }
      st_chunk(addr, o[0], o[1], o[2], o[3]);
    }
  } else {
#pragma unroll
    for (int cc = 0; cc < kCh; ++cc) st_f16_sat(tile + tile_off(part * kCh + cc, pos), fmaf(xt[cc], rstd, nmr));
  }
  return rstd;  // (no closing barrier: consecutive calls alternate between the two exchange buffers)
}

// Sum of the float2 partials the kBwdParts threads of a position left in `xchg` (fixed order).
__device__ __forceinline__ void sum_partials(uint32_t xchg, int pos, float& a, float& b) {
  a = 0.f, b = 0.f;
#pragma unroll
  for (int k = 0; k < kBwdParts; ++k) {
    float x, y;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(x), "=f"(y) : "r"(xchg + (k * 128 + pos) * 8));
    a += x, b += y;
  }
}

// Sum the per-thread column partials of a CTA over its 128 positions: `acc` holds this thread's channels (part
// `part`) for two vectors; scratch is float[256][129] (a tile region, padded against bank conflicts).
template <int NCH>
__device__ __forceinline__ void flush_colsums(const float (&a0)[NCH], const float (&a1)[NCH], uint8_t* scratch, int pos,
                                              int part, float* out0, float* out1) {
  float* s = reinterpret_cast<float*>(scratch);
  // rows: (vector * 128 + channel), columns: position
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    s[(0 * 128 + part * NCH + c) * 129 + pos] = a0[c];
    s[(1 * 128 + part * NCH + c) * 129 + pos] = a1[c];
  }
  __syncthreads();
  const int r = threadIdx.x;  // 0..255: vector r / 128, channel r % 128 (channels beyond 4 * NCH do not exist)
  if (r < 256 && (r & 127) < NCH * kBwdParts) {
    float sum = 0.f;
    for (int p = 0; p < 128; ++p) sum += s[r * 129 + p];
    (r < 128 ? out0 : out1)[r & 127] = sum;
  }
  __syncthreads();
}

struct BwdEpilogueParams {
  int tiles_per_row;   // ceil(N / 128)
  int num_tiles;       // B * N * tiles_per_row
  int n;               // N
  const float* consts;      // [2][128]: d_out = W_out beta_out + bias_out, d_gate = W_gate beta_in + bias_gate
  const float* grad_scale;  // [2]: c, 1 / c
  const uint16_t* drop_scale;  // [B][N][128] bf16 or null
  float eps_in;
  float eps_out;       // scaled by 2^-8: tri is stored times 2^-4
  float* part_m;       // [grid][2][128][128]: per-CTA partial sums of dproj^T t_hat and dgate^T x_hat
  float* part_s;       // [grid][2][128]: per-CTA column sums of dproj and dgate
  // the two-launch form for an output LayerNorm over 256 channels (MODE 1: first 128 channels, MODE 2: the others)
  const float2* ext_stats;  // [B*N][N]: mean and rstd of the stored t over all 256 channels
  float2* ln_part;          // [B*N][N]: MODE 1 writes its sums of d t_hat and d t_hat * t_hat; MODE 2 adds its own and
                            // writes back the two means over 256 channels
  const uint16_t* p_part;   // [B*N][N][128] fp16, MODE 2: the first launch's part of the output projection
  int* status;
};

// Epilogue backward. Inputs: tri [B*N][128][N] fp16 (times 2^-4), z and dy [B*N][N][128] bf16. Outputs:
//   dtri [B*N][128][N] fp16 = c * d loss / d t,  dxg [B*N][N][128] fp16 = c * (d loss / d x_hat through the output gate)
// and the per-CTA partials. Shared memory: W_out' , W_gate' (fp16, gamma folded), then four tiles: t, z, dy, dgate.
//
// MODE 0: the whole operator (128 contracted channels). MODE 1 / 2: the bidirectional module, whose output LayerNorm
// and projection span 256 channels held in two tensors; two launches with the statistics given (`ext_stats`):
//   MODE 1 (first tensor):  proj part = t_hat_1 Wo_1'^T + d_1 -> through map_dx (fp16); dproj; d t_hat_1 = dproj Wo_1'
//                           written raw through map_dt; its two LayerNorm-backward sums -> ln_part; Mo_1.
//   MODE 2 (second tensor): proj = part + t_hat_2 Wo_2'^T + d_2; dproj, dgate; d t_hat_2, dxg, Mo_2, Mg; the
//                           LayerNorm backward of its own 128 channels with the sums over all 256 (means -> ln_part);
//                           `bwd_ln_finish_kernel` then finishes the first tensor's gradient.
template <int MODE, int C = 128>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_epilogue_kernel(const __grid_constant__ CUtensorMap map_t, const __grid_constant__ CUtensorMap map_z,
                    const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_wo,
                    const __grid_constant__ CUtensorMap map_wg, const __grid_constant__ CUtensorMap map_dt,
                    const __grid_constant__ CUtensorMap map_dx, const BwdEpilogueParams p) {
  // C = d_pair: the channels of z, dy, dproj, dgate and the rows of both weight matrices (128, or 64 for the narrow pair
  // stacks; MODE 0 only). The contracted width (channels of t) is 128 in both cases.
  static_assert(C == 128 || (C == 64 && MODE == 0), "d_pair is 128, or 64 with one output tensor");
  constexpr int kZCh = C / kBwdParts;   // z-side channels per thread
  constexpr int kZChunks = kZCh / 8;
  constexpr int kZHalves = C / 64;      // 64-channel halves of a [pos][C] tile
  constexpr uint32_t kWHalf = C * 128;  // bytes of one 64-wide k half of a weight matrix with C rows
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t wo_s = smem_base, wg_s = smem_base + kBwdTile;
  const uint32_t tiles_s = smem_base + 2 * kBwdTile;  // four tile buffers whose roles rotate from tile to tile
  const uint32_t xchg = smem_base + 6 * kBwdTile;
  const uint32_t const_s = xchg + kBwdXchg;
  const uint32_t bar_base = const_s + 1024;
  const uint32_t w_full = bar_base, tz_full = bar_base + 8, mma_bar = bar_base + 16, dy_full = bar_base + 24;
  const uint32_t sums_done = bar_base + 48;  // every thread arrives once it has read the gradient tiles for the column sums
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 6 * kBwdTile + kBwdXchg + 1024 + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* const_ptr = reinterpret_cast<float*>(smem + 6 * kBwdTile + kBwdXchg);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = warp & 3, part = warp >> 2;
  const int pos = q * 32 + lane;
  const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    mbar_init(tz_full, 1);
    mbar_init(dy_full, 1);
    mbar_init(mma_bar, 1);
    mbar_init(sums_done, kBwdThreads);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_t);
    prefetch_tmap(&map_z);
    prefetch_tmap(&map_dy);
    prefetch_tmap(&map_dt);
    prefetch_tmap(&map_dx);
  }
  if (threadIdx.x < 256) const_ptr[threadIdx.x] = p.consts[threadIdx.x];
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const float gc = p.grad_scale[0];

  if (threadIdx.x == 0) {
    // Wo' [C, 128] as two k halves, Wg' [C, C] as C / 64 k halves
    mbar_arrive_expect_tx(w_full, (2 + kZHalves) * kWHalf);
#pragma unroll
    for (int kh = 0; kh < 2; ++kh) tma_load_2d(wo_s + kh * kWHalf, &map_wo, w_full, kh * 64, 0);
#pragma unroll
    for (int kh = 0; kh < kZHalves; ++kh) tma_load_2d(wg_s + kh * kWHalf, &map_wg, w_full, kh * 64, 0);
  }
  // Column sums of dproj and dgate (the bias / beta terms of the weight gradients): gathered from the fp16 tiles while
  // the gradient GEMMs run, this thread taking the 16-byte chunk `sum_chunk` (eight channels) of four position rows.
  const int sum_chunk = threadIdx.x & 15, sum_rows = (threadIdx.x >> 4) * 4;
  float acc_so[8], acc_sg[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc_so[c] = 0.f, acc_sg[c] = 0.f;

  // Buffer roles of tile `it`: t, z, dy, dgate = buffers (0, 1, 2, 3) for even it and (2, 3, 0, 1) for odd it. The
  // outputs of a tile are written over its t and z buffers and stored from there; its dy and dgate buffers are free
  // once the gradient GEMMs are done, and receive the next tile's t and z while this tile finishes. The next tile's dy
  // goes into this tile's t buffer as soon as the store has read it.
  auto issue_tz = [&](int tile_i, int it_i) {
    const int row_i = tile_i / p.tiles_per_row;
    const int j_i = (tile_i - row_i * p.tiles_per_row) * 128;
    const uint32_t t_i = tiles_s + ((it_i & 1) * 2) * kBwdTile, z_i = t_i + kBwdTile;
    mbar_arrive_expect_tx(tz_full, kBwdTile + kZHalves * 16384);
#pragma unroll
    for (int kh = 0; kh < 2; ++kh) tma_load_3d(t_i + kh * 16384, &map_t, tz_full, j_i + kh * 64, 0, row_i);
#pragma unroll
    for (int kh = 0; kh < kZHalves; ++kh) tma_load_3d(z_i + kh * 16384, &map_z, tz_full, kh * 64, j_i, row_i);
  };
  bool ok = true;
  int it = 0;
  int tz_pending = -1, dy_pending = -1;  // thread 0: iteration whose copies are in flight, or -1
  if (threadIdx.x == 0 && static_cast<int>(blockIdx.x) < p.num_tiles) {
    issue_tz(blockIdx.x, 0);
    tz_pending = 0;
  }
  for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
    const int row = tile / p.tiles_per_row;
    const int j0 = (tile - row * p.tiles_per_row) * 128;
    const uint32_t t_s = tiles_s + ((it & 1) * 2) * kBwdTile, z_s = t_s + kBwdTile;
    const uint32_t dy_s = tiles_s + (((it & 1) ^ 1) * 2) * kBwdTile, dg_s = dy_s + kBwdTile;
    if (it == 0) ok &= thread_wait(w_full, 0, abort_flag, p.status, kDevTimeoutMma);
    ok &= thread_wait(tz_full, it & 1, abort_flag, p.status, kDevTimeoutStats);
    if (threadIdx.x == 0) tz_pending = -1;
    // ---- phase 1: normalise t (rows = channels) and z (rows = positions) in place
    float rstd_out;
    if constexpr (MODE == 0) {
      rstd_out = normalise_tile<false, false>(t_s, xchg, pos, part, p.eps_out);
    } else {
      float2 st = make_float2(0.f, 0.f);
      if (j0 + pos < p.n) st = p.ext_stats[static_cast<size_t>(row) * p.n + j0 + pos];
      rstd_out = st.y;
      const float nmr = -st.x * st.y;
#pragma unroll 8
      for (int cc = 0; cc < kBwdCh; ++cc) {
        const uint32_t addr = t_s + tile_off(part * kBwdCh + cc, pos);
        st_f16_sat(addr, fmaf(ld_f16(addr), st.y, nmr));
      }
    }
    if (threadIdx.x == 0) {
      // this tile's dy and dgate buffers held the previous tile's outputs: their store (issued a normalisation pass
      // ago) must have read them before the dy copy lands there
      bulk_wait_read<0>();
      mbar_arrive_expect_tx(dy_full, kZHalves * 16384);
#pragma unroll
      for (int kh = 0; kh < kZHalves; ++kh) tma_load_3d(dy_s + kh * 16384, &map_dy, dy_full, kh * 64, j0, row);
      dy_pending = it;
    }
    normalise_tile<true, true, C>(z_s, xchg + kBwdXchgHalf, pos, part, p.eps_in);  // (the other exchange buffer)
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- phase 2: P = t_hat Wo'^T (columns 0-127), G = x_hat Wg'^T (columns 128-255)
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc_p = umma_idesc(128, C, true, false, kFmtF16, kFmtF16);
      constexpr uint32_t idesc_g = umma_idesc(128, C, false, false, kFmtF16, kFmtF16);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t kb = static_cast<uint64_t>((ks & 3) * 2);
        umma_bf16(tmem_base, umma_desc_mnmajor(t_s + ks * 2048, 16384), umma_desc_kmajor(wo_s + (ks >> 2) * kWHalf) + kb,
                  idesc_p, ks != 0 ? 1u : 0u);
      }
#pragma unroll
      for (int ks = 0; ks < C / 16; ++ks) {
        const uint64_t kb = static_cast<uint64_t>((ks & 3) * 2);
        umma_bf16(tmem_base + 128, umma_desc_kmajor(z_s + (ks >> 2) * 16384) + kb,
                  umma_desc_kmajor(wg_s + (ks >> 2) * kWHalf) + kb, idesc_g, ks != 0 ? 1u : 0u);
      }
      umma_commit(mma_bar);
    }
    // per-thread global operands of phase 3 (MODE 2: the first launch's part of the projection; the dropout scale),
    // requested before the waits
    const int j = j0 + pos;
    uint4 ppv[kZChunks], scv[kZChunks];
#pragma unroll
    for (int ch = 0; ch < kZChunks; ++ch) {
      ppv[ch] = make_uint4(0u, 0u, 0u, 0u);
      scv[ch] = make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);  // bf16 ones
    }
    if constexpr (MODE == 2) {
      if (j < p.n)
        ldg_chunks(reinterpret_cast<const uint4*>(p.p_part + (static_cast<size_t>(row) * p.n + j) * C + part * kZCh), true,
                   ppv);  // the workspace is 1024-byte aligned
    }
    if (p.drop_scale != nullptr && j < p.n) {
      const int b = row / p.n;
      ldg_chunks(reinterpret_cast<const uint4*>(p.drop_scale + (static_cast<size_t>(b) * p.n + j) * C + part * kZCh),
                 (reinterpret_cast<uintptr_t>(p.drop_scale) & 31u) == 0, scv);
    }
    ok &= thread_wait(mma_bar, 0, abort_flag, p.status, kDevTimeoutEpilogue);
    ok &= thread_wait(dy_full, it & 1, abort_flag, p.status, kDevTimeoutStats);
    if (threadIdx.x == 0) dy_pending = -1;
    tc_fence_after();
    // ---- phase 3: dproj = c du gate, dgate = c du proj gate (1 - gate); du = dy (* dropout scale)
    {
      uint32_t vp[kZChunks][8], vg[kZChunks][8];
#pragma unroll
      for (int ch = 0; ch < kZChunks; ++ch) {
        tmem_ld8(tmem_base + lane_sel + part * kZCh + ch * 8, vp[ch]);
        tmem_ld8(tmem_base + lane_sel + 128 + part * kZCh + ch * 8, vg[ch]);
      }
      tmem_ld_wait();
#pragma unroll
      for (int ch = 0; ch < kZChunks; ++ch) {
        const uint32_t addr = tile_chunk(pos, part * kZChunks + ch);
        const uint4 dyv = ld_chunk(dy_s + addr);
        float co[8], cg[8];  // the eight channels' constants (the same addresses for the whole warp)
        {
          const float4* cp = reinterpret_cast<const float4*>(const_ptr + part * kZCh + ch * 8);
          const float4 a0 = cp[0], a1 = cp[1], b0 = cp[32], b1 = cp[33];
          co[0] = a0.x, co[1] = a0.y, co[2] = a0.z, co[3] = a0.w, co[4] = a1.x, co[5] = a1.y, co[6] = a1.z, co[7] = a1.w;
          cg[0] = b0.x, cg[1] = b0.y, cg[2] = b0.z, cg[3] = b0.w, cg[4] = b1.x, cg[5] = b1.y, cg[6] = b1.z, cg[7] = b1.w;
        }
        const uint32_t pw[4] = {ppv[ch].x, ppv[ch].y, ppv[ch].z, ppv[ch].w};
        const uint32_t dw[4] = {dyv.x, dyv.y, dyv.z, dyv.w};
        const uint32_t sw[4] = {scv[ch].x, scv[ch].y, scv[ch].z, scv[ch].w};
        uint32_t op[4], og[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 d2 = bf16x2_to_float2(dw[t]);
          const float2 s2 = bf16x2_to_float2(sw[t]);
          const float2 p2 = f16x2_to_float2(pw[t]);
          float dpv[2], dgv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float proj = __uint_as_float(vp[ch][t * 2 + e]) + co[t * 2 + e] + (e == 0 ? p2.x : p2.y);
            const float gate = sigmoid_fast(__uint_as_float(vg[ch][t * 2 + e]) + cg[t * 2 + e]);
            const float du = (e == 0 ? d2.x * s2.x : d2.y * s2.y) * gc;
            dpv[e] = du * gate;
            dgv[e] = MODE == 1 ? proj : dpv[e] * fmaf(-proj, gate, proj);  // MODE 1 hands its part of proj on
          }
          op[t] = pack_f16x2_sat(make_float2(dpv[0], dpv[1]));
          og[t] = pack_f16x2_sat(make_float2(dgv[0], dgv[1]));
        }
        st_chunk(dy_s + addr, op[0], op[1], op[2], op[3]);
        // MODE 1: the part of proj leaves through the z buffer (x_hat is only needed by the G GEMM, which is done)
        st_chunk((MODE == 1 ? z_s : dg_s) + addr, og[0], og[1], og[2], og[3]);
        if constexpr (C == 64) {
          // the weight-gradient GEMMs read these tiles as 128-row operands: rows 64-127 (the second 64-channel block) are zero
          const uint32_t zaddr = tile_chunk(pos, 8 + part * kZChunks + ch);
          st_chunk(dy_s + zaddr, 0u, 0u, 0u, 0u);
          st_chunk(dg_s + zaddr, 0u, 0u, 0u, 0u);
        }
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    // ---- phase 4: dt_hat = dproj Wo' (0-127), dxg = dgate Wg' (128-255); Mo += dproj^T t_hat (256-383),
    //      Mg += dgate^T x_hat (384-511)
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc_d = umma_idesc(128, 128, false, true, kFmtF16, kFmtF16);   // d t_hat: N = 128
      constexpr uint32_t idesc_dx = umma_idesc(128, C, false, true, kFmtF16, kFmtF16);    // d x_hat: N = C
      constexpr uint32_t idesc_mo = umma_idesc(128, 128, true, false, kFmtF16, kFmtF16);
      constexpr uint32_t idesc_mg = umma_idesc(128, C, true, true, kFmtF16, kFmtF16);
      const uint32_t accum = it != 0 ? 1u : 0u;
#pragma unroll
      for (int ks = 0; ks < C / 16; ++ks) {  // K = the C channels of dproj; Wo' read MN-major: its k halves are the N blocks
        const uint64_t kb = static_cast<uint64_t>((ks & 3) * 2);
        umma_bf16(tmem_base, umma_desc_kmajor(dy_s + (ks >> 2) * 16384) + kb, umma_desc_mnmajor(wo_s + ks * 2048, kWHalf),
                  idesc_d, ks != 0 ? 1u : 0u);
      }
      if constexpr (MODE != 1) {
#pragma unroll
        for (int ks = 0; ks < C / 16; ++ks) {
          const uint64_t kb = static_cast<uint64_t>((ks & 3) * 2);
          umma_bf16(tmem_base + 128, umma_desc_kmajor(dg_s + (ks >> 2) * 16384) + kb,
                    umma_desc_mnmajor(wg_s + ks * 2048, kWHalf), idesc_dx, ks != 0 ? 1u : 0u);
        }
      }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t kb = static_cast<uint64_t>((ks & 3) * 2);
        umma_bf16(tmem_base + 256, umma_desc_mnmajor(dy_s + ks * 2048, 16384),
                  umma_desc_kmajor(t_s + (ks >> 2) * 16384) + kb, idesc_mo, (ks != 0 ? 1u : 0u) | accum);
      }
      if constexpr (MODE != 1) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          umma_bf16(tmem_base + 384, umma_desc_mnmajor(dg_s + ks * 2048, 16384), umma_desc_mnmajor(z_s + ks * 2048, 16384),
                    idesc_mg, (ks != 0 ? 1u : 0u) | accum);
        }
      }
      umma_commit(mma_bar);
    }
    if (sum_chunk < C / 8) {  // column sums of the two fp16 tiles the GEMMs are reading
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const uint32_t addr = tile_chunk(sum_rows + r, sum_chunk);
        const uint4 a = ld_chunk(dy_s + addr);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 x = f16x2_to_float2(aw[t]);
          acc_so[2 * t] += x.x, acc_so[2 * t + 1] += x.y;
        }
        if constexpr (MODE != 1) {
          const uint4 b = ld_chunk(dg_s + addr);
          const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 x = f16x2_to_float2(bw[t]);
            acc_sg[2 * t] += x.x, acc_sg[2 * t + 1] += x.y;
          }
        }
      }
    }
    mbar_arrive(sums_done);
    ok &= thread_wait(mma_bar, 1, abort_flag, p.status, kDevTimeoutEpilogue);
    tc_fence_after();
    if (threadIdx.x == 0 && tile + static_cast<int>(gridDim.x) < p.num_tiles) {
      // into this tile's dy and dgate buffers: the GEMMs have finished with them, and so must every thread's column sums
      ok &= thread_wait(sums_done, it & 1, abort_flag, p.status, kDevTimeoutEpilogue);
      issue_tz(tile + gridDim.x, it + 1);
      tz_pending = it + 1;
    }
    // ---- phase 5: LayerNorm backward of the output normalisation, in place over t_hat; dxg over x_hat
    {
      const bool inside = j0 + pos < p.n;
      float2 other = make_float2(0.f, 0.f);  // MODE 2: the first launch's sums (read before the barrier below)
      if constexpr (MODE == 2) {
        if (inside) other = p.ln_part[static_cast<size_t>(row) * p.n + j0 + pos];
      }
      float s1 = 0.f, s2 = 0.f;
      float th[kBwdCh];                 // this thread's t_hat values and its d t_hat, both kept for the second pass
      uint32_t dtv[kBwdChunks][8];
#pragma unroll
      for (int ch = 0; ch < kBwdChunks; ++ch) tmem_ld8(tmem_base + lane_sel + part * kBwdCh + ch * 8, dtv[ch]);
#pragma unroll
      for (int cc = 0; cc < kBwdCh; ++cc) th[cc] = ld_f16(t_s + tile_off(part * kBwdCh + cc, pos));
      tmem_ld_wait();
#pragma unroll
      for (int ch = 0; ch < kBwdChunks; ++ch) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float d = __uint_as_float(dtv[ch][e]);
          s1 += d;
          s2 = fmaf(d, th[ch * 8 + e], s2);
        }
      }
      asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xchg + (part * 128 + pos) * 8), "f"(s1), "f"(s2) : "memory");
      named_bar_sync(1, kBwdThreads);
      float m1, m2;
      sum_partials(xchg, pos, m1, m2);
      if constexpr (MODE == 1) {
        if (part == 0 && inside) p.ln_part[static_cast<size_t>(row) * p.n + j0 + pos] = make_float2(m1, m2);
      } else if constexpr (MODE == 2) {
        m1 = (m1 + other.x) * (1.0f / 256.0f), m2 = (m2 + other.y) * (1.0f / 256.0f);
        if (part == 0 && inside) p.ln_part[static_cast<size_t>(row) * p.n + j0 + pos] = make_float2(m1, m2);
      } else {
        m1 *= 1.0f / 128.0f, m2 *= 1.0f / 128.0f;
      }
      const float rs = rstd_out * 0.0625f;  // d / d t of the stored t / 16
#pragma unroll
      for (int ch = 0; ch < kBwdChunks; ++ch) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t addr = t_s + tile_off(part * kBwdCh + ch * 8 + e, pos);
          if constexpr (MODE == 1) st_f16_sat(addr, __uint_as_float(dtv[ch][e]));  // finished by bwd_ln_finish_kernel
          else st_f16_sat(addr, rs * (__uint_as_float(dtv[ch][e]) - m1 - th[ch * 8 + e] * m2));
        }
      }
      if constexpr (MODE != 1) {
        uint32_t xg[kZChunks][8];
#pragma unroll
        for (int ch = 0; ch < kZChunks; ++ch) tmem_ld8(tmem_base + lane_sel + 128 + part * kZCh + ch * 8, xg[ch]);
        tmem_ld_wait();
#pragma unroll
        for (int ch = 0; ch < kZChunks; ++ch) {
          const uint32_t(&x)[8] = xg[ch];
          st_chunk(z_s + tile_chunk(pos, part * kZChunks + ch),
                   pack_f16x2_sat(make_float2(__uint_as_float(x[0]), __uint_as_float(x[1]))),
                   pack_f16x2_sat(make_float2(__uint_as_float(x[2]), __uint_as_float(x[3]))),
                   pack_f16x2_sat(make_float2(__uint_as_float(x[4]), __uint_as_float(x[5]))),
                   pack_f16x2_sat(make_float2(__uint_as_float(x[6]), __uint_as_float(x[7]))));
        }
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    ok = __syncthreads_and(ok ? 1 : 0) != 0;  // a thread that gave up takes the whole CTA out here
    if (!ok) break;
    if (threadIdx.x == 0) {
#pragma unroll
      for (int kh = 0; kh < 2; ++kh)
        if (j0 + kh * 64 < p.n) tma_store_3d(&map_dt, t_s + kh * 16384, j0 + kh * 64, 0, row);
#pragma unroll
      for (int kh = 0; kh < kZHalves; ++kh) tma_store_3d(&map_dx, z_s + kh * 16384, kh * 64, j0, row);
      bulk_commit();
    }
  }
  if (threadIdx.x == 0) {
    if (!ok) {  // a wait gave up: copies in flight must land before the CTA exits
      const long long t0 = clock64();
      while (!mbar_try_wait(w_full, 0) || (tz_pending >= 0 && !mbar_try_wait(tz_full, tz_pending & 1)) ||
             (dy_pending >= 0 && !mbar_try_wait(dy_full, dy_pending & 1))) {
        if (clock64() - t0 > kWaitLimitCycles) {
          atomicCAS(p.status, 0, kDevTimeoutDrain);
          break;
        }
      }
    }
    bulk_wait<0>();
  }
  __syncthreads();
  if (ok && it > 0) {
    // weight-gradient accumulators: lane = output row of the matrix, this thread's 64 columns
    tc_fence_after();
    float* pm = p.part_m + static_cast<size_t>(blockIdx.x) * 2 * 128 * 128;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
      for (int ch = 0; ch < kBwdChunks; ++ch) {
        uint32_t v[8];
        tmem_ld8(tmem_base + lane_sel + 256 + m * 128 + part * kBwdCh + ch * 8, v);
        tmem_ld_wait();
        float4* dst = reinterpret_cast<float4*>(pm + (m * 128 + pos) * 128 + part * kBwdCh + ch * 8);
        dst[0] = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]), __uint_as_float(v[3]));
        dst[1] = make_float4(__uint_as_float(v[4]), __uint_as_float(v[5]), __uint_as_float(v[6]), __uint_as_float(v[7]));
      }
    }
  }
  {  // the 32 row groups of a channel, fixed order; every tile region is free by now
    float* sc = reinterpret_cast<float*>(smem);  // [32 row groups][2][128]
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      sc[((threadIdx.x >> 4) * 2 + 0) * 128 + sum_chunk * 8 + c] = acc_so[c];
      sc[((threadIdx.x >> 4) * 2 + 1) * 128 + sum_chunk * 8 + c] = acc_sg[c];
    }
    __syncthreads();
    if (threadIdx.x < 256 && (threadIdx.x & 127) < C) {
      float sum = 0.f;
      for (int g = 0; g < 32; ++g) sum += sc[g * 256 + threadIdx.x];
      p.part_s[static_cast<size_t>(blockIdx.x) * 2 * 128 + threadIdx.x] = sum;
    }
    __syncthreads();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Mean and rstd of the stored t over the 256 channels of two tensors [rows][128][N] (fp16), one thread per row and
// group of eight columns: stats[row][j] = {mean, rsqrt(var + eps)} (eps already scaled like the stored t). Eight
// channels' loads are in flight per thread.
__global__ void __launch_bounds__(256) bwd_ln_stats_kernel(const uint4* t0, const uint4* t1, int n, long long groups, float eps,
                                                           float2* stats) {
  const long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (g >= groups) return;
  const int per_row = n / 8;
  const long long row = g / per_row;
  const int jc = static_cast<int>(g - row * per_row);
  float pv[8], s1[8], s2[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) pv[e] = 0.f, s1[e] = 0.f, s2[e] = 0.f;
  for (int c0 = 0; c0 < 256; c0 += 8) {
    const uint4* src = (c0 < 128 ? t0 : t1) + (row * 128 + (c0 & 127)) * per_row + jc;
    uint4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = __ldg(src + static_cast<long long>(k) * per_row);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 x = f16x2_to_float2(w[t]);
        if (c0 == 0 && k == 0) pv[2 * t] = x.x, pv[2 * t + 1] = x.y;
        const float d0 = x.x - pv[2 * t], d1 = x.y - pv[2 * t + 1];
        s1[2 * t] += d0, s1[2 * t + 1] += d1;
        s2[2 * t] = fmaf(d0, d0, s2[2 * t]), s2[2 * t + 1] = fmaf(d1, d1, s2[2 * t + 1]);
      }
    }
  }
  float4* dst = reinterpret_cast<float4*>(stats + row * n + jc * 8);  // 64-byte aligned: n is a multiple of 8
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    float m[2], r[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      m[u] = pv[e + u] + s1[e + u] * (1.0f / 256.0f);
      const float var = fmaxf(s2[e + u] - s1[e + u] * s1[e + u] * (1.0f / 256.0f), 0.f) * (1.0f / 256.0f);
      r[u] = rsqrtf(var + eps);
    }
    dst[e >> 1] = make_float4(m[0], r[0], m[1], r[1]);
  }
}

// Finishes the first tensor's gradient of the 256-channel LayerNorm backward, in place over the raw d t_hat the MODE 1
// launch left in dt [rows][128][N] (fp16, times c): dt = rstd / 16 * (d t_hat - m1 - t_hat m2), t_hat recomputed from t.
// One thread per row, group of eight columns and group of 16 channels: the eight positions' statistics are read once.
constexpr int kLnFinishChannels = 16;
__global__ void __launch_bounds__(256) bwd_ln_finish_kernel(uint4* dt, const uint4* t, const float2* stats, const float2* means,
                                                            int n, long long threads) {
  const long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (g >= threads) return;
  const int per_row = n / 8;
  const long long rg = g / per_row;  // row * (128 / kLnFinishChannels) + channel group
  const int jc = static_cast<int>(g - rg * per_row);
  const long long row = rg / (128 / kLnFinishChannels);
  const int c_first = static_cast<int>(rg - row * (128 / kLnFinishChannels)) * kLnFinishChannels;
  float mean[8], k0[8], k1[8], m1[8];
  {
    const float4* sp = reinterpret_cast<const float4*>(stats + row * n + jc * 8);
    const float4* mp = reinterpret_cast<const float4*>(means + row * n + jc * 8);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 st = __ldg(sp + q), mm = __ldg(mp + q);
      mean[2 * q] = st.x, k0[2 * q] = st.y * 0.0625f, k1[2 * q] = st.y * mm.y, m1[2 * q] = mm.x;
      mean[2 * q + 1] = st.z, k0[2 * q + 1] = st.w * 0.0625f, k1[2 * q + 1] = st.w * mm.w, m1[2 * q + 1] = mm.z;
    }
  }
  const long long base = (row * 128 + c_first) * per_row + jc;
#pragma unroll
  for (int c0 = 0; c0 < kLnFinishChannels; c0 += 4) {
    uint4 dv[4], tv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      dv[k] = dt[base + static_cast<long long>(c0 + k) * per_row];
      tv[k] = __ldg(t + base + static_cast<long long>(c0 + k) * per_row);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t dw[4] = {dv[k].x, dv[k].y, dv[k].z, dv[k].w}, tw[4] = {tv[k].x, tv[k].y, tv[k].z, tv[k].w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 d = f16x2_to_float2(dw[q]);
        const float2 x = f16x2_to_float2(tw[q]);
        const float r0 = k0[2 * q] * (d.x - m1[2 * q] - (x.x - mean[2 * q]) * k1[2 * q]);
        const float r1 = k0[2 * q + 1] * (d.y - m1[2 * q + 1] - (x.y - mean[2 * q + 1]) * k1[2 * q + 1]);
        o[q] = pack_f16x2_sat(make_float2(r0, r1));
      }
      dt[base + static_cast<long long>(c0 + k) * per_row] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

struct BwdPrologueParams {
  int tiles_per_row;
  int num_tiles;
  int n;
  const float* consts;        // [2][128]: d_value = W beta_in + bias, d_gate likewise (this side's two matrices)
  const float* grad_scale;    // [2]: c, 1 / c
  const uint8_t* token_mask;  // [B][N] or null
  const uint8_t* pair_mask;   // [B][N][N] or null
  const uint16_t* dx_in;      // [B*N][N][128] fp16: c * d loss / d x_hat gathered so far (read)
  const uint16_t* dy;         // LAST only: upstream gradient [B*N][N][128] bf16 (the residual path), or null
  float eps_in;
  float* part_m;              // [grid][2][128][128]: partial dvalue^T x_hat, dgate^T x_hat
  float* part_s;              // [grid][2][128]
  int* status;
};

// Prologue backward for one side (left or right). Inputs: z [B*N][N][128] bf16, dO = the contraction's gradient for
// this side [B*N][128][N] fp16 (times c / 16). It recomputes value / gate, forms dvalue = dO sig m, dgate = dO value
// sig (1 - sig) m, adds dvalue W_v' + dgate W_g' to the running d x_hat, and accumulates the two weight gradients.
// !LAST: the running d x_hat (fp16, times c) is written back through map_out. LAST: the input LayerNorm's backward
// and the residual finish d loss / d z (bf16, unscaled) through map_out.
template <bool LAST, int C = 128>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_prologue_kernel(const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_do,
                    const __grid_constant__ CUtensorMap map_wv, const __grid_constant__ CUtensorMap map_wg,
                    const __grid_constant__ CUtensorMap map_out, const BwdPrologueParams p) {
  // C = d_pair: the channels of z, d x_hat, dz and the columns of both weight matrices (128, or 64 for the narrow pair
  // stacks). The contracted width (channels of dO, rows of the weight matrices) is 128 in both cases.
  static_assert(C == 128 || C == 64, "d_pair is 128 or 64");
  constexpr int kZCh = C / kBwdParts;   // z-side channels per thread
  constexpr int kZChunks = kZCh / 8;
  constexpr int kZHalves = C / 64;      // 64-channel halves of a [pos][C] tile = k halves of a [128][C] weight matrix
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t wv_s = smem_base, wg_s = smem_base + kBwdTile;
  const uint32_t tiles_s = smem_base + 2 * kBwdTile;  // four tile buffers whose roles rotate from tile to tile
  const uint32_t xchg = smem_base + 6 * kBwdTile;
  const uint32_t const_s = xchg + kBwdXchg;
  const uint32_t bar_base = const_s + 1024;
  const uint32_t w_full = bar_base, z_full = bar_base + 8, mma_bar = bar_base + 16, do_full = bar_base + 24;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 6 * kBwdTile + kBwdXchg + 1024 + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = warp & 3, part = warp >> 2;
  const int pos = q * 32 + lane;
  const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    mbar_init(z_full, 1);   // a tile's z and dO copies are issued and awaited at different times
    mbar_init(do_full, 1);
    mbar_init(mma_bar, 2);  // two issuing threads commit to it in every GEMM round
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_z);
    prefetch_tmap(&map_do);
    prefetch_tmap(&map_out);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const float gc_inv = p.grad_scale[1];
  const float c_value = p.consts[pos], c_gate_half = 0.5f * p.consts[128 + pos];  // this thread's channel

  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(w_full, 2 * kZHalves * 16384);
#pragma unroll
    for (int kh = 0; kh < kZHalves; ++kh) {
      tma_load_2d(wv_s + kh * 16384, &map_wv, w_full, kh * 64, 0);
      tma_load_2d(wg_s + kh * 16384, &map_wg, w_full, kh * 64, 0);
    }
  }
  // Phases 2-3 work on the transposed projections (TMEM lanes = contracted channels, columns = positions): a thread
  // owns channel `pos` (its lane) and the position quarter `part`, so its constants and its column sums are scalars
  // and dO, stored [channel][position], is read in 16-byte runs of positions.
  float acc_sv = 0.f, acc_sg = 0.f;
  // validity of a tile's positions, one bit each: [2][4] words (tile parity, 32 positions per word). The mask bytes of
  // the NEXT tile are requested by the first four warps before a GEMM wait and turned into the words after it, so that
  // their latency is off the path.
  uint32_t* valid_words = reinterpret_cast<uint32_t*>(smem + 6 * kBwdTile + kBwdXchg + 1024 + 64);
  auto mask_bytes = [&](int tile_i, bool& in_range, uint32_t& m_i, uint32_t& m_j, uint32_t& m_p) {
    const int row_i = tile_i / p.tiles_per_row;
    const int j_i = (tile_i - row_i * p.tiles_per_row) * 128 + pos;
    const int b = row_i / p.n;
    const int i = row_i - b * p.n;
    in_range = j_i < p.n;
    m_i = 1u, m_j = 1u, m_p = 1u;
    if (in_range) {
      if (p.token_mask != nullptr) {
        m_i = p.token_mask[static_cast<size_t>(b) * p.n + i];
        m_j = p.token_mask[static_cast<size_t>(b) * p.n + j_i];
      }
      if (p.pair_mask != nullptr) m_p = p.pair_mask[(static_cast<size_t>(b) * p.n + i) * p.n + j_i];
    }
  };
  auto publish_valid = [&](int it_i, bool in_range, uint32_t m_i, uint32_t m_j, uint32_t m_p) {
    const uint32_t word = __ballot_sync(0xFFFFFFFFu, in_range && m_i != 0u && m_j != 0u && m_p != 0u);
    if (lane == 0) valid_words[(it_i & 1) * 4 + q] = word;
  };

  // Buffer roles (z, dO, dvalue, dgate) of tile `it`, one nibble each, period 4: the next tile's z and dO are copied
  // into this tile's dO buffer (free after phase 3) and dgate buffer (free after the gradient GEMMs) while this tile
  // finishes; its dvalue scratch is this tile's z buffer and its dgate scratch this tile's dvalue buffer, which holds
  // the output until the store has read it.
  auto role = [&](int it_i, int r) {
    const uint32_t rr = static_cast<uint32_t>(0x1302012320313210ull >> (16 * (it_i & 3))) & 0xFFFFu;
    return tiles_s + ((rr >> (4 * r)) & 0xFu) * kBwdTile;
  };
  auto issue_z = [&](int tile_i, int it_i) {
    const int row_i = tile_i / p.tiles_per_row;
    const int j_i = (tile_i - row_i * p.tiles_per_row) * 128;
    const uint32_t z_i = role(it_i, 0);
    mbar_arrive_expect_tx(z_full, kZHalves * 16384);
#pragma unroll
    for (int kh = 0; kh < kZHalves; ++kh) tma_load_3d(z_i + kh * 16384, &map_z, z_full, kh * 64, j_i, row_i);
  };
  auto issue_do = [&](int tile_i, int it_i) {
    const int row_i = tile_i / p.tiles_per_row;
    const int j_i = (tile_i - row_i * p.tiles_per_row) * 128;
    const uint32_t do_i = role(it_i, 1);
    mbar_arrive_expect_tx(do_full, kBwdTile);
#pragma unroll
    for (int kh = 0; kh < 2; ++kh) tma_load_3d(do_i + kh * 16384, &map_do, do_full, j_i + kh * 64, 0, row_i);
  };
  // The single-thread jobs of a tile sit on three different warps so that they do not queue behind one another: the MMA
  // issue (threads 0 and 32), the TMA loads of the next tile (thread 96) and the TMA store with its bulk group (thread 64).
  const bool load_thread = threadIdx.x == 96, store_thread = threadIdx.x == 64;
  // tile -> (row, column block) without a division per tile
  const int step_rows = static_cast<int>(gridDim.x) / p.tiles_per_row;
  const int step_cols = static_cast<int>(gridDim.x) - step_rows * p.tiles_per_row;
  int row = static_cast<int>(blockIdx.x) / p.tiles_per_row;
  int jt = static_cast<int>(blockIdx.x) - row * p.tiles_per_row;
  bool ok = true;
  int it = 0;
  int z_pending = -1, do_pending = -1;  // load thread: iteration whose copy is in flight, or -1
  if (load_thread && static_cast<int>(blockIdx.x) < p.num_tiles) {
    issue_z(blockIdx.x, 0);
    issue_do(blockIdx.x, 0);
    z_pending = 0, do_pending = 0;
  }
  if (part == 0 && static_cast<int>(blockIdx.x) < p.num_tiles) {
    bool in0;
    uint32_t a0, b0, c0;
    mask_bytes(blockIdx.x, in0, a0, b0, c0);
    publish_valid(0, in0, a0, b0, c0);
  }
  for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
    if (it != 0) {
      row += step_rows, jt += step_cols;
      if (jt >= p.tiles_per_row) jt -= p.tiles_per_row, ++row;
    }
    const int j0 = jt * 128;
    const uint32_t z_s = role(it, 0), do_s = role(it, 1), dv_s = role(it, 2), dg_s = role(it, 3);
    const int j = j0 + pos;
    if (it == 0) ok &= thread_wait(w_full, 0, abort_flag, p.status, kDevTimeoutMma);
    ok &= thread_wait(z_full, it & 1, abort_flag, p.status, kDevTimeoutStats);
    if (load_thread) z_pending = -1;
    // ---- phase 1: x_hat in place
    const float rstd_in = normalise_tile<true, true, C>(z_s, xchg, pos, part, p.eps_in);
    // this tile's dgate scratch held the previous tile's output: its store must have read it before phase 3 (the
    // barrier that closes phase 1 orders this wait before every thread's phase 3)
    if (store_thread) bulk_wait_read<0>();
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- phase 2: value^T = Wv' x_hat^T (columns 0-127), gate^T = Wg' x_hat^T (128-255): lanes = contracted channels
    // (the GEMMs of a round are issued by two threads, one per accumulator group: one thread's issue rate does not
    // keep the tensor pipe busy)
    if (threadIdx.x == 0 || threadIdx.x == 32) {
      const int m = threadIdx.x >> 5;
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc(128, 128, false, false, kFmtF16, kFmtF16);
#pragma unroll
      for (int ks = 0; ks < C / 16; ++ks) {
        const uint64_t kb = static_cast<uint64_t>((ks & 3) * 2);
        umma_bf16(tmem_base + m * 128, umma_desc_kmajor((m == 0 ? wv_s : wg_s) + (ks >> 2) * 16384) + kb,
                  umma_desc_kmajor(z_s + (ks >> 2) * 16384) + kb, idesc, ks != 0 ? 1u : 0u);
      }
      umma_commit(mma_bar);
    }
    bool nx_in = false;
    uint32_t nx_i = 1u, nx_j = 1u, nx_p = 1u;
    const bool has_next = tile + static_cast<int>(gridDim.x) < p.num_tiles;
    if (part == 0 && has_next) mask_bytes(tile + gridDim.x, nx_in, nx_i, nx_j, nx_p);
    ok &= thread_wait(mma_bar, 0, abort_flag, p.status, kDevTimeoutEpilogue);
    tc_fence_after();
    if (part == 0 && has_next) publish_valid(it + 1, nx_in, nx_i, nx_j, nx_p);
    ok &= thread_wait(do_full, it & 1, abort_flag, p.status, kDevTimeoutStats);
    if (load_thread) do_pending = -1;
    // ---- phase 3: dvalue, dgate for this thread's channel and 32 positions, stored [channel][position]
    {
      const uint32_t vbits = valid_words[(it & 1) * 4 + part];
      uint32_t vv[32], vg[32];
      tmem_ld32(tmem_base + lane_sel + part * 32, vv);
      tmem_ld32(tmem_base + lane_sel + 128 + part * 32, vg);
      uint4 dov[4];
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) dov[k4] = ld_chunk(do_s + tile_chunk(pos, part * 4 + k4));
      tmem_ld_wait();
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        const uint32_t dw[4] = {dov[k4].x, dov[k4].y, dov[k4].z, dov[k4].w};
        uint32_t ov[4], og[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float2 d_o = f16x2_to_float2(dw[t]);
          const int e0 = k4 * 8 + 2 * t;
          if (vbits != 0xFFFFFFFFu) {
            d_o.x = ((vbits >> e0) & 1u) ? d_o.x : 0.f;
            d_o.y = ((vbits >> (e0 + 1)) & 1u) ? d_o.y : 0.f;
          }
          float dv2[2], dg2[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const float val = __uint_as_float(vv[e0 + u]) + c_value;
            const float th = tanh_approx(fmaf(__uint_as_float(vg[e0 + u]), 0.5f, c_gate_half));
            const float sg = fmaf(th, 0.5f, 0.5f);
            const float sg16 = fmaf(th, 8.0f, 8.0f);  // the contraction's outputs are stored times 2^-4
            dv2[u] = (u == 0 ? d_o.x : d_o.y) * sg16;
            dg2[u] = dv2[u] * fmaf(-val, sg, val);
            acc_sv += dv2[u];
            acc_sg += dg2[u];
          }
          ov[t] = pack_f16x2_sat(make_float2(dv2[0], dv2[1]));
          og[t] = pack_f16x2_sat(make_float2(dg2[0], dg2[1]));
        }
        const uint32_t addr = tile_chunk(pos, part * 4 + k4);
        st_chunk(dv_s + addr, ov[0], ov[1], ov[2], ov[3]);
        st_chunk(dg_s + addr, og[0], og[1], og[2], og[3]);
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (load_thread && tile + static_cast<int>(gridDim.x) < p.num_tiles) {
      issue_z(tile + gridDim.x, it + 1);  // into this tile's dO buffer, read for the last time in phase 3
      z_pending = it + 1;
    }
    // ---- phase 4: d x_hat = dvalue Wv' + dgate Wg' (columns 0-127, lanes = positions); Mv += dvalue^T x_hat (256-383),
    // Mg += dgate^T x_hat (384-511). dvalue / dgate are [channel][position] tiles: MN-major as the A operand of the
    // first pair of GEMMs (M = positions), K-major as that of the second (M = channels, K = positions).
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc_d = umma_idesc(128, C, true, true, kFmtF16, kFmtF16);
#pragma unroll
      for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          umma_bf16(tmem_base, umma_desc_mnmajor((m == 0 ? dv_s : dg_s) + ks * 2048, 16384),
                    umma_desc_mnmajor((m == 0 ? wv_s : wg_s) + ks * 2048, 16384), idesc_d, (m | ks) != 0 ? 1u : 0u);
        }
      }
      umma_commit(mma_bar);
    } else if (threadIdx.x == 32) {
      tc_fence_after();
      constexpr uint32_t idesc_m = umma_idesc(128, C, false, true, kFmtF16, kFmtF16);
      const uint32_t accum = it != 0 ? 1u : 0u;
#pragma unroll
      for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t kb = static_cast<uint64_t>((ks & 3) * 2);
          umma_bf16(tmem_base + 256 + m * 128, umma_desc_kmajor((m == 0 ? dv_s : dg_s) + (ks >> 2) * 16384) + kb,
                    umma_desc_mnmajor(z_s + ks * 2048, 16384), idesc_m, (ks != 0 ? 1u : 0u) | accum);
        }
      }
      umma_commit(mma_bar);
    }
    // the running d x_hat of this thread's channels: requested now, used after the GEMM round
    const bool inside = j < p.n;
    uint4 dx_prev[kZChunks];
#pragma unroll
    for (int ch = 0; ch < kZChunks; ++ch) dx_prev[ch] = make_uint4(0u, 0u, 0u, 0u);
    if (inside) {
      const uint4* src = reinterpret_cast<const uint4*>(p.dx_in + (static_cast<size_t>(row) * p.n + j) * C + part * kZCh);
      ldg_chunks(src, true, dx_prev);  // the workspace is 1024-byte aligned
    }
    uint4 dy_res[LAST ? kZChunks : 2];  // LAST: the residual branch's share of dz, requested at the same time
    if constexpr (LAST) {
#pragma unroll
      for (int ch = 0; ch < kZChunks; ++ch) dy_res[ch] = make_uint4(0u, 0u, 0u, 0u);
      if (p.dy != nullptr && inside) {
        const uint4* dyp = reinterpret_cast<const uint4*>(p.dy + (static_cast<size_t>(row) * p.n + j) * C + part * kZCh);
        ldg_chunks(dyp, (reinterpret_cast<uintptr_t>(p.dy) & 31u) == 0, dy_res);
      }
    }
    ok &= thread_wait(mma_bar, 1, abort_flag, p.status, kDevTimeoutEpilogue);
    tc_fence_after();
    if (load_thread && tile + static_cast<int>(gridDim.x) < p.num_tiles) {
      issue_do(tile + gridDim.x, it + 1);  // into this tile's dgate buffer, free once the gradient GEMMs are done
      do_pending = it + 1;
    }
    // ---- phase 5: add the running d x_hat; !LAST: write it back, LAST: LayerNorm backward + residual -> dz
    {
      float tot[kZCh];
      float s1 = 0.f, s2 = 0.f;
      uint32_t vt[kZChunks][8];
#pragma unroll
      for (int ch = 0; ch < kZChunks; ++ch) tmem_ld8(tmem_base + lane_sel + part * kZCh + ch * 8, vt[ch]);
      tmem_ld_wait();
#pragma unroll
      for (int ch = 0; ch < kZChunks; ++ch) {
        const uint32_t(&v)[8] = vt[ch];
        const uint4 in = dx_prev[ch];
        uint4 xh = make_uint4(0u, 0u, 0u, 0u);
        if constexpr (LAST) xh = ld_chunk(z_s + tile_chunk(pos, part * kZChunks + ch));
        const uint32_t iw[4] = {in.x, in.y, in.z, in.w};
        const uint32_t xw[4] = {xh.x, xh.y, xh.z, xh.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 a = f16x2_to_float2(iw[t]);
          const float t0 = __uint_as_float(v[2 * t]) + a.x, t1 = __uint_as_float(v[2 * t + 1]) + a.y;
          tot[ch * 8 + 2 * t] = t0;
          tot[ch * 8 + 2 * t + 1] = t1;
          if constexpr (LAST) {
            const float2 x = f16x2_to_float2(xw[t]);
            s1 += t0 + t1;
            s2 = fmaf(t0, x.x, fmaf(t1, x.y, s2));
          }
        }
      }
      if constexpr (!LAST) {
#pragma unroll
        for (int ch = 0; ch < kZChunks; ++ch)
          st_chunk(dv_s + tile_chunk(pos, part * kZChunks + ch), pack_f16x2_sat(make_float2(tot[ch * 8], tot[ch * 8 + 1])),
                   pack_f16x2_sat(make_float2(tot[ch * 8 + 2], tot[ch * 8 + 3])),
                   pack_f16x2_sat(make_float2(tot[ch * 8 + 4], tot[ch * 8 + 5])),
                   pack_f16x2_sat(make_float2(tot[ch * 8 + 6], tot[ch * 8 + 7])));
      } else {
        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xchg + kBwdXchgHalf + (part * 128 + pos) * 8), "f"(s1), "f"(s2)
                     : "memory");
        named_bar_sync(1, kBwdThreads);
        float m1, m2;
        sum_partials(xchg + kBwdXchgHalf, pos, m1, m2);
        m1 *= 1.0f / C, m2 *= 1.0f / C;
        const float rs = rstd_in * gc_inv;
#pragma unroll
        for (int ch = 0; ch < kZChunks; ++ch) {
          const uint4 xh = ld_chunk(z_s + tile_chunk(pos, part * kZChunks + ch));
          const uint4 dyv = dy_res[ch];
          const uint32_t xw[4] = {xh.x, xh.y, xh.z, xh.w};
          const uint32_t dw[4] = {dyv.x, dyv.y, dyv.z, dyv.w};
          uint32_t o[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 x = f16x2_to_float2(xw[t]);
            const float2 r = bf16x2_to_float2(dw[t]);
            o[t] = pack_bf16x2(fmaf(rs, tot[ch * 8 + 2 * t] - m1 - x.x * m2, r.x),
                               fmaf(rs, tot[ch * 8 + 2 * t + 1] - m1 - x.y * m2, r.y));
          }
          st_chunk(dv_s + tile_chunk(pos, part * kZChunks + ch), o[0], o[1], o[2], o[3]);
        }
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    ok = __syncthreads_and(ok ? 1 : 0) != 0;  // a thread that gave up takes the whole CTA out here
    if (!ok) break;
    if (store_thread) {
#pragma unroll
      for (int kh = 0; kh < kZHalves; ++kh) tma_store_3d(&map_out, dv_s + kh * 16384, kh * 64, j0, row);
      bulk_commit();
    }
  }
  if (store_thread) bulk_wait<0>();
  if (load_thread) {
    if (!ok) {  // a wait gave up: copies in flight must land before the CTA exits
      const long long t0 = clock64();
      while (!mbar_try_wait(w_full, 0) || (z_pending >= 0 && !mbar_try_wait(z_full, z_pending & 1)) ||
             (do_pending >= 0 && !mbar_try_wait(do_full, do_pending & 1))) {
        if (clock64() - t0 > kWaitLimitCycles) {
          atomicCAS(p.status, 0, kDevTimeoutDrain);
          break;
        }
      }
    }
  }
  __syncthreads();
  if (ok && it > 0) {
    tc_fence_after();
    float* pm = p.part_m + static_cast<size_t>(blockIdx.x) * 2 * 128 * 128;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
      for (int ch = 0; ch < kBwdChunks; ++ch) {
        uint32_t v[8];
        tmem_ld8(tmem_base + lane_sel + 256 + m * 128 + part * kBwdCh + ch * 8, v);
        tmem_ld_wait();
        float4* dst = reinterpret_cast<float4*>(pm + (m * 128 + pos) * 128 + part * kBwdCh + ch * 8);
        dst[0] = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]), __uint_as_float(v[3]));
        dst[1] = make_float4(__uint_as_float(v[4]), __uint_as_float(v[5]), __uint_as_float(v[6]), __uint_as_float(v[7]));
      }
    }
  }
  {  // column sums: the four position quarters of a channel, fixed order
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xchg + (part * 128 + pos) * 8), "f"(acc_sv), "f"(acc_sg) : "memory");
    __syncthreads();
    if (threadIdx.x < 128) {
      float a, b;
      sum_partials(xchg, threadIdx.x, a, b);
      float* ps = p.part_s + static_cast<size_t>(blockIdx.x) * 2 * 128;
      ps[threadIdx.x] = a;
      ps[128 + threadIdx.x] = b;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------ small kernels
// Largest |dy| (bf16) as the bits of a non-negative float: `amax_bits` must be zero before the launch.
__global__ void __launch_bounds__(256) bwd_amax_kernel(const uint4* dy, size_t n_chunks, unsigned int* amax_bits) {
  // |x| of a bf16 pair compares like the unsigned integer of its bits with the sign cleared, so the maximum is taken on
  // the packed halves; four loads per thread in flight
  uint32_t mx = 0u;
  auto fold = [&](const uint4& v) {
    const uint32_t w[4] = {v.x & 0x7FFF7FFFu, v.y & 0x7FFF7FFFu, v.z & 0x7FFF7FFFu, v.w & 0x7FFF7FFFu};
#pragma unroll
    for (int t = 0; t < 4; ++t) mx = __vmaxu2(mx, w[t]);
  };
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  for (; i + 3 * step < n_chunks; i += 4 * step) {
    const uint4 v0 = __ldg(dy + i), v1 = __ldg(dy + i + step), v2 = __ldg(dy + i + 2 * step), v3 = __ldg(dy + i + 3 * step);
    fold(v0), fold(v1), fold(v2), fold(v3);
  }
  for (; i < n_chunks; i += step) fold(__ldg(dy + i));
  const uint32_t top = (mx >> 16) > (mx & 0xFFFFu) ? (mx >> 16) : (mx & 0xFFFFu);
  float m = __uint_as_float(top << 16);  // NaN or infinity bits stay above 3e38 and are rejected below
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
  if ((threadIdx.x & 31) == 0 && m > 0.f && m <= 3.0e38f) atomicMax(amax_bits, __float_as_uint(m));
}
// scale[0] = c = the power of two that brings max |dy| into [8, 16), scale[1] = 1 / c (c = 1 for a zero gradient)
__global__ void bwd_scale_kernel(const unsigned int* amax_bits, float* scale) {
  const float amax = __uint_as_float(*amax_bits);
  float c = 1.0f;
  if (amax > 0.f) {
    int e = 0;
    frexpf(amax, &e);           // amax = f * 2^e, f in [0.5, 1)
    e = 4 - e;                  // amax * 2^(4 - e) in [8, 16)
    e = e > 100 ? 100 : (e < -100 ? -100 : e);
    c = ldexpf(1.0f, e);
  }
  scale[0] = c;
  scale[1] = 1.0f / c;
}

// Weights for the backward kernels: all six matrices (PackArgs order: left, left gate, right, right gate, out, gate)
// as dense fp16 [128][128] with the LayerNorm gamma of their input folded in, W'[r][k] = W[r][k] gamma[k], and
// d[m][r] = sum_k W[r][k] beta[k] + bias[m][r] (fp32) behind them. One warp per matrix row.
constexpr size_t kBwdPackedD = 6 * 32768;
constexpr size_t kBwdPackedBytes = kBwdPackedD + 3072;  // 199680, a multiple of 1024
__global__ void __launch_bounds__(128) bwd_pack_kernel(const PackArgs a, uint8_t* packed) {
  const int gw = blockIdx.x * 4 + (threadIdx.x >> 5);  // 0 .. 767
  const int lane = threadIdx.x & 31;
  const int m = gw >> 7, row = gw & 127;
  const int n_rows = m < 4 ? 128 : a.c;  // a.c = d_pair: matrices 0..3 are [128, c], 4 (out) is [c, 128], 5 (gate) [c, c]
  const int k = m == 4 ? 128 : a.c;
  if (row >= n_rows) return;
  const bool active = lane * 4 < k;
  const float* gamma = (m == 4) ? a.ln_out_w : a.ln_in_w;
  const float* beta = (m == 4) ? a.ln_out_b : a.ln_in_b;
  float w[4] = {0.f, 0.f, 0.f, 0.f};
  if (!active) {
  } else if (a.f32_weights) {
    const float4 v = reinterpret_cast<const float4*>(static_cast<const float*>(a.w[m]) + static_cast<size_t>(row) * a.ld[m])[lane];
    w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
  } else {
    const uint2 v = reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(a.w[m]) + static_cast<size_t>(row) * a.ld[m])[lane];
    w[0] = bf16_lo(v.x), w[1] = bf16_hi(v.x), w[2] = bf16_lo(v.y), w[3] = bf16_hi(v.y);
  }
  const float4 g = active ? reinterpret_cast<const float4*>(gamma)[lane] : make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 b = active ? reinterpret_cast<const float4*>(beta)[lane] : make_float4(0.f, 0.f, 0.f, 0.f);
  const float gg[4] = {g.x, g.y, g.z, g.w}, bb[4] = {b.x, b.y, b.z, b.w};
  float d = 0.f;
  uint16_t o[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    o[t] = __half_as_ushort(__float2half_rn(fminf(fmaxf(w[t] * gg[t], -65504.f), 65504.f)));
    d = fmaf(w[t], bb[t], d);
  }
  if (active) {
    uint2 ov;
    ov.x = static_cast<uint32_t>(o[0]) | (static_cast<uint32_t>(o[1]) << 16);
    ov.y = static_cast<uint32_t>(o[2]) | (static_cast<uint32_t>(o[3]) << 16);
    reinterpret_cast<uint2*>(packed + static_cast<size_t>(m) * 32768)[row * (k / 4) + lane] = ov;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, off);
  if (lane == 0)
    reinterpret_cast<float*>(packed + kBwdPackedD)[m * 128 + row] = d + (a.bias[m] != nullptr ? a.bias[m][row] : 0.f);
}

// Sum of element e over the partials g, g + 4, g + 8, ... (four loads in flight, fixed order of additions).
__device__ __forceinline__ float sum_every_fourth(const float* parts, size_t stride, int n_parts, int e, int g) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int i = g;
  for (; i + 12 < n_parts; i += 16) {
    const float a = parts[static_cast<size_t>(i) * stride + e], b = parts[static_cast<size_t>(i + 4) * stride + e];
    const float c = parts[static_cast<size_t>(i + 8) * stride + e], d = parts[static_cast<size_t>(i + 12) * stride + e];
    s0 += a, s1 += b, s2 += c, s3 += d;
  }
  for (; i < n_parts; i += 4) s0 += parts[static_cast<size_t>(i) * stride + e];
  return (s0 + s1) + (s2 + s3);
}

// M[e] and S[e] = sums over the CTAs' partials in a fixed order (deterministic). Blocks 0 .. 511 take M (2 x 128 x 128
// values), blocks 512 .. 515 take S (2 x 128 values).
__global__ void __launch_bounds__(256) bwd_reduce_kernel(const float* part_m, const float* part_s, int n_parts, float* m_out,
                                                         float* s_out) {
  // grid = 512 blocks for M (64 elements each) + 4 for S; a block's four groups of 64 threads take every fourth partial
  // and are combined in a fixed order
  __shared__ float comb[4][64];
  const bool is_s = blockIdx.x >= 512;
  const float* parts = is_s ? part_s : part_m;
  const size_t stride = is_s ? 2 * 128 : 2 * 128 * 128;
  const int el = threadIdx.x & 63, g = threadIdx.x >> 6;
  const int e = (is_s ? blockIdx.x - 512 : blockIdx.x) * 64 + el;
  comb[g][el] = sum_every_fourth(parts, stride, n_parts, e, g);
  __syncthreads();
  if (g == 0) (is_s ? s_out : m_out)[e] = (comb[0][el] + comb[1][el]) + (comb[2][el] + comb[3][el]);
}

// Parameter gradients from the reduced sums M[m] = dOut_m^T x_hat (times c) and S[m] = column sums of dOut_m (times c):
//   dW_m[r][k] = (M[m][r][k] gamma[k] + S[m][r] beta[k]) / c
//   dgamma[k]  = sum_m sum_r W_m[r][k] M[m][r][k] / c,   dbeta[k] = sum_m sum_r W_m[r][k] S[m][r] / c
// over the matrices that read that LayerNorm (the output one: matrix 4; the input one: the other five).
// One call covers one set of six 128 x 128 matrices ("half": the unidirectional module has one, the bidirectional module
// two, whose matrices are row or column blocks of the module's wider parameters, hence the leading dimensions).
// Grid (6 matrices, 8 blocks of 16 rows), thread = column k; the LayerNorm sums leave as partials [6][8][2][128] that
// bwd_finalize_ln_kernel adds in a fixed order.
struct BwdFinalArgs {
  PackArgs w;           // raw weights (this half's blocks, with their leading dimensions) and LayerNorm parameters
  const float* m_all;   // [6][128][128]
  const float* s_all;   // [6][128]
  const float* scale;   // [2]
  float* dw[6];         // fp32 gradient blocks
  int dw_ld[6];         // their leading dimensions
  float* ln_part;       // [6][8][2][128]
  unsigned mask;        // bit m set: matrix m is present in this half
};
__global__ void __launch_bounds__(128) bwd_finalize_kernel(const BwdFinalArgs a) {
  const int k = threadIdx.x, m = blockIdx.x, rb = blockIdx.y;
  if (((a.mask >> m) & 1u) == 0u) return;
  const int n_rows = m < 4 ? 128 : a.w.c, n_cols = m == 4 ? 128 : a.w.c;  // a.w.c = d_pair
  float* part0 = a.ln_part + ((m * 8 + rb) * 2 + 0) * 128 + k;
  float* part1 = a.ln_part + ((m * 8 + rb) * 2 + 1) * 128 + k;
  if (k >= n_cols || rb * 16 >= n_rows) {
    *part0 = 0.f, *part1 = 0.f;
    return;
  }
  const float cinv = a.scale[1];
  const float gamma = (m == 4 ? a.w.ln_out_w : a.w.ln_in_w)[k];
  const float beta = (m == 4 ? a.w.ln_out_b : a.w.ln_in_b)[k];
  float ag = 0.f, ab = 0.f;
#pragma unroll 4
  for (int r = rb * 16; r < rb * 16 + 16; ++r) {
    const size_t wi = static_cast<size_t>(r) * a.w.ld[m] + k;
    const float w = a.w.f32_weights ? static_cast<const float*>(a.w.w[m])[wi]
                                    : __uint_as_float(static_cast<uint32_t>(static_cast<const uint16_t*>(a.w.w[m])[wi]) << 16);
    const float mv = a.m_all[(m * 128 + r) * 128 + k] * cinv;
    const float sv = a.s_all[m * 128 + r] * cinv;
    a.dw[m][static_cast<size_t>(r) * a.dw_ld[m] + k] = fmaf(mv, gamma, sv * beta);
    ag = fmaf(w, mv, ag);
    ab = fmaf(w, sv, ab);
  }
  *part0 = ag;
  *part1 = ab;
}
struct BwdLnArgs {
  const float* ln_part[2];  // per half
  unsigned mask[2];
  int halves;
  float* d_ln_in_w;   // [128]
  float* d_ln_in_b;
  float* d_ln_out_w;  // [128 * halves]: half h at + 128 h
  float* d_ln_out_b;
  int c;              // d_pair
};
__global__ void __launch_bounds__(128) bwd_finalize_ln_kernel(const BwdLnArgs a) {
  const int k = threadIdx.x;
  float g_in = 0.f, b_in = 0.f;
  for (int h = 0; h < a.halves; ++h) {
    float g_out = 0.f, b_out = 0.f;
    for (int m = 0; m < 6; ++m) {
      if (((a.mask[h] >> m) & 1u) == 0u) continue;
      float ag = 0.f, ab = 0.f;
      for (int rb = 0; rb < 8; ++rb) {
        ag += a.ln_part[h][((m * 8 + rb) * 2 + 0) * 128 + k];
        ab += a.ln_part[h][((m * 8 + rb) * 2 + 1) * 128 + k];
      }
      if (m == 4) g_out += ag, b_out += ab;
      else g_in += ag, b_in += ab;
    }
    a.d_ln_out_w[h * 128 + k] = g_out;
    a.d_ln_out_b[h * 128 + k] = b_out;
  }
  if (k < a.c) {  // the input LayerNorm has d_pair channels
    a.d_ln_in_w[k] = g_in;
    a.d_ln_in_b[k] = b_in;
  }
}

}  // namespace trimul
