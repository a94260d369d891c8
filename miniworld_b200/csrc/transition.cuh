// Pair Transition (the SwiGLU feed-forward that follows the triangle update in every Pairformer block):
//
//   y[pos, :] = x[pos, :] + W_s ( SiLU(W_a x_hat) * (W_b x_hat) ),   x_hat = LayerNorm(x[pos, :])
//
// with C = 128 channels and a hidden width of 512 (n = 4), all linears bias-free. 393 kFLOP per position against
// 512 bytes of compulsory traffic: the kernel is bound by the tensor cores, and what limits it in practice is the
// 384 KiB of weights every tile of positions has to meet. Persistent CTA pairs (tcgen05 cta_group::2): a pair works
// on 256 consecutive positions (128 per CTA) and walks the hidden dimension in eight blocks of 64 units; per block
// each CTA loads only HALF of the block's weights (CTA 0 the 64 rows of W_a, CTA 1 the 64 rows of W_b, and each its
// 64 output rows of W_s), 24 KiB, because the MMAs of a pair read the B operand from both CTAs' shared memory.
//
//   G1(block): D1[pos, 0:64 | 64:128] = x_hat[pos, :] * [0.5 W_a(block) ; W_b(block)]^T     (M 256, N 128, K 128)
//   SwiGLU   : h[pos, u] = a2 (1 + tanh a2) * b,  a2 = D1[pos, u] (= a / 2),  b = D1[pos, 64 + u]   -> fp16, into TMEM
//   G2(block): D2[pos, :] += h[pos, 0:64] * W_s[:, block]^T                (M 256, N 128, K 64, A operand from TMEM)
//
// Tensor memory (512 columns per CTA): D1[0], D1[1] (128 each) and D2[0], D2[1] (128 each, alternating by tile).
// h never touches shared memory: the SwiGLU threads store it with tcgen05.st into the first 64 columns of the D2
// buffer that is NOT accumulating during the tile (H[g] = 32 columns per group: 64 fp16 per lane), and G2 reads its A
// operand from there. Two groups of SwiGLU warps take alternate blocks (group g: blocks with k & 1 == g, D1[g],
// H[g]), so the tensor pipe runs G1 of block k+1 and G2 of block k-1 while block k is turned into h; a D1 buffer is
// free as soon as its values are in registers, an H buffer once G2 of its block is complete. A separate group of
// warps writes the tile's y = x + D2, so the SwiGLU groups never leave the block loop; the first h of a tile waits
// until that group has read the D2 buffer h is about to borrow.
// LayerNorm is done once per tile by dedicated warps, in place on the loaded tile (fp32 statistics, affine applied,
// rounded to fp16 for the tensor cores); the residual re-reads x from global memory (L2) at the end of the tile.
//
// Warp roles (1024 threads per CTA, 64 registers each): warp 0 weight producer, warp 1 issuer of the G1 MMAs (leader
// CTA) / TMEM owner, warp 2 input-tile producer, warp 3 issuer of the G2 MMAs (leader CTA), warps 4-11 LayerNorm (four
// of them took 19 k cycles per tile next to the busy SwiGLU warps instead of 4 k alone), warps 12-19 and 20-27 the two
// SwiGLU groups (two threads per position, 32 hidden units each per block in two passes of 16), warps 28-31 the output
// group. Three input stages let LayerNorm of tile t + 2 run while tile t is still being written out.
// G1 and G2 have an issuing thread each: issuing one 256 x 128 x 16 MMA costs about as long as it runs, so a single
// thread that also waits for the SwiGLU warps between the two GEMMs leaves the tensor pipe idle half of the time.
// Only mbarrier signals cross between the two CTAs. All waits are bounded.
#pragma once

#include "ptx.cuh"

namespace trimul {

struct TransitionParams {
  long long positions;  // rows of x / y
  int num_tiles;        // ceil(positions / 256): one tile per CTA pair and step
  const float* ln_w;    // [128] LayerNorm gamma
  const float* ln_b;    // [128] LayerNorm beta
  const __nv_bfloat16* x;  // the input again, for the residual
  float eps;
  int residual;
  int* status;
};

constexpr int kTrThreads = 1024;
constexpr int kTrBlocks = 8;            // hidden blocks of 64 units
constexpr int kTrWStages = 5;
constexpr int kTrXStages = 3;           // input tiles in flight: LayerNorm of tile t + 2 runs while tile t is still being written out
constexpr int kTrWStageBytes = 24576;   // 16 KiB of W_a or W_b rows + 8 KiB of W_s rows
constexpr int kTrXBytes = 32768;        // 128 positions x 128 channels, 16-bit
constexpr int kTrBarBytes = 256;
constexpr int kTrSmemBytes = kTrXStages * kTrXBytes + kTrWStages * kTrWStageBytes + kTrBarBytes + 1024;
constexpr uint32_t kTrColD2 = 256;      // tensor-memory columns: D1[b] at b * 128, D2[b] at kTrColD2 + b * 128

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTrThreads, 1)
transition_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                  const __grid_constant__ CUtensorMap map_wab, const __grid_constant__ CUtensorMap map_ws,
                  const TransitionParams p) {
  constexpr int WS = kTrWStages;
  constexpr int XS = kTrXStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t x_base = smem_base;
  const uint32_t w_base = x_base + XS * kTrXBytes;
  const uint32_t bar_base = w_base + WS * kTrWStageBytes;
  // barriers ("leader": only the copy in CTA 0 is used; "both": the MMA commit signals the copy in each CTA)
  auto x_full = [&](int s) { return bar_base + 8u * (0 + s); };          // own: this CTA's tile has landed
  auto xn_ready = [&](int s) { return bar_base + 8u * (XS + s); };       // leader: 16 LayerNorm warps (8 per CTA)
  auto x_empty = [&](int s) { return bar_base + 8u * (2 * XS + s); };    // own: the tile's y has been stored
  constexpr int B0 = 3 * XS;
  auto w_full = [&](int s) { return bar_base + 8u * (B0 + s); };         // leader: bytes of both CTAs
  auto blk_done = [&](int s) { return bar_base + 8u * (B0 + WS + s); };  // both: G2 of the block in weight stage s is complete
  auto d1_full = [&](int b) { return bar_base + 8u * (B0 + 2 * WS + b); };       // both
  auto d1_empty = [&](int b) { return bar_base + 8u * (B0 + 2 * WS + 2 + b); };  // leader: 8 warps (group b of both CTAs)
  auto h_full = [&](int b) { return bar_base + 8u * (B0 + 2 * WS + 4 + b); };    // leader: 8 warps (group b of both CTAs)
  auto d2_full = [&](int b) { return bar_base + 8u * (B0 + 2 * WS + 6 + b); };   // both
  auto d2_empty = [&](int b) { return bar_base + 8u * (B0 + 2 * WS + 8 + b); };  // leader: 8 warps (output group of both CTAs)
  auto d2_read = [&](int b) { return bar_base + 8u * (B0 + 2 * WS + 10 + b); };  // own: this CTA's output group has read D2[b]
  constexpr int kBarOff = XS * kTrXBytes + WS * kTrWStageBytes;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kBarOff + 8 * (B0 + 2 * WS + 12));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < XS; ++s) {
      mbar_init(x_full(s), 1);
      mbar_init(xn_ready(s), 16);
      mbar_init(x_empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(d1_full(s), 1);
      mbar_init(d1_empty(s), 16);
      mbar_init(h_full(s), 16);
      mbar_init(d2_full(s), 1);
      mbar_init(d2_empty(s), 8);
      mbar_init(d2_read(s), 4);
    }
    for (int s = 0; s < WS; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(blk_done(s), 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_x);
    prefetch_tmap(&map_y);
    prefetch_tmap(&map_wab);
    prefetch_tmap(&map_ws);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before any signal crosses
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tiles of this pair: tile index t_local = 0, 1, ... <-> global tile pair + t_local * num_pairs
  const int my_tiles = pair < p.num_tiles ? (p.num_tiles - pair + num_pairs - 1) / num_pairs : 0;

  if (warp == 0) {
    // ------------------------------------------------------------ weight producer (both CTAs): 8 blocks per tile
    if (lane == 0) {
      const long long total = static_cast<long long>(my_tiles) * kTrBlocks;
      for (long long gb = 0; gb < total; ++gb) {
        const int slot = static_cast<int>(gb % WS);
        const uint32_t ph = static_cast<uint32_t>((gb / WS) & 1);
        if (!mbar_wait(blk_done(slot), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) break;
        const int hb = static_cast<int>(gb % kTrBlocks);
        if (rank == 0) mbar_arrive_expect_tx(w_full(slot), 2 * kTrWStageBytes);  // bytes of both CTAs
        const uint32_t bar = map_to_cta(w_full(slot), 0);
        const uint32_t ws = w_base + slot * kTrWStageBytes;
        // [0.5 W_a ; W_b] packed per block: rows hb*128 .. +63 are W_a's units, +64 .. +127 W_b's; two 64-wide k halves
        const int row_ab = hb * 128 + static_cast<int>(rank) * 64;
        tma_load_2d_pair(ws, &map_wab, bar, 0, row_ab);
        tma_load_2d_pair(ws + 8192, &map_wab, bar, 64, row_ab);
        // W_s [128 out, 512]: this CTA's 64 output rows, the block's 64 hidden units
        tma_load_2d_pair(ws + 16384, &map_ws, bar, hb * 64, static_cast<int>(rank) * 64);
      }
      // Drain (leader: its barriers count the bytes of both CTAs; the closing cluster barrier keeps CTA 1 alive).
      if (rank == 0) {
        const long long pending = total < WS ? total : WS;
        for (long long back = 1; back <= pending; ++back) {
          const long long gb = total - back;
          const long long t0 = clock64();
          while (!mbar_try_wait(w_full(static_cast<int>(gb % WS)), static_cast<uint32_t>((gb / WS) & 1))) {
            if (*abort_flag != 0 || clock64() - t0 > kWaitLimitCycles) {
              atomicCAS(p.status, 0, kDevTimeoutDrain);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ input-tile producer (both CTAs)
    if (lane == 0) {
      for (int t = 0; t < my_tiles; ++t) {
        const int s = t % XS;
        const uint32_t ph = (t / XS) & 1;
        if (!mbar_wait(x_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) break;
        const int tile = pair + t * num_pairs;
        const int row0 = tile * 256 + static_cast<int>(rank) * 128;  // rows past the end read as zero
        mbar_arrive_expect_tx(x_full(s), kTrXBytes);
        tma_load_2d(x_base + s * kTrXBytes, &map_x, x_full(s), 0, row0);
        tma_load_2d(x_base + s * kTrXBytes + 16384, &map_x, x_full(s), 64, row0);
      }
      // every tile loaded here is consumed by this CTA's LayerNorm warps before the kernel ends: nothing to drain
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ issuer of G1 (leader CTA only)
    // D1[gb & 1] = x_hat * [W_a ; W_b](block)^T, as soon as the weights are there and the SwiGLU group of that buffer
    // has taken its previous contents into registers.
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc(256, 128, false, false, kFmtF16, kFmtF16);
      const long long total = static_cast<long long>(my_tiles) * kTrBlocks;
      for (long long gb = 0; gb < total; ++gb) {
        const int t = static_cast<int>(gb / kTrBlocks);
        const int hb = static_cast<int>(gb % kTrBlocks);
        const int s = t % XS;
        if (hb == 0 && !mbar_wait(xn_ready(s), (t / XS) & 1, abort_flag, p.status, kDevTimeoutMma)) break;
        const int slot = static_cast<int>(gb % WS);
        if (!mbar_wait(w_full(slot), static_cast<uint32_t>((gb / WS) & 1), abort_flag, p.status, kDevTimeoutMma)) break;
        const int b = static_cast<int>(gb & 1);
        if (!mbar_wait(d1_empty(b), static_cast<uint32_t>(((gb >> 1) & 1) ^ 1), abort_flag, p.status, kDevTimeoutMma)) break;
        tc_fence_after();
        const uint32_t xs = x_base + s * kTrXBytes;
        const uint32_t ws = w_base + slot * kTrWStageBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t da = umma_desc_kmajor(xs + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2);
          const uint64_t db = umma_desc_kmajor(ws + (ks >> 2) * 8192) + static_cast<uint64_t>((ks & 3) * 2);
          umma_pair(tmem_base + b * 128, da, db, idesc, ks != 0 ? 1u : 0u);
        }
        umma_commit_pair(d1_full(b));
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------ issuer of G2 (leader CTA only)
    // D2 += H[gb & 1] * W_s(block)^T once the SwiGLU warps of both CTAs have written h. G1 of the same block completed
    // before h could be computed, so one commit after G2 says that the block's weight stage and its H buffer are free.
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc(256, 128, false, false, kFmtF16, kFmtF16);
      const long long total = static_cast<long long>(my_tiles) * kTrBlocks;
      for (long long gb = 0; gb < total; ++gb) {
        const int t = static_cast<int>(gb / kTrBlocks);
        const int hb = static_cast<int>(gb % kTrBlocks);
        const int b = static_cast<int>(gb & 1);
        const int slot = static_cast<int>(gb % WS);
        // D2[t & 1] last held tile t - 2 (and lent its first columns to h during tile t - 1, whose G2s this thread has
        // issued before): wait until the output group has read tile t - 2 out of it
        if (hb == 0 && !mbar_wait(d2_empty(t & 1), ((t >> 1) & 1) ^ 1u, abort_flag, p.status, kDevTimeoutMma)) break;
        if (!mbar_wait(h_full(b), static_cast<uint32_t>((gb >> 1) & 1), abort_flag, p.status, kDevTimeoutMma)) break;
        tc_fence_after();
        const uint32_t ws = w_base + slot * kTrWStageBytes + 16384;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // H[b][(hb >> 1) & 1]: 32 of the 128 columns of the D2 buffer that is idle during this tile (two buffers per
          // SwiGLU group, used in turn); 8 columns = 16 fp16 per 16-deep MMA
          const uint32_t a_tmem = tmem_base + kTrColD2 + ((t + 1) & 1) * 128 + ((hb >> 1) & 1) * 64 + b * 32 + ks * 8;
          const uint64_t db = umma_desc_kmajor(ws) + static_cast<uint64_t>(ks * 2);
          umma_pair_ta(tmem_base + kTrColD2 + (t & 1) * 128, a_tmem, db, idesc, (hb | ks) != 0 ? 1u : 0u);
        }
        umma_commit_pair(blk_done(slot));
        if (hb == kTrBlocks - 1) umma_commit_pair(d2_full(t & 1));
      }
    }
  } else if (warp < 12) {
    // ------------------------------------------------------------ LayerNorm of this CTA's 128 positions, in place
    // Eight threads per position (16 channels each, their gamma / beta in registers), four passes of 32 positions.
    const int ts = threadIdx.x - 128;  // 0 .. 255
    const int sub = ts & 7;            // 16-byte chunk: channels 8*sub .. 8*sub+7 of each 64-channel half
    const int slot = ts >> 3;          // position slot inside a pass
    float2 g[8], b[8];
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int c = half * 64 + sub * 8 + 2 * t;
        g[half * 4 + t] = make_float2(p.ln_w[c], p.ln_w[c + 1]);
        b[half * 4 + t] = make_float2(p.ln_b[c], p.ln_b[c + 1]);
      }
    for (int t = 0; t < my_tiles; ++t) {
      const int s = t % XS;
      if (!mbar_wait_warp(x_full(s), (t / XS) & 1, abort_flag, p.status, kDevTimeoutStats)) break;
      const uint32_t xs = x_base + s * kTrXBytes;
#pragma unroll 2
      for (int pass = 0; pass < 4; ++pass) {
        const int pos = pass * 32 + slot;
        const uint32_t addr = xs + pos * 128 + ((sub ^ (pos & 7)) << 4);
        uint32_t w[8];
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                     : "r"(addr + 16384));
        float2 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = bf16x2_to_float2(w[i]);
        const float2 a01 = __fadd2_rn(__fadd2_rn(v[0], v[1]), __fadd2_rn(v[2], v[3]));
        const float2 a23 = __fadd2_rn(__fadd2_rn(v[4], v[5]), __fadd2_rn(v[6], v[7]));
        const float2 acc = __fadd2_rn(a01, a23);
        float sum = acc.x + acc.y;
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
        const float mean = sum * (1.0f / 128.0f);
        const float2 nmean = make_float2(-mean, -mean);
        float2 q0 = make_float2(0.f, 0.f), q1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          v[i] = __fadd2_rn(v[i], nmean);
          v[i + 1] = __fadd2_rn(v[i + 1], nmean);
          q0 = __ffma2_rn(v[i], v[i], q0);
          q1 = __ffma2_rn(v[i + 1], v[i + 1], q1);
        }
        const float2 q2 = __fadd2_rn(q0, q1);
        float ssq = q2.x + q2.y;
        ssq += __shfl_xor_sync(0xFFFFFFFFu, ssq, 1);
        ssq += __shfl_xor_sync(0xFFFFFFFFu, ssq, 2);
        ssq += __shfl_xor_sync(0xFFFFFFFFu, ssq, 4);
        const float rstd = rsqrtf(ssq * (1.0f / 128.0f) + p.eps);
        const float2 rstd2 = make_float2(rstd, rstd);
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = pack_f16x2_sat(__ffma2_rn(__fmul2_rn(v[i], rstd2), g[i], b[i]));
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr + 16384), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                     : "memory");
      }
      fence_proxy_async_smem();  // x_hat was written through the generic proxy; the MMA reads it through the async one
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(xn_ready(s), rank);
    }
  } else if (warp < 28) {
    // ------------------------------------------------------------ SwiGLU groups (8 warps each)
    // Thread = one position (TMEM lane) and half of the block's 64 hidden units, in two passes of 16.
    const int grp = (warp - 12) >> 3;  // 0: even blocks, 1: odd blocks
    const int uh = ((warp - 12) >> 2) & 1;  // which 32 units
    const int q = warp & 3;            // TMEM lane quarter this warp may access
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_d1 = tmem_base + lane_off + grp * 128 + uh * 32;
    for (int t = 0; t < my_tiles; ++t) {
      // h of this tile borrows the D2 buffer that is not accumulating: H[grp][0 / 1] = 32 columns each, used in turn, so
      // that a block's h never waits for the G2 of the group's previous block
      const int hbuf = (t + 1) & 1;
      const uint32_t t_h0 = tmem_base + lane_off + kTrColD2 + hbuf * 128 + grp * 32 + uh * 16;
      bool alive = true;
#pragma unroll 1
      for (int hb = grp; hb < kTrBlocks; hb += 2) {
        const long long gb = static_cast<long long>(t) * kTrBlocks + hb;
        const uint32_t bph = static_cast<uint32_t>((gb >> 1) & 1);
        if (!mbar_wait_warp(d1_full(grp), bph, abort_flag, p.status, kDevTimeoutEpilogue)) {
          alive = false;
          break;
        }
        tc_fence_after();
        uint32_t o[16];
#pragma unroll
        for (int pq = 0; pq < 2; ++pq) {
          uint32_t va[16], vb[16];
          tmem_ld16(t_d1 + pq * 16, va);
          tmem_ld16(t_d1 + 64 + pq * 16, vb);
          tmem_ld_wait();
          if (pq == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(d1_empty(grp), rank);  // D1[grp] may be overwritten by block gb + 2
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float2 a2 = make_float2(__uint_as_float(va[2 * i]), __uint_as_float(va[2 * i + 1]));
            const float2 bb = make_float2(__uint_as_float(vb[2 * i]), __uint_as_float(vb[2 * i + 1]));
            const float2 th = make_float2(tanh_approx(a2.x), tanh_approx(a2.y));  // (the packed fp16 form measured no faster)
            o[pq * 8 + i] = pack_f16x2_sat(__fmul2_rn(__ffma2_rn(th, a2, a2), bb));
          }
        }
        // this H buffer is free once G2 of block gb - 4 (weight stage (gb - 4) % WS) is complete (block gb + 1, the next
        // one in the same stage, cannot have completed yet: its G2 is issued after this block's); the first h of a tile
        // also waits until this CTA's output group has read tile t - 1 out of the D2 buffer that h borrows
        const uint32_t t_h = t_h0 + ((hb >> 1) & 1) * 64;
        if (gb >= 4) {
          const long long pb = gb - 4;
          if (!mbar_wait_warp(blk_done(static_cast<int>(pb % WS)), static_cast<uint32_t>((pb / WS) & 1), abort_flag, p.status,
                              kDevTimeoutEpilogue)) {
            alive = false;
            break;
          }
        }
        if (hb == grp && t >= 1) {
          // tile t - 1 accumulated in D2[(t - 1) & 1] = D2[hbuf]; it is that buffer's use number (t - 1) / 2
          if (!mbar_wait_warp(d2_read(hbuf), static_cast<uint32_t>(((t - 1) >> 1) & 1), abort_flag, p.status,
                              kDevTimeoutEpilogue)) {
            alive = false;
            break;
          }
        }
        tc_fence_after();
        tmem_st16(t_h, o);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_leader(h_full(grp), rank);
      }
      if (!alive) break;
    }
  } else {
    // ------------------------------------------------------------ output group: y = x + D2 per tile
    // Thread = one position and all 128 channels, in eight passes of 16 (the residual is fetched one pass ahead).
    const int q = warp & 3;
    const int pos = q * 32 + lane;
    const bool store_thread = warp == 28 && lane == 0;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    for (int t = 0; t < my_tiles; ++t) {
      const int s = t % XS;
      const int tile = pair + t * num_pairs;
      const long long grow = static_cast<long long>(tile) * 256 + static_cast<long long>(rank) * 128 + pos;
      const bool in_range = grow < p.positions;
      const uint4* xp = reinterpret_cast<const uint4*>(p.x + (in_range ? grow : 0) * 128);
      uint4 xr[2][2];
#pragma unroll
      for (int c = 0; c < 2; ++c) xr[0][c] = (p.residual && in_range) ? __ldg(xp + c) : make_uint4(0u, 0u, 0u, 0u);
      {
        const bool got = mbar_wait_warp(d2_full(t & 1), (t >> 1) & 1, abort_flag, p.status, kDevTimeoutEpilogue);
        if (!named_bar_and(1, 128, got)) break;
      }
      tc_fence_after();
      const uint32_t xs = x_base + s * kTrXBytes;  // x_hat is dead (every G1 of the tile has completed): reuse for y
      const uint32_t t_d2 = tmem_base + lane_off + kTrColD2 + (t & 1) * 128;
#pragma unroll
      for (int ps = 0; ps < 8; ++ps) {
        if (ps < 7) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
            xr[(ps + 1) & 1][c] = (p.residual && in_range) ? __ldg(xp + (ps + 1) * 2 + c) : make_uint4(0u, 0u, 0u, 0u);
        }
        uint32_t v[16];
        tmem_ld16(t_d2 + ps * 16, v);
        tmem_ld_wait();
        if (ps == 7) {
          // D2[t & 1] has been read: h of tile t + 1 may borrow it (this CTA's SwiGLU groups), and the G2s of tile
          // t + 2 may accumulate into it (the leader's issuer)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(d2_read(t & 1));
            mbar_arrive_leader(d2_empty(t & 1), rank);
          }
        }
        const uint32_t yrow = xs + (ps >> 2) * 16384 + pos * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint4 xv = xr[ps & 1][c];
          const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 d = make_float2(__uint_as_float(v[8 * c + 2 * i]), __uint_as_float(v[8 * c + 2 * i + 1]));
            o[i] = pack_bf16x2(__fadd2_rn(d, bf16x2_to_float2(xw[i])));
          }
          const uint32_t addr = yrow + ((((ps & 3) * 2 + c) ^ (pos & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                       : "memory");
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(1, 128);
      if (store_thread) {
        const int row0 = tile * 256 + static_cast<int>(rank) * 128;
        if (row0 < p.positions) {  // rows past the end are clipped by the copy; a tile wholly past it is skipped
          tma_store_2d(&map_y, xs, 0, row0);
          tma_store_2d(&map_y, xs + 16384, 64, row0);
        }
        bulk_commit();
        bulk_wait_read<0>();
        mbar_arrive(x_empty(s));
      }
    }
    if (store_thread) bulk_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers or read its operands
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Weight packing for transition_kernel: [0.5 W_a ; W_b] interleaved per block of 64 hidden units as fp16
// ([8 blocks][128 rows][128]), W_s as fp16 [128][512], then gamma and beta (fp32[128] each).
constexpr size_t kTrPackedAbBytes = 1024 * 128 * 2;
constexpr size_t kTrPackedWsBytes = 128 * 512 * 2;
constexpr size_t kTrPackedLnOff = kTrPackedAbBytes + kTrPackedWsBytes;
constexpr size_t kTrPackedBytes = kTrPackedLnOff + 1024;

struct TransitionPackArgs {
  const void* w_a;  // [512, 128]
  const void* w_b;  // [512, 128]
  const void* w_s;  // [128, 512]
  const float* ln_w;
  const float* ln_b;
  int f32_weights;
};

__device__ __forceinline__ float load_weight(const void* w, size_t idx, int f32) {
  return f32 ? static_cast<const float*>(w)[idx] : __bfloat162float(static_cast<const __nv_bfloat16*>(w)[idx]);
}

__global__ void __launch_bounds__(256) transition_pack_kernel(const TransitionPackArgs a, uint8_t* packed) {
  const int i = blockIdx.x * 256 + threadIdx.x;  // 0 .. 196607
  __half* ab = reinterpret_cast<__half*>(packed);
  __half* ws = reinterpret_cast<__half*>(packed + kTrPackedAbBytes);
  if (i < 1024 * 128) {
    const int row = i >> 7, col = i & 127;
    const int hb = row >> 7, r = row & 127;
    const float v = r < 64 ? 0.5f * load_weight(a.w_a, static_cast<size_t>(hb * 64 + r) * 128 + col, a.f32_weights)
                           : load_weight(a.w_b, static_cast<size_t>(hb * 64 + r - 64) * 128 + col, a.f32_weights);
    ab[i] = __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
  } else if (i < 1024 * 128 + 128 * 512) {
    const int j = i - 1024 * 128;
    ws[j] = __float2half_rn(fminf(fmaxf(load_weight(a.w_s, j, a.f32_weights), -65504.f), 65504.f));
  }
  if (i < 128) {
    reinterpret_cast<float*>(packed + kTrPackedLnOff)[i] = a.ln_w[i];
    reinterpret_cast<float*>(packed + kTrPackedLnOff)[128 + i] = a.ln_b[i];
  }
}

}  // namespace trimul
