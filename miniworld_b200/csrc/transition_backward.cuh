// Backward of the pair Transition  y = x + squeeze(SiLU(expand_a(LN x)) * expand_b(LN x)),  hidden width 512.
//
// One launch per block of 128 hidden units (four launches): the weight gradients of a block (expand_a, expand_b and
// squeeze: three 128 x 128 accumulators) stay in tensor memory over all position tiles of a CTA, which leaves one
// 128-column working region; the running d x_hat is carried between the launches in HBM (fp16, in place) and the last
// launch finishes the LayerNorm backward and the residual. Structure as in backward.cuh: one CTA per SM, 512 threads
// (four per position, 32 hidden units or channels each), tiles of 128 positions, phases separated by CTA-wide barriers,
// one thread issuing TMA copies and MMAs. Per tile and block j:
//   x_hat = LN(x) and dy * c as fp16 tiles (c: the power-of-two gradient scale of backward.cuh)
//   dh = dy Ws_j      -> registers        a = x_hat Wa_j'^T + ca -> registers        b = x_hat Wb_j'^T + cb
//   da = dh b silu'(a),  db = dh silu(a),  h = silu(a) b     (one scratch tile, used three times in turn)
//   d x_hat (+)= da Wa_j' + db Wb_j'        Ma_j += da^T x_hat     Mb_j += db^T x_hat     dWs_j += dy^T h
// Wa' = Wa gamma, Wb' = Wb gamma (fp16), ca = Wa beta, cb = Wb beta; the column sums of da and db (the beta terms of
// the weight gradients) are read back from the scratch tile by a thread per hidden unit and kept in a register.
#pragma once

#include "backward.cuh"

namespace trimul {

struct BwdTransitionParams {
  int num_tiles;          // ceil(positions / 128)
  long long positions;
  int block;              // hidden block j of this launch (0..3)
  const float* consts;    // [2][512]: ca, cb
  const float* grad_scale;
  const uint16_t* dx_in;  // [positions][128] fp16: c * d loss / d x_hat gathered by the earlier launches (not FIRST)
  float eps;
  int residual;
  float* part_m;          // [grid][3][128][128]: Ma_j, Mb_j, dWs_j partials
  float* part_s;          // [grid][2][4][128]: column sums of da and db per position quarter
  int* status;
};

constexpr int kTrBwdSmemBytes = 6 * kBwdTile + kBwdXchg + 1024 + 256 + 1024;

template <bool FIRST, bool LAST>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_transition_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_dy,
                      const __grid_constant__ CUtensorMap map_wa, const __grid_constant__ CUtensorMap map_wb,
                      const __grid_constant__ CUtensorMap map_ws, const __grid_constant__ CUtensorMap map_out,
                      const BwdTransitionParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t wa_s = smem_base, wb_s = wa_s + kBwdTile, ws_s = wb_s + kBwdTile;
  const uint32_t x_s = ws_s + kBwdTile, y_s = x_s + kBwdTile, s_s = y_s + kBwdTile;  // x_hat, dy * c, scratch
  const uint32_t xchg = smem_base + 6 * kBwdTile;
  const uint32_t bar_base = xchg + kBwdXchg + 1024;
  const uint32_t w_full = bar_base, in_full = bar_base + 8, mma_bar = bar_base + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 6 * kBwdTile + kBwdXchg + 1024 + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* const_ptr = reinterpret_cast<float*>(smem + 6 * kBwdTile + kBwdXchg);  // ca_j[128], cb_j[128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = warp & 3, part = warp >> 2;
  const int pos = q * 32 + lane;
  const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    mbar_init(in_full, 1);
    mbar_init(mma_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_x);
    prefetch_tmap(&map_dy);
    prefetch_tmap(&map_out);
  }
  if (threadIdx.x < 256) const_ptr[threadIdx.x] = p.consts[(threadIdx.x >> 7) * 512 + p.block * 128 + (threadIdx.x & 127)];
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const float gc = p.grad_scale[0], gc_inv = p.grad_scale[1];

  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(w_full, 3 * kBwdTile);
#pragma unroll
    for (int kh = 0; kh < 2; ++kh) {
      tma_load_2d(wa_s + kh * 16384, &map_wa, w_full, kh * 64, p.block * 128);  // Wa' rows of block j, [128 hid][128 k]
      tma_load_2d(wb_s + kh * 16384, &map_wb, w_full, kh * 64, p.block * 128);
      tma_load_2d(ws_s + kh * 16384, &map_ws, w_full, p.block * 128 + kh * 64, 0);  // Ws columns of block j, [128 c][128 hid]
    }
  }
  // column sums of da and db: this thread's 16-byte chunk (eight hidden units) of four position rows of the scratch tile
  const int sum_chunk = threadIdx.x & 15, sum_rows = (threadIdx.x >> 4) * 4;
  float sa_acc[8], sb_acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) sa_acc[c] = 0.f, sb_acc[c] = 0.f;

  bool ok = true;
  int it = 0;
  bool loads_pending = false;
  uint32_t mma_phase = 0;
  auto mma_wait = [&]() {
    // per thread, no CTA-wide barrier: a thread that gives up carries on and the CTA leaves at the tile's last barrier
    const bool got = thread_wait(mma_bar, mma_phase, abort_flag, p.status, kDevTimeoutEpilogue);
    mma_phase ^= 1u;
    return got;
  };
  // adds this thread's share of the scratch tile's column sums
  auto column_sum = [&](float (&acc)[8]) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint4 a = ld_chunk(s_s + tile_chunk(sum_rows + r, sum_chunk));
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 x = f16x2_to_float2(aw[t]);
        acc[2 * t] += x.x, acc[2 * t + 1] += x.y;
      }
    }
  };
  auto issue_inputs = [&](int p0_i) {  // thread 0
    mbar_arrive_expect_tx(in_full, 2 * kBwdTile);
#pragma unroll
    for (int kh = 0; kh < 2; ++kh) {
      tma_load_2d(y_s + kh * 16384, &map_dy, in_full, kh * 64, p0_i);
      tma_load_2d(x_s + kh * 16384, &map_x, in_full, kh * 64, p0_i);
    }
    loads_pending = true;
  };
  for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
    const int p0 = tile * 128;
    if (threadIdx.x == 0) {
      if (!loads_pending) issue_inputs(p0);  // (not LAST: requested while the previous tile finished)
    }
    if (it == 0) ok &= thread_wait(w_full, 0, abort_flag, p.status, kDevTimeoutMma);
    ok &= thread_wait(in_full, it & 1, abort_flag, p.status, kDevTimeoutStats);
    loads_pending = false;  // (only thread 0's copy is read)
    // ---- dy * c as fp16 in place (x_hat follows while the first GEMM runs)
#pragma unroll
    for (int ch = 0; ch < kBwdChunks; ++ch) {
      const uint32_t addr = y_s + tile_chunk(pos, part * kBwdChunks + ch);
      const uint4 v = ld_chunk(addr);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t o[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 d = bf16x2_to_float2(w[t]);
        o[t] = pack_f16x2_sat(make_float2(d.x * gc, d.y * gc));
      }
      st_chunk(addr, o[0], o[1], o[2], o[3]);
    }
    // the previous tile's store has read the scratch tile (rewritten after the third GEMM round; the barrier below
    // orders this wait before every thread's writes)
    if (threadIdx.x == 0) bulk_wait_read<0>();
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- dh = dy Ws_j (A: dy K-major over c; B: Ws_j [c rows][hid] read MN-major) -> working columns 0-127
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc(128, 128, false, true, kFmtF16, kFmtF16);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_bf16(tmem_base, umma_desc_kmajor(y_s + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2),
                  umma_desc_mnmajor(ws_s + ks * 2048, 16384), idesc, ks != 0 ? 1u : 0u);
      umma_commit(mma_bar);
    }
    // ---- x_hat in place, in the shadow of the dh GEMM (which reads dy and Ws only)
    const float rstd_in = normalise_tile<true, true, 128>(x_s, xchg, pos, part, p.eps);
    fence_proxy_async_smem();
    ok &= mma_wait();
    tc_fence_after();
    float dh[kBwdCh];
#pragma unroll
    for (int ch = 0; ch < kBwdChunks; ++ch) {
      uint32_t v[8];
      tmem_ld8(tmem_base + lane_sel + part * kBwdCh + ch * 8, v);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 8; ++e) dh[ch * 8 + e] = __uint_as_float(v[e]);
    }
    tc_fence_before();
    __syncthreads();
    // ---- a = x_hat Wa_j'^T
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc(128, 128, false, false, kFmtF16, kFmtF16);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t kb = static_cast<uint64_t>((ks & 3) * 2);
        umma_bf16(tmem_base, umma_desc_kmajor(x_s + (ks >> 2) * 16384) + kb, umma_desc_kmajor(wa_s + (ks >> 2) * 16384) + kb,
                  idesc, ks != 0 ? 1u : 0u);
      }
      umma_commit(mma_bar);
    }
    ok &= mma_wait();
    tc_fence_after();
    float av[kBwdCh];
#pragma unroll
    for (int ch = 0; ch < kBwdChunks; ++ch) {
      uint32_t v[8];
      tmem_ld8(tmem_base + lane_sel + part * kBwdCh + ch * 8, v);
      tmem_ld_wait();
      {
        const float4* cp = reinterpret_cast<const float4*>(const_ptr + part * kBwdCh + ch * 8);
        const float4 c0 = cp[0], c1 = cp[1];
        const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) av[ch * 8 + e] = __uint_as_float(v[e]) + cc[e];
      }
    }
    tc_fence_before();
    __syncthreads();
    // ---- b = x_hat Wb_j'^T; then da -> scratch tile, db and h kept packed in registers
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc(128, 128, false, false, kFmtF16, kFmtF16);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t kb = static_cast<uint64_t>((ks & 3) * 2);
        umma_bf16(tmem_base, umma_desc_kmajor(x_s + (ks >> 2) * 16384) + kb, umma_desc_kmajor(wb_s + (ks >> 2) * 16384) + kb,
                  idesc, ks != 0 ? 1u : 0u);
      }
      umma_commit(mma_bar);
    }
    ok &= mma_wait();
    tc_fence_after();
    uint32_t db_p[kBwdCh / 2], h_p[kBwdCh / 2];
#pragma unroll
    for (int ch = 0; ch < kBwdChunks; ++ch) {
      uint32_t v[8];
      tmem_ld8(tmem_base + lane_sel + part * kBwdCh + ch * 8, v);
      tmem_ld_wait();
      uint32_t da_p[4];
      const float4* cbp = reinterpret_cast<const float4*>(const_ptr + 128 + part * kBwdCh + ch * 8);
      const float4 cb0 = cbp[0], cb1 = cbp[1];
      const float cbv[8] = {cb0.x, cb0.y, cb0.z, cb0.w, cb1.x, cb1.y, cb1.z, cb1.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float dav[2], dbv[2], hv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i = ch * 8 + t * 2 + e;
          const float b = __uint_as_float(v[t * 2 + e]) + cbv[t * 2 + e];
          const float a = av[i];
          const float sg = sigmoid_fast(a);
          const float silu = a * sg;
          const float dsilu = sg * fmaf(a, 1.0f - sg, 1.0f);
          dav[e] = dh[i] * b * dsilu;
          dbv[e] = dh[i] * silu;
          hv[e] = silu * b;
        }
        da_p[t] = pack_f16x2_sat(make_float2(dav[0], dav[1]));
        db_p[ch * 4 + t] = pack_f16x2_sat(make_float2(dbv[0], dbv[1]));
        h_p[ch * 4 + t] = pack_f16x2_sat(make_float2(hv[0], hv[1]));
      }
      st_chunk(s_s + tile_chunk(pos, part * kBwdChunks + ch), da_p[0], da_p[1], da_p[2], da_p[3]);
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    // ---- d x_hat = da Wa_j' (working columns), Ma += da^T x_hat (columns 128-255)
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc_d = umma_idesc(128, 128, false, true, kFmtF16, kFmtF16);
      constexpr uint32_t idesc_m = umma_idesc(128, 128, true, true, kFmtF16, kFmtF16);
      const uint32_t accum = it != 0 ? 1u : 0u;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_bf16(tmem_base, umma_desc_kmajor(s_s + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2),
                  umma_desc_mnmajor(wa_s + ks * 2048, 16384), idesc_d, ks != 0 ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_bf16(tmem_base + 128, umma_desc_mnmajor(s_s + ks * 2048, 16384), umma_desc_mnmajor(x_s + ks * 2048, 16384),
                  idesc_m, (ks != 0 ? 1u : 0u) | accum);
      umma_commit(mma_bar);
    }
    column_sum(sa_acc);  // reads the tile the MMAs read
    ok &= mma_wait();
    named_bar_sync(1, kBwdThreads);  // every thread's column-sum reads come before the tile is rewritten
    // ---- db -> scratch; d x_hat += db Wb_j', Mb += db^T x_hat (columns 256-383)
#pragma unroll
    for (int ch = 0; ch < kBwdChunks; ++ch)
      st_chunk(s_s + tile_chunk(pos, part * kBwdChunks + ch), db_p[ch * 4], db_p[ch * 4 + 1], db_p[ch * 4 + 2], db_p[ch * 4 + 3]);
    fence_proxy_async_smem();
    __syncthreads();
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc_d = umma_idesc(128, 128, false, true, kFmtF16, kFmtF16);
      constexpr uint32_t idesc_m = umma_idesc(128, 128, true, true, kFmtF16, kFmtF16);
      const uint32_t accum = it != 0 ? 1u : 0u;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_bf16(tmem_base, umma_desc_kmajor(s_s + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2),
                  umma_desc_mnmajor(wb_s + ks * 2048, 16384), idesc_d, 1u);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_bf16(tmem_base + 256, umma_desc_mnmajor(s_s + ks * 2048, 16384), umma_desc_mnmajor(x_s + ks * 2048, 16384),
                  idesc_m, (ks != 0 ? 1u : 0u) | accum);
      umma_commit(mma_bar);
    }
    column_sum(sb_acc);
    ok &= mma_wait();
    named_bar_sync(1, kBwdThreads);
    // ---- h -> scratch; dWs_j += dy^T h (columns 384-511; lanes = channels c, columns = hidden units)
#pragma unroll
    for (int ch = 0; ch < kBwdChunks; ++ch)
      st_chunk(s_s + tile_chunk(pos, part * kBwdChunks + ch), h_p[ch * 4], h_p[ch * 4 + 1], h_p[ch * 4 + 2], h_p[ch * 4 + 3]);
    fence_proxy_async_smem();
    __syncthreads();
    if (threadIdx.x == 0) {
      tc_fence_after();
      constexpr uint32_t idesc_m = umma_idesc(128, 128, true, true, kFmtF16, kFmtF16);
      const uint32_t accum = it != 0 ? 1u : 0u;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_bf16(tmem_base + 384, umma_desc_mnmajor(y_s + ks * 2048, 16384), umma_desc_mnmajor(s_s + ks * 2048, 16384),
                  idesc_m, (ks != 0 ? 1u : 0u) | accum);
      umma_commit(mma_bar);
    }
    // the earlier launches' running d x_hat for this thread: requested now, used after the GEMM round
    const long long gp = static_cast<long long>(p0) + pos;
    const bool inside = gp < p.positions;
    uint4 dx_prev[kBwdChunks];
#pragma unroll
    for (int ch = 0; ch < kBwdChunks; ++ch) dx_prev[ch] = make_uint4(0u, 0u, 0u, 0u);
    if constexpr (!FIRST) {
      if (inside) {
        const uint4* src = reinterpret_cast<const uint4*>(p.dx_in + gp * 128 + part * kBwdCh);
        ldg_chunks(src, true, dx_prev);  // the workspace is 1024-byte aligned
      }
    }
    ok &= mma_wait();
    tc_fence_after();
    if constexpr (!LAST) {
      // x_hat and dy * c have been read for the last time: the next tile's inputs land while this one finishes
      if (threadIdx.x == 0 && tile + static_cast<int>(gridDim.x) < p.num_tiles) issue_inputs((tile + gridDim.x) * 128);
    }
    // ---- the running d x_hat: add the earlier launches' sum; LAST: LayerNorm backward + residual -> dx (bf16)
    {
      float tot[kBwdCh];
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int ch = 0; ch < kBwdChunks; ++ch) {
        uint32_t v[8];
        tmem_ld8(tmem_base + lane_sel + part * kBwdCh + ch * 8, v);
        const uint4 in = dx_prev[ch];
        uint4 xh = make_uint4(0u, 0u, 0u, 0u);
        if constexpr (LAST) xh = ld_chunk(x_s + tile_chunk(pos, part * kBwdChunks + ch));
        tmem_ld_wait();
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
        for (int ch = 0; ch < kBwdChunks; ++ch)
          st_chunk(s_s + tile_chunk(pos, part * kBwdChunks + ch), pack_f16x2_sat(make_float2(tot[ch * 8], tot[ch * 8 + 1])),
                   pack_f16x2_sat(make_float2(tot[ch * 8 + 2], tot[ch * 8 + 3])),
                   pack_f16x2_sat(make_float2(tot[ch * 8 + 4], tot[ch * 8 + 5])),
                   pack_f16x2_sat(make_float2(tot[ch * 8 + 6], tot[ch * 8 + 7])));
      } else {
        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xchg + kBwdXchgHalf + (part * 128 + pos) * 8), "f"(s1), "f"(s2)
                     : "memory");
        named_bar_sync(1, kBwdThreads);
        float m1, m2;
        sum_partials(xchg + kBwdXchgHalf, pos, m1, m2);
        m1 *= 1.0f / 128.0f, m2 *= 1.0f / 128.0f;
        const float rs = rstd_in * gc_inv;
        const float res = p.residual ? gc_inv : 0.f;  // the dy tile holds dy * c
#pragma unroll
        for (int ch = 0; ch < kBwdChunks; ++ch) {
          const uint4 xh = ld_chunk(x_s + tile_chunk(pos, part * kBwdChunks + ch));
          const uint4 dyv = ld_chunk(y_s + tile_chunk(pos, part * kBwdChunks + ch));
          const uint32_t xw[4] = {xh.x, xh.y, xh.z, xh.w};
          const uint32_t dw[4] = {dyv.x, dyv.y, dyv.z, dyv.w};
          uint32_t o[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 x = f16x2_to_float2(xw[t]);
            const float2 r = f16x2_to_float2(dw[t]);
            o[t] = pack_bf16x2(fmaf(rs, tot[ch * 8 + 2 * t] - m1 - x.x * m2, r.x * res),
                               fmaf(rs, tot[ch * 8 + 2 * t + 1] - m1 - x.y * m2, r.y * res));
          }
          st_chunk(s_s + tile_chunk(pos, part * kBwdChunks + ch), o[0], o[1], o[2], o[3]);
        }
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    ok = __syncthreads_and(ok ? 1 : 0) != 0;  // a thread that gave up takes the whole CTA out here
    if (!ok) break;
    if (threadIdx.x == 0) {
#pragma unroll
      for (int kh = 0; kh < 2; ++kh) tma_store_2d(&map_out, s_s + kh * 16384, kh * 64, p0);
      bulk_commit();
    }
  }
  if (threadIdx.x == 0) {
    if (loads_pending || !ok) {
      const long long t0 = clock64();
      while (!mbar_try_wait(w_full, 0) || (loads_pending && !mbar_try_wait(in_full, it & 1))) {
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
    tc_fence_after();
    float* pm = p.part_m + static_cast<size_t>(blockIdx.x) * 3 * 128 * 128;
#pragma unroll
    for (int m = 0; m < 3; ++m) {
#pragma unroll
      for (int ch = 0; ch < kBwdChunks; ++ch) {
        uint32_t v[8];
        tmem_ld8(tmem_base + lane_sel + 128 + m * 128 + part * kBwdCh + ch * 8, v);
        tmem_ld_wait();
        float4* dst = reinterpret_cast<float4*>(pm + (m * 128 + pos) * 128 + part * kBwdCh + ch * 8);
        dst[0] = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]), __uint_as_float(v[3]));
        dst[1] = make_float4(__uint_as_float(v[4]), __uint_as_float(v[5]), __uint_as_float(v[6]), __uint_as_float(v[7]));
      }
    }
  }
  {  // the 32 row groups of a hidden unit, fixed order (every tile region is free by now); the sums go to quarter 0
    float* sc = reinterpret_cast<float*>(smem);  // [32 row groups][2][128]
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      sc[((threadIdx.x >> 4) * 2 + 0) * 128 + sum_chunk * 8 + c] = sa_acc[c];
      sc[((threadIdx.x >> 4) * 2 + 1) * 128 + sum_chunk * 8 + c] = sb_acc[c];
    }
    __syncthreads();
    float* ps = p.part_s + static_cast<size_t>(blockIdx.x) * 2 * 512;
    float sum = 0.f;
    if (threadIdx.x < 256)
      for (int g = 0; g < 32; ++g) sum += sc[g * 256 + threadIdx.x];
    __syncthreads();
    // [vector][quarter][hidden unit]: threads 0-255 hold (vector, unit); quarters 1-3 are zero
    if (threadIdx.x < 256) ps[(threadIdx.x >> 7) * 512 + (threadIdx.x & 127)] = sum;
    else ps[((threadIdx.x - 256) >> 7) * 512 + 128 + (threadIdx.x & 127)] = 0.f;
    ps[(threadIdx.x >> 8) * 512 + 256 + (threadIdx.x & 255)] = 0.f;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------- small kernels
// Packed weights of the Transition's backward: Wa' = fp16(Wa gamma) [512][128], Wb' likewise, Ws fp16 [128][512],
// then ca = Wa beta [512], cb = Wb beta [512] (fp32). One warp per row of Wa / Wb; Ws converted elementwise.
constexpr size_t kTrBwdWa = 0, kTrBwdWb = 512 * 128 * 2, kTrBwdWs = 2 * 512 * 128 * 2, kTrBwdConst = 3 * 512 * 128 * 2;
constexpr size_t kTrBwdPackedBytes = kTrBwdConst + 2 * 512 * 4;  // 397312, a multiple of 1024
struct TrBwdPackArgs {
  const void* w_a;
  const void* w_b;
  const void* w_s;
  const float* ln_w;
  const float* ln_b;
  int f32_weights;
};
__device__ __forceinline__ float tr_load_w(const void* w, size_t i, int f32) {
  return f32 ? static_cast<const float*>(w)[i]
             : __uint_as_float(static_cast<uint32_t>(static_cast<const uint16_t*>(w)[i]) << 16);
}
__global__ void __launch_bounds__(128) tr_bwd_pack_kernel(const TrBwdPackArgs a, uint8_t* packed) {
  const int gw = blockIdx.x * 4 + (threadIdx.x >> 5);  // 0 .. 1535: rows of Wa (0-511), Wb (512-1023), then Ws rows by 4
  const int lane = threadIdx.x & 31;
  if (gw < 1024) {
    const int m = gw >> 9, row = gw & 511;
    const void* w = m == 0 ? a.w_a : a.w_b;
    float d = 0.f;
    uint16_t o[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int k = lane * 4 + t;
      const float v = tr_load_w(w, static_cast<size_t>(row) * 128 + k, a.f32_weights);
      o[t] = __half_as_ushort(__float2half_rn(fminf(fmaxf(v * a.ln_w[k], -65504.f), 65504.f)));
      d = fmaf(v, a.ln_b[k], d);
    }
    uint2 ov;
    ov.x = static_cast<uint32_t>(o[0]) | (static_cast<uint32_t>(o[1]) << 16);
    ov.y = static_cast<uint32_t>(o[2]) | (static_cast<uint32_t>(o[3]) << 16);
    reinterpret_cast<uint2*>(packed + (m == 0 ? kTrBwdWa : kTrBwdWb))[row * 32 + lane] = ov;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, off);
    if (lane == 0) reinterpret_cast<float*>(packed + kTrBwdConst)[m * 512 + row] = d;
  } else {
    // Ws [128][512]: warp gw - 1024 (0 .. 511) converts 128 consecutive elements
    const size_t base = static_cast<size_t>(gw - 1024) * 128;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const size_t i = base + lane * 4 + t;
      const float v = tr_load_w(a.w_s, i, a.f32_weights);
      reinterpret_cast<uint16_t*>(packed + kTrBwdWs)[i] = __half_as_ushort(__float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f)));
    }
  }
}

// m_out[e] (3 x 128 x 128 values: blocks 0 .. 767) and s_out[e] (2 x 512 values: blocks 768 .. 783) = sums over the CTAs'
// partials; a block covers 64 elements, its four groups of 64 threads take every fourth partial and are combined in a
// fixed order.
__global__ void __launch_bounds__(256) tr_bwd_reduce_kernel(const float* part_m, const float* part_s, int n_parts, float* m_out,
                                                            float* s_out) {
  __shared__ float comb[4][64];
  const bool is_s = blockIdx.x >= 768;
  const float* parts = is_s ? part_s : part_m;
  const size_t stride = is_s ? 2 * 512 : 3 * 128 * 128;
  const int el = threadIdx.x & 63, g = threadIdx.x >> 6;
  const int e = (is_s ? blockIdx.x - 768 : blockIdx.x) * 64 + el;
  comb[g][el] = sum_every_fourth(parts, stride, n_parts, e, g);
  __syncthreads();
  if (g == 0) (is_s ? s_out : m_out)[e] = (comb[0][el] + comb[1][el]) + (comb[2][el] + comb[3][el]);
}

// Parameter gradients of the Transition from the reduced sums of all four blocks:
//   m_all [4][3][128][128] (Ma_j, Mb_j: [hidden][k]; dWs_j: [c][hidden]), s_all [4][2][4][128] (column sums per quarter)
//   dWa[j*128+r][k] = (Ma_j[r][k] gamma[k] + sa_j[r] beta[k]) / c, dWb likewise, dWs[c][j*128+h] = dWs_j[c][h] / c
//   dgamma[k] = sum_j sum_r (Wa Ma + Wb Mb) / c,  dbeta[k] = sum_j sum_r (Wa sa + Wb sb) / c
// Grid (4 blocks j, 8 row groups of 16), thread = column; LayerNorm partials [4][8][2][128] added by tr_bwd_final_ln_kernel.
struct TrBwdFinalArgs {
  TrBwdPackArgs w;
  const float* m_all;
  const float* s_all;
  const float* scale;
  float* d_wa;    // [512][128]
  float* d_wb;    // [512][128]
  float* d_ws;    // [128][512]
  float* ln_part; // [4][8][2][128]
  float* d_ln_w;  // [128]
  float* d_ln_b;
};
__global__ void __launch_bounds__(128) tr_bwd_final_kernel(const TrBwdFinalArgs a) {
  const int k = threadIdx.x, j = blockIdx.x, rb = blockIdx.y;
  const float cinv = a.scale[1];
  const float gamma = a.w.ln_w[k], beta = a.w.ln_b[k];
  float ag = 0.f, ab = 0.f;
  for (int r = rb * 16; r < rb * 16 + 16; ++r) {
    const float* sq = a.s_all + static_cast<size_t>(j) * 2 * 512;
    const float sa = (sq[r] + sq[128 + r] + sq[256 + r] + sq[384 + r]) * cinv;
    const float sb = (sq[512 + r] + sq[512 + 128 + r] + sq[512 + 256 + r] + sq[512 + 384 + r]) * cinv;
    const float ma = a.m_all[((static_cast<size_t>(j) * 3 + 0) * 128 + r) * 128 + k] * cinv;
    const float mb = a.m_all[((static_cast<size_t>(j) * 3 + 1) * 128 + r) * 128 + k] * cinv;
    const size_t wi = static_cast<size_t>(j * 128 + r) * 128 + k;
    const float wa = tr_load_w(a.w.w_a, wi, a.w.f32_weights), wb = tr_load_w(a.w.w_b, wi, a.w.f32_weights);
    a.d_wa[wi] = fmaf(ma, gamma, sa * beta);
    a.d_wb[wi] = fmaf(mb, gamma, sb * beta);
    ag = fmaf(wa, ma, fmaf(wb, mb, ag));
    ab = fmaf(wa, sa, fmaf(wb, sb, ab));
    // dWs: row c = r (of this row group), column block j, column h = k
    a.d_ws[static_cast<size_t>(r) * 512 + j * 128 + k] = a.m_all[((static_cast<size_t>(j) * 3 + 2) * 128 + r) * 128 + k] * cinv;
  }
  a.ln_part[((j * 8 + rb) * 2 + 0) * 128 + k] = ag;
  a.ln_part[((j * 8 + rb) * 2 + 1) * 128 + k] = ab;
}
__global__ void __launch_bounds__(128) tr_bwd_final_ln_kernel(const TrBwdFinalArgs a) {
  const int k = threadIdx.x;
  float g = 0.f, b = 0.f;
  for (int i = 0; i < 32; ++i) {
    g += a.ln_part[(i * 2 + 0) * 128 + k];
    b += a.ln_part[(i * 2 + 1) * 128 + k];
  }
  a.d_ln_w[k] = g;
  a.d_ln_b[k] = b;
}

}  // namespace trimul
