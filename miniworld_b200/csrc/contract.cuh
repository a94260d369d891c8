// Per-channel triangle contraction on tcgen05 tensor cores.
//
//   outgoing: t[b,i,h,j] = sum_k a[b,i,h,k] * b[b,j,h,k]     (both operands K-major in shared memory)
//   incoming: t[b,i,h,j] = sum_k a[b,k,h,i] * b[b,k,h,j]     (both operands MN-major, no transpose pass)
//   mixed:    t[b,i,h,j] = sum_k a[b,i,h,k] * b[b,k,h,j]     (a K-major, b MN-major: a plain per-plane product,
//                                                              which the gradients of the two forms above need)
//
// a, b and t are stored "row-plane": [B, rows, H, N] fp16 (for each row a [H, N] slab), so the rows of
// a row-sharded operand gathered from several ranks are one uniform strided dimension.  fp16 rather than
// bf16: the tensor-core rate is the same and the three extra mantissa bits are what keeps the module
// output within its max-abs bound; t is stored as t * 2^-4, saturated to the fp16 range (the output
// LayerNorm that consumes it is scale invariant once its eps is scaled by 2^-8).
//
// One persistent CTA per SM walks output tiles of 128 x BN in plane-major order (all tiles of one
// (b, h) plane before the next, so the plane's operands stay in L2).  Warp roles: warp 0 = TMA
// producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 = epilogue (TMEM -> fp16 -> swizzled shared
// staging -> TMA store).  Two TMEM accumulators of BN columns let the epilogue of one tile overlap the
// mainloop of the next.
#pragma once

#include "ptx.cuh"

namespace trimul {

struct ContractParams {
  int H;          // channels per batch sample
  int planes;     // B * H
  int m_tiles;    // output row tiles (128 rows)
  int n_tiles;    // output column tiles (BN columns)
  int num_kb;     // 64-deep k blocks
  int a_col_off;  // incoming only: first output row, as a column offset into a's inner dimension
  int n_cols;     // output columns (N)
  int m_rows;     // output rows of this call
  int* status;
};

// Output destinations of the channel-sharded multi-GPU form (CTA-pair kernel only): output row r belongs to GPU
// r / rows_per_owner, and every box_rows-row slice of a finished tile is stored (plain TMA store, peer memory over
// NVLink for the other GPUs) into that owner's buffer [rows_per_owner][channels][N] at row r % rows_per_owner.
// n == 0: one destination, the `tri` tensor map of the call.
constexpr int kMaxOwners = 8;
struct TriOwners {
  CUtensorMap m[kMaxOwners];
  int n;
  int rows_per_owner;
  int box_rows;  // 128, 64 or 32; divides rows_per_owner
};

constexpr int kContractThreads = 192;
constexpr int kContractStages = 4;
constexpr int kBM = 128;
constexpr int kBK = 64;

constexpr int kContractOutgoing = 0;
constexpr int kContractIncoming = 1;
constexpr int kContractMixed = 2;

constexpr float kTriScale = 0.0625f;  // t is stored as t * 2^-4

// two fp32 accumulators -> scaled, saturated fp16 pair
__device__ __forceinline__ uint32_t pack_tri(uint32_t lo_bits, uint32_t hi_bits) {
  return pack_f16x2_sat(
      __fmul2_rn(make_float2(__uint_as_float(lo_bits), __uint_as_float(hi_bits)), make_float2(kTriScale, kTriScale)));
}

template <int BN>
struct ContractSmem {
  static constexpr int kABytes = kBM * kBK * 2;             // 16 KiB
  static constexpr int kBBytes = BN * kBK * 2;              // BN * 128 B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = 2 * 128 * 128;       // two 64-column sub-tiles
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kContractStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};

template <int BN, int MODE>
__global__ void __launch_bounds__(kContractThreads, 1)
contract_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_t, const ContractParams p) {
  using L = ContractSmem<BN>;
  constexpr int S = kContractStages;
  constexpr bool A_MN = MODE == kContractIncoming;  // A operand MN-major (its k index is the tensor's row)
  constexpr bool B_MN = MODE != kContractOutgoing;  // B operand MN-major
  constexpr uint32_t kTmemCols = (2 * BN > 256) ? 512u : 256u;
  constexpr uint32_t kAccStride = kTmemCols / 2;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_base = smem_base;
  const uint32_t staging_base = smem_base + S * L::kStageBytes;
  const uint32_t bar_base = staging_base + L::kStagingBytes;
  // barriers: full[S], empty[S], tmem_full[2], tmem_empty[2]; then tmem base word, abort word
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_aligned + S * L::kStageBytes + L::kStagingBytes + 8 * (2 * S + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    prefetch_tmap(&map_t);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_plane = p.m_tiles * p.n_tiles;
  const int num_tiles = p.planes * tiles_per_plane;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      int issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const int plane = tile / tiles_per_plane;
        const int r = tile - plane * tiles_per_plane;
        const int mt = r / p.n_tiles;
        const int nt = r - mt * p.n_tiles;
        const int bb = plane / p.H;
        const int hh = plane - bb * p.H;
        const int m0 = mt * kBM;
        const int n0 = nt * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full_bar(s), L::kStageBytes);
          const uint32_t sa = stage_base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
          const int k0 = kb * kBK;
          if constexpr (!A_MN) {
            tma_load_4d(sa, &map_a, full_bar(s), k0, m0, hh, bb);
          } else {
#pragma unroll
            for (int hf = 0; hf < kBM / 64; ++hf)
              tma_load_4d(sa + hf * 8192, &map_a, full_bar(s), p.a_col_off + m0 + 64 * hf, k0, hh, bb);
          }
          if constexpr (!B_MN) {
            tma_load_4d(sb, &map_b, full_bar(s), k0, n0, hh, bb);
          } else {
#pragma unroll
            for (int hf = 0; hf < BN / 64; ++hf)
              tma_load_4d(sb + hf * 8192, &map_b, full_bar(s), n0 + 64 * hf, k0, hh, bb);
          }
          ++issued;
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      // Drain: every copy this thread started must have landed before the CTA may exit.
      const int pending = issued < S ? issued : S;
      for (int q = 0; q < pending; ++q) {
        if (s == 0) {
          s = S;
          ph ^= 1u;
        }
        --s;
        const long long t0 = clock64();
        while (!mbar_try_wait(full_bar(s), ph)) {
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
      constexpr uint32_t idesc = umma_idesc(kBM, BN, A_MN, B_MN, kFmtF16, kFmtF16);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.status, kDevTimeoutMma)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccStride;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, kDevTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = stage_base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
          // descriptor start-address step per 16-deep MMA, in 16-byte units: 32 bytes along a K-major row, sixteen
          // 128-byte rows of an MN-major tile
          const uint64_t da = A_MN ? umma_desc_mnmajor(sa, 8192) : umma_desc_kmajor(sa);
          const uint64_t db = B_MN ? umma_desc_mnmajor(sb, 8192) : umma_desc_kmajor(sb);
          constexpr uint32_t kstep_a = A_MN ? (2048 >> 4) : (32 >> 4);
          constexpr uint32_t kstep_b = B_MN ? (2048 >> 4) : (32 >> 4);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            umma_bf16(d_tmem, da + static_cast<uint64_t>(k * kstep_a), db + static_cast<uint64_t>(k * kstep_b), idesc,
                      (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5)
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;       // output row inside the tile
    const bool store_thread = (threadIdx.x == 64);
    int it = 0;
    int group_counter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
      const int plane = tile / tiles_per_plane;
      const int r = tile - plane * tiles_per_plane;
      const int mt = r / p.n_tiles;
      const int nt = r - mt * p.n_tiles;
      const int bb = plane / p.H;
      const int hh = plane - bb * p.H;
      const int m0 = mt * kBM;
      const int n0 = nt * BN;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      const bool got = mbar_wait_warp(tfull_bar(acc), acc_ph, abort_flag, p.status, kDevTimeoutEpilogue);
      if (!named_bar_and(1, 128, got)) break;  // the four warps leave together or not at all
      tc_fence_after();
      const uint32_t t_acc = tmem_base + acc * kAccStride + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int g = 0; g < BN / 64; ++g, ++group_counter) {
        const uint32_t buf = staging_base + (group_counter & 1) * 16384u;
        if (store_thread) bulk_wait_read<1>();
        named_bar_sync(1, 128);
        uint32_t v0[32], v1[32];
        tmem_ld32(t_acc + g * 64, v0);
        tmem_ld32(t_acc + g * 64 + 32, v1);
        tmem_ld_wait();
        if (g == BN / 64 - 1) {
          // all TMEM reads of this accumulator are done: hand it back to the MMA issuer
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
        const uint32_t row_addr = buf + row * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 w;
          w.x = pack_tri(v0[8 * c + 0], v0[8 * c + 1]);
          w.y = pack_tri(v0[8 * c + 2], v0[8 * c + 3]);
          w.z = pack_tri(v0[8 * c + 4], v0[8 * c + 5]);
          w.w = pack_tri(v0[8 * c + 6], v0[8 * c + 7]);
          const uint32_t addr = row_addr + ((c ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w)
                       : "memory");
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 w;
          w.x = pack_tri(v1[8 * c + 0], v1[8 * c + 1]);
          w.y = pack_tri(v1[8 * c + 2], v1[8 * c + 3]);
          w.z = pack_tri(v1[8 * c + 4], v1[8 * c + 5]);
          w.w = pack_tri(v1[8 * c + 6], v1[8 * c + 7]);
          const uint32_t addr = row_addr + (((c + 4) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w)
                       : "memory");
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (store_thread) {
          const int col0 = n0 + g * 64;
          if (col0 < p.n_cols) tma_store_4d(&map_t, buf, col0, m0, hh, bb);
          bulk_commit();
        }
      }
    }
    if (store_thread) bulk_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace trimul
