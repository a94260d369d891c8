// Triangle contraction with CTA pairs (tcgen05 cta_group::2): one 256 x BN output tile per pair of SMs.
//
// Same math, layouts and tile order as contract.cuh. Two CTAs of a 2-CTA cluster share every MMA: each
// supplies its own 128 rows of the A operand and its own half (BN/2 rows) of the B operand from its own
// shared memory, and each receives its 128 x BN slice of the accumulator in its own TMEM. Per 64-deep k
// block a CTA therefore loads 16 KiB + BN/2 * 128 B instead of 16 KiB + BN * 128 B: a third less L2 -> SM
// traffic and shared-memory read bandwidth for the same tensor work, which is what the single-CTA kernel
// is short of. No data is broadcast between the CTAs; only mbarrier signals cross:
//   * both producers' TMA loads report their bytes to the leader CTA's `full` barrier,
//   * the leader's MMA thread commits to the `empty` / `tmem_full` barriers of both CTAs,
//   * both CTAs' epilogue warps arrive on the leader's `tmem_empty` barrier.
#pragma once

#include "contract.cuh"

namespace trimul {

constexpr int kPairStages = 6;

template <int BN>
struct PairSmem {
  static constexpr int kABytes = kBM * kBK * 2;         // 16 KiB: this CTA's 128 rows of A
  static constexpr int kBBytes = (BN / 2) * kBK * 2;    // this CTA's half of B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = 2 * 128 * 128;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kPairStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};

// ContractParams::m_tiles counts 256-row pair tiles here.
template <int BN, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kContractThreads, 1)
contract_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_t, const __grid_constant__ TriOwners own,
                     const ContractParams p) {
  using L = PairSmem<BN>;
  constexpr int S = kPairStages;
  constexpr bool A_MN = MODE == kContractIncoming;  // A operand MN-major (its k index is the tensor's row)
  constexpr bool B_MN = MODE != kContractOutgoing;  // B operand MN-major
  constexpr uint32_t kTmemCols = (2 * BN > 256) ? 512u : 256u;
  constexpr uint32_t kAccStride = kTmemCols / 2;
  constexpr int kHalfN = BN / 2;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_base = smem_base;
  const uint32_t staging_base = smem_base + S * L::kStageBytes;
  const uint32_t bar_base = staging_base + L::kStagingBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  uint32_t* tmem_slot =
      reinterpret_cast<uint32_t*>(smem_aligned + S * L::kStageBytes + L::kStagingBytes + 8 * (2 * S + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader (issues the MMAs)
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // four epilogue warps in each of the two CTAs
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    prefetch_tmap(&map_t);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before any signal crosses
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_plane = p.m_tiles * p.n_tiles;
  const int num_tiles = p.planes * tiles_per_plane;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      int issued = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        const int plane = tile / tiles_per_plane;
        const int r = tile - plane * tiles_per_plane;
        const int mt = r / p.n_tiles;
        const int nt = r - mt * p.n_tiles;
        const int bb = plane / p.H;
        const int hh = plane - bb * p.H;
        const int m0 = mt * 256 + static_cast<int>(rank) * kBM;    // this CTA's rows of A / of the output
        const int n0 = nt * BN + static_cast<int>(rank) * kHalfN;  // this CTA's half of B
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) {
            ok = false;
            break;
          }
          if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * L::kStageBytes);  // bytes of both CTAs
          const uint32_t lead_full = map_to_cta(full_bar(s), 0);
          const uint32_t sa = stage_base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
          const int k0 = kb * kBK;
          if constexpr (!A_MN) {
            tma_load_4d_pair(sa, &map_a, lead_full, k0, m0, hh, bb);
          } else {
#pragma unroll
            for (int hf = 0; hf < kBM / 64; ++hf)
              tma_load_4d_pair(sa + hf * 8192, &map_a, lead_full, p.a_col_off + m0 + 64 * hf, k0, hh, bb);
          }
          if constexpr (!B_MN) {
            tma_load_4d_pair(sb, &map_b, lead_full, k0, n0, hh, bb);
          } else {
#pragma unroll
            for (int hf = 0; hf < kHalfN / 64; ++hf)
              tma_load_4d_pair(sb + hf * 8192, &map_b, lead_full, n0 + 64 * hf, k0, hh, bb);
          }
          ++issued;
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      // Drain (leader: its `full` barriers count the bytes of both CTAs; the closing cluster barrier keeps the
      // other CTA alive until then).
      if (rank == 0) {
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
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc(256, BN, A_MN, B_MN, kFmtF16, kFmtF16);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++it) {
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
          const uint64_t da = A_MN ? umma_desc_mnmajor(sa, 8192) : umma_desc_kmajor(sa);
          const uint64_t db = B_MN ? umma_desc_mnmajor(sb, 8192) : umma_desc_kmajor(sb);
          constexpr uint32_t kstep_a = A_MN ? (2048 >> 4) : (32 >> 4);
          constexpr uint32_t kstep_b = B_MN ? (2048 >> 4) : (32 >> 4);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            umma_pair(d_tmem, da + static_cast<uint64_t>(k * kstep_a), db + static_cast<uint64_t>(k * kstep_b), idesc,
                      (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(s));
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) umma_commit_pair(tfull_bar(acc));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5), both CTAs
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool store_thread = (threadIdx.x == 64);
    int it = 0;
    int group_counter = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
      const int plane = tile / tiles_per_plane;
      const int r = tile - plane * tiles_per_plane;
      const int mt = r / p.n_tiles;
      const int nt = r - mt * p.n_tiles;
      const int bb = plane / p.H;
      const int hh = plane - bb * p.H;
      const int m0 = mt * 256 + static_cast<int>(rank) * kBM;
      const int n0 = nt * BN;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      const bool got = mbar_wait_warp(tfull_bar(acc), acc_ph, abort_flag, p.status, kDevTimeoutEpilogue);
      if (!named_bar_and(1, 128, got)) break;
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
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
        }
        const uint32_t row_addr = buf + row * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t addr = row_addr + ((c ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_tri(v0[8 * c + 0], v0[8 * c + 1])),
                       "r"(pack_tri(v0[8 * c + 2], v0[8 * c + 3])), "r"(pack_tri(v0[8 * c + 4], v0[8 * c + 5])),
                       "r"(pack_tri(v0[8 * c + 6], v0[8 * c + 7]))
                       : "memory");
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t addr = row_addr + (((c + 4) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_tri(v1[8 * c + 0], v1[8 * c + 1])),
                       "r"(pack_tri(v1[8 * c + 2], v1[8 * c + 3])), "r"(pack_tri(v1[8 * c + 4], v1[8 * c + 5])),
                       "r"(pack_tri(v1[8 * c + 6], v1[8 * c + 7]))
                       : "memory");
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (store_thread) {
          const int col0 = n0 + g * 64;
          if (own.n == 0) {
            if (col0 < p.n_cols && m0 < p.m_rows) tma_store_4d(&map_t, buf, col0, m0, hh, bb);
          } else if (col0 < p.n_cols) {
            // each slice of rows to the GPU that owns those rows (a slice never straddles two owners)
            for (int r0 = 0; r0 < kBM && m0 + r0 < p.m_rows; r0 += own.box_rows) {
              const int owner = (m0 + r0) / own.rows_per_owner;
              tma_store_4d(&own.m[owner], buf + r0 * 128, col0, m0 + r0 - owner * own.rows_per_owner, hh, 0);
            }
          }
          bulk_commit();
        }
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
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace trimul
