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
// Persistent CTA pairs (tcgen05 cta_group::2), one pair per two SMs, walk tiles of 128 consecutive columns j
// of one pair row (b, i). The GEMMs are issued as D^T[h, pos] = W[h, c] * x_hat^T[c, pos], so TMEM lanes are
// channels and columns are positions: each epilogue thread owns one channel and writes runs of consecutive
// positions, which is exactly the row-plane layout [B, rows, H, N] of the outputs (written as fp16; masked
// cells are exactly zero).
//
// The two CTAs of a pair split the OUTPUTS: CTA 0 produces `left`, CTA 1 produces `right`, each holding only
// its own two matrices (64 KiB), which leaves room for five input stages and two staging buffers. Every MMA
// spans both CTAs (M = 256: rows 0-127 are CTA 0's matrix, rows 128-255 CTA 1's matrix at the same
// shared-memory offset; N = 128 positions, of which each CTA loads and normalises 64). So per tile each CTA
//   * loads and LayerNorms 64 positions,
//   * receives proj / gate accumulators of ITS output for all 128 positions in its own TMEM (2 x 128 columns,
//     double-buffered: the MMAs of tile t+1 overlap the epilogue of tile t),
//   * gates, masks and stores 128 channels x 128 positions of its output.
// Only mbarrier signals cross between the CTAs (statistics-done and accumulator-free arrive on the leader's
// barriers; the leader's MMA commits release both CTAs' barriers); no tile is broadcast. A single-CTA version
// of this kernel (all four matrices resident, two input stages) measured 3 % slower at N = 768.
//
// Outputs leave through a swizzled shared-memory staging tile and TMA stores (full 128-byte rows);
// direct per-thread 16-byte stores to 128 different channel rows ran the store path at a third of this.
//
// Warp roles (864 threads per CTA):
//   warp 0        TMA producer (input tiles, this CTA's weights once)
//   warp 1        MMA issuer (leader CTA) / TMEM owner
//   warps 2-9     LayerNorm: 8 threads per position (16 channels each, their gamma / beta in registers), two
//                 passes of 32 positions computed as independent chains; normalises the tile in place.
//   warps 10-25   epilogue: two groups of eight warps on alternate tiles (one thread per channel x 64 positions:
//                 TMEM -> tanh gate -> mask -> staging -> TMA store)
//   warp 26       validity bitmap of the tile
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

// Where the outputs go. Each output has a list of destination tensor maps; a finished tile [128 channels][128
// positions] of local row r is stored to every destination d of its list at row r + row_shift, taking the
// channels d * smem_step / 128 ... of the staging tile (smem_step = 0: every destination gets all 128 channels).
//   one GPU:            one destination per output, the [B*rows, 128, N] buffers, row_shift 0
//   rows over GPUs:     `right` additionally to the peers' gathered copies [N, 128, N] (row_shift = first local row)
//   channels over GPUs: destination d = the GPU that contracts channel group d; it receives the 128/P channels of
//                       its group for this GPU's rows, in its [N, 128/P, N] buffer (smem_step = 128/P channel rows)
// Peer destinations are plain (non-multicast) TMA stores over NVLink; they replace a separate collective pass.
constexpr int kMaxDst = 8;
struct OutputMaps {
  CUtensorMap left[kMaxDst];
  CUtensorMap right[kMaxDst];
  int n_left, n_right;
  int step_left, step_right;    // bytes between the destinations' channel slices in a 16 KiB half staging tile
  int shift_left, shift_right;  // added to the row coordinate
  // One GPU: the same two outputs with a box of 32 channel rows, so that every epilogue warp stores the 32 rows it
  // wrote by itself and the warps of a group never wait for one another (warp_store != 0).
  CUtensorMap left_warp, right_warp;
  int warp_store;
};

constexpr int kProThreads = 864;
constexpr int kProStages = 5;
constexpr int kProRing = 8;              // mask ring entries (>= stages + 3)
constexpr int kProRingBytes = 272;       // 64 pair-mask words + 4 ballots
constexpr int kProStageOutBytes = 2 * 32768;  // two staging buffers of [128 channels][128 positions]
constexpr int kProBarBytes = 256;
// C = d_pair, the channels of the input tensor (128, or 64 for the narrow pair stacks); the outputs always have 128
// channels. The shared-memory budget is that of C = 128 for both.
constexpr int kProSmemBytes =
    2 * 32768 + kProStages * 16384 + kProStageOutBytes + kProRing * kProRingBytes + kProBarBytes + 1024;

template <bool HAS_BIAS, int C = 128>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kProThreads, 1)
prologue_kernel(const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ OutputMaps out, const PrologueParams p) {
  static_assert(C == 128 || C == 64, "d_pair is 128 or 64");
  constexpr int S = kProStages;
  constexpr int kHalves = C / 64;              // 64-channel (128-byte) halves of an input row
  constexpr int kProWBytes = 2 * 128 * C * 2;  // this CTA's proj and gate matrices, [128, C] fp16 each
  constexpr int kProZBytes = 64 * C * 2;       // 64 positions x C channels, 16-bit
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t w_base = smem_base;
  const uint32_t z_base = smem_base + kProWBytes;
  const uint32_t stage_out_base = z_base + S * kProZBytes;
  const uint32_t ring_base = stage_out_base + kProStageOutBytes;
  const uint32_t bar_base = ring_base + kProRing * kProRingBytes;
  uint32_t* ring_ptr = reinterpret_cast<uint32_t*>(smem + kProWBytes + S * kProZBytes + kProStageOutBytes);
  // barriers: w_full (leader), z_full[S] (own), xn_ready[S] (leader), z_empty[S] (both), acc_full[2] (both),
  // acc_empty[2] (leader)
  const uint32_t w_full = bar_base;
  auto z_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto xn_ready = [&](int s) { return bar_base + 8u * (1 + S + s); };
  auto z_empty = [&](int s) { return bar_base + 8u * (1 + 2 * S + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (1 + 3 * S + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (1 + 3 * S + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kProWBytes + S * kProZBytes + kProStageOutBytes +
                                                    kProRing * kProRingBytes + 8 * (1 + 3 * S + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: leader, produces `left`; 1: produces `right`
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int s = 0; s < S; ++s) {
      mbar_init(z_full(s), 1);
      mbar_init(xn_ready(s), 18);  // eight LayerNorm warps and the mask warp of each CTA
      mbar_init(z_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full(a), 1);
      mbar_init(acc_empty(a), 16);  // the eight warps of epilogue group a in each CTA
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&map_z);
    prefetch_tmap(&map_w);
    prefetch_tmap(&out.left[0]);
    prefetch_tmap(&out.right[0]);
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      // this CTA's two matrices: packed order is left, left gate, right, right gate
      if (rank == 0) mbar_arrive_expect_tx(w_full, 2 * kProWBytes);  // bytes of both CTAs
      const uint32_t lead_w = map_to_cta(w_full, 0);
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int kh = 0; kh < kHalves; ++kh)
          tma_load_2d_pair(w_base + m * (kProWBytes / 2) + kh * 16384, &map_w, lead_w, kh * 64,
                           (static_cast<int>(rank) * 2 + m) * 128);
      int s = 0;
      uint32_t ph = 0;
      int issued = 0;
      for (int tile = pair; tile < p.num_tiles; tile += num_pairs) {
        if (!mbar_wait(z_empty(s), ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) break;
        const int row = tile / p.tiles_per_row;
        const int j0 = (tile - row * p.tiles_per_row) * 128 + static_cast<int>(rank) * 64;  // this CTA's 64 positions
        mbar_arrive_expect_tx(z_full(s), kProZBytes);
#pragma unroll
        for (int kh = 0; kh < kHalves; ++kh) tma_load_3d(z_base + s * kProZBytes + kh * 8192, &map_z, z_full(s), kh * 64, j0, row);
        ++issued;
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
      // Drain every copy this thread started before the CTA may exit (the weights report to the leader, whose
      // MMA thread waits for them; the closing cluster barrier keeps this CTA alive until then).
      if (rank == 0) {
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
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc(256, 128, false, false, kFmtF16, kFmtF16);
      bool ok = mbar_wait(w_full, 0, abort_flag, p.status, kDevTimeoutMma);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      for (int tile = pair; ok && tile < p.num_tiles; tile += num_pairs, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(xn_ready(s), ph, abort_flag, p.status, kDevTimeoutMma)) break;
        if (!mbar_wait(acc_empty(buf), ((it >> 1) & 1) ^ 1u, abort_flag, p.status, kDevTimeoutMma)) break;
        tc_fence_after();
        const uint32_t zs = z_base + s * kProZBytes;
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const uint32_t d_tmem = tmem_base + buf * 256 + m * 128;
          const uint32_t wm = w_base + m * (kProWBytes / 2);
#pragma unroll
          for (int ks = 0; ks < C / 16; ++ks) {
            const uint64_t da = umma_desc_kmajor(wm + (ks >> 2) * 16384) + static_cast<uint64_t>((ks & 3) * 2);
            const uint64_t db = umma_desc_kmajor(zs + (ks >> 2) * 8192) + static_cast<uint64_t>((ks & 3) * 2);
            umma_pair(d_tmem, da, db, idesc, ks != 0 ? 1u : 0u);
          }
        }
        umma_commit_pair(acc_full(buf));
        umma_commit_pair(z_empty(s));
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp < 10) {
#include "prologue_stats.inc"
  } else if (warp < 26) {
#include "prologue_epilogue.inc"
  } else {
#include "prologue_mask.inc"
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

}  // namespace trimul
