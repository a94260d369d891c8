// C-ABI entry points of the B200 triangle-multiplication forward path (see include/b200_trimul.h).
// Host side only builds tensor maps, checks arguments and launches; all arithmetic is in the kernels.

#include "../../include/b200_trimul.h"

#include <atomic>
#include <mutex>

#include "contract.cuh"
#include "contract_pair.cuh"
#include "epilogue.cuh"
#include "epilogue_wide.cuh"
#include "prologue.cuh"
#include "transition.cuh"

namespace trimul {

constexpr int kC = 128;
constexpr size_t kStatusBytes = 1024;
constexpr size_t kPackedMatrixBytes = 6 * 32768;
constexpr size_t kPackedD1Off = kPackedMatrixBytes;            // float[4][128]
constexpr size_t kPackedC3Off = kPackedMatrixBytes + 2048;     // float4[128]
constexpr size_t kPackedLnOff = kPackedMatrixBytes + 4096;     // float[2][128]: input LayerNorm gamma, beta
constexpr size_t kPackedBytes = kPackedMatrixBytes + 5120;     // 201728, a multiple of 1024

static thread_local int tl_last_cuda_error = 0;

#define TRIMUL_CUDA(expr)                             \
  do {                                                \
    cudaError_t _e = (expr);                          \
    if (_e != cudaSuccess) {                          \
      tl_last_cuda_error = static_cast<int>(_e);      \
      return B200_TRIMUL_E_CUDA;                      \
    }                                                 \
  } while (0)

// ---------------------------------------------------------------------------------------------
// Weight packing: one warp per matrix row. C = d_pair (128 or 64); the contracted width is 128 in both cases.
//   matrices 0..3 (left, left gate, right, right gate) [128, C]: W' = fp16(0.5 W), d = 0.5 bias
//     (the prologue applies the input LayerNorm affine itself; gamma_in / beta_in are copied alongside)
//   matrix 4 (out)  [C, 128]: W' = fp16(0.5 W gamma_out), s = rowsum(W'), d = 0.5 (W beta_out + bias)
//   matrix 5 (gate) [C, C]:   W' = bf16(0.5 W gamma_in),  s = rowsum(W'), d = 0.5 (W beta_in + bias)
// Packed matrices are dense and follow one another: 0..3 at m * 128 * C * 2 bytes, 4 after them, 5 after 4.
struct PackArgs {
  const void* w[6];
  int ld[6];  // elements between consecutive rows of w[m] (128 for a matrix of its own, more for a column slice)
  const float* bias[6];
  const float* ln_in_w;
  const float* ln_in_b;
  const float* ln_out_w;
  const float* ln_out_b;
  int f32_weights;
  int c;  // d_pair
};

__host__ __device__ inline size_t packed_matrix_offset(int m, int c) {
  return m <= 4 ? static_cast<size_t>(m) * 128 * c * 2 : static_cast<size_t>(4) * 128 * c * 2 + static_cast<size_t>(c) * 128 * 2;
}

__global__ void __launch_bounds__(128) pack_kernel(const PackArgs a, uint8_t* packed) {
  const int gw = blockIdx.x * 4 + (threadIdx.x >> 5);  // 0 .. 767
  const int lane = threadIdx.x & 31;
  const int m = gw >> 7;
  const int row = gw & 127;
  const int n_rows = m < 4 ? 128 : a.c;
  const int k = m == 4 ? 128 : a.c;  // row length
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
  const float gg[4] = {g.x, g.y, g.z, g.w};
  const float bb[4] = {b.x, b.y, b.z, b.w};
  float s = 0.f, d = 0.f;
  uint16_t o[4];
  // Both operands of an MMA share one 16-bit format. Matrices 0..3 meet the fp16 x_hat and matrix 4 the
  // fp16 t tile, so they are fp16 (three more mantissa bits than bf16; |0.5 W gamma| is far from 65504).
  // Matrix 5 meets the module's raw bf16 input, so it is bf16.
  const bool fold = m >= 4;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float v = fold ? 0.5f * w[t] * gg[t] : 0.5f * w[t];
    if (m == 5) {
      const __nv_bfloat16 r = __float2bfloat16_rn(v);
      o[t] = __bfloat16_as_ushort(r);
      s += __bfloat162float(r);
    } else {
      const __half r = __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
      o[t] = __half_as_ushort(r);
      s += __half2float(r);
    }
    if (fold) d = fmaf(w[t], bb[t], d);
  }
  if (gw == 0 && active) {
    reinterpret_cast<float4*>(packed + kPackedLnOff)[lane] = g;
    reinterpret_cast<float4*>(packed + kPackedLnOff + 512)[lane] = b;
  }
  if (active) {
    uint2 ov;
    ov.x = static_cast<uint32_t>(o[0]) | (static_cast<uint32_t>(o[1]) << 16);
    ov.y = static_cast<uint32_t>(o[2]) | (static_cast<uint32_t>(o[3]) << 16);
    reinterpret_cast<uint2*>(packed + packed_matrix_offset(m, a.c))[row * (k / 4) + lane] = ov;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
    d += __shfl_xor_sync(0xFFFFFFFFu, d, off);
  }
  if (lane == 0) {
    const float bias = a.bias[m] != nullptr ? a.bias[m][row] : 0.f;
    d = 0.5f * (d + bias);  // d is the folded W beta term for matrices 4 and 5, zero for the others
    if (m < 4) {
      reinterpret_cast<float*>(packed + kPackedD1Off)[m * 128 + row] = d;
    } else {
      float* c3 = reinterpret_cast<float*>(packed + kPackedC3Off) + row * 4;
      if (m == 5) {
        c3[0] = s;
        c3[1] = d;
      } else {
        c3[2] = s;
        c3[3] = d;
      }
    }
  }
}

// Sum of the incoming-direction partial results of several GPUs for the rows one GPU owns:
// tri[e] = sum_s src[s][e] over `count` 16-byte groups of eight fp16 values, fp32 accumulation in source order,
// one saturating rounding. Sources may be peer memory: they are read with plain 16-byte loads.
constexpr int kMaxReduceSrc = 8;
struct ReduceSrc {
  const uint4* p[kMaxReduceSrc];
  int n;
};

__device__ __forceinline__ uint32_t pack_sat(float a, float b) { return pack_f16x2_sat(make_float2(a, b)); }

__global__ void __launch_bounds__(512) reduce_partials_kernel(const ReduceSrc src, uint4* __restrict__ tri, size_t count) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t e = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < count; e += stride) {
    float acc[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) acc[t] = 0.f;
    uint4 v[kMaxReduceSrc];
#pragma unroll
    for (int s = 0; s < kMaxReduceSrc; ++s)
      if (s < src.n) v[s] = src.p[s][e];  // all loads in flight before the first use
#pragma unroll
    for (int s = 0; s < kMaxReduceSrc; ++s) {
      if (s < src.n) {
        const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = f16x2_to_float2(w[t]);
          acc[2 * t] += f.x;
          acc[2 * t + 1] += f.y;
        }
      }
    }
    uint4 o;
    o.x = pack_sat(acc[0], acc[1]);
    o.y = pack_sat(acc[2], acc[3]);
    o.z = pack_sat(acc[4], acc[5]);
    o.w = pack_sat(acc[6], acc[7]);
    tri[e] = o;
  }
}

// Barrier between GPUs through flag arrays in peer memory (see b200_trimul_peer_barrier). Thread t talks to GPU t.
struct PeerFlags {
  int* p[8];
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerFlags f, int rank, int world, int epoch,
                                                          long long limit_cycles, int* status) {
  const int t = threadIdx.x;
  if (t >= world || t == rank) return;
  // the kernels before this one on the stream have completed, so their stores to peer memory have been performed
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f.p[t] + rank), "r"(epoch) : "memory");
  const int* mine = f.p[rank] + t;
  const long long t0 = clock64();
  while (true) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= epoch) break;
    if (clock64() - t0 > limit_cycles) {  // bounded: report and leave, the context stays usable
      atomicCAS(status, 0, kDevTimeoutPeerBarrier);
      break;
    }
    __nanosleep(200);
  }
}

// ---------------------------------------------------------------------------------------------
// Host helpers
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static std::once_flag once;
  static EncodeTiledFn fn = nullptr;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

// bf16 tensor map with 128-byte swizzle. dims[0] is the contiguous dimension; strides (bytes) are for
// dims[1..rank-1].
static int make_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                    const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) {
    tl_last_cuda_error = static_cast<int>(cudaErrorNotSupported);
    return B200_TRIMUL_E_CUDA;
  }
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5];
  cuuint32_t e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
    if (i > 0) s[i - 1] = strides[i - 1];
  }
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s,
                  b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    tl_last_cuda_error = 100000 + static_cast<int>(r);
    return B200_TRIMUL_E_CUDA;
  }
  return B200_TRIMUL_OK;
}

struct DeviceInfo {
  int sms;
  int cc_major;
  int device;
};

constexpr int kMaxDevices = 64;

// SM count and compute capability of the current device; queried once per device and process.
static int device_info(DeviceInfo* info) {
  static std::atomic<int> cached_sms[kMaxDevices];  // 0 = not queried yet
  static std::atomic<int> cached_cc[kMaxDevices];
  int dev = 0;
  TRIMUL_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return B200_TRIMUL_E_DEVICE;
  info->device = dev;
  int sms = cached_sms[dev].load(std::memory_order_acquire);
  if (sms == 0) {
    int cc = 0;
    TRIMUL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    TRIMUL_CUDA(cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev));
    cached_cc[dev].store(cc, std::memory_order_relaxed);
    cached_sms[dev].store(sms, std::memory_order_release);
  }
  info->sms = sms;
  info->cc_major = cached_cc[dev].load(std::memory_order_relaxed);
  if (info->cc_major != 10) return B200_TRIMUL_E_DEVICE;
  return B200_TRIMUL_OK;
}

// Opt a kernel in to its dynamic shared-memory size, once per kernel and device (the attribute belongs to the
// function in a device's context; setting it again is harmless, so a benign race between two threads is fine).
template <typename K>
static int set_smem(K kernel, int bytes, int device) {
  struct Slot {
    std::atomic<const void*> fn{nullptr};
    std::atomic<unsigned long long> devices{0};
  };
  static Slot slots[64];
  const void* key = reinterpret_cast<const void*>(kernel);
  const unsigned long long bit = 1ull << device;
  for (Slot& s : slots) {
    const void* cur = s.fn.load(std::memory_order_acquire);
    if (cur == nullptr) {
      const void* expected = nullptr;
      if (!s.fn.compare_exchange_strong(expected, key, std::memory_order_acq_rel) && expected != key) continue;
      cur = key;
    }
    if (cur != key) continue;
    if (s.devices.load(std::memory_order_acquire) & bit) return B200_TRIMUL_OK;
    TRIMUL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    s.devices.fetch_or(bit, std::memory_order_release);
    return B200_TRIMUL_OK;
  }
  TRIMUL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));  // table full
  return B200_TRIMUL_OK;
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

static int check_bn(int B, int N) {
  if (B < 1 || N < 8) return B200_TRIMUL_E_SHAPE;
  if (N % 8 != 0) return B200_TRIMUL_E_UNSUPPORTED;
  if (static_cast<long long>(B) * N > 0x7FFFFFFFll / 128) return B200_TRIMUL_E_SHAPE;
  return B200_TRIMUL_OK;
}

static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static size_t plane_tensor_bytes(int B, int rows, int N) {
  return round_up(static_cast<size_t>(B) * rows * kC * N * 2, 1024);
}

// Column tile width of the contraction: the candidate that wastes the fewest padded columns.
static int choose_bn(int N) {
  const int cands[3] = {256, 192, 128};
  int best = 256;
  long long best_pad = -1;
  for (int c : cands) {
    const long long padded = static_cast<long long>((N + c - 1) / c) * c;
    if (best_pad < 0 || padded < best_pad) {
      best_pad = padded;
      best = c;
    }
  }
  return best;
}

template <int BN, int MODE>
static int launch_contract(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mt, const ContractParams& p,
                           const DeviceInfo& info, cudaStream_t stream) {
  const int sms = info.sms;
  auto kernel = contract_kernel<BN, MODE>;
  constexpr int smem = ContractSmem<BN>::kTotal;
  int rc = set_smem(kernel, smem, info.device);
  if (rc != B200_TRIMUL_OK) return rc;
  const long long tiles = static_cast<long long>(p.planes) * p.m_tiles * p.n_tiles;
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  kernel<<<grid, kContractThreads, smem, stream>>>(ma, mb, mt, p);
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

template <int BN, int MODE>
static int launch_contract_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mt,
                                const TriOwners& own, const ContractParams& p, const DeviceInfo& info,
                                cudaStream_t stream) {
  const int sms = info.sms;
  auto kernel = contract_pair_kernel<BN, MODE>;
  constexpr int smem = PairSmem<BN>::kTotal;
  int rc = set_smem(kernel, smem, info.device);
  if (rc != B200_TRIMUL_OK) return rc;
  const long long tiles = static_cast<long long>(p.planes) * p.m_tiles * p.n_tiles;
  const long long pairs = tiles < sms / 2 ? tiles : sms / 2;
  kernel<<<static_cast<int>(2 * pairs), kContractThreads, smem, stream>>>(ma, mb, mt, own, p);  // clusters of two CTAs
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

}  // namespace trimul

#include "backward.cuh"  // after PackArgs
#include "transition_backward.cuh"

using namespace trimul;

extern "C" {

int b200_trimul_version(void) { return 100; }

const char* b200_trimul_strerror(int code) {
  switch (code) {
    case B200_TRIMUL_OK: return "ok";
    case B200_TRIMUL_E_NULL: return "a required pointer is null";
    case B200_TRIMUL_E_SHAPE: return "bad shape, row range or direction";
    case B200_TRIMUL_E_UNSUPPORTED: return "unsupported size: N a multiple of 8 and d_pair = d_hidden = 128 (or d_pair = 64 with 128 contracted channels in total) are required";
    case B200_TRIMUL_E_ALIGN: return "pointer not aligned (16 bytes; workspace and packed weights 1024)";
    case B200_TRIMUL_E_WORKSPACE: return "workspace too small";
    case B200_TRIMUL_E_CUDA: return "CUDA call failed (see b200_trimul_last_cuda_error)";
    case B200_TRIMUL_E_DEVICE: return "device is not sm_100";
    case B200_TRIMUL_E_TOO_LARGE:
      return "problem does not fit the built-in scratch of b200_trimul_forward_static (B * N * N <= 16384)";
    case kDevTimeoutProducer: return "device: copy producer gave up waiting";
    case kDevTimeoutMma: return "device: MMA issuer gave up waiting";
    case kDevTimeoutEpilogue: return "device: epilogue gave up waiting";
    case kDevTimeoutStats: return "device: statistics warps gave up waiting";
    case kDevTimeoutDrain: return "device: copies still in flight at exit";
    case kDevTimeoutPeerBarrier: return "device: barrier between GPUs gave up waiting for a peer";
    default: return "unknown status";
  }
}

int b200_trimul_last_cuda_error(void) { return tl_last_cuda_error; }

size_t b200_trimul_packed_bytes(void) { return kPackedBytes; }

int b200_trimul_workspace_layout(int B, int N, size_t out_offsets[5]) {
  if (out_offsets == nullptr) return B200_TRIMUL_E_NULL;
  int rc = check_bn(B, N);
  if (rc != B200_TRIMUL_OK) return rc;
  const size_t t = plane_tensor_bytes(B, N, N);
  out_offsets[0] = 0;
  out_offsets[1] = kStatusBytes;
  out_offsets[2] = kStatusBytes + kPackedBytes;
  out_offsets[3] = out_offsets[2] + t;
  out_offsets[4] = out_offsets[3] + t;
  return B200_TRIMUL_OK;
}

int b200_trimul_workspace_bytes(int B, int N, int d_pair, int d_hidden, int direction, size_t* out_bytes) {
  if (out_bytes == nullptr) return B200_TRIMUL_E_NULL;
  if (direction != B200_TRIMUL_OUTGOING && direction != B200_TRIMUL_INCOMING && direction != B200_TRIMUL_BIDIRECTIONAL)
    return B200_TRIMUL_E_SHAPE;
  // supported widths: d_pair = d_hidden = 128 (every direction); d_pair = 64 with 128 contracted channels in total,
  // i.e. d_hidden = 128 for one direction or d_hidden = 64 per direction for the bidirectional module
  const bool wide = d_pair == kC && d_hidden == kC;
  const bool narrow = d_pair == 64 && d_hidden == (direction == B200_TRIMUL_BIDIRECTIONAL ? 64 : kC);
  if (!wide && !narrow) return B200_TRIMUL_E_UNSUPPORTED;
  size_t off[5];
  int rc = b200_trimul_workspace_layout(B, N, off);
  if (rc != B200_TRIMUL_OK) return rc;
  *out_bytes = off[4] + plane_tensor_bytes(B, N, N);
  // bidirectional: a second packed block and a second tri tensor (left / right are reused by the two halves)
  if (direction == B200_TRIMUL_BIDIRECTIONAL && wide) *out_bytes += kPackedBytes + plane_tensor_bytes(B, N, N);
  return B200_TRIMUL_OK;
}

int b200_trimul_clear_status(int* status, void* cuda_stream) {
  if (status == nullptr) return B200_TRIMUL_E_NULL;
  TRIMUL_CUDA(cudaMemsetAsync(status, 0, 64, static_cast<cudaStream_t>(cuda_stream)));
  return B200_TRIMUL_OK;
}

int b200_trimul_read_status(const int* status, void* cuda_stream, int* host_status) {
  if (status == nullptr || host_status == nullptr) return B200_TRIMUL_E_NULL;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  TRIMUL_CUDA(cudaMemcpyAsync(host_status, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
  TRIMUL_CUDA(cudaStreamSynchronize(stream));
  return B200_TRIMUL_OK;
}

// Launch the pack kernel. w / bias in MATRIX order: left, left gate, right, right gate, out, gate.
static int pack_impl(const void* const w[6], const int ld[6], int weight_dtype, const float* ln_in_w, const float* ln_in_b,
                     const float* ln_out_w, const float* ln_out_b, const float* const bias[6], void* packed,
                     void* cuda_stream, int c = kC) {
  if (!ln_in_w || !ln_in_b || !ln_out_w || !ln_out_b || !packed) return B200_TRIMUL_E_NULL;
  if (weight_dtype != B200_TRIMUL_DTYPE_BF16 && weight_dtype != B200_TRIMUL_DTYPE_F32) return B200_TRIMUL_E_SHAPE;
  PackArgs a;
  for (int i = 0; i < 6; ++i) {
    if (!w[i]) return B200_TRIMUL_E_NULL;
    if (!aligned(w[i], 16)) return B200_TRIMUL_E_ALIGN;
    a.w[i] = w[i];
    a.ld[i] = ld[i];
    a.bias[i] = bias[i];
  }
  if (!aligned(ln_in_w, 16) || !aligned(ln_in_b, 16) || !aligned(ln_out_w, 16) || !aligned(ln_out_b, 16))
    return B200_TRIMUL_E_ALIGN;
  if (!aligned(packed, 1024)) return B200_TRIMUL_E_ALIGN;
  a.ln_in_w = ln_in_w;
  a.ln_in_b = ln_in_b;
  a.ln_out_w = ln_out_w;
  a.ln_out_b = ln_out_b;
  a.f32_weights = weight_dtype == B200_TRIMUL_DTYPE_F32;
  a.c = c;
  pack_kernel<<<192, 128, 0, static_cast<cudaStream_t>(cuda_stream)>>>(a, static_cast<uint8_t*>(packed));
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

int b200_trimul_pack_weights(const void* w_left, const void* w_left_gate, const void* w_right,
                             const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                             const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                             const float* ln_out_b, const void* const* bias_opt, void* packed, void* cuda_stream) {
  const void* w[6] = {w_left, w_left_gate, w_right, w_right_gate, w_out, w_gate};
  const int ld[6] = {kC, kC, kC, kC, kC, kC};
  const float* bias[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  if (bias_opt != nullptr) {
    // ABI order: left, left_gate, right, right_gate, gate, out  ->  matrix order: ..., out (4), gate (5)
    for (int i = 0; i < 4; ++i) bias[i] = static_cast<const float*>(bias_opt[i]);
    bias[5] = static_cast<const float*>(bias_opt[4]);
    bias[4] = static_cast<const float*>(bias_opt[5]);
  }
  return pack_impl(w, ld, weight_dtype, ln_in_w, ln_in_b, ln_out_w, ln_out_b, bias, packed, cuda_stream);
}

// Bidirectional module: the four left / right matrices are [256, 128] (rows 0-127 feed the outgoing contraction, rows
// 128-255 the incoming one), ln_out has 256 entries, w_out is [128, 256]. Two packed blocks of the ordinary layout:
// `packed_out` serves stage 1 of the outgoing half and stage 3 (its matrix 4 is W_out[:, 0:128] folded with
// gamma_out[0:128]; its constants carry the output bias), `packed_in` serves stage 1 of the incoming half and
// holds W_out[:, 128:256] as its matrix 4. Stage 3 adds the two blocks' s_out / d_out constants.
int b200_trimul_pack_weights_bidir(const void* w_left, const void* w_left_gate, const void* w_right,
                                   const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                                   const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                                   const float* ln_out_b, const void* const* bias_opt, void* packed_out,
                                   void* packed_in, void* cuda_stream) {
  if (!w_left || !w_left_gate || !w_right || !w_right_gate || !w_gate || !w_out || !ln_out_w || !ln_out_b)
    return B200_TRIMUL_E_NULL;
  if (weight_dtype != B200_TRIMUL_DTYPE_BF16 && weight_dtype != B200_TRIMUL_DTYPE_F32) return B200_TRIMUL_E_SHAPE;
  const size_t es = weight_dtype == B200_TRIMUL_DTYPE_F32 ? 4 : 2;
  auto rows128 = [&](const void* base) { return static_cast<const uint8_t*>(base) + static_cast<size_t>(kC) * kC * es; };
  const float* b[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  if (bias_opt != nullptr)
    for (int i = 0; i < 6; ++i) b[i] = static_cast<const float*>(bias_opt[i]);
  const int ld[6] = {kC, kC, kC, kC, 2 * kC, kC};
  {
    const void* w[6] = {w_left, w_left_gate, w_right, w_right_gate, w_out, w_gate};
    const float* bias[6] = {b[0], b[1], b[2], b[3], b[5], b[4]};
    int rc = pack_impl(w, ld, weight_dtype, ln_in_w, ln_in_b, ln_out_w, ln_out_b, bias, packed_out, cuda_stream);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  const void* w[6] = {rows128(w_left), rows128(w_left_gate), rows128(w_right), rows128(w_right_gate),
                      static_cast<const uint8_t*>(w_out) + kC * es, w_gate};
  const float* bias[6] = {b[0] ? b[0] + kC : nullptr, b[1] ? b[1] + kC : nullptr, b[2] ? b[2] + kC : nullptr,
                          b[3] ? b[3] + kC : nullptr, nullptr, nullptr};
  return pack_impl(w, ld, weight_dtype, ln_in_w, ln_in_b, ln_out_w + kC, ln_out_b + kC, bias, packed_in, cuda_stream);
}

// Where stage 1 writes (see OutputMaps): kLocal - left / right are [B, rows, 128, N]; kGatherRight (B = 1) - left is
// [rows, 128, N], every right destination a gathered copy [N, 128, N]; kChannels (B = 1) - destination d of either
// output is the [N, 128/n, N] buffer of the GPU that contracts channel group d.
enum PrologueMode { kLocal, kGatherRight, kChannels };

static int prologue_impl(const void* z, const void* packed, const uint8_t* token_mask, const uint8_t* pair_mask,
                         void* const* left_dst, int n_left, void* const* right_dst, int n_right, PrologueMode mode,
                         int B, int N, int row_begin, int rows, float eps_in, int has_bias, int* status,
                         void* cuda_stream, int d_pair = kC) {
  if (d_pair != kC && d_pair != 64) return B200_TRIMUL_E_UNSUPPORTED;
  if (!z || !packed || !left_dst || !right_dst || !status) return B200_TRIMUL_E_NULL;
  if (n_left < 1 || n_left > kMaxDst || n_right < 1 || n_right > kMaxDst) return B200_TRIMUL_E_SHAPE;
  if (mode != kLocal && B != 1) return B200_TRIMUL_E_SHAPE;
  if (mode == kChannels && (n_left != n_right || kC % n_left != 0 || (kC / n_left) % 8 != 0)) return B200_TRIMUL_E_SHAPE;
  int rc = check_bn(B, N);
  if (rc != B200_TRIMUL_OK) return rc;
  if (rows < 1 || row_begin < 0 || row_begin + rows > N) return B200_TRIMUL_E_SHAPE;
  if (!aligned(z, 16) || !aligned(packed, 1024)) return B200_TRIMUL_E_ALIGN;
  DeviceInfo info;
  rc = device_info(&info);
  if (rc != B200_TRIMUL_OK) return rc;

  CUtensorMap map_z, map_w;
  OutputMaps out;
  {
    const uint64_t dp = static_cast<uint64_t>(d_pair);
    const uint64_t dims[3] = {dp, static_cast<uint64_t>(N), static_cast<uint64_t>(B) * rows};
    const uint64_t strides[2] = {dp * 2ull, static_cast<uint64_t>(N) * dp * 2ull};
    const uint32_t box[3] = {64, 64, 1};  // each CTA of a pair loads 64 of a tile's 128 positions
    rc = make_map(&map_z, z, 3, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  {
    // outputs, row-plane: [rows][channels][N columns]
    const uint64_t n64 = static_cast<uint64_t>(N);
    const uint64_t ch = mode == kChannels ? static_cast<uint64_t>(kC / n_left) : static_cast<uint64_t>(kC);
    const uint64_t strides[2] = {n64 * 2ull, n64 * ch * 2ull};
    const uint32_t box[3] = {64, static_cast<uint32_t>(ch), 1};
    const uint64_t dims_local[3] = {n64, ch, static_cast<uint64_t>(B) * rows};
    const uint64_t dims_all[3] = {n64, ch, n64};
    for (int d = 0; d < n_left; ++d) {
      if (!left_dst[d]) return B200_TRIMUL_E_NULL;
      if (!aligned(left_dst[d], 16)) return B200_TRIMUL_E_ALIGN;
      rc = make_map(&out.left[d], left_dst[d], 3, mode == kChannels ? dims_all : dims_local, strides, box);
      if (rc != B200_TRIMUL_OK) return rc;
    }
    for (int d = 0; d < n_right; ++d) {
      if (!right_dst[d]) return B200_TRIMUL_E_NULL;
      if (!aligned(right_dst[d], 16)) return B200_TRIMUL_E_ALIGN;
      rc = make_map(&out.right[d], right_dst[d], 3, mode == kLocal ? dims_local : dims_all, strides, box);
      if (rc != B200_TRIMUL_OK) return rc;
    }
    out.n_left = n_left;
    out.n_right = n_right;
    out.step_left = out.step_right = mode == kChannels ? static_cast<int>(ch) * 128 : 0;
    out.shift_left = mode == kChannels ? row_begin : 0;
    out.shift_right = mode == kLocal ? 0 : row_begin;
    out.warp_store = 0;
    if (mode == kLocal && n_left == 1 && n_right == 1) {
      const uint32_t box_w[3] = {64, 32, 1};
      rc = make_map(&out.left_warp, left_dst[0], 3, dims_local, strides, box_w);
      if (rc != B200_TRIMUL_OK) return rc;
      rc = make_map(&out.right_warp, right_dst[0], 3, dims_local, strides, box_w);
      if (rc != B200_TRIMUL_OK) return rc;
      out.warp_store = 1;
    }
  }
  {
    // the four left / right matrices [128, d_pair], one after the other at the start of the packed block
    const uint64_t dims[2] = {static_cast<uint64_t>(d_pair), 4ull * 128};
    const uint64_t strides[1] = {static_cast<uint64_t>(d_pair) * 2ull};
    const uint32_t box[2] = {64, 128};
    rc = make_map(&map_w, packed, 2, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  PrologueParams p;
  p.batch = B;
  p.rows = rows;
  p.n = N;
  p.row_offset = row_begin;
  p.tiles_per_row = (N + 127) / 128;
  p.num_tiles = B * rows * p.tiles_per_row;
  p.token_mask = token_mask;
  p.pair_mask = pair_mask;
  p.d1 = reinterpret_cast<const float*>(static_cast<const uint8_t*>(packed) + kPackedD1Off);
  p.ln_w = reinterpret_cast<const float*>(static_cast<const uint8_t*>(packed) + kPackedLnOff);
  p.ln_b = p.ln_w + 128;
  p.eps = eps_in;
  p.status = status;
  const int pairs = p.num_tiles < info.sms / 2 ? p.num_tiles : info.sms / 2;
  const int grid = 2 * pairs;  // clusters of two CTAs: CTA 0 produces `left`, CTA 1 `right`
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
#define TRIMUL_LAUNCH_PROLOGUE(BIAS, DP)                                                              \
  do {                                                                                               \
    rc = set_smem(prologue_kernel<BIAS, DP>, kProSmemBytes, info.device);                            \
    if (rc != B200_TRIMUL_OK) return rc;                                                             \
    prologue_kernel<BIAS, DP><<<grid, kProThreads, kProSmemBytes, stream>>>(map_z, map_w, out, p);   \
  } while (0)
  if (d_pair == kC) {
    if (has_bias) TRIMUL_LAUNCH_PROLOGUE(true, 128);
    else TRIMUL_LAUNCH_PROLOGUE(false, 128);
  } else {
    if (has_bias) TRIMUL_LAUNCH_PROLOGUE(true, 64);
    else TRIMUL_LAUNCH_PROLOGUE(false, 64);
  }
#undef TRIMUL_LAUNCH_PROLOGUE
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

int b200_trimul_prologue(const void* z, const void* packed, const uint8_t* token_mask, const uint8_t* pair_mask,
                         void* left, void* right, int B, int N, int row_begin, int rows, float eps_in, int has_bias,
                         int* status, void* cuda_stream) {
  void* l[1] = {left};
  void* r[1] = {right};
  return prologue_impl(z, packed, token_mask, pair_mask, l, 1, r, 1, kLocal, B, N, row_begin, rows, eps_in, has_bias,
                       status, cuda_stream);
}

int b200_trimul_prologue_push(const void* z, const void* packed, const uint8_t* token_mask, const uint8_t* pair_mask,
                              void* left, void* right_all, void* const* right_all_peers, int n_peers, int N,
                              int row_begin, int rows, float eps_in, int has_bias, int* status, void* cuda_stream) {
  if (n_peers < 0 || n_peers > kMaxDst - 1 || (n_peers > 0 && !right_all_peers)) return B200_TRIMUL_E_SHAPE;
  void* l[1] = {left};
  void* r[kMaxDst] = {right_all};
  for (int d = 0; d < n_peers; ++d) r[1 + d] = right_all_peers[d];
  return prologue_impl(z, packed, token_mask, pair_mask, l, 1, r, 1 + n_peers, kGatherRight, 1, N, row_begin, rows,
                       eps_in, has_bias, status, cuda_stream);
}

int b200_trimul_prologue_channels(const void* z, const void* packed, const uint8_t* token_mask, void* const* left_groups,
                                  void* const* right_groups, int groups, int N, int row_begin, int rows, float eps_in,
                                  int has_bias, int* status, void* cuda_stream) {
  return prologue_impl(z, packed, token_mask, nullptr, left_groups, groups, right_groups, groups, kChannels, 1, N,
                       row_begin, rows, eps_in, has_bias, status, cuda_stream);
}

// Contraction for output rows row_begin .. row_begin+rows-1. `k_rows` only matters for the incoming direction: the
// number of pair rows k that left / right hold and the sum runs over (N for the full update, a rank's own rows for a
// partial sum). `channels` is the channel count of the operands (128, or a group of 128/P in the channel-sharded
// form). With n_owners > 0 (all rows, B = 1) the result does not go to `tri` but, row block by row block, to
// owner_dst[s] + slot * (N/n_owners) * channels * N * 2 bytes: slot `slot` of GPU s's [n_owners][N/n_owners][channels][N].
// `row_channels` (0 = `channels`): channels per pair row in memory when the call works on a sub-range of them (left,
// right and tri then point at the first channel of the range).
// internal third operand form of contract_impl (not a module direction): t[i][j] = sum_k a[i][k] b[k][j] per plane
constexpr int kDirMixed = 3;

static int contract_impl(const void* left, const void* right, void* tri, void* const* owner_dst, int n_owners, int slot,
                         int channels, int B, int N, int row_begin, int rows, int k_rows, int direction, int* status,
                         void* cuda_stream, int row_channels = 0) {
  if (!left || !right || !status) return B200_TRIMUL_E_NULL;
  if (n_owners == 0 && !tri) return B200_TRIMUL_E_NULL;
  if (n_owners < 0 || n_owners > kMaxOwners || (n_owners > 0 && !owner_dst)) return B200_TRIMUL_E_SHAPE;
  if (channels < 8 || channels > kC || channels % 8 != 0) return B200_TRIMUL_E_SHAPE;
  int rc = check_bn(B, N);
  if (rc != B200_TRIMUL_OK) return rc;
  if (rows < 1 || row_begin < 0 || row_begin + rows > N) return B200_TRIMUL_E_SHAPE;
  if (k_rows < 1 || k_rows > N) return B200_TRIMUL_E_SHAPE;
  if (direction != B200_TRIMUL_OUTGOING && direction != B200_TRIMUL_INCOMING && direction != kDirMixed)
    return B200_TRIMUL_E_SHAPE;
  if (direction == kDirMixed && (k_rows != N || n_owners != 0)) return B200_TRIMUL_E_SHAPE;
  if (!aligned(left, 16) || !aligned(right, 16) || (tri && !aligned(tri, 16))) return B200_TRIMUL_E_ALIGN;
  DeviceInfo info;
  rc = device_info(&info);
  if (rc != B200_TRIMUL_OK) return rc;
  // operand forms: a is MN-major (its k index is the tensor's row) for the incoming contraction only, b for the
  // incoming and the mixed one
  const bool a_mn = direction == B200_TRIMUL_INCOMING;
  const bool b_mn = direction != B200_TRIMUL_OUTGOING;
  // CTA pairs work on 256-row tiles: used when that pads the rows by at most a quarter.
  const int pair_rows = (rows + 255) / 256 * 256;
  const bool use_pair = rows >= 256 && (pair_rows - rows) * 4 <= rows;
  const int bn = use_pair ? ((N + 255) / 256 * 256 <= (N + 127) / 128 * 128 ? 256 : 128) : choose_bn(N);
  const uint64_t n64 = static_cast<uint64_t>(N);
  const uint64_t ch64 = static_cast<uint64_t>(channels);
  const uint64_t row_stride = static_cast<uint64_t>(row_channels > 0 ? row_channels : channels) * n64 * 2;  // bytes between pair rows
  const uint64_t h_stride = n64 * 2;
  const uint64_t left_rows = a_mn ? static_cast<uint64_t>(k_rows) : static_cast<uint64_t>(rows);
  const uint64_t right_rows = b_mn ? static_cast<uint64_t>(k_rows) : n64;

  CUtensorMap map_a, map_b, map_t;
  {
    const uint64_t dims[4] = {n64, left_rows, ch64, static_cast<uint64_t>(B)};
    const uint64_t strides[3] = {row_stride, h_stride, left_rows * row_stride};
    const uint32_t box_out[4] = {64, 128, 1, 1};
    const uint32_t box_in[4] = {64, 64, 1, 1};
    rc = make_map(&map_a, left, 4, dims, strides, a_mn ? box_in : box_out);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  {
    const uint64_t dims[4] = {n64, right_rows, ch64, static_cast<uint64_t>(B)};
    const uint64_t strides[3] = {row_stride, h_stride, right_rows * row_stride};
    const uint32_t box_out[4] = {64, static_cast<uint32_t>(use_pair ? bn / 2 : bn), 1, 1};  // a CTA of a pair loads half
    const uint32_t box_in[4] = {64, 64, 1, 1};
    rc = make_map(&map_b, right, 4, dims, strides, b_mn ? box_in : box_out);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  TriOwners own;
  own.n = n_owners;
  own.rows_per_owner = 0;
  own.box_rows = 128;
  if (n_owners == 0) {
    const uint64_t dims[4] = {n64, static_cast<uint64_t>(rows), ch64, static_cast<uint64_t>(B)};
    const uint64_t strides[3] = {row_stride, h_stride, static_cast<uint64_t>(rows) * row_stride};
    const uint32_t box[4] = {64, 128, 1, 1};
    rc = make_map(&map_t, tri, 4, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  } else {
    // only the CTA-pair kernel stores per owner; every 32-row slice must belong to one owner
    if (!use_pair || B != 1 || row_begin != 0 || rows != N || slot < 0 || slot >= n_owners) return B200_TRIMUL_E_SHAPE;
    if (N % n_owners != 0 || (N / n_owners) % 32 != 0) return B200_TRIMUL_E_SHAPE;
    const int rpo = N / n_owners;
    own.rows_per_owner = rpo;
    own.box_rows = rpo % 128 == 0 ? 128 : (rpo % 64 == 0 ? 64 : 32);
    const uint64_t dims[4] = {n64, static_cast<uint64_t>(rpo), ch64, 1};
    const uint64_t strides[3] = {row_stride, h_stride, static_cast<uint64_t>(rpo) * row_stride};
    const uint32_t box[4] = {64, static_cast<uint32_t>(own.box_rows), 1, 1};
    for (int s2 = 0; s2 < n_owners; ++s2) {
      if (!owner_dst[s2]) return B200_TRIMUL_E_NULL;
      if (!aligned(owner_dst[s2], 16)) return B200_TRIMUL_E_ALIGN;
      uint8_t* base = static_cast<uint8_t*>(owner_dst[s2]) + static_cast<size_t>(slot) * rpo * row_stride;
      rc = make_map(&own.m[s2], base, 4, dims, strides, box);
      if (rc != B200_TRIMUL_OK) return rc;
    }
    map_t = own.m[0];  // unused by the kernel in this form, but a valid descriptor
  }
  ContractParams p;
  p.H = channels;
  p.planes = B * channels;
  p.m_tiles = use_pair ? pair_rows / 256 : (rows + kBM - 1) / kBM;
  p.m_rows = rows;
  p.n_tiles = (N + bn - 1) / bn;
  p.num_kb = ((b_mn ? k_rows : N) + kBK - 1) / kBK;  // rows past k_rows read as zero (TMA out-of-bounds fill)
  p.a_col_off = a_mn ? row_begin : 0;
  p.n_cols = N;
  p.status = status;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
#define TRIMUL_CONTRACT_MODE(MODE)                                                                       \
  do {                                                                                                   \
    if (use_pair) {                                                                                      \
      if (bn == 256) return launch_contract_pair<256, MODE>(map_a, map_b, map_t, own, p, info, stream); \
      return launch_contract_pair<128, MODE>(map_a, map_b, map_t, own, p, info, stream);                \
    }                                                                                                    \
    if (bn == 256) return launch_contract<256, MODE>(map_a, map_b, map_t, p, info, stream);             \
    if (bn == 192) return launch_contract<192, MODE>(map_a, map_b, map_t, p, info, stream);             \
    return launch_contract<128, MODE>(map_a, map_b, map_t, p, info, stream);                            \
  } while (0)
  if (direction == B200_TRIMUL_OUTGOING) TRIMUL_CONTRACT_MODE(kContractOutgoing);
  if (direction == B200_TRIMUL_INCOMING) TRIMUL_CONTRACT_MODE(kContractIncoming);
  TRIMUL_CONTRACT_MODE(kContractMixed);
#undef TRIMUL_CONTRACT_MODE
}

int b200_trimul_contract(const void* left, const void* right, void* tri, int B, int N, int row_begin, int rows,
                         int direction, int* status, void* cuda_stream) {
  return contract_impl(left, right, tri, nullptr, 0, 0, kC, B, N, row_begin, rows, N, direction, status, cuda_stream);
}

int b200_trimul_contract_backward(const void* dtri, const void* left, const void* right, void* dleft, void* dright, int B,
                                  int N, int direction, int* status, void* cuda_stream) {
  if (!dtri || !left || !right || !dleft || !dright) return B200_TRIMUL_E_NULL;
  int rc;
  if (direction == B200_TRIMUL_OUTGOING) {
    // t_ij = sum_k l_ik r_jk:  dl_ik = sum_j dt_ij r_jk (mixed),  dr_jk = sum_i dt_ij l_ik (the incoming form)
    rc = contract_impl(dtri, right, dleft, nullptr, 0, 0, kC, B, N, 0, N, N, kDirMixed, status, cuda_stream);
    if (rc != B200_TRIMUL_OK) return rc;
    return contract_impl(dtri, left, dright, nullptr, 0, 0, kC, B, N, 0, N, N, B200_TRIMUL_INCOMING, status, cuda_stream);
  }
  if (direction == B200_TRIMUL_INCOMING) {
    // t_ij = sum_k l_ki r_kj:  dl_ki = sum_j r_kj dt_ij (the outgoing form),  dr_kj = sum_i l_ki dt_ij (mixed)
    rc = contract_impl(right, dtri, dleft, nullptr, 0, 0, kC, B, N, 0, N, N, B200_TRIMUL_OUTGOING, status, cuda_stream);
    if (rc != B200_TRIMUL_OK) return rc;
    return contract_impl(left, dtri, dright, nullptr, 0, 0, kC, B, N, 0, N, N, kDirMixed, status, cuda_stream);
  }
  return B200_TRIMUL_E_SHAPE;
}

int b200_trimul_contract_partial(const void* left, const void* right, void* tri_partial, int B, int N, int k_rows,
                                 int* status, void* cuda_stream) {
  return contract_impl(left, right, tri_partial, nullptr, 0, 0, kC, B, N, 0, N, k_rows, B200_TRIMUL_INCOMING, status,
                       cuda_stream);
}

int b200_trimul_contract_channels(const void* left_group, const void* right_group, void* const* tri_owners, int groups,
                                  int group, int N, int direction, int* status, void* cuda_stream) {
  if (groups < 1 || groups > kMaxOwners || kC % groups != 0) return B200_TRIMUL_E_SHAPE;
  return contract_impl(left_group, right_group, nullptr, tri_owners, groups, group, kC / groups, 1, N, 0, N, N, direction,
                       status, cuda_stream);
}

int b200_trimul_peer_barrier(int* const* flags, int rank, int world, int epoch, int timeout_ms, int* status,
                             void* cuda_stream) {
  if (!flags || !status) return B200_TRIMUL_E_NULL;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || timeout_ms < 1) return B200_TRIMUL_E_SHAPE;
  DeviceInfo info;
  int rc = device_info(&info);
  if (rc != B200_TRIMUL_OK) return rc;
  PeerFlags f;
  for (int r = 0; r < 8; ++r) {
    f.p[r] = r < world ? flags[r] : nullptr;
    if (r < world && !f.p[r]) return B200_TRIMUL_E_NULL;
  }
  // SM clock cycles at the nominal maximum clock of a B200 (1965 MHz); querying the clock attribute costs about a
  // millisecond per call, and the limit only has to be of the right order
  const long long limit = static_cast<long long>(timeout_ms) * 1965000ll;
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(f, rank, world, epoch, limit, status);
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

int b200_trimul_reduce_partials(void* tri, const void* const* partials, int n_src, int N, int row_begin, int rows,
                                void* cuda_stream) {
  if (!tri || !partials) return B200_TRIMUL_E_NULL;
  if (n_src < 1 || n_src > kMaxReduceSrc) return B200_TRIMUL_E_SHAPE;
  int rc = check_bn(1, N);
  if (rc != B200_TRIMUL_OK) return rc;
  if (rows < 1 || row_begin < 0 || row_begin + rows > N) return B200_TRIMUL_E_SHAPE;
  if (!aligned(tri, 16)) return B200_TRIMUL_E_ALIGN;
  DeviceInfo info;
  rc = device_info(&info);
  if (rc != B200_TRIMUL_OK) return rc;
  const size_t row_bytes = static_cast<size_t>(kC) * N * 2;  // a multiple of 16: N is a multiple of 8
  ReduceSrc src;
  src.n = n_src;
  for (int s = 0; s < kMaxReduceSrc; ++s) {
    if (s < n_src) {
      if (!partials[s]) return B200_TRIMUL_E_NULL;
      if (!aligned(partials[s], 16)) return B200_TRIMUL_E_ALIGN;
      src.p[s] = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(partials[s]) + row_bytes * row_begin);
    } else {
      src.p[s] = nullptr;
    }
  }
  const size_t count = row_bytes * rows / 16;
  const int grid = info.sms * 4;
  reduce_partials_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(cuda_stream)>>>(src, static_cast<uint4*>(tri), count);
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

// `groups` = 1: tri is [B*rows][128][N]. groups = P (B = 1): tri is [P][rows][128/P][N], channel group g of every row
// in slab g (what the channel-sharded contraction of GPU g stored there).
static int epilogue_impl(const void* tri, const void* z, const void* packed, void* y, int B, int N, int rows, int groups,
                         float eps_in, float eps_out, int residual, int* status, void* cuda_stream, int d_pair = kC) {
  if (!tri || !z || !packed || !y || !status) return B200_TRIMUL_E_NULL;
  if (d_pair != kC && d_pair != 64) return B200_TRIMUL_E_UNSUPPORTED;
  if (groups < 1 || groups > 8 || kC % groups != 0 || (groups > 1 && B != 1)) return B200_TRIMUL_E_SHAPE;
  int rc = check_bn(B, N);
  if (rc != B200_TRIMUL_OK) return rc;
  if (rows < 1 || rows > N) return B200_TRIMUL_E_SHAPE;
  if (!aligned(tri, 16) || !aligned(z, 16) || !aligned(y, 16) || !aligned(packed, 1024)) return B200_TRIMUL_E_ALIGN;
  DeviceInfo info;
  rc = device_info(&info);
  if (rc != B200_TRIMUL_OK) return rc;
  const uint64_t n64 = static_cast<uint64_t>(N);
  const uint64_t nrows = static_cast<uint64_t>(B) * rows;

  CUtensorMap map_t, map_z, map_y, map_wo, map_wg;
  {
    const uint64_t cg = static_cast<uint64_t>(kC / groups);
    const uint64_t dims[4] = {n64, cg, static_cast<uint64_t>(groups), nrows};
    const uint64_t strides[3] = {n64 * 2, nrows * cg * n64 * 2, cg * n64 * 2};
    const uint32_t box[4] = {64, static_cast<uint32_t>(cg), static_cast<uint32_t>(groups), 1};
    rc = make_map(&map_t, tri, 4, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  const uint64_t dp = static_cast<uint64_t>(d_pair);
  {
    const uint64_t dims[3] = {dp, n64, nrows};
    const uint64_t strides[2] = {dp * 2ull, n64 * dp * 2ull};
    const uint32_t box[3] = {64, 128, 1};
    rc = make_map(&map_z, z, 3, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = make_map(&map_y, y, 3, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  {
    // Wo' [d_pair, 128] and Wg' [d_pair, d_pair] of the packed block, each loaded in 64-wide k halves
    const uint8_t* pk = static_cast<const uint8_t*>(packed);
    const uint64_t dims_o[2] = {128ull, dp};
    const uint64_t strides_o[1] = {128 * 2ull};
    const uint64_t dims_g[2] = {dp, dp};
    const uint64_t strides_g[1] = {dp * 2ull};
    const uint32_t box[2] = {64, static_cast<uint32_t>(d_pair)};
    rc = make_map(&map_wo, pk + packed_matrix_offset(4, d_pair), 2, dims_o, strides_o, box);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = make_map(&map_wg, pk + packed_matrix_offset(5, d_pair), 2, dims_g, strides_g, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  EpilogueParams p;
  p.tiles_per_row = (N + 127) / 128;
  p.num_tiles = static_cast<int>(nrows) * p.tiles_per_row;
  p.c3 = reinterpret_cast<const float4*>(static_cast<const uint8_t*>(packed) + kPackedC3Off);
  p.eps_in = eps_in;
  p.eps_out = eps_out * (kTriScale * kTriScale);  // tri arrives scaled by kTriScale
  p.residual = residual;
  p.status = status;
  const int grid = p.num_tiles < info.sms ? p.num_tiles : info.sms;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (d_pair == kC) {
    rc = set_smem(epilogue_kernel<128>, kEpiSmemBytes, info.device);
    if (rc != B200_TRIMUL_OK) return rc;
    epilogue_kernel<128><<<grid, kEpilogueThreads, kEpiSmemBytes, stream>>>(map_t, map_z, map_y, map_wo, map_wg, p);
  } else {
    rc = set_smem(epilogue_kernel<64>, kEpiSmemBytes, info.device);
    if (rc != B200_TRIMUL_OK) return rc;
    epilogue_kernel<64><<<grid, kEpilogueThreads, kEpiSmemBytes, stream>>>(map_t, map_z, map_y, map_wo, map_wg, p);
  }
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

int b200_trimul_epilogue(const void* tri, const void* z, const void* packed, void* y, int B, int N, int rows,
                         float eps_in, float eps_out, int residual, int* status, void* cuda_stream) {
  return epilogue_impl(tri, z, packed, y, B, N, rows, 1, eps_in, eps_out, residual, status, cuda_stream);
}

int b200_trimul_epilogue_groups(const void* tri_groups, const void* z, const void* packed, void* y, int N, int rows,
                                int groups, float eps_in, float eps_out, int residual, int* status, void* cuda_stream) {
  return epilogue_impl(tri_groups, z, packed, y, 1, N, rows, groups, eps_in, eps_out, residual, status, cuda_stream);
}

}  // extern "C"

template <int KCH, bool SCALED>
static int launch_epilogue_wide(const CUtensorMap& mt0, const CUtensorMap& mt1, const CUtensorMap& mz, const CUtensorMap& my,
                                const CUtensorMap& mw0, const CUtensorMap& mw1, const EpilogueWideParams& p,
                                const DeviceInfo& info, cudaStream_t stream) {
  auto kernel = epilogue_wide_kernel<KCH, SCALED>;
  int rc = set_smem(kernel, kWideSmemBytes, info.device);
  if (rc != B200_TRIMUL_OK) return rc;
  const int grid = p.num_tiles < info.sms ? p.num_tiles : info.sms;
  kernel<<<grid, kEpilogueThreads, kWideSmemBytes, stream>>>(mt0, mt1, mz, my, mw0, mw1, p);
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

extern "C" {

int b200_trimul_epilogue_wide(const void* tri, const void* tri_in, const void* z, const void* packed,
                              const void* packed_in, const void* drop_scale, void* y, int B, int N, int rows,
                              float eps_in, float eps_out, int residual, int* status, void* cuda_stream) {
  if (!tri || !z || !packed || !y || !status) return B200_TRIMUL_E_NULL;
  const bool bidir = tri_in != nullptr;
  if (bidir && !packed_in) return B200_TRIMUL_E_NULL;
  int rc = check_bn(B, N);
  if (rc != B200_TRIMUL_OK) return rc;
  if (rows < 1 || rows > N) return B200_TRIMUL_E_SHAPE;
  if (!aligned(tri, 16) || !aligned(z, 16) || !aligned(y, 16) || !aligned(packed, 1024)) return B200_TRIMUL_E_ALIGN;
  if (bidir && (!aligned(tri_in, 16) || !aligned(packed_in, 1024))) return B200_TRIMUL_E_ALIGN;
  if (drop_scale && !aligned(drop_scale, 16)) return B200_TRIMUL_E_ALIGN;
  DeviceInfo info;
  rc = device_info(&info);
  if (rc != B200_TRIMUL_OK) return rc;
  const uint64_t n64 = static_cast<uint64_t>(N);
  const uint64_t nrows = static_cast<uint64_t>(B) * rows;
  CUtensorMap map_t0, map_t1, map_z, map_y, map_w0, map_w1;
  {
    const uint64_t dims[3] = {n64, static_cast<uint64_t>(kC), nrows};
    const uint64_t strides[2] = {n64 * 2, static_cast<uint64_t>(kC) * n64 * 2};
    const uint32_t box[3] = {64, 64, 1};  // one chunk half: 64 positions of 64 channels
    rc = make_map(&map_t0, tri, 3, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = make_map(&map_t1, bidir ? tri_in : tri, 3, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(kC), n64, nrows};
    const uint64_t strides[2] = {kC * 2ull, n64 * kC * 2ull};
    const uint32_t box[3] = {64, 128, 1};
    rc = make_map(&map_z, z, 3, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = make_map(&map_y, y, 3, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(kC), 6ull * 128};
    const uint64_t strides[1] = {kC * 2ull};
    const uint32_t box[2] = {64, 128};
    rc = make_map(&map_w0, packed, 2, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = make_map(&map_w1, bidir ? packed_in : packed, 2, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  EpilogueWideParams p;
  p.tiles_per_row = (N + 127) / 128;
  p.num_tiles = static_cast<int>(nrows) * p.tiles_per_row;
  p.rows_per_sample = rows;
  p.n = N;
  p.c3_a = reinterpret_cast<const float4*>(static_cast<const uint8_t*>(packed) + kPackedC3Off);
  p.c3_b = reinterpret_cast<const float4*>(static_cast<const uint8_t*>(bidir ? packed_in : packed) + kPackedC3Off);
  p.drop_scale = static_cast<const __nv_bfloat16*>(drop_scale);
  p.eps_in = eps_in;
  p.eps_out = eps_out * (kTriScale * kTriScale);  // tri arrives scaled by kTriScale
  p.residual = residual;
  p.status = status;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (bidir) {
    if (drop_scale) return launch_epilogue_wide<4, true>(map_t0, map_t1, map_z, map_y, map_w0, map_w1, p, info, stream);
    return launch_epilogue_wide<4, false>(map_t0, map_t1, map_z, map_y, map_w0, map_w1, p, info, stream);
  }
  if (drop_scale) return launch_epilogue_wide<2, true>(map_t0, map_t1, map_z, map_y, map_w0, map_w1, p, info, stream);
  return launch_epilogue_wide<2, false>(map_t0, map_t1, map_z, map_y, map_w0, map_w1, p, info, stream);
}

int b200_trimul_forward_ex(const void* z, const void* w_left, const void* w_left_gate, const void* w_right,
                           const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                           const float* ln_in_w, const float* ln_in_b, const float* ln_out_w, const float* ln_out_b,
                           const void* const* bias_opt, const uint8_t* token_mask, const uint8_t* pair_mask,
                           const void* drop_scale, void* y, void* workspace, size_t workspace_bytes, int B, int N,
                           int d_pair, int d_hidden, int direction, float eps_in, float eps_out, int residual,
                           void* cuda_stream) {
  if (!z || !y || !workspace) return B200_TRIMUL_E_NULL;
  size_t need = 0;
  int rc = b200_trimul_workspace_bytes(B, N, d_pair, d_hidden, direction, &need);
  if (rc != B200_TRIMUL_OK) return rc;
  if (workspace_bytes < need) return B200_TRIMUL_E_WORKSPACE;
  if (!aligned(workspace, 1024)) return B200_TRIMUL_E_ALIGN;
  size_t off[5];
  rc = b200_trimul_workspace_layout(B, N, off);
  if (rc != B200_TRIMUL_OK) return rc;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* status = reinterpret_cast<int*>(ws + off[0]);
  void* packed = ws + off[1];
  void* left = ws + off[2];
  void* right = ws + off[3];
  void* tri = ws + off[4];
  rc = b200_trimul_clear_status(status, cuda_stream);
  if (rc != B200_TRIMUL_OK) return rc;
  int has_bias = 0;
  if (bias_opt != nullptr)
    for (int i = 0; i < 4; ++i) has_bias |= bias_opt[i] != nullptr;
  if (d_pair == 64) {
    // Narrow pair stacks: 64 input channels, 128 contracted channels in one [rows, 128, N] tensor. The parameter
    // shapes are to_left / to_left_gate / to_right / to_right_gate [128, 64], ln_out [128], to_out [64, 128],
    // to_gate [64, 64] for both forms; the bidirectional module contracts channels 0-63 outgoing and 64-127 incoming.
    if (drop_scale != nullptr) return B200_TRIMUL_E_UNSUPPORTED;
    if (!w_left || !w_left_gate || !w_right || !w_right_gate || !w_gate || !w_out) return B200_TRIMUL_E_NULL;
    const void* w[6] = {w_left, w_left_gate, w_right, w_right_gate, w_out, w_gate};
    const int ld[6] = {64, 64, 64, 64, kC, 64};
    const float* bias[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    if (bias_opt != nullptr) {
      for (int i = 0; i < 4; ++i) bias[i] = static_cast<const float*>(bias_opt[i]);
      bias[5] = static_cast<const float*>(bias_opt[4]);
      bias[4] = static_cast<const float*>(bias_opt[5]);
    }
    rc = pack_impl(w, ld, weight_dtype, ln_in_w, ln_in_b, ln_out_w, ln_out_b, bias, packed, cuda_stream, 64);
    if (rc != B200_TRIMUL_OK) return rc;
    void* l[1] = {left};
    void* r[1] = {right};
    rc = prologue_impl(z, packed, token_mask, pair_mask, l, 1, r, 1, kLocal, B, N, 0, N, eps_in, has_bias, status,
                       cuda_stream, 64);
    if (rc != B200_TRIMUL_OK) return rc;
    if (direction == B200_TRIMUL_BIDIRECTIONAL) {
      const size_t half = static_cast<size_t>(64) * N * 2;  // bytes from channel 0 to channel 64 of a pair row
      rc = contract_impl(left, right, tri, nullptr, 0, 0, 64, B, N, 0, N, N, B200_TRIMUL_OUTGOING, status, cuda_stream, kC);
      if (rc != B200_TRIMUL_OK) return rc;
      rc = contract_impl(static_cast<uint8_t*>(left) + half, static_cast<uint8_t*>(right) + half,
                         static_cast<uint8_t*>(tri) + half, nullptr, 0, 0, 64, B, N, 0, N, N, B200_TRIMUL_INCOMING, status,
                         cuda_stream, kC);
    } else {
      rc = b200_trimul_contract(left, right, tri, B, N, 0, N, direction, status, cuda_stream);
    }
    if (rc != B200_TRIMUL_OK) return rc;
    return epilogue_impl(tri, z, packed, y, B, N, N, 1, eps_in, eps_out, residual, status, cuda_stream, 64);
  }
  if (direction == B200_TRIMUL_BIDIRECTIONAL) {
    // workspace tail: second tri tensor, then the second packed block
    const size_t plane = plane_tensor_bytes(B, N, N);
    void* tri_in = ws + off[4] + plane;
    void* packed_in = ws + off[4] + 2 * plane;
    rc = b200_trimul_pack_weights_bidir(w_left, w_left_gate, w_right, w_right_gate, w_gate, w_out, weight_dtype, ln_in_w,
                                        ln_in_b, ln_out_w, ln_out_b, bias_opt, packed, packed_in, cuda_stream);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = b200_trimul_prologue(z, packed, token_mask, pair_mask, left, right, B, N, 0, N, eps_in, has_bias, status,
                              cuda_stream);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = b200_trimul_contract(left, right, tri, B, N, 0, N, B200_TRIMUL_OUTGOING, status, cuda_stream);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = b200_trimul_prologue(z, packed_in, token_mask, pair_mask, left, right, B, N, 0, N, eps_in, has_bias, status,
                              cuda_stream);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = b200_trimul_contract(left, right, tri_in, B, N, 0, N, B200_TRIMUL_INCOMING, status, cuda_stream);
    if (rc != B200_TRIMUL_OK) return rc;
    return b200_trimul_epilogue_wide(tri, tri_in, z, packed, packed_in, drop_scale, y, B, N, N, eps_in, eps_out, residual,
                                     status, cuda_stream);
  }
  rc = b200_trimul_pack_weights(w_left, w_left_gate, w_right, w_right_gate, w_gate, w_out, weight_dtype, ln_in_w,
                                ln_in_b, ln_out_w, ln_out_b, bias_opt, packed, cuda_stream);
  if (rc != B200_TRIMUL_OK) return rc;
  rc = b200_trimul_prologue(z, packed, token_mask, pair_mask, left, right, B, N, 0, N, eps_in, has_bias, status,
                            cuda_stream);
  if (rc != B200_TRIMUL_OK) return rc;
  rc = b200_trimul_contract(left, right, tri, B, N, 0, N, direction, status, cuda_stream);
  if (rc != B200_TRIMUL_OK) return rc;
  if (drop_scale != nullptr)
    return b200_trimul_epilogue_wide(tri, nullptr, z, packed, nullptr, drop_scale, y, B, N, N, eps_in, eps_out, residual,
                                     status, cuda_stream);
  return b200_trimul_epilogue(tri, z, packed, y, B, N, N, eps_in, eps_out, residual, status, cuda_stream);
}

int b200_trimul_forward(const void* z, const void* w_left, const void* w_left_gate, const void* w_right,
                        const void* w_right_gate, const void* w_gate, const void* w_out, int weight_dtype,
                        const float* ln_in_w, const float* ln_in_b, const float* ln_out_w, const float* ln_out_b,
                        const void* const* bias_opt, const uint8_t* token_mask, const uint8_t* pair_mask, void* y,
                        void* workspace, size_t workspace_bytes, int B, int N, int d_pair, int d_hidden,
                        int direction, float eps_in, float eps_out, int residual, void* cuda_stream) {
  return b200_trimul_forward_ex(z, w_left, w_left_gate, w_right, w_right_gate, w_gate, w_out, weight_dtype, ln_in_w,
                                ln_in_b, ln_out_w, ln_out_b, bias_opt, token_mask, pair_mask, nullptr, y, workspace,
                                workspace_bytes, B, N, d_pair, d_hidden, direction, eps_in, eps_out, residual,
                                cuda_stream);
}

// --------------------------------------------------------------------------------------------- pair Transition
size_t b200_transition_packed_bytes(void) { return kTrPackedBytes; }

int b200_transition_pack_weights(const void* w_expand_a, const void* w_expand_b, const void* w_squeeze, int weight_dtype,
                                 const float* ln_w, const float* ln_b, void* packed, void* cuda_stream) {
  if (!w_expand_a || !w_expand_b || !w_squeeze || !ln_w || !ln_b || !packed) return B200_TRIMUL_E_NULL;
  if (weight_dtype != B200_TRIMUL_DTYPE_BF16 && weight_dtype != B200_TRIMUL_DTYPE_F32) return B200_TRIMUL_E_SHAPE;
  if (!aligned(packed, 1024)) return B200_TRIMUL_E_ALIGN;
  TransitionPackArgs a;
  a.w_a = w_expand_a;
  a.w_b = w_expand_b;
  a.w_s = w_squeeze;
  a.ln_w = ln_w;
  a.ln_b = ln_b;
  a.f32_weights = weight_dtype == B200_TRIMUL_DTYPE_F32;
  transition_pack_kernel<<<(1024 * 128 + 128 * 512) / 256, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      a, static_cast<uint8_t*>(packed));
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

int b200_transition_forward(const void* x, const void* packed, void* y, long long positions, int d, int n, float eps,
                            int residual, int* status, void* cuda_stream) {
  if (!x || !packed || !y || !status) return B200_TRIMUL_E_NULL;
  if (d != kC || n != 4) return B200_TRIMUL_E_UNSUPPORTED;
  if (positions < 1 || positions > 0x7FFFFFFFll - 512) return B200_TRIMUL_E_SHAPE;
  if (!aligned(x, 16) || !aligned(y, 16) || !aligned(packed, 1024)) return B200_TRIMUL_E_ALIGN;
  DeviceInfo info;
  int rc = device_info(&info);
  if (rc != B200_TRIMUL_OK) return rc;
  CUtensorMap map_x, map_y, map_wab, map_ws;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(kC), static_cast<uint64_t>(positions)};
    const uint64_t strides[1] = {kC * 2ull};
    const uint32_t box[2] = {64, 128};
    rc = make_map(&map_x, x, 2, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
    rc = make_map(&map_y, y, 2, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(kC), 1024ull};
    const uint64_t strides[1] = {kC * 2ull};
    const uint32_t box[2] = {64, 64};
    rc = make_map(&map_wab, packed, 2, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  {
    const uint64_t dims[2] = {512ull, static_cast<uint64_t>(kC)};
    const uint64_t strides[1] = {512 * 2ull};
    const uint32_t box[2] = {64, 64};
    rc = make_map(&map_ws, static_cast<const uint8_t*>(packed) + kTrPackedAbBytes, 2, dims, strides, box);
    if (rc != B200_TRIMUL_OK) return rc;
  }
  TransitionParams p;
  p.positions = positions;
  p.num_tiles = static_cast<int>((positions + 255) / 256);
  p.ln_w = reinterpret_cast<const float*>(static_cast<const uint8_t*>(packed) + kTrPackedLnOff);
  p.ln_b = p.ln_w + 128;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.eps = eps;
  p.residual = residual;
  p.status = status;
  rc = set_smem(transition_kernel, kTrSmemBytes, info.device);
  if (rc != B200_TRIMUL_OK) return rc;
  const int pairs = p.num_tiles < info.sms / 2 ? p.num_tiles : info.sms / 2;
  transition_kernel<<<2 * pairs, kTrThreads, kTrSmemBytes, static_cast<cudaStream_t>(cuda_stream)>>>(map_x, map_y, map_wab,
                                                                                                   map_ws, p);
  TRIMUL_CUDA(cudaGetLastError());
  return B200_TRIMUL_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Forward for callers that must not allocate device memory.
//
// Some hosts of this library cannot hand it a workspace: an inference server whose memory pool already
// owns all of HBM (a late cudaMalloc fails, and even a successful one synchronises the whole device in
// the middle of a latency-critical loop), or a plug-in running under a host program that forbids
// allocation after start-up. For them the scratch of a small forward lives in the library image itself:
// a file-scope device array, reserved on every GPU that loads the library until the process exits.
//
// Host code may not treat the array's name as a device address (it is only a host-side handle of the
// symbol), so the address is looked up with cudaGetSymbolAddress once per device, with that device
// current, the first time the entry point runs there; that first call should therefore be made before
// any stream capture begins. All calls on a device share the one array: it keeps whatever the last call
// left in it, the status words are cleared at the start of every call, everything else is overwritten
// before it is read, and two calls that overlap on the GPU (different streams, or different host
// threads) race on it.
namespace trimul {

constexpr long long kStaticMaxCells = 16384;  // B * N * N, e.g. one 128-token sample or four 64-token ones
constexpr size_t kStaticPlaneBytes = static_cast<size_t>(kStaticMaxCells) * kC * 2;  // 4 MiB per intermediate
constexpr size_t kStaticWorkspaceBytes = kStatusBytes + kPackedBytes + 3 * kStaticPlaneBytes;
constexpr size_t kStaticScratchBytes = kStaticWorkspaceBytes + 1024;  // slack to reach 1024-byte alignment

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];  // 12.2 MiB per GPU

static std::mutex g_static_mutex;
static void* g_static_ptr[kMaxDevices] = {};

// Device address of the scratch on the current device, rounded up to 1024 bytes (set up on first use).
static int static_scratch(void** out) {
  int dev = 0;
  TRIMUL_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return B200_TRIMUL_E_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* raw = nullptr;
    TRIMUL_CUDA(cudaGetSymbolAddress(&raw, g_static_scratch));
    if (raw == nullptr) return B200_TRIMUL_E_CUDA;
    const uintptr_t a = (reinterpret_cast<uintptr_t>(raw) + 1023u) & ~static_cast<uintptr_t>(1023u);
    g_static_ptr[dev] = reinterpret_cast<void*>(a);
  }
  *out = g_static_ptr[dev];
  return B200_TRIMUL_OK;
}

}  // namespace trimul

extern "C" int b200_trimul_forward_static(const void* z, const void* w_left, const void* w_left_gate,
                                          const void* w_right, const void* w_right_gate, const void* w_gate,
                                          const void* w_out, int weight_dtype, const float* ln_in_w,
                                          const float* ln_in_b, const float* ln_out_w, const float* ln_out_b,
                                          const void* const* bias_opt, const uint8_t* token_mask,
                                          const uint8_t* pair_mask, void* y, int B, int N, int d_pair, int d_hidden,
                                          int direction, float eps_in, float eps_out, int residual,
                                          int** device_status_out, void* cuda_stream) {
  if (!z || !y) return B200_TRIMUL_E_NULL;
  size_t need = 0;
  int rc = b200_trimul_workspace_bytes(B, N, d_pair, d_hidden, direction, &need);
  if (rc != B200_TRIMUL_OK) return rc;
  if (static_cast<long long>(B) * N * N > kStaticMaxCells || need > kStaticWorkspaceBytes) return B200_TRIMUL_E_TOO_LARGE;
  DeviceInfo info;
  rc = device_info(&info);  // a device of another architecture is reported as such, before the symbol look-up fails on it
  if (rc != B200_TRIMUL_OK) return rc;
  void* scratch = nullptr;
  rc = static_scratch(&scratch);
  if (rc != B200_TRIMUL_OK) return rc;
  if (device_status_out != nullptr) *device_status_out = static_cast<int*>(scratch);
  return b200_trimul_forward(z, w_left, w_left_gate, w_right, w_right_gate, w_gate, w_out, weight_dtype, ln_in_w,
                             ln_in_b, ln_out_w, ln_out_b, bias_opt, token_mask, pair_mask, y, scratch,
                             kStaticWorkspaceBytes, B, N, d_pair, d_hidden, direction, eps_in, eps_out, residual,
                             cuda_stream);
}

#include "backward_host.inc"
#include "transition_backward_host.inc"
