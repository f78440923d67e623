// Persistent, warp-specialised tcgen05 GEMM for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T  (both operands K-major).
//
//   kind 0  bf16 x bf16 -> fp32 accumulate in TMEM -> bf16
//   kind 1  FP8 e4m3 x e4m3 with DeepSeek-style block scales: A carries one fp32 scale per row per 128-wide
//           K group, B one fp32 scale per 128x128 tile.  Every 128-K group is accumulated on the tensor cores
//           into a fresh TMEM buffer and folded into fp32 registers as  acc += partial * a_scale * b_scale
//           (two-level accumulation; same numerics as the reference's fp8_gemm_t_blockscaled kernel,
//           kernels/gb10/common/fp8_gemm_t_blockscaled.cu:15-17, which does it with mma.sync).
//
// Roles (320 threads, one CTA per SM, static round-robin over work items):
//   warp 0      TMA producer: 128B-swizzled A/B tiles into a multi-stage shared-memory ring
//   warp 1      TMEM owner + single-thread tcgen05.mma issuer, two TMEM accumulator buffers
//   warps 2..9  epilogue: tcgen05.ld, scale folding, bf16 conversion, global stores, split-K reduction
//
// Split-K: a work item is (k-split, n-tile, m-tile).  Partials go to an fp32 workspace; the CTA that finishes
// a tile last (ticket counter) sums the partials in split order, so results do not depend on timing.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "host_api.h"

namespace atlas {

constexpr int kBlockM = 128;
constexpr int kRowBytes = 128;            // one swizzle row = one BLOCK_K slice
constexpr int kEpiWarps = 8;
constexpr int kGemmThreads = 32 * (2 + kEpiWarps);

template <int BLOCK_N>
struct GemmCfg {
  static constexpr int kABytes = kBlockM * kRowBytes;
  static constexpr int kBBytes = BLOCK_N * kRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BLOCK_N == 256 ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BLOCK_N < 32 ? 32 : 2 * BLOCK_N;
  static constexpr int kHalf = BLOCK_N / 2;             // columns per epilogue thread
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 512 /*barriers*/;
};

struct GemmParams {
  void* C;
  const float* a_scale;
  const float* b_scale;
  float* workspace;
  int* counters;
  status_t* status;
  long long ldc;
  long long sa_m, sa_k;     // a_scale strides (elements) over rows / k-groups
  int M, N, K;
  int k_blocks;             // number of 128-byte K slices
  int splits, kb_per_split;
  int m_tiles, n_tiles;
  int b_scale_ld;           // k-groups per row of b_scale
  int vec_ok;               // 16-byte stores into C are legal
};

template <int BLOCK_N, bool FP8>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
  using Cfg = GemmCfg<BLOCK_N>;
  constexpr int kStages = Cfg::kStages;
  constexpr int HALF = Cfg::kHalf;
  constexpr int kElemsPerRow = FP8 ? 128 : 64;          // BLOCK_K in elements
  constexpr uint32_t kIdesc = make_idesc(kBlockM, BLOCK_N, FP8 ? 0u : 1u);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile int* ticket_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kEpiWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_items = p.m_tiles * p.n_tiles * p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int m_tile = item % p.m_tiles;
        const int rest = item / p.m_tiles;
        const int n_tile = rest % p.n_tiles;
        const int split = rest / p.n_tiles;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, 0x100)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          mbar_expect_tx(&full[stage], Cfg::kStageBytes);
          tma_load_2d(sa, &tmap_a, &full[stage], kb * kElemsPerRow, m_tile * kBlockM);
          tma_load_2d(sa + Cfg::kABytes, &tmap_b, &full[stage], kb * kElemsPerRow, n_tile * BLOCK_N);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // give copies that are already in flight time to land before the CTA's shared memory goes away
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc_iter = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int split = item / (p.m_tiles * p.n_tiles);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        if (!FP8) {
          const uint32_t buf = acc_iter & 1u, aph = (acc_iter >> 1) & 1u;
          if (!mbar_wait(&acc_empty[buf], aph ^ 1u, abort_flag, p.status, 0x200)) { ok = false; break; }
          tc_fence_after();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          uint32_t buf = acc_iter & 1u;
          if (FP8) {
            const uint32_t aph = (acc_iter >> 1) & 1u;
            if (!mbar_wait(&acc_empty[buf], aph ^ 1u, abort_flag, p.status, 0x201)) { ok = false; break; }
          }
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 0x202)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + Cfg::kABytes);
          const uint32_t d = tmem_base + buf * BLOCK_N;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t accum = FP8 ? (k > 0) : (kb > kb0 || k > 0);
            if (FP8) umma_f8(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, accum);
            else     umma_f16(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, accum);
          }
          umma_commit(&empty[stage]);
          if (FP8) { umma_commit(&acc_full[buf]); ++acc_iter; }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (!FP8) { umma_commit(&acc_full[acc_iter & 1u]); ++acc_iter; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps)
    const int e = warp - 2;
    const int lane_group = warp & 3;                 // TMEM lanes this warp may touch: [32*lane_group, +32)
    const int half = e >> 2;                         // which half of the tile's columns
    const int row_in_tile = lane_group * 32 + lane;
    const uint32_t t_lane = (uint32_t)(lane_group * 32) << 16;
    const int epi_tid = threadIdx.x - 64;
    uint32_t acc_iter = 0;
    bool ok = true;
    float acc[HALF];
    // This loop never exits early: the split-K path below uses named barriers that need all eight warps.
    // Once a wait has failed (`ok` false) the remaining items only walk the barriers.
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const int m_tile = item % p.m_tiles;
      const int rest = item / p.m_tiles;
      const int n_tile = rest % p.n_tiles;
      const int split = rest / p.n_tiles;
      const int kb0 = split * p.kb_per_split;
      const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
      const int m = m_tile * kBlockM + row_in_tile;
      const int n_base = n_tile * BLOCK_N + half * HALF;
      if (!ok) {
        // fall through to the write-out barriers without touching TMEM
      } else if (FP8) {
#pragma unroll
        for (int i = 0; i < HALF; ++i) acc[i] = 0.f;
        const float* bs = p.b_scale + (size_t)(n_base / 128) * p.b_scale_ld;
        const bool row_ok = m < p.M;
        const bool col_ok = n_base < p.N;
        float s_next = (row_ok && col_ok && kb0 < kb1) ? p.a_scale[m * p.sa_m + kb0 * p.sa_k] * __ldg(bs + kb0) : 0.f;
        for (int kb = kb0; kb < kb1; ++kb) {
          const float s = s_next;
          if (kb + 1 < kb1 && row_ok && col_ok) s_next = p.a_scale[m * p.sa_m + (kb + 1) * p.sa_k] * __ldg(bs + kb + 1);
          const uint32_t buf = acc_iter & 1u, aph = (acc_iter >> 1) & 1u;
          if (!mbar_wait(&acc_full[buf], aph, abort_flag, p.status, 0x300)) { ok = false; break; }
          tc_fence_after();
          const uint32_t taddr = tmem_base + t_lane + buf * BLOCK_N + half * HALF;
#pragma unroll
          for (int c = 0; c < HALF / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(r[i]), s, acc[c * 32 + i]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          ++acc_iter;
        }
      } else {
        const uint32_t buf = acc_iter & 1u, aph = (acc_iter >> 1) & 1u;
        if (mbar_wait(&acc_full[buf], aph, abort_flag, p.status, 0x301)) {
          tc_fence_after();
          const uint32_t taddr = tmem_base + t_lane + buf * BLOCK_N + half * HALF;
#pragma unroll
          for (int c = 0; c < HALF / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[c * 32 + i] = __uint_as_float(r[i]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          ++acc_iter;
        } else {
          ok = false;
        }
      }

      // ---- write out
      if (p.splits == 1) {
        if (ok && m < p.M) {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.ldc;
#pragma unroll
          for (int j = 0; j < HALF; j += 8) {
            const int n = n_base + j;
            if (p.vec_ok && n + 8 <= p.N) {
              uint4 v;
              v.x = pack_bf16x2(acc[j + 0], acc[j + 1]);
              v.y = pack_bf16x2(acc[j + 2], acc[j + 3]);
              v.z = pack_bf16x2(acc[j + 4], acc[j + 5]);
              v.w = pack_bf16x2(acc[j + 6], acc[j + 7]);
              *reinterpret_cast<uint4*>(crow + n) = v;
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (n + i < p.N) crow[n + i] = __float2bfloat16_rn(acc[j + i]);
            }
          }
        }
      } else {
        // fp32 partial -> workspace[split][m][n], then ticket; last arriver reduces in split order
        const size_t plane = (size_t)p.M * p.N;
        if (ok && m < p.M) {
          float* wrow = p.workspace + (size_t)split * plane + (size_t)m * p.N;
#pragma unroll
          for (int j = 0; j < HALF; ++j)
            if (n_base + j < p.N) wrow[n_base + j] = acc[j];
        }
        __threadfence();
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        const int tile_id = n_tile * p.m_tiles + m_tile;
        if (epi_tid == 0) *ticket_slot = atomicAdd(&p.counters[tile_id], 1);
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        const int ticket = *ticket_slot;
        if (ticket == p.splits - 1) {
          __threadfence();
          if (ok && m < p.M) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.ldc;
#pragma unroll 4
            for (int j = 0; j < HALF; ++j) {
              const int n = n_base + j;
              if (n < p.N) {
                float s = 0.f;
                for (int sp = 0; sp < p.splits; ++sp)
                  s += __ldcg(p.workspace + (size_t)sp * plane + (size_t)m * p.N + n);
                crow[n] = __float2bfloat16_rn(s);
              }
            }
          }
          if (epi_tid == 0) p.counters[tile_id] = 0;     // ready for the next launch
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ================================================================================ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

struct TmapKey {
  const void* ptr;
  uint64_t rows, cols, ld;
  uint32_t box_rows, esize;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && esize == o.esize;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.cols * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= (k.ld + k.box_rows * 131 + k.esize) * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
    return h;
  }
};

// Row-major [rows, cols] matrix with leading dimension `ld` (elements), tiles of box_rows x 128 bytes,
// 128-byte swizzle.  Cached: weights never move and graph-captured activations live at fixed addresses.
static int make_tmap_kmajor(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                            uint32_t box_rows, uint32_t esize) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key{ptr, rows, cols, ld, box_rows, esize};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -10;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esize};
  cuuint32_t box[2] = {128u / esize, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -11;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

template <int BLOCK_N, bool FP8>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BLOCK_N>;
  static bool attr_done = false;
  auto kern = gemm_tcgen05_kernel<BLOCK_N, FP8>;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return -20;
    attr_done = true;
  }
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace atlas

using namespace atlas;

// kind: 0 = bf16, 1 = fp8 block-scaled.  Strides are in elements.  `workspace` needs splits*M*N floats and
// `counters` m_tiles*n_tiles zero-initialised ints when splits > 1.  Returns 0 or a negative error code.
extern "C" int atlas_gemm(int kind, const void* A, const void* B, void* C, const float* a_scale, long long sa_m,
                          long long sa_k, const float* b_scale, int b_scale_ld, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, int block_n, int splits, float* workspace, int* counters,
                          int num_sms, unsigned long long* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const uint32_t esize = kind == 1 ? 1 : 2;
  const int elems_per_row = 128 / esize;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
  if ((lda * esize) % 16 || (ldb * esize) % 16) return -2;
  if (kind == 1 && (K % 128)) return -3;
  if (block_n != 64 && block_n != 128 && block_n != 256) return -4;
  CUtensorMap ta, tb;
  int rc = make_tmap_kmajor(&ta, A, M, K, lda, kBlockM, esize);
  if (rc) return rc;
  rc = make_tmap_kmajor(&tb, B, N, K, ldb, block_n, esize);
  if (rc) return rc;
  GemmParams p;
  p.C = C; p.a_scale = a_scale; p.b_scale = b_scale; p.workspace = workspace; p.counters = counters;
  p.status = status; p.ldc = ldc; p.sa_m = sa_m; p.sa_k = sa_k; p.M = M; p.N = N; p.K = K;
  p.k_blocks = (K + elems_per_row - 1) / elems_per_row;
  if (splits < 1) splits = 1;
  if (splits > p.k_blocks) splits = p.k_blocks;
  p.kb_per_split = (p.k_blocks + splits - 1) / splits;
  p.splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  if (p.splits > 1 && (!workspace || !counters)) return -5;
  p.m_tiles = (M + kBlockM - 1) / kBlockM;
  p.n_tiles = (N + block_n - 1) / block_n;
  p.b_scale_ld = b_scale_ld;
  p.vec_ok = ((ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
  const long long items = (long long)p.m_tiles * p.n_tiles * p.splits;
  int grid = (int)(items < num_sms ? items : num_sms);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (kind == 1) {
    if (block_n == 64) return launch_gemm<64, true>(ta, tb, p, grid, st);
    if (block_n == 128) return launch_gemm<128, true>(ta, tb, p, grid, st);
    return launch_gemm<256, true>(ta, tb, p, grid, st);
  }
  if (block_n == 64) return launch_gemm<64, false>(ta, tb, p, grid, st);
  if (block_n == 128) return launch_gemm<128, false>(ta, tb, p, grid, st);
  return launch_gemm<256, false>(ta, tb, p, grid, st);
}
