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
//   warp 0       TMA producer: 128B-swizzled A/B tiles into a multi-stage shared-memory ring
//   warp 1       TMEM owner + single-thread tcgen05.mma issuer, ring of up to four TMEM accumulator buffers
//   warps 2..9   epilogue: tcgen05.ld, scale folding, bf16 conversion, global stores, split-K reduction
//
// Split-K: a work item is (k-split, n-tile, m-tile).  Partials go to an fp32 workspace; the CTA that finishes
// a tile last (ticket counter) sums the partials in split order, so results do not depend on timing.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "host_api.h"
#include "tmap.h"

namespace atlas {

constexpr int kBlockM = 128;
constexpr int kRowBytes = 128;            // one swizzle row = one BLOCK_K slice
constexpr int kCtrlWarps = 2;            // warp 0: TMA producer, warp 1: MMA issuer
constexpr int kRowsPerReadyFlag = 8;     // granularity of the "rows have arrived" flags of a gathered A operand
// Epilogue warps: eight (two per TMEM lane quadrant) or sixteen.  The FP8 path keeps the whole accumulator of a tile in
// registers across its per-k-group folds: 128 x 256 / (32 x warps) floats per thread, i.e. 128 with eight warps (fits
// the 200-register budget of a 320-thread CTA) and 64 with sixteen (112-register budget of a 576-thread CTA).
__host__ __device__ constexpr int epi_warps(int block_n, bool fp8) { return (fp8 && block_n == 256) ? 16 : 8; }
// The fused-collective variants carry one more warp that raises the peers' flags (see the signal warp in the kernel);
// warps are allocated four at a time, so ten and eleven warps cost the same.
__host__ __device__ constexpr int gemm_threads_w(int warps, bool fuse = false) { return 32 * (kCtrlWarps + warps + (fuse ? 1 : 0)); }

template <int BLOCK_N>
struct GemmCfg {
  static constexpr int kABytes = kBlockM * kRowBytes;
  static constexpr int kBBytes = BLOCK_N * kRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BLOCK_N == 256 ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int kAccStages = (512 / BLOCK_N) < 4 ? (512 / BLOCK_N) : 4;   // TMEM accumulator ring depth
  static constexpr int kTmemCols = kAccStages * BLOCK_N;
  // Activation scales travel in their own ring, deeper than the tile ring: the producer runs at most kStages k-groups
  // ahead of the tensor cores and those at most kAccStages ahead of the epilogue, so a slot is never overwritten
  // before the epilogue has read it and the tile stages can be recycled as soon as their MMAs retire.
  static constexpr int kScaleSlots = kStages + kAccStages + 1;
  static constexpr int kScaleRingBytes = kScaleSlots * kBlockM * 4;   // per slot: 128 activation scales (fp32)
  static constexpr int kBScaleMax = 512;                          // k-groups of one split kept in shared memory
  static constexpr int kBScaleBytes = 2 * 2 * kBScaleMax * 4;     // double-buffered over tiles, two 128-column groups
  static constexpr int kXchBytes = 2 * 4 * kBlockM * 4;           // fused epilogues: per-row partial (max, sum of squares) of up to four column slices
  static constexpr int kSmemBytes = kStages * kStageBytes + kScaleRingBytes + kBScaleBytes + kXchBytes + 1024 /*align*/ + 512 /*barriers*/;
};

struct GemmParams {
  void* C;
  const float* a_scale;
  const float* b_scale;
  float* workspace;
  int* counters;
  status_t* status;
  long long ldc;
  long long sa_k;           // a_scale is k-group major: scale(m, g) = a_scale[g * sa_k + m]; sa_k % 4 == 0, rows padded to 128
  int M, N, K;
  int k_blocks;             // number of 128-byte K slices
  int splits, kb_per_split;
  int m_tiles, n_tiles;
  int b_scale_ld;           // k-groups per row of b_scale
  int vec_ok;               // 16-byte stores into C are legal
  int cluster_splits;       // > 1: the K splits of a tile are the CTAs of one thread-block cluster (one item per CTA, a
                            // single m-tile): partials meet in distributed shared memory instead of the workspace and
                            // every CTA finishes 128 / cluster_splits rows of the tile (see cluster_tail)
  int a_box_rows;           // rows of A one tile copy carries (8..128): decode-size problems copy only the rows that exist,
                            // the rest of the 128-row operand slot keeps stale bytes whose output rows are never stored
  // grouped (MoE) mode: rows are expert-sorted and every expert's segment is padded to a multiple of 128 rows, so
  // m-tile i covers rows [128 i, 128 i + 128) and belongs to expert tile_expert[i]; B is the stack [E * expert_n, K].
  // fused all-reduce (row-parallel GEMM): peers' symmetric areas, see the FUSE_AR path of the kernel
  uint8_t* ar_data[8];
  uint32_t* ar_flags[8];
  unsigned int* ar_state;       // [0] epoch of the last finished call, [1] CTAs finished in this call
  long long ar_max_cycles;
  size_t ar_part_src_stride;    // bytes between two source ranks' partial regions
  size_t ar_result_off;         // byte offset of the [M, N] bf16 result inside the area
  int ar_rank, ar_world, ar_max_tiles;
  int prefetch_b;               // k-slices of B to request into L2 ahead of the tile ring (0 = off)
  int ar_mode;                  // 0 = two-shot (owner reduces, result pushed back), 1 = one-shot (partials pushed to all),
                                // 2 = reduce-scatter (partials pushed to the row block's owner, nothing comes back)
  int rs_tiles_per_rank;        // mode 2: m-tiles (128-row blocks) owned by each rank, in rank order
  int rs_rows_per_rank;         // mode 2, > 0: a single m-tile whose ROWS are owned rank by rank in groups of this many rows
                                // (a multiple of 8; decode-size steps): every row goes to its own owner, and the tile's flag is
                                // raised at every rank that owns some of its rows
  // gathered A operand (sequence-parallel all-gather -> GEMM): rows of A are written into this rank's memory by their
  // owners; one flag per group of kRowsPerReadyFlag rows carries the epoch of the gather that filled it
  const uint32_t* a_ready;
  const unsigned int* a_ready_epoch;
  size_t ar_parity_stride;      // one-shot: bytes between the two epoch-parity halves of the partial area
  // ---- fused epilogues (epi_mode != 0 replaces the bf16 store of C)
  //   1  C = [gate | up] of a SwiGLU projection (B is the stack [gate rows; up rows], N = 2 * act_cols): the tile takes 32-row
  //      chunks of gate and up alternately, the epilogue computes silu(gate) * up, quantises it to FP8 in 128-wide groups
  //      and stores rows + scales (scales k-group major, like every activation scale of this library)
  //   2  C + residual -> residual (in place); (new residual * norm weight) quantised to FP8 in 128-wide groups -> q_out /
  //      s_out; per-row sums of squares of each column tile -> ss_out[n_tile][row].  The row's 1/rms factor is NOT
  //      applied here: RMSNorm's per-row factor commutes with the next linear layer, whose GEMM applies it (ss_in).
  // ss_in (any mode): this GEMM's A operand is such a deferred-norm activation: every output row is multiplied by
  // rsqrt(sum_j ss_in[j][row] * ss_inv_h + ss_eps) before anything else happens to it.
  int epi_mode;
  int act_cols;                 // mode 1: number of activation columns (= N / 2)
  uint8_t* q_out; long long ldq;
  float* s_out; long long s_ld;
  __nv_bfloat16* residual; long long ldr;
  const __nv_bfloat16* norm_w; int norm_plus_one;
  float* ss_out; long long ss_out_ld;
  const float* ss_in; int ss_in_parts; long long ss_in_ld; float ss_inv_h, ss_eps;
  // phase trace (nullptr = off): 32 words per CTA; [0] / [12] the global nanosecond timer at entry / exit, the rest SM
  // cycle counts: [1] entry, [2] barriers + TMEM ready, [3] previous kernel done, [4] first copies issued, [5] first tile
  // landed, [6] last MMA committed, [8] last fold done, [9] split-K ticket known (cluster form: every CTA of the cluster
  // past its k loop), [10] output stored, [11] exit; cluster split-K tail: [19] partial rows sent, [20] all partials here,
  // [21] rows summed.  Nothing is stamped inside the per-slice loops of the epilogue warps: their register budget is
  // what the fold needs.
  unsigned long long* timeline;
  const int* tile_expert;       // nullptr = plain GEMM
  const int* num_m_tiles_ptr;   // device-side tile count (the host cannot know it)
  int expert_n;                 // output features per expert
  long long b_scale_expert_stride;
};

ATLAS_DEVICE void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

ATLAS_DEVICE void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
ATLAS_DEVICE uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
ATLAS_DEVICE bool wait_flag_eq(const uint32_t* p, uint32_t want, status_t* status, uint32_t site, long long max_cycles) {
  const long long t0 = clock64();
  // epochs only grow: a peer that is already one call ahead has written want + 1, which also ends the wait
  while ((int32_t)(ld_acquire_sys_u32(p) - want) < 0) {
    if (clock64() - t0 > max_cycles) { report_status(status, kFlagTimeout, site); return false; }
    __nanosleep(20);
  }
  return true;
}

// FUSE_AR: the GEMM is one rank's share of a row-parallel (K-sharded) projection.  Tile t belongs to rank t % world.
//   GEMM phase   the epilogue stores its bf16 partial tile into the OWNER's partial region [this rank][t / world]
//                (peer stores over NVLink) and raises part_flag[t][this rank] at the owner.
//   reduce phase for each tile it owns a rank waits for all ranks' flags, sums the partials in rank order and stores
//                the finished tile into EVERY rank's result area, then raises final_flag[t] everywhere.
//   drain        a rank leaves the kernel once it has seen final_flag of every tile, so the next kernel in the stream
//                finds the whole [M, N] result in its own memory.
// Transfers therefore overlap the math tile by tile; flags carry the call's epoch, so nothing is ever reset.
// acc{0,1} += v{0,1} * s on the packed fp32 pipe (one instruction for two lanes of the accumulator)
ATLAS_DEVICE void ffma2(float& a0, float& a1, uint32_t v0, uint32_t v1, uint64_t s2) {
  asm("{\n\t.reg .b64 a, v;\n\t"
      "mov.b64 a, {%0, %1};\n\t"
      "mov.b64 v, {%2, %3};\n\t"
      "fma.rn.f32x2 a, v, %4, a;\n\t"
      "mov.b64 {%0, %1}, a;\n\t}\n"
      : "+f"(a0), "+f"(a1)
      : "r"(v0), "r"(v1), "l"(s2));
}
ATLAS_DEVICE uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

// Work item -> (m-tile, n-tile, K split).  Cluster mode: consecutive CTAs are the splits of one n-tile.
struct ItemPos { int m_tile, n_tile, split; };
ATLAS_DEVICE ItemPos item_pos(const GemmParams& p, int item, int m_tiles) {
  ItemPos r;
  if (p.cluster_splits > 1) {
    r.m_tile = 0; r.n_tile = item / p.cluster_splits; r.split = item % p.cluster_splits;
  } else {
    r.m_tile = item % m_tiles;
    const int rest = item / m_tiles;
    r.n_tile = rest % p.n_tiles; r.split = rest / p.n_tiles;
  }
  return r;
}

// Split-K tail of a 128 x 128 tile whose S splits form a thread-block cluster.  On entry every epilogue thread holds its
// row's 64 partial sums (`acc`, thread = (row_in_tile, half)) and every CTA of the cluster is past its k loop, so the
// operand rings are free.  The partial rows are scattered into the ring of the CTA that finishes them (CTA c takes rows
// [c R, c R + R), R = 128 / S; 16-byte blocks XOR-swizzled by row so that neither side has bank conflicts), a cluster
// barrier publishes them, and each CTA sums its rows in split order with 256 / R threads per row: row-contiguous residual
// and output accesses, S times the parallelism of a last-ticket reduction, no global workspace, atomics or fences.
template <int S>
ATLAS_DEVICE void cluster_tail(const GemmParams& p, uint8_t* smem, const float (&acc)[64], int split, int half, int row_in_tile,
                               int epi_tid, int n_tile, int M_rows, unsigned long long* tl) {
  constexpr int kN = 128, R = kBlockM / S, TPR = 256 / R, CPT = kN / TPR;      // S = 4: 32 rows, 8 threads x 16 columns
  float* xbuf = reinterpret_cast<float*>(smem);                                 // [S][R][128] fp32
  {
    const int dst_cta = row_in_tile / R, lr = row_in_tile % R;
    const uint32_t remote = cluster_map_shared(smem_u32(xbuf) + (uint32_t)((split * R + lr) * kN * 4), (uint32_t)dst_cta);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int c4 = (half * 16 + j) ^ (lr & 31);
      st_cluster_f32x4(remote + c4 * 16, acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
    }
  }
  if (tl && epi_tid == 0) tl[19] = clock64();
  cluster_sync_all();
  if (tl && epi_tid == 0) tl[20] = clock64();
  const int fr = epi_tid / TPR, seg = epi_tid % TPR;
  const int gm = split * R + fr;                         // the tile is the only m-tile
  const int n0 = n_tile * kN + seg * CPT;
  float v[CPT];
#pragma unroll
  for (int i = 0; i < CPT; ++i) v[i] = 0.f;
#pragma unroll
  for (int s = 0; s < S; ++s) {
    const float* rowp = xbuf + (s * R + fr) * kN;
#pragma unroll
    for (int j = 0; j < CPT / 4; ++j) {
      const int c4 = (seg * (CPT / 4) + j) ^ (fr & 31);
      const float4 t = *reinterpret_cast<const float4*>(rowp + c4 * 4);
      v[4 * j] += t.x; v[4 * j + 1] += t.y; v[4 * j + 2] += t.z; v[4 * j + 3] += t.w;
    }
  }
  if (tl && epi_tid == 0) tl[21] = clock64();
  const bool live = gm < M_rows;
  if (p.ss_in != nullptr && live) {
    float t = 0.f;
    for (int j = 0; j < p.ss_in_parts; ++j) t += __ldg(p.ss_in + (size_t)j * p.ss_in_ld + gm);
    const float rstd = rsqrtf(t * p.ss_inv_h + p.ss_eps);
#pragma unroll
    for (int i = 0; i < CPT; ++i) v[i] *= rstd;
  }
  if (p.epi_mode == 2) {
    float amax = 0.f, ss = 0.f;
    if (live) {
      __nv_bfloat16* rrow = p.residual + (size_t)gm * p.ldr + n0;
      uint4 rv[CPT / 8], wv[CPT / 8];
#pragma unroll
      for (int j = 0; j < CPT / 8; ++j) {
        rv[j] = *reinterpret_cast<const uint4*>(rrow + 8 * j);
        wv[j] = __ldg(reinterpret_cast<const uint4*>(p.norm_w + n0 + 8 * j));
      }
#pragma unroll
      for (int j = 0; j < CPT / 8; ++j) {
        const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rv[j]);
        const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv[j]);
        uint4 ov;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 r2 = __bfloat1622float2(rh[i]);
          oh[i] = __floats2bfloat162_rn(v[8 * j + 2 * i] + r2.x, v[8 * j + 2 * i + 1] + r2.y);
          const float2 h2 = __bfloat1622float2(oh[i]);          // the rounded residual stream is what gets normalised
          ss += h2.x * h2.x + h2.y * h2.y;
          float2 w2 = __bfloat1622float2(wh[i]);
          if (p.norm_plus_one) { w2.x += 1.f; w2.y += 1.f; }
          v[8 * j + 2 * i] = h2.x * w2.x; v[8 * j + 2 * i + 1] = h2.y * w2.y;
          amax = fmaxf(amax, fmaxf(fabsf(v[8 * j + 2 * i]), fabsf(v[8 * j + 2 * i + 1])));
        }
        *reinterpret_cast<uint4*>(rrow + 8 * j) = ov;
      }
    }
    // the TPR threads of a row are neighbouring lanes
#pragma unroll
    for (int off = 1; off < TPR; off <<= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
      ss += __shfl_xor_sync(0xffffffffu, ss, off);
    }
    if (live) {
      const float sc = fmaxf(amax, 1e-20f) / 448.f;
      const float inv = __frcp_rn(sc);
      uint32_t w[CPT / 4];
#pragma unroll
      for (int j = 0; j < CPT / 4; ++j) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * inv, v[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * inv, v[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        w[j] = lo | (hi << 16);
      }
      uint4* dst = reinterpret_cast<uint4*>(p.q_out + (size_t)gm * p.ldq + n0);
#pragma unroll
      for (int j = 0; j < CPT / 16; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
      if (seg == 0) {
        p.s_out[(size_t)(n0 >> 7) * p.s_ld + gm] = sc;
        p.ss_out[(size_t)n_tile * p.ss_out_ld + gm] = ss;
      }
    }
  } else if (live) {
    __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)gm * p.ldc + n0;
#pragma unroll
    for (int j = 0; j < CPT / 8; ++j) {
      uint4 o;
      o.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]); o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
      o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]); o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
      *reinterpret_cast<uint4*>(crow + 8 * j) = o;
    }
  }
}

// TRACE compiles the phase stamps of GemmParams::timeline in; the kernels that serve traffic are built without them (a
// few extra instructions in the single-thread producer / MMA loops were worth 5 % of a prefill-size GEMM).
template <int BLOCK_N, bool FP8, bool FUSE_AR = false, int EPW = epi_warps(BLOCK_N, FP8), bool TRACE = false>
__global__ void __launch_bounds__(gemm_threads_w(EPW, FUSE_AR), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
  using Cfg = GemmCfg<BLOCK_N>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kEpiWarps = EPW;
  constexpr int kParts = kEpiWarps / 4;                 // column slices of a tile, one per warp of a lane quadrant
  constexpr int HALF = BLOCK_N / kParts;                // columns per epilogue thread
  constexpr int kElemsPerRow = FP8 ? 128 : 64;          // BLOCK_K in elements
  constexpr uint32_t kIdesc = make_idesc(kBlockM, BLOCK_N, FP8 ? 0u : 1u);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kScaleSlots = Cfg::kScaleSlots;
  float* sc_ring = reinterpret_cast<float*>(smem + kStages * Cfg::kStageBytes);        // [kScaleSlots][128]
  float* bs_smem = sc_ring + kScaleSlots * kBlockM;                                     // [2][kBScaleMax]
  float* xch = bs_smem + Cfg::kBScaleBytes / 4;                                        // [2][4][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + Cfg::kScaleRingBytes + Cfg::kBScaleBytes + Cfg::kXchBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;
  constexpr int kAcc = Cfg::kAccStages;
  uint64_t* acc_empty = acc_full + kAcc;
  uint64_t* sc_full = acc_empty + kAcc;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sc_full + kScaleSlots);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile int* ticket_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);
  // reduce-scatter mode: epilogue -> signal warp handshake (two slots), so that the system-scope release that publishes
  // a tile's peer stores is not paid by the warps that fold the next tile
  uint64_t* sig_full = reinterpret_cast<uint64_t*>(tmem_slot + 4);
  uint64_t* sig_free = sig_full + 2;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  unsigned long long* const tl = (TRACE && p.timeline) ? p.timeline + (size_t)blockIdx.x * 32 : nullptr;
  if (tl && threadIdx.x == 0) {
    unsigned long long g;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(g));
    tl[0] = g;
    tl[1] = clock64();
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < kScaleSlots; ++s) mbar_init(&sc_full[s], 1);
    for (int b = 0; b < kAcc; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kEpiWarps);
    }
    if (FUSE_AR) {
      for (int b = 0; b < 2; ++b) { mbar_init(&sig_full[b], kEpiWarps); mbar_init(&sig_free[b], 1); }
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  // Weight tiles do not depend on the previous kernel in the stream, so the producer asks for the first ones (L2 only)
  // before waiting for that kernel: their HBM latency overlaps its tail.  `pf_*` is a cursor over this CTA's
  // (item, k-slice) sequence that stays p.prefetch_b slices ahead of the ring's loads.
  int pf_item = blockIdx.x, pf_kb = 0, pf_kb1 = 0, pf_row = 0, pf_ahead = 0;
  const bool pf_on = p.prefetch_b > 0 && p.tile_expert == nullptr;
  const int pf_total = p.m_tiles * p.n_tiles * p.splits;
  auto pf_enter = [&]() {
    if (pf_item < pf_total) {
      const ItemPos ip = item_pos(p, pf_item, p.m_tiles);
      const int split = ip.split;
      pf_row = ip.n_tile * BLOCK_N;
      pf_kb = split * p.kb_per_split;
      pf_kb1 = min(p.k_blocks, pf_kb + p.kb_per_split);
    }
  };
  auto pf_step = [&]() {            // request one slice and advance the cursor
    if (pf_item >= pf_total) return;
    tma_prefetch_l2_2d(&tmap_b, pf_kb * kElemsPerRow, pf_row);
    if (++pf_kb >= pf_kb1) { pf_item += gridDim.x; pf_enter(); }
  };
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (pf_on) {
      pf_enter();
      for (; pf_ahead < p.prefetch_b; ++pf_ahead) pf_step();
    }
  }
  chain_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tl && threadIdx.x == 0) tl[2] = clock64();
  chain_wait();                         // barriers, TMEM and descriptors are set up; global memory from here on
  if (tl && threadIdx.x == 0) tl[3] = clock64();

  const int m_tiles = p.tile_expert ? *p.num_m_tiles_ptr : p.m_tiles;
  const int total_items = m_tiles * p.n_tiles * p.splits;
  const int M_rows = p.tile_expert ? m_tiles * kBlockM : p.M;
  const uint32_t ar_epoch = FUSE_AR ? p.ar_state[0] + 1u : 0u;
  uint32_t* const part_flags = FUSE_AR ? p.ar_flags[p.ar_rank] : nullptr;                       // [tile][src]
  (void)part_flags;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the work items; lane 0 issues the copies.  When A is a gathered operand the warp first polls
    // the arrival flags of the tile's row groups (one flag per lane) and remembers which m-tiles it has seen complete.
    uint32_t stage = 0, phase = 0, sc_slot = 0;
    bool ok = true;
    uint32_t seen[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};         // m-tiles known to be complete (up to 256)
    const uint32_t want_epoch = p.a_ready ? *p.a_ready_epoch : 0u;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const ItemPos ip = item_pos(p, item, m_tiles);
      const int m_tile = ip.m_tile;
      if (p.a_ready != nullptr && !((m_tile < 256) && (seen[m_tile >> 5] >> (m_tile & 31) & 1u))) {
        constexpr int kGroups = kBlockM / kRowsPerReadyFlag;      // 16 flags per m-tile
        const int row = m_tile * kBlockM + lane * kRowsPerReadyFlag;
        bool mine = true;
        if (lane < kGroups && row < p.M)
          mine = wait_flag_eq(p.a_ready + (size_t)m_tile * kGroups + lane, want_epoch, p.status, 0x620, p.ar_max_cycles);
        ok = __all_sync(0xffffffffu, mine);
        if (!ok) { if (lane == 0) *abort_flag = 1u; break; }
        if (m_tile < 256) seen[m_tile >> 5] |= 1u << (m_tile & 31);
        // the rows were written by other GPUs' ordinary stores and are read below by the copy engine
        asm volatile("fence.proxy.async;\n" ::: "memory");
      }
      if (lane == 0) {
        const int n_tile = ip.n_tile;
        const int split = ip.split;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, 0x100)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          mbar_expect_tx(&full[stage], p.a_box_rows * kRowBytes + Cfg::kBBytes);
          if (FP8) {
            mbar_expect_tx(&sc_full[sc_slot], kBlockM * 4);
            bulk_g2s(sc_ring + sc_slot * kBlockM, p.a_scale + (long long)kb * p.sa_k + m_tile * kBlockM, kBlockM * 4,
                     &sc_full[sc_slot]);
            if (++sc_slot == kScaleSlots) sc_slot = 0;
          }
          tma_load_2d(sa, &tmap_a, &full[stage], kb * kElemsPerRow, m_tile * kBlockM);
          if (p.epi_mode == 1) {
            // 32-row chunks, gate and up alternating, so that an epilogue thread's 64 columns are 32 gate values and
            // the 32 up values of the same activation columns (the tensor map of B has a 32-row box in this mode)
            const int a0 = n_tile * (BLOCK_N / 2);
#pragma unroll
            for (int c = 0; c < BLOCK_N / 32; ++c)
              tma_load_2d(sa + Cfg::kABytes + c * 32 * kRowBytes, &tmap_b, &full[stage], kb * kElemsPerRow,
                          ((c & 1) ? p.act_cols : 0) + a0 + (c >> 1) * 32);
          } else {
            tma_load_2d(sa + Cfg::kABytes, &tmap_b, &full[stage], kb * kElemsPerRow,
                        (p.tile_expert ? p.tile_expert[m_tile] * p.expert_n : 0) + n_tile * BLOCK_N);
          }
          if (pf_on) pf_step();
          if (tl && item == (int)blockIdx.x && kb == kb0) tl[4] = clock64();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    if (!ok && lane == 0) {
      // give copies that are already in flight time to land before the CTA's shared memory goes away
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    if (p.cluster_splits > 1) {            // the epilogue warps' two cluster barriers need every thread of the CTA
      __syncwarp();
      cluster_sync_all();
      cluster_sync_all();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc_iter = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int split = item_pos(p, item, m_tiles).split;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        if (!FP8) {
          const uint32_t buf = acc_iter % kAcc, aph = (acc_iter / kAcc) & 1u;
          if (!mbar_wait(&acc_empty[buf], aph ^ 1u, abort_flag, p.status, 0x200)) { ok = false; break; }
          tc_fence_after();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          const uint32_t buf = acc_iter % kAcc;
          if (FP8) {
            const uint32_t aph = (acc_iter / kAcc) & 1u;
            if (!mbar_wait(&acc_empty[buf], aph ^ 1u, abort_flag, p.status, 0x201)) { ok = false; break; }
          }
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 0x202)) { ok = false; break; }
          tc_fence_after();
          if (tl && item == (int)blockIdx.x && kb == kb0) tl[5] = clock64();
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
        if (!FP8) { umma_commit(&acc_full[acc_iter % kAcc]); ++acc_iter; }
        if (tl) tl[6] = clock64();
      }
    }
    if (p.cluster_splits > 1) {
      __syncwarp();
      cluster_sync_all();
      cluster_sync_all();
    }
  } else if (FUSE_AR && warp == kCtrlWarps + kEpiWarps) {
    // ------------------------------------------------------------------ signal warp (reduce-scatter mode)
    // For every tile, in the CTA's item order: wait until all epilogue warps have issued the tile's peer stores, then
    // raise the tile's flag at the owner with a system-scope release (cumulative over those stores through the
    // barrier).  The release waits for the stores to be acknowledged over NVLink; here that costs nobody anything.
    if (p.ar_mode == 2 && p.rs_rows_per_rank > 0) {
      // row-level ownership: lane o tells rank o, for every rank that owns rows of the (only) m-tile
      const int n_owners = min(p.ar_world, (M_rows + p.rs_rows_per_rank - 1) / p.rs_rows_per_rank);
      uint32_t it = 0;
      bool live = true;
      for (int item = blockIdx.x; item < total_items && live; item += gridDim.x, ++it) {
        const uint32_t slot = it & 1u, ph = (it >> 1) & 1u;
        bool got = true;
        if (lane == 0) got = mbar_wait(&sig_full[slot], ph, abort_flag, p.status, 0x630);
        live = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (!live) break;
        const int n_tile = (item / m_tiles) % p.n_tiles;
        if (lane < n_owners && *abort_flag == 0u)
          st_release_sys_u32(p.ar_flags[lane] + (size_t)n_tile * 8 + p.ar_rank, ar_epoch);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sig_free[slot]);
      }
    } else if (p.ar_mode == 2 && lane == 0) {
      uint32_t it = 0;
      for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it) {
        const uint32_t slot = it & 1u, ph = (it >> 1) & 1u;
        if (!mbar_wait(&sig_full[slot], ph, abort_flag, p.status, 0x630)) break;
        const int m_tile = item % m_tiles;
        const int n_tile = (item / m_tiles) % p.n_tiles;
        const int owner = min(m_tile / p.rs_tiles_per_rank, p.ar_world - 1);
        const int local_tile = m_tile - owner * p.rs_tiles_per_rank;
        if (*abort_flag == 0u)
          st_release_sys_u32(p.ar_flags[owner] + ((size_t)local_tile * p.n_tiles + n_tile) * 8 + p.ar_rank, ar_epoch);
        mbar_arrive(&sig_free[slot]);
      }
    }
  } else if (warp >= kCtrlWarps) {
    // ------------------------------------------------------------------ epilogue
    const int e = warp - kCtrlWarps;
    const int lane_group = warp & 3;                 // TMEM lanes this warp may touch: [32*lane_group, +32)
    const int half = e >> 2;                         // which column slice of the tile
    const int row_in_tile = lane_group * 32 + lane;
    const uint32_t t_lane = (uint32_t)(lane_group * 32) << 16;
    const int epi_tid = threadIdx.x - 32 * kCtrlWarps;
    uint32_t acc_iter = 0;
    uint32_t tile_iter = 0;
    uint32_t sc_slot = 0, sc_phase = 0;      // mirrors the producer's position in the activation-scale ring
    uint32_t rs_it = 0;                      // tiles handed to the signal warp (reduce-scatter mode)
    bool ok = true;
    float acc[HALF];
    // This loop never exits early: the split-K path below uses named barriers that need all eight warps.
    // Once a wait has failed (`ok` false) the remaining items only walk the barriers.
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const ItemPos ip = item_pos(p, item, m_tiles);
      const int m_tile = ip.m_tile;
      const int n_tile = ip.n_tile;
      const int split = ip.split;
      const int kb0 = split * p.kb_per_split;
      const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
      const int m = m_tile * kBlockM + row_in_tile;
      const int n_base = n_tile * BLOCK_N + half * HALF;
      // Weight scales of this tile's k range -> shared memory (one row per 128-column group of the tile).  The
      // buffer alternates between tiles so that the single barrier below also protects the previous tile's readers.
      // Every epilogue warp runs this for every item, whatever `ok` says.
      float* bs_buf = bs_smem + (tile_iter & 1u) * 2 * Cfg::kBScaleMax;
      ++tile_iter;
      if (FP8) {
        const int nkb = kb1 - kb0;
        const int kRows = (BLOCK_N > 128 || p.epi_mode == 1) ? 2 : 1;
        for (int i = epi_tid; i < kRows * nkb; i += 32 * kEpiWarps) {
          const int r = i / nkb, g = i - r * nkb;
          // SwiGLU mode: row 0 = the gate rows' block, row 1 = the up rows' block of this tile's activation columns
          const int nb = p.epi_mode == 1 ? ((r ? p.act_cols : 0) + n_tile * (BLOCK_N / 2)) / 128 : (n_tile * BLOCK_N) / 128 + r;
          const float* bsrc = p.b_scale + (p.tile_expert ? (size_t)p.tile_expert[m_tile] * p.b_scale_expert_stride : 0);
          bs_buf[r * Cfg::kBScaleMax + g] = (nb * 128 < p.N) ? __ldg(bsrc + (size_t)nb * p.b_scale_ld + kb0 + g) : 0.f;
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
      }
      if (!ok) {
        // fall through to the write-out barriers without touching TMEM
      } else if (FP8) {
#pragma unroll
        for (int i = 0; i < HALF; ++i) acc[i] = 0.f;
        const float* bs_row = bs_buf + (p.epi_mode == 1 ? 0 : ((half * HALF) / 128) * Cfg::kBScaleMax);
        const float* bs_row_up = bs_buf + Cfg::kBScaleMax;          // SwiGLU mode: scales of the up rows
        for (int kb = kb0; kb < kb1; ++kb) {
          const uint32_t buf = acc_iter % kAcc, aph = (acc_iter / kAcc) & 1u;
          if (!mbar_wait(&acc_full[buf], aph, abort_flag, p.status, 0x300)) { ok = false; break; }
          tc_fence_after();
          if (!mbar_wait(&sc_full[sc_slot], sc_phase, abort_flag, p.status, 0x302)) { ok = false; break; }
          const float a_s = sc_ring[sc_slot * kBlockM + row_in_tile];
          const float s = a_s * bs_row[kb - kb0];
          if (++sc_slot == kScaleSlots) { sc_slot = 0; sc_phase ^= 1u; }
          const uint32_t taddr = tmem_base + t_lane + buf * BLOCK_N + half * HALF;
          // Pull the partial tile into registers with back-to-back tcgen05.ld, hand the TMEM buffer back to the
          // MMA issuer as soon as the loads have landed, and only then fold the scales in.
          // Chunks of the tile row go TMEM -> registers -> packed FMAs; the TMEM buffer returns to the MMA issuer as
          // soon as the last chunk's load has landed.  The chunk width is what the register budget leaves next to the
          // accumulators: 64 columns for a 64-column thread, 32 for 128 columns, 16 under the 112-register budget.
          constexpr int kChunk = kEpiWarps > 8 ? 16 : (HALF > 64 ? 32 : 64);
          const uint64_t s2 = pack_f32x2(s, s);
          uint64_t s2_up = s2;
          if (HALF == 64 && p.epi_mode == 1) { const float su = a_s * bs_row_up[kb - kb0]; s2_up = pack_f32x2(su, su); }
#pragma unroll
          for (int c0 = 0; c0 < HALF; c0 += kChunk) {
            uint32_t r[kChunk];
            if constexpr (kChunk == 16) {
              tmem_ld_32x32b_x16(taddr + c0, r);
            } else {
#pragma unroll
              for (int c = 0; c < kChunk / 32; ++c) tmem_ld_32x32b_x32(taddr + c0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
            }
            tmem_ld_wait();
            if (c0 + kChunk >= HALF) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[buf]);
            }
#pragma unroll
            for (int i = 0; i < kChunk; i += 2)
              ffma2(acc[c0 + i], acc[c0 + i + 1], r[i], r[i + 1], (HALF == 64 && c0 + i >= 32) ? s2_up : s2);
          }
          ++acc_iter;
        }
      } else {
        const uint32_t buf = acc_iter % kAcc, aph = (acc_iter / kAcc) & 1u;
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
      if (tl && epi_tid == 0) tl[8] = clock64();
      if constexpr (BLOCK_N == 128 && HALF == 64 && !FUSE_AR) {
        if (p.cluster_splits > 1) {
          // (a wait that ran out leaves rubbish in this CTA's partial; the status word already says so)
          cluster_sync_all();              // every CTA of the cluster is past its k loop: the operand rings are free
          if (tl && epi_tid == 0) tl[9] = clock64();
          if (p.cluster_splits == 4) cluster_tail<4>(p, smem, acc, split, half, row_in_tile, epi_tid, n_tile, M_rows, tl);
          else                       cluster_tail<2>(p, smem, acc, split, half, row_in_tile, epi_tid, n_tile, M_rows, tl);
          continue;
        }
      }
      bool do_store = ok;
      if (p.splits > 1) {
        // fp32 partials go to the workspace in fragment order (float4 index j4, then epilogue thread), so every
        // store and load below is a fully coalesced 512-byte warp access; the CTA that takes the last ticket of
        // the tile sums the partials in split order.
        float4* ws4 = reinterpret_cast<float4*>(p.workspace);
        const size_t tiles = (size_t)m_tiles * p.n_tiles;
        const size_t tile_id = (size_t)n_tile * m_tiles + m_tile;
        constexpr size_t kFrag4 = (size_t)(32 * kEpiWarps) * (HALF / 4);
        const bool row_live = m < M_rows;                      // rows past the problem's edge carry nothing worth moving
        if (ok && row_live) {
          float4* dst = ws4 + ((size_t)split * tiles + tile_id) * kFrag4 + epi_tid;
#pragma unroll
          for (int j4 = 0; j4 < HALF / 4; ++j4)
            dst[(size_t)j4 * (32 * kEpiWarps)] = make_float4(acc[4 * j4], acc[4 * j4 + 1], acc[4 * j4 + 2], acc[4 * j4 + 3]);
        }
        __threadfence();
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        if (epi_tid == 0) *ticket_slot = atomicAdd(&p.counters[tile_id], 1);
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        const int ticket = *ticket_slot;
        do_store = ok && ticket == p.splits - 1;
        if (ticket == p.splits - 1) {
          __threadfence();
          if (ok && row_live) {
#pragma unroll
            for (int i = 0; i < HALF; ++i) acc[i] = 0.f;
            for (int sp = 0; sp < p.splits; ++sp) {
              const float4* src = ws4 + ((size_t)sp * tiles + tile_id) * kFrag4 + epi_tid;
#pragma unroll
              for (int j4 = 0; j4 < HALF / 4; ++j4) {
                const float4 v = __ldcg(src + (size_t)j4 * (32 * kEpiWarps));
                acc[4 * j4] += v.x; acc[4 * j4 + 1] += v.y; acc[4 * j4 + 2] += v.z; acc[4 * j4 + 3] += v.w;
              }
            }
          }
          if (epi_tid == 0) p.counters[tile_id] = 0;     // ready for the next launch
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
      }
      if (tl && epi_tid == 0) tl[9] = clock64();
      bool store_now = do_store;
      if (FUSE_AR && p.ar_mode == 1) {
        // ---- one-shot: this tile's bf16 partial goes to every peer (fragment order: 16-byte vector jv of epilogue
        // thread r sits at vector index jv * 128 + r, so a warp's store covers 512 contiguous bytes), one flag per
        // (tile, source) follows, and the same threads then add the peers' partials, which arrive in this rank's own
        // memory, to their registers in rank order (identical bits on every rank) and store C locally.
        const int tile_id = n_tile * m_tiles + m_tile;
        const int n_tiles_all = m_tiles * p.n_tiles;
        constexpr int kVec = HALF / 8;
        constexpr size_t kTileBytes = (size_t)kBlockM * BLOCK_N * 2;
        const size_t par_off = (size_t)(ar_epoch & 1u) * p.ar_parity_stride;
        const size_t one_flags = (size_t)p.ar_max_tiles * 9;
        const size_t frag = (size_t)(half * kVec) * kBlockM + row_in_tile;
        const bool live = do_store && m < M_rows;
        uint4 mine[kVec];
        if (live) {
#pragma unroll
          for (int jv = 0; jv < kVec; ++jv) {
            mine[jv].x = pack_bf16x2(acc[8 * jv + 0], acc[8 * jv + 1]);
            mine[jv].y = pack_bf16x2(acc[8 * jv + 2], acc[8 * jv + 3]);
            mine[jv].z = pack_bf16x2(acc[8 * jv + 4], acc[8 * jv + 5]);
            mine[jv].w = pack_bf16x2(acc[8 * jv + 6], acc[8 * jv + 7]);
          }
          for (int dst = 0; dst < p.ar_world; ++dst) {
            if (dst == p.ar_rank) continue;
            uint4* d = reinterpret_cast<uint4*>(p.ar_data[dst] + par_off +
                                                ((size_t)p.ar_rank * n_tiles_all + tile_id) * kTileBytes) + frag;
#pragma unroll
            for (int jv = 0; jv < kVec; ++jv) d[(size_t)jv * kBlockM] = mine[jv];
          }
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        if (do_store && epi_tid < p.ar_world && epi_tid != p.ar_rank) {
          st_release_sys_u32(p.ar_flags[epi_tid] + one_flags + (size_t)tile_id * 8 + p.ar_rank, ar_epoch);
          if (!wait_flag_eq(p.ar_flags[p.ar_rank] + one_flags + (size_t)tile_id * 8 + epi_tid, ar_epoch, p.status, 0x610,
                            p.ar_max_cycles))
            *abort_flag = 1u;
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        store_now = do_store && *abort_flag == 0u;
        if (live && store_now) {
#pragma unroll
          for (int i = 0; i < HALF; ++i) acc[i] = 0.f;
          // sources are taken a few at a time so that their loads are in flight together; the adds keep rank order
          constexpr int kSrcBatch = kVec <= 4 ? 4 : 2;
          for (int s0 = 0; s0 < p.ar_world; s0 += kSrcBatch) {
            uint4 raw[kSrcBatch][kVec];
#pragma unroll
            for (int b = 0; b < kSrcBatch; ++b) {
              const int src = s0 + b;
              if (src >= p.ar_world) break;
              const uint4* sp = reinterpret_cast<const uint4*>(p.ar_data[p.ar_rank] + par_off +
                                                               ((size_t)src * n_tiles_all + tile_id) * kTileBytes) + frag;
#pragma unroll
              for (int jv = 0; jv < kVec; ++jv) raw[b][jv] = src == p.ar_rank ? mine[jv] : __ldcg(sp + (size_t)jv * kBlockM);
            }
#pragma unroll
            for (int b = 0; b < kSrcBatch; ++b) {
              if (s0 + b >= p.ar_world) break;
#pragma unroll
              for (int jv = 0; jv < kVec; ++jv) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[b][jv]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = __bfloat1622float2(h[i]);
                  acc[8 * jv + 2 * i] += f.x;
                  acc[8 * jv + 2 * i + 1] += f.y;
                }
              }
            }
          }
        }
      } else if (FUSE_AR && p.ar_mode == 2) {
        // ---- reduce-scatter: the bf16 partial goes into the row block owner's area [source rank][local row][N]
        // (row-major, so the owner's reduce + norm kernel streams whole rows); one flag per (tile, source) follows.
        store_now = false;
        const int owner = min(m_tile / p.rs_tiles_per_rank, p.ar_world - 1);
        const int local_tile = m_tile - owner * p.rs_tiles_per_rank;
        __nv_bfloat16* dbase = reinterpret_cast<__nv_bfloat16*>(p.ar_data[owner] + (size_t)p.ar_rank * p.ar_part_src_stride) +
                               (size_t)local_tile * kBlockM * p.N;
        // row-level ownership (one m-tile): row r belongs to rank r / rows_per_rank and is its local row r % rows_per_rank
        const int rpr = p.rs_rows_per_rank;
        auto row_dst = [&](int r_in_tile) -> __nv_bfloat16* {
          if (rpr <= 0) return dbase + (size_t)r_in_tile * p.N;
          const int o = min(r_in_tile / rpr, p.ar_world - 1);
          return reinterpret_cast<__nv_bfloat16*>(p.ar_data[o] + (size_t)p.ar_rank * p.ar_part_src_stride) +
                 (size_t)(r_in_tile - o * rpr) * p.N;
        };
        if constexpr (HALF == 64) {
          // A thread holds 64 consecutive columns of ONE row, so a warp-wide 16-byte store would touch 32 rows: 32
          // separate 16-byte writes, which NVLink carries poorly.  The eight 16-byte vectors are transposed across each
          // group of eight lanes first (butterfly of shuffles): afterwards eight neighbouring lanes hold the eight
          // vectors of one row and every store instruction writes four whole 128-byte row segments.
          uint4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[j].x = pack_bf16x2(acc[8 * j + 0], acc[8 * j + 1]);
            v[j].y = pack_bf16x2(acc[8 * j + 2], acc[8 * j + 3]);
            v[j].z = pack_bf16x2(acc[8 * j + 4], acc[8 * j + 5]);
            v[j].w = pack_bf16x2(acc[8 * j + 6], acc[8 * j + 7]);
          }
#pragma unroll
          for (int sft = 4; sft >= 1; sft >>= 1) {
            const bool up = (lane & sft) != 0;
#pragma unroll
            for (int a = 0; a < 8; ++a) {
              if (a & sft) continue;
              const uint4 snd = up ? v[a] : v[a | sft];
              uint4 rcv;
              rcv.x = __shfl_xor_sync(0xffffffffu, snd.x, sft);
              rcv.y = __shfl_xor_sync(0xffffffffu, snd.y, sft);
              rcv.z = __shfl_xor_sync(0xffffffffu, snd.z, sft);
              rcv.w = __shfl_xor_sync(0xffffffffu, snd.w, sft);
              if (up) v[a] = rcv; else v[a | sft] = rcv;
            }
          }
          // now v[i] = vector (lane & 7) of row 8 * (lane >> 3) + i of this warp's 32 rows
          const int col = n_base + 8 * (lane & 7);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r_in_tile = lane_group * 32 + 8 * (lane >> 3) + i;
            if (ok && m_tile * kBlockM + r_in_tile < M_rows && col + 8 <= p.N)
              *reinterpret_cast<uint4*>(row_dst(r_in_tile) + col) = v[i];
          }
        } else if (ok && m < M_rows) {
          __nv_bfloat16* drow = row_dst(row_in_tile);
#pragma unroll
          for (int j = 0; j < HALF; j += 8) {
            const int n = n_base + j;
            if (n + 8 <= p.N) {
              uint4 v;
              v.x = pack_bf16x2(acc[j + 0], acc[j + 1]);
              v.y = pack_bf16x2(acc[j + 2], acc[j + 3]);
              v.z = pack_bf16x2(acc[j + 4], acc[j + 5]);
              v.w = pack_bf16x2(acc[j + 6], acc[j + 7]);
              *reinterpret_cast<uint4*>(drow + n) = v;
            }
          }
        }
        // hand the tile to the signal warp: slot (item count & 1), reused once the signal warp has released it
        {
          const uint32_t slot = rs_it & 1u, round = rs_it >> 1;
          __syncwarp();
          if (lane == 0) {
            if (round > 0 && !mbar_wait(&sig_free[slot], (round - 1) & 1u, abort_flag, p.status, 0x631)) ok = false;
            mbar_arrive(&sig_full[slot]);
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          ++rs_it;
        }
      } else if (FUSE_AR) {
        store_now = false;
        const int tile_id = n_tile * m_tiles + m_tile;
        const int owner = tile_id % p.ar_world;
        if (ok && m < M_rows) {
          uint8_t* tile_base = p.ar_data[owner] + (size_t)p.ar_rank * p.ar_part_src_stride +
                               (size_t)(tile_id / p.ar_world) * (kBlockM * BLOCK_N * 2);
          uint4* dst = reinterpret_cast<uint4*>(tile_base + ((size_t)row_in_tile * BLOCK_N + half * HALF) * 2);
#pragma unroll
          for (int j = 0; j < HALF; j += 8) {
            uint4 v;
            v.x = pack_bf16x2(acc[j + 0], acc[j + 1]);
            v.y = pack_bf16x2(acc[j + 2], acc[j + 3]);
            v.z = pack_bf16x2(acc[j + 4], acc[j + 5]);
            v.w = pack_bf16x2(acc[j + 6], acc[j + 7]);
            dst[j / 8] = v;
          }
        }
        // the release store below is cumulative over the epilogue warps' stores ordered before it by the barrier
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        if (epi_tid == 0)
          st_release_sys_u32(p.ar_flags[owner] + (size_t)tile_id * 8 + p.ar_rank, ar_epoch);
      }
      // ---- deferred RMSNorm factor of the A operand: one multiplier per output row
      if (p.ss_in != nullptr && store_now && m < M_rows) {
        float t = 0.f;
        for (int j = 0; j < p.ss_in_parts; ++j) t += __ldg(p.ss_in + (size_t)j * p.ss_in_ld + m);
        const float rstd = rsqrtf(t * p.ss_inv_h + p.ss_eps);
#pragma unroll
        for (int i = 0; i < HALF; ++i) acc[i] *= rstd;
      }
      if (HALF == 64 && p.epi_mode == 1) {
        // ---- SwiGLU + FP8 group quantisation: acc[0..31] = gate, acc[32..63] = up of activation columns
        // a0 + 32 * half + i; the four column slices of the 256-wide tile share one 128-wide quantisation group
        constexpr int kPartsPerGroup = 256 / BLOCK_N == 1 ? 4 : 2;       // 128-wide tiles hold half a group: not used
        const bool live = store_now && m < M_rows;
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float g = acc[i], u = acc[32 + i];
          const float v = __bfloat162float(__float2bfloat16_rn(__fdividef(g, 1.f + __expf(-g)) * u));
          acc[i] = v;
          amax = fmaxf(amax, fabsf(v));
        }
        xch[half * kBlockM + row_in_tile] = amax;
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        const int g0 = (half / kPartsPerGroup) * kPartsPerGroup;
#pragma unroll
        for (int j = 0; j < kPartsPerGroup; ++j) amax = fmaxf(amax, xch[(g0 + j) * kBlockM + row_in_tile]);
        if (live) {
          const float sc = fmaxf(amax, 1e-10f) / 448.f;
          const float inv = __frcp_rn(sc);
          const int col = n_tile * (BLOCK_N / 2) + half * 32;
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(acc[4 * j] * inv, acc[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(acc[4 * j + 2] * inv, acc[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
            w[j] = lo | (hi << 16);
          }
          uint4* dst = reinterpret_cast<uint4*>(p.q_out + (size_t)m * p.ldq + col);
          dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
          dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
          if (half == g0) p.s_out[(size_t)(col >> 7) * p.s_ld + m] = sc;
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));      // the exchange area is reused by the next tile
      } else if (HALF == 64 && p.epi_mode == 2) {
        // ---- residual add + RMSNorm weight + FP8 group quantisation + per-row sum of squares of this column tile
        constexpr int kPartsPerGroup = 2;                               // two 64-column threads per 128-wide group
        const bool live = store_now && m < M_rows;
        float amax = 0.f, ss = 0.f;
        if (live) {
          __nv_bfloat16* rrow = p.residual + (size_t)m * p.ldr + n_base;
#pragma unroll
          for (int j = 0; j < HALF; j += 8) {
            const uint4 rv = *reinterpret_cast<const uint4*>(rrow + j);
            const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rv);
            uint4 ov;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 r2 = __bfloat1622float2(rh[i]);
              oh[i] = __floats2bfloat162_rn(acc[j + 2 * i] + r2.x, acc[j + 2 * i + 1] + r2.y);
              const float2 h2 = __bfloat1622float2(oh[i]);          // the rounded residual stream is what gets normalised
              acc[j + 2 * i] = h2.x; acc[j + 2 * i + 1] = h2.y;
              ss += h2.x * h2.x + h2.y * h2.y;
            }
            *reinterpret_cast<uint4*>(rrow + j) = ov;
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(p.norm_w + n_base + j));
            const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float2 w2 = __bfloat1622float2(wh[i]);
              if (p.norm_plus_one) { w2.x += 1.f; w2.y += 1.f; }
              acc[j + 2 * i] *= w2.x; acc[j + 2 * i + 1] *= w2.y;
              amax = fmaxf(amax, fmaxf(fabsf(acc[j + 2 * i]), fabsf(acc[j + 2 * i + 1])));
            }
          }
        }
        xch[half * kBlockM + row_in_tile] = amax;
        xch[(4 + half) * kBlockM + row_in_tile] = ss;
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        const int g0 = (half / kPartsPerGroup) * kPartsPerGroup;
#pragma unroll
        for (int j = 0; j < kPartsPerGroup; ++j) amax = fmaxf(amax, xch[(g0 + j) * kBlockM + row_in_tile]);
        if (live) {
          const float sc = fmaxf(amax, 1e-20f) / 448.f;
          const float inv = __frcp_rn(sc);
          uint4* dst = reinterpret_cast<uint4*>(p.q_out + (size_t)m * p.ldq + n_base);
#pragma unroll
          for (int v4 = 0; v4 < HALF / 16; ++v4) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int b = v4 * 16 + j * 4;
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(acc[b] * inv, acc[b + 1] * inv), __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(acc[b + 2] * inv, acc[b + 3] * inv), __NV_SATFINITE, __NV_E4M3);
              w[j] = lo | (hi << 16);
            }
            dst[v4] = make_uint4(w[0], w[1], w[2], w[3]);
          }
          if (half == g0) p.s_out[(size_t)(n_base >> 7) * p.s_ld + m] = sc;
          if (half == 0) {
            float t = 0.f;
#pragma unroll
            for (int j = 0; j < kParts; ++j) t += xch[(4 + j) * kBlockM + row_in_tile];      // fixed order
            p.ss_out[(size_t)n_tile * p.ss_out_ld + m] = t;
          }
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
      } else
      if (store_now && m < M_rows) {
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
    }
    if (tl && epi_tid == 0) tl[10] = clock64();
    if (FUSE_AR && p.ar_mode != 0) {
      // nothing to drain.  One-shot: partial areas alternate with the epoch parity, and a rank can only be one call
      // ahead.  Reduce-scatter: the owner's reduce kernel waits on the tile flags, and a peer cannot reach its next
      // reduce-scatter GEMM before it has consumed every row this rank gathers from those partials.
      asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
      if (epi_tid == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(&p.ar_state[1], 1u);
        if (done == gridDim.x - 1) {
          p.ar_state[1] = 0;
          __threadfence();
          p.ar_state[0] = ar_epoch;
        }
      }
    } else if (FUSE_AR) {
      const int n_tiles_all = m_tiles * p.n_tiles;
      uint32_t* my_flags = p.ar_flags[p.ar_rank];
      uint32_t* final_base_off = nullptr;
      (void)final_base_off;
      const size_t final_off = (size_t)p.ar_max_tiles * 8;          // final flags follow the [tile][src] flags
      constexpr int kVecPerRow = BLOCK_N / 8;
      // ---- reduce phase: owned tiles rank + world * j, shared round-robin among this rank's CTAs
      for (int j = blockIdx.x; p.ar_rank + p.ar_world * j < n_tiles_all; j += gridDim.x) {
        const int tile_id = p.ar_rank + p.ar_world * j;
        if (epi_tid < p.ar_world) {
          if (!wait_flag_eq(my_flags + (size_t)tile_id * 8 + epi_tid, ar_epoch, p.status, 0x600, p.ar_max_cycles))
            *abort_flag = 1u;
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        const bool good = *abort_flag == 0u;
        const int m0 = (tile_id % m_tiles) * kBlockM, n0 = (tile_id / m_tiles) * BLOCK_N;
        if (good) {
          for (int v = epi_tid; v < kBlockM * kVecPerRow; v += 32 * kEpiWarps) {
            const int r = v / kVecPerRow, c8 = v % kVecPerRow;
            const int gm = m0 + r, gn = n0 + c8 * 8;
            if (gm >= M_rows || gn >= p.N) continue;
            float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            uint4 raws[8];
#pragma unroll
            for (int src = 0; src < 8; ++src)                 // all loads first, then the adds in rank order
              if (src < p.ar_world)
                raws[src] = *reinterpret_cast<const uint4*>(
                    p.ar_data[p.ar_rank] + (size_t)src * p.ar_part_src_stride + (size_t)j * (kBlockM * BLOCK_N * 2) +
                    ((size_t)r * BLOCK_N + c8 * 8) * 2);
#pragma unroll
            for (int src = 0; src < 8; ++src) {               // fixed order: identical bits on every rank
              if (src >= p.ar_world) break;
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raws[src]);
#pragma unroll
              for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); sum[2 * i] += f.x; sum[2 * i + 1] += f.y; }
            }
            uint4 o;
            o.x = pack_bf16x2(sum[0], sum[1]); o.y = pack_bf16x2(sum[2], sum[3]);
            o.z = pack_bf16x2(sum[4], sum[5]); o.w = pack_bf16x2(sum[6], sum[7]);
            for (int dst = 0; dst < p.ar_world; ++dst)
              *reinterpret_cast<uint4*>(p.ar_data[dst] + p.ar_result_off + ((size_t)gm * p.N + gn) * 2) = o;
          }
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
        if (epi_tid < p.ar_world) st_release_sys_u32(p.ar_flags[epi_tid] + final_off + tile_id, ar_epoch);
      }
      // ---- drain: see every tile's final flag before leaving
      for (int t = blockIdx.x * (32 * kEpiWarps) + epi_tid; t < n_tiles_all; t += gridDim.x * (32 * kEpiWarps)) {
        if (*abort_flag) break;
        if (!wait_flag_eq(my_flags + final_off + t, ar_epoch, p.status, 0x601, p.ar_max_cycles)) *abort_flag = 1u;
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kEpiWarps));
      if (epi_tid == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(&p.ar_state[1], 1u);
        if (done == gridDim.x - 1) {
          p.ar_state[1] = 0;
          __threadfence();
          p.ar_state[0] = ar_epoch;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (tl && threadIdx.x == 0) {
    unsigned long long g;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(g));
    tl[11] = clock64();
    tl[12] = g;
  }
}

// Trace buffer for the next launches of this library's tcgen05 GEMMs (32 words per CTA, see GemmParams::timeline);
// nullptr switches tracing off again.  Meant for single launches under a microbenchmark, not for serving.
static unsigned long long* g_gemm_timeline = nullptr;
extern "C" void atlas_gemm_set_timeline(unsigned long long* buf) { g_gemm_timeline = buf; }

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
  uint32_t box_rows, esize, box_bytes;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && esize == o.esize &&
           box_bytes == o.box_bytes;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.cols * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= (k.ld + k.box_rows * 131 + k.esize + k.box_bytes * 7919) * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
    return h;
  }
};

// Row-major [rows, cols] matrix with leading dimension `ld` (elements), tiles of box_rows x 128 bytes,
// 128-byte swizzle.  Cached: weights never move and graph-captured activations live at fixed addresses.
int make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                 uint32_t esize, uint32_t box_bytes, bool swizzle128) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key{ptr, rows, cols, ld, box_rows, esize, box_bytes | (swizzle128 ? 0x80000000u : 0u)};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -10;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esize};
  cuuint32_t box[2] = {box_bytes / esize, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -11;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

static int make_tmap_kmajor(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                            uint32_t box_rows, uint32_t esize) {
  return make_tmap_2d(out, ptr, rows, cols, ld, box_rows, esize, 128u, true);
}

template <int BLOCK_N, bool FP8, bool FUSE_AR = false, int EPW = epi_warps(BLOCK_N, FP8)>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BLOCK_N>;
  auto kern = gemm_tcgen05_kernel<BLOCK_N, FP8, FUSE_AR, EPW, false>;
  if constexpr (!FUSE_AR) {
    if (p.timeline != nullptr) kern = gemm_tcgen05_kernel<BLOCK_N, FP8, FUSE_AR, EPW, true>;
  }
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), Cfg::kSmemBytes) != cudaSuccess) return -20;
  if (p.cluster_splits > 1)
    return launch_chain_cluster(true, (unsigned)p.cluster_splits, kern, dim3(grid), dim3(gemm_threads_w(EPW, FUSE_AR)),
                                (size_t)Cfg::kSmemBytes, st, ta, tb, p) == cudaSuccess ? 0 : -21;
  return launch_chain_if(p.m_tiles <= 2 && p.tile_expert == nullptr, kern, dim3(grid), dim3(gemm_threads_w(EPW, FUSE_AR)),
                         (size_t)Cfg::kSmemBytes, st, ta, tb, p) == cudaSuccess ? 0 : -21;
}

// Rows of A per tile copy: a problem of at most 64 rows copies the next power of two of its row count (at least 8)
// instead of the whole 128-row slot.  A CTA's copy engine ingests ~50 bytes per clock whatever the tile, so at decode
// sizes the 16 KB activation tile (the same for every CTA, mostly padding) was taking a third to two thirds of the
// ingest that the weight stream needs (ATLAS_GEMM_ABOX=0 restores whole-slot copies).
static int a_box_for(int M) {
  static const bool on = [] { const char* e = getenv("ATLAS_GEMM_ABOX"); return !(e && e[0] == '0'); }();
  if (!on || M > 64) return kBlockM;
  int b = 8;
  while (b < M) b <<= 1;
  return b;
}

// Split-K through thread-block clusters (ATLAS_GEMM_CLUSTER=0 keeps the workspace + last-ticket reduction everywhere)
static bool cluster_splitk_enabled() {
  static const bool on = [] { const char* e = getenv("ATLAS_GEMM_CLUSTER"); return !(e && e[0] == '0'); }();
  return on;
}

// k-slices of weights requested into L2 ahead of the tile ring for decode-size GEMMs (ATLAS_GEMM_PREFETCH, 0 = off)
static int prefetch_depth() {
  static const int d = [] {
    const char* e = getenv("ATLAS_GEMM_PREFETCH");
    const int v = e ? atoi(e) : 0;   // off: on B200 the extra requests compete with the ring for TMA throughput (slower)
    return v < 0 ? 0 : (v > 64 ? 64 : v);
  }();
  return d;
}

// Epilogue warps of the 256-wide FP8 tile (ATLAS_GEMM_EPW256 = 8 or 16)
static int wide_fp8_epilogue_warps() {
  static const int w = [] {
    const char* e = getenv("ATLAS_GEMM_EPW256");
    return (e && atoi(e) == 8) ? 8 : 16;
  }();
  return w;
}

}  // namespace atlas

using namespace atlas;

// kind: 0 = bf16, 1 = fp8 block-scaled.  Strides are in elements.  For kind 1, a_scale is k-group major
// (scale(m, g) = a_scale[g * sa_k + m]) with sa_k a multiple of 4 and at least m_tiles*128, so that a 128-row
// slice is one aligned bulk copy.  With splits > 1, `workspace` needs splits*m_tiles*n_tiles*128*block_n floats and
// `counters` m_tiles*n_tiles zero-initialised ints.  Returns 0 or a negative error code.
static int gemm_impl(int kind, const void* A, const void* B, void* C, const float* a_scale, long long sa_m,
                     long long sa_k, const float* b_scale, int b_scale_ld, int M, int N, int K, long long lda,
                     long long ldb, long long ldc, int block_n, int splits, float* workspace, int* counters,
                     int num_sms, unsigned long long* status, void* stream, const uint32_t* a_ready,
                     const unsigned int* a_ready_epoch, long long max_cycles, const AtlasEpilogue* epi = nullptr) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const uint32_t esize = kind == 1 ? 1 : 2;
  const int elems_per_row = 128 / esize;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
  if ((lda * esize) % 16 || (ldb * esize) % 16) return -2;
  if (kind == 1 && (K % 128)) return -3;
  if (block_n != 64 && block_n != 128 && block_n != 256) return -4;
  const int epi_mode = epi ? epi->mode : 0;
  if (epi_mode < 0 || epi_mode > 2) return -40;
  if (epi_mode != 0) {
    // fused epilogues exist for the FP8 kernels whose epilogue threads hold 64 columns of a row
    if (kind != 1 || !epi->q_out || !epi->s_out || (epi->ldq % 16) || (reinterpret_cast<uintptr_t>(epi->q_out) & 15)) return -41;
    if (block_n == 256 && wide_fp8_epilogue_warps() != 16) return -42;
    if (epi_mode == 1 && (block_n != 256 || (N % 256) || ((N / 2) % 128))) return -43;
    if (epi_mode == 2 && ((block_n != 128 && block_n != 256) || (N % block_n) || !epi->residual || !epi->norm_w || !epi->ss_out ||
                          (epi->ldr % 8) || (reinterpret_cast<uintptr_t>(epi->residual) & 15) ||
                          (reinterpret_cast<uintptr_t>(epi->norm_w) & 15)))
      return -44;
  }
  CUtensorMap ta, tb;
  const int a_box = a_box_for(M);
  int rc = make_tmap_kmajor(&ta, A, M, K, lda, a_box, esize);
  if (rc) return rc;
  rc = make_tmap_kmajor(&tb, B, N, K, ldb, epi_mode == 1 ? 32 : block_n, esize);
  if (rc) return rc;
  GemmParams p = {};
  p.timeline = g_gemm_timeline;
  p.a_box_rows = a_box;
  p.C = C; p.a_scale = a_scale; p.b_scale = b_scale; p.workspace = workspace; p.counters = counters;
  p.status = status; p.ldc = ldc; p.sa_k = sa_k; p.M = M; p.N = N; p.K = K;
  p.epi_mode = epi_mode;
  if (epi) {
    p.act_cols = N / 2; p.q_out = reinterpret_cast<uint8_t*>(epi->q_out); p.ldq = epi->ldq; p.s_out = epi->s_out; p.s_ld = epi->s_ld;
    p.residual = reinterpret_cast<__nv_bfloat16*>(epi->residual); p.ldr = epi->ldr;
    p.norm_w = reinterpret_cast<const __nv_bfloat16*>(epi->norm_w); p.norm_plus_one = epi->norm_plus_one;
    p.ss_out = epi->ss_out; p.ss_out_ld = epi->ss_out_ld;
    p.ss_in = epi->ss_in; p.ss_in_parts = epi->ss_in_parts; p.ss_in_ld = epi->ss_in_ld; p.ss_inv_h = epi->ss_inv_h; p.ss_eps = epi->ss_eps;
  }
  p.tile_expert = nullptr; p.num_m_tiles_ptr = nullptr; p.expert_n = 0; p.b_scale_expert_stride = 0;
  p.ar_state = nullptr; p.ar_world = 1; p.ar_rank = 0; p.ar_mode = 0; p.ar_parity_stride = 0; p.prefetch_b = 0;
  p.rs_tiles_per_rank = 1; p.a_ready = a_ready; p.a_ready_epoch = a_ready_epoch;
  p.ar_max_cycles = max_cycles > 0 ? max_cycles : kMbarMaxCycles;
  p.k_blocks = (K + elems_per_row - 1) / elems_per_row;
  if (splits < 1) splits = 1;
  if (splits > p.k_blocks) splits = p.k_blocks;
  p.kb_per_split = (p.k_blocks + splits - 1) / splits;
  p.splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  if (p.splits > 1 && (!workspace || !counters)) return -5;
  p.m_tiles = (M + kBlockM - 1) / kBlockM;
  p.n_tiles = epi_mode == 1 ? (N / 2) / (block_n / 2) : (N + block_n - 1) / block_n;
  if (kind == 1) {
    if (sa_m != 1 || (sa_k % 4) || sa_k < (long long)p.m_tiles * kBlockM) return -6;
    if ((reinterpret_cast<uintptr_t>(a_scale) & 15)) return -7;
    if (p.kb_per_split > 512) return -8;
  }
  p.b_scale_ld = b_scale_ld;
  p.vec_ok = ((ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
  const long long items = (long long)p.m_tiles * p.n_tiles * p.splits;
  int grid = (int)(items < num_sms ? items : num_sms);
  // One m-tile, 128-wide tiles, 2 or 4 splits and a CTA for every (tile, split): the splits of a tile run as a cluster
  // and meet in distributed shared memory (cluster_tail) instead of in the global workspace.
  p.cluster_splits = 1;
  if (cluster_splitk_enabled() && p.m_tiles == 1 && block_n == 128 && (p.splits == 2 || p.splits == 4) && items <= num_sms &&
      (epi_mode == 2 || (epi_mode == 0 && p.vec_ok)) && (N % 128) == 0 && a_ready == nullptr)
    p.cluster_splits = p.splits;
  p.prefetch_b = p.m_tiles <= 2 ? prefetch_depth() : 0;      // weights read once from HBM: run ahead of the ring in L2
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (kind == 1) {
    if (block_n == 64) return launch_gemm<64, true>(ta, tb, p, grid, st);
    if (block_n == 128) return launch_gemm<128, true>(ta, tb, p, grid, st);
    if (wide_fp8_epilogue_warps() == 8) return launch_gemm<256, true, false, 8>(ta, tb, p, grid, st);
    return launch_gemm<256, true>(ta, tb, p, grid, st);
  }
  if (block_n == 64) return launch_gemm<64, false>(ta, tb, p, grid, st);
  if (block_n == 128) return launch_gemm<128, false>(ta, tb, p, grid, st);
  return launch_gemm<256, false>(ta, tb, p, grid, st);
}

extern "C" int atlas_gemm(int kind, const void* A, const void* B, void* C, const float* a_scale, long long sa_m,
                          long long sa_k, const float* b_scale, int b_scale_ld, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, int block_n, int splits, float* workspace, int* counters,
                          int num_sms, unsigned long long* status, void* stream) {
  return gemm_impl(kind, A, B, C, a_scale, sa_m, sa_k, b_scale, b_scale_ld, M, N, K, lda, ldb, ldc, block_n, splits, workspace,
                   counters, num_sms, status, stream, nullptr, nullptr, 0);
}

// All-gather -> GEMM: the rows of A (and their scales) are written into this rank's memory by the ranks that own them;
// `a_ready` holds one flag per 8 rows and a row group is complete once its flag has reached *a_ready_epoch.  The TMA
// producer polls the flags of a tile's rows before it loads the tile, so the GEMM starts on the rows that are already
// there and the gather overlaps the math.  Everything else is atlas_gemm.
extern "C" int atlas_gemm_gathered(int kind, const void* A, const void* B, void* C, const float* a_scale, long long sa_m,
                                   long long sa_k, const float* b_scale, int b_scale_ld, int M, int N, int K, long long lda,
                                   long long ldb, long long ldc, int block_n, int splits, float* workspace, int* counters,
                                   int num_sms, unsigned long long* status, void* stream, const void* a_ready,
                                   const unsigned int* a_ready_epoch, long long max_cycles) {
  if (!a_ready || !a_ready_epoch) return -30;
  return gemm_impl(kind, A, B, C, a_scale, sa_m, sa_k, b_scale, b_scale_ld, M, N, K, lda, ldb, ldc, block_n, splits, workspace,
                   counters, num_sms, status, stream, reinterpret_cast<const uint32_t*>(a_ready), a_ready_epoch, max_cycles);
}

// atlas_gemm with a fused epilogue and / or a deferred RMSNorm factor on the A operand (see AtlasEpilogue in host_api.h
// and the epi_mode notes in GemmParams).  `C` is unused when epi->mode != 0.
extern "C" int atlas_gemm_fused(int kind, const void* A, const void* B, void* C, const float* a_scale, long long sa_m,
                                long long sa_k, const float* b_scale, int b_scale_ld, int M, int N, int K, long long lda,
                                long long ldb, long long ldc, int block_n, int splits, float* workspace, int* counters,
                                int num_sms, unsigned long long* status, void* stream, const AtlasEpilogue* epi,
                                const void* a_ready, const unsigned int* a_ready_epoch, long long max_cycles) {
  if (!epi) return -40;
  return gemm_impl(kind, A, B, C, a_scale, sa_m, sa_k, b_scale, b_scale_ld, M, N, K, lda, ldb, ldc, block_n, splits, workspace,
                   counters, num_sms, status, stream, reinterpret_cast<const uint32_t*>(a_ready), a_ready_epoch, max_cycles, epi);
}

// Grouped (MoE) GEMM: C[r, :] = A[r, :] * B[e(r)]^T for expert-sorted rows.  `A` has `max_rows` rows (a multiple of
// 128); m-tile i covers rows [128 i, 128 i + 128) and uses expert tile_expert[i]; *num_m_tiles (device memory) says how
// many tiles are live.  `B` is the expert stack [E * N, K]; b_scale is [E, ceil(N/128), K/128].
extern "C" int atlas_gemm_grouped(int kind, const void* A, const void* B, void* C, const float* a_scale, long long sa_k,
                                  const float* b_scale, int max_rows, int N, int K, int E, long long lda, long long ldb,
                                  long long ldc, int block_n, const int* tile_expert, const int* num_m_tiles,
                                  int num_sms, unsigned long long* status, void* stream) {
  if (max_rows <= 0 || N <= 0 || K <= 0 || E <= 0) return 0;
  if (max_rows % kBlockM) return -9;
  const uint32_t esize = kind == 1 ? 1 : 2;
  const int elems_per_row = 128 / esize;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
  if ((lda * esize) % 16 || (ldb * esize) % 16) return -2;
  if (kind == 1 && (K % 128)) return -3;
  if (block_n != 64 && block_n != 128 && block_n != 256) return -4;
  if (N % block_n) return -10;            // a tile must not straddle two experts' rows of B
  CUtensorMap ta, tb;
  int rc = make_tmap_kmajor(&ta, A, max_rows, K, lda, kBlockM, esize);
  if (rc) return rc;
  rc = make_tmap_kmajor(&tb, B, (uint64_t)E * N, K, ldb, block_n, esize);
  if (rc) return rc;
  GemmParams p = {};
  p.timeline = g_gemm_timeline;
  p.a_box_rows = kBlockM;
  p.C = C; p.a_scale = a_scale; p.b_scale = b_scale; p.workspace = nullptr; p.counters = nullptr;
  p.status = status; p.ldc = ldc; p.sa_k = sa_k; p.M = max_rows; p.N = N; p.K = K;
  p.k_blocks = (K + elems_per_row - 1) / elems_per_row;
  p.splits = 1; p.kb_per_split = p.k_blocks;
  p.m_tiles = max_rows / kBlockM;
  p.n_tiles = N / block_n;
  p.b_scale_ld = p.k_blocks;
  p.vec_ok = ((ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
  p.tile_expert = tile_expert; p.num_m_tiles_ptr = num_m_tiles; p.expert_n = N;
  p.ar_state = nullptr; p.ar_world = 1; p.ar_rank = 0; p.ar_mode = 0; p.ar_parity_stride = 0; p.prefetch_b = 0;
  p.rs_tiles_per_rank = 1; p.a_ready = nullptr; p.a_ready_epoch = nullptr; p.ar_max_cycles = kMbarMaxCycles;
  p.b_scale_expert_stride = (long long)((N + 127) / 128) * p.k_blocks;
  if (kind == 1) {
    if ((sa_k % 4) || sa_k < max_rows || (reinterpret_cast<uintptr_t>(a_scale) & 15)) return -6;
    if (p.kb_per_split > 512) return -8;
  }
  const long long items = (long long)p.m_tiles * p.n_tiles;
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

// Row-parallel GEMM fused with its all-reduce.  Every rank calls this with its K-shard of A and B.
//   mode 0 (two-shot): tile t is reduced by rank t % world and the sum is pushed to everyone; the [M, N] bf16 result
//     appears at `*result_off_out` inside every rank's fused area (row-major, ld = N).  Uses the upper half of the area:
//     [world partial regions of part_src_stride bytes][result]; flags [max_tiles][8] partial + [max_tiles] final.
//   mode 1 (one-shot): every rank pushes each partial tile to all peers and sums all partials itself into `C` (a plain
//     local tensor).  One flag exchange instead of two; (world - 1) x the NVLink bytes, so meant for small outputs.
//     Uses the lower half of the area, split into two epoch-parity quarters of [world][tiles] tiles; flags
//     [max_tiles][8] at word offset 9 * max_tiles.  K may be split (`splits`, `workspace`, `counters` as in atlas_gemm).
// The grid is the same on every rank by construction.
extern "C" int atlas_gemm_allreduce(int kind, const void* A, const void* B, const float* a_scale, long long sa_k,
                                    const float* b_scale, int b_scale_ld, int M, int N, int K, long long lda,
                                    long long ldb, int block_n, void* const* data, void* const* flags, int rank,
                                    int world, unsigned int* state, size_t area_bytes, int max_tiles, size_t* result_off_out,
                                    int num_sms, long long max_cycles, unsigned long long* status, void* stream, int mode,
                                    void* C, long long ldc, int splits, float* workspace, int* counters,
                                    const AtlasEpilogue* epi) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const uint32_t esize = kind == 1 ? 1 : 2;
  const int elems_per_row = 128 / esize;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
  if ((lda * esize) % 16 || (ldb * esize) % 16) return -2;
  if (kind == 1 && (K % 128)) return -3;
  if (block_n != 64 && block_n != 128) return -4;
  if (N % 8 || world < 1 || world > 8) return -5;
  if (mode != 0 && mode != 1) return -13;
  // The one-shot form ends with the full sum in the epilogue threads' registers, so the residual + norm + FP8 epilogue
  // (mode 2 of AtlasEpilogue) applies to it unchanged: every rank updates its own copy of the residual stream and writes
  // its own quantised activations (identical bits everywhere, the partials are added in rank order).
  const int epi_mode = epi ? epi->mode : 0;
  if (epi_mode != 0) {
    if (epi_mode != 2 || mode != 1 || kind != 1 || block_n != 128 || (N % 128)) return -44;
    if (!epi->q_out || !epi->s_out || !epi->residual || !epi->norm_w || !epi->ss_out || (epi->ldq % 16) || (epi->ldr % 8) ||
        ((reinterpret_cast<uintptr_t>(epi->q_out) | reinterpret_cast<uintptr_t>(epi->residual) |
          reinterpret_cast<uintptr_t>(epi->norm_w)) & 15) || epi->ss_in)
      return -44;
  }
  CUtensorMap ta, tb;
  const int a_box = a_box_for(M);
  int rc = make_tmap_kmajor(&ta, A, M, K, lda, a_box, esize);
  if (rc) return rc;
  rc = make_tmap_kmajor(&tb, B, N, K, ldb, block_n, esize);
  if (rc) return rc;
  GemmParams p = {};
  p.timeline = g_gemm_timeline;
  p.a_box_rows = a_box;
  p.C = nullptr; p.a_scale = a_scale; p.b_scale = b_scale; p.workspace = nullptr; p.counters = nullptr;
  p.status = status; p.ldc = N; p.sa_k = sa_k; p.M = M; p.N = N; p.K = K;
  p.epi_mode = epi_mode;
  if (epi_mode == 2) {
    p.q_out = reinterpret_cast<uint8_t*>(epi->q_out); p.ldq = epi->ldq; p.s_out = epi->s_out; p.s_ld = epi->s_ld;
    p.residual = reinterpret_cast<__nv_bfloat16*>(epi->residual); p.ldr = epi->ldr;
    p.norm_w = reinterpret_cast<const __nv_bfloat16*>(epi->norm_w); p.norm_plus_one = epi->norm_plus_one;
    p.ss_out = epi->ss_out; p.ss_out_ld = epi->ss_out_ld;
  }
  p.k_blocks = (K + elems_per_row - 1) / elems_per_row;
  p.splits = 1; p.kb_per_split = p.k_blocks;
  if (mode == 1) {
    if (!C && epi_mode == 0) return -14;
    if (splits < 1) splits = 1;
    if (splits > p.k_blocks) splits = p.k_blocks;
    p.kb_per_split = (p.k_blocks + splits - 1) / splits;
    p.splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;
    if (p.splits > 1 && (!workspace || !counters)) return -5;
    p.C = C; p.ldc = ldc; p.workspace = workspace; p.counters = counters;
  }
  p.m_tiles = (M + kBlockM - 1) / kBlockM;
  p.n_tiles = (N + block_n - 1) / block_n;
  p.b_scale_ld = b_scale_ld;
  p.vec_ok = mode == 1 ? (((ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0) : 1;
  p.tile_expert = nullptr; p.num_m_tiles_ptr = nullptr; p.expert_n = 0; p.b_scale_expert_stride = 0;
  p.rs_tiles_per_rank = 1; p.a_ready = nullptr; p.a_ready_epoch = nullptr;
  if (kind == 1) {
    if ((sa_k % 4) || sa_k < (long long)p.m_tiles * kBlockM || (reinterpret_cast<uintptr_t>(a_scale) & 15)) return -6;
    if (p.kb_per_split > 512) return -8;
  }
  const int tiles = p.m_tiles * p.n_tiles;
  if (tiles > max_tiles) return -11;
  const size_t tile_bytes = (size_t)kBlockM * block_n * 2;
  const size_t half_area = (area_bytes / 2) & ~(size_t)255;
  size_t base_off = 0;
  p.ar_mode = mode;
  p.ar_parity_stride = 0;
  p.ar_part_src_stride = 0;
  p.ar_result_off = 0;
  if (mode == 0) {
    base_off = half_area;
    p.ar_part_src_stride = (size_t)((tiles + world - 1) / world) * tile_bytes;
    p.ar_result_off = ((size_t)world * p.ar_part_src_stride + 255) & ~(size_t)255;
    if (p.ar_result_off + (size_t)M * N * 2 > half_area) return -12;
    if (result_off_out) *result_off_out = base_off + p.ar_result_off;
  } else {
    p.ar_parity_stride = (half_area / 2) & ~(size_t)255;
    if ((size_t)world * tiles * tile_bytes > p.ar_parity_stride) return -12;
    if (result_off_out) *result_off_out = 0;
  }
  for (int i = 0; i < 8; ++i) {
    p.ar_data[i] = i < world ? reinterpret_cast<uint8_t*>(data[i]) + base_off : nullptr;
    p.ar_flags[i] = i < world ? reinterpret_cast<uint32_t*>(flags[i]) : nullptr;
  }
  p.ar_state = state; p.ar_rank = rank; p.ar_world = world; p.ar_max_tiles = max_tiles;
  p.ar_max_cycles = max_cycles > 0 ? max_cycles : 2000ll * 1000ll * 1000ll;
  const long long items = (long long)tiles * p.splits;
  int grid = (int)(items < num_sms ? items : num_sms);
  p.prefetch_b = p.m_tiles <= 2 ? prefetch_depth() : 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (kind == 1) {
    if (block_n == 64) return launch_gemm<64, true, true>(ta, tb, p, grid, st);
    return launch_gemm<128, true, true>(ta, tb, p, grid, st);
  }
  if (block_n == 64) return launch_gemm<64, false, true>(ta, tb, p, grid, st);
  return launch_gemm<128, false, true>(ta, tb, p, grid, st);
}

// Row-parallel GEMM fused with the reduce-scatter of its output (sequence-parallel tensor parallelism).  Rank r owns the
// row blocks (m-tiles of 128 rows) [r * tiles_per_rank, (r + 1) * tiles_per_rank).  Every rank computes its K-shard's
// partial of the whole [M, N] output; the epilogue stores each bf16 partial tile into the OWNER's area with peer stores,
//   data[owner] + rank * part_src_stride + ((m_tile - owner * tiles_per_rank) * 128 + row) * N * 2,
// and raises flags[owner][((m_tile - owner * tiles_per_rank) * n_tiles + n_tile) * 8 + rank] to the call's epoch
// (state[0] + 1; state[0] holds that epoch once the kernel has finished).  Nothing is reduced here and nothing comes
// back: atlas_sp_reduce_norm_gather on the owner sums the partials.  `flag_words` is the capacity of a flag area.
extern "C" int atlas_gemm_reduce_scatter(int kind, const void* A, const void* B, const float* a_scale, long long sa_k,
                                         const float* b_scale, int b_scale_ld, int M, int N, int K, long long lda,
                                         long long ldb, int block_n, void* const* data, void* const* flags, int rank,
                                         int world, unsigned int* state, size_t part_src_stride, int tiles_per_rank,
                                         size_t flag_words, int num_sms, long long max_cycles, unsigned long long* status,
                                         void* stream, int* n_tiles_out, int rows_per_rank) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const uint32_t esize = kind == 1 ? 1 : 2;
  const int elems_per_row = 128 / esize;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
  if ((lda * esize) % 16 || (ldb * esize) % 16) return -2;
  if (kind == 1 && (K % 128)) return -3;
  if (block_n != 64 && block_n != 128 && block_n != 256) return -4;
  if (block_n == 256 && (kind != 1 || wide_fp8_epilogue_warps() != 16)) return -4;    // the wide tile exists for FP8 only
  if (N % 8 || world < 1 || world > 8 || tiles_per_rank < 1) return -5;
  CUtensorMap ta, tb;
  const int a_box = kBlockM;
  int rc = make_tmap_kmajor(&ta, A, M, K, lda, a_box, esize);
  if (rc) return rc;
  rc = make_tmap_kmajor(&tb, B, N, K, ldb, block_n, esize);
  if (rc) return rc;
  GemmParams p = {};
  p.timeline = g_gemm_timeline;
  p.a_box_rows = a_box;
  p.C = nullptr; p.a_scale = a_scale; p.b_scale = b_scale; p.workspace = nullptr; p.counters = nullptr;
  p.status = status; p.ldc = N; p.sa_k = sa_k; p.M = M; p.N = N; p.K = K;
  p.k_blocks = (K + elems_per_row - 1) / elems_per_row;
  p.splits = 1; p.kb_per_split = p.k_blocks;
  p.m_tiles = (M + kBlockM - 1) / kBlockM;
  p.n_tiles = (N + block_n - 1) / block_n;
  if (n_tiles_out) *n_tiles_out = p.n_tiles;
  p.b_scale_ld = b_scale_ld; p.vec_ok = 1;
  p.tile_expert = nullptr; p.num_m_tiles_ptr = nullptr; p.expert_n = 0; p.b_scale_expert_stride = 0;
  p.a_ready = nullptr; p.a_ready_epoch = nullptr;
  if (kind == 1) {
    if ((sa_k % 4) || sa_k < (long long)p.m_tiles * kBlockM || (reinterpret_cast<uintptr_t>(a_scale) & 15)) return -6;
    if (p.kb_per_split > 512) return -8;
  }
  if ((long long)tiles_per_rank * world < p.m_tiles) return -11;                        // every row block needs an owner
  if ((size_t)tiles_per_rank * p.n_tiles * 8 > flag_words) return -12;
  if ((size_t)tiles_per_rank * kBlockM * N * 2 > part_src_stride) return -12;
  p.ar_mode = 2; p.rs_tiles_per_rank = tiles_per_rank;
  // row-level ownership: one m-tile, groups of rows_per_rank rows (a multiple of 8) owned rank by rank
  if (rows_per_rank > 0 && (rows_per_rank % 8 || M > kBlockM || tiles_per_rank != 1 || (long long)rows_per_rank * world < M)) return -15;
  p.rs_rows_per_rank = rows_per_rank > 0 ? rows_per_rank : 0;
  p.ar_parity_stride = 0; p.ar_part_src_stride = part_src_stride; p.ar_result_off = 0;
  for (int i = 0; i < 8; ++i) {
    p.ar_data[i] = i < world ? reinterpret_cast<uint8_t*>(data[i]) : nullptr;
    p.ar_flags[i] = i < world ? reinterpret_cast<uint32_t*>(flags[i]) : nullptr;
  }
  p.ar_state = state; p.ar_rank = rank; p.ar_world = world; p.ar_max_tiles = 0;
  p.ar_max_cycles = max_cycles > 0 ? max_cycles : kMbarMaxCycles;
  const long long items = (long long)p.m_tiles * p.n_tiles;
  int grid = (int)(items < num_sms ? items : num_sms);
  p.prefetch_b = 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (kind == 1) {
    if (block_n == 64) return launch_gemm<64, true, true>(ta, tb, p, grid, st);
    if (block_n == 256) return launch_gemm<256, true, true, 16>(ta, tb, p, grid, st);
    return launch_gemm<128, true, true>(ta, tb, p, grid, st);
  }
  if (block_n == 64) return launch_gemm<64, false, true>(ta, tb, p, grid, st);
  return launch_gemm<128, false, true>(ta, tb, p, grid, st);
}
