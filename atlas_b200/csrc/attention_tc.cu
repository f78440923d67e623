// Prefill (chunk) attention over the paged FP8 KV cache on the 5th-generation tensor cores (head_dim 128, 16-token
// pages).  One CTA per (128-row query tile, kv head); the G = Hq/Hkv query heads that share the kv head are packed into
// the tile's rows (row = token * G + head), so every K/V page is fetched and widened once for all of them.
//
//   warp 0       producer: TMA load of the Q tile (3-D box: 64 dims x G heads x 128/G tokens, 128-byte swizzle) and
//                bulk copies of the K / V pages of each 128-token KV tile into a three-stage staging ring; sixteen
//                lanes issue one page copy each, block-table entries are fetched one tile ahead
//   warp 1       tcgen05.mma issuer (kind::f16): S_j = Q K_j^T into one of two TMEM buffers, O += P_j V_j into a third
//   warps 2..5   converters: FP8 pages -> f16 operand tiles in the 128-byte-swizzled K-major layout the MMA reads
//                (K: rows = tokens, V: rows = head dims; V pages are stored transposed in the cache, so both are
//                16-byte-in, two-chunks-out moves)
//   warps 6..13  softmax: two threads per query row, 64 score columns each (warps w and w + 4 share the TMEM lanes of a
//                row group).  A thread pulls its half row out of TMEM at once, the two halves agree on the row max
//                through a spare TMEM column and an mbarrier per row group, P goes to shared memory as the A operand of
//                the PV product, and O is rescaled in TMEM lazily (only when a row's max has grown by more than 2^8
//                since its reference point was set), each thread its own 64 columns
//
// Q is converted to f16 once (softmax scale, K scale and log2(e) folded in), so S is already in the exp2 domain; the V
// scale is applied with the final 1/l.  QK_{j+1} is issued before PV_j, so the tensor cores work on the next score tile
// while the softmax warps handle the current one.  Every wait is bounded (status word + early exit).
//
// Reference ops replaced: inferspark_prefill_paged_fp8.cu / prefill_paged_compute.cuh (mma.sync FA2, QK^T in bf16 and
// P.V in fp16) and the FlashInfer ragged-prefill wrapper.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "host_api.h"

namespace atlas {

constexpr int kTcD = 128;                 // head dim
constexpr int kTcRows = 128;              // query rows per tile (tokens * G)
constexpr int kTcKv = 128;                // kv tokens per tile
constexpr int kTcPage = 16;
constexpr int kTcPages = kTcKv / kTcPage;
constexpr int kTcThreads = 448;
constexpr int kSub = 16 * 1024;           // one 128-row x 64-element f16 sub-tile
constexpr int kPageBytes = kTcPage * kTcD;        // 2 KB (fp8)
constexpr int kStageBytes = 2 * kTcPages * kPageBytes;   // K pages then V pages: 32 KB
constexpr int kTcStages = 3;

struct TcAttnParams {
  __nv_bfloat16* out; long long ldo;
  // q_out != nullptr: write the rows as FP8 with one scale per (row, head) -- a head is one 128-wide quantisation group of
  // the output projection's A operand -- instead of bf16 `out`; scale of (row, head) at s_out[head * s_ld + row]
  uint8_t* q_out; long long ldqo;
  float* s_out; long long s_ld;
  const uint8_t* k_cache; const uint8_t* v_cache;
  const int* block_tables; int bt_ld;
  const int* seq_lens; const int* query_start_loc;
  const int* tile_seq; const int* tile_q0;
  float qk_scale_log2, v_scale;
  int Hq, Hkv, G;
  int total_tokens;
  status_t* status;
};

ATLAS_DEVICE void bulk_copy_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
ATLAS_DEVICE void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
ATLAS_DEVICE void tmem_st_32x32b_x1(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};\n" ::"r"(taddr), "r"(v) : "memory");
}
ATLAS_DEVICE void tmem_ld_32x32b_x1(uint32_t taddr, uint32_t& v) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];\n" : "=r"(v) : "r"(taddr) : "memory");
}
ATLAS_DEVICE void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
ATLAS_DEVICE uint32_t fp8x2_to_h2(uint32_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(r) : "h"((uint16_t)v));
  return r;
}
ATLAS_DEVICE float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
ATLAS_DEVICE uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// 16 fp8 bytes -> 16 f16 in two 16-byte chunks
ATLAS_DEVICE void widen16(const uint4 v, uint4& lo, uint4& hi) {
  lo.x = fp8x2_to_h2(v.x); lo.y = fp8x2_to_h2(v.x >> 16); lo.z = fp8x2_to_h2(v.y); lo.w = fp8x2_to_h2(v.y >> 16);
  hi.x = fp8x2_to_h2(v.z); hi.y = fp8x2_to_h2(v.z >> 16); hi.z = fp8x2_to_h2(v.w); hi.w = fp8x2_to_h2(v.w >> 16);
}

// 14 warps are accounted as 16 (warps are allocated four at a time), so 128 registers per thread is the ceiling
__global__ void __launch_bounds__(kTcThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                       // 2 sub-tiles: [128 rows][64 dims]
  uint8_t* sK = smem + 2 * kSub;            // 2 sub-tiles: [128 tokens][64 dims]
  uint8_t* sV = smem + 4 * kSub;            // 2 sub-tiles: [128 dims][64 tokens]
  uint8_t* sP = smem + 6 * kSub;            // 2 sub-tiles: [128 rows][64 tokens]
  uint8_t* sStage = smem + 8 * kSub;        // kTcStages x (8 K pages + 8 V pages)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStage + kTcStages * kStageBytes);
  uint64_t* q_full = bars;                  // 1
  uint64_t* stg_full = bars + 1;            // [kTcStages] tx
  uint64_t* stg_empty = bars + 1 + kTcStages;   // [kTcStages] 4 converter warps
  uint64_t* k_ready = bars + 1 + 2 * kTcStages; // 4 converter warps
  uint64_t* k_free = k_ready + 1;           // commit after QK
  uint64_t* v_ready = k_ready + 2;          // 4 converter warps
  uint64_t* pv_done = k_ready + 3;          // commit after PV: V tile, P tile and O are free / stable
  uint64_t* s_full = k_ready + 4;           // [2] commit after QK
  uint64_t* s_free = k_ready + 6;           // [2] 8 softmax warps
  uint64_t* p_ready = k_ready + 8;          // 8 softmax warps
  uint64_t* q_conv = k_ready + 9;           // 12 warps (converters + softmax) finished the in-place Q conversion
  uint64_t* x_ready = k_ready + 10;         // [2 parities][4 row groups] the two softmax warps of a row group exchanged a value
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(k_ready + 18);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.G;
  const int tok_per_tile = kTcRows / G;
  const int b = p.tile_seq[blockIdx.x];
  const int q0 = p.tile_q0[blockIdx.x];
  const int kvh = blockIdx.y;
  const int L = p.seq_lens[b];
  const int q_row0 = p.query_start_loc[b];
  const int q_len = p.query_start_loc[b + 1] - q_row0;
  const int ctx0 = L - q_len;                                   // absolute position of the chunk's first query
  const int last_tok = min(q0 + tok_per_tile, q_len) - 1;       // last live query token of the tile (chunk-relative)
  const int kv_hi = min(L, ctx0 + last_tok + 1);                // causal bound: keys [0, kv_hi)
  const int n_kv = (kv_hi + kTcKv - 1) / kTcKv;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kTcStages; ++s) { mbar_init(&stg_full[s], 1); mbar_init(&stg_empty[s], 4); }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_free[s], 8); }
    mbar_init(k_ready, 4); mbar_init(k_free, 1); mbar_init(v_ready, 4); mbar_init(pv_done, 1); mbar_init(p_ready, 8);
    mbar_init(q_conv, 12);
    for (int s = 0; s < 8; ++s) mbar_init(&x_ready[s], 2);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  if (warp == 0 && lane == 0) tma_prefetch_desc(&tmap_q);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;            // two score buffers: columns [0,128) and [128,256)
  const uint32_t tO = tmem_base + 256;      // output accumulator: columns [256,384)
  const uint32_t tX = tmem_base + 384;      // four columns through which the two threads of a row exchange a value

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp)
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * kSub);
      tma_load_3d(sQ, &tmap_q, q_full, 0, kvh * G, q_row0 + q0);
      tma_load_3d(sQ + kSub, &tmap_q, q_full, 64, kvh * G, q_row0 + q0);
    }
    const int* bt = p.block_tables + (long long)b * p.bt_ld;
    const int n_pages = (L + kTcPage - 1) / kTcPage;
    const int pi = lane & 7;                          // lanes 0..7 copy K pages, 8..15 V pages
    int blk_next = (lane < 16 && pi < n_pages) ? bt[pi] : 0;
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int blk = blk_next;
      const int pg_next = (j + 1) * kTcPages + pi;
      if (lane < 16 && j + 1 < n_kv && pg_next < n_pages) blk_next = bt[pg_next];     // one tile ahead of its use
      const int live = min(kTcPages, n_pages - j * kTcPages);
      if (lane == 0) {
        ok = mbar_wait(&stg_empty[stage], phase ^ 1u, abort_flag, p.status, 0x800);
        if (ok) mbar_expect_tx(&stg_full[stage], (uint32_t)live * 2u * kPageBytes);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane < 16 && pi < live) {
        const long long page = (long long)blk * p.Hkv + kvh;
        uint8_t* dst = sStage + stage * kStageBytes + ((lane < 8 ? 0 : kTcPages) + pi) * kPageBytes;
        bulk_copy_g2s(dst, (lane < 8 ? p.k_cache : p.v_cache) + page * kPageBytes, kPageBytes, &stg_full[stage]);
      }
      if (++stage == kTcStages) { stage = 0; phase ^= 1u; }
    }
    if (!ok)
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t kIdesc = make_idesc(kTcRows, 128, 0u);       // f16 x f16 -> f32, M = 128, N = 128
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 0x810) && mbar_wait(q_conv, 0, abort_flag, p.status, 0x811);
      auto issue_pv = [&](int i) -> bool {
        if (!mbar_wait(p_ready, i & 1, abort_flag, p.status, 0x812)) return false;
        if (!mbar_wait(v_ready, i & 1, abort_flag, p.status, 0x813)) return false;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t ad = make_smem_desc_sw128(aP + (ks >> 2) * kSub) + 2 * (ks & 3);
          const uint64_t bd = make_smem_desc_sw128(aV + (ks >> 2) * kSub) + 2 * (ks & 3);
          umma_f16(tO, ad, bd, kIdesc, (i > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(pv_done);
        return true;
      };
      for (int j = 0; j < n_kv && ok; ++j) {
        const int sb = j & 1;
        if (!mbar_wait(k_ready, j & 1, abort_flag, p.status, 0x814)) { ok = false; break; }
        if (!mbar_wait(&s_free[sb], ((j >> 1) & 1) ^ 1u, abort_flag, p.status, 0x815)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t ad = make_smem_desc_sw128(aQ + (ks >> 2) * kSub) + 2 * (ks & 3);
          const uint64_t bd = make_smem_desc_sw128(aK + (ks >> 2) * kSub) + 2 * (ks & 3);
          umma_f16(tS + sb * 128, ad, bd, kIdesc, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        umma_commit(k_free);
        if (j > 0) ok = issue_pv(j - 1);
      }
      if (ok && n_kv > 0) issue_pv(n_kv - 1);
    }
  } else {
    // ------------------------------------------------------------------ converters (warps 2..5) and softmax (6..13)
    const bool is_conv = warp < 6;
    const int t128 = threadIdx.x - 64;                            // converters: 0..127
    bool ok = true;
    // Q: bf16 -> f16 in place (element-wise, so the swizzled layout is untouched), scaled into the exp2 domain
    if (!mbar_wait(q_full, 0, abort_flag, p.status, 0x820)) ok = false;
    if (ok) {
      const int t384 = threadIdx.x - 64;                          // 0..383 over both roles
      uint4* q4 = reinterpret_cast<uint4*>(sQ);
      for (int i = t384; i < 2 * kSub / 16; i += 384) {
        uint4 v = q4[i];
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[e]));
          w[e] = pack_h2(f.x * p.qk_scale_log2, f.y * p.qk_scale_log2);
        }
        q4[i] = v;
      }
      fence_proxy_async();
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(q_conv);

    if (is_conv) {
      const int r = t128;                    // K: token row of the tile; V: head-dim row
      const int sw = r & 7;
      // K_{j+1} is converted before V_j: the next score tile can then be issued while the softmax warps are still
      // working on the current one (V_j has to wait for the previous PV product anyway).
      auto conv_k = [&](int j) -> bool {
        const int s = j % kTcStages;
        if (!mbar_wait(&stg_full[s], (j / kTcStages) & 1, abort_flag, p.status, 0x821)) return false;
        if (j > 0 && !mbar_wait(k_free, (j - 1) & 1, abort_flag, p.status, 0x822)) return false;
        const int kv0 = j * kTcKv;
        // consecutive threads take consecutive 16-byte pieces of the staged pages (no bank conflicts on the read):
        // piece i = row (token) i / 8, dims (i % 8) * 16 .. + 15
        const uint4* src = reinterpret_cast<const uint4*>(sStage + s * kStageBytes);
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {
          const int i = k8 * 128 + r;
          const int trow = i >> 3, c = i & 7, tsw = trow & 7;
          uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
          if (kv0 + trow < L) widen16(src[i], lo, hi);
          uint8_t* rowp = sK + (c >> 2) * kSub + (trow >> 3) * 1024 + tsw * 128;
          const int ch = (c & 3) * 2;
          *reinterpret_cast<uint4*>(rowp + ((ch ^ tsw) << 4)) = lo;
          *reinterpret_cast<uint4*>(rowp + (((ch + 1) ^ tsw) << 4)) = hi;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(k_ready);
        return true;
      };
      auto conv_v = [&](int j) -> bool {
        const int s = j % kTcStages;
        const int kv0 = j * kTcKv;
        const uint8_t* stg = sStage + s * kStageBytes;
        // row r = head dim r, page pg holds tokens kv0 + 16 pg .. + 15 as 16 contiguous bytes
        if (j > 0 && !mbar_wait(pv_done, (j - 1) & 1, abort_flag, p.status, 0x823)) return false;
        uint8_t* row0 = sV + (r >> 3) * 1024 + sw * 128;
#pragma unroll
        for (int pg = 0; pg < kTcPages; ++pg) {
          const int t0 = kv0 + pg * kTcPage;
          uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
          if (t0 < L) {
            uint4 v = *reinterpret_cast<const uint4*>(stg + (kTcPages + pg) * kPageBytes + r * kTcPage);
            if (t0 + kTcPage > L) {                 // the sequence ends inside this page: clear the tail bytes
              uint8_t* bytes = reinterpret_cast<uint8_t*>(&v);
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (t0 + i >= L) bytes[i] = 0;
            }
            widen16(v, lo, hi);
          }
          uint8_t* rowp = row0 + (pg >> 2) * kSub;
          const int ch = (pg & 3) * 2;
          *reinterpret_cast<uint4*>(rowp + ((ch ^ sw) << 4)) = lo;
          *reinterpret_cast<uint4*>(rowp + (((ch + 1) ^ sw) << 4)) = hi;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) { mbar_arrive(v_ready); mbar_arrive(&stg_empty[s]); }
        return true;
      };
      if (ok && n_kv > 0) ok = conv_k(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) ok = conv_k(j + 1);
        if (ok) ok = conv_v(j);
      }
    } else {
      // ---------------------------------------------------------------- softmax, two threads per query row
      const int lane_group = warp & 3;                           // the TMEM lanes a warp may touch: 32 * (warp % 4) ..
      const int half = (warp - 6) >> 2;                          // 0: score / output columns [0, 64), 1: [64, 128)
      const int col0 = half * 64;
      const int row = lane_group * 32 + lane;
      const uint32_t t_lane = (uint32_t)(lane_group * 32) << 16;
      // One value per thread to the other thread of the same row: written to a TMEM column of the row's lane, handed
      // over by a two-warp mbarrier, read back by the partner.  Slots alternate, and a slot is written again only after
      // the barrier of the exchange in between, which the partner reaches after its read.
      int xn = 0;
      auto exchange = [&](float mine, float& other) -> bool {
        const int par = xn & 1;
        uint64_t* xb = &x_ready[par * 4 + lane_group];
        tmem_st_32x32b_x1(tX + t_lane + par * 2 + half, __float_as_uint(mine));
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(xb);
        if (!mbar_wait(xb, (xn >> 1) & 1, abort_flag, p.status, 0x833)) return false;
        tc_fence_after();
        uint32_t o;
        tmem_ld_32x32b_x1(tX + t_lane + par * 2 + (half ^ 1), o);
        tmem_ld_wait();
        other = __uint_as_float(o);
        ++xn;
        return true;
      };
      const int tok = q0 + row / G;                              // chunk-relative query token of this row
      const int head = kvh * G + row % G;
      const bool row_live = tok < q_len;
      const int pos = ctx0 + tok;                                // absolute position: keys [0, pos] are visible
      float m = -INFINITY, l = 0.f;
      const int sw = row & 7;
      uint8_t* prow0 = sP + half * kSub + (row >> 3) * 1024 + sw * 128;      // this half's 64 columns are one sub-tile
      for (int j = 0; j < n_kv && ok; ++j) {
        const int sb = j & 1;
        const int kv0 = j * kTcKv;
        if (!mbar_wait(&s_full[sb], (j >> 1) & 1, abort_flag, p.status, 0x830)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ts = tS + sb * 128 + t_lane;
        const int vis = row_live ? min(pos + 1, L) - kv0 : 0;     // columns [0, vis) of this tile are visible to the row
        // ---- this thread's half of the score row into registers, both loads in flight together, then release the buffer
        uint32_t sr[2][32];
#pragma unroll
        for (int c = 0; c < 2; ++c) tmem_ld_32x32b_x32(ts + col0 + c * 32, sr[c]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[sb]);
        // tiles below the diagonal need no masking at all (same for every row of the warp)
        const bool full = __all_sync(0xffffffffu, vis >= col0 + 64);
        if (!full) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + c * 32 + i >= vis) sr[c][i] = 0xff800000u;  // -inf: exp2 gives exactly 0 below
        }
        // four independent chains (a single running max would serialise 128 dependent instructions)
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sr[c][i]));
        float mx_other;
        if (!exchange(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])), mx_other)) { ok = false; break; }
        const float mx = fmaxf(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])), mx_other);    // the same in both halves
        // Lazy rescaling: the reference point m only moves when the row max grew by more than 2^8 (P stays below 256,
        // far inside f16 range), so the O accumulator in TMEM is rarely touched after the first tiles.
        float m_new = m, alpha = 1.f;
        if (mx > m + 8.f) {                   // also the first visible tile of a row (m = -inf)
          m_new = mx;
          alpha = (m == -INFINITY) ? 0.f : fast_exp2(m - mx);
        }
        // ---- the previous PV product must have retired before P is overwritten or O is rescaled
        if (j > 0) {
          if (!mbar_wait(pv_done, (j - 1) & 1, abort_flag, p.status, 0x831)) { ok = false; break; }
          tc_fence_after();
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(tO + t_lane + col0 + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32b_x32(tO + t_lane + col0 + c * 32, r);
            }
            tmem_st_wait();
          }
        }
        // ---- p = exp2(s - m) (masked scores are -inf), row sum over four independent chains, P (f16) into the
        //      A-operand layout
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        const float mref = (m_new == -INFINITY) ? 0.f : m_new;       // dead rows: -inf - 0 stays -inf, p = 0
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint8_t* rowp = prow0;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float e[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              e[i] = fast_exp2(__uint_as_float(sr[c][q * 8 + i]) - mref);
              sum4[i & 3] += e[i];
            }
            uint4 o;
            o.x = pack_h2(e[0], e[1]); o.y = pack_h2(e[2], e[3]); o.z = pack_h2(e[4], e[5]); o.w = pack_h2(e[6], e[7]);
            const int ch = c * 4 + q;
            *reinterpret_cast<uint4*>(rowp + ((ch ^ sw) << 4)) = o;
          }
        }
        const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        l = l * alpha + sum;
        m = m_new;
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
      }
      // ---- epilogue: O / l * v_scale -> bf16, each thread its 64 columns; l is the sum of the two halves' row sums
      float l_other = 0.f;
      if (ok && n_kv > 0) ok = exchange(l, l_other);
      l += l_other;
      if (ok && n_kv > 0 && mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag, p.status, 0x832)) {
        tc_fence_after();
        const float inv = (l > 0.f) ? p.v_scale / l : 0.f;
        if (p.q_out != nullptr) {
          // the whole output row in registers (as the score rows were), rounded to bf16 like the unfused path's
          // output, then one scale for the row's 128 values
          uint32_t r[2][32];
#pragma unroll
          for (int c = 0; c < 2; ++c) tmem_ld_32x32b_x32(tO + t_lane + col0 + c * 32, r[c]);
          tmem_ld_wait();
          float amax = 0.f;
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float v = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[c][i]) * inv));
              r[c][i] = __float_as_uint(v);
              amax = fmaxf(amax, fabsf(v));
            }
          float amax_other = 0.f;
          const bool got = exchange(amax, amax_other);           // every thread takes part, live row or not
          amax = fmaxf(amax, amax_other);
          if (row_live && got) {
            const float sc = fmaxf(amax, 1e-10f) / 448.f;
            const float qinv = __frcp_rn(sc);
            uint8_t* qrow = p.q_out + (long long)(q_row0 + tok) * p.ldqo + head * kTcD + col0;
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int b = q * 16 + j * 4;
                  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__uint_as_float(r[c][b]) * qinv, __uint_as_float(r[c][b + 1]) * qinv), __NV_SATFINITE, __NV_E4M3);
                  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__uint_as_float(r[c][b + 2]) * qinv, __uint_as_float(r[c][b + 3]) * qinv), __NV_SATFINITE, __NV_E4M3);
                  w[j] = lo | (hi << 16);
                }
                *reinterpret_cast<uint4*>(qrow + c * 32 + q * 16) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            if (half == 0) p.s_out[(long long)head * p.s_ld + q_row0 + tok] = sc;
          }
        } else {
        __nv_bfloat16* orow = p.out + (long long)(q_row0 + tok) * p.ldo + head * kTcD + col0;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tO + t_lane + col0 + c * 32, r);
          tmem_ld_wait();
          if (row_live) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
              o.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
              o.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
              o.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
            }
          }
        }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ================================================================================ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn tc_encode_fn() {
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

}  // namespace atlas

using namespace atlas;

// Chunk attention on tcgen05.  `num_tiles` query tiles of 128/G tokens each, described by (sequence index, first query
// token of the tile inside the sequence's chunk).  Covers head_dim 128, 16-token pages, an FP8 cache, G = Hq/Hkv in
// {1,2,4,8} and no sliding window; returns ATLAS_ATTN_TC_UNSUPPORTED (1) otherwise so that the caller can use the
// general kernel.
extern "C" int atlas_attn_prefill_tc(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                                     const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                                     const int* query_start_loc, const int* tile_seq, const int* tile_q0, int num_tiles,
                                     int total_tokens, float scale, float k_scale, float v_scale, int Hq, int Hkv, int D,
                                     int block_size, int window, unsigned long long* status, void* stream, void* q_out,
                                     long long ldqo, float* s_out, long long s_ld) {
  if (num_tiles <= 0) return 0;
  if (D != kTcD || block_size != kTcPage || window > 0 || Hq % Hkv) return 1;
  if (q_out != nullptr && (!s_out || (ldqo % 16) || (reinterpret_cast<uintptr_t>(q_out) & 15))) return 1;
  const int G = Hq / Hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8) return 1;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (ldq * 2) % 16) return 1;
  if (q_out == nullptr && ((ldo % 8) || (reinterpret_cast<uintptr_t>(out) & 15))) return 1;
  EncodeTiledFn enc = tc_encode_fn();
  if (!enc) return -10;
  // Q as [tokens][heads][dims]: box = 64 dims x G heads x 128/G tokens -> 128 rows of 128 bytes, row = token * G + head
  CUtensorMap tq;
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)Hq, (cuuint64_t)total_tokens};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)ldq * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(kTcRows / G)};
  cuuint32_t estr[3] = {1, 1, 1};
  if (enc(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -11;
  TcAttnParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.q_out = reinterpret_cast<uint8_t*>(q_out); p.ldqo = ldqo; p.s_out = s_out; p.s_ld = s_ld;
  p.k_cache = reinterpret_cast<const uint8_t*>(k_cache); p.v_cache = reinterpret_cast<const uint8_t*>(v_cache);
  p.block_tables = block_tables; p.bt_ld = bt_ld; p.seq_lens = seq_lens; p.query_start_loc = query_start_loc;
  p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.qk_scale_log2 = scale * k_scale * 1.4426950408889634f; p.v_scale = v_scale;
  p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.total_tokens = total_tokens; p.status = status;
  constexpr int kSmem = 8 * kSub + kTcStages * kStageBytes + 256 + 1024;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(attn_prefill_tc_kernel), kSmem) != cudaSuccess) return -20;
  dim3 grid(num_tiles, Hkv);
  attn_prefill_tc_kernel<<<grid, kTcThreads, kSmem, reinterpret_cast<cudaStream_t>(stream)>>>(tq, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
