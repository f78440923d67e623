// What a weight stream costs on its own: every CTA walks `k_blocks` tile copies (box_rows rows x 128 bytes each, TMA,
// 128-byte swizzle) through a ring of `stages` shared-memory slots and does nothing with them but hand the slot back.
// The same bytes can be laid out the way a [N, K] FP8 weight lies in memory (a tile's rows are `ld` bytes apart, one
// k slice of every row per copy) or packed tile by tile (ld = 128: a copy reads one contiguous block).  Comparing the two
// at the GEMM kernels' ring depths separates what the memory system gives for each access pattern from what the GEMM
// pipeline adds (used by `python -m atlas_b200.bench.microbench --only stream`).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "tmap.h"

namespace atlas {

__global__ void __launch_bounds__(64, 1)
tma_stream_probe_kernel(const __grid_constant__ CUtensorMap tmap, int box_rows, int stages, int k_blocks, int tiles,
                        int packed, int pieces, status_t* status, unsigned long long* sink) {
  extern __shared__ uint8_t probe_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(probe_raw) + 1023) & ~uintptr_t(1023));
  const int slot_bytes = box_rows * 128;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * slot_bytes);
  uint64_t* empty = full + stages;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(empty + stages);
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) {
    uint32_t stage = 0, phase = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, status, 0x900)) return;
        mbar_expect_tx(&full[stage], slot_bytes);
        // weight layout: column kb * 128 of rows [tile * box_rows, +box_rows); packed: rows of 128 bytes, tile after tile
        // a slot is filled by `pieces` copies of box_rows / pieces rows each (the tensor map's box is one piece)
        const int pr = box_rows / pieces;
        for (int pc = 0; pc < pieces; ++pc) {
          uint8_t* dst = smem + (size_t)stage * slot_bytes + (size_t)pc * pr * 128;
          if (packed) tma_load_2d(dst, &tmap, &full[stage], 0, (tile * k_blocks + kb) * box_rows + pc * pr);
          else        tma_load_2d(dst, &tmap, &full[stage], kb * 128, tile * box_rows + pc * pr);
        }
        if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1 && lane == 0) {
    uint32_t stage = 0, phase = 0;
    unsigned long long acc = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(&full[stage], phase, abort_flag, status, 0x901)) return;
        acc += *reinterpret_cast<volatile unsigned long long*>(smem + (size_t)stage * slot_bytes);
        mbar_arrive(&empty[stage]);
        if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
      }
    }
    if (acc == 0x1234567887654321ull) *sink = acc;       // keeps the reads alive
  }
}

// The same walk with per-thread 16-byte asynchronous copies (cp.async, no copy engine): every warp streams its own
// `chunk_bytes` chunks (chunk index = warp-global index + k * total warps) through a private ring of `depth` chunks.
__global__ void __launch_bounds__(128)
cpasync_stream_probe_kernel(const uint8_t* __restrict__ data, int chunk_bytes, int depth, int chunks_per_warp, unsigned long long* sink) {
  extern __shared__ __align__(128) uint8_t probe_cp[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * 4;
  const int gw = blockIdx.x * 4 + warp;
  uint8_t* ring = probe_cp + (size_t)warp * depth * chunk_bytes;
  auto issue = [&](int k) {
    const uint8_t* src = data + ((size_t)gw + (size_t)k * warps_total) * chunk_bytes;
    uint8_t* dst = ring + (size_t)(k % depth) * chunk_bytes;
    for (int off = lane * 16; off < chunk_bytes; off += 512)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst + off)), "l"(src + off) : "memory");
  };
  for (int k = 0; k < depth - 1 && k < chunks_per_warp; ++k) {
    issue(k);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }
  unsigned long long acc = 0;
  for (int k = 0; k < chunks_per_warp; ++k) {
    if (k + depth - 1 < chunks_per_warp) issue(k + depth - 1);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    // all but the newest depth - 1 groups are complete: chunk k has landed
    switch (depth - 1) {
      case 1: asm volatile("cp.async.wait_group 1;\n" ::: "memory"); break;
      case 2: asm volatile("cp.async.wait_group 2;\n" ::: "memory"); break;
      case 3: asm volatile("cp.async.wait_group 3;\n" ::: "memory"); break;
      case 5: asm volatile("cp.async.wait_group 5;\n" ::: "memory"); break;
      case 7: asm volatile("cp.async.wait_group 7;\n" ::: "memory"); break;
      default: asm volatile("cp.async.wait_group 0;\n" ::: "memory"); break;
    }
    __syncwarp();
    acc += *reinterpret_cast<volatile unsigned long long*>(ring + (size_t)(k % depth) * chunk_bytes + lane * 8);
    __syncwarp();
  }
  if (acc == 0x1234567887654321ull) *sink = acc;
}

}  // namespace atlas

using namespace atlas;

// `ctas` CTAs of four warps; every warp walks chunks_per_warp chunks of chunk_bytes (a multiple of 512) with `depth`
// (2, 3, 4, 6 or 8) chunks in flight.  The walk covers ctas * 4 * chunks_per_warp * chunk_bytes <= data_bytes.
extern "C" int atlas_probe_cpasync_stream(const void* data, long long data_bytes, int ctas, int chunk_bytes, int depth,
                                          int chunks_per_warp, unsigned long long* sink, void* stream) {
  if (ctas <= 0 || chunk_bytes < 512 || chunk_bytes % 512 || chunks_per_warp <= 0) return -1;
  if (depth != 2 && depth != 3 && depth != 4 && depth != 6 && depth != 8) return -1;
  if ((long long)ctas * 4 * chunks_per_warp * chunk_bytes > data_bytes) return -3;
  const size_t smem = (size_t)4 * depth * chunk_bytes;
  if (smem > 200 * 1024) return -2;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(cpasync_stream_probe_kernel), (int)smem) != cudaSuccess) return -20;
  cpasync_stream_probe_kernel<<<ctas, 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(data), chunk_bytes, depth, chunks_per_warp, sink);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// `data` (data_bytes long) holds rows_total * ld bytes (weight layout: rows_total = tiles * box_rows rows of ld = k_blocks * 128 bytes;
// packed: rows_total = tiles * k_blocks * box_rows rows of 128 bytes).  Returns 0 or a negative code.
extern "C" int atlas_probe_tma_stream(const void* data, long long data_bytes, int tiles, int k_blocks, int box_rows, int stages,
                                      int packed, int ctas, int pieces, unsigned long long* status, unsigned long long* sink,
                                      void* stream) {
  if (tiles <= 0 || k_blocks <= 0 || box_rows < 8 || box_rows > 256 || stages < 1 || stages > 16) return -1;
  if ((long long)tiles * k_blocks * box_rows * 128 > data_bytes) return -3;        // the walk must stay inside the buffer
  if (pieces < 1 || box_rows % pieces || (box_rows / pieces) % 8) return -1;
  const size_t smem = (size_t)stages * box_rows * 128 + 1024 + 512;
  if (smem > 227 * 1024) return -2;
  CUtensorMap tm;
  int rc;
  const uint32_t piece_rows = (uint32_t)(box_rows / pieces);
  if (packed) rc = make_tmap_2d(&tm, data, (uint64_t)tiles * k_blocks * box_rows, 128, 128, piece_rows, 1, 128u, true);
  else        rc = make_tmap_2d(&tm, data, (uint64_t)tiles * box_rows, (uint64_t)k_blocks * 128, (uint64_t)k_blocks * 128, piece_rows,
                                1, 128u, true);
  if (rc) return rc;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(tma_stream_probe_kernel), (int)smem) != cudaSuccess) return -20;
  tma_stream_probe_kernel<<<ctas, 64, smem, reinterpret_cast<cudaStream_t>(stream)>>>(tm, box_rows, stages, k_blocks, tiles, packed,
                                                                                     pieces, status, sink);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
