// Pipelined checkpoint reader: worker threads pread fixed-size chunks with O_DIRECT into 4 KiB-aligned bounce buffers
// and copy them to the destination (typically pinned host memory that a CUDA stream then uploads), so the page cache
// is bypassed and the disk queue stays full.  Unaligned heads / tails and filesystems that refuse O_DIRECT use
// buffered reads.
// Reference behaviour: crates/spark-runtime/src/fast_weights/{mod,direct_io}.rs (O_DIRECT pipelined loader).
#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include <errno.h>
#include <fcntl.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <thread>
#include <vector>

#include "runtime_api.h"

namespace {
constexpr long long kAlign = 4096;

long long pread_all(int fd, char* dst, long long len, long long off) {
  long long done = 0;
  while (done < len) {
    ssize_t r = pread(fd, dst + done, (size_t)(len - done), (off_t)(off + done));
    if (r < 0) {
      if (errno == EINTR) continue;
      return -errno;
    }
    if (r == 0) break;
    done += r;
  }
  return done;
}
}  // namespace

extern "C" long long atlas_read_file(const char* path, long long offset, long long len, void* dst, int threads,
                                     long long chunk) {
  if (len <= 0) return 0;
  if (threads < 1) threads = 1;
  if (threads > 64) threads = 64;
  if (chunk < kAlign) chunk = 8ll << 20;
  chunk = (chunk + kAlign - 1) / kAlign * kAlign;
  int fd_direct = open(path, O_RDONLY | O_DIRECT);
  int fd_plain = open(path, O_RDONLY);
  if (fd_plain < 0) {
    const int e = errno;
    if (fd_direct >= 0) close(fd_direct);
    return -e;
  }
  const long long nchunks = (len + chunk - 1) / chunk;
  std::atomic<long long> next{0}, total{0}, err{0};
  auto work = [&]() {
    void* bounce = nullptr;
    if (fd_direct >= 0 && posix_memalign(&bounce, kAlign, (size_t)chunk + kAlign) != 0) bounce = nullptr;
    for (;;) {
      const long long c = next.fetch_add(1);
      if (c >= nchunks || err.load()) break;
      const long long lo = offset + c * chunk;
      const long long n = (c == nchunks - 1) ? (offset + len - lo) : chunk;
      char* out = static_cast<char*>(dst) + (lo - offset);
      long long got = -1;
      if (bounce) {
        // widen to aligned bounds, read, copy the wanted window
        const long long alo = lo / kAlign * kAlign;
        const long long ahi = (lo + n + kAlign - 1) / kAlign * kAlign;
        long long r = pread_all(fd_direct, static_cast<char*>(bounce), ahi - alo, alo);
        if (r >= (lo - alo) + 1) {
          long long avail = r - (lo - alo);
          if (avail > n) avail = n;
          memcpy(out, static_cast<char*>(bounce) + (lo - alo), (size_t)avail);
          got = avail;
        }
      }
      if (got < 0) got = pread_all(fd_plain, out, n, lo);
      if (got < 0) { err.store(got); break; }
      total.fetch_add(got);
      if (got < n) break;      // end of file
    }
    free(bounce);
  };
  std::vector<std::thread> pool;
  for (int t = 1; t < threads; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
  if (fd_direct >= 0) close(fd_direct);
  close(fd_plain);
  return err.load() ? err.load() : total.load();
}
