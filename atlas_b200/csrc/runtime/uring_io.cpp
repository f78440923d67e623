// Batched positional I/O of fixed-size records through one io_uring (raw system calls, no liburing): the file tier of the
// KV cache moves every block of a parked sequence with one submission instead of one pread / pwrite per block, so the
// device queue holds many requests at once.  A ring is created per call (a few tens of microseconds against batches of
// megabytes), which keeps the entry point re-entrant without shared state.  Short transfers are resubmitted for the
// remainder; any failed request fails the call.  Where the kernel or the sandbox refuses io_uring the caller keeps
// its pread / pwrite loop (`atlas_uring_available`).
// Reference behaviour: crates/spark-storage/src/high_speed_swap.rs (io_uring queue of NVMe block reads / writes).
#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include <errno.h>
#include <linux/io_uring.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <vector>

#include "runtime_api.h"

namespace {

int sys_setup(unsigned entries, io_uring_params* p) { return (int)syscall(__NR_io_uring_setup, entries, p); }
int sys_enter(int fd, unsigned to_submit, unsigned min_complete, unsigned flags) {
  return (int)syscall(__NR_io_uring_enter, fd, to_submit, min_complete, flags, nullptr, 0);
}

struct Ring {
  int fd = -1;
  void* sq_map = MAP_FAILED; size_t sq_len = 0;
  void* cq_map = MAP_FAILED; size_t cq_len = 0;
  io_uring_sqe* sqes = (io_uring_sqe*)MAP_FAILED; size_t sqes_len = 0;
  unsigned *sq_head = nullptr, *sq_tail = nullptr, *sq_mask = nullptr, *sq_array = nullptr;
  unsigned *cq_head = nullptr, *cq_tail = nullptr, *cq_mask = nullptr;
  io_uring_cqe* cqes = nullptr;
  unsigned entries = 0;

  int open(unsigned want) {
    io_uring_params p;
    memset(&p, 0, sizeof(p));
    fd = sys_setup(want, &p);
    if (fd < 0) return -errno;
    entries = p.sq_entries;
    sq_len = p.sq_off.array + p.sq_entries * sizeof(unsigned);
    cq_len = p.cq_off.cqes + p.cq_entries * sizeof(io_uring_cqe);
    const bool single = (p.features & IORING_FEAT_SINGLE_MMAP) != 0;
    if (single) sq_len = cq_len = (sq_len > cq_len ? sq_len : cq_len);
    sq_map = mmap(nullptr, sq_len, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_SQ_RING);
    if (sq_map == MAP_FAILED) return -errno;
    if (single) {
      cq_map = sq_map;
    } else {
      cq_map = mmap(nullptr, cq_len, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_CQ_RING);
      if (cq_map == MAP_FAILED) return -errno;
    }
    sqes_len = p.sq_entries * sizeof(io_uring_sqe);
    sqes = (io_uring_sqe*)mmap(nullptr, sqes_len, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_SQES);
    if (sqes == (io_uring_sqe*)MAP_FAILED) return -errno;
    char* sq = (char*)sq_map;
    sq_head = (unsigned*)(sq + p.sq_off.head); sq_tail = (unsigned*)(sq + p.sq_off.tail);
    sq_mask = (unsigned*)(sq + p.sq_off.ring_mask); sq_array = (unsigned*)(sq + p.sq_off.array);
    char* cq = (char*)cq_map;
    cq_head = (unsigned*)(cq + p.cq_off.head); cq_tail = (unsigned*)(cq + p.cq_off.tail);
    cq_mask = (unsigned*)(cq + p.cq_off.ring_mask); cqes = (io_uring_cqe*)(cq + p.cq_off.cqes);
    return 0;
  }

  ~Ring() {
    if (sqes != (io_uring_sqe*)MAP_FAILED) munmap(sqes, sqes_len);
    if (cq_map != MAP_FAILED && cq_map != sq_map) munmap(cq_map, cq_len);
    if (sq_map != MAP_FAILED) munmap(sq_map, sq_len);
    if (fd >= 0) close(fd);
  }
};

struct Req {
  long long off; char* buf; long long left;
};

}  // namespace

extern "C" int atlas_uring_available(void) {
  static std::atomic<int> cached{-1};
  int v = cached.load();
  if (v < 0) {
    Ring r;
    v = r.open(2) == 0 ? 1 : 0;
    cached.store(v);
  }
  return v;
}

// n records of `bytes_each` at file offsets offsets[i] <-> bufs[i]; write != 0 writes the buffers to the file.  At most
// `depth` requests are in flight.  Returns the bytes moved (n * bytes_each) or -errno.
extern "C" long long atlas_uring_rw(int fd, int write, int n, const long long* offsets, void* const* bufs, long long bytes_each,
                                    int depth) {
  if (n <= 0 || bytes_each <= 0) return 0;
  if (depth < 1) depth = 1;
  if (depth > 256) depth = 256;
  Ring ring;
  const int rc = ring.open((unsigned)(depth < n ? depth : n));
  if (rc != 0) return rc;
  std::vector<Req> reqs((size_t)n);
  for (int i = 0; i < n; ++i) reqs[(size_t)i] = Req{offsets[i], (char*)bufs[i], bytes_each};
  std::vector<int> todo;                      // request indices waiting for a submission slot (new or remainder)
  todo.reserve((size_t)n);
  for (int i = n - 1; i >= 0; --i) todo.push_back(i);
  int inflight = 0, done = 0;
  long long err = 0;
  while (done < n) {
    unsigned queued = 0;
    unsigned tail = *ring.sq_tail;
    while (!todo.empty() && inflight + (int)queued < (int)ring.entries && err == 0) {
      const int i = todo.back();
      todo.pop_back();
      const unsigned idx = tail & *ring.sq_mask;
      io_uring_sqe* s = &ring.sqes[idx];
      memset(s, 0, sizeof(*s));
      s->opcode = write ? IORING_OP_WRITE : IORING_OP_READ;
      s->fd = fd;
      s->addr = (unsigned long long)(uintptr_t)reqs[(size_t)i].buf;
      s->len = (unsigned)(reqs[(size_t)i].left > (1ll << 30) ? (1ll << 30) : reqs[(size_t)i].left);
      s->off = (unsigned long long)reqs[(size_t)i].off;
      s->user_data = (unsigned long long)i;
      ring.sq_array[idx] = idx;
      ++tail;
      ++queued;
    }
    if (queued) __atomic_store_n(ring.sq_tail, tail, __ATOMIC_RELEASE);
    if (queued == 0 && inflight == 0) break;            // an error stopped new submissions and nothing is pending
    int r;
    do {
      r = sys_enter(ring.fd, queued, 1, IORING_ENTER_GETEVENTS);
    } while (r < 0 && errno == EINTR);
    if (r < 0) return -errno;
    inflight += (int)queued;
    unsigned head = *ring.cq_head;
    const unsigned ctail = __atomic_load_n(ring.cq_tail, __ATOMIC_ACQUIRE);
    while (head != ctail) {
      const io_uring_cqe* c = &ring.cqes[head & *ring.cq_mask];
      const int i = (int)c->user_data;
      --inflight;
      if (c->res < 0) {
        if (err == 0) err = c->res;
        ++done;
      } else if (c->res == 0) {                          // end of file before the record was complete
        if (err == 0) err = -EIO;
        ++done;
      } else {
        Req& q = reqs[(size_t)i];
        q.off += c->res; q.buf += c->res; q.left -= c->res;
        if (q.left > 0 && err == 0) todo.push_back(i); else ++done;
      }
      ++head;
    }
    __atomic_store_n(ring.cq_head, head, __ATOMIC_RELEASE);
  }
  return err != 0 ? err : (long long)n * bytes_each;
}
