// Host runtime of the engine as a plain C ABI (bound from Python with ctypes): paged-KV block pool with reference
// counts, block-granular radix tree (prefix cache index) with LRU leaf eviction, process-wide fault latch, and a
// pipelined O_DIRECT file reader for checkpoint shards.  No CUDA here; device state stays with the caller.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- block pool ------------------------------------------------------------------------------------------------
typedef struct atlas_pool atlas_pool;
atlas_pool* atlas_pool_create(int num_blocks, int block_size);
void atlas_pool_destroy(atlas_pool*);
int atlas_pool_num_free(const atlas_pool*);
int atlas_pool_block_size(const atlas_pool*);
int atlas_pool_ref_count(const atlas_pool*, int block);
// Takes n blocks (FIFO order of the free list) into out[]; returns 0, or -1 when fewer than n are free (nothing taken).
int atlas_pool_alloc(atlas_pool*, int n, int* out);
// +1 on each block; -2 if one of them is free (nothing changed).
int atlas_pool_inc_ref(atlas_pool*, const int* blocks, int n);
// -1 on each block; returns how many went back to the free list, or -2 on a double free (processing stops there).
int atlas_pool_free(atlas_pool*, const int* blocks, int n);
// 0 when the free list and the reference counts agree.
int atlas_pool_check(const atlas_pool*);

// ---- radix tree over whole blocks of token ids --------------------------------------------------------------------
typedef struct atlas_radix atlas_radix;
atlas_radix* atlas_radix_create(atlas_pool* pool);
void atlas_radix_destroy(atlas_radix*);
// Longest cached prefix of tokens[0..n) in whole blocks, leaving at least one token uncomputed and at most max_tokens
// (negative = no limit).  Writes block ids to blocks_out and opaque node handles to nodes_out (capacity cap); every
// returned block gets one pool reference and every node one pin.  Returns the number of blocks matched.
int atlas_radix_match(atlas_radix*, uint64_t ns, const int32_t* tokens, int n, int max_tokens, int* blocks_out,
                      uint64_t* nodes_out, int cap);
void atlas_radix_release(atlas_radix*, const uint64_t* nodes, int n);
// Publishes the full blocks of a sequence (blocks[j] holds tokens [j*bs, (j+1)*bs)); new nodes take a pool reference.
// Returns the number of nodes created.
int atlas_radix_insert(atlas_radix*, uint64_t ns, const int32_t* tokens, int n, const int* blocks, int nblocks);
// Evicts least-recently-used unpinned leaves until `want` blocks have been returned to the pool; returns the count.
int atlas_radix_evict(atlas_radix*, int want);
int atlas_radix_num_nodes(const atlas_radix*);
int atlas_radix_evictable(const atlas_radix*);

// ---- fault latch (one shot, process wide) ----------------------------------------------------------------------------
// Returns 1 if this call tripped it, 0 if it was already tripped (the first reason sticks).
int atlas_fault_trip(const char* reason);
int atlas_fault_tripped(void);
// Copies the reason (NUL terminated, truncated to cap) and returns its full length; 0 when not tripped.
int atlas_fault_reason(char* out, int cap);
void atlas_fault_reset_for_tests(void);

// ---- pipelined direct-I/O reader -----------------------------------------------------------------------------------------
// Reads [offset, offset+len) of `path` into dst with `threads` workers issuing O_DIRECT preads of `chunk` bytes through
// aligned bounce buffers (falls back to buffered reads where O_DIRECT is refused).  Returns bytes read or -errno.
long long atlas_read_file(const char* path, long long offset, long long len, void* dst, int threads, long long chunk);

#ifdef __cplusplus
}
#endif
