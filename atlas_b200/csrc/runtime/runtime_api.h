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

// ---- batched record I/O through io_uring (uring_io.cpp) ----------------------------------------------------------------
// 1 when this kernel / sandbox lets the process create an io_uring.
int atlas_uring_available(void);
// n records of bytes_each at offsets[i] of fd <-> bufs[i] (write != 0: buffers to file), at most depth requests in
// flight.  Returns n * bytes_each or -errno.
long long atlas_uring_rw(int fd, int write, int n, const long long* offsets, void* const* bufs, long long bytes_each, int depth);

// ---- grammar-constrained decoding (grammar.cpp) ------------------------------------------------------------------------
typedef struct atlas_grammar atlas_grammar;
typedef struct atlas_vocab atlas_vocab;
typedef struct atlas_matcher atlas_matcher;
// EBNF text -> grammar (NULL on a syntax error, message copied to err).  `root` names the start rule ("root" if empty).
atlas_grammar* atlas_grammar_compile(const char* text, const char* root, char* err, int errcap);
void atlas_grammar_destroy(atlas_grammar*);
int atlas_grammar_num_rules(const atlas_grammar*);
// Token t is bytes[offsets[t] .. offsets[t+1]); tokens without bytes (specials) are never allowed by a grammar.
atlas_vocab* atlas_vocab_create(const uint8_t* bytes, const int64_t* offsets, int n_tokens);
void atlas_vocab_destroy(atlas_vocab*);
int atlas_vocab_num_nodes(const atlas_vocab*);
atlas_matcher* atlas_matcher_create(const atlas_grammar*, const atlas_vocab*);
void atlas_matcher_destroy(atlas_matcher*);
int atlas_matcher_can_end(const atlas_matcher*);
int atlas_matcher_exhausted(const atlas_matcher*);
int atlas_matcher_mask(atlas_matcher*, uint32_t* bits, int n_words);
int atlas_matcher_accept_bytes(atlas_matcher*, const uint8_t* bytes, int n);
int atlas_matcher_rollback(atlas_matcher*, int n);
int atlas_matcher_num_stacks(const atlas_matcher*);

#ifdef __cplusplus
}
#endif
