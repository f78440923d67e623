// C ABI of the sm_100a kernel library (libatlas_b200_kernels.so).  Every function takes raw device pointers,
// element strides and a CUDA stream handle, launches asynchronously and returns 0 or a negative error code.
// The Python binding (atlas_b200/ops/cuda.py) calls these through ctypes.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- library state
int atlas_init(int device);                                   // allocates the per-device status word
unsigned long long* atlas_status_ptr(int device);
unsigned long long atlas_read_status(int device, int clear);  // synchronises the device
int atlas_num_sms(int device);

// ---- GEMM (gemm.cu)
int atlas_gemm(int kind, const void* A, const void* B, void* C, const float* a_scale, long long sa_m,
               long long sa_k, const float* b_scale, int b_scale_ld, int M, int N, int K, long long lda,
               long long ldb, long long ldc, int block_n, int splits, float* workspace, int* counters,
               int num_sms, unsigned long long* status, void* stream);

// Fused epilogue of atlas_gemm_fused (FP8 block-scaled GEMMs).
//   mode 0  plain bf16 store of C (only the deferred-norm factor below is applied)
//   mode 1  B = [gate rows; up rows] (N = 2 * I): silu(gate) * up, FP8 e4m3 in 128-wide groups -> q_out [M, I] (row stride
//           ldq) and s_out (scale(m, g) = s_out[g * s_ld + m])
//   mode 2  C + residual -> residual (in place, row stride ldr); (residual * norm_w [+1]) FP8-quantised -> q_out / s_out;
//           per-row sum of squares of every column tile -> ss_out[tile * ss_out_ld + m].  The 1/rms factor of the row is
//           left to the GEMM that consumes q_out, which gets the same array as ss_in.
//   ss_in   (any mode) deferred RMSNorm factor of the A operand: every output row m is scaled by
//           rsqrt(sum_{j < ss_in_parts} ss_in[j * ss_in_ld + m] * ss_inv_h + ss_eps).
typedef struct AtlasEpilogue {
  int mode;
  void* q_out; long long ldq;
  float* s_out; long long s_ld;
  void* residual; long long ldr;
  const void* norm_w; int norm_plus_one;
  float* ss_out; long long ss_out_ld;
  const float* ss_in; int ss_in_parts; long long ss_in_ld; float ss_inv_h; float ss_eps;
} AtlasEpilogue;

// ---- fused elementwise / norm / rope / KV write (elementwise.cu)
int atlas_rmsnorm(const void* x, long long ldx, const void* residual, long long ldr, const void* w, void* res_out,
                  long long ldro, void* y, long long ldy, void* q, long long ldq, float* scale, long long scale_ld,
                  int T, int H, float eps, int plus_one, void* stream);
int atlas_silu_mul(const void* gu, long long ld, int T, int I, void* y, long long ldy, void* q, long long ldq,
                   float* scale, long long scale_ld, const int* live_tiles, void* stream);
int atlas_quant_fp8(const void* x, long long ld, int T, int K, void* q, long long ldq, float* scale,
                    long long scale_ld, void* stream);
int atlas_rope_kv_write(void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                        const int* positions, const float* rope, const void* q_norm_w, const void* k_norm_w,
                        void* k_cache, void* v_cache, const int* slot_mapping, int T, int Hq, int Hkv, int D,
                        int rotary_dim, int block_size, int kv_fp8, int plus_one, float eps, float k_scale,
                        float v_scale, void* stream);
int atlas_wht_d128(void* x, long long ld, int T, int H, void* stream);
int atlas_gated_rmsnorm(const void* x, long long ldx, const void* z, long long ldz, const void* w, void* y,
                        long long ldy, int T, int H, int D, float eps, void* stream);

// ---- MoE (moe.cu) and grouped GEMM (gemm.cu)
int atlas_gelu_tanh_mul(const void* gu, long long ld, int T, int I, void* y, long long ldy, void* q, long long ldq,
                        float* scale, long long scale_ld, void* stream);
int atlas_moe_route(const void* logits, long long ld, int is_bf16, int T, int E, int k, int norm, int sigmoid,
                    float* w_out, int* id_out, void* stream);
int atlas_moe_route_ex(const void* logits, long long ld, int is_bf16, int T, int E, int k, int norm, int score_mode,
                       const float* sel_bias, int n_group, int topk_group, const int* hash_table, const int* token_ids,
                       float out_scale, float* w_out, int* id_out, void* stream);
int atlas_moe_align(const int* topk_ids, int T, int k, int e_lo, int E_local, int* slot_of, int* row_token,
                    int* tile_expert, int* num_tiles, int max_rows, unsigned long long* status, void* stream);
int atlas_moe_gather(const void* x, long long ldx, const int* row_token, const int* num_tiles, int max_rows, int H,
                     void* y, void* q, float* scale, long long scale_ld, void* stream);
int atlas_moe_combine(const void* y, long long ldy, const int* slot_of, const float* topk_w, int T, int k, int H,
                      const void* addend, long long ld_add, void* out, long long ldo, void* stream);
int atlas_moe_dispatch_prep(const int* topk_ids, int pairs, int experts_per_rank, int world, int* send_off, int* pos,
                            void* stream);
int atlas_moe_dispatch_pack(const void* x, long long ldx, const int* topk_ids, const int* pos, int T, int k, int H,
                            void* send, int row_bytes, void* stream);
int atlas_moe_recv_ids(const void* recv, int row_bytes, int H, const int* recv_off, int world, int cap_rows, int* ids,
                       void* stream);
int atlas_gemm_w4a16(const void* A, const void* packed, const void* bscale, const float* gscale, void* C, int M, int N,
                     int K, long long lda, long long ldc, int block_n, int num_sms, unsigned long long* status,
                     void* stream);
int atlas_gemm_w4a16_grouped(const void* A, const void* packed, const void* bscale, const float* gscale, void* C,
                             int max_rows, int N, int K, int E, long long lda, long long ldc, int block_n,
                             const int* tile_expert, const int* num_m_tiles, int num_sms, unsigned long long* status,
                             void* stream);
int atlas_gemm_grouped(int kind, const void* A, const void* B, void* C, const float* a_scale, long long sa_k,
                       const float* b_scale, int max_rows, int N, int K, int E, long long lda, long long ldb,
                       long long ldc, int block_n, const int* tile_expert, const int* num_m_tiles, int num_sms,
                       unsigned long long* status, void* stream);

// ---- Gated DeltaNet (gdn.cu)
int atlas_gdn_conv(const void* x, long long ldx, const void* w, int C, int W, const void* conv_state,
                   const int* seq_of_token, const int* query_start_loc, const int* state_slots,
                   const unsigned char* has_state, void* y, long long ldy, int T, void* stream);
int atlas_gdn_conv_state(const void* x, long long ldx, int C, int W, void* conv_state, const int* query_start_loc,
                         const int* state_slots, const unsigned char* has_state, const int* limit, const int* snap_rows,
                         const int* snap_slots, int num_snaps_per_seq, int B, void* stream);
int atlas_gdn_recurrent(const void* y, long long ldy, const void* a, long long lda, const void* b, long long ldb,
                        const float* A_log, const float* dt_bias, float* h, void* out, long long ldo,
                        const int* query_start_loc, const int* state_slots, const unsigned char* has_state,
                        const int* limit, const int* snap_rows, const int* snap_slots, int num_snaps_per_seq, int B,
                        int Hk, int Hv, int Dk, int Dv, int commit, void* stream);

// ---- peer-memory collectives (comm.cu)
int atlas_symm_alloc(size_t bytes, void** ptr);
int atlas_symm_free(void* ptr);
int atlas_ipc_export(void* ptr, void* handle64);
int atlas_ipc_open(const void* handle64, void** ptr);
int atlas_ipc_close(void* ptr);
int atlas_allreduce_bf16(int kind, void* const* data, void* const* flags, int rank, int world, const void* in, void* out,
                         size_t n_bytes, size_t slot_bytes, unsigned int* state, int blocks, unsigned long long* status,
                         long long max_cycles, void* stream);
int atlas_alltoall_rows(void* const* data, void* const* flags, int rank, int world, const void* in, const int* send_off,
                        void* out, int* recv_off, int row_bytes, int region_rows, size_t slot_bytes, unsigned int* state,
                        int blocks, unsigned long long* status, long long max_cycles, void* stream);

// ---- attention (attention.cu)
int atlas_attn_decode(const void* q, long long ldq, void* out, long long ldo, const void* k_cache, const void* v_cache,
                      const int* block_tables, int bt_ld, const int* seq_lens, const int* query_start_loc,
                      int seq_base, int B, float scale, float k_scale, float v_scale, int Hq, int Hkv, int D,
                      int block_size, int window, int num_splits, float* part_o, float* part_ml,
                      unsigned long long* status, void* stream);
int atlas_attn_decode_q8(const void* q, long long ldq, void* q_out, long long ldqo, float* s_out, long long s_ld,
                         const void* k_cache, const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                         const int* query_start_loc, int seq_base, int B, float scale, float k_scale, float v_scale,
                         int Hq, int Hkv, int block_size, int window, int num_splits, float* part_o, float* part_ml,
                         unsigned long long* status, void* stream);
int atlas_attn_prefill(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                       const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                       const int* query_start_loc, const int* tile_seq, const int* tile_q0, int num_tiles, float scale,
                       float k_scale, float v_scale, int Hq, int Hkv, int D, int block_size, int window, void* stream);

// ---- sampling (sampling.cu)
int atlas_argmax(const void* logits, long long ld, int B, int V, int is_bf16, long long* out, float* out_val,
                 void* stream);
int atlas_sample(const void* logits, long long ld, int B, int V, int is_bf16, const float* temperature,
                 const int* top_k, const float* top_p, const float* min_p, const float* uniform, long long* out,
                 void* stream);
int atlas_spec_accept(const long long* draft, const long long* target, int B, int K, int* n_acc, void* stream);
int atlas_logit_edits(float* logits, long long ld, int B, int V, const void* edits, int n, void* stream);

#ifdef __cplusplus
}
#endif
