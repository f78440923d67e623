// C ABI of the sm_100a kernel library (libatlas_b200_kernels.so).  Every function takes raw device pointers,
// element strides and a CUDA stream handle, launches asynchronously and returns 0 or a negative error code.
// The Python binding (atlas_b200/ops/cuda.py) calls these through ctypes.
#pragma once
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

// ---- fused elementwise / norm / rope / KV write (elementwise.cu)
int atlas_rmsnorm(const void* x, long long ldx, const void* residual, long long ldr, const void* w, void* res_out,
                  long long ldro, void* y, long long ldy, void* q, long long ldq, float* scale, long long scale_ld,
                  int T, int H, float eps, int plus_one, void* stream);
int atlas_silu_mul(const void* gu, long long ld, int T, int I, void* y, long long ldy, void* q, long long ldq,
                   float* scale, long long scale_ld, void* stream);
int atlas_quant_fp8(const void* x, long long ld, int T, int K, void* q, long long ldq, float* scale,
                    long long scale_ld, void* stream);
int atlas_rope_kv_write(void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                        const int* positions, const float* rope, const void* q_norm_w, const void* k_norm_w,
                        void* k_cache, void* v_cache, const int* slot_mapping, int T, int Hq, int Hkv, int D,
                        int rotary_dim, int block_size, int kv_fp8, int plus_one, float eps, float k_scale,
                        float v_scale, void* stream);
int atlas_gated_rmsnorm(const void* x, long long ldx, const void* z, long long ldz, const void* w, void* y,
                        long long ldy, int T, int H, int D, float eps, void* stream);

// ---- attention (attention.cu)
int atlas_attn_decode(const void* q, long long ldq, void* out, long long ldo, const void* k_cache, const void* v_cache,
                      const int* block_tables, int bt_ld, const int* seq_lens, const int* query_start_loc,
                      int seq_base, int B, float scale, float k_scale, float v_scale, int Hq, int Hkv, int D,
                      int block_size, int window, int num_splits, float* part_o, float* part_ml,
                      unsigned long long* status, void* stream);
int atlas_attn_prefill(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                       const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                       const int* query_start_loc, const int* tile_seq, const int* tile_q0, int num_tiles, float scale,
                       float k_scale, float v_scale, int Hq, int Hkv, int D, int block_size, int window, void* stream);

// ---- sampling (sampling.cu)
int atlas_argmax(const void* logits, long long ld, int B, int V, int is_bf16, long long* out, void* stream);
int atlas_sample(const void* logits, long long ld, int B, int V, int is_bf16, const float* temperature,
                 const int* top_k, const float* top_p, const float* min_p, const float* uniform, long long* out,
                 void* stream);
int atlas_spec_accept(const long long* draft, const long long* target, int B, int K, int* n_acc, void* stream);

#ifdef __cplusplus
}
#endif
