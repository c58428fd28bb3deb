// Launchers of the non-attention operators on Q1_0 weights (bp_q1_ops.cu). A Q1_0 tensor
// [n rows][k inputs] is n * k / 128 blocks of one f16 scale and 128 sign bits; on the device it is
// held as the reference's two arrays (scales, sign bytes: src/model.rs manifest d_offset / qs_offset)
// plus, for the tensors the one-token path multiplies, the sign words re-laid out for the matvec kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

struct bp_q1_tensor {
  const __half* d;      // block scales [n][k / 128]
  const uint8_t* qs;    // sign bytes [n][k / 128][16], bit e of a block = weight e (1 = +d, 0 = -d)
  const void* bits;     // re-laid-out sign words [n][k / 128] (uint4), or null
  uint32_t k, n;
};

void bp_q1_set_matvec_rows(uint32_t rows_per_lane);  // tuning aid: 0 = by tensor height, else 1, 2 or 4
cudaError_t bp_q1_relayout(cudaStream_t s, const uint8_t* qs, void* out, uint64_t n_blocks);
cudaError_t bp_q1_matvec(bool pdl, cudaStream_t s, const bp_q1_tensor& w, const __half* x, __half* y, bool accumulate);
cudaError_t bp_q1_matvec_normed(bool pdl, cudaStream_t s, const bp_q1_tensor* w, __half* const* out, uint32_t n_ranges,
                                const __half* x, const __half* w_norm, float eps);
cudaError_t bp_q1_matvec_normed_silu(bool pdl, cudaStream_t s, const bp_q1_tensor& w_gate, const bp_q1_tensor& w_up, __half* out,
                                     const __half* x, const __half* w_norm, float eps);
cudaError_t bp_q1_matvec_silu(bool pdl, cudaStream_t s, const bp_q1_tensor& w, const __half* gate, const __half* up, __half* y,
                              bool accumulate);
cudaError_t bp_q1_rms_norm(bool pdl, cudaStream_t s, const __half* in, __half* out, const __half* w, uint32_t group_size,
                           uint32_t n_groups, float eps);
cudaError_t bp_q1_silu_mul(bool pdl, cudaStream_t s, const __half* gate, const __half* up, __half* out, uint64_t n);
cudaError_t bp_q1_embed(bool pdl, cudaStream_t s, const bp_q1_tensor& w, const uint32_t* tokens, uint32_t m, __half* x);
cudaError_t bp_q1_quantize_q8(bool pdl, cudaStream_t s, const __half* x, uint32_t k, uint32_t m, float* d_out, int8_t* qs_out);
// err: device-visible error word that a bounded wait of the tensor-core kernel stores a code in when it gives
// up (null: a word of the library's own, read and cleared by bp_q1_take_error); wait_limit 0 = default.
cudaError_t bp_q1_matmul(bool pdl, cudaStream_t s, const bp_q1_tensor& w, uint32_t m, const float* a_d, const int8_t* a_qs, __half* y,
                         bool accumulate, uint32_t* err = nullptr, uint32_t wait_limit = 0);
cudaError_t bp_q1_matmul_multi(bool pdl, cudaStream_t s, const bp_q1_tensor* w, __half* const* y, uint32_t n_w, uint32_t m, const float* a_d,
                               const int8_t* a_qs, bool accumulate, uint32_t* err = nullptr, uint32_t wait_limit = 0);
void bp_q1_set_matmul_variant(uint32_t variant);  // tuning aid: 0 = by batch size (1 or 2), 1 = dp4a, 2 = mma.sync, 3 = tcgen05
cudaError_t bp_q1_take_error(uint32_t* code);     // synchronous; 0 = no wait gave up since the last call
cudaError_t bp_q1_topk(bool pdl, cudaStream_t s, const __half* logits, uint32_t n, uint32_t k, float* out_val, uint32_t* out_idx);
