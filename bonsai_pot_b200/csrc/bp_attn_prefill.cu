// Batched-prefill causal attention over the Q8_0 KV cache. Replaces
// attention.wgsl (dispatch_attention with is_prefill = 1, src/forward.rs:501-532).
#include "bp_common.cuh"

cudaError_t bp_launch_scalar_attention(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                                       __half* out, uint32_t cur_pos, uint32_t m, bool is_prefill,
                                       uint32_t* launches);

uint32_t bp_prefill_stage_tokens() { return 64; }
cudaError_t bp_prefill_init(bp_attn_ctx*) { return cudaSuccess; }

cudaError_t bp_launch_prefill(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                              __half* out, uint32_t m, uint32_t* launches) {
  return bp_launch_scalar_attention(c, s, layer, q, out, m, m, true, launches);
}
