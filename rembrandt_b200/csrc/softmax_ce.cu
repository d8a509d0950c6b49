// Fused softmax + cross-entropy head: one warp per sample does max, sum-exp, weighted loss,
// arg-max / accuracy count and the gradient  delta[b,k] = w_b (p[b,k] - 1[k = y_b])  in one pass.
// Replaces the reference's cuDNN softmax + batch_map_softmax_kl_backward + batch_map_softmax_kl_loss1 +
// batch_blockreduce_sum + batch_blockreduce_argmax sequence (src/operator/loss.rs:118-237), without its
// K <= 1024 and B <= 1024 limits.
#include "common.cuh"

namespace rb {

__global__ void softmax_ce_kernel(const bf16* __restrict__ logits, int B, int K, int ld,
                                  const int* __restrict__ labels, const float* __restrict__ weights, float w_scalar,
                                  bf16* __restrict__ delta, float* __restrict__ probs, float* __restrict__ loss_sum,
                                  int* __restrict__ correct, float* __restrict__ loss_per, int* __restrict__ argmax_out,
                                  const float* __restrict__ cat_weights) {
  const int warps_per_block = blockDim.x >> 5;
  const int b = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  const bf16* row = logits + (long long)b * ld;
  float mx = -INFINITY;
  int am = 0;
  for (int k = lane; k < K; k += 32) {
    const float v = bf2f(row[k]);
    if (v > mx) { mx = v; am = k; }
  }
  // arg-max across the warp (smallest index wins ties)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, mx, o);
    const int oi = __shfl_xor_sync(0xffffffffu, am, o);
    if (ov > mx || (ov == mx && oi < am)) { mx = ov; am = oi; }
  }
  float se = 0.f;
  for (int k = lane; k < K; k += 32) se += __expf(bf2f(row[k]) - mx);
  se = warp_sum(se);
  const float inv = 1.f / se;
  const int y = labels[b];
  const float w = weights ? weights[b] : w_scalar;
  if (delta || probs) {
    for (int k = lane; k < ld; k += 32) {
      float pk = 0.f;
      if (k < K) pk = __expf(bf2f(row[k]) - mx) * inv;
      if (probs && k < K) probs[(long long)b * K + k] = pk;
      if (delta) {
        float d = 0.f;
        if (k < K) {
          d = w * (pk - (k == y ? 1.f : 0.f));
          if (cat_weights) d *= cat_weights[k];
        }
        delta[(long long)b * ld + k] = f2bf(d);
      }
    }
  }
  if (lane == 0) {
    float l = 0.f;
    if (y >= 0 && y < K) l = -(bf2f(row[y]) - mx - __logf(se));
    if (loss_per) loss_per[b] = l;
    if (argmax_out) argmax_out[b] = am;
    if (loss_sum) atomicAdd(loss_sum, w * l);
    if (correct && am == y) atomicAdd(correct, 1);
  }
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_softmax_ce(const void* logits, int B, int K, int ld, const int* labels, const float* weights, float w_scalar,
                  void* delta, float* probs, float* loss_sum, int* correct, float* loss_per, int* argmax_out,
                  const float* cat_weights, cudaStream_t st) {
  const int wpb = 4;
  softmax_ce_kernel<<<(B + wpb - 1) / wpb, wpb * 32, 0, st>>>((const bf16*)logits, B, K, ld, labels, weights, w_scalar,
                                                             (bf16*)delta, probs, loss_sum, correct, loss_per,
                                                             argmax_out, cat_weights);
  return RB_LAUNCH_OK();
}

}  // extern "C"
