// Fused softmax + cross-entropy head: one warp per sample does max, sum-exp, weighted loss,
// arg-max / accuracy count and the gradient  delta[b,k] = w_b (p[b,k] - 1[k = y_b])  in one pass.
// Replaces the reference's cuDNN softmax + batch_map_softmax_kl_backward + batch_map_softmax_kl_loss1 +
// batch_blockreduce_sum + batch_blockreduce_argmax sequence (src/operator/loss.rs:118-237), without its
// K <= 1024 and B <= 1024 limits.
#include "launch.cuh"
#include "common.cuh"

namespace rb {

// Rows are (sample, head) pairs: a sample carries L heads of K logits each, head l at columns [l K, (l+1) K) of its
// row of `ld` columns (L = 1 is the plain softmax head; L > 1 the k-step look-ahead heads). `mask` (optional,
// [B L][K] bytes) marks the admissible categories: the others get probability zero and the rest is renormalised
// (the legal-move masks of the reference's gen-2 softmax head). A head whose label is negative is skipped: zero
// delta, no loss. Accuracy and arg-max are those of head 0.
// `soft` (optional, [B L][K] floats) replaces the one-hot target by a distribution q (a teacher's probabilities):
// delta = w (p - q), loss = -sum_k q_k log p_k; accuracy then compares with the label as before.
__global__ void softmax_ce_kernel(const bf16* __restrict__ logits, int B, int K, int ld, int L,
                                  const int* __restrict__ labels, const float* __restrict__ weights, float w_scalar,
                                  bf16* __restrict__ delta, float* __restrict__ probs, float* __restrict__ loss_sum,
                                  int* __restrict__ correct, float* __restrict__ loss_per, int* __restrict__ argmax_out,
                                  const float* __restrict__ cat_weights, const uint8_t* __restrict__ mask,
                                  const float* __restrict__ soft) {
  pdl_prolog();
  const int warps_per_block = blockDim.x >> 5;
  const int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= B * L) return;
  const int b = r / L, l = r - b * L;
  const bf16* row = logits + (long long)b * ld + (long long)l * K;
  const uint8_t* mrow = mask ? mask + (long long)r * K : nullptr;
  float mx = -INFINITY;
  int am = 0;
  for (int k = lane; k < K; k += 32) {
    if (mrow && !mrow[k]) continue;
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
  for (int k = lane; k < K; k += 32)
    if (!mrow || mrow[k]) se += __expf(bf2f(row[k]) - mx);
  se = warp_sum(se);
  const float inv = se > 0.f ? 1.f / se : 0.f;
  const int y = labels[r];
  const bool live = soft ? true : (y >= 0 && y < K);
  const float w = weights ? weights[b] : w_scalar;
  const float* q = soft ? soft + (long long)r * K : nullptr;
  float soft_loss = 0.f;
  if (q) {
    const float lse = mx + __logf(se);
    for (int k = lane; k < K; k += 32)
      if ((!mrow || mrow[k]) && q[k] > 0.f) soft_loss -= q[k] * (bf2f(row[k]) - lse);
    soft_loss = warp_sum(soft_loss);
  }
  if (delta || probs) {
    // the last head also clears the padding columns behind the heads
    const int kend = (l == L - 1) ? ld - l * K : K;
    for (int k = lane; k < kend; k += 32) {
      float pk = 0.f;
      if (k < K && (!mrow || mrow[k])) pk = __expf(bf2f(row[k]) - mx) * inv;
      if (probs && k < K) probs[(long long)r * K + k] = pk;
      if (delta) {
        float d = 0.f;
        if (k < K && live) {
          d = w * (pk - (q ? q[k] : (k == y ? 1.f : 0.f)));
          if (cat_weights) d *= cat_weights[k];
        }
        delta[(long long)b * ld + (long long)l * K + k] = f2bf(d);
      }
    }
  }
  if (lane == 0) {
    float lo = 0.f;
    if (q) lo = soft_loss;
    else if (live) lo = -(bf2f(row[y]) - mx - __logf(se));
    if (loss_per) loss_per[r] = lo;
    if (argmax_out && l == 0) argmax_out[b] = am;
    if (loss_sum && live) atomicAdd(loss_sum, w * lo);
    if (correct && l == 0 && am == y) atomicAdd(correct, 1);
  }
}

// Categorical heads of the second layer generation other than softmax + cross-entropy. Their backward kernels live
// outside the reference's tree; what is restated here follows from the call sites (src/layer_new.rs:2249-2258
// `batch_map_softmax_ind_backward(probs, K, B, labels, weights, delta)`, :2703-2738 `batch_blockreduce_sum` of the
// raw inputs followed by `batch_map_antilogistic_forward(in, K, B, sums, out)` and
// `batch_map_antilogistic_kl_backward(out, K, B, labels, weights, delta)`, and src/operator/loss.rs:322-333
// `batch_map_marginalized_softmax_ind_backward(probs, K, B, weights, category_weights, delta)`):
//   objective 1  softmax indicator: p = softmax(x); the objective is the probability mass on the target,
//                R = sum_k t_k p_k with t the one-hot label or, marginalised, a weight per category;
//                loss = 1 - R, delta_j = w p_j (R - t_j)   (for a one-hot target: w p_y (p_j - [j = y]))
//   objective 2  "antilogistic" + KL: the inputs are non-negative scores normalised by their plain sum,
//                v_k = x_k / S, S = sum_k x_k (the forward kernel receives exactly that sum);
//                loss = -log v_y, delta_j = w (1 / S - [j = y] / x_y)
//   objective 3  "antilogistic" indicator: loss = 1 - v_y, delta_j = w (x_y - [j = y] S) / S^2
// One warp per sample; masks as in the softmax head; arg-max / accuracy on the normalised values.
__global__ void categorical_obj_kernel(const bf16* __restrict__ x, int B, int K, int ld, const int* __restrict__ labels,
                                       const float* __restrict__ weights, float w_scalar, bf16* __restrict__ delta,
                                       float* __restrict__ probs, float* __restrict__ loss_sum,
                                       int* __restrict__ correct, int* __restrict__ argmax_out,
                                       const uint8_t* __restrict__ mask, const float* __restrict__ target_w,
                                       int objective) {
  pdl_prolog();
  const int warps_per_block = blockDim.x >> 5;
  const int b = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  const bf16* row = x + (long long)b * ld;
  const uint8_t* mrow = mask ? mask + (long long)b * K : nullptr;
  const bool soft = objective == 1;
  float mx = -INFINITY;
  int am = 0;
  for (int k = lane; k < K; k += 32) {
    if (mrow && !mrow[k]) continue;
    const float v = bf2f(row[k]);
    if (v > mx) { mx = v; am = k; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, mx, o);
    const int oi = __shfl_xor_sync(0xffffffffu, am, o);
    if (ov > mx || (ov == mx && oi < am)) { mx = ov; am = oi; }
  }
  // normaliser: sum of exponentials (softmax) or plain sum of the clipped scores
  float s = 0.f;
  for (int k = lane; k < K; k += 32)
    if (!mrow || mrow[k]) s += soft ? __expf(bf2f(row[k]) - mx) : fmaxf(bf2f(row[k]), 0.f);
  s = warp_sum(s);
  const float eps = 1e-6f;
  const float inv = soft ? (s > 0.f ? 1.f / s : 0.f) : 1.f / fmaxf(s, eps);
  const int y = labels ? labels[b] : -1;
  const bool live = target_w != nullptr || (y >= 0 && y < K && (!mrow || mrow[y]));
  const float w = weights ? weights[b] : w_scalar;
  // mass on the target
  float r = 0.f;
  for (int k = lane; k < K; k += 32) {
    if (mrow && !mrow[k]) continue;
    const float t = target_w ? target_w[k] : (k == y ? 1.f : 0.f);
    if (t != 0.f) r += t * (soft ? __expf(bf2f(row[k]) - mx) : fmaxf(bf2f(row[k]), 0.f)) * inv;
  }
  r = warp_sum(r);
  const float xy = (!soft && live && !target_w) ? fmaxf(bf2f(row[y]), eps) : 1.f;
  if (delta || probs) {
    for (int k = lane; k < ld; k += 32) {
      float vk = 0.f;
      if (k < K && (!mrow || mrow[k])) vk = (soft ? __expf(bf2f(row[k]) - mx) : fmaxf(bf2f(row[k]), 0.f)) * inv;
      if (probs && k < K) probs[(long long)b * K + k] = vk;
      if (delta) {
        float d = 0.f;
        if (k < K && live && (!mrow || mrow[k])) {
          const float t = target_w ? target_w[k] : (k == y ? 1.f : 0.f);
          // scores below zero are clipped (no gradient); a target without any mass gives the KL form no gradient
          const bool clipped = !soft && bf2f(row[k]) < 0.f;
          if (objective == 1) d = w * vk * (r - t);
          else if (clipped) d = 0.f;
          else if (objective == 2) d = r > eps ? w * (inv - t / xy) : 0.f;
          else d = w * (r - t) * inv;
        }
        delta[(long long)b * ld + k] = f2bf(d);
      }
    }
  }
  if (lane == 0) {
    const float lo = !live ? 0.f : (objective == 2 ? -__logf(fmaxf(r, eps)) : 1.f - r);
    if (argmax_out) argmax_out[b] = am;
    if (loss_sum && live) atomicAdd(loss_sum, w * lo);
    if (correct && am == y) atomicAdd(correct, 1);
  }
}

// Draw one category per sample from softmax(x / temperature) restricted to the admissible categories: the
// Boltzmann sampling of the first-generation softmax head (src/layer.rs:2456, a prefix-sum CDF kernel followed by a
// uniform draw). One warp per sample: maximum, normaliser, one Philox uniform per (seed, step, sample), then a
// running inclusive prefix sum over chunks of 32 categories; the first category whose cumulative mass exceeds the
// draw wins (the last admissible one if rounding leaves the draw above the total).
__global__ void sample_categories_kernel(const bf16* __restrict__ x, int B, int K, int ld,
                                         const uint8_t* __restrict__ mask, float inv_temperature, uint64_t seed,
                                         uint32_t step, int* __restrict__ out) {
  pdl_prolog();
  const int warps_per_block = blockDim.x >> 5;
  const int b = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  const bf16* row = x + (long long)b * ld;
  const uint8_t* mrow = mask ? mask + (long long)b * K : nullptr;
  float mx = -INFINITY;
  for (int k = lane; k < K; k += 32)
    if (!mrow || mrow[k]) mx = fmaxf(mx, bf2f(row[k]) * inv_temperature);
  mx = warp_max(mx);
  float se = 0.f;
  for (int k = lane; k < K; k += 32)
    if (!mrow || mrow[k]) se += __expf(bf2f(row[k]) * inv_temperature - mx);
  se = warp_sum(se);
  uint32_t r4[4];
  Philox::gen(seed, (uint64_t)b, step, r4);
  const float target = u32_to_unit(r4[0]) * se;
  float running = 0.f;
  int pick = -1, last_ok = -1;
  for (int k0 = 0; k0 < K && pick < 0; k0 += 32) {
    const int k = k0 + lane;
    const bool ok = k < K && (!mrow || mrow[k]);
    const float e = ok ? __expf(bf2f(row[k]) * inv_temperature - mx) : 0.f;
    float scan = e;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, scan, o);
      if (lane >= o) scan += up;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, ok && running + scan > target);
    const unsigned oks = __ballot_sync(0xffffffffu, ok);
    if (oks) last_ok = k0 + 31 - __clz(oks);
    if (hit) pick = k0 + __ffs(hit) - 1;
    running += __shfl_sync(0xffffffffu, scan, 31);
  }
  if (lane == 0) out[b] = pick >= 0 ? pick : last_ok;
}

// Element-wise regression / binary heads on [B][K] outputs with float targets [B][K]:
//   mode 0  logistic:  p = sigmoid(x), loss = -(t log p + (1-t) log(1-p)), delta = w (p - t); "correct" counts
//           samples whose first output lies on the target's side of 0.5
//   mode 1  L2:        loss = 0.5 (x - t)^2, delta = w (x - t)
// (the gen-2 logistic indicator head, src/layer_new.rs, and the gen-1 L2LossLayer, src/layer.rs).
__global__ void pointwise_loss_kernel(const bf16* __restrict__ x, int B, int K, int ld, const float* __restrict__ target,
                                      const float* __restrict__ weights, float w_scalar, bf16* __restrict__ delta,
                                      float* __restrict__ loss_sum, int* __restrict__ correct, int mode) {
  pdl_prolog();
  const int warps_per_block = blockDim.x >> 5;
  const int b = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  const float w = weights ? weights[b] : w_scalar;
  float loss = 0.f;
  for (int k = lane; k < ld; k += 32) {
    float d = 0.f;
    if (k < K) {
      const float v = bf2f(x[(long long)b * ld + k]), t = target[(long long)b * K + k];
      if (mode == 0) {
        // log(1 + exp(-|v|)) form keeps both logs finite
        const float sp = __logf(1.f + __expf(-fabsf(v)));
        const float log_p = (v >= 0.f ? 0.f : v) - sp, log_q = (v >= 0.f ? -v : 0.f) - sp;
        loss -= t * log_p + (1.f - t) * log_q;
        d = w * (1.f / (1.f + __expf(-v)) - t);
      } else {
        loss += 0.5f * (v - t) * (v - t);
        d = w * (v - t);
      }
    }
    if (delta) delta[(long long)b * ld + k] = f2bf(d);
  }
  loss = warp_sum(loss);
  if (lane == 0) {
    if (loss_sum) atomicAdd(loss_sum, w * loss);
    if (correct && mode == 0) {
      const float v = bf2f(x[(long long)b * ld]), t = target[(long long)b * K];
      if ((v > 0.f) == (t > 0.5f)) atomicAdd(correct, 1);
    }
  }
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_softmax_ce(const void* logits, int B, int K, int ld, int L, const int* labels, const float* weights,
                  float w_scalar, void* delta, float* probs, float* loss_sum, int* correct, float* loss_per,
                  int* argmax_out, const float* cat_weights, const void* mask, const float* soft, cudaStream_t st) {
  if (L < 1 || (long long)L * K > ld) return -10;
  const int wpb = 4;
  launch_pdl(softmax_ce_kernel, (B * L + wpb - 1) / wpb, wpb * 32, 0, st, (const bf16*)logits, B, K, ld, L, labels,
             weights, w_scalar, (bf16*)delta, probs, loss_sum, correct, loss_per, argmax_out, cat_weights,
             (const uint8_t*)mask, soft);
  return RB_LAUNCH_OK();
}

int rb_categorical_loss(const void* x, int B, int K, int ld, const int* labels, const float* weights, float w_scalar,
                        void* delta, float* probs, float* loss_sum, int* correct, int* argmax_out, const void* mask,
                        const float* target_w, int objective, cudaStream_t st) {
  if (objective < 1 || objective > 3 || K > ld || (!labels && !target_w)) return -10;
  if (objective != 1 && target_w) return -10;      // the marginalised form exists for the softmax indicator only
  const int wpb = 4;
  launch_pdl(categorical_obj_kernel, (B + wpb - 1) / wpb, wpb * 32, 0, st, (const bf16*)x, B, K, ld, labels, weights,
             w_scalar, (bf16*)delta, probs, loss_sum, correct, argmax_out, (const uint8_t*)mask, target_w, objective);
  return RB_LAUNCH_OK();
}

int rb_sample_categories(const void* x, int B, int K, int ld, const void* mask, float temperature,
                         unsigned long long seed, unsigned int step, int* out, cudaStream_t st) {
  if (K > ld || !(temperature > 0.f)) return -10;
  const int wpb = 4;
  launch_pdl(sample_categories_kernel, (B + wpb - 1) / wpb, wpb * 32, 0, st, (const bf16*)x, B, K, ld,
             (const uint8_t*)mask, 1.f / temperature, seed, step, out);
  return RB_LAUNCH_OK();
}

int rb_pointwise_loss(const void* x, int B, int K, int ld, const float* target, const float* weights, float w_scalar,
                      void* delta, float* loss_sum, int* correct, int mode, cudaStream_t st) {
  if (mode < 0 || mode > 1 || K > ld) return -10;
  const int wpb = 4;
  launch_pdl(pointwise_loss_kernel, (B + wpb - 1) / wpb, wpb * 32, 0, st, (const bf16*)x, B, K, ld, target, weights,
             w_scalar, (bf16*)delta, loss_sum, correct, mode);
  return RB_LAUNCH_OK();
}

}  // extern "C"
