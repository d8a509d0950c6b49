// The momentum rules as one device function, shared by the single-GPU fused optimizer (sgd_fused.cu) and the
// communication kernels that apply the update in the same pass as the gradient reduction (comm_p2p.cu).
//
// Rules (src/opt/sgd/new.rs:377-463 of the reference), g' = grad_scale * g + l2 * w :
//   0 Zero             v = -lr g'            w += v
//   1 Update           v = mu v - lr g'      w += v
//   2 UpdateNesterov   w is stored at the look-ahead point w + mu v:
//                      w -= mu v_old ; v = mu v_old - lr g' ; w += v ; w += mu v
//   3 Gradient         v = mu v + g'         w -= lr v
//   4 GradientNesterov v = mu v + g'         w -= lr g' + lr mu v
//   5 GradDecay        w -= lr g' ; g = mu g'   (gen-2 rule, src/opt_new.rs:321-327; no velocity buffer)
// phase bits: 1 = regularise + accumulate into v, 2 = apply to w, 4 = zero g.
#pragma once

namespace rb {

struct SgdHyper {
  float lr, mu, l2, grad_scale;
  int mode, phase;
};

__device__ __forceinline__ void sgd_elem(float& w, float& g, float& v, const SgdHyper& a) {
  const bool acc = a.phase & 1, upd = a.phase & 2, zero = a.phase & 4;
  const float gp = a.grad_scale * g + a.l2 * w;
  switch (a.mode) {
    case 0:
    case 1:
      if (acc) v = (a.mode == 0 ? 0.f : a.mu * v) - a.lr * gp;
      if (upd) w += v;
      break;
    case 2:
      if (acc) { w -= a.mu * v; v = a.mu * v - a.lr * gp; }
      if (upd) w += v + a.mu * v;
      break;
    case 3:
      if (acc) v = a.mu * v + gp;
      if (upd) w -= a.lr * v;
      break;
    case 4:
      if (acc) v = a.mu * v + gp;
      if (upd) w -= a.lr * gp + a.lr * a.mu * v;
      break;
    case 5:
      if (upd) { w -= a.lr * gp; g = a.mu * gp; }   // the decay belongs to the applying phase: once per step
      break;
  }
  if (zero && a.mode != 5) g = 0.f;
}

}  // namespace rb
