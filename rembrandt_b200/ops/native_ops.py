"""Thin, allocation-free Python fronts of the CUDA kernels.

Conventions shared by every function here:

* activations are bf16, NHWC, with the channel count padded (``pad_channels``); padded channels hold zeros;
* convolution filters are ``[Kout][R*S][Cp]`` (bf16 compute copy, fp32 master/gradient);
* affine weights are ``[out][in_pad]`` row-major, which is the reference's ``[in,out]`` first-dimension-fastest
  array (src/operator/mod.rs:1024-1034);
* every function launches on the current torch stream and writes into caller-provided tensors.

The functions raise ``NativeError`` if a launcher reports a problem; there is no eager fallback.
"""
from __future__ import annotations

import torch

from .. import _native
from .._native import check, ptr, stream_handle

EPI_BF16, EPI_F32_STORE, EPI_F32_ATOMIC = 0, 1, 2
LAUNCHES = _native.LAUNCH_COUNT


def pad_channels(c: int) -> int:
    """Channel padding rule: a multiple of 64 is kept, anything else is rounded up to a multiple of 32."""
    if c % 64 == 0:
        return c
    return (c + 31) // 32 * 32


_status_words: dict[int, torch.Tensor] = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device uint32 word in which kernels record a bounded wait that ran out (0 = healthy)."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev not in _status_words:
        _status_words[dev] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
    return _status_words[dev]


def read_status() -> int:
    return int(status_word().item())


# ------------------------------------------------------------------ GEMM / convolution (tcgen05)
GEMM_WORKSPACE_BYTES = 40 << 20
_gemm_workspaces: dict = {}


def gemm_workspace() -> torch.Tensor:
    """Zeroed fp32 scratch of the tensor-core kernel for (device, current stream): the partial sums of work items that
    are cut along the reduction pass through it, and the kernel that finishes those items clears it again. Launches
    that share a workspace must be ordered on one stream, hence one workspace per stream."""
    key = (torch.cuda.current_device(), stream_handle())
    ws = _gemm_workspaces.get(key)
    if ws is None:
        ws = _gemm_workspaces[key] = torch.zeros(GEMM_WORKSPACE_BYTES // 4, dtype=torch.float32, device="cuda")
    return ws


def gemm_set_option(name: str, value: int) -> None:
    """Planner switch of the tensor-core kernel by name (force_mt, force_resident, force_halo, force_taps, force_tail,
    force_wide, bk32, bn_cap, a_split, b_split, autotune, deterministic); initial values come from RB_GEMM_<NAME> at first use."""
    if _native.cuda().rb_gemm_set_option(name.encode(), int(value)) != 0:
        raise KeyError(name)


def gemm_get_option(name: str) -> int:
    import ctypes as C_
    v = C_.c_int(0)
    if _native.cuda().rb_gemm_get_option(name.encode(), C_.byref(v)) != 0:
        raise KeyError(name)
    return v.value


class gemm_options:
    """``with gemm_options(force_mt=2, force_resident=0): ...`` sets planner switches and restores them on exit."""

    def __init__(self, **kw):
        self.kw, self.saved = kw, {}

    def __enter__(self):
        for k, v in self.kw.items():
            self.saved[k] = gemm_get_option(k)
            gemm_set_option(k, v)
        return self

    def __exit__(self, *exc):
        for k, v in self.saved.items():
            gemm_set_option(k, v)
        return False


class gemm_tuning:
    """While active, a launch of a forward / data-grad shape that has no cached plan times its candidate tile plans
    (it synchronises the stream: never inside a graph capture) and caches the fastest. A network does this at build
    time on scratch operands (`tune_conv`); outside this block launches never measure anything."""

    def __enter__(self):
        _native.cuda().rb_gemm_tune_mode(1)
        return self

    def __exit__(self, *exc):
        _native.cuda().rb_gemm_tune_mode(0)
        return False


def gemm_role_profile():
    """Cycles the roles of one CTA of the tensor-core kernel spent waiting since the last call ([A producer, B
    producer, MMA issuer on operands, MMA issuer on the epilogue, whole run, ...]); None unless the library was built
    with -DRB_GEMM_PROFILE."""
    import ctypes as C_
    buf = (C_.c_ulonglong * 8)()
    rc = _native.cuda().rb_gemm_role_profile(C_.cast(buf, C_.c_void_p))
    return list(buf) if rc == 0 else None


def gemm_last_launch() -> dict:
    """Tile plan of the most recent tensor-core launch of this process (after tuning: the plan that won)."""
    import ctypes as C_
    buf = (C_.c_int * 9)()
    _native.cuda().rb_gemm_last_launch(C_.cast(buf, C_.c_void_p))
    names = ("sub_tiles", "split_k", "resident_b", "tail_parts", "cta_pairs", "tile_width", "a_mode", "stages", "grid")
    return dict(zip(names, buf))


def gemm_clear_plans() -> None:
    _native.cuda().rb_gemm_clear_plans()


def gemm_tc(a, a_mn, lda, b, b_mn, ldb, M, N, K, d, ldd, epi=EPI_BF16, bias=None, relu=False, mask_src=None,
            n_valid=0, n_store=0, split_k=0, bn_cap=0):
    ws = gemm_workspace() if epi == EPI_BF16 else None
    rc = _native.cuda().rb_gemm_tc(ptr(a), int(a_mn), lda, ptr(b), int(b_mn), ldb, M, N, K, ptr(d), ldd, epi,
                                   ptr(bias), int(relu), ptr(mask_src), n_valid, n_store, split_k, bn_cap,
                                   ptr(ws), ws.numel() * 4 if ws is not None else 0,
                                   ptr(status_word()), stream_handle())
    check(rc, "rb_gemm_tc")


def conv_fprop_tc(x, N, H, W, Cp, w, Kout, R, S, stride, pad_h, pad_w, P, Q, y, ldy, bias=None, relu=False,
                  mask_src=None, n_valid=0, n_store=0):
    ws = gemm_workspace()
    rc = _native.cuda().rb_conv_fprop_tc(ptr(x), N, H, W, Cp, ptr(w), Kout, R, S, stride, pad_h, pad_w, P, Q, ptr(y),
                                         ldy, ptr(bias), int(relu), ptr(mask_src), n_valid, n_store,
                                         ptr(ws), ws.numel() * 4, ptr(status_word()), stream_handle())
    check(rc, "rb_conv_fprop_tc")


_tuned_convs: set = set()


def tune_conv(N, H, W, Cp, Kout, R, S, stride, pad_h, pad_w, P, Q, ldy, relu=False, has_bias=False, has_mask=False,
              n_valid=0, n_store=0):
    """Measure the tile plans of one convolution shape (forward form; a stride-1 data-grad is the same call with the
    roles of input and output exchanged) on scratch operands and cache the winner; later launches of the shape only
    look the plan up. Idempotent per shape and process."""
    key = (torch.cuda.current_device(), N, H, W, Cp, Kout, R, S, stride, pad_h, pad_w, P, Q, ldy, bool(has_mask),
           n_valid, n_store)
    if key in _tuned_convs:
        return
    _tuned_convs.add(key)
    dev = "cuda"
    x = torch.zeros((N, H, W, Cp), dtype=torch.bfloat16, device=dev)
    w = torch.zeros((max(Kout, n_store), R * S, Cp), dtype=torch.bfloat16, device=dev)
    y = torch.zeros((N * P * Q, ldy), dtype=torch.bfloat16, device=dev)
    bias = torch.zeros(max(Kout, n_store), dtype=torch.float32, device=dev) if has_bias else None
    mask = torch.zeros_like(y) if has_mask else None
    with gemm_tuning():
        conv_fprop_tc(x, N, H, W, Cp, w, Kout, R, S, stride, pad_h, pad_w, P, Q, y, ldy, bias=bias, relu=relu,
                      mask_src=mask, n_valid=n_valid, n_store=n_store)
    torch.cuda.current_stream().synchronize()


def conv_wgrad_tc(x, N, H, W, Cp, dy, lddy, Kout, R, S, stride, pad_h, pad_w, P, Q, dw, split_k=0):
    rc = _native.cuda().rb_conv_wgrad_tc(ptr(x), N, H, W, Cp, ptr(dy), lddy, Kout, R, S, stride, pad_h, pad_w, P, Q,
                                         ptr(dw), split_k, ptr(status_word()), stream_handle())
    check(rc, "rb_conv_wgrad_tc")


def conv_direct_fwd(x, w, bias, y, N, H, W, Cp, Kout, Kp, R, S, stride, pad_h, pad_w, P, Q, relu):
    check(_native.cuda().rb_conv_direct_fwd(ptr(x), ptr(w), ptr(bias), ptr(y), N, H, W, Cp, Kout, Kp, R, S, stride,
                                            pad_h, pad_w, P, Q, int(relu), stream_handle()), "rb_conv_direct_fwd")


def conv_direct_dgrad(dy, w, dx, mask_src, N, H, W, Cp, Kout, Kp, R, S, stride, pad_h, pad_w, P, Q):
    check(_native.cuda().rb_conv_direct_dgrad(ptr(dy), ptr(w), ptr(dx), ptr(mask_src), N, H, W, Cp, Kout, Kp, R, S,
                                              stride, pad_h, pad_w, P, Q, stream_handle()), "rb_conv_direct_dgrad")


def conv_direct_wgrad(x, dy, dw, N, H, W, Cp, Kout, Kp, R, S, stride, pad_h, pad_w, P, Q):
    check(_native.cuda().rb_conv_direct_wgrad(ptr(x), ptr(dy), ptr(dw), N, H, W, Cp, Kout, Kp, R, S, stride, pad_h,
                                              pad_w, P, Q, stream_handle()), "rb_conv_direct_wgrad")


def pack_dgrad_filters(w16, wt16, Kout, Kp, RS, Cp):
    check(_native.cuda().rb_pack_dgrad_filters(ptr(w16), ptr(wt16), Kout, Kp, RS, Cp, stream_handle()),
          "rb_pack_dgrad_filters")


def zero_s2d_structural(dw, Kout, R2, Cp, f, cin, ksize):
    check(_native.cuda().rb_zero_s2d_structural(ptr(dw), Kout, R2, Cp, f, cin, ksize, stream_handle()),
          "rb_zero_s2d_structural")


# ------------------------------------------------------------------ memory-bound operators
def gemv_sparse(w, n, k, transposed, val, ind, nnz, y, alpha=1.0, beta=0.0):
    """y = beta * y + alpha * W x for x given by `nnz` (value, index) pairs; W fp32 [n][k], or [k][n] if `transposed`."""
    check(_native.cuda().rb_gemv_sparse(ptr(w), n, k, int(bool(transposed)), ptr(val), ptr(ind), nnz, float(alpha),
                                        float(beta), ptr(y), stream_handle()), "rb_gemv_sparse")


def colsum(x, rows, ld, cols, out):
    check(_native.cuda().rb_colsum(ptr(x), rows, ld, cols, ptr(out), stream_handle()), "rb_colsum")


def bias_act(acc, rows, ld, n_valid, bias, relu, y, mask_src=None, rezero=True):
    check(_native.cuda().rb_bias_act(ptr(acc), rows, ld, n_valid, ptr(bias), int(relu), ptr(y), ptr(mask_src),
                                     int(rezero), stream_handle()), "rb_bias_act")


def dropout(x, y, n, p, seed, stream_id, mask_src=None, step_ptr=None):
    check(_native.cuda().rb_dropout(ptr(x), ptr(y), ptr(mask_src), n, float(p), int(seed) & (2**64 - 1),
                                    int(stream_id) & 0xFFFFFFFF, ptr(step_ptr), stream_handle()), "rb_dropout")


def relu_mask(d, y, n):
    check(_native.cuda().rb_relu_mask(ptr(d), ptr(y), n, stream_handle()), "rb_relu_mask")


ACT_LOGISTIC, ACT_TANH, ACT_BOUNDED_RECT, ACT_RECT, ACT_SCALED_LOGISTIC = 1, 2, 3, 4, 5


def act_fwd(y, rows, ld, n_valid, kind, bound=0.0):
    """y = f(y) in place on the first `n_valid` columns of a bf16 [rows][ld] buffer (logistic, tanh, clipped ReLU)."""
    check(_native.cuda().rb_act_fwd(ptr(y), rows, ld, n_valid, kind, float(bound), stream_handle()), "rb_act_fwd")


def act_bwd(d, y, rows, ld, n_valid, kind, bound=0.0):
    """d *= f'(y) in place, with the slope written in terms of the output y."""
    check(_native.cuda().rb_act_bwd(ptr(d), ptr(y), rows, ld, n_valid, kind, float(bound), stream_handle()),
          "rb_act_bwd")


def count_above(x, threshold, out):
    """out[0] (int64, device) += number of elements of the bf16 / fp32 tensor `x` with |x| > threshold."""
    check(_native.cuda().rb_count_above(ptr(x), x.numel(), int(x.dtype == torch.float32), float(threshold), ptr(out),
                                        stream_handle()), "rb_count_above")


def add_bf16(a, b, n):
    check(_native.cuda().rb_add_bf16(ptr(a), ptr(b), n, stream_handle()), "rb_add_bf16")


def f32_to_bf16(x, y, n):
    check(_native.cuda().rb_f32_to_bf16(ptr(x), ptr(y), n, stream_handle()), "rb_f32_to_bf16")


def pool_fwd(x, y, idx, N, H, W, C, P, Q, k, stride, pad, is_max, relu):
    check(_native.cuda().rb_pool_fwd(ptr(x), ptr(y), ptr(idx), N, H, W, C, P, Q, k, stride, pad, int(is_max),
                                     int(relu), stream_handle()), "rb_pool_fwd")


def pool_bwd(dy, idx, y_relu, dx, mask_src, N, H, W, C, P, Q, k, stride, pad, is_max):
    check(_native.cuda().rb_pool_bwd(ptr(dy), ptr(idx), ptr(y_relu), ptr(dx), ptr(mask_src), N, H, W, C, P, Q, k,
                                     stride, pad, int(is_max), stream_handle()), "rb_pool_bwd")


def lrn_fwd(x, y, pixels, C, size, alpha_eff, beta, k):
    check(_native.cuda().rb_lrn_fwd(ptr(x), ptr(y), pixels, C, size, alpha_eff, beta, k, stream_handle()),
          "rb_lrn_fwd")


def lrn_bwd(x, dy, dx, mask_src, pixels, C, size, alpha_eff, beta, k):
    check(_native.cuda().rb_lrn_bwd(ptr(x), ptr(dy), ptr(dx), ptr(mask_src), pixels, C, size, alpha_eff, beta, k,
                                    stream_handle()), "rb_lrn_bwd")


def softmax_ce(logits, B, K, ld, labels, weights, w_scalar, delta, probs=None, loss_sum=None, correct=None,
               loss_per=None, argmax_out=None, cat_weights=None, mask=None, heads=1, soft=None):
    """`heads` > 1: every sample carries that many blocks of K logits (labels [B, heads], negative = skip).
    `mask`: uint8 [B * heads, K], zero marks a category that must get probability zero.
    `soft`: float32 [B * heads, K] target distribution that replaces the one-hot label (distillation)."""
    check(_native.cuda().rb_softmax_ce(ptr(logits), B, K, ld, int(heads), ptr(labels), ptr(weights), float(w_scalar),
                                       ptr(delta), ptr(probs), ptr(loss_sum), ptr(correct), ptr(loss_per),
                                       ptr(argmax_out), ptr(cat_weights), ptr(mask), ptr(soft), stream_handle()),
          "rb_softmax_ce")


def sample_categories(x, B, K, ld, mask, temperature, seed, step, out):
    """out[b] (int32) = one draw from softmax(x[b] / temperature) over the categories whose mask byte is non-zero."""
    check(_native.cuda().rb_sample_categories(ptr(x), B, K, ld, ptr(mask), float(temperature), int(seed) & (2**64 - 1),
                                              int(step) & 0xFFFFFFFF, ptr(out), stream_handle()),
          "rb_sample_categories")


OBJ_SOFTMAX_IND, OBJ_ANTILOGISTIC_KL, OBJ_ANTILOGISTIC_IND = 1, 2, 3


def categorical_loss(x, B, K, ld, labels, weights, w_scalar, delta, objective, probs=None, loss_sum=None, correct=None,
                     argmax_out=None, mask=None, target_w=None):
    """Categorical heads other than softmax + cross-entropy (csrc/softmax_ce.cu, `categorical_obj_kernel`):
    softmax indicator (one-hot label, or `target_w` [K] = a weight per category), antilogistic + KL, antilogistic
    indicator."""
    check(_native.cuda().rb_categorical_loss(ptr(x), B, K, ld, ptr(labels), ptr(weights), float(w_scalar), ptr(delta),
                                             ptr(probs), ptr(loss_sum), ptr(correct), ptr(argmax_out), ptr(mask),
                                             ptr(target_w), int(objective), stream_handle()), "rb_categorical_loss")


def pointwise_loss(x, B, K, ld, target, weights, w_scalar, delta, loss_sum=None, correct=None, mode=0):
    """mode 0: logistic (binary cross-entropy on logits), mode 1: L2; targets float32 [B, K]."""
    check(_native.cuda().rb_pointwise_loss(ptr(x), B, K, ld, ptr(target), ptr(weights), float(w_scalar), ptr(delta),
                                           ptr(loss_sum), ptr(correct), int(mode), stream_handle()),
          "rb_pointwise_loss")


def sgd_fused(w, g, v, w16, n, lr, mu, l2, grad_scale, mode, phase=7):
    check(_native.cuda().rb_sgd_fused(ptr(w), ptr(g), ptr(v), ptr(w16), n, lr, mu, l2, grad_scale, mode, phase,
                                      stream_handle()), "rb_sgd_fused")


def sgd_fused_grid(w, g, v, w16, n, lr, mu, l2, grad_scale, mode, phase=7, blocks=296, threads=128):
    """The fused SGD sweep with an explicit grid (small blocks that co-reside with the GEMM CTAs)."""
    check(_native.cuda().rb_sgd_fused_grid(ptr(w), ptr(g), ptr(v), ptr(w16), n, lr, mu, l2, grad_scale, mode, phase,
                                           int(blocks), int(threads), stream_handle()), "rb_sgd_fused_grid")


def axpy_shadow(w, v, w16, n, s):
    check(_native.cuda().rb_axpy_shadow(ptr(w), ptr(v), ptr(w16), n, float(s), stream_handle()), "rb_axpy_shadow")


def axpby(x, y, n, a, b):
    check(_native.cuda().rb_axpby(ptr(x), ptr(y), n, float(a), float(b), stream_handle()), "rb_axpby")


def input_u8(src, mean, dst, N, C, H, W, crop_h, crop_w, OH, OW, Cp, f, lo_y, hi_y, lo_x, hi_x, random_crop,
             random_flip, per_batch, scale, mean_scale, pca_sigma, pca_vals, pca_vecs, seed, step, step_ptr=None):
    import ctypes as C_
    pv = (C_.c_float * 3)(*pca_vals) if pca_vals is not None else None
    pe = (C_.c_float * 9)(*pca_vecs) if pca_vecs is not None else None
    check(_native.cuda().rb_input_u8(ptr(src), ptr(mean), ptr(dst), N, C, H, W, crop_h, crop_w, OH, OW, Cp, f, lo_y,
                                     hi_y, lo_x, hi_x, int(random_crop), int(random_flip), int(per_batch),
                                     float(scale), float(mean_scale), float(pca_sigma),
                                     C_.cast(pv, C_.c_void_p) if pv is not None else None,
                                     C_.cast(pe, C_.c_void_p) if pe is not None else None,
                                     int(seed) & (2**64 - 1), int(step) & 0xFFFFFFFF, ptr(step_ptr), stream_handle()),
          "rb_input_u8")


def var_input_u8(src, shapes, dst, draws, in_stride, N, C, crop_h, crop_w, Cp, f, ep, OH, OW, scale_lower, scale_upper,
                 train, random_flip, per_batch, scale, mean, pca_sigma, pca_vals, pca_vecs, seed, step, step_ptr=None):
    """Variable-size input: bicubic rescale + crop + flip + mean + lighting noise in one kernel (csrc/var_input.cu)."""
    import ctypes as C_
    mv = (C_.c_float * 4)(*(list(mean) + [0.0] * 4)[:4]) if mean is not None else None
    pv = (C_.c_float * 3)(*pca_vals) if pca_vals is not None else None
    pe = (C_.c_float * 9)(*pca_vecs) if pca_vecs is not None else None
    cast = lambda a: C_.cast(a, C_.c_void_p) if a is not None else None
    check(_native.cuda().rb_var_input_u8(ptr(src), ptr(shapes), ptr(dst), ptr(draws), int(in_stride), N, C, crop_h,
                                         crop_w, Cp, f, ep, OH, OW, scale_lower, scale_upper, int(train),
                                         int(random_flip), int(per_batch), float(scale), cast(mv), float(pca_sigma),
                                         cast(pv), cast(pe), int(seed) & (2**64 - 1), int(step) & 0xFFFFFFFF,
                                         ptr(step_ptr), stream_handle()), "rb_var_input_u8")


def synth_normal(dst, pixels, C, Cp, seed, step):
    check(_native.cuda().rb_synth_normal(ptr(dst), pixels, C, Cp, int(seed) & (2**64 - 1), int(step) & 0xFFFFFFFF,
                                         stream_handle()), "rb_synth_normal")


def synth_labels(labels, n, classes, seed, step):
    check(_native.cuda().rb_synth_labels(ptr(labels), n, classes, int(seed) & (2**64 - 1), int(step) & 0xFFFFFFFF,
                                         stream_handle()), "rb_synth_labels")


def bn_fwd_train(x, rows, C, c_valid, sums, eps, factor, mean, istd, run_mean, run_var, gamma, beta, residual, y,
                 relu, avg_kind=0, step_ptr=None):
    """avg_kind 1 (cumulative) / 2 (exponential, 1 at step 0) derive the averaging factor from the device-side step
    counter `step_ptr`, so that a captured graph keeps averaging correctly; 0 uses `factor` as given."""
    check(_native.cuda().rb_bn_fwd_train(ptr(x), rows, C, c_valid, ptr(sums), eps, factor, ptr(mean), ptr(istd),
                                         ptr(run_mean), ptr(run_var), ptr(gamma), ptr(beta), ptr(residual), ptr(y),
                                         int(relu), int(avg_kind), ptr(step_ptr), stream_handle()), "rb_bn_fwd_train")


def bn_fwd_infer(x, rows, C, c_valid, eps, run_mean, run_var, istd_tmp, gamma, beta, residual, y, relu):
    check(_native.cuda().rb_bn_fwd_infer(ptr(x), rows, C, c_valid, eps, ptr(run_mean), ptr(run_var), ptr(istd_tmp),
                                         ptr(gamma), ptr(beta), ptr(residual), ptr(y), int(relu), stream_handle()),
          "rb_bn_fwd_infer")


def bn_bwd(x, dy, y_relu, rows, C, c_valid, sums, mean, istd, gamma, dgamma, dbeta, dx):
    check(_native.cuda().rb_bn_bwd(ptr(x), ptr(dy), ptr(y_relu), rows, C, c_valid, ptr(sums), ptr(mean), ptr(istd),
                                   ptr(gamma), ptr(dgamma), ptr(dbeta), ptr(dx), stream_handle()), "rb_bn_bwd")
